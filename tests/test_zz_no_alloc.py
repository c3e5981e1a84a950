"""The allocation-free dense entry point against the allocating one, through the C ABI.

f3m_rbf_dense_f32_static is for callers that may not allocate device memory at run time (all memory
owned by the host application's pool, or a no-allocation rule in a latency-critical loop); it keeps its
scratch in a fixed array of the library.  Two calls in a row with different sizes check that what one call
leaves in the shared array does not leak into the next, and an oversized problem must be refused."""
import ctypes

import pytest
import torch

from cases import rel_l2

pytestmark = pytest.mark.gpu


def _call(fn, X, Y, b, ls):
    out = torch.empty(X.shape[0], b.shape[1], device=X.device, dtype=torch.float32)
    st = fn(X.data_ptr(), X.shape[0], Y.data_ptr(), Y.shape[0], b.data_ptr(), b.shape[1], X.shape[1], ctypes.c_float(ls),
            out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return st, out


def test_static_entry_matches_allocating_entry(cuda):
    from f3m_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(21)
    # second call: fewer sources, more columns, another dimension -> stale rows of the first call must not matter
    for (n, m, d, r, ls) in [(3000, 50000, 3, 1, 0.7), (1500, 9000, 5, 3, 1.3)]:
        X = torch.rand(n, d, generator=g).to(cuda)
        Y = torch.rand(m, d, generator=g).to(cuda)
        b = torch.randn(m, r, generator=g).to(cuda)
        st_a, ref = _call(L.f3m_rbf_dense_f32, X, Y, b, ls)
        st_b, out = _call(L.f3m_rbf_dense_f32_static, X, Y, b, ls)
        torch.cuda.synchronize()
        assert st_a == 0 and st_b == 0, L.f3m_last_error()
        assert rel_l2(out.cpu(), ref.cpu()) <= 2e-6
    # beyond the fixed capacity: a clear error, nothing computed
    m_big = 4 * 1024 * 1024 // 4 + 1
    X = torch.rand(8, 3, device=cuda)
    Y = torch.rand(m_big, 3, device=cuda)
    b = torch.randn(m_big, 1, device=cuda)
    st, _ = _call(L.f3m_rbf_dense_f32_static, X, Y, b, 1.0)
    assert st == 7      # F3M_ERR_TOO_LARGE
    assert b"f3m_rbf_dense_f32_static holds" in L.f3m_last_error()
