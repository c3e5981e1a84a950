"""Operator surface of the engine: the classes the reference defines in experiments/FFM_classes.py,
with the same constructor arguments, methods and error behaviour, running on libf3m.so.

  FFM(X, Y=None, ls, min_points, nr_of_interpolation, eff_var_limit, var_compression,
      small_field_points, device)            experiments/FFM_classes.py:8-126
  obj @ b, obj.forward(X, Y, b), obj.grad(b), obj.chunk_forward_transpose / chunk_forward_example,
  obj.update_ls(ls)
  benchmark_matmul(X, Y, ls, device) @ b      experiments/FFM_classes.py:264-323 (exact dense op, float32)
  benchmark_matmul_double(...)                experiments/FFM_classes.py:325-383 (float64)
  block_FFM_matmul(...)                       experiments/FFM_classes.py:385-435
  par_FFM_block(...)                          experiments/FFM_classes.py:128-211

Differences, all on purpose: pykeops is not needed at import; a product whose X and Y are the tensors
given at construction reuses the tree and the interaction lists between calls (the reference rebuilds
them for every product); dimensions above 5 raise instead of printing.
"""
from __future__ import annotations

import torch

from . import engine
from ._lib import MATH_FASTMATH, FLAG_NEAR_MOMENTS

MAX_DIM = 5


class FFM:
    def __init__(self, X, Y=None, ls=1.0, min_points=1000, nr_of_interpolation=64, eff_var_limit=0.15,
                 var_compression=False, small_field_points=1000, device="cuda:0", math_mode=MATH_FASTMATH,
                 near_moments=False):
        # math_mode and near_moments are additions to the reference's arguments: the numeric flavour of the box
        # index / far test, and the optional evaluation of near sums by box moments (see include/f3m.h)
        self.X = X.float().to(device)
        if torch.is_tensor(Y):
            self.Y = Y.float().to(device)
        else:
            self.Y = self.X          # shared tree: K(X, X)
        self.d = self.X.shape[1]
        if not 1 <= self.d <= MAX_DIM:
            raise ValueError(f"dimension {self.d} not supported (1..{MAX_DIM})")
        self.ls = float(ls)
        self.min_points = float(min_points)
        self.nr_of_interpolation = int(nr_of_interpolation)
        self.eff_var_limit = float(eff_var_limit)
        self.var_compression = var_compression
        self.device = device
        self.small_field_points = small_field_points
        self.math_mode = math_mode
        self.near_moments = bool(near_moments)
        self._plan = None
        self._plan_key = None

    # ---- parameters ----------------------------------------------------------------------------
    def _params(self):
        return engine.make_params(self.ls, self.min_points, self.nr_of_interpolation, self.var_compression,
                                  self.eff_var_limit, self.small_field_points, self.math_mode,
                                  flags=FLAG_NEAR_MOMENTS if self.near_moments else 0)

    def update_ls(self, ls):
        if not ls > 0:
            raise AssertionError("ls must be positive")
        self.ls = float(ls)

    # ---- products ------------------------------------------------------------------------------
    def __matmul__(self, b):
        self.b = b.float().to(self.device)
        return self.forward(self.X, self.Y, self.b)

    def grad(self, b):
        self.b = b.float().to(self.device)
        return self.forward_grad(self.X, self.Y, self.b)

    def _check(self, X, Y, b):
        assert X.device == Y.device == b.device == torch.device(self.device)
        self.device = str(self.device)
        if not (Y.shape[1] == X.shape[1] and Y.shape[0] == b.shape[0]):
            raise AssertionError("shapes of X, Y and b do not match")

    def plan(self, X=None, Y=None):
        """Tree + lists for (X, Y); cached while the tensors and the parameters stay the same."""
        X = self.X if X is None else X
        Y = self.Y if Y is None else Y
        key = (X.data_ptr(), X._version, tuple(X.shape), Y.data_ptr(), Y._version, tuple(Y.shape), self.ls,
               self.min_points, self.nr_of_interpolation, self.eff_var_limit, bool(self.var_compression),
               self.small_field_points, self.math_mode, self.near_moments)
        if self._plan is None or self._plan_key != key:
            if self._plan is not None:
                self._plan.close()
            self._plan = engine.Plan(X, None if engine.is_shared(X, Y) else Y, self._params())
            self._plan_key = key
        return self._plan

    def forward(self, X, Y, b):
        self._check(X, Y, b)
        own = engine.is_shared(self.X, X) and engine.is_shared(self.Y, Y)   # the tensors given at construction
        if own:
            return self.plan(X, Y).apply(b)
        return engine.kmvm(X, None if engine.is_shared(X, Y) else Y, b, self._params())

    def forward_grad(self, X, Y, b):
        if not (Y.shape[1] == X.shape[1] and Y.shape[0] == b.shape[0]):
            raise AssertionError("shapes of X, Y and b do not match")
        return engine.rbf_dense(X, Y, b, self.ls, grad=True)

    def chunk_forward_transpose(self, b, chunks=10):
        """K(Y, X) b summed over chunks of X (experiments/FFM_classes.py:54-61)."""
        self.b = b.float().to(self.device)
        res = 0.0
        for bc, yc in zip(torch.chunk(self.b, dim=0, chunks=chunks), torch.chunk(self.X, dim=0, chunks=chunks)):
            res = res + self.forward(self.Y, yc, bc)
        return res

    def chunk_forward_example(self, b, chunks=10):
        """K(X, Y) b summed over chunks of Y (experiments/FFM_classes.py:63-70)."""
        self.b = b.float().to(self.device)
        res = 0.0
        for bc, yc in zip(torch.chunk(self.b, dim=0, chunks=chunks), torch.chunk(self.Y, dim=0, chunks=chunks)):
            res = res + self.forward(self.X, yc, bc)
        return res


class benchmark_matmul:
    """Exact dense product in float32 (experiments/FFM_classes.py:264-323)."""
    _dtype = torch.float32

    def __init__(self, X, Y=None, ls=1.0, device="cuda:0"):
        self.device = device
        self.X = X.to(self._dtype).to(device)
        self.Y = Y.to(self._dtype).to(device) if torch.is_tensor(Y) else self.X
        self.ls = float(ls)
        self.d = self.X.shape[1]
        if not 1 <= self.d <= MAX_DIM:
            raise ValueError(f"dimension {self.d} not supported (1..{MAX_DIM})")

    def __matmul__(self, b):
        self.b = b.to(self._dtype).to(self.device)
        return self.forward(self.X, self.Y, self.b)

    def forward(self, X, Y, b):
        if not (Y.shape[1] == X.shape[1] and Y.shape[0] == b.shape[0]):
            raise AssertionError("shapes of X, Y and b do not match")
        return engine.rbf_dense(X, Y, b, self.ls)


class benchmark_matmul_double(benchmark_matmul):
    """Exact dense product in float64 (experiments/FFM_classes.py:325-383), with a double-precision exponential."""
    _dtype = torch.float64


class block_FFM_matmul(FFM):
    """Blocked product accumulated on the host (experiments/FFM_classes.py:385-435): K is split into
    blocks_X x blocks_Y tiles and each tile is one product of its own.  (The reference passes None as Y on
    diagonal blocks, which its own forward cannot handle; here diagonal blocks use the shared-tree product.)"""

    def __init__(self, X, Y=None, ls=1.0, min_points=1000, nr_of_interpolation=64, eff_var_limit=0.15,
                 var_compression=False, small_field_points=1000, device="cuda:0", blocks_X=1, blocks_Y=1):
        super().__init__(X=X, Y=Y, ls=ls, min_points=min_points, nr_of_interpolation=nr_of_interpolation,
                         eff_var_limit=eff_var_limit, var_compression=var_compression,
                         small_field_points=small_field_points, device=device)
        self.blocks_X = blocks_X
        self.blocks_Y = blocks_Y
        self._xy_mode = torch.is_tensor(Y)

    def __matmul__(self, b):
        b = b.float().to(self.device)
        out = []
        if self._xy_mode:
            ys = torch.chunk(self.Y, self.blocks_Y, dim=0)
            bs = torch.chunk(b, self.blocks_Y, dim=0)
            for x in torch.chunk(self.X, self.blocks_X, dim=0):
                acc = torch.zeros(x.shape[0], b.shape[1])
                for y, bc in zip(ys, bs):
                    acc += self.forward(x.contiguous(), y.contiguous(), bc.contiguous()).cpu()
                out.append(acc)
        else:
            xs = [x.contiguous() for x in torch.chunk(self.X, self.blocks_X, dim=0)]
            bs = torch.chunk(b, self.blocks_X, dim=0)
            for i, x in enumerate(xs):
                acc = torch.zeros(x.shape[0], b.shape[1])
                for j, y in enumerate(xs):
                    acc += self.forward(x, x if i == j else y, bs[j].contiguous()).cpu()
                out.append(acc)
        return torch.cat(out, dim=0)


class par_FFM_block:
    """Independent block products spread over several GPUs (experiments/FFM_classes.py:128-211): K is cut
    into len(devices) x len(devices) blocks, block (x_i, y_j) runs on devices[i], and calling the object
    returns the list of block results in the reference's job order (outer loop over y blocks, inner over x
    blocks) without summing them, as the reference does.  One host thread per device instead of one
    process per device; for a product that is summed and sharded by target boxes see f3m_b200.parallel."""

    def __init__(self, X, b, Y=None, ls=1.0, min_points=1000, nr_of_interpolation=64, eff_var_limit=0.15,
                 var_compression=False, small_field_points=1000, devices=(0,)):
        self.X = X.float()
        self.b = b.float()
        self.Y = Y.float() if torch.is_tensor(Y) else self.X
        self.d = self.X.shape[1]
        if not 1 <= self.d <= MAX_DIM:
            raise ValueError(f"dimension {self.d} not supported (1..{MAX_DIM})")
        self.ls, self.min_points = float(ls), float(min_points)
        self.nr_of_interpolation, self.eff_var_limit = int(nr_of_interpolation), float(eff_var_limit)
        self.var_compression, self.small_field_points = var_compression, small_field_points
        self.devices = list(devices)
        self.par_fac = len(self.devices)
        ys = torch.chunk(self.Y, self.par_fac, dim=0)
        xs = torch.chunk(self.X, self.par_fac, dim=0)
        bs = torch.chunk(self.b, self.par_fac, dim=0)
        self.jobs_list = [(x.clone(), y.clone(), bb.clone(), dev) for y, bb in zip(ys, bs) for x, dev in zip(xs, self.devices)]

    def update_ls(self, ls):
        if not ls > 0:
            raise AssertionError("ls must be positive")
        self.ls = float(ls)

    def forward(self, X, Y, b, device):
        dev = torch.device("cuda", int(device))
        X, Y, b = X.to(dev), Y.to(dev), b.to(dev)
        if not (Y.shape[1] == X.shape[1] and Y.shape[0] == b.shape[0]):
            raise AssertionError("shapes of X, Y and b do not match")
        prm = engine.make_params(self.ls, self.min_points, self.nr_of_interpolation, self.var_compression,
                                 self.eff_var_limit, self.small_field_points)
        with torch.cuda.device(dev):
            return engine.kmvm(X, Y, b, prm)

    def __call__(self):
        from concurrent.futures import ThreadPoolExecutor
        results = [None] * len(self.jobs_list)
        by_device = {}
        for k, job in enumerate(self.jobs_list):
            by_device.setdefault(job[3], []).append(k)

        def run(keys):
            for k in keys:
                results[k] = self.forward(*self.jobs_list[k])

        with ThreadPoolExecutor(max_workers=len(by_device)) as ex:
            list(ex.map(run, by_device.values()))
        return results
