"""B200-native F3M engine: Gaussian kernel matrix-vector products on hand-written sm_100a kernels
behind a C ABI (include/f3m.h).  Importing the package loads libf3m.so and fails if it is absent."""
from . import _lib

_lib.lib()   # no fallback: a missing library is an import error

from .FFM_classes import FFM, benchmark_matmul, benchmark_matmul_double, block_FFM_matmul, par_FFM_block  # noqa: E402
from . import engine  # noqa: E402

__all__ = ["FFM", "benchmark_matmul", "benchmark_matmul_double", "block_FFM_matmul", "par_FFM_block", "engine"]
