"""`from F3M_src.FFM_classes import *` as the reference's callers write it."""
from f3m_b200.FFM_classes import *  # noqa: F401,F403
from f3m_b200.FFM_classes import FFM, benchmark_matmul, benchmark_matmul_double, block_FFM_matmul, par_FFM_block  # noqa: F401
