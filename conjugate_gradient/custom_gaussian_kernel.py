"""Stand-in for the reference's FALKON kernel glue (conjugate_gradient/custom_gaussian_kernel.py): the same
products (mmv, dmmv) on the B200 engine, without the third-party `falkon` base class."""
from f3m_b200.solvers import F3MGaussianKernel as custom_GaussianKernel, Falkon  # noqa: F401
