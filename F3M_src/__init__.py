"""Import-name compatibility: callers of the reference import `F3M_src.FFM_classes`
(conjugate_gradient/custom_gaussian_kernel.py:6)."""
