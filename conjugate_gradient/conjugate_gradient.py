"""`from conjugate_gradient.conjugate_gradient import ...` as the reference's scripts write it
(conjugate_gradient/gp_experiment_object.py); the implementations live in f3m_b200/solvers.py."""
from f3m_b200.solvers import (ConjugateGradientSolver, PreConditionedConjugateGradientSolver, nystrom_preconditioner,  # noqa: F401
                              subsample_inducing_points, build_tridiagonalization_matrices, calculate_log_kxx,
                              get_GP_likelihood)
