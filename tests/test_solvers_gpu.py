"""Callers of the KMVM operator: conjugate gradients and FALKON, checked against dense float64 solves.
(The reference takes FALKON's preconditioner and CG loop from the third-party `falkon` package, which is
not available: parity with `falkon` itself is unpinned; the linear algebra is checked directly.)"""
import pytest
import torch

from cases import rel_l2

pytestmark = pytest.mark.gpu


def test_conjugate_gradient_solves_regularised_system(cuda):
    from conjugate_gradient.conjugate_gradient import ConjugateGradientSolver, PreConditionedConjugateGradientSolver, nystrom_preconditioner
    from F3M_src.FFM_classes import FFM
    g = torch.Generator().manual_seed(0)
    X = torch.rand(6000, 3, generator=g)
    b = torch.randn(6000, 2, generator=g).to(cuda)
    ls, lamb = 0.3, 5.0        # well conditioned: the products carry an interpolation error of ~1e-5
    op = FFM(X, ls=ls, min_points=200, nr_of_interpolation=125, small_field_points=125, device="cuda:0")
    a, alphas, betas = ConjugateGradientSolver("torch", op, b, lamb=lamb, eps=1e-7, max_its=300)
    Xd = X.double().to(cuda)
    K = torch.exp(-torch.cdist(Xd, Xd).pow(2) / (2 * ls * ls)) + lamb * torch.eye(6000, device=cuda, dtype=torch.float64)
    exact = torch.linalg.solve(K, b.double())
    assert rel_l2(a.cpu(), exact.cpu()) <= 1e-3
    assert alphas.shape[1] == 2 and alphas.shape == betas.shape and alphas.shape[0] >= 3
    pre = nystrom_preconditioner(op.X, m_fac=2.0, lamb=lamb, generator=torch.Generator().manual_seed(1))
    pre.calculate_constants_gaussian(ls)
    u, _, _ = PreConditionedConjugateGradientSolver("torch", pre, op, b, lamb=lamb, eps=1e-7, max_its=300)
    assert rel_l2(u.cpu(), exact.cpu()) <= 1e-3


def test_falkon_matches_direct_nystrom_solve(cuda):
    from conjugate_gradient.custom_gaussian_kernel import custom_GaussianKernel, Falkon
    g = torch.Generator().manual_seed(3)
    n, m, ls, lam = 40000, 300, 0.4, 1e-3
    X = torch.rand(n, 3, generator=g)
    y = (torch.sin(4 * X[:, 0]) * torch.cos(3 * X[:, 1]) + X[:, 2] ** 2 + 0.1 * torch.randn(n, generator=g))[:, None]
    kern = custom_GaussianKernel(ls, min_points=500, var_compression=False, interpolation_nr=125)
    model = Falkon(kern, penalty=lam, M=m, maxiter=40, seed=5).fit(X, y)
    # dense float64 solve of (K_nm^T K_nm + lam n K_mm) alpha = K_nm^T y with the same centres
    C = model.ny_points_.double()
    Xd, yd = X.double().to(cuda), y.double().to(cuda)
    Knm = torch.exp(-torch.cdist(Xd, C).pow(2) / (2 * ls * ls))
    Kmm = torch.exp(-torch.cdist(C, C).pow(2) / (2 * ls * ls))
    H = Knm.t() @ Knm + lam * n * Kmm
    alpha = torch.linalg.solve(H, Knm.t() @ yd)
    Xt = torch.rand(5000, 3, generator=g)
    pred_exact = torch.exp(-torch.cdist(Xt.double().to(cuda), C).pow(2) / (2 * ls * ls)) @ alpha
    pred = model.predict(Xt)
    assert rel_l2(pred.cpu(), pred_exact.cpu()) <= 1e-2
    truth = (torch.sin(4 * Xt[:, 0]) * torch.cos(3 * Xt[:, 1]) + Xt[:, 2] ** 2)[:, None]
    assert rel_l2(pred.cpu(), truth) <= 1e-1       # it actually learns the function
