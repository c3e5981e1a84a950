"""Solvers that consume the KMVM operator: conjugate gradients and FALKON kernel ridge regression.

They mirror the callers of the reference:

  ConjugateGradientSolver / PreConditionedConjugateGradientSolver / nystrom_preconditioner
      conjugate_gradient/conjugate_gradient.py:91-208   (same arguments and return values; the unused
      `binding` argument is kept so that existing call sites run unchanged)
  F3MGaussianKernel.mmv / dmmv
      conjugate_gradient/custom_gaussian_kernel.py:45-89 (custom_GaussianKernel.mmv_ / dmmv_)
  Falkon
      conjugate_gradient/custom_falkon.py:119-244 with the solver of
      conjugate_gradient/custom_conjugate_gradient_falkon.py:45-189.

The reference takes centre selection, the preconditioner and the CG loop from the third-party `falkon`
package, which is not part of it; here they are written out from the formulas in the reference's own
docstring (custom_conjugate_gradient_falkon.py:104-114): preconditioner B = n^(-1/2) T^-1 A^-1 with
K_mm = T^T T and A^T A = T T^T / m + lambda I, system B^T H B beta = B^T K_nm^T y / n with
H = K_nm^T K_nm / n + lambda K_mm.  Results of this class are checked against a direct float64 solve of
the same normal equations, not against `falkon` itself.

The trees of K_nm and K_mn are built once and reused by every CG iteration (the reference rebuilds them
in every product and splits K_mn into 48 chunked products, custom_gaussian_kernel.py:85).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch

from .FFM_classes import FFM


# ------------------------------------------------------------------------------------------------
# conjugate gradients on  (K + lamb I) a = b
# ------------------------------------------------------------------------------------------------
def ConjugateGradientSolver(binding, kmvm_object, b, lamb=1e-2, eps=1e-6, max_its=1000, verbose=False):
    """Plain CG, one system per column of b (conjugate_gradient.py:172-208).  Returns (a, alphas, betas);
    the step sizes feed the Lanczos log-determinant estimate of get_GP_likelihood."""
    def linop(p):
        return kmvm_object @ p + lamb * p

    a = torch.zeros_like(b)
    r = b.clone()
    nr2 = (r ** 2).mean(dim=0, keepdim=True)
    p = r.clone()
    scale = b.abs().sum(dim=0, keepdim=True)
    alphas, betas = [], []
    for _ in range(max_its):
        Mp = linop(p)
        alp = nr2 / (p * Mp).mean(dim=0, keepdim=True)
        a += alp * p
        r -= alp * Mp
        err = (r.abs().sum(dim=0, keepdim=True) / scale).mean().item()
        if verbose:
            print(err)
        if err < eps:
            break
        nr2new = (r ** 2).mean(dim=0, keepdim=True)
        beta = nr2new / nr2
        p = r + beta * p
        nr2 = nr2new
        alphas.append(alp)
        betas.append(beta)
    A = torch.cat(alphas, 0) if alphas else torch.zeros(0, b.shape[1], device=b.device)
    B = torch.cat(betas, 0) if betas else torch.zeros(0, b.shape[1], device=b.device)
    return a, A, B


def subsample_inducing_points(X, m_fac=1.0, generator=None):
    m = int(round(m_fac * X.shape[0] ** 0.5))
    idx = torch.randperm(X.shape[0], generator=generator)[:m]
    return X[idx.to(X.device)].clone()


def _gaussian(A, B, ls):
    return torch.exp(-torch.cdist(A, B).pow(2) / (2 * ls * ls))


def _gaussian_blocked(C, ls, dtype, rows=8192):
    """K(C, C) in `dtype`, filled block of rows by block of rows (distances in float64) so that no second m x m array
    exists while it is built."""
    m = C.shape[0]
    K = torch.empty(m, m, device=C.device, dtype=dtype)
    Cd = C.double()
    for s0 in range(0, m, rows):
        K[s0:s0 + rows] = _gaussian(Cd[s0:s0 + rows], Cd, ls).to(dtype)
    return K


class nystrom_preconditioner:
    """P = lamb I + K_nm K_mm^-1 K_mn applied through the Woodbury identity (conjugate_gradient.py:91-109)."""

    def __init__(self, X, m_fac=1.0, lamb=1e-2, generator=None):
        self.X = X
        self.x_m = subsample_inducing_points(X, m_fac, generator)
        self.lamb = lamb

    def calculate_constants(self, memory_kernel: Callable):
        """memory_kernel(A, B) returns the dense kernel block (a tensor, or an object with .evaluate())."""
        def dense(A, B):
            k = memory_kernel(A, B)
            return k.evaluate() if hasattr(k, "evaluate") else k
        # float64: K_mm of a smooth kernel is close to singular, a float32 inverse of the sum is not usable
        k_xm = dense(self.X, self.x_m).double()
        self.small_in_mem = dense(self.x_m, self.x_m).double() + k_xm.t() @ k_xm / self.lamb
        self.inside_inverse = torch.linalg.inv(self.small_in_mem)

    def calculate_constants_gaussian(self, ls: float):
        self.calculate_constants(lambda A, B: _gaussian(A, B, ls))

    def apply_predcond(self, ffm_obj, b):
        right = ffm_obj.forward(self.x_m, self.X, b) / self.lamb
        mid = (self.inside_inverse @ right.double()).float()
        left = ffm_obj.forward(self.X, self.x_m, mid)
        return (b - left) / self.lamb


def PreConditionedConjugateGradientSolver(binding, preconditioner, kmvm_object, b, lamb=1e-3, eps=1e-6, max_its=1000,
                                          verbose=False):
    """Preconditioned CG (conjugate_gradient.py:111-141); returns (u, alphas, betas)."""
    def linop(p):
        return kmvm_object @ p + lamb * p

    u = torch.zeros_like(b)
    r = b.clone()
    z = preconditioner.apply_predcond(ffm_obj=kmvm_object, b=r)
    d = z.clone()
    scale = b.abs().sum().item()
    nz2 = (z * r).mean(dim=0, keepdim=True)
    alphas, betas = [], []
    for _ in range(max_its):
        err = (r.abs().sum() / scale).item()
        if verbose:
            print(err)
        if err < eps:
            break
        v = linop(d)
        alp = nz2 / (d * v).mean(dim=0, keepdim=True)
        u += alp * d
        r -= alp * v
        z = preconditioner.apply_predcond(ffm_obj=kmvm_object, b=r)
        nz2new = (z * r).mean(dim=0, keepdim=True)
        beta = nz2new / nz2
        d = z + beta * d
        nz2 = nz2new.clone()
        alphas.append(alp)
        betas.append(beta)
    A = torch.cat(alphas, 0) if alphas else torch.zeros(0, b.shape[1], device=b.device)
    B = torch.cat(betas, 0) if betas else torch.zeros(0, b.shape[1], device=b.device)
    return u, A, B


def build_tridiagonalization_matrices(alphas, betas):
    """Lanczos tridiagonal matrices of the CG run, one per column (conjugate_gradient.py:155-170): with step lengths
    a_k and ratios b_k of one column, T has diagonal 1/a_k + b_{k-1}/a_{k-1} (second term absent for k = 0) and
    off-diagonal sqrt(b_k)/a_k, k >= 1.  All columns are assembled at once as a batch."""
    a, b = alphas.t(), betas.t()                                  # (columns, iterations)
    k = a.shape[1]
    diag = a.reciprocal()
    if k > 1:
        diag[:, 1:] += torch.nan_to_num(b[:, 1:] / a[:, 1:], nan=0.0)     # b and a of iteration k, as the reference pairs them
        off = b[:, 1:].sqrt() / a[:, 1:]
    T = torch.diag_embed(diag)
    if k > 1:
        T = T + torch.diag_embed(off, offset=1) + torch.diag_embed(off, offset=-1)
    return T


def calculate_log_kxx(T_list):
    """Mean over the columns of the log of the largest Ritz value (conjugate_gradient.py:143-147)."""
    return torch.linalg.eigvalsh(T_list)[:, -1].log().mean().item()


def get_GP_likelihood(alpha, y, alpha_mat, beta_mat):
    """conjugate_gradient.py:149-153: spectral term of the Lanczos matrices minus the data fit alpha . y."""
    spectral = calculate_log_kxx(build_tridiagonalization_matrices(alpha_mat, beta_mat))
    return spectral - float((alpha * y).sum())


# ------------------------------------------------------------------------------------------------
# FALKON
# ------------------------------------------------------------------------------------------------
class F3MGaussianKernel:
    """K(X1, X2) v and K(X1, X2)^T (K(X1, X2) v + w) with the treecode (custom_gaussian_kernel.py:45-89).
    Defaults follow custom_GaussianKernel: var_compression on, small_field_points = interpolation_nr,
    min_points = 4^d."""

    def __init__(self, sigma: float, min_points: Optional[float] = None, var_compression: bool = True,
                 interpolation_nr: int = 64, eff_var_limit: float = 0.3, device="cuda:0"):
        self.ls = float(sigma)
        self.min_points = min_points
        self.var_compression = var_compression
        self.interpolation_nr = interpolation_nr
        self.eff_var_limit = eff_var_limit
        self.device = device
        self._nm = None      # K(X1, X2)
        self._mn = None      # K(X2, X1)
        self._key = None

    def _operators(self, X1, X2):
        # The key holds the caller's tensors themselves (identity, not address: an address can be recycled by another
        # tensor of the same shape once the first is freed) and every parameter the operators are built with.
        key = (X1, X1._version, X2, X2._version, self.ls, self.min_points, self.interpolation_nr, self.var_compression,
               self.eff_var_limit)
        same = self._key is not None and len(self._key) == len(key) and all(
            (a is b) if torch.is_tensor(a) else (a == b) for a, b in zip(self._key, key))
        if not same:
            mp = self.min_points if self.min_points is not None else 4 ** X1.shape[1]
            kw = dict(ls=self.ls, min_points=mp, nr_of_interpolation=self.interpolation_nr, eff_var_limit=self.eff_var_limit,
                      var_compression=self.var_compression, small_field_points=self.interpolation_nr, device=self.device)
            self._nm = FFM(X1, X2, **kw)
            self._mn = FFM(self._nm.Y, self._nm.X, **kw)
            self._key = key
        return self._nm, self._mn

    def mmv(self, X1, X2, v):
        nm, _ = self._operators(X1, X2)
        return nm @ v

    def dmmv(self, X1, X2, v, w):
        """K^T (K v + w); v or w may be None (dmmv_, custom_gaussian_kernel.py:57-89)."""
        nm, mn = self._operators(X1, X2)
        if v is None:
            res = w.float().to(self.device)
        else:
            res = nm @ v
            if w is not None:
                res = res + w.float().to(self.device)
        return mn @ res


class Falkon:
    """Nystrom kernel ridge regression solved with preconditioned CG (custom_falkon.py:119-244)."""

    def __init__(self, kernel: F3MGaussianKernel, penalty: float, M: int, maxiter: int = 20, seed: int = 0,
                 jitter: float = 1e-6):
        self.kernel, self.penalty, self.M, self.maxiter, self.seed, self.jitter = kernel, penalty, M, maxiter, seed, jitter
        self.alpha_ = None
        self.ny_points_ = None

    def fit(self, X: torch.Tensor, Y: torch.Tensor):
        dev = self.kernel.device
        X = X.float().to(dev)
        Y = Y.float().to(dev)
        if Y.dim() == 1:
            Y = Y[:, None]
        n, m = X.shape[0], self.M
        g = torch.Generator().manual_seed(self.seed)
        C = X[torch.randperm(n, generator=g)[:m].to(dev)].contiguous()
        ls, lam = self.kernel.ls, self.penalty
        # preconditioner: K_mm = T^T T,  A^T A = T T^T / m + lambda I.  Two m x m factors are kept; they are float64 up
        # to m = 20000 and float32 beyond (m = 1e5: 2 x 40 GB instead of 2 x 80 GB, which would leave no room for the
        # products), and every m x m step reuses the buffer of its input.
        fdt = torch.float64 if m <= 20000 else torch.float32
        T = _gaussian_blocked(C, ls, fdt)
        T.diagonal().add_(self.jitter * m)
        torch.linalg.cholesky(T, upper=True, out=T)
        T.triu_()
        A = torch.empty_like(T)
        torch.mm(T, T.t(), out=A)
        A.div_(m)
        A.diagonal().add_(lam)
        torch.linalg.cholesky(A, upper=True, out=A)
        A.triu_()
        solve_tri = torch.linalg.solve_triangular

        def solve(M_, v, upper):   # right-hand sides stay float64; the factor's precision is the preconditioner's
            return solve_tri(M_, v.to(fdt), upper=upper).double()
        invT = lambda v: solve(T, v, True)
        invTt = lambda v: solve(T.t(), v, False)
        invA = lambda v: solve(A, v, True)
        invAt = lambda v: solve(A.t(), v, False)

        def op(beta):   # falkon_mmv (custom_conjugate_gradient_falkon.py:144-160)
            v = invA(beta)
            cc = self.kernel.dmmv(X, C, invT(v).float(), None).double() / n
            return invAt(invTt(cc) + lam * v)

        rhs = invAt(invTt(self.kernel.dmmv(X, C, None, Y / n).double()))
        beta = torch.zeros_like(rhs)
        r = rhs.clone()
        p = r.clone()
        rs = (r * r).sum(0, keepdim=True)
        for _ in range(self.maxiter):
            Ap = op(p)
            alp = rs / (p * Ap).sum(0, keepdim=True)
            beta += alp * p
            r -= alp * Ap
            rs_new = (r * r).sum(0, keepdim=True)
            p = r + (rs_new / rs) * p
            rs = rs_new
        self.alpha_ = invT(invA(beta)).float()
        self.ny_points_ = C
        return self

    def predict(self, X: torch.Tensor) -> torch.Tensor:
        X = X.float().to(self.kernel.device)
        pred = FFM(X, self.ny_points_, ls=self.kernel.ls, min_points=self.kernel.min_points or 4 ** X.shape[1],
                   nr_of_interpolation=self.kernel.interpolation_nr, eff_var_limit=self.kernel.eff_var_limit,
                   var_compression=self.kernel.var_compression, small_field_points=self.kernel.interpolation_nr,
                   device=self.kernel.device)
        return pred @ self.alpha_
