"""Module with the function table of the reference's extension `ffm_3d_float`
(F3M_src/pybinder_setup.cu:17-73): FFM_XY_FLOAT_d, rbf_float_d, rbf_double_d, rbf_float_d_grad for
d = 1..5, same positional arguments, running on libf3m.so.  Code that imports the extension
directly (`import ffm_3d_float as load_obj`, experiments/FFM_classes.py:6) keeps working."""
from __future__ import annotations

from . import engine


def _ffm_xy(X, Y, b, device, ls, min_points, nr_of_interpolation, var_compression, eff_var_limit, small_field_limit):
    prm = engine.make_params(ls, min_points, nr_of_interpolation, var_compression, eff_var_limit, small_field_limit)
    return engine.kmvm(X, None if engine.is_shared(X, Y) else Y, b, prm)


def _rbf(X, Y, b, ls, shared=True):
    return engine.rbf_dense(X, Y, b, ls)


def _rbf_grad(X, Y, b, ls, shared=True):
    return engine.rbf_dense(X, Y, b, ls, grad=True)


def _dim_checked(fn, d):
    def call(X, *a, **k):
        if X.shape[1] != d:
            raise ValueError(f"expected {d}-dimensional points, got {X.shape[1]}")
        return fn(X, *a, **k)
    return call


for _d in range(1, 6):
    globals()[f"FFM_XY_FLOAT_{_d}"] = _dim_checked(_ffm_xy, _d)
    globals()[f"rbf_float_{_d}"] = _dim_checked(_rbf, _d)
    globals()[f"rbf_double_{_d}"] = _dim_checked(_rbf, _d)
    globals()[f"rbf_float_{_d}_grad"] = _dim_checked(_rbf_grad, _d)
