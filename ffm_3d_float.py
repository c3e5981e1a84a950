"""`import ffm_3d_float` as experiments/FFM_classes.py:6 of the reference writes it."""
from f3m_b200.ffm_3d_float import *  # noqa: F401,F403
import f3m_b200.ffm_3d_float as _m
globals().update({k: v for k, v in vars(_m).items() if k.startswith(("FFM_XY_FLOAT_", "rbf_"))})
