"""ny_b200: B200 (sm_100a) engine for ny's IBP / CROWN / beta-CROWN bound-propagation path.

The numeric work is done by hand-written CUDA kernels behind the C ABI in include/nyb200.h;
this package is the Python host mirror of ny's engine interface over that ABI.
"""
from .engine import B200Engine, Conv2d, ConvTransposeParams, EngineError, SPLIT_DTYPE, Network, lower_projection_block  # noqa: F401
