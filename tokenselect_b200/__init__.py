"""tokenselect_b200: decode-time token selection + sparse paged attention as sm_100a CUDA kernels
behind a C ABI (``include/tokenselect_b200.h``), with the host-side mirror of the reference patcher's
decode surface.  No CPU path: the CUDA library is required."""
from .engine import TokenSelectConfig, TokenSelectEngine, rotary_tables  # noqa: F401
from ._lib import TokenSelectError, TS_FLAG_DENSE, TS_FLAG_RECOMPUTE, TS_FLAG_REUSE  # noqa: F401

__all__ = ["TokenSelectConfig", "TokenSelectEngine", "TokenSelectError", "rotary_tables",
           "TS_FLAG_DENSE", "TS_FLAG_RECOMPUTE", "TS_FLAG_REUSE"]
