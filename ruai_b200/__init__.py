"""ruai_b200: the quantized-inference path of ruai on B200 (sm_100a).

`ruai_b200.nn` mirrors the reference's `ruai::nn` names for this path; the work
is done by libruai_b200.so (csrc/, C ABI in include/ruai_b200.h).
"""
from . import _lib, nn  # noqa: F401
from ._lib import RuaiError  # noqa: F401

__all__ = ["nn", "RuaiError"]
