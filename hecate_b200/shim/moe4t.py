"""`moe4t` of the reference (runtime/tier/moe4/moe4t.cu:526-530): tcgen05 prefill kernels and their scratch."""
from ..moe import HmoeError
from ..moe import moe4t_forward as forward
from ..moe import moe4t_scratch as scratch

__all__ = ["forward", "scratch", "gemm"]


def gemm(*args, **kwargs):
    raise HmoeError("moe4t.gemm: the reference's single raw grouped GEMM (a test entry) is not provided; forward() runs both fused GEMMs")
