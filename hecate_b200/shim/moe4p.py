"""`moe4p` of the reference (runtime/tier/moe4/moe4p.cu:220-245): mid-size prefill. The same tcgen05 kernels serve every row count."""
from ..moe import moe4p_forward as forward
from ..moe import moe4p_scratch as scratch

__all__ = ["forward", "scratch"]
