"""`cn` of the reference (runtime/tier/cn.cu:190-232): the combine fused into the next layer's input norm."""
from ..moe import HmoeError
from ..moe import combine_norm

__all__ = ["combine_norm", "combine_norm_pdl"]


def combine_norm_pdl(*args, **kwargs):
    raise HmoeError("cn.combine_norm_pdl: its CPU / RTX done flags have no counterpart here; use combine_norm")
