"""`moe4` of the reference (runtime/tier/moe4/moe4.cu:916-925): decode kernels, scratch, combine, dequant."""
from ..moe import HmoeError
from ..moe import moe4_combine as combine
from ..moe import moe4_dequant as dequant
from ..moe import moe4_forward as forward
from ..moe import moe4_scratch as scratch

__all__ = ["forward", "scratch", "combine", "dequant", "handoff", "stage"]


def handoff(*args, **kwargs):
    raise HmoeError("moe4.handoff: the mailbox hand-off to the reference's other processors has no counterpart here")


def stage(*args, **kwargs):
    raise HmoeError("moe4.stage: host staging for the reference's other processors has no counterpart here")
