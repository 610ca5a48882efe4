"""ctypes binding of libhecate_moe_b200.so (the C ABI declared in include/hecate_moe.h).

There is no fallback: if the library is missing it is built with nvcc, and if it cannot be loaded the import of any
compute entry point raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# HECATE_MOE_LIB selects another build of the same library (e.g. a debug or experimental build)
LIB_PATH = os.environ.get("HECATE_MOE_LIB") or os.path.join(_HERE, "csrc", "libhecate_moe_b200.so")
_lib = None

F16, BF16, F32, F16_FRAG = 0, 1, 2, 3


class HmoeError(RuntimeError):
    pass


class LayerStruct(C.Structure):
    _fields_ = [("H", C.c_int32), ("I", C.c_int32), ("n_experts", C.c_int32), ("topk", C.c_int32),
                ("group", C.c_int32), ("scale_dtype", C.c_int32)] + \
               [(n, C.c_void_p) for n in ("gate_w", "up_w", "down_w", "gate_s", "up_s", "down_s",
                                          "sh_gate_w", "sh_up_w", "sh_down_w", "sh_gate_s", "sh_up_s", "sh_down_s")] + \
               [("shared_format", C.c_int32)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            from .csrc import build
            build.build()
        L = C.CDLL(LIB_PATH)
        L.hmoe_last_error.restype = C.c_char_p
        L.hmoe_launch_count.restype = C.c_int64
        for n in ("hmoe_router_ws_bytes", "hmoe_decode_ws_bytes", "hmoe_prefill_ws_bytes", "hmoe_permute_ws_bytes", "hmoe_prefill_sorted_ws_bytes",
                  "hmoe_ep_stage_bytes", "hmoe_prefill_ep_stage_bytes", "hmoe_short_prefill_ws_bytes", "hmoe_forward_ws_bytes"):
            getattr(L, n).restype = C.c_size_t
        _lib = L
    return _lib


def check(rc):
    if rc != 0:
        raise HmoeError(f"hecate_moe error {rc}: {lib().hmoe_last_error().decode()}")


def vp(x):
    """device/host pointer argument from an int, a tensor (data_ptr) or None"""
    if x is None:
        return C.c_void_p(0)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    return C.c_void_p(int(x))
