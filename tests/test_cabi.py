"""The C ABI library loads without a GPU and exports every function that include/hecate_moe.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "hecate_moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hmoe_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_all_declared_symbols():
    from hecate_b200 import _lib
    L = _lib.lib()
    names = declared_functions()
    assert "hmoe_decode" in names and "hmoe_router" in names and len(names) >= 10
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/hecate_moe.h but not exported"


def test_host_only_entry_points():
    from hecate_b200 import _lib
    L = _lib.lib()
    assert L.hmoe_version() >= 100
    assert L.hmoe_decode_ws_bytes(ctypes.c_int(6144), ctypes.c_int(2048)) > 4_000_000
    assert L.hmoe_router_ws_bytes(ctypes.c_int(16), ctypes.c_int(256)) >= 16 * 256 * 4
    # the built-in scratch of hmoe_decode_noalloc is 5 MiB: the benchmark shape fits, the next larger ones do not
    five = 5 << 20
    assert L.hmoe_decode_ws_bytes(ctypes.c_int(6144), ctypes.c_int(2048)) <= five
    assert L.hmoe_decode_ws_bytes(ctypes.c_int(6144), ctypes.c_int(2304)) > five
    assert L.hmoe_decode_ws_bytes(ctypes.c_int(8192), ctypes.c_int(2304)) > five
    # argument errors are reported as codes with a message, never thrown
    rc = L.hmoe_combine(None, None, None, ctypes.c_int64(4), None, None)
    assert rc == 1 and b"hmoe_combine" in L.hmoe_last_error()


def test_forward_workspace_covers_every_path():
    """hmoe_forward's workspace is sized for the largest of the three paths it may take for up to R rows; the short path takes
    1..640 rows and the dispatcher hands over to the grouped GEMMs somewhere between the decode limit and that."""
    from hecate_b200 import _lib
    L = _lib.lib()
    ci = ctypes.c_int
    H, I = 6144, 2048
    short = lambda r: L.hmoe_short_prefill_ws_bytes(ci(r), ci(H), ci(I), ci(8))
    fwd = lambda r, q=0: L.hmoe_forward_ws_bytes(ci(r), ci(8), ci(256), ci(H), ci(I), ci(q))
    assert short(0) == 0 and short(641) == 0 and short(640) > short(64) > short(1) > 0
    assert short(64) >= 64 * 9 * 2 * I * 4                       # the per-pick gate / up sums
    limit = L.hmoe_forward_short_rows()
    assert 16 < limit <= 640
    assert fwd(0) == 0
    assert fwd(16) >= L.hmoe_decode_ws_bytes(ci(H), ci(I))
    assert fwd(limit) >= short(limit) and fwd(100) >= short(100)
    for r in (16, 100, limit, 4096):
        for q in (0, 1):
            assert fwd(r, q) >= L.hmoe_prefill_ws_bytes(ci(r), ci(8), ci(256), ci(H), ci(I), ci(q))
    assert fwd(4096) >= fwd(limit) >= fwd(17) >= fwd(16)          # one workspace serves every smaller call
    # argument errors come back as codes before anything touches a device
    st = _lib.LayerStruct()
    st.H, st.I, st.n_experts, st.topk, st.group, st.scale_dtype = H, I, 1, 8, 0, 2
    assert L.hmoe_forward(ctypes.byref(st), None, 0, None, None, 0, 0, 1, 0, None, None, ctypes.c_size_t(0), None) == 1
    assert L.hmoe_short_prefill(ctypes.byref(st), None, 0, None, None, 641, 0, 1, 0, None, None, ctypes.c_size_t(0), None) == 1
    assert b"hmoe_short_prefill" in L.hmoe_last_error()


def test_noalloc_size_check_needs_no_gpu():
    """Shapes beyond the built-in scratch are refused before anything touches a device."""
    from hecate_b200 import _lib
    L = _lib.lib()
    st = _lib.LayerStruct()
    st.H, st.I, st.n_experts, st.topk, st.group, st.scale_dtype = 6144, 2304, 1, 8, 0, 2
    rc = L.hmoe_decode_noalloc(ctypes.byref(st), None, 0, None, None, 1, 0, 1, 0, None, None, None)
    assert rc == 4 and b"built-in scratch" in L.hmoe_last_error()


def test_layer_struct_matches_header():
    from hecate_b200 import _lib
    assert ctypes.sizeof(_lib.LayerStruct) == 6 * 4 + 12 * 8 + 8          # six ints, twelve pointers, shared_format + padding
    assert _lib.LayerStruct.shared_format.offset == 6 * 4 + 12 * 8
