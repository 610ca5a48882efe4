"""TEST INFRASTRUCTURE: python face of the CPU checker (oracle/hmoe_oracle.cpp) and of the reference engine build.

Only tests, the smoke test and the benchmark's CPU-baseline leg import this module. The shipped package never does.
"""
import ctypes as C
import importlib.util
import os
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


class _Expert(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("g", "u", "d", "gs", "us", "ds")]


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "hmoe_oracle.so")
        if not os.path.exists(path):
            from . import build
            build.build_oracle()
        L = C.CDLL(path)
        L.orc_moe_forward.restype = C.c_int
        L.orc_router.restype = C.c_int
        L.orc_row_blocks.restype = C.c_int
        L.orc_threads.restype = C.c_int
        L.orc_det_expf.restype = C.c_float
        L.orc_det_expf.argtypes = [C.c_float]
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def unpack_rowmajor(q, N, K):
    q = np.ascontiguousarray(q, dtype=np.uint8)
    out = np.empty(N * K // 2, dtype=np.uint8)
    lib().orc_unpack_u4(_p(q), C.c_int(N), C.c_int(K), _p(out))
    return out.reshape(N, K // 2)


def pack_from_rowmajor(rm, N, K):
    rm = np.ascontiguousarray(rm, dtype=np.uint8)
    out = np.empty(N * K // 2, dtype=np.uint8)
    lib().orc_pack_u4(_p(rm), C.c_int(N), C.c_int(K), _p(out))
    return out


def q8_roundtrip(v):
    v = np.ascontiguousarray(v, dtype=np.float32)
    out = np.empty_like(v)
    lib().orc_q8_roundtrip(_p(v), C.c_int(v.size), _p(out))
    return out


class Expert:
    """Host copy of one expert for the checker: row-major nibbles + fp32 scales [K/G][N]."""

    def __init__(self, gq, uq, dq, gs, us, ds, H, I, packed=True):
        f = (lambda q, N, K: unpack_rowmajor(q, N, K)) if packed else (lambda q, N, K: np.ascontiguousarray(q, dtype=np.uint8))
        self.g, self.u, self.d = f(gq, I, H), f(uq, I, H), f(dq, H, I)
        self.gs, self.us, self.ds = (np.ascontiguousarray(s, dtype=np.float32) for s in (gs, us, ds))

    def struct(self):
        return _Expert(*(a.ctypes.data for a in (self.g, self.u, self.d, self.gs, self.us, self.ds)))


def moe_forward(H, I, G, x_f16, sel, rw_f16, lo, experts, shared=None, mode=0, topk=None):
    """x_f16 [R][H] float16, sel int64 [R][topk], rw float16 [R][topk]; experts = list of Expert for ids lo.. .
    mode 0 = reference arithmetic (int8 activations), 1 = exact. Returns float32 [R][H]."""
    x = np.ascontiguousarray(x_f16, dtype=np.float16)
    sel = np.ascontiguousarray(sel, dtype=np.int64)
    rw = np.ascontiguousarray(rw_f16, dtype=np.float16)
    R = x.shape[0]
    topk = sel.shape[1] if topk is None else topk
    arr = (_Expert * max(1, len(experts)))(*[e.struct() for e in experts])
    sh = shared.struct() if shared is not None else None
    out = np.zeros((R, H), dtype=np.float32)
    rc = lib().orc_moe_forward(C.c_int(H), C.c_int(I), C.c_int(G), C.c_int(R), C.c_int(topk), _p(x), _p(sel), _p(rw), C.c_int(lo),
                               C.c_int(len(experts)), arr, C.byref(sh) if sh is not None else None, C.c_int(mode), _p(out))
    if rc:
        raise ValueError(f"oracle: bad shape (rc {rc})")
    return out


def router(x_bits, x_bf16, wt_bits, w_bf16, bias, topk, scale, want_logits=False):
    """x_bits uint16 [R][K], wt_bits uint16 [E][K] (fp16 or bf16 bit patterns). Returns sel int64, rw float16 (, logits)."""
    x = np.ascontiguousarray(x_bits, dtype=np.uint16)
    w = np.ascontiguousarray(wt_bits, dtype=np.uint16)
    R, K = x.shape
    E = w.shape[0]
    b = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
    sel = np.empty((R, topk), dtype=np.int64)
    rw = np.empty((R, topk), dtype=np.uint16)
    lg = np.empty((R, E), dtype=np.float32) if want_logits else None
    rc = lib().orc_router(_p(x), C.c_int(int(x_bf16)), _p(w), C.c_int(int(w_bf16)), _p(b) if b is not None else None, C.c_int(R),
                          C.c_int(K), C.c_int(E), C.c_int(topk), C.c_float(scale), _p(sel), _p(rw), _p(lg) if lg is not None else None)
    if rc:
        raise ValueError("oracle router: bad shape")
    return (sel, rw.view(np.float16), lg) if want_logits else (sel, rw.view(np.float16))


def permute(sel, rw_f16, E):
    sel = np.ascontiguousarray(sel, dtype=np.int64)
    rw = np.ascontiguousarray(rw_f16, dtype=np.float16)
    R, topk = sel.shape
    n = R * topk
    order, tok, eid = (np.empty(n, dtype=np.int32) for _ in range(3))
    wt = np.empty(n, dtype=np.float32)
    counts = np.empty(E, dtype=np.int32)
    lib().orc_permute(_p(sel), _p(rw), C.c_int(R), C.c_int(topk), C.c_int(E), _p(order), _p(tok), _p(eid), _p(wt), _p(counts))
    return order, tok, eid, wt, counts


def row_blocks(counts, bm, balance):
    counts = np.ascontiguousarray(counts, dtype=np.int32)
    n = lib().orc_row_blocks(_p(counts), C.c_int(counts.size), C.c_int(bm), C.c_int(int(balance)), None)
    rbt = np.zeros((n, 4), dtype=np.int32)
    lib().orc_row_blocks(_p(counts), C.c_int(counts.size), C.c_int(bm), C.c_int(int(balance)), _p(rbt))
    return rbt


def threads():
    return lib().orc_threads()


# ----------------------------------------------------------------------------------------------------------------------
# The reference CPU engine itself (oracle/_ref, built from the reference's own source by oracle/build.py)

def ref_available(variant="avx2"):
    """Is the reference engine's build `variant` ("avx2", "vnni", "scalar": oracle/build.py) present and runnable on this host?"""
    from . import build
    if variant == "vnni" and not build.host_has_vnni():
        return False
    return os.path.exists(build.ref_module_path(variant))


class RefEngine:
    """Drives the reference engine in its legacy (non-slot) mode the way the reference's own test does
    (tools/dev/test_grace_picks.py:25-42): a 256-byte int32 flag block (ISSUE word 0, meta [layer, rows] at byte 64,
    DONE at byte 128), x fp16 [8][6144], sel int64 [8][8], rw fp16 [8][8], out fp32 [8][6144]. H, I and 8 rows are fixed
    by the engine. One engine per build variant and process (its pool is a singleton of the module)."""
    H, I = 6144, 2048

    def __init__(self, experts, lo, threads=8, core0=0, variant="avx2"):
        import torch
        from . import build
        spec = importlib.util.spec_from_file_location(build.REF_VARIANTS[variant][0], build.ref_module_path(variant))
        self.mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(self.mod)
        self.torch = torch
        T = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        self.keep = [[T(getattr(e, k)) for e in experts] for k in ("g", "u", "d")]
        self.keep += [[T(np.ascontiguousarray(getattr(e, k).reshape(-1))) for e in experts] for k in ("gs", "us", "ds")]
        self.mod.add_layer(0, lo, -1, *self.keep)
        self.flags = torch.zeros(64, dtype=torch.int32)
        self.xs = torch.zeros(8, self.H, dtype=torch.half)
        self.sel = torch.zeros(8, 8, dtype=torch.long)
        self.rw = torch.zeros(8, 8, dtype=torch.half)
        self.out = torch.zeros(8, self.H)
        fp = self.flags.data_ptr()
        self.mod.start(fp, fp + 64, fp + 128, self.xs.data_ptr(), self.sel.data_ptr(), self.rw.data_ptr(), self.out.data_ptr(),
                       threads, core0, 0, 0, 0, 0, 0)
        time.sleep(0.2)
        self.gen = 0
        self.threads = threads

    def job(self, x_f16, sel, rw_f16, timeout=120.0):
        """One job of R <= 8 rows; returns (out float32 [R][H], seconds from ISSUE to DONE)."""
        t = self.torch
        R = x_f16.shape[0]
        self.xs[:R] = t.from_numpy(np.ascontiguousarray(x_f16, dtype=np.float16))
        self.sel[:R] = t.from_numpy(np.ascontiguousarray(sel, dtype=np.int64))
        self.rw[:R] = t.from_numpy(np.ascontiguousarray(rw_f16, dtype=np.float16))
        self.flags[16] = 0
        self.flags[17] = R
        self.gen += 1
        t0 = time.perf_counter()
        self.flags[0] = self.gen
        while int(self.flags[32]) != self.gen:
            if time.perf_counter() - t0 > timeout:
                raise RuntimeError("reference engine job timed out")
        dt = time.perf_counter() - t0
        return self.out[:R].clone().numpy(), dt

    def stop(self):
        self.mod.stop()


def combine_norm(f, o, y, o2, r, w, eps, cbias=0.0, cscale=1.0, threads=1024):
    """CPU restatement of the combine fused into the next input norm (runtime/tier/cn.cu:50-105), float32 throughout and in the
    kernel's order: a = ((f + y) + o) + o2; r' = a + r; per thread t the squares of float4 columns t, t + 1024, ... are added
    with fused multiply-adds (x, y, z, w in turn), the 32 lanes of a warp are summed by a butterfly (xor 16 .. 1), the 32 warp
    sums by a second one; xn = fp16(r' * (w + cbias) * (rsqrt(sum / H + eps) * cscale)). Returns (r', xn, sum of squares).
    f, o, o2 may be None; w float32 [H] (the fp16 / bf16 weight widened). The reciprocal square root here is exact; the GPU's
    is a 2-ulp approximation, so xn may differ in its last bit."""
    y = np.asarray(y, dtype=np.float32)
    rows, H = y.shape
    a = np.zeros_like(y) if f is None else np.asarray(f, dtype=np.float32).copy()
    a = a + y
    if o is not None:
        a = a + np.asarray(o, dtype=np.float32)
    if o2 is not None:
        a = a + np.asarray(o2, dtype=np.float32)
    rn = (a + np.asarray(r, dtype=np.float32)).astype(np.float32)
    cols = H // 4
    sums = np.zeros((rows, threads), dtype=np.float32)
    fma = lambda x, s: (x.astype(np.float64) * x.astype(np.float64) + s.astype(np.float64)).astype(np.float32)
    for k in range((cols + threads - 1) // threads):
        c = np.arange(threads) + k * threads
        ok = c < cols
        for j in range(4):
            x = np.zeros((rows, threads), dtype=np.float32)
            x[:, ok] = rn[:, 4 * c[ok] + j]
            sums = np.where(ok[None, :], fma(x, sums), sums)
    def butterfly(v):                      # v [rows][n_groups][32]
        for off in (16, 8, 4, 2, 1):
            v = (v + v[..., np.arange(32) ^ off]).astype(np.float32)
        return v
    warp = butterfly(sums.reshape(rows, threads // 32, 32))[..., 0]                 # [rows][32 warps]
    total = butterfly(warp.reshape(rows, 1, 32))[:, 0, 0]
    rmf = (np.float32(1.0) / np.sqrt((total / np.float32(H) + np.float32(eps)).astype(np.float32), dtype=np.float32)).astype(np.float32) * np.float32(cscale)
    ww = (np.asarray(w, dtype=np.float32) + np.float32(cbias)).astype(np.float32) if cbias != 0.0 else np.asarray(w, dtype=np.float32)
    xn = ((rn * ww[None, :]).astype(np.float32) * rmf[:, None]).astype(np.float32).astype(np.float16)
    return rn, xn, total
