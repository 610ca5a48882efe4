"""Host-side mirror of the reference's operator surface for the MoE expert path, on top of the C ABI.

The functions keep the names, argument order and meaning of the reference's extension modules so that its dispatcher
(runtime/tier/tier_split.py) could call them unchanged:

    moe4_forward / moe4_scratch / moe4_combine / moe4_dequant   runtime/tier/moe4/moe4.cu:817-911
    router_fused                                                runtime/core/exl3_router.py:134-146

torch is used for device memory and the current stream only. All compute happens in libhecate_moe_b200.so; a missing
library is an error, never a fallback.
"""
import ctypes as C

import torch

from . import _lib
from ._lib import BF16, F16, F16_FRAG, F32, HmoeError, LayerStruct, check, lib, vp

MAX_DECODE_ROWS = 16


def _stream(dev):
    return C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)


def _dt(t):
    if t.dtype == torch.float16:
        return F16
    if t.dtype == torch.bfloat16:
        return BF16
    raise HmoeError(f"expected fp16 or bf16, got {t.dtype}")


def launch_count():
    return int(lib().hmoe_launch_count())


class ExpertTables:
    """The six device pointer tables of one layer's local experts (as tier_split.py:210-214,246 builds them) plus the
    optional shared expert. Keeps the weight tensors alive."""

    def __init__(self, H, I, topk, gate, up, down, gate_s, up_s, down_s, group=0, shared=None, device=None, shared_i8=False):
        dev = device or gate[0].device
        self.H, self.I, self.topk, self.group, self.n = H, I, topk, group, len(gate)
        self.scale_dtype = F32 if group == 0 else BF16
        want = torch.float32 if group == 0 else torch.bfloat16
        for s in list(gate_s) + list(up_s) + list(down_s):
            if s.dtype != want:
                raise HmoeError(f"scales must be {want} for group {group}")
        self.keep = [gate, up, down, gate_s, up_s, down_s, shared]
        tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
        self.tabs = {k: tab(v) for k, v in zip(("gate_w", "up_w", "down_w", "gate_s", "up_s", "down_s"),
                                               (gate, up, down, gate_s, up_s, down_s))}
        self.shared = shared   # (gq, uq, dq, gs, us, ds) tensors or None
        self.shared_i8 = bool(shared_i8)   # shared expert in the reference's int8 format (layout.pack_i8, fp32 row scales)

    def struct(self):
        s = LayerStruct()
        s.H, s.I, s.n_experts, s.topk, s.group, s.scale_dtype = self.H, self.I, self.n, self.topk, self.group, self.scale_dtype
        for k, t in self.tabs.items():
            setattr(s, k, t.data_ptr())
        s.shared_format = 1 if (self.shared is not None and self.shared_i8) else 0
        if self.shared is not None:
            for k, t in zip(("sh_gate_w", "sh_up_w", "sh_down_w", "sh_gate_s", "sh_up_s", "sh_down_s"), self.shared):
                setattr(s, k, t.data_ptr())
        return s


def decode_workspace(H, I, device):
    """Zero-filled scratch of the decode path (the counterpart of moe4.scratch, moe4.cu:897-902)."""
    n = lib().hmoe_decode_ws_bytes(C.c_int(H), C.c_int(I))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def decode(tables, x, sel, rw, y, ws, lo=0, n_local=None, act_quant=False):
    """y[R][H] (fp32) += experts(x) for the rows' selections; R <= 16. Only ids in [lo, lo + n_local) contribute."""
    R = x.shape[0]
    if not (x.is_contiguous() and sel.is_contiguous() and rw.is_contiguous() and y.is_contiguous()):
        raise HmoeError("decode: tensors must be contiguous")
    if sel.dtype != torch.int64 or rw.dtype != torch.float16 or y.dtype != torch.float32:
        raise HmoeError("decode: sel int64, rw fp16, y fp32 required")
    if x.shape[1] != tables.H or sel.shape[1] != tables.topk or y.shape[-1] != tables.H:
        raise HmoeError("decode: shape")
    st = tables.struct()
    check(lib().hmoe_decode(C.byref(st), vp(x), C.c_int(_dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(lo),
                            C.c_int(tables.n if n_local is None else n_local), C.c_int(int(act_quant)), vp(y), vp(ws),
                            C.c_size_t(ws.numel()), _stream(x.device)))
    return y


def prefill_workspace(R, topk, n_local, H, I, device, act_quant=False):
    n = lib().hmoe_prefill_ws_bytes(C.c_int(R), C.c_int(topk), C.c_int(n_local), C.c_int(H), C.c_int(I), C.c_int(int(act_quant)))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def prefill(tables, x, sel, rw, out, ws, lo=0, n_local=None, act_quant=False):
    """out[R][H] (fp32) += experts(x) for any number of rows: permutation on the device, then the two grouped tcgen05 GEMMs
    (the counterpart of tier_split._prefill_gb300 + moe4t.forward, tier_split.py:427-462, moe4t.cu:498-524)."""
    R = x.shape[0]
    if not (x.is_contiguous() and sel.is_contiguous() and rw.is_contiguous() and out.is_contiguous()):
        raise HmoeError("prefill: tensors must be contiguous")
    if sel.dtype != torch.int64 or rw.dtype != torch.float16 or out.dtype != torch.float32:
        raise HmoeError("prefill: sel int64, rw fp16, out fp32 required")
    st = tables.struct()
    check(lib().hmoe_prefill(C.byref(st), vp(x), C.c_int(_dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(lo),
                             C.c_int(tables.n if n_local is None else n_local), C.c_int(int(act_quant)), vp(out), vp(ws),
                             C.c_size_t(ws.numel()), _stream(x.device)))
    return out


def _rows_call(fn, name, tables, x, sel, rw, out, ws, lo, n_local, act_quant):
    R = x.shape[0]
    if not (x.is_contiguous() and sel.is_contiguous() and rw.is_contiguous() and out.is_contiguous()):
        raise HmoeError(name + ": tensors must be contiguous")
    if sel.dtype != torch.int64 or rw.dtype != torch.float16 or out.dtype != torch.float32:
        raise HmoeError(name + ": sel int64, rw fp16, out fp32 required")
    if x.shape[1] != tables.H or sel.shape[1] != tables.topk or out.shape[-1] != tables.H:
        raise HmoeError(name + ": shape")
    st = tables.struct()
    check(fn(C.byref(st), vp(x), C.c_int(_dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(lo),
             C.c_int(tables.n if n_local is None else n_local), C.c_int(int(act_quant)), vp(out), vp(ws),
             C.c_size_t(ws.numel()), _stream(x.device)))
    return out


def short_prefill_workspace(R, H, I, topk, device):
    n = lib().hmoe_short_prefill_ws_bytes(C.c_int(R), C.c_int(H), C.c_int(I), C.c_int(topk))
    if n == 0:
        raise HmoeError("short_prefill_workspace: rows must be 1..640")
    return torch.zeros(n, dtype=torch.uint8, device=device)


def short_prefill(tables, x, sel, rw, out, ws, lo=0, n_local=None, act_quant=False):
    """out[R][H] (fp32) += experts(x) for 1..640 rows through the decode streaming kernels, the whole call as one tile list
    (the counterpart of tier_split._hot_prefill's 8-row chunks of moe4.forward, tier_split.py:341-355)."""
    return _rows_call(lib().hmoe_short_prefill, "short_prefill", tables, x, sel, rw, out, ws, lo, n_local, act_quant)


def forward_short_rows():
    """Calls of 17 .. this many rows take the short path in `forward`."""
    return int(lib().hmoe_forward_short_rows())


def forward_workspace(R, topk, n_local, H, I, device, act_quant=False):
    n = lib().hmoe_forward_ws_bytes(C.c_int(R), C.c_int(topk), C.c_int(n_local), C.c_int(H), C.c_int(I), C.c_int(int(act_quant)))
    if n == 0:
        raise HmoeError("forward_workspace: rows >= 1, topk 1..8")
    return torch.zeros(n, dtype=torch.uint8, device=device)


def forward(tables, x, sel, rw, out, ws, lo=0, n_local=None, act_quant=False):
    """out[R][H] (fp32) += experts(x) for any number of rows; the library picks decode, short prefill or the grouped GEMMs
    by the row count, as tier_submit / _hot_prefill do among the reference's kernels (tier_split.py:341-364,543-546).
    ws: forward_workspace(R_max, ...), good for every call of up to R_max rows."""
    return _rows_call(lib().hmoe_forward, "forward", tables, x, sel, rw, out, ws, lo, n_local, act_quant)


def moe4t_scratch(device, npos, H=6144, I=2048, act_quant=False):
    """moe4t.scratch(device, npos) -> [gu, ar, d] (moe4t.cu:490-495). Here one workspace tensor stands for all three (it holds
    the gathered inputs and the intermediate activations); the other two entries keep call sites that unpack three working."""
    n = lib().hmoe_prefill_sorted_ws_bytes(C.c_int(int(npos)), C.c_int(H), C.c_int(I), C.c_int(int(act_quant)))
    # `ar` and `d` are zero-stride views of one element with the reference's shapes, so call sites that reshape them
    # (d.view(1, ps, H), tier_split.py:459) keep working without the memory
    ar = torch.zeros(1, dtype=torch.float16, device=device).expand(int(npos), I)
    d = torch.zeros(1, dtype=torch.float32, device=device).expand(int(npos), H)
    return [torch.zeros(n, dtype=torch.uint8, device=device), ar, d]


def moe4t_forward(x, tok, eid, wt, rbt, gw, uw, dw, gs, us, ds, gu, ar, d, out, *, I=2048, group=0, act_quant=False):
    """moe4t.forward / moe4p.forward with the reference's argument order (moe4t.cu:498-500): x fp16/bf16 [rows][H], tok / eid
    int32 [npos] and wt fp32 [npos] in sorted-pick order, rbt int32 [nrb][4] on the device, six int64 pointer tables, the
    workspace from moe4t_scratch as `gu` (`ar`, `d` ignored), out fp32 [rows][H] added into. eid is not read: the expert of a
    pick is the expert of its row block."""
    npos, nrb, H = int(tok.numel()), int(rbt.shape[0]), x.shape[1]
    if npos == 0:
        return
    if tok.dtype != torch.int32 or wt.dtype != torch.float32 or rbt.dtype != torch.int32 or out.dtype != torch.float32:
        raise HmoeError("moe4t: shapes")
    s = LayerStruct()
    s.H, s.I, s.n_experts, s.topk, s.group = H, I, int(gw.numel()), 8, group
    s.scale_dtype = F32 if group == 0 else BF16
    for k, t in zip(("gate_w", "up_w", "down_w", "gate_s", "up_s", "down_s"), (gw, uw, dw, gs, us, ds)):
        setattr(s, k, t.data_ptr())
    check(lib().hmoe_prefill_sorted(C.byref(s), vp(x), C.c_int(_dt(x)), vp(tok), vp(wt), vp(rbt.contiguous()), C.c_int(nrb), C.c_int(npos),
                                    C.c_int(int(gw.numel())), C.c_int(int(act_quant)), vp(out), vp(gu), C.c_size_t(gu.numel()),
                                    _stream(x.device)))


moe4p_forward, moe4p_scratch = moe4t_forward, moe4t_scratch


def permute(sel, rw, n_local, lo=0, shared_rows=0, bm=256, balance=True):
    """Device permutation of the picks (stable sort by expert id) and the row-block table. Returns a dict of tensors:
    order, tok, eid, wt, counts, rbt (first `nrb` rows valid), total, nrb."""
    R, topk = sel.shape
    dev = sel.device
    cap = R * topk + shared_rows
    maxrb = cap // bm + n_local + 2
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=dev)
    order, tok, eid, wt = i32(cap), i32(cap), i32(cap), torch.zeros(cap, dtype=torch.float32, device=dev)
    counts, rbt, plan = i32(n_local + 1), i32(maxrb * 4), i32(4)
    nb = lib().hmoe_permute_ws_bytes(C.c_int(R), C.c_int(topk), C.c_int(n_local))
    ws = torch.zeros(nb, dtype=torch.uint8, device=dev)
    check(lib().hmoe_permute(vp(sel), vp(rw), C.c_int(R), C.c_int(topk), C.c_int(lo), C.c_int(n_local), C.c_int(shared_rows),
                             C.c_int(bm), C.c_int(int(balance)), vp(order), vp(tok), vp(eid), vp(wt), vp(counts), vp(rbt), vp(plan), vp(ws),
                             C.c_size_t(nb), _stream(dev)))
    total, nrb = (int(v) for v in plan[:2].cpu())
    return dict(order=order[:total], tok=tok[:total], eid=eid[:total], wt=wt[:total], counts=counts, rbt=rbt.view(-1, 4)[:nrb],
                total=total, nrb=nrb)


def set_profiling(on):
    check(lib().hmoe_set_profiling(C.c_int(int(on))))


def decode_phase_times():
    """ms of (prepare, gate_up, down), averaged over the decode calls made since profiling was switched on (at most the last
    32; waits for them)."""
    out = (C.c_float * 3)()
    check(lib().hmoe_decode_phase_times(out))
    return tuple(out)


def ws_status(ws):
    out = C.c_uint32(0)
    check(lib().hmoe_ws_status(vp(ws), C.byref(out), _stream(ws.device)))
    return out.value


def route_distinct(ws):
    """Diagnostic: the number of distinct routed experts the last decode call on workspace `ws` served on this device (the first
    word of the work list, which follows the 256-byte status block). Synchronises."""
    import torch
    torch.cuda.synchronize(ws.device)
    return int(ws[256:260].view(torch.int32).item())


def route_tiles(ws):
    """Diagnostic: (distinct routed experts, 8-pick tiles) of the work list the last decode or short-prefill call left in `ws`.
    Synchronises."""
    import torch
    torch.cuda.synchronize(ws.device)
    m, nt = ws[256:264].view(torch.int32).tolist()
    return int(m), int(nt)


# ----------------------------------------------------------------------------------------------------------------------
# reference-named entry points

def moe4_scratch(device, H=6144, I=2048):
    """moe4.scratch(device) -> five tensors (moe4.cu:897-902). Only the first is used here (the decode workspace); the
    other four stand in for the reference's gu32 / counters / y32 so call sites can keep unpacking five."""
    e = torch.zeros(1, dtype=torch.int32, device=device)
    return [decode_workspace(H, I, device), e, e, e, e]


def moe4_forward(x, sel, rw, n_hot, gate_w, up_w, down_w, gate_s, up_s, down_s, act, gu32, ctr_a, y32, ctr_b, y, blocks,
                 blocks_a, lo, sh_gw=0, sh_uw=0, sh_dw=0, sh_gs=0, sh_us=0, sh_ds=0, xf=0, *, I=2048, group=0, act_quant=False,
                 shared_i8=False):
    """moe4.forward with the reference's argument order (moe4.cu:828-833,916-920). gate_w .. down_s are int64 device
    tables of pointers; `act` is the workspace from moe4_scratch; gu32, ctr_a, y32, ctr_b, blocks, blocks_a are accepted and
    ignored (this implementation needs no counters and sizes its own grid). Up to 16 rows. The shared expert pointers
    are int4 in the routed experts' format, or with shared_i8 the reference's int8 copies (tier_split.py:495-514). xf = 1: x
    is the fp16 copy in the MMA column order that the reference's norm + router kernel writes (moe4.cu:68-72)."""
    if xf and x.dtype != torch.float16:
        raise HmoeError("moe4_forward: fragment-order input (xf) must be fp16")
    R, H = x.shape
    s = LayerStruct()
    s.H, s.I, s.n_experts, s.topk, s.group = H, I, int(n_hot), sel.shape[1], group
    s.scale_dtype = F32 if group == 0 else BF16
    for k, t in zip(("gate_w", "up_w", "down_w", "gate_s", "up_s", "down_s"), (gate_w, up_w, down_w, gate_s, up_s, down_s)):
        setattr(s, k, t.data_ptr())
    for k, p in zip(("sh_gate_w", "sh_up_w", "sh_down_w", "sh_gate_s", "sh_up_s", "sh_down_s"), (sh_gw, sh_uw, sh_dw, sh_gs, sh_us, sh_ds)):
        setattr(s, k, int(p) or None)
    s.shared_format = 1 if (shared_i8 and sh_gw) else 0
    if sel.dtype != torch.int64 or not sel.is_contiguous():
        raise HmoeError("moe4: selection must be contiguous int64")
    check(lib().hmoe_decode(C.byref(s), vp(x), C.c_int(F16_FRAG if xf else _dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(int(lo)), C.c_int(int(n_hot)),
                            C.c_int(int(act_quant)), vp(y), vp(act), C.c_size_t(act.numel()), _stream(x.device)))


def moe4_combine(f, o_ptr, y, rows, o2_ptr, done_ptr=0):
    """moe4.combine (moe4.cu:817-824): f += y (+ o) (+ o2); y = 0. done_ptr (a flag another device raises) is not
    supported: there is no second device behind this path."""
    if done_ptr:
        raise HmoeError("moe4_combine: done flag not supported")
    if f.dtype != torch.float32 or not f.is_contiguous():
        raise HmoeError("moe4_combine: f must be contiguous fp32")
    n = int(rows) * f.shape[-1]
    check(lib().hmoe_combine(vp(f), vp(o_ptr or None), vp(y), C.c_int64(n), vp(o2_ptr or None), _stream(f.device)))


def combine_norm(f, o_ptr, y, rows, o2_ptr, done_ptr, r, w, xn, eps, cbias=0.0, cscale=1.0):
    """combine_norm (runtime/tier/cn.cu:190-210): the layer's combine fused into the next layer's input norm. f fp32 [rows][H]
    or None; y the accumulator (zeroed here); r fp32 residual, updated in place; w the norm weight (fp16 / bf16 [H]); xn fp16
    out. done_ptr (a flag another device raises) is not supported."""
    if done_ptr:
        raise HmoeError("combine_norm: done flag not supported")
    if r.dtype != torch.float32 or xn.dtype != torch.float16 or not (r.is_contiguous() and xn.is_contiguous() and w.is_contiguous()):
        raise HmoeError("combine_norm: shapes / dtypes")
    Hn = r.shape[-1]
    if w.numel() != Hn or xn.shape[-1] != Hn or y.shape[-1] != Hn:
        raise HmoeError("combine_norm: shapes / dtypes")
    check(lib().hmoe_combine_norm(vp(f), vp(o_ptr or None), vp(y), vp(o2_ptr or None), vp(r), vp(w), C.c_int(_dt(w)), vp(xn), C.c_int(int(rows)),
                                  C.c_int(Hn), C.c_float(eps), C.c_float(cbias), C.c_float(cscale), _stream(r.device)))


def moe4_dequant(q, sc, N, K, group=0):
    """moe4.dequant(q, sc, N, K) -> fp16 [N][K] (moe4.cu:904-911)."""
    out = torch.empty((N, K), dtype=torch.float16, device=q.device)
    check(lib().hmoe_dequant(vp(q), vp(sc), C.c_int(group), C.c_int(F32 if group == 0 else BF16), C.c_int(N), C.c_int(K), vp(out),
                             _stream(q.device)))
    return out


_router_ws = {}


def router_fused(x, wt, bias, logits, ctr, sel, rw, topk, scale):
    """router_fused(x, wt, bias, logits, ctr, sel, rw, topk, scale) (exl3_router.py:134-146). `logits` and `ctr` (the
    reference's self-cleaning scratch) are accepted and ignored; any number of rows."""
    H = x.shape[-1]
    R = x.numel() // H
    E = wt.shape[0]
    need = lib().hmoe_router_ws_bytes(C.c_int(R), C.c_int(E))
    key = (x.device, )
    ws = _router_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _router_ws[key] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=x.device)
    if not (x.is_contiguous() and wt.is_contiguous()):
        raise HmoeError("router_fused: shape / dtype")
    check(lib().hmoe_router(vp(x), C.c_int(_dt(x)), vp(wt), C.c_int(_dt(wt)), vp(bias), C.c_int(R), C.c_int(H), C.c_int(E),
                            C.c_int(int(topk)), C.c_float(float(scale)), vp(sel), vp(rw), vp(ws), C.c_size_t(ws.numel()),
                            _stream(x.device)))
    return sel, rw


def router_decode(tables, x, wt, bias, sel, rw, scale, y, ws, lo=0, n_local=None, act_quant=False):
    """router_fused followed by decode on its output, in three launches instead of four (hmoe_router_decode): what the
    reference's hooks do back to back per layer (routing_fn, then cpu_split_submit). sel / rw are written; y += experts(x)."""
    R, H = x.shape
    E = wt.shape[0]
    need = lib().hmoe_router_ws_bytes(C.c_int(R), C.c_int(E))
    rws = _router_ws.get((x.device, ))
    if rws is None or rws.numel() < need:
        rws = _router_ws[(x.device, )] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=x.device)
    if not (x.is_contiguous() and wt.is_contiguous() and sel.is_contiguous() and rw.is_contiguous() and y.is_contiguous()):
        raise HmoeError("router_decode: tensors must be contiguous")
    if sel.dtype != torch.int64 or rw.dtype != torch.float16 or y.dtype != torch.float32 or H != tables.H or sel.shape[1] != tables.topk:
        raise HmoeError("router_decode: sel int64 [R][topk], rw fp16, y fp32 required")
    st = tables.struct()
    check(lib().hmoe_router_decode(C.byref(st), vp(x), C.c_int(_dt(x)), vp(wt), C.c_int(_dt(wt)), vp(bias), C.c_int(R), C.c_int(E),
                                   C.c_float(float(scale)), vp(sel), vp(rw), vp(rws), C.c_size_t(rws.numel()), C.c_int(lo),
                                   C.c_int(tables.n if n_local is None else n_local), C.c_int(int(act_quant)), vp(y), vp(ws),
                                   C.c_size_t(ws.numel()), _stream(x.device)))
    return y


def norm_route(y, r, w, xn, wt, bias, sel, rw, topk, scale, eps, cbias=0.0, cscale=1.0, r_out=None):
    """Residual add + input norm + router in one launch (the reference's norm_route, runtime/core/exl3_normroute.py:16-65, without
    its hand-off arguments): r' = r + y (y may be None) -> r_out (or dropped), xn = fp16 norm of r', (sel, rw) = router(xn)."""
    H = r.shape[-1]
    R = r.numel() // H
    E = wt.shape[0]
    need = lib().hmoe_router_ws_bytes(C.c_int(R), C.c_int(E))
    ws = _router_ws.get((r.device, ))
    if ws is None or ws.numel() < need:
        ws = _router_ws[(r.device, )] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=r.device)
    if r.dtype != torch.float32 or xn.dtype != torch.float16 or not (r.is_contiguous() and xn.is_contiguous() and wt.is_contiguous() and w.is_contiguous()):
        raise HmoeError("norm_route: shapes / dtypes")
    check(lib().hmoe_norm_router(vp(y), vp(r), vp(r_out), vp(w), C.c_int(_dt(w)), vp(xn), vp(wt), C.c_int(_dt(wt)), vp(bias), C.c_int(R), C.c_int(H),
                                 C.c_int(E), C.c_int(int(topk)), C.c_float(float(scale)), C.c_float(eps), C.c_float(cbias), C.c_float(cscale),
                                 vp(sel), vp(rw), vp(ws), C.c_size_t(ws.numel()), _stream(r.device)))
    return sel, rw


def fill_bytes(t, seed, stream_id):
    """Fill a uint8 tensor (numel % 8 == 0) with the synthetic generator's bytes for (seed, stream_id)."""
    check(lib().hmoe_fill_bytes(vp(t), C.c_size_t(t.numel() * t.element_size()), C.c_uint64(seed), C.c_uint64(stream_id),
                                _stream(t.device)))
    return t
