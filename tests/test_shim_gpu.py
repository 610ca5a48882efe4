"""The reference-named modules (hecate_b200.shim: moe4, moe4t, moe4p, cn) called with the argument lists of the reference
dispatcher's own call sites, verbatim: runtime/tier/tier_split.py:352-353 (decode chunk), :563-568 (tier_submit, with and without
the fragment-order input xf), :587 (moe4.combine), :458-459 (moe4t.forward), and runtime/tier/cn.cu:190 (combine_norm).
Results are checked against the CPU checker (exact mode, the reference GPU kernels' own gate: norm-relative < 2e-3)."""
import types

import numpy as np
import pytest

from helpers import HostLayer, errors, random_routing
from hecate_b200 import layout, synth

pytestmark = pytest.mark.gpu
H_, I_ = 6144, 2048
NORM_REL = 2e-3


@pytest.fixture(scope="module")
def world(oracle):
    """What tier_split keeps per layer (Hh: the pointer tables and the expert count) and per process (T: scratch, the decode
    accumulator, grid sizes), built the way its loader does but on seeded synthetic experts."""
    import torch
    from hecate_b200.shim import moe4
    dev = torch.device("cuda:0")
    hl = HostLayer(31, 0, H_, I_, range(8), 0, shared=False)
    tabs = hl.upload(dev)
    Hh = types.SimpleNamespace(n=tabs.n, hot=tabs.n, far=0, tab=tabs.tabs)
    T = types.SimpleNamespace(scr=moe4.scratch(dev), y=torch.zeros(8, H_, dtype=torch.float, device=dev), blocks=296, blocks_a=444)
    return dev, hl, tabs, Hh, T, hl.oracle_experts(oracle)[0]


def _inputs(dev, R, seed):
    import torch
    x = (synth.activations(seed, 0, R, H_) * 0.5).astype(np.float16)
    sel, rw = random_routing(seed + 1, R, 8)
    return x, sel, rw, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)


def test_decode_call_sites(oracle, world):
    import torch
    from hecate_b200.shim import moe4
    dev, hl, tabs, Hh, T, ex = world
    bsz = 5
    x, sel, rw, y, selected_experts, routing_weights = _inputs(dev, bsz, 80)
    ref = oracle.moe_forward(H_, I_, 0, x, sel, rw, 0, ex, None, mode=1)
    # tier_split.py:567-568 (tier_submit, decode rows, no shared-expert pointers)
    yh = T.y[:bsz]; shp = ()
    moe4.forward(y, selected_experts.view(bsz, -1).contiguous(), routing_weights.view(bsz, -1).contiguous(),
                 Hh.hot if Hh.far else Hh.n, Hh.tab["gate_w"], Hh.tab["up_w"], Hh.tab["down_w"],
                 Hh.tab["gate_s"], Hh.tab["up_s"], Hh.tab["down_s"], *T.scr, yh, T.blocks, T.blocks_a, 0, *shp)
    assert errors(yh.cpu().numpy(), ref)[2] < NORM_REL
    # tier_split.py:587 (tier_combine, hot band only): f += y, y = 0
    final_hidden_states = torch.full((bsz, H_), 0.25, dtype=torch.float, device=dev)
    f2 = final_hidden_states.view(-1, final_hidden_states.shape[-1]); rows = bsz
    moe4.combine(f2, 0, T.y, rows, 0, 0)
    assert errors(f2.cpu().numpy() - 0.25, ref)[2] < NORM_REL and float(T.y.abs().max()) == 0.0
    # tier_split.py:563-565: the same call with the input in the MMA column order (xf = 1), as the norm + router kernel writes it
    xf = torch.from_numpy(layout.frag_order_row(x)).to(dev)
    moe4.forward(xf[:bsz], selected_experts.view(bsz, -1).contiguous(), routing_weights.view(bsz, -1).contiguous(),
                 Hh.hot if Hh.far else Hh.n, Hh.tab["gate_w"], Hh.tab["up_w"], Hh.tab["down_w"],
                 Hh.tab["gate_s"], Hh.tab["up_s"], Hh.tab["down_s"], *T.scr, yh, T.blocks, T.blocks_a, 0, *shp, xf=1)
    assert errors(yh.cpu().numpy(), ref)[2] < NORM_REL
    yh.zero_()
    # tier_split.py:347-353 (_hot_prefill, up to 64 rows in chunks of 8)
    R = 19
    x, sel, rw, y, sel_t, rw_t = _inputs(dev, R, 82)
    ref = oracle.moe_forward(H_, I_, 0, x, sel, rw, 0, ex, None, mode=1)
    out = torch.empty(R, H_, dtype=torch.float, device=y.device)
    sel_t = sel_t.contiguous(); rw_t = rw_t.contiguous()
    for c in range(0, R, 8):
        n = min(8, R - c)
        yh = out[c:c + n]; yh.zero_()
        moe4.forward(y[c:c + n], sel_t[c:c + n], rw_t[c:c + n], Hh.n, Hh.tab["gate_w"], Hh.tab["up_w"], Hh.tab["down_w"],
                     Hh.tab["gate_s"], Hh.tab["up_s"], Hh.tab["down_s"], *T.scr, yh, T.blocks, T.blocks_a, 0)
    assert errors(out.cpu().numpy(), ref)[2] < NORM_REL


@pytest.mark.parametrize("name", ["moe4t", "moe4p"])
def test_prefill_call_site(oracle, world, name):
    """tier_split.py:436-459 (_prefill_gb300, int4 branch) with the host-side permutation the reference does."""
    import importlib
    import torch
    from baseline.ref_gpu import pick_groups
    mod = importlib.import_module(f"hecate_b200.shim.{name}")
    dev, hl, tabs, Hh, T, ex = world
    R = 300
    x, sel_np, rw_np, y, sel, rw = _inputs(dev, R, 84)
    K8 = sel.shape[-1]; fs = sel.reshape(-1)
    order = torch.argsort(fs, stable=True)
    allc = torch.bincount(fs, minlength=Hh.n).tolist()
    out = torch.zeros(y.shape[0], H_, dtype=torch.float, device=y.device)
    ps = 16384
    gu, ar, d = mod.scratch(y.device, ps)
    c4 = allc[:Hh.n]; n4 = sum(c4)
    seg = order[:n4]
    tok = (seg // K8).int(); eid = fs[seg].int(); wt = rw.reshape(-1)[seg].float()
    t = Hh.tab
    for p0, p1, rbt in pick_groups(c4, ps, 256, True):
        mod.forward(y, tok[p0:p1], eid[p0:p1], wt[p0:p1], torch.from_numpy(rbt).pin_memory().to(y.device, non_blocking=True),
                    t["gate_w"], t["up_w"], t["down_w"], t["gate_s"], t["up_s"], t["down_s"], gu, ar, d.view(1, ps, H_), out)
    rows = [0, 77, 299]
    ref = oracle.moe_forward(H_, I_, 0, x[rows], sel_np[rows], rw_np[rows], 0, ex, None, mode=1)
    assert errors(out[rows].cpu().numpy(), ref)[2] < NORM_REL


def test_combine_norm_call_site(oracle):
    import torch
    from hecate_b200.shim import cn
    dev = torch.device("cuda:0")
    rows = 4
    n = lambda s, k: (synth.normal(90, s, rows * H_).reshape(rows, H_) * k).astype(np.float32)
    f, y, r = n(1, 0.3), n(2, 0.5), n(3, 2.0)
    w = torch.from_numpy((1.0 + 0.1 * synth.normal(91, 6, H_)).astype(np.float32)).to(dev).to(torch.bfloat16)
    rn, xn_ref, _ = oracle.combine_norm(f, None, y, None, r, w.float().cpu().numpy(), 1e-6, 0.0, 1.0)
    ft, yt, rt = (torch.from_numpy(a).to(dev) for a in (f, y, r))
    xn = torch.empty(rows, H_, dtype=torch.float16, device=dev)
    cn.combine_norm(ft, 0, yt, rows, 0, 0, rt, w, xn, 1e-6, 0.0, 1.0)              # argument order of runtime/tier/cn.cu:190-191
    assert np.array_equal(rt.cpu().numpy(), rn)
    assert np.abs(xn.cpu().numpy().astype(np.float32) - xn_ref.astype(np.float32)).max() <= 2.0 ** -10 * np.abs(xn_ref.astype(np.float32)).max()
    with pytest.raises(Exception):
        cn.combine_norm_pdl()
