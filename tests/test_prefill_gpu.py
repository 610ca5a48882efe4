"""Prefill path on the GPU: device permutation (bit-exact) and the tcgen05 grouped GEMMs (tolerance) against the CPU checker,
and against the decode path at the benchmark's full shapes."""
import numpy as np
import pytest

from helpers import HostLayer, errors
from hecate_b200 import synth

pytestmark = pytest.mark.gpu

NORM_REL_EXACT = 2e-3      # the reference GPU kernels' own gate against an exact evaluation (tools/quant/test_moe4_rtx.py:70)
MAX_REL = 1e-2             # the benchmark definition's bar against the CPU engine, max|a-b| / max|b|
MEAN_ABS = 1e-3            # the same definition's bar on mean|a-b| / mean|b|; the int8 mode carries code x scale as fp16 hi + lo


@pytest.fixture(scope="module")
def dev():
    import torch
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


@pytest.mark.parametrize("R,E,lo,nl,shared,bm,balance,zipf", [
    (1, 8, 0, 8, 0, 64, True, 0.0), (40, 8, 0, 8, 0, 64, True, 0.0), (300, 64, 0, 64, 300, 256, True, 1.1),
    (300, 64, 16, 32, 0, 64, False, 1.1), (1000, 256, 64, 32, 1000, 256, True, 1.3), (8192, 256, 0, 256, 8192, 256, True, 1.1),
    (32768, 256, 0, 256, 0, 256, True, 1.3)])
def test_permutation_bit_exact(oracle, dev, R, E, lo, nl, shared, bm, balance, zipf):
    """Stable sort by expert id, tok / eid / wt, counts and row blocks equal the checker's (tier_split.py:404-412,
    rtx_split.py:236-255); ids outside [lo, lo + n_local) are dropped; the shared expert's rows follow as expert n_local."""
    import torch
    from hecate_b200 import moe
    sel, rw = synth.zipf_routing(1, 0, R, E, 8, zipf)
    p = moe.permute(torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), nl, lo=lo, shared_rows=shared, bm=bm, balance=balance)
    fs = sel.reshape(-1)
    keep = np.nonzero((fs >= lo) & (fs < lo + nl))[0]
    if lo == 0 and nl == E:
        o, tok, eid, wt, counts = oracle.permute(sel, rw, E)                      # the checker's own permutation
    else:
        o = keep[np.argsort(fs[keep], kind="stable")].astype(np.int32)
        tok, eid, wt = (o // 8).astype(np.int32), (fs[o] - lo).astype(np.int32), rw.reshape(-1)[o].astype(np.float32)
        counts = np.bincount(fs[keep] - lo, minlength=nl).astype(np.int32)
    n = len(o)
    assert p["total"] == n + shared
    assert np.array_equal(p["order"][:n].cpu().numpy(), o)
    assert np.array_equal(p["tok"][:n].cpu().numpy(), tok)
    assert np.array_equal(p["eid"][:n].cpu().numpy(), eid)
    assert np.array_equal(p["wt"][:n].cpu().numpy(), wt)
    assert np.array_equal(p["counts"][:nl].cpu().numpy(), counts)
    cc = np.concatenate([counts, [shared]]).astype(np.int32) if shared else counts
    assert np.array_equal(p["rbt"].cpu().numpy(), oracle.row_blocks(cc, bm, balance))
    if shared:
        assert np.array_equal(p["tok"][n:].cpu().numpy(), np.arange(shared, dtype=np.int32))
        assert bool((p["eid"][n:] == nl).all()) and bool((p["wt"][n:] == 1).all())


def _prefill(oracle, dev, H, I, E, R, group, shared, aq, zipf, seed=0, lo=0, n_local=None):
    import torch
    from hecate_b200 import moe
    hl = HostLayer(seed, 0, H, I, range(E), group, shared)
    tabs = hl.upload(dev)
    x = synth.activations(seed + 1, 0, R, H).astype(np.float16)
    sel, rw = synth.zipf_routing(seed + 2, 0, R, E + lo, 8, zipf)
    ex, sh = hl.oracle_experts(oracle)
    n_local = E if n_local is None else n_local
    ref = oracle.moe_forward(H, I, group, x, sel, rw, lo, ex[:n_local], sh, mode=0 if aq else 1)
    ws = moe.prefill_workspace(R, 8, n_local, H, I, dev, act_quant=aq)
    out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out, ws, lo=lo,
                n_local=n_local, act_quant=aq)
    assert moe.ws_status(ws) == 0
    return errors(out.cpu().numpy(), ref)


@pytest.mark.parametrize("group", [0, 128])
@pytest.mark.parametrize("R,zipf,shared", [(1, 0.0, False), (40, 0.0, True), (300, 1.1, True), (777, 1.3, False)])
def test_prefill_exact_mode_small(oracle, dev, group, R, zipf, shared):
    e = _prefill(oracle, dev, 256, 128, 8, R, group, shared, False, zipf)
    assert e[2] < NORM_REL_EXACT, e


@pytest.mark.parametrize("group", [0, 128])
def test_prefill_int8_mode(oracle, dev, group):
    e = _prefill(oracle, dev, 512, 256, 16, 700, group, True, True, 1.1)
    assert e[0] < MAX_REL and e[1] < MEAN_ABS, e


def test_prefill_int8_mode_full_width(oracle, dev):
    """The benchmark's widths (6144 x 2048), few experts and rows so that the CPU checker finishes in seconds."""
    e = _prefill(oracle, dev, 6144, 2048, 8, 64, 128, True, True, 0.0)
    assert e[0] < MAX_REL and e[1] < MEAN_ABS, e


def test_prefill_band_filter(oracle, dev):
    e = _prefill(oracle, dev, 256, 128, 8, 200, 128, False, False, 0.0, lo=4, n_local=5)
    assert e[2] < NORM_REL_EXACT, e


def test_prefill_row_block_edges(oracle, dev):
    """Experts with exactly 256 / 257 / 0 picks: row blocks of 256, 129 + 128, and none."""
    import torch
    from hecate_b200 import moe
    H, I, E = 256, 128, 8
    R = 300
    sel = np.zeros((R, 8), dtype=np.int64)
    for r in range(R):
        first = 0 if r < 256 else 1                       # expert 0: 256 picks; expert 1: 257 picks (rows 0..212 pick it too)
        others = [2, 3, 4, 5, 6, 100 + r % 3, 200]        # foreign ids are dropped; expert 7 never picked
        sel[r] = [first] + others
    for r in range(213):
        sel[r, 7] = 1
    rw = (synth.uniform(5, 1, R * 8).reshape(R, 8) * 0.3 + 0.05).astype(np.float16)
    hl = HostLayer(0, 0, H, I, range(E), 128, False)
    tabs = hl.upload(dev)
    x = synth.activations(1, 0, R, H).astype(np.float16)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 128, x, sel, rw, 0, ex, None, mode=1)
    ws = moe.prefill_workspace(R, 8, E, H, I, dev)
    out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out, ws)
    assert moe.ws_status(ws) == 0
    assert errors(out.cpu().numpy(), ref)[2] < NORM_REL_EXACT


@pytest.mark.parametrize("n", [1, 15, 16, 17, 63, 64, 65, 127, 128, 129, 191, 192, 193, 255])
def test_prefill_pick_counts_around_the_input_box_size(oracle, dev, n):
    """One expert with exactly n picks (the input tile is loaded as boxes of 64 rows, the MMA runs over n rounded up to 16): the
    rows behind the block belong to another expert's block and must neither be read into the result nor written."""
    import torch
    from hecate_b200 import moe
    H, I, E = 256, 128, 8
    R = 300
    sel = np.full((R, 8), 1000, dtype=np.int64)             # ids no expert holds
    sel[:n, 0] = 2                                          # expert 2: n picks
    sel[:, 1] = 5                                           # expert 5: every row (its blocks follow expert 2's in the gathered order)
    rw = (synth.uniform(6, 1, R * 8).reshape(R, 8) * 0.3 + 0.05).astype(np.float16)
    hl = HostLayer(0, 0, H, I, range(E), 128, False)
    tabs = hl.upload(dev)
    x = synth.activations(2, 0, R, H).astype(np.float16)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 128, x, sel, rw, 0, ex, None, mode=1)
    ws = moe.prefill_workspace(R, 8, E, H, I, dev)
    out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out, ws)
    assert moe.ws_status(ws) == 0
    assert errors(out.cpu().numpy(), ref)[2] < NORM_REL_EXACT


def test_prefill_adds_into_out_and_is_linear_in_weights(dev):
    """out is added into; doubling every routing weight doubles the routed part (the shared expert's part stays)."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 256, 128, 8, 100
    hl = HostLayer(0, 0, H, I, range(E), 128, False)
    tabs = hl.upload(dev)
    x = torch.from_numpy(synth.activations(1, 0, R, H)).to(dev).half()
    sel, rw = synth.zipf_routing(3, 0, R, E, 8, 0.0)
    st, rt = torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
    ws = moe.prefill_workspace(R, 8, E, H, I, dev)
    a = torch.zeros(R, H, device=dev); moe.prefill(tabs, x, st, rt, a, ws)
    b = torch.full((R, H), 3.0, device=dev); moe.prefill(tabs, x, st, (rt.float() * 2).half(), b, ws)
    assert errors((b - 3.0).cpu().numpy(), (2 * a).cpu().numpy())[2] < 1e-3


def test_prefill_matches_decode_at_full_shape(dev):
    """H = 6144, I = 2048, 32 experts + shared, 1024 rows with Zipf routing: sampled rows equal the decode path (which is
    checked against the CPU engine) within the fp16 rounding of the two paths."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 6144, 2048, 32, 1024
    per = I * H // 2
    pool = torch.empty((E + 1) * 3 * per, dtype=torch.uint8, device=dev)
    moe.fill_bytes(pool, 7, 99)
    view = lambda e, k: pool[(e * 3 + k) * per:(e * 3 + k + 1) * per]
    g = torch.Generator(device=dev); g.manual_seed(1)
    sc = lambda N, K: (torch.randn(E + 1, N // 64, K // 128, 64, device=dev, generator=g) * 0.5 - 4.0).exp().to(torch.bfloat16)
    gs, us, ds = sc(I, H), sc(I, H), sc(H, I)
    tabs = moe.ExpertTables(H, I, 8, [view(e, 0) for e in range(E)], [view(e, 1) for e in range(E)], [view(e, 2) for e in range(E)],
                            list(gs[:E]), list(us[:E]), list(ds[:E]), group=128,
                            shared=(view(E, 0), view(E, 1), view(E, 2), gs[E], us[E], ds[E]), device=dev)
    x = torch.from_numpy(synth.activations(1, 0, R, H)).to(dev).to(torch.bfloat16)
    sel, rw = synth.zipf_routing(3, 0, R, E, 8, 1.1)
    st, rt = torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
    ws = moe.prefill_workspace(R, 8, E, H, I, dev)
    out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, x, st, rt, out, ws)
    assert moe.ws_status(ws) == 0
    rows = torch.arange(0, R, R // 16, device=dev)[:16]
    wsd = moe.decode_workspace(H, I, dev)
    y = torch.zeros(16, H, device=dev)
    moe.decode(tabs, x[rows].contiguous(), st[rows].contiguous(), rt[rows].contiguous(), y, wsd)
    assert errors(out[rows].cpu().numpy(), y.cpu().numpy())[2] < 1e-3


def test_reference_calling_convention_moe4t_forward(oracle, dev):
    """moe4t_forward with tok / wt / rbt prepared on the host exactly as the reference's dispatcher does
    (tier_split.py:433-457: stable argsort, bincount, pick_groups with 256-pick balanced blocks)."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 256, 128, 8, 500
    hl = HostLayer(0, 0, H, I, range(E), 0, False)
    tabs = hl.upload(dev)
    x = synth.activations(1, 0, R, H).astype(np.float16)
    sel, rw = synth.zipf_routing(2, 0, R, E, 8, 1.1)
    order, tok, eid, wt, counts = oracle.permute(sel, rw, E)
    rbt = oracle.row_blocks(counts, 256, True)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x, sel, rw, 0, ex, None, mode=1)
    scr = moe.moe4t_scratch(dev, len(tok), H, I)
    out = torch.zeros(R, H, device=dev)
    t = tabs.tabs
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    moe.moe4t_forward(T(x), T(tok), T(eid), T(wt), T(rbt), t["gate_w"], t["up_w"], t["down_w"], t["gate_s"], t["up_s"], t["down_s"], *scr, out, I=I)
    assert errors(out.cpu().numpy(), ref)[2] < NORM_REL_EXACT
