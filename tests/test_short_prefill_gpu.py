"""Short prefill on the GPU (1..640 rows as one tile list for the streaming kernels) against the CPU checker, against the
grouped GEMMs at the benchmark's widths, and the row-count dispatch of `forward`."""
import numpy as np
import pytest

from helpers import HostLayer, errors
from hecate_b200 import synth

pytestmark = pytest.mark.gpu

NORM_REL_EXACT = 2e-3      # the reference GPU kernels' own gate against an exact evaluation (tools/quant/test_moe4_rtx.py:70)
MAX_REL = 1e-2             # the benchmark definition's bar against the CPU engine, max|a-b| / max|b|
MEAN_ABS = 1e-3            # the same definition's bar on mean|a-b| / mean|b|


@pytest.fixture(scope="module")
def dev():
    import torch
    assert torch.cuda.is_available()
    return torch.device("cuda:0")


def _short(oracle, dev, H, I, E, R, group, shared, aq, zipf, seed=0, lo=0, n_local=None, sel=None, call="short"):
    import torch
    from hecate_b200 import moe
    hl = HostLayer(seed, 0, H, I, range(E), group, shared)
    tabs = hl.upload(dev)
    x = synth.activations(seed + 1, 0, R, H).astype(np.float16)
    s0, rw = synth.zipf_routing(seed + 2, 0, R, E + lo, 8, zipf)
    sel = s0 if sel is None else sel
    ex, sh = hl.oracle_experts(oracle)
    n_local = E if n_local is None else n_local
    ref = oracle.moe_forward(H, I, group, x, sel, rw, lo, ex[:n_local], sh, mode=0 if aq else 1)
    out = torch.zeros(R, H, device=dev)
    args = (tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out)
    if call == "short":
        ws = moe.short_prefill_workspace(R, H, I, 8, dev)
        moe.short_prefill(*args, ws, lo=lo, n_local=n_local, act_quant=aq)
    else:
        ws = moe.forward_workspace(max(R, 800), 8, n_local, H, I, dev, act_quant=aq)      # one workspace for every row count
        moe.forward(*args, ws, lo=lo, n_local=n_local, act_quant=aq)
    assert moe.ws_status(ws) == 0
    return errors(out.cpu().numpy(), ref)


@pytest.mark.parametrize("group", [0, 128])
@pytest.mark.parametrize("R,zipf,shared", [(1, 0.0, False), (17, 0.0, True), (40, 1.1, True), (100, 0.0, False), (255, 1.3, True), (257, 0.0, True), (640, 1.1, True)])
def test_short_prefill_exact_mode_small(oracle, dev, group, R, zipf, shared):
    """Few experts, so every expert gets many 8-pick tiles (640 rows over 8 experts: 80 tiles each under uniform routing, 80 of
    the shared expert; row numbers beyond 255)."""
    e = _short(oracle, dev, 256, 128, 8, R, group, shared, False, zipf)
    assert e[2] < NORM_REL_EXACT, e


@pytest.mark.parametrize("E,R", [(16, 100), (256, 64)])
def test_short_prefill_int8_mode(oracle, dev, E, R):
    """The CPU engine's int8 activation round trips; 256 experts: most tiles hold one or two picks."""
    e = _short(oracle, dev, 512, 256, E, R, 128, True, True, 0.0)
    assert e[0] < MAX_REL and e[1] < MEAN_ABS, e


def test_short_prefill_full_width(oracle, dev):
    """The benchmark's widths (6144 x 2048: three column chunks per item), few experts so that the CPU checker finishes in seconds."""
    e = _short(oracle, dev, 6144, 2048, 8, 40, 128, True, True, 0.0)
    assert e[0] < MAX_REL and e[1] < MEAN_ABS, e


def test_short_prefill_band_filter(oracle, dev):
    e = _short(oracle, dev, 256, 128, 8, 90, 128, False, False, 0.0, lo=4, n_local=5)
    assert e[2] < NORM_REL_EXACT, e


def test_short_prefill_repeated_picks_and_idle_experts(oracle, dev):
    """A row that picks one expert twice gets two tile columns (both weights count); experts nobody picks emit no tile;
    an expert with exactly 8 and one with exactly 9 picks."""
    R, E = 30, 8
    sel = np.full((R, 8), 1000, dtype=np.int64)             # ids no expert holds
    sel[:, 0] = 3; sel[:, 1] = 3                            # expert 3 twice per row: 60 picks
    sel[:8, 2] = 5                                          # exactly one full tile
    sel[:9, 3] = 6                                          # one full tile and one single pick
    e = _short(oracle, dev, 256, 128, E, R, 128, True, False, 0.0, sel=sel)
    assert e[2] < NORM_REL_EXACT, e


def test_short_prefill_no_local_picks(dev):
    """Nothing selected locally and no shared expert: out stays as it was."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 256, 128, 8, 20
    tabs = HostLayer(0, 0, H, I, range(E), 128, False).upload(dev)
    x = torch.from_numpy(synth.activations(1, 0, R, H)).to(dev).half()
    sel = torch.full((R, 8), 77, dtype=torch.int64, device=dev)
    rw = torch.full((R, 8), 0.125, dtype=torch.float16, device=dev)
    out = torch.full((R, H), 2.5, device=dev)
    ws = moe.short_prefill_workspace(R, H, I, 8, dev)
    moe.short_prefill(tabs, x, sel, rw, out, ws)
    assert moe.ws_status(ws) == 0
    assert bool((out == 2.5).all())


def test_short_prefill_argument_errors(dev):
    import torch
    from hecate_b200 import moe
    H, I, E = 256, 128, 8
    tabs = HostLayer(0, 0, H, I, range(E), 128, False).upload(dev)
    with pytest.raises(moe.HmoeError):
        moe.short_prefill_workspace(641, H, I, 8, dev)
    R = 40
    x = torch.zeros(R, H, dtype=torch.float16, device=dev)
    sel = torch.zeros(R, 8, dtype=torch.int64, device=dev); rw = torch.zeros(R, 8, dtype=torch.float16, device=dev)
    out = torch.zeros(R, H, device=dev)
    small = moe.short_prefill_workspace(R - 1, H, I, 8, dev)
    with pytest.raises(moe.HmoeError):
        moe.short_prefill(tabs, x, sel, rw, out, small)


@pytest.mark.parametrize("R", [8, 16, 17, 64, 300, 384, 385, 700])
def test_forward_picks_a_path_by_row_count(oracle, dev, R):
    """decode (<= 16 rows), short prefill, grouped GEMMs (> forward_short_rows()): one entry point, one workspace, the same result."""
    from hecate_b200 import moe
    assert 16 < moe.forward_short_rows() <= 640
    e = _short(oracle, dev, 256, 128, 8, R, 128, True, False, 1.1, call="forward")
    assert e[2] < NORM_REL_EXACT, e


def test_short_prefill_matches_grouped_gemms_at_full_shape(dev):
    """H = 6144, I = 2048, 64 experts + shared, 96 rows: the short path and the grouped GEMMs agree within the fp16 rounding of the two."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 6144, 2048, 64, 96
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
    a = torch.zeros(R, H, device=dev); b = torch.zeros(R, H, device=dev)
    wsp = moe.prefill_workspace(R, 8, E, H, I, dev)
    moe.prefill(tabs, x, st, rt, a, wsp)
    wss = moe.short_prefill_workspace(R, H, I, 8, dev)
    moe.short_prefill(tabs, x, st, rt, b, wss)
    assert moe.ws_status(wsp) == 0 and moe.ws_status(wss) == 0
    assert errors(b.cpu().numpy(), a.cpu().numpy())[2] < 1e-3


def test_short_prefill_random_against_decode_chunks(dev):
    """Random row counts, expert counts, bands, scale formats and routings (repeated picks inside a row, a few very hot experts):
    the short path equals the decode call in 16-row chunks, which shares its streaming kernels but not its set-up code."""
    import torch
    from hecate_b200 import moe
    rng = np.random.default_rng(7)
    H, I = 256, 128
    layers = {}
    for it in range(60):
        E = int(rng.choice([8, 32, 256])); shared = bool(rng.integers(2)); group = int(rng.choice([0, 128]))
        key = (E, shared, group)
        if key not in layers:
            layers[key] = HostLayer(3, 0, H, I, range(E), group, shared).upload(dev)
        tabs = layers[key]
        R = int(rng.integers(1, 641))
        lo = int(rng.integers(0, E)) if rng.integers(3) == 0 else 0
        n_local = int(rng.integers(1, E - lo + 1)) if lo or rng.integers(3) == 0 else E
        mode = int(rng.integers(3))
        if mode == 0:
            sel = rng.integers(0, E, size=(R, 8))
        elif mode == 1:
            sel = np.stack([rng.permutation(E)[:8] for _ in range(R)])
        else:
            sel = np.minimum((rng.pareto(1.0, size=(R, 8)) * 2).astype(np.int64), E - 1)
        sel = sel.astype(np.int64)
        rw = (rng.random((R, 8)) * 0.3 + 0.02).astype(np.float16)
        aq = bool(rng.integers(2)) and mode == 1      # repeated picks: decode sums their weights before the int8 round trip, the short path after
        x = torch.from_numpy(synth.activations(100 + it, 0, R, H)).to(dev).half()
        st, rt = torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
        a = torch.zeros(R, H, device=dev); b = torch.zeros(R, H, device=dev)
        ws = moe.short_prefill_workspace(R, H, I, 8, dev)
        moe.short_prefill(tabs, x, st, rt, a, ws, lo=lo, n_local=n_local, act_quant=aq)
        wsd = moe.decode_workspace(H, I, dev)
        for c in range(0, R, 16):
            n = min(16, R - c)
            moe.decode(tabs, x[c:c + n], st[c:c + n], rt[c:c + n], b[c:c + n], wsd, lo=lo, n_local=n_local, act_quant=aq)
        assert moe.ws_status(ws) == 0
        # the work list: one tile per eight picks of a local expert (a repeated pick counts twice), the shared expert's rows behind them
        local = sel[(sel >= lo) & (sel < lo + n_local)] - lo
        counts = np.bincount(local, minlength=n_local)
        want_tiles = int(((counts + 7) // 8).sum()) + ((R + 7) // 8 if shared else 0)
        assert moe.route_tiles(ws) == (int((counts > 0).sum()), want_tiles), (it, moe.route_tiles(ws), want_tiles)
        err = float((a - b).norm()) / (float(b.norm()) or 1.0)
        assert err < 2e-3, (it, E, shared, group, R, lo, n_local, mode, aq, err)


def test_forward_reuses_one_workspace_across_paths(oracle, dev):
    """Calls of different sizes, alternating among the three paths, on ONE workspace sized for the largest: what one path leaves
    behind in the shared scratch must not matter to the next (both activation modes)."""
    import torch
    from hecate_b200 import moe
    H, I, E = 256, 128, 8
    hl = HostLayer(0, 0, H, I, range(E), 128, True)
    tabs = hl.upload(dev)
    ex, sh = hl.oracle_experts(oracle)
    for aq in (False, True):
        ws = moe.forward_workspace(700, 8, E, H, I, dev, act_quant=aq)
        for k, R in enumerate([300, 8, 700, 64, 16, 500, 17, 1, 384, 385]):
            x = synth.activations(30 + k, 0, R, H).astype(np.float16)
            sel, rw = synth.zipf_routing(40 + k, 0, R, E, 8, 1.1)
            ref = oracle.moe_forward(H, I, 128, x, sel, rw, 0, ex, sh, mode=0 if aq else 1)
            out = torch.zeros(R, H, device=dev)
            moe.forward(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out, ws, act_quant=aq)
            assert moe.ws_status(ws) == 0
            e = errors(out.cpu().numpy(), ref)
            assert (e[0] < MAX_REL and e[1] < MEAN_ABS) if aq else e[2] < NORM_REL_EXACT, (aq, R, e)
