"""Parity of the CUDA decode path (through the C ABI) with the CPU checker."""
import numpy as np
import pytest

from helpers import HostLayer, errors, int8_close, random_routing
from hecate_b200 import synth

pytestmark = pytest.mark.gpu

# tolerances: the benchmark definition's bar against the CPU engine (int8 activation mode), with the errors normalised as
# max|a-b| / max|b| and mean|a-b| / mean|b|; and the reference GPU kernel's own gate against an exact evaluation
# (norm-relative < 2e-3, tools/quant/test_moe4_rtx.py:70) for the fp16-activation mode.
MAX_REL, MEAN_ABS, NORM_REL_EXACT = 1e-2, 1e-3, 2e-3


@pytest.fixture(scope="module")
def dev():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def run_case(oracle, dev, H, I, E, R, group, shared, act_quant, seed=0, lo=0, n_local=None, x_dtype="float16", sel_rw=None, calls=1):
    import torch
    from hecate_b200 import moe
    hl = HostLayer(seed, 0, H, I, range(E), group, shared)
    tabs = hl.upload(dev)
    x = synth.activations(seed + 1, 0, R, H)
    sel, rw = sel_rw if sel_rw is not None else random_routing(seed + R, R, E + lo)
    ex, sh = hl.oracle_experts(oracle)
    n_local = E if n_local is None else n_local
    ref = oracle.moe_forward(H, I, group, x.astype(np.float16), sel, rw, lo, ex[:n_local], sh, mode=0 if act_quant else 1)
    ws = moe.decode_workspace(H, I, dev)
    xt = torch.from_numpy(x).to(dev).to(getattr(torch, x_dtype))
    st, rt = torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
    outs = []
    for _ in range(calls):
        y = torch.zeros(R, H, device=dev)
        moe.decode(tabs, xt, st, rt, y, ws, lo=lo, n_local=n_local, act_quant=act_quant)
        outs.append(y.cpu().numpy())
    assert moe.ws_status(ws) == 0
    return outs, ref


@pytest.mark.parametrize("group", [0, 128])
@pytest.mark.parametrize("R", [1, 2, 3, 5, 8, 9, 13, 16])
def test_tiny_shapes_int8_mode(oracle, dev, group, R):
    (got,), ref = run_case(oracle, dev, 256, 128, 8, R, group, True, True)
    e = errors(got, ref)
    assert int8_close(e), e        # the int8 mode follows the CPU engine far inside the required bar


@pytest.mark.parametrize("group", [0, 128])
@pytest.mark.parametrize("R", [1, 4, 8, 16])
def test_tiny_shapes_exact_mode(oracle, dev, group, R):
    (got,), ref = run_case(oracle, dev, 512, 256, 16, R, group, True, False)
    assert errors(got, ref)[2] < NORM_REL_EXACT


def test_no_shared_expert_and_bf16_input(oracle, dev):
    (got,), ref = run_case(oracle, dev, 512, 256, 16, 7, 128, False, True, x_dtype="bfloat16")
    e = errors(got, ref)
    assert e[0] < MAX_REL and e[1] < MEAN_ABS


def test_band_filter_lo_n_local(oracle, dev):
    """Only ids in [lo, lo + n_local) contribute (moe4.cu:93); foreign ids are ignored."""
    (got,), ref = run_case(oracle, dev, 256, 128, 8, 6, 0, False, True, lo=5, n_local=6)
    e = errors(got, ref)
    assert int8_close(e), e


def test_rows_without_local_picks_and_duplicates(oracle, dev):
    """A row with no local pick stays zero; a row that picks one expert twice gets the summed weight."""
    R, E = 4, 8
    sel = np.array([[100, 101, 102, 103, 104, 105, 106, 107], [0, 0, 1, 2, 3, 4, 5, 6], [7, 6, 5, 4, 3, 2, 1, 0], [1, 100, 100, 100, 100, 100, 100, 100]], dtype=np.int64)
    rw = (synth.uniform(3, 1, R * 8).reshape(R, 8) * 0.3 + 0.05).astype(np.float16)
    (got,), ref = run_case(oracle, dev, 256, 128, E, R, 128, False, True, sel_rw=(sel, rw))
    assert np.all(got[0] == 0) and np.all(ref[0] == 0)
    e = errors(got, ref)
    assert int8_close(e), e


def test_hot_expert_more_than_eight_rows(oracle, dev):
    """An expert picked by > 8 rows is processed as two 8-row tiles."""
    R, E = 16, 8
    sel = np.tile(np.arange(8, dtype=np.int64), (R, 1))
    rw = (synth.uniform(4, 1, R * 8).reshape(R, 8) * 0.3 + 0.05).astype(np.float16)
    (got,), ref = run_case(oracle, dev, 256, 128, E, R, 128, True, True, sel_rw=(sel, rw))
    e = errors(got, ref)
    assert int8_close(e), e


def test_repeated_calls_reuse_workspace(oracle, dev):
    """Three calls in a row on one workspace give the same result (the scratch needs no cleaning between calls), as the
    reference's test checks for its counters (tools/quant/test_moe4_rtx.py:59-65)."""
    outs, ref = run_case(oracle, dev, 512, 256, 16, 5, 128, True, True, calls=3)
    assert np.array_equal(outs[0], outs[1]) or errors(outs[1], outs[0])[0] < 1e-6
    assert int8_close(errors(outs[2], ref))


def test_poisoned_workspace(oracle, dev):
    """NaN-filled scratch (except the status word) does not leak into the result."""
    import torch
    from hecate_b200 import moe
    H, I, E, R = 256, 128, 8, 5
    hl = HostLayer(0, 0, H, I, range(E), 128, True)
    tabs = hl.upload(dev)
    x = synth.activations(1, 0, R, H); sel, rw = random_routing(2, R, E)
    ex, sh = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 128, x.astype(np.float16), sel, rw, 0, ex, sh, mode=0)
    ws = moe.decode_workspace(H, I, dev)
    ws[256:] = 0xFF
    y = torch.zeros(R, H, device=dev)
    moe.decode(tabs, torch.from_numpy(x).to(dev).half(), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws, act_quant=True)
    assert int8_close(errors(y.cpu().numpy(), ref))


@pytest.mark.parametrize("group,aq", [(128, True), (128, False), (0, True)])
def test_full_shape(oracle, dev, group, aq):
    """H = 6144, I = 2048 with 12 experts + shared, 16 rows: the benchmark's shapes on a small expert set."""
    (got,), ref = run_case(oracle, dev, 6144, 2048, 12, 16, group, True, aq, seed=3)
    e = errors(got, ref)
    if aq:
        assert e[0] < MAX_REL and e[1] < MEAN_ABS, e
    else:
        assert e[2] < NORM_REL_EXACT, e


@pytest.mark.parametrize("aq", [True, False])
def test_single_token_full_width(oracle, dev, aq):
    """One token (the reference's own CPU-tier decode case): H = 6144, I = 2048, top-8 of 16 experts + shared."""
    (got,), ref = run_case(oracle, dev, 6144, 2048, 16, 1, 128, True, aq, seed=7)
    e = errors(got, ref)
    assert (e[0] < MAX_REL and e[1] < MEAN_ABS) if aq else e[2] < NORM_REL_EXACT, e


@pytest.mark.parametrize("H,I", [(6272, 256), (512, 2176)])
def test_shapes_beyond_the_register_resident_path(oracle, dev, H, I):
    """H > 6144 or I > 2048: a tile's activation fragments no longer fit in registers and the call takes the kernels that
    fetch them stage by stage."""
    (got,), ref = run_case(oracle, dev, H, I, 8, 11, 128, True, True, seed=5)
    assert int8_close(errors(got, ref)), errors(got, ref)


@pytest.mark.parametrize("R,H,I,E,aq", [(16, 6144, 2048, 32, False), (5, 6144, 2048, 32, True), (1, 512, 256, 32, True), (13, 1024, 256, 64, False)])
def test_router_decode_in_one_call_equals_the_two_calls(oracle, dev, R, H, I, E, aq):
    """hmoe_router_decode (the router's launch also does the decode call's set-up step) against hmoe_router followed by
    hmoe_decode: the same selection and weights bit for bit, the same output up to the order of the fp32 atomic additions; and
    against the CPU checker."""
    import torch
    from hecate_b200 import moe
    hl = HostLayer(9, 0, H, I, range(E), 128, True)
    tabs = hl.upload(dev)
    x = synth.activations(40 + R, 0, R, H)
    xt = torch.from_numpy(x).to(dev).to(torch.bfloat16)
    wt = torch.from_numpy(synth.router_weight(41, 0, E, H)).to(dev).to(torch.bfloat16)
    bias = torch.from_numpy(synth.router_bias(41, 0, E, 0.05)).to(dev)
    ws = moe.decode_workspace(H, I, dev)
    sel1 = torch.empty(R, 8, dtype=torch.int64, device=dev); rw1 = torch.empty(R, 8, dtype=torch.float16, device=dev)
    y1 = torch.zeros(R, H, device=dev)
    moe.router_fused(xt, wt, bias, None, None, sel1, rw1, 8, 1.5)
    moe.decode(tabs, xt, sel1, rw1, y1, ws, act_quant=aq)
    ws2 = moe.decode_workspace(H, I, dev)
    for _ in range(2):                                        # twice: the counters inside the library return to zero
        sel2 = torch.full((R, 8), -7, dtype=torch.int64, device=dev); rw2 = torch.zeros(R, 8, dtype=torch.float16, device=dev)
        y2 = torch.zeros(R, H, device=dev)
        moe.router_decode(tabs, xt, wt, bias, sel2, rw2, 1.5, y2, ws2, act_quant=aq)
        assert torch.equal(sel1, sel2) and torch.equal(rw1.view(torch.int16), rw2.view(torch.int16))
        assert moe.ws_status(ws2) == 0
        e = errors(y2.cpu().numpy(), y1.cpu().numpy())
        assert int8_close(e) if aq else e[2] < 1e-3, e
    ex, sh = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 128, x.astype(np.float16), sel2.cpu().numpy(), rw2.cpu().numpy(), 0, ex, sh, mode=0 if aq else 1)
    e = errors(y2.cpu().numpy(), ref)
    assert (e[0] < MAX_REL and e[1] < MEAN_ABS) if aq else e[2] < NORM_REL_EXACT, e


def test_accumulates_into_y_and_combine(oracle, dev):
    import torch
    from hecate_b200 import moe
    H, I, E, R = 256, 128, 8, 4
    hl = HostLayer(0, 0, H, I, range(E), 0, False)
    tabs = hl.upload(dev)
    x = synth.activations(1, 0, R, H); sel, rw = random_routing(2, R, E)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x.astype(np.float16), sel, rw, 0, ex, None, mode=0)
    ws = moe.decode_workspace(H, I, dev)
    y = torch.full((R, H), 2.0, device=dev)
    moe.decode(tabs, torch.from_numpy(x).to(dev).half(), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws, act_quant=True)
    assert int8_close(errors(y.cpu().numpy() - 2.0, ref))
    f = torch.full((R, H), 1.0, device=dev); o = torch.full((R, H), 0.5, device=dev); o2 = torch.full((R, H), 0.25, device=dev)
    yc = y.clone()
    moe.moe4_combine(f, o.data_ptr(), y, R, o2.data_ptr())
    assert torch.equal(f, ((torch.full_like(f, 1.0) + yc) + 0.5) + 0.25) and torch.count_nonzero(y) == 0


def test_reference_named_entry_points(oracle, dev):
    """moe4_forward with the reference's positional argument order, moe4_scratch, moe4_dequant."""
    import torch
    from hecate_b200 import moe, layout
    H, I, E, R = 256, 128, 8, 3
    hl = HostLayer(0, 0, H, I, range(E), 0, True)
    tabs = hl.upload(dev)
    x = synth.activations(1, 0, R, H); sel, rw = random_routing(2, R, E)
    ex, sh = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x.astype(np.float16), sel, rw, 0, ex, sh, mode=1)
    scr = moe.moe4_scratch(dev, H, I)
    y = torch.zeros(R, H, device=dev)
    t = tabs.tabs
    shp = [p.data_ptr() for p in tabs.shared]
    moe.moe4_forward(torch.from_numpy(x).to(dev).half(), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), E,
                     t["gate_w"], t["up_w"], t["down_w"], t["gate_s"], t["up_s"], t["down_s"], *scr, y, 296, 296, 0, *shp, I=I)
    assert errors(y.cpu().numpy(), ref)[2] < NORM_REL_EXACT
    w = moe.moe4_dequant(tabs.keep[0][2], tabs.keep[3][2], I, H).cpu().numpy().astype(np.float64)
    assert np.abs(w - layout.dequant(hl.ex[2]["gq"], hl.ex[2]["gs"], I, H)).max() < 2e-3 * np.abs(w).max()
    hg = HostLayer(0, 0, H, I, range(2), 128, False)
    tg = hg.upload(dev)
    wg = moe.moe4_dequant(tg.keep[2][1], tg.keep[5][1], H, I, group=128).cpu().numpy().astype(np.float64)
    assert np.abs(wg - layout.dequant(hg.ex[1]["dq"], hg.ex[1]["ds"], H, I)).max() < 2e-3 * np.abs(wg).max()


def test_argument_errors(dev):
    import torch
    from hecate_b200 import moe
    hl = HostLayer(0, 0, 256, 128, range(2), 0, False)
    tabs = hl.upload(dev)
    ws = moe.decode_workspace(256, 128, dev)
    x = torch.zeros(17, 256, dtype=torch.float16, device=dev)
    sel = torch.zeros(17, 8, dtype=torch.int64, device=dev); rw = torch.zeros(17, 8, dtype=torch.float16, device=dev)
    y = torch.zeros(17, 256, device=dev)
    with pytest.raises(moe.HmoeError, match="rows"):
        moe.decode(tabs, x, sel, rw, y, ws)
    with pytest.raises(moe.HmoeError, match="workspace"):
        moe.decode(tabs, x[:4], sel[:4], rw[:4], y[:4], ws[:1024])
