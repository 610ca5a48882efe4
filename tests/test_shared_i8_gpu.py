"""The shared expert in the reference's int8 format (dense GEMV fragment order, one fp32 scale per row) beside int4 routed
experts: the decode and the prefill result equal the routed experts' result plus an exact evaluation of the int8 expert."""
import numpy as np
import pytest

from helpers import HostLayer, errors, random_routing
from hecate_b200 import layout, synth

pytestmark = pytest.mark.gpu
NORM_REL_EXACT = 2e-3      # the reference GPU kernels' own gate against an exact evaluation (tools/quant/test_moe4_rtx.py:70)


def _int8_expert(seed, H, I):
    mk = lambda s, N, K: (synth.rand_bytes(seed, s, N * K).reshape(N, K).astype(np.uint8), (np.exp(synth.normal(seed, s + 50, N) * 0.5 - 7.5)).astype(np.float32))
    return mk(1, I, H), mk(2, I, H), mk(3, H, I)


def _shared_exact(x, ex):
    (gc, gs), (uc, us), (dc, ds) = ex
    w = lambda c, s: (c.astype(np.float64) - 128.0) * s[:, None].astype(np.float64)
    xd = x.astype(np.float64)
    g, u = xd @ w(gc, gs).T, xd @ w(uc, us).T
    return (g / (1.0 + np.exp(-g)) * u) @ w(dc, ds).T


@pytest.mark.parametrize("H,I,R,group", [(256, 128, 5, 128), (512, 256, 16, 0), (6144, 2048, 16, 128), (6144, 2048, 3, 128)])
def test_int8_shared_expert(oracle, H, I, R, group):
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    E = 8
    hl = HostLayer(9, 0, H, I, range(E), group, False)
    base = hl.upload(dev)
    ex8 = _int8_expert(13, H, I)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    shared = tuple(up(layout.pack_i8(c)) for c, _ in ex8) + tuple(up(s) for _, s in ex8)
    tabs = moe.ExpertTables(H, I, 8, *[base.keep[i] for i in range(6)], group=group, shared=shared, device=dev, shared_i8=True)
    x = synth.activations(3, 0, R, H).astype(np.float16); sel, rw = random_routing(4, R, E)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, group, x, sel, rw, 0, ex, None, mode=1).astype(np.float64) + _shared_exact(x, ex8)
    ws = moe.decode_workspace(H, I, dev)
    for call in range(2):                     # twice on one workspace: the per-pick buffer is cleared by every call
        y = torch.zeros(R, H, device=dev)
        moe.decode(tabs, up(x), up(sel), up(rw), y, ws)
        assert moe.ws_status(ws) == 0
        assert errors(y.cpu().numpy(), ref)[2] < NORM_REL_EXACT, (call, errors(y.cpu().numpy(), ref))


@pytest.mark.parametrize("H,I,R,group", [(256, 128, 40, 128), (512, 256, 300, 0), (6144, 2048, 200, 128)])
def test_int8_shared_expert_in_prefill(oracle, H, I, R, group):
    """The grouped GEMMs take the same int8 shared expert: its tiles are staged from the int8 fragment order and scaled per row in
    the read-out, beside routed experts of either scale format."""
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    E = 8
    hl = HostLayer(9, 0, H, I, range(E), group, False)
    base = hl.upload(dev)
    ex8 = _int8_expert(13, H, I)
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    shared = tuple(up(layout.pack_i8(c)) for c, _ in ex8) + tuple(up(s) for _, s in ex8)
    tabs = moe.ExpertTables(H, I, 8, *[base.keep[i] for i in range(6)], group=group, shared=shared, device=dev, shared_i8=True)
    x = synth.activations(3, 0, R, H).astype(np.float16); sel, rw = random_routing(4, R, E)
    ex, _ = hl.oracle_experts(oracle)
    rows = np.unique(np.concatenate([np.arange(min(R, 6)), [R // 2, R - 1]]))
    ref = oracle.moe_forward(H, I, group, x[rows], sel[rows], rw[rows], 0, ex, None, mode=1).astype(np.float64) + _shared_exact(x[rows], ex8)
    ws = moe.prefill_workspace(R, 8, E, H, I, dev)
    for call in range(2):
        y = torch.zeros(R, H, device=dev)
        moe.prefill(tabs, up(x), up(sel), up(rw), y, ws)
        assert moe.ws_status(ws) == 0
        got = y.cpu().numpy()
        assert errors(got[rows], ref)[2] < NORM_REL_EXACT, (call, errors(got[rows], ref))
    # and the decode kernels agree with the grouped GEMMs on the first 16 rows
    yd = torch.zeros(16 if R >= 16 else R, H, device=dev); n = yd.shape[0]
    moe.decode(tabs, up(x[:n]), up(sel[:n]), up(rw[:n]), yd, moe.decode_workspace(H, I, dev))
    assert errors(got[:n], yd.cpu().numpy().astype(np.float64))[2] < NORM_REL_EXACT
    # and so does the short path, which runs the int8 shared expert sixteen rows at a time (37 rows: 16 + 16 + 5)
    ns = min(R, 37)
    ys = torch.zeros(ns, H, device=dev)
    wss = moe.short_prefill_workspace(ns, H, I, 8, dev)
    for call in range(2):
        ys.zero_()
        moe.short_prefill(tabs, up(x[:ns]), up(sel[:ns]), up(rw[:ns]), ys, wss)
        assert moe.ws_status(wss) == 0
        assert errors(ys.cpu().numpy().astype(np.float64), got[:ns])[2] < NORM_REL_EXACT, call
    # in the int8 activation mode the streaming kernels do not take the int8 shared expert; `forward` sends such a call to the grouped GEMMs
    with pytest.raises(moe.HmoeError):
        moe.short_prefill(tabs, up(x[:ns]), up(sel[:ns]), up(rw[:ns]), ys, wss, act_quant=True)
    with pytest.raises(moe.HmoeError):
        moe.decode(tabs, up(x[:n]), up(sel[:n]), up(rw[:n]), yd, moe.decode_workspace(H, I, dev), act_quant=True)
    wsf = moe.forward_workspace(ns, 8, E, H, I, dev, act_quant=True)
    yq = torch.zeros(ns, H, device=dev); yp = torch.zeros(ns, H, device=dev)
    moe.forward(tabs, up(x[:ns]), up(sel[:ns]), up(rw[:ns]), yq, wsf, act_quant=True)
    moe.prefill(tabs, up(x[:ns]), up(sel[:ns]), up(rw[:ns]), yp, moe.prefill_workspace(ns, 8, E, H, I, dev, act_quant=True), act_quant=True)
    assert moe.ws_status(wsf) == 0 and errors(yq.cpu().numpy(), yp.cpu().numpy())[2] < 1e-5       # the same kernels; the sums' order differs
