"""Parity of this library's kernels with the reference's OWN GPU kernels, run on the same device: router_k
(runtime/core/exl3_router.py:21-131), combine_norm (runtime/tier/cn.cu:50-105), the moe4 decode kernels
(runtime/tier/moe4/moe4.cu:828-895) and the moe4t tcgen05 prefill kernels (runtime/tier/moe4/moe4t.cu:498-524). The reference
modules are built unchanged for sm_100a by baseline/build_ref_gpu.py into baseline/_ref; a test is skipped when its module is
not there. Shapes follow the reference's own GPU test (tools/quant/test_moe4_rtx.py:59-70: rows 1, 3, 4, 5, 8, x = randn * 0.5,
rw = rand, gate: norm-relative error < 2e-3).
"""
import numpy as np
import pytest

from helpers import HostLayer, errors, random_routing
from hecate_b200 import synth

pytestmark = pytest.mark.gpu
H, I = 6144, 2048
NORM_REL = 2e-3


@pytest.fixture(scope="module")
def ref():
    import torch
    from baseline import ref_gpu
    assert torch.cuda.is_available()
    return ref_gpu.RefGpu(torch.device("cuda:0"))


@pytest.fixture(scope="module")
def layer(oracle):
    """16 full-width experts in the reference's format (one fp32 scale per row), no shared expert."""
    import torch
    hl = HostLayer(21, 0, H, I, range(16), 0, shared=False)
    return hl, hl.upload(torch.device("cuda:0")), hl.oracle_experts(oracle)[0]


def _margins(x16, w16, bias, topk):
    """fp64 keys: the gap between the topk-th and the next key per row (a near-tie shows as a tiny margin)."""
    logit = x16.astype(np.float64) @ w16.astype(np.float64).T
    key = 1.0 / (1.0 + np.exp(-logit)) + (0.0 if bias is None else bias.astype(np.float64)[None, :])
    s = -np.sort(-key, axis=1)
    return s[:, topk - 1] - s[:, topk]


@pytest.mark.parametrize("R", [2, 3, 5, 8])
@pytest.mark.parametrize("bias_sigma", [0.0, 0.1])
def test_router_against_reference_router(ref, R, bias_sigma):
    """Same selected experts as router_k (as sets and in order), weights within one fp16 ulp. router_k sums split-K partials
    with atomics (order not fixed) and uses the fast exponential, so its keys differ from ours in the last bits: a row whose
    top-8 / top-9 margin is below that noise could legitimately differ; the margins are printed and such rows are excused."""
    import torch
    from hecate_b200 import moe
    if ref.rt is None:
        pytest.skip("reference router not built")
    dev = torch.device("cuda:0")
    E, topk = 256, 8
    x = synth.activations(40 + R, 0, R, H).astype(np.float16)
    w = synth.router_weight(0, 0, E, H).astype(np.float16)              # the benchmark's router weight as fp16 (router_k takes fp16 only)
    bias = synth.router_bias(41, 0, E, bias_sigma) if bias_sigma else None
    xt, wt = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    bt = None if bias is None else torch.from_numpy(bias).to(dev)
    rsel, rrw = ref.router(xt, wt, bt, topk, 2.5)
    sel = torch.empty(R, topk, dtype=torch.int64, device=dev); rw = torch.empty(R, topk, dtype=torch.float16, device=dev)
    moe.router_fused(xt, wt, bt, None, None, sel, rw, topk, 2.5)
    torch.cuda.synchronize()
    m = _margins(x, w, bias, topk)
    print(f"router R={R} bias_sigma={bias_sigma}: top-{topk}/{topk + 1} key margin per row " + " ".join(f"{v:.1e}" for v in m))
    a, b = sel.cpu().numpy(), rsel.cpu().numpy()
    for r in range(R):
        if m[r] < 1e-5:
            continue                                                   # near-tie: either choice is within router_k's own noise
        assert set(a[r]) == set(b[r]), (r, a[r], b[r], m[r])
        fa, fb = rw[r].cpu().float().numpy(), rrw[r].cpu().float().numpy()
        wa = dict(zip(a[r].tolist(), fa.tolist())); wb = dict(zip(b[r].tolist(), fb.tolist()))
        for e in wa:
            assert abs(wa[e] - wb[e]) <= max(abs(wb[e]), 2.0 ** -14) * 2.0 ** -10, (r, e, wa[e], wb[e])
    assert (m >= 1e-5).any()


@pytest.mark.parametrize("rows,wdt,with_o", [(8, "bfloat16", True), (3, "float16", False), (16, "bfloat16", False)])
def test_combine_norm_against_reference_kernel(ref, rows, wdt, with_o):
    """hmoe_combine_norm against the reference's combine_norm on the same inputs: the residual bit for bit (the contract the
    reference states for its own kernel pair), the normalised rows to one fp16 ulp (the reference is built with fast-math)."""
    import torch
    from hecate_b200 import moe
    if ref.cn is None:
        pytest.skip("reference cn module not built")
    dev = torch.device("cuda:0")
    n = lambda s, k: torch.from_numpy((synth.normal(50 + rows, s, rows * H).reshape(rows, H) * k).astype(np.float32)).to(dev)
    f, y, r = n(1, 0.3), n(2, 0.5), n(3, 2.0)
    o, o2 = (n(4, 0.2), n(5, 0.1)) if with_o else (None, None)
    w = torch.from_numpy((1.0 + 0.1 * synth.normal(51, 6, H)).astype(np.float32)).to(dev).to(getattr(torch, wdt))
    y1, r1, xn1 = y.clone(), r.clone(), torch.empty(rows, H, dtype=torch.float16, device=dev)
    ref.combine_norm(f, o, y1, o2, r1, w, xn1, 1e-6, 0.0, 1.0)
    y2, r2, xn2 = y.clone(), r.clone(), torch.empty(rows, H, dtype=torch.float16, device=dev)
    moe.combine_norm(f, 0 if o is None else o.data_ptr(), y2, rows, 0 if o2 is None else o2.data_ptr(), 0, r2, w, xn2, 1e-6, 0.0, 1.0)
    torch.cuda.synchronize()
    assert torch.equal(r1, r2) and float(y2.abs().max()) == 0.0 and float(y1.abs().max()) == 0.0
    a, b = xn2.float(), xn1.float()
    ulp = torch.clamp(b.abs(), min=2.0 ** -14) * 2.0 ** -10
    assert bool(((a - b).abs() <= ulp).all())
    assert float((a != b).float().mean()) < 0.02


@pytest.mark.parametrize("R", [1, 3, 4, 5, 8, 16])
def test_decode_against_reference_moe4(oracle, ref, layer, R):
    """hmoe_decode (fp16 activations, per-row scales) against moe4.forward on the same seeded inputs; both against the exact
    evaluation by the CPU checker. 16 rows run on the reference as two 8-row calls (its kernels take at most 8)."""
    import torch
    from hecate_b200 import moe
    if ref.moe4 is None:
        pytest.skip("reference moe4 module not built")
    hl, tabs, ex = layer
    dev = torch.device("cuda:0")
    x = (synth.activations(60 + R, 0, R, H) * 0.5).astype(np.float16)
    sel, rw = random_routing(61 + R, R, 16)
    xt, st, rt = torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
    out_ref = torch.zeros(R, H, device=dev)
    ref.decode(tabs, xt, st, rt, out_ref)
    ws = moe.decode_workspace(H, I, dev)
    y = torch.zeros(R, H, device=dev)
    moe.decode(tabs, xt, st, rt, y, ws)
    torch.cuda.synchronize()
    assert moe.ws_status(ws) == 0
    exact = oracle.moe_forward(H, I, 0, x, sel, rw, 0, ex, None, mode=1)
    e_ours, e_ref = errors(y.cpu().numpy(), exact), errors(out_ref.cpu().numpy(), exact)
    e_pair = errors(y.cpu().numpy(), out_ref.cpu().numpy())
    print(f"decode R={R}: ours vs exact {e_ours[2]:.2e}, moe4 vs exact {e_ref[2]:.2e}, ours vs moe4 {e_pair[2]:.2e}")
    assert e_ours[2] < NORM_REL and e_ref[2] < NORM_REL and e_pair[2] < NORM_REL


@pytest.mark.parametrize("R,zipf", [(40, 0.0), (300, 1.1), (1024, 0.0)])
def test_prefill_against_reference_moe4t(oracle, ref, layer, R, zipf):
    """hmoe_prefill (device permutation + tcgen05 grouped GEMMs) against moe4t.forward driven as the reference's dispatcher
    drives it (host argsort + pick groups); both against the exact evaluation on a sample of rows."""
    import torch
    from hecate_b200 import moe
    if ref.moe4t is None:
        pytest.skip("reference moe4t module not built")
    hl, tabs, ex = layer
    dev = torch.device("cuda:0")
    x = (synth.activations(70 + R, 0, R, H) * 0.5).astype(np.float16)
    sel, rw = synth.zipf_routing(71 + R, 0, R, 16, 8, zipf)
    xt, st, rt = torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev)
    out_ref = ref.prefill(tabs, xt, st, rt)
    ws = moe.prefill_workspace(R, 8, 16, H, I, dev)
    out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, xt, st, rt, out, ws)
    torch.cuda.synchronize()
    assert moe.ws_status(ws) == 0
    rows = np.unique(np.linspace(0, R - 1, 6).astype(int))
    exact = oracle.moe_forward(H, I, 0, x[rows], sel[rows], rw[rows], 0, ex, None, mode=1)
    a, b = out.cpu().numpy(), out_ref.cpu().numpy()
    e_ours, e_ref, e_pair = errors(a[rows], exact), errors(b[rows], exact), errors(a, b)
    print(f"prefill R={R}: ours vs exact {e_ours[2]:.2e}, moe4t vs exact {e_ref[2]:.2e}, ours vs moe4t {e_pair[2]:.2e}")
    assert e_ours[2] < NORM_REL and e_ref[2] < NORM_REL and e_pair[2] < NORM_REL
