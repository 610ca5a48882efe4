"""The CUDA router selects the same experts and writes the same fp16 weights as the CPU checker, bit for bit."""
import numpy as np
import pytest

from hecate_b200 import synth

pytestmark = pytest.mark.gpu


def _run(oracle, R, H, E, topk, xbf, wbf, bias_sigma, scale, seed):
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    x = synth.activations(seed, 0, R, H); w = synth.router_weight(seed, 0, E, H)
    bias = synth.router_bias(seed, 0, E, bias_sigma) if bias_sigma is not None else None
    xt = torch.from_numpy(x).to(dev).to(torch.bfloat16 if xbf else torch.float16)
    wt = torch.from_numpy(w).to(dev).to(torch.bfloat16 if wbf else torch.float16)
    sel = torch.empty(R, topk, dtype=torch.int64, device=dev); rw = torch.empty(R, topk, dtype=torch.float16, device=dev)
    moe.router_fused(xt, wt, None if bias is None else torch.from_numpy(bias).to(dev), None, None, sel, rw, topk, scale)
    bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)
    osel, orw = oracle.router(bits(xt), xbf, bits(wt), wbf, bias, topk, scale)
    assert np.array_equal(osel, sel.cpu().numpy())
    assert np.array_equal(orw.view(np.uint16), bits(rw))


@pytest.mark.parametrize("R", [1, 2, 8, 16, 33])
def test_router_bit_exact_benchmark_shape(oracle, R):
    _run(oracle, R, 6144, 256, 8, 1, 1, 0.0, 1.0, seed=R)


@pytest.mark.parametrize("xbf,wbf", [(0, 0), (0, 1), (1, 0)])
def test_router_dtypes_bias_scale(oracle, xbf, wbf):
    _run(oracle, 5, 1024, 64, 6, xbf, wbf, 0.1, 2.5, seed=7)
    _run(oracle, 3, 256, 32, 8, xbf, wbf, None, 1.0, seed=8)


def test_router_large_rows(oracle):
    _run(oracle, 1000, 512, 128, 8, 1, 1, 0.05, 1.0, seed=9)


def test_fill_matches_numpy_generator():
    import torch
    from hecate_b200 import moe
    t = torch.empty(8192, dtype=torch.uint8, device="cuda:0")
    moe.fill_bytes(t, 5, synth.stream_id(2, "down_q", 17))
    assert np.array_equal(t.cpu().numpy(), synth.rand_bytes(5, synth.stream_id(2, "down_q", 17), 8192))


@pytest.mark.parametrize("R,H,wbf,with_y", [(16, 6144, True, True), (5, 6144, False, False), (3, 512, True, True), (9, 1024, False, True)])
def test_norm_route_equals_norm_then_router(R, H, wbf, with_y):
    """Residual add + norm + router in one launch gives, bit for bit, what the norm kernel followed by the router gives."""
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    E, topk = 256, 8
    g = lambda s, n: torch.from_numpy(synth.normal(31, s, n).astype(np.float32)).to(dev)
    r = g(1, R * H).view(R, H) * 2.0
    y = g(2, R * H).view(R, H) * 0.5 if with_y else None
    nw = (1.0 + 0.1 * g(3, H)).to(torch.bfloat16 if wbf else torch.float16)
    wt = torch.from_numpy(synth.router_weight(4, 0, E, H)).to(dev).to(torch.bfloat16 if wbf else torch.float16)
    bias = torch.from_numpy(synth.router_bias(4, 0, E, 0.05)).to(dev)
    # separate: combine_norm (a = y, r += a, xn), then the router on xn
    r1 = r.clone(); y1 = y.clone() if y is not None else torch.zeros(R, H, device=dev)
    xn1 = torch.empty(R, H, dtype=torch.float16, device=dev)
    moe.combine_norm(None, 0, y1, R, 0, 0, r1, nw, xn1, 1e-6, 0.0, 1.0)
    sel1 = torch.empty(R, topk, dtype=torch.int64, device=dev); rw1 = torch.empty(R, topk, dtype=torch.float16, device=dev)
    moe.router_fused(xn1, wt, bias, None, None, sel1, rw1, topk, 2.5)
    # fused
    xn2 = torch.empty(R, H, dtype=torch.float16, device=dev); r2 = torch.empty(R, H, device=dev)
    sel2 = torch.empty(R, topk, dtype=torch.int64, device=dev); rw2 = torch.empty(R, topk, dtype=torch.float16, device=dev)
    moe.norm_route(y, r, nw, xn2, wt, bias, sel2, rw2, topk, 2.5, 1e-6, r_out=r2)
    assert torch.equal(r2, r1) and torch.equal(xn2, xn1)
    assert torch.equal(sel2, sel1) and torch.equal(rw2.view(torch.int16), rw1.view(torch.int16))


@pytest.mark.parametrize("R,H,wbf,with_y,cbias", [(16, 6144, True, True, 0.0), (4, 6144, False, False, 1.0), (7, 1024, True, True, 0.0)])
def test_norm_route_against_the_checker(oracle, R, H, wbf, with_y, cbias):
    """hmoe_norm_router against the CPU checker alone (no other kernel of this library involved): the residual sum bit for
    bit and the normalised rows to one fp16 ulp against the checker's combine_norm restatement; the selection and the fp16
    weights bit for bit against the checker's router applied to the rows the kernel wrote."""
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    E, topk, scale = 256, 8, 2.5
    g = lambda s, n: synth.normal(33, s, n).astype(np.float32)
    r = g(1, R * H).reshape(R, H) * 2.0
    y = g(2, R * H).reshape(R, H) * 0.5 if with_y else None
    nw_t = torch.from_numpy(1.0 + 0.1 * g(3, H)).to(dev).to(torch.bfloat16 if wbf else torch.float16)
    wt_t = torch.from_numpy(synth.router_weight(5, 0, E, H)).to(dev).to(torch.bfloat16 if wbf else torch.float16)
    bias = synth.router_bias(5, 0, E, 0.05)
    xn = torch.empty(R, H, dtype=torch.float16, device=dev); r_out = torch.empty(R, H, device=dev)
    sel = torch.empty(R, topk, dtype=torch.int64, device=dev); rw = torch.empty(R, topk, dtype=torch.float16, device=dev)
    moe.norm_route(None if y is None else torch.from_numpy(y).to(dev), torch.from_numpy(r).to(dev), nw_t, xn, wt_t, torch.from_numpy(bias).to(dev),
                   sel, rw, topk, scale, 1e-6, cbias=cbias, r_out=r_out)
    torch.cuda.synchronize()
    rn, xn_ref, _ = oracle.combine_norm(None, None, y if y is not None else np.zeros_like(r), None, r, nw_t.float().cpu().numpy(), 1e-6, cbias, 1.0)
    assert np.array_equal(r_out.cpu().numpy(), rn)
    got = xn.cpu().numpy().astype(np.float32)
    ulp = np.maximum(np.abs(xn_ref.astype(np.float32)), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(got - xn_ref.astype(np.float32)) <= ulp)
    bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)
    osel, orw = oracle.router(bits(xn), 0, bits(wt_t), int(wbf), bias, topk, scale)
    assert np.array_equal(osel, sel.cpu().numpy())
    assert np.array_equal(orw.view(np.uint16), bits(rw))
