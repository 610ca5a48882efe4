"""The combine fused into the next input norm: CPU restatement against plain formulas (CPU), CUDA kernel against the
restatement (GPU): the residual bit for bit, the normalised rows to one fp16 ulp."""
import numpy as np
import pytest

from hecate_b200 import synth


def _inputs(rows, H, seed=0, with_f=True, with_o=True):
    n = lambda s: (synth.normal(seed, s, rows * H).reshape(rows, H)).astype(np.float32)
    f = n(1) * 0.3 if with_f else None
    y, r = n(2) * 0.5, n(3) * 2.0
    o = n(4) * 0.2 if with_o else None
    o2 = n(5) * 0.1 if with_o else None
    w = (1.0 + 0.1 * synth.normal(seed, 6, H)).astype(np.float32)
    return f, o, y, o2, r, w


def test_restatement_against_plain_formulas(oracle):
    f, o, y, o2, r, w = _inputs(3, 6144)
    w16 = w.astype(np.float16).astype(np.float32)
    rn, xn, total = oracle.combine_norm(f, o, y, o2, r, w16, 1e-6, 0.0, 1.0)
    a = ((f + y) + o) + o2
    assert np.array_equal(rn, a + r)                                                  # fixed order of fp32 additions
    ref = rn.astype(np.float64) * w16 / np.sqrt((rn.astype(np.float64) ** 2).mean(1) + 1e-6)[:, None]
    assert np.allclose(total, (rn.astype(np.float64) ** 2).sum(1), rtol=1e-6)
    assert np.abs(xn.astype(np.float64) - ref).max() <= np.abs(ref).max() * 2.0 ** -10


@pytest.mark.gpu
@pytest.mark.parametrize("H,rows,wdt,with_f,with_o,cbias,cscale", [(6144, 16, "bfloat16", True, True, 0.0, 1.0), (6144, 3, "float16", False, False, 1.0, 0.5),
                                                                    (256, 5, "float16", True, False, 0.0, 1.0), (7168, 2, "bfloat16", True, True, 0.0, 1.0)])
def test_kernel_against_restatement(oracle, H, rows, wdt, with_f, with_o, cbias, cscale):
    import torch
    from hecate_b200 import moe
    dev = torch.device("cuda:0")
    f, o, y, o2, r, w = _inputs(rows, H, seed=H + rows, with_f=with_f, with_o=with_o)
    wt = torch.from_numpy(w).to(dev).to(getattr(torch, wdt))
    w32 = wt.float().cpu().numpy()
    rn, xn, _ = oracle.combine_norm(f, o, y, o2, r, w32, 1e-6, cbias, cscale)
    td = lambda a: None if a is None else torch.from_numpy(a).to(dev)
    ft, ot, yt, o2t, rt = td(f), td(o), td(y), td(o2), td(r)
    xnt = torch.empty(rows, H, dtype=torch.float16, device=dev)
    moe.combine_norm(ft, 0 if ot is None else ot.data_ptr(), yt, rows, 0 if o2t is None else o2t.data_ptr(), 0, rt, wt, xnt, 1e-6, cbias, cscale)
    assert float(yt.abs().max()) == 0.0                                               # the accumulator is cleared
    assert np.array_equal(rt.cpu().numpy(), rn)                                       # residual: bit for bit
    if ft is not None:
        assert np.array_equal(ft.cpu().numpy(), f)                                    # f is not written
    got = xnt.cpu().numpy()
    ulp = np.maximum(np.abs(xn.astype(np.float32)), 2.0 ** -14) * 2.0 ** -10           # one fp16 ulp (at least the subnormal step)
    assert np.all(np.abs(got.astype(np.float32) - xn.astype(np.float32)) <= ulp)
    assert (got != xn).mean() < 0.02                                                  # and nearly all values identical
