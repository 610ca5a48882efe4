"""Edge cases of the decode and prefill paths on the GPU: nothing to do, one row, zero weights, large activations."""
import numpy as np
import pytest

from helpers import HostLayer, errors, int8_close, random_routing
from hecate_b200 import synth

pytestmark = pytest.mark.gpu
H, I, E = 256, 128, 8


@pytest.fixture(scope="module")
def setup():
    import torch
    from oracle import oracle as O
    dev = torch.device("cuda:0")
    hl = HostLayer(0, 0, H, I, range(E), 128, False)
    return dev, hl, hl.upload(dev), hl.oracle_experts(O)[0], O


def test_no_local_pick_leaves_output_untouched(setup):
    import torch
    from hecate_b200 import moe
    dev, hl, tabs, ex, O = setup
    R = 3
    x = torch.from_numpy(synth.activations(1, 0, R, H)).to(dev).half()
    sel = torch.full((R, 8), 100, dtype=torch.int64, device=dev); rw = torch.full((R, 8), 0.1, dtype=torch.float16, device=dev)
    ws = moe.decode_workspace(H, I, dev); y = torch.zeros(R, H, device=dev)
    moe.decode(tabs, x, sel, rw, y, ws)
    assert float(y.abs().max()) == 0.0 and moe.ws_status(ws) == 0
    wsp = moe.prefill_workspace(R, 8, E, H, I, dev); out = torch.zeros(R, H, device=dev)
    moe.prefill(tabs, x, sel, rw, out, wsp)
    assert float(out.abs().max()) == 0.0 and moe.ws_status(wsp) == 0
    p = moe.permute(sel, rw, E)
    assert p["total"] == 0 and p["nrb"] == 0


def test_single_row_prefill(setup):
    import torch
    from hecate_b200 import moe
    dev, hl, tabs, ex, O = setup
    x = synth.activations(1, 0, 1, H).astype(np.float16); sel, rw = random_routing(3, 1, E)
    out = torch.zeros(1, H, device=dev); wsp = moe.prefill_workspace(1, 8, E, H, I, dev)
    moe.prefill(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), out, wsp)
    ref = O.moe_forward(H, I, 128, x, sel, rw, 0, ex, None, mode=1)
    assert errors(out.cpu().numpy(), ref)[2] < 2e-3


def test_zero_routing_weights_give_zero(setup):
    import torch
    from hecate_b200 import moe
    dev, hl, tabs, ex, O = setup
    sel, rw = random_routing(4, 5, E); rw[:] = 0
    x = torch.from_numpy(synth.activations(2, 0, 5, H)).to(dev).half()
    ws = moe.decode_workspace(H, I, dev); y = torch.zeros(5, H, device=dev)
    moe.decode(tabs, x, torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws)
    assert float(y.abs().max()) == 0.0


@pytest.mark.parametrize("scale", [0.3, 4.0])
def test_activation_scales_like_the_reference_test(setup, scale):
    """The reference's engine test draws x with scales 0.3, 1 and 4 (tools/dev/test_grace_picks.py:61)."""
    import torch
    from hecate_b200 import moe
    dev, hl, tabs, ex, O = setup
    x = synth.activations(2, 0, 8, H, scale).astype(np.float16); sel, rw = random_routing(5, 8, E)
    ws = moe.decode_workspace(H, I, dev); y = torch.zeros(8, H, device=dev)
    moe.decode(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws, act_quant=True)
    ref = O.moe_forward(H, I, 128, x, sel, rw, 0, ex, None, mode=0)
    e = errors(y.cpu().numpy(), ref)
    assert int8_close(e), e
