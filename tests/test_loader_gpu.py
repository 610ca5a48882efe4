"""Experts loaded from layer files on disk give the same decode result as the same experts uploaded from memory, for the
per-row format, the group format written by the converter, an expert-parallel shard and a placement permutation."""
import numpy as np
import pytest

from helpers import HostLayer, errors, int8_close, random_routing
from hecate_b200 import loader, synth

pytestmark = pytest.mark.gpu
H, I, E = 256, 128, 8


def _write(tmp_path, hl, shared_id=None):
    t = {}
    for e, d in zip(hl.ids, hl.ex):
        for m, c in zip(loader.MATS, "gud"):
            t[f"{e}.{m}.q"] = d[c + "q"]; t[f"{e}.{m}.s"] = d[c + "s"].reshape(-1).astype(np.float32)
    if shared_id is not None:
        for m, c in zip(loader.MATS, "gud"):
            t[f"{shared_id}.{m}.q"] = hl.sh[c + "q"]; t[f"{shared_id}.{m}.s"] = hl.sh[c + "s"].reshape(-1).astype(np.float32)
    loader.write_layer(str(tmp_path / "layer0.safetensors"), t)


def _decode(tabs, x, sel, rw, dev, lo=0, n_local=None):
    import torch
    from hecate_b200 import moe
    ws = moe.decode_workspace(H, I, dev); y = torch.zeros(x.shape[0], H, device=dev)
    moe.decode(tabs, torch.from_numpy(x).to(dev), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws, lo=lo, n_local=n_local,
               act_quant=True)
    assert moe.ws_status(ws) == 0
    return y.cpu().numpy()


def test_per_row_files_and_shared_expert(tmp_path, oracle):
    import torch
    dev = torch.device("cuda:0")
    hl = HostLayer(5, 0, H, I, range(E), 0, True)
    _write(tmp_path, hl, shared_id=256)
    tabs = loader.load_layer(str(tmp_path), 0, H, I, dev, shared=256)
    assert tabs.n == E and tabs.group == 0
    x = synth.activations(1, 0, 6, H).astype(np.float16); sel, rw = random_routing(2, 6, E)
    ex, sh = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x, sel, rw, 0, ex, sh, mode=0)
    assert int8_close(errors(_decode(tabs, x, sel, rw, dev), ref))


def test_shard_and_placement(tmp_path, oracle):
    import torch
    dev = torch.device("cuda:0")
    hl = HostLayer(6, 0, H, I, range(E), 0, False)
    _write(tmp_path, hl)
    perm = [3, 1, 7, 0, 2, 6, 5, 4]
    tabs = loader.load_layer(str(tmp_path), 0, H, I, dev, placement={"perm": perm}, rank=1, world=2)      # positions 4..7 = experts 2, 6, 5, 4
    assert tabs.n == 4
    x = synth.activations(1, 0, 5, H).astype(np.float16); sel, rw = random_routing(3, 5, E)              # sel = router positions
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x, sel, rw, 4, [ex[perm[p]] for p in range(4, 8)], None, mode=0)
    assert int8_close(errors(_decode(tabs, x, sel, rw, dev, lo=4, n_local=4), ref))


def test_converted_group_files(tmp_path, oracle):
    import torch
    dev = torch.device("cuda:0")
    hl = HostLayer(7, 0, H, I, range(E), 0, False)
    _write(tmp_path, hl)
    loader.convert_to_g128(str(tmp_path), str(tmp_path / "g"), 0, H, I)
    tabs = loader.load_layer(str(tmp_path / "g"), 0, H, I, dev)
    assert tabs.group == 128
    x = synth.activations(1, 0, 4, H).astype(np.float16); sel, rw = random_routing(4, 4, E)
    ex, _ = hl.oracle_experts(oracle)
    ref = oracle.moe_forward(H, I, 0, x, sel, rw, 0, ex, None, mode=0)
    e = errors(_decode(tabs, x, sel, rw, dev), ref)
    assert e[0] < 1e-2 and e[1] < 6e-3, e          # the row scales were rounded to bf16 (2^-9 relative each)
