"""Layer files on disk (the reference's `layer{L}.safetensors` container and key scheme), the quantisation recipes and the
per-row -> group-128 conversion."""
import importlib.util
import json
import os
import struct

import numpy as np
import pytest

from hecate_b200 import layout, loader, synth

HERE = os.path.dirname(os.path.abspath(__file__))
H, I = 256, 128


def _make_layer(tmp_path, experts, layer=3, split=False):
    tensors = {}
    for e in experts:
        for m in loader.MATS:
            N, K = (I, H) if m != "down" else (H, I)
            tensors[f"{e}.{m}.q"] = synth.packed_codes(7, layer, m + "_q", e, N, K)
            tensors[f"{e}.{m}.s"] = synth.scales(7, layer, m + "_s", e, N, K, K).reshape(-1).astype(np.float32)
    if split:
        names = sorted(tensors)
        loader.write_layer(str(tmp_path / f"layer{layer}.safetensors"), {k: tensors[k] for k in names[::2]})
        loader.write_layer(str(tmp_path / f"layer{layer}.r1.safetensors"), {k: tensors[k] for k in names[1::2]})
    else:
        loader.write_layer(str(tmp_path / f"layer{layer}.safetensors"), tensors)
    return tensors


@pytest.mark.parametrize("split", [False, True])
def test_round_trip_and_parts(tmp_path, split):
    t = _make_layer(tmp_path, [0, 1, 5, 9], split=split)
    lf = loader.LayerFiles(str(tmp_path), 3)
    assert lf.expert_ids() == [0, 1, 5, 9] and set(lf.keys()) == set(t)
    for k, v in t.items():
        got = lf.get(k)
        assert got.dtype == v.dtype and got.shape == v.shape and np.array_equal(got, v)
    with pytest.raises(KeyError):
        lf.get("2.gate.q")
    with pytest.raises(FileNotFoundError):
        loader.LayerFiles(str(tmp_path), 4)


def test_container_is_the_safetensors_format(tmp_path):
    """If the safetensors package is present, it reads what write_layer wrote, and the reader reads what it writes."""
    if importlib.util.find_spec("safetensors") is None:
        pytest.skip("safetensors not installed")
    from safetensors.numpy import load_file, save_file
    t = _make_layer(tmp_path, [0, 1])
    back = load_file(str(tmp_path / "layer3.safetensors"))
    assert set(back) == set(t) and all(np.array_equal(back[k], t[k]) for k in t)
    save_file({k: np.ascontiguousarray(v) for k, v in t.items()}, str(tmp_path / "layer8.safetensors"))
    lf = loader.LayerFiles(str(tmp_path), 8)
    assert all(np.array_equal(lf.get(k), t[k]) for k in t)


def test_malformed_files_are_rejected(tmp_path):
    p = tmp_path / "layer0.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(loader.FormatError):
        loader.read_header(str(p))
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(loader.FormatError):
        loader.read_header(str(p))
    hdr = json.dumps({"0.gate.q": {"dtype": "U8", "shape": [64], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 10)               # data shorter than the offsets say
    with pytest.raises(loader.FormatError):
        loader.read_header(str(p))
    hdr = json.dumps({"0.gate.q": {"dtype": "U8", "shape": [65], "data_offsets": [0, 64]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 64)               # shape does not match the byte count
    with pytest.raises(loader.FormatError):
        loader.read_header(str(p))
    p.write_bytes(struct.pack("<Q", 5) + b"nope!" + b"\0" * 8)
    with pytest.raises(loader.FormatError):
        loader.read_header(str(p))


def test_row_scales_match_the_reference_recipe():
    """quant.npz holds the scales the reference's scales_mse chose for the seeded matrix (tests/golden/make_golden.py)."""
    g = np.load(os.path.join(HERE, "golden", "quant.npz"))
    assert np.allclose(g["u4f"], np.array(loader.U4F, dtype=np.float32))
    # the matrix is regenerated from its seed (as the generator does)
    w = synth.normal(21, 5150, 24 * 256).reshape(24, 256).astype(np.float32) * (10.0 ** np.linspace(-3, 1, 24, dtype=np.float32))[:, None]
    s = loader.row_scales(w)
    assert s.dtype == np.float32 and np.allclose(s, g["scales"], rtol=2e-6, atol=0)


def test_quantize_rows_reconstruction():
    w = (synth.normal(3, 99, 128 * 256).reshape(128, 256) * 0.02).astype(np.float32)
    q, s = loader.quantize_rows(w)
    codes = layout.unpack_u4(q, 128, 256).astype(np.float32) - 8
    err = np.sqrt(np.mean((codes * s[:, None] - w) ** 2)) / np.sqrt(np.mean(w ** 2))
    assert codes.min() >= -8 and codes.max() <= 7 and err < 0.13          # 4-bit uniform quantiser on gaussian rows: ~0.10-0.12


def test_quantize_g128_and_scale_order():
    w = (synth.normal(4, 98, 128 * 256).reshape(128, 256) * np.linspace(0.01, 0.05, 256, dtype=np.float32)[None, :]).astype(np.float32)
    q, sbits = loader.quantize_g128(w)
    assert sbits.shape == (2, 2, 64) and sbits.dtype == np.uint16
    s = layout.group_scales_logical(loader._bf16_to_f32(sbits), 128)                     # [K/128][N]
    codes = layout.unpack_u4(q, 128, 256).astype(np.float32) - 8
    rec = codes * np.repeat(s.T, 128, axis=1)
    err_g = np.sqrt(np.mean((rec - w) ** 2))
    qr, sr = loader.quantize_rows(w)
    err_r = np.sqrt(np.mean(((layout.unpack_u4(qr, 128, 256).astype(np.float32) - 8) * sr[:, None] - w) ** 2))
    assert err_g < err_r                                    # column-dependent magnitudes: a scale per group fits better


def test_convert_to_g128_keeps_values(tmp_path):
    t = _make_layer(tmp_path, [0, 2])
    out = tmp_path / "g128"
    loader.convert_to_g128(str(tmp_path), str(out), 3, H, I)
    lf = loader.LayerFiles(str(out), 3)
    assert lf.dtype("0.gate.s") == "BF16" and lf.get("0.gate.s").shape == (I // 64, H // 128, 64)
    for e in (0, 2):
        for m in loader.MATS:
            N, K = (I, H) if m != "down" else (H, I)
            assert np.array_equal(lf.get(f"{e}.{m}.q"), t[f"{e}.{m}.q"])
            s = layout.group_scales_logical(loader._bf16_to_f32(lf.get(f"{e}.{m}.s")), N)    # [K/128][N]
            row = t[f"{e}.{m}.s"]
            assert np.all(np.abs(s - row[None, :]) <= np.abs(row[None, :]) * 2.0 ** -8)


def test_placement_file(tmp_path):
    p = tmp_path / "place.json"
    p.write_text(json.dumps({"3": {"perm": [2, 0, 1, 3], "hot": 2, "far": 1, "first": 3}, "4": {"perm": [0, 0, 1, 2]}}))
    assert loader.load_placement(str(p), 3)["perm"] == [2, 0, 1, 3]
    with pytest.raises(loader.FormatError):
        loader.load_placement(str(p), 4)
    with pytest.raises(loader.FormatError):
        loader.load_placement(str(p), 5)
