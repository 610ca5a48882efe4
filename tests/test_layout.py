"""Packed int4 layout: the package's numpy functions, the checker's C functions and the reference's own packer agree."""
import os

import numpy as np

from hecate_b200 import layout, synth

G = os.path.join(os.path.dirname(__file__), "golden")


def test_pack_matches_reference_packer(oracle):
    z = np.load(os.path.join(G, "layout.npz"))
    codes, packed, rm = z["codes"], z["packed"], z["rowmajor"]
    N, K = codes.shape
    assert np.array_equal(layout.pack_u4(codes), packed)                 # reference pack_u4 output
    assert np.array_equal(layout.unpack_u4(packed, N, K), codes)         # reference _unpack_moe4 output
    assert np.array_equal(layout.rowmajor_i4(packed, N, K), rm)          # reference _rowmajor_i4 output
    assert np.array_equal(oracle.unpack_rowmajor(packed, N, K), rm)
    assert np.array_equal(oracle.pack_from_rowmajor(rm, N, K), packed)


def test_roundtrip_random():
    for N, K, seed in [(64, 64, 1), (128, 256, 2), (192, 128, 3)]:
        codes = (synth.rand_bytes(seed, 1, N * K) & 15).reshape(N, K).astype(np.uint8)
        q = layout.pack_u4(codes)
        assert q.shape == (N * K // 2,)
        assert np.array_equal(layout.unpack_u4(q, N, K), codes)


def test_byte_formula():
    """The explicit index formula of the layout (one byte = two rows 8 apart, same column)."""
    N, K = 128, 128
    codes = (synth.rand_bytes(9, 2, N * K) & 15).reshape(N, K).astype(np.uint8)
    q = layout.pack_u4(codes)
    KB = K // 64
    rng = np.random.default_rng(0)
    for n, k in zip(rng.integers(0, N, 200), rng.integers(0, K, 200)):
        gr, s, rh, g = n // 64, (n % 64) // 16, (n % 16) // 8, n % 8
        kb, t, h, qq, cc = k // 64, (k % 64) // 16, (k % 16) // 8, (k % 8) // 2, k % 2
        b = ((((((gr * KB + kb) * 4 + s) * 8 + g) * 4 + qq) * 4 + t) * 2 + cc) * 2 + h
        assert (q[b] >> (4 * rh)) & 15 == codes[n, k]


def test_group_scale_order_roundtrip():
    s = synth.scales(0, 0, "gate_s", 3, 256, 512, 128)
    d = layout.group_scales_device_order(s)
    assert d.shape == (4, 4, 64)
    assert np.array_equal(layout.group_scales_logical(d, 256), s)
    gr, kg, j, g = 2, 1, 5, 3
    assert d[gr, kg, g * 8 + j] == s[kg, gr * 64 + j * 8 + g]


def test_dequant_matches_definition():
    N, K = 64, 128
    q = synth.packed_codes(0, 0, "gate_q", 0, N, K)
    s = synth.scales(0, 0, "gate_s", 0, N, K, 128)
    w = layout.dequant(q, s, N, K)
    c = layout.unpack_u4(q, N, K).astype(np.float64) - 8
    assert np.allclose(w[:, :128], c[:, :128] * s[0][:, None].astype(np.float64))
    assert c.min() >= -8 and c.max() <= 7


def test_frag_order_row():
    v = np.arange(128)
    w = layout.frag_order_row(v)
    # word p (values 2p, 2p+1) of block 0 sits at q*8 + t*2 + h with t = p // 8, h = (p % 8) // 4, q = p % 4
    for p in range(32):
        t, h, qq = p // 8, (p % 8) // 4, p % 4
        pos = qq * 8 + t * 2 + h
        assert w[2 * pos] == 2 * p and w[2 * pos + 1] == 2 * p + 1
    assert sorted(w[64:]) == list(range(64, 128))


def test_int8_layout_matches_the_reference_packer():
    """layout_i8.npz holds what the reference's own _pack wrote for seeded codes (tests/golden/make_golden.py)."""
    import os
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layout_i8.npz"))
    assert np.array_equal(layout.pack_i8(g["codes"]), g["packed"])
    assert np.array_equal(layout.unpack_i8(g["packed"], *g["codes"].shape), g["codes"])
