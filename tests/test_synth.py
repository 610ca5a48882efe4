import numpy as np

from hecate_b200 import synth


def test_streams_are_reproducible_and_distinct():
    a = synth.rand_bytes(0, synth.stream_id(0, "gate_q", 3), 4096)
    b = synth.rand_bytes(0, synth.stream_id(0, "gate_q", 3), 4096)
    c = synth.rand_bytes(0, synth.stream_id(0, "up_q", 3), 4096)
    assert np.array_equal(a, b) and not np.array_equal(a, c)
    assert synth.u64(1, 2, 4)[2] == synth.u64(1, 2, 1, offset=2)[0]


def test_known_words():
    """Pinned words of the generator (the CUDA fill kernel is checked against the same function on the GPU)."""
    w = synth.u64(0, 0, 2)
    assert w.dtype == np.uint64
    z = 0  # splitmix64 finaliser of 0 + G, twice, by hand
    M = (1 << 64) - 1

    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & M
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
        return z ^ (z >> 31)
    base = mix(0)
    assert int(w[0]) == mix(base) and int(w[1]) == mix((base + 1) & M)


def test_distributions():
    z = synth.normal(0, 5, 200000)
    assert abs(z.mean()) < 0.01 and abs(z.std() - 1) < 0.01
    s = synth.scales(0, 0, "gate_s", 0, 512, 1024, 128)
    assert s.shape == (8, 512)
    assert abs(np.log(s.astype(np.float64)).mean() + 4) < 0.02 and abs(np.log(s.astype(np.float64)).std() - 0.5) < 0.02
    x = synth.activations(0, 0, 4, 1024)
    assert np.array_equal(x.astype(np.float16).astype(np.float32), x)          # exactly representable in fp16
    assert np.array_equal(synth.bf16_bits_to_f32(synth.to_bf16_bits(x)), x)     # and in bf16
    codes = synth.packed_codes(0, 0, "gate_q", 0, 256, 256)
    nib = np.concatenate([codes & 15, codes >> 4])
    assert np.abs(np.bincount(nib, minlength=16) / nib.size - 1 / 16).max() < 0.01
