"""Seeded synthetic inputs for the MoE expert path (weights, scales, activations, router, routing).

Everything derives from one counter-based generator, `u64(seed, stream, index)` (splitmix64 finaliser applied twice), so
a tensor's contents depend only on (seed, stream id, element index): the numpy code here and the CUDA fill kernel
(`hmoe_fill_bytes`) produce identical bytes, and nothing depends on torch's or numpy's own RNG streams.

Distributions follow the benchmark configuration: int4 codes uniform (the packed bytes are uniform, which makes every
nibble uniform in [0, 15], i.e. values uniform in [-8, 7]); scales lognormal(mu=-4, sigma=0.5) rounded to bf16;
activations N(0, 1) rounded to bf16 (and representable in fp16, see `activations`); router weight N(0, 0.02) in bf16.
"""
import numpy as np

_M = np.uint64(0xFFFFFFFFFFFFFFFF)
_G = np.uint64(0x9E3779B97F4A7C15)
_C1 = np.uint64(0xBF58476D1CE4E5B9)
_C2 = np.uint64(0x94D049BB133111EB)

# stream ids: (layer, kind, expert) -> one 64-bit stream number
KIND = {"gate_q": 1, "up_q": 2, "down_q": 3, "gate_s": 4, "up_s": 5, "down_s": 6, "x": 7, "router_w": 8, "router_b": 9,
        "route": 10, "rw": 11}
SHARED = 4095  # expert index used for the shared expert's streams


def stream_id(layer, kind, expert=0):
    return (int(layer) << 24) | (KIND[kind] << 12) | int(expert)


def _mix(z):
    with np.errstate(over="ignore"):
        z = (z + _G) & _M
        z = ((z ^ (z >> np.uint64(30))) * _C1) & _M
        z = ((z ^ (z >> np.uint64(27))) * _C2) & _M
        return z ^ (z >> np.uint64(31))


def u64(seed, stream, n, offset=0):
    """n 64-bit words: word i = mix(mix(seed * G + stream) + offset + i)."""
    with np.errstate(over="ignore"):
        base = _mix(np.array([(int(seed) * 0x9E3779B97F4A7C15 + int(stream)) & 0xFFFFFFFFFFFFFFFF], dtype=np.uint64))[0]
        idx = np.arange(offset, offset + n, dtype=np.uint64)
        return _mix((idx + base) & _M)


def rand_bytes(seed, stream, nbytes):
    """nbytes uniform bytes (nbytes % 8 == 0): little-endian bytes of the stream's words."""
    assert nbytes % 8 == 0
    return u64(seed, stream, nbytes // 8).view(np.uint8)


def uniform(seed, stream, n, offset=0):
    """float64 in (0, 1)."""
    return ((u64(seed, stream, n, offset) >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def normal(seed, stream, n):
    """float64 standard normal (Box-Muller on two words per value)."""
    u = uniform(seed, stream, 2 * n)
    return np.sqrt(-2.0 * np.log(u[0::2])) * np.cos(2.0 * np.pi * u[1::2])


def to_bf16_bits(v):
    """float array -> uint16 bf16 bit patterns, round to nearest even."""
    b = np.asarray(v, dtype=np.float32).view(np.uint32)
    r = ((b >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return ((b + r) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def packed_codes(seed, layer, kind, expert, N, K):
    """Packed int4 codes of one matrix in the operator layout: N*K/2 uniform bytes."""
    return rand_bytes(seed, stream_id(layer, kind, expert), N * K // 2)


def scales(seed, layer, kind, expert, N, K, G):
    """Scales exp(-4 + 0.5 z) rounded to bf16, returned as float32 [K/G][N] (column-group major). G == K: one per row."""
    z = normal(seed, stream_id(layer, kind, expert), (K // G) * N)
    return bf16_bits_to_f32(to_bf16_bits(np.exp(-4.0 + 0.5 * z))).reshape(K // G, N)


def activations(seed, layer, R, H, scale=1.0):
    """N(0, scale) rounded to bf16, as float32 [R][H]. Values below fp16's normal range are flushed to zero so the same
    numbers are exactly representable in both bf16 and fp16 (the reference path computes in fp16)."""
    v = bf16_bits_to_f32(to_bf16_bits(normal(seed, stream_id(layer, "x"), R * H) * scale))
    v = np.where(np.abs(v) < 6.103515625e-05, np.float32(0), v)
    return np.clip(v, -65504.0, 65504.0).astype(np.float32).reshape(R, H)


def router_weight(seed, layer, E, H):
    """N(0, 0.02) rounded to bf16, float32 [E][H]."""
    return bf16_bits_to_f32(to_bf16_bits(normal(seed, stream_id(layer, "router_w"), E * H) * 0.02)).reshape(E, H)


def router_bias(seed, layer, E, sigma=0.0):
    if sigma == 0.0:
        return np.zeros(E, dtype=np.float32)
    return (normal(seed, stream_id(layer, "router_b"), E) * sigma).astype(np.float32)


def zipf_routing(seed, layer, R, E, topk, s):
    """Per-token top-k without replacement from expert popularity p_e ~ 1/(e+1)^s (Gumbel top-k); weights are random
    positive numbers renormalised per token and rounded to fp16. s == 0 gives uniform routing.
    Returns sel int64 [R][topk] (selection order = descending perturbed score), rw float16 [R][topk]."""
    logp = -float(s) * np.log(np.arange(1, E + 1, dtype=np.float64))
    u = uniform(seed, stream_id(layer, "route"), R * E).reshape(R, E)
    score = logp[None, :] - np.log(-np.log(u))
    sel = np.argsort(-score, axis=1, kind="stable")[:, :topk].astype(np.int64)
    w = uniform(seed, stream_id(layer, "rw"), R * topk).reshape(R, topk) + 0.05
    rw = (w / w.sum(1, keepdims=True)).astype(np.float16)
    return sel, rw
