"""The packed int4 weight layout of the operator surface, on the host (numpy).

A matrix W[N][K] of 4-bit codes c in [0, 15] (value c - 8) is stored in the order the reference's packer writes
(tools/quant/gptq_int4.py:74-77, inverse runtime/tier/tier_split.py:98-101): with KB = K / 64,

    byte b = ((((((gr*KB + kb)*4 + s)*8 + g)*4 + q)*4 + t)*2 + cc)*2 + h,   nibble rh (0 = low)

holds row n = gr*64 + s*16 + rh*8 + g and column k = kb*64 + t*16 + h*8 + q*2 + cc. Read as 16-byte words, word
((gr*KB + kb)*4 + s)*32 + lane with lane = g*4 + q is what lane `lane` of a warp feeds to four m16n8k16 MMAs (one 32-bit
word per 16 columns). 64 rows x 64 columns form one contiguous 2 KB unit and all units of a 64-row group are contiguous.

Scales: fp32 [N] for the reference's one-scale-per-row format. For the group-quantised format the logical tensor is
[K/G][N]; on the device it is stored bf16 [N/64][K/G][64] with row r of a 64-row group at position (r % 8) * 8 + r / 8
(`group_scales_device_order`), so one 16-byte load gives an MMA lane the scales of its eight rows.
"""
import numpy as np


def pack_u4(codes):
    """codes uint8 [N][K] in [0, 15] -> packed uint8 [N*K/2]."""
    N, K = codes.shape
    assert N % 64 == 0 and K % 64 == 0
    c = codes.reshape(N // 64, 4, 2, 8, K // 64, 4, 2, 4, 2)      # gr s rh g kb t h q cc
    c = c.transpose(0, 4, 1, 3, 7, 5, 8, 6, 2).reshape(-1, 2)     # gr kb s g q t cc h | rh
    return (c[:, 0] | (c[:, 1] << 4)).astype(np.uint8)


def unpack_u4(q, N, K):
    """packed uint8 [N*K/2] -> codes uint8 [N][K]."""
    q = np.asarray(q, dtype=np.uint8).reshape(-1)
    c = np.stack((q & 15, q >> 4), axis=-1).reshape(N // 64, K // 64, 4, 8, 4, 4, 2, 2, 2)   # gr kb s g q t cc h rh
    return c.transpose(0, 2, 8, 3, 1, 5, 7, 4, 6).reshape(N, K)


def rowmajor_i4(q, N, K):
    """packed -> row-major nibbles [N][K/2], low nibble = even column (the CPU engine's format, tier_split.py:103-106)."""
    c = unpack_u4(q, N, K)
    return (c[:, 0::2] | (c[:, 1::2] << 4)).astype(np.uint8)


def dequant(q, scales, N, K):
    """packed codes + scales [K/G][N] -> float64 [N][K]."""
    c = unpack_u4(q, N, K).astype(np.float64) - 8.0
    s = np.asarray(scales, dtype=np.float64).reshape(-1, N)
    G = K // s.shape[0]
    return c * np.repeat(s.T, G, axis=1)


def frag_order_row(v):
    """Reorder the last axis (multiple of 64 values) into the order the kernels read an activation row in: inside
    every 64-column block the 32 two-value words p = t*8 + h*4 + q move to q*8 + t*2 + h, so that the eight words one
    lane needs for the block's four m16n8k16 steps are contiguous."""
    v = np.asarray(v)
    K = v.shape[-1]
    w = v.reshape(*v.shape[:-1], K // 64, 4, 2, 4, 2)            # kb t h q pair
    return w.swapaxes(-4, -2).swapaxes(-3, -2).reshape(v.shape)  # kb q t h pair


def group_scales_device_order(s):
    """logical scales [K/G][N] -> device order [N/64][K/G][64] (row r of a group at (r % 8) * 8 + r // 8)."""
    s = np.asarray(s)
    KG, N = s.shape
    t = s.reshape(KG, N // 64, 8, 8)                 # kg, gr, j (= r // 8), g (= r % 8)
    return np.ascontiguousarray(t.transpose(1, 0, 3, 2)).reshape(N // 64, KG, 64)


def group_scales_logical(d, N):
    """inverse of group_scales_device_order: [N/64][K/G][64] -> [K/G][N]."""
    d = np.asarray(d).reshape(N // 64, -1, 8, 8)     # gr, kg, g, j
    return np.ascontiguousarray(d.transpose(1, 0, 3, 2)).reshape(-1, N)


def pack_i8(codes):
    """codes uint8 [N][K] (value = code - 128) -> the reference's dense int8 fragment order, N % 64 == 0, K % 32 == 0
    (runtime/core/hecate_runtime.py:43-48 with four strips per group): byte
    ((((((((gr * K/32 + kb) * 4 + s) * 8 + g) * 4 + q) * 2 + t) * 2 + h) * 2 + c) * 2 + rh holds row gr*64 + s*16 + rh*8 + g,
    column kb*32 + t*16 + h*8 + q*2 + c."""
    codes = np.asarray(codes, dtype=np.uint8)
    N, K = codes.shape
    assert N % 64 == 0 and K % 32 == 0
    v = codes.reshape(N // 64, 4, 2, 8, K // 32, 2, 2, 4, 2)               # gr, s, rh, g, kb, t, h, q, c
    return np.ascontiguousarray(v.transpose(0, 4, 1, 3, 7, 5, 6, 8, 2)).reshape(-1)


def unpack_i8(q, N, K):
    """inverse of pack_i8 -> codes uint8 [N][K]."""
    v = np.asarray(q, dtype=np.uint8).reshape(N // 64, K // 32, 4, 8, 4, 2, 2, 2, 2)   # gr, kb, s, g, q, t, h, c, rh
    return np.ascontiguousarray(v.transpose(0, 2, 8, 3, 1, 5, 6, 4, 7)).reshape(N, K)

