"""On-disk int4 expert files -> expert tables in HBM.

The reference keeps one safetensors file per layer, `layer{L}.safetensors` (plus optional `layer{L}.r*.safetensors` parts),
with keys `"{id}.{gate,up,down}.{q,s}"`: `q` the packed codes (uint8, N*K/2 bytes in the operator's fragment order), `s`
one fp32 scale per output row (runtime/tier/tier_split.py:18-19,207-214). A placement file maps router positions to expert
ids: `{layer: {"perm": [ids], "hot": n, "far": m, "first": n + m}}` (tier_split.py:17; tools/placement). Here:

  * `LayerFiles` reads those files without any dependency (the container format is a JSON header in front of raw
    little-endian tensors) and hands out zero-copy numpy views of a memory map;
  * `load_layer` uploads the experts a rank serves and builds the six pointer tables (`hecate_b200.moe.ExpertTables`), for
    the whole layer or for one expert-parallel shard;
  * `write_layer` writes files in the same format (tests, tools);
  * `quantize_rows` restates the reference's per-row recipe (`scales_mse`, tools/quant/gptq_int4.py:62-71: the scale that
    minimises the squared error over eight candidates rms / f), `quantize_g128` applies the same recipe per group of 128
    input columns for the group format, and `convert_to_g128` rewrites per-row files as group files (codes unchanged,
    the row scale repeated per group and rounded to bf16: values change by at most 2^-9 relative).

Group-format files use the same keys; their `s` is bf16 `[N/64][K/128][64]` in the order the kernels read
(`layout.group_scales_device_order`), so a scale tensor is uploaded as it lies in the file.
"""
import glob
import json
import os
import struct

import numpy as np

from . import layout

_DTYPES = {"U8": (np.uint8, 1), "I8": (np.int8, 1), "F32": (np.float32, 4), "F16": (np.float16, 2), "BF16": (np.uint16, 2),
           "I32": (np.int32, 4), "I64": (np.int64, 8), "U16": (np.uint16, 2)}
U4F = (2.4, 2.6, 2.8, 3.0, 3.2, 3.4, 3.7, 4.0)       # candidate divisors of the row rms (tools/quant/gptq_int4.py:38)
MATS = ("gate", "up", "down")


class FormatError(ValueError):
    pass


def read_header(path):
    """-> (entries, data_start): entries[name] = (dtype string, shape tuple, begin, end) with offsets relative to data_start."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise FormatError(f"{path}: shorter than a safetensors header")
        n = struct.unpack("<Q", raw)[0]
        if n < 2 or 8 + n > size:
            raise FormatError(f"{path}: header length {n} does not fit the file")
        try:
            hdr = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise FormatError(f"{path}: header is not JSON ({e})")
    out = {}
    for name, d in hdr.items():
        if name == "__metadata__":
            continue
        dt, shape, (b, e) = d["dtype"], tuple(int(v) for v in d["shape"]), d["data_offsets"]
        if dt not in _DTYPES:
            raise FormatError(f"{path}: tensor {name} has unsupported dtype {dt}")
        if b < 0 or e < b or 8 + n + e > size or int(np.prod(shape, dtype=np.int64)) * _DTYPES[dt][1] != e - b:
            raise FormatError(f"{path}: tensor {name} has inconsistent offsets")
        out[name] = (dt, shape, int(b), int(e))
    return out, 8 + n


class LayerFiles:
    """The tensors of `layer{L}.safetensors` and its `layer{L}.r*.safetensors` parts in a directory, as numpy views of
    memory maps (bf16 tensors come back as uint16 bit patterns)."""

    def __init__(self, u4dir, layer):
        self.paths = sorted(glob.glob(os.path.join(u4dir, f"layer{layer}.safetensors")) + glob.glob(os.path.join(u4dir, f"layer{layer}.r*.safetensors")))
        if not self.paths:
            raise FileNotFoundError(f"no layer{layer}.safetensors under {u4dir}")
        self.where = {}
        self.maps = []
        for i, p in enumerate(self.paths):
            entries, start = read_header(p)
            self.maps.append((np.memmap(p, dtype=np.uint8, mode="r"), start))
            for k, v in entries.items():
                self.where[k] = (i, v)

    def keys(self):
        return self.where.keys()

    def dtype(self, name):
        return self.where[name][1][0]

    def get(self, name):
        if name not in self.where:
            raise KeyError(f"{name} is not in {self.paths}")
        i, (dt, shape, b, e) = self.where[name]
        mm, start = self.maps[i]
        return mm[start + b:start + e].view(_DTYPES[dt][0]).reshape(shape)

    def expert_ids(self):
        return sorted({int(k.split(".")[0]) for k in self.where if k.split(".")[0].isdigit()})


def write_layer(path, tensors, bf16=()):
    """Writes `tensors` (name -> numpy array) as one safetensors file; names listed in `bf16` hold uint16 bit patterns and are
    labelled BF16."""
    names = sorted(tensors)
    rev = {np.dtype(np.uint8): "U8", np.dtype(np.int8): "I8", np.dtype(np.float32): "F32", np.dtype(np.float16): "F16",
           np.dtype(np.int32): "I32", np.dtype(np.int64): "I64", np.dtype(np.uint16): "U16"}
    hdr, off = {}, 0
    for n in names:
        a = np.ascontiguousarray(tensors[n])
        dt = "BF16" if n in bf16 else rev[a.dtype]
        hdr[n] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + a.nbytes]}
        off += a.nbytes
    blob = json.dumps(hdr, separators=(",", ":")).encode("utf-8")
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for n in names:
            f.write(np.ascontiguousarray(tensors[n]).tobytes())


# ----------------------------------------------------------------------------------------------------------------------
def _best_scale(W, axis_len):
    """W [..., K] float64/32 -> scale [...] minimising sum((W - clip(round(W / s), -8, 7) * s)^2) over s = rms / f, f in U4F;
    ties keep the earlier candidate (the reference's strict `e < best_e`)."""
    W = np.asarray(W, dtype=np.float32)
    s0 = np.maximum(np.sqrt(np.mean(W * W, axis=-1, dtype=np.float32)), np.float32(1e-12)).astype(np.float32)
    best_e = best_s = None
    for f in U4F:
        s = (s0 / np.float32(f)).astype(np.float32)
        q = np.clip(np.rint(W / s[..., None]), -8, 7)
        e = np.sum((W - q * s[..., None]) ** 2, axis=-1, dtype=np.float32)
        if best_e is None:
            best_e, best_s = e, s
        else:
            m = e < best_e
            best_e = np.where(m, e, best_e); best_s = np.where(m, s, best_s)
    return best_s.astype(np.float32)


def row_scales(W):
    """W fp32 [..., N, K] -> fp32 [..., N]: the scale the reference's scales_mse picks for every row."""
    return _best_scale(W, np.asarray(W).shape[-1])


def quantize_rows(W):
    """W fp32 [N][K] -> (packed codes uint8 [N*K/2], scale fp32 [N]): the reference's per-row format, round-to-nearest codes."""
    W = np.asarray(W, dtype=np.float32)
    s = row_scales(W)
    codes = (np.clip(np.rint(W / s[:, None]), -8, 7) + 8).astype(np.uint8)
    return layout.pack_u4(codes), s


def _bf16_round(a):
    u = np.asarray(a, dtype=np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def _bf16_to_f32(bits):
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize_g128(W, group=128):
    """W fp32 [N][K] -> (packed codes, scale bits uint16 bf16 in device order [N/64][K/128][64]); the codes are taken against
    the bf16-rounded scale, so that (code - 8) * stored scale is the best reconstruction available."""
    W = np.asarray(W, dtype=np.float32)
    N, K = W.shape
    Wg = W.reshape(N, K // group, group)
    s = _bf16_to_f32(_bf16_round(_best_scale(Wg, group)))                   # [N][K/G]
    s = np.where(s > 0, s, np.float32(2.0 ** -126))
    codes = (np.clip(np.rint(Wg / s[..., None]), -8, 7) + 8).astype(np.uint8).reshape(N, K)
    dev = layout.group_scales_device_order(np.ascontiguousarray(s.T))       # helper takes [K/G][N]
    return layout.pack_u4(codes), _bf16_round(dev).reshape(N // 64, K // group, 64)


def convert_to_g128(src_dir, dst_dir, layer, H, I, group=128):
    """Rewrites layer `layer`'s per-row files as one group-format file: codes unchanged, every row scale repeated over the
    row's K/128 groups and rounded to bf16."""
    lf = LayerFiles(src_dir, layer)
    out, bf = {}, []
    for e in lf.expert_ids():
        for m in MATS:
            N, K = (I, H) if m != "down" else (H, I)
            q = np.asarray(lf.get(f"{e}.{m}.q")).reshape(-1)
            s = np.asarray(lf.get(f"{e}.{m}.s"), dtype=np.float32).reshape(-1)
            if q.size != N * K // 2 or s.size != N:
                raise FormatError(f"expert {e} {m}: sizes do not match N = {N}, K = {K}")
            rep = np.repeat(s[None, :], K // group, axis=0)                  # [K/G][N]
            out[f"{e}.{m}.q"] = q
            out[f"{e}.{m}.s"] = _bf16_round(layout.group_scales_device_order(rep)).reshape(N // 64, K // group, 64)
            bf.append(f"{e}.{m}.s")
    os.makedirs(dst_dir, exist_ok=True)
    write_layer(os.path.join(dst_dir, f"layer{layer}.safetensors"), out, bf16=bf)


# ----------------------------------------------------------------------------------------------------------------------
def load_layer(u4dir, layer, H, I, device, topk=8, placement=None, rank=0, world=1, shared=None):
    """Experts of `layer` into HBM on `device` -> hecate_b200.moe.ExpertTables.

    placement: the layer's entry of the placement file (or None): router position i is expert `perm[i]`. Without it the
    positions are the file's expert ids in ascending order. With world > 1 the rank keeps positions
    [rank * n / world, (rank + 1) * n / world) (`hecate_b200.ep.shard_plan`), so local slot j is position lo + j.
    shared: None, or the id under which the shared expert is stored (same format as a routed expert).
    The format is read off the scale tensors: F32 [N] = per row (group 0), BF16 [N/64][K/128][64] = group 128."""
    import torch
    from . import moe
    lf = LayerFiles(u4dir, layer)
    ids = [int(e) for e in placement["perm"]] if placement is not None else [e for e in lf.expert_ids() if e != shared]
    n = len(ids)
    if n % world:
        raise ValueError("the number of experts must be a multiple of the world size")
    lo, n_local = rank * (n // world), n // world
    fmt = lf.dtype(f"{ids[0]}.gate.s")
    group = 0 if fmt == "F32" else 128
    if fmt not in ("F32", "BF16"):
        raise FormatError(f"scale dtype {fmt} is neither the per-row (F32) nor the group (BF16) format")

    def up(e, m, t):
        a = np.asarray(lf.get(f"{e}.{m}.{t}"))
        N, K = (I, H) if m != "down" else (H, I)
        want = N * K // 2 if t == "q" else (N if group == 0 else N * K // 128)
        if a.size != want:
            raise FormatError(f"{e}.{m}.{t}: {a.size} elements, expected {want}")
        x = torch.from_numpy(np.ascontiguousarray(a).reshape(-1)).to(device)
        return x if t == "q" or group == 0 else x.view(torch.bfloat16)

    cols = {k: [] for k in ("gq", "uq", "dq", "gs", "us", "ds")}
    for e in ids[lo:lo + n_local]:
        for m, c in zip(MATS, "gud"):
            cols[c + "q"].append(up(e, m, "q")); cols[c + "s"].append(up(e, m, "s"))
    sh = None
    if shared is not None:
        sh = tuple(up(shared, m, t) for t in ("q", "s") for m in MATS)
    return moe.ExpertTables(H, I, topk, cols["gq"], cols["uq"], cols["dq"], cols["gs"], cols["us"], cols["ds"], group=group,
                            shared=sh, device=device)


def load_placement(path, layer):
    """The entry of layer `layer` in a placement file ({layer: {"perm": [...], "hot": n, "far": m, "first": n + m}})."""
    with open(path) as f:
        d = json.load(f)
    e = d.get(str(layer), d.get(layer))
    if e is None or "perm" not in e:
        raise FormatError(f"{path}: no placement for layer {layer}")
    if sorted(e["perm"]) != list(range(len(e["perm"]))):
        raise FormatError(f"{path}: perm of layer {layer} is not a permutation")
    return e


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="rewrite per-row int4 layer files in the group-128 bf16 format")
    ap.add_argument("src"); ap.add_argument("dst"); ap.add_argument("--layer", type=int, required=True)
    ap.add_argument("--hidden", type=int, default=6144); ap.add_argument("--inter", type=int, default=2048)
    a = ap.parse_args()
    convert_to_g128(a.src, a.dst, a.layer, a.hidden, a.inter)
