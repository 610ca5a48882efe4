"""Generates the golden fixtures of tests/golden from the reference itself. Run in a container that has the reference
tree (HECATE_REFERENCE_ROOT, or a folder `reference` beside this repository) and the oracle/_ref build:

    python tests/golden/make_golden.py

Writes
  cpuband_jobs.npz   outputs of the reference CPU expert engine (runtime/tier/cpuband.cpp, compiled unchanged by
                     oracle/build.py) on seeded jobs; inputs are regenerated from the seeds by hecate_b200.synth
  pick_groups.json   row-block tables returned by the reference's pick_groups (runtime/tier/rtx_split.py:236-255), executed
                     from its source text
  layout.npz         bytes written by the reference's pack_u4 (tools/quant/gptq_int4.py:74-77) and codes recovered by its
                     _unpack_moe4 / _rowmajor_i4 (runtime/tier/tier_split.py:98-106), executed from their source text
  layout_i8.npz      bytes written by the reference's int8 packer (runtime/core/hecate_runtime.py:43-48), `--only i8`
  quant.npz          scales chosen by the reference's per-row recipe scales_mse (tools/quant/gptq_int4.py:62-71, with its
                     candidate list U4F, :38), executed from its source text on a seeded matrix (`--only quant` writes just this)
No reference source is copied: the functions are compiled from the files where they lie at generation time only.
"""
import ast
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from hecate_b200 import synth  # noqa: E402
from oracle import build, oracle as O  # noqa: E402

REF = build.ref_root() or ""

# the seeded engine jobs, shared with tests/test_oracle_golden.py
JOB_SEED, JOB_LO, JOB_EXPERTS = 11, 144, 6
JOBS = [dict(R=1, scale=1.0), dict(R=3, scale=0.3), dict(R=5, scale=1.0), dict(R=8, scale=4.0)]


def job_inputs(j, spec):
    """x fp16 [R][6144], sel int64 [R][8] (a mix of band ids 144..149 and foreign ids), rw fp16 [R][8]."""
    R = spec["R"]
    x = synth.activations(JOB_SEED + j, 0, R, 6144, spec["scale"]).astype(np.float16)
    u = synth.uniform(JOB_SEED + j, 777, R * 8).reshape(R, 8)
    sel = np.zeros((R, 8), dtype=np.int64)
    for r in range(R):
        pool = list(range(JOB_LO - 3, JOB_LO + JOB_EXPERTS + 3))
        order = np.argsort(synth.uniform(JOB_SEED + j, 900 + r, len(pool)), kind="stable")
        sel[r] = [pool[i] for i in order[:8]]
    rw = (u * 0.4 + 0.01).astype(np.float16)
    return x, sel, rw


def job_experts():
    H, I = 6144, 2048
    ex = []
    for e in range(JOB_EXPERTS):
        ex.append(O.Expert(synth.packed_codes(JOB_SEED, 0, "gate_q", e, I, H), synth.packed_codes(JOB_SEED, 0, "up_q", e, I, H),
                           synth.packed_codes(JOB_SEED, 0, "down_q", e, H, I), synth.scales(JOB_SEED, 0, "gate_s", e, I, H, H),
                           synth.scales(JOB_SEED, 0, "up_s", e, I, H, H), synth.scales(JOB_SEED, 0, "down_s", e, H, I, I), H, I))
    return ex


def _function_from(path, name, glb):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            exec(compile(mod, path, "exec"), glb)
            return glb[name]
    raise KeyError(name)


def _assignment_from(path, name, glb):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id == name for t in node.targets):
            exec(compile(ast.Module(body=[node], type_ignores=[]), path, "exec"), glb)
            return glb[name]
    raise KeyError(name)


def quant_matrix():
    """The seeded matrix of quant.npz: 24 rows x 256 columns, rows of very different magnitude."""
    w = synth.normal(21, 5150, 24 * 256).reshape(24, 256).astype(np.float32)
    return w * (10.0 ** np.linspace(-3, 1, 24, dtype=np.float32))[:, None]


def write_quant():
    import torch
    path = os.path.join(REF, "tools/quant/gptq_int4.py")
    glb = {"torch": torch, "dev": "cpu"}
    _assignment_from(path, "U4F", glb)
    scales_mse = _function_from(path, "scales_mse", glb)
    W = quant_matrix()
    s = scales_mse(torch.from_numpy(W)).numpy()
    np.savez_compressed(os.path.join(HERE, "quant.npz"), scales=s, u4f=glb["U4F"].numpy())
    print("quant.npz written")


def write_layout_i8():
    """layout_i8.npz: bytes written by the reference's int8 packer _pack and codes recovered by its _codes
    (runtime/core/hecate_runtime.py:38-48), executed from their source text."""
    import torch
    path = os.path.join(REF, "runtime/core/hecate_runtime.py")
    glb = {"torch": torch}
    pack = _function_from(path, "_pack", glb)
    codes_of = _function_from(path, "_codes", glb)
    N, K = 128, 96
    codes = synth.rand_bytes(6, 424242, N * K).reshape(N, K).astype(np.uint8)
    q, spw = pack(torch.from_numpy(codes))
    assert spw == 4 and np.array_equal(codes_of(q, N, K, spw).numpy(), codes)
    np.savez_compressed(os.path.join(HERE, "layout_i8.npz"), codes=codes, packed=q.numpy())
    print("layout_i8.npz written")


def main():
    import torch
    if "--only" in sys.argv:
        what = sys.argv[sys.argv.index("--only") + 1]
        return write_quant() if what == "quant" else write_layout_i8()
    build.build_oracle(); assert build.build_ref(), "needs the reference tree"
    # 1. engine jobs
    ex = job_experts()
    eng = O.RefEngine(ex, JOB_LO, threads=min(8, os.cpu_count() or 1))
    outs = {}
    for j, spec in enumerate(JOBS):
        x, sel, rw = job_inputs(j, spec)
        out, _ = eng.job(x, sel, rw)
        outs[f"out{j}"] = out
        outs[f"xsum{j}"] = np.array([x.astype(np.float64).sum(), float(sel.sum()), rw.astype(np.float64).sum()])
    eng.stop()
    np.savez_compressed(os.path.join(HERE, "cpuband_jobs.npz"), **outs)
    # 2. pick_groups
    pg = _function_from(os.path.join(REF, "runtime/tier/rtx_split.py"), "pick_groups", {"np": np})
    cases = []
    fixed = [([3, 0, 130, 5, 70], 64), ([300, 2], 256), ([0, 0, 0], 64), ([64], 64), ([65], 64), ([1] * 7, 256), ([257, 0, 512, 511], 256)]
    for c, bm in fixed:
        for bal in (False, True):
            g = list(pg(c, 1 << 30, bm, bal))
            cases.append(dict(counts=c, bm=bm, balance=bal, rbt=[x.tolist() for _, _, x in g][0] if g else [], span=[g[0][0], g[0][1]] if g else [0, 0]))
    for seed in range(6):
        c = (synth.uniform(seed, 4242, 40) ** 3 * 700).astype(int).tolist()
        for bm in (64, 256):
            for bal in (False, True):
                g = list(pg(c, 1 << 30, bm, bal))
                cases.append(dict(counts=c, bm=bm, balance=bal, rbt=g[0][2].tolist(), span=[g[0][0], g[0][1]]))
    json.dump(cases, open(os.path.join(HERE, "pick_groups.json"), "w"))
    # 3. layout
    pack_u4 = _function_from(os.path.join(REF, "tools/quant/gptq_int4.py"), "pack_u4", {"torch": torch})
    glb = {"torch": torch}
    unpack = _function_from(os.path.join(REF, "runtime/tier/tier_split.py"), "_unpack_moe4", glb)
    rowmajor = _function_from(os.path.join(REF, "runtime/tier/tier_split.py"), "_rowmajor_i4", glb)
    N, K = 128, 192
    codes = (synth.rand_bytes(5, 31337, N * K) & 15).reshape(N, K).astype(np.uint8)
    q = pack_u4(torch.from_numpy(codes)).numpy()
    assert np.array_equal(unpack(torch.from_numpy(q), N, K).numpy(), codes)
    rm = rowmajor(torch.from_numpy(q), N, K).numpy()
    np.savez_compressed(os.path.join(HERE, "layout.npz"), codes=codes, packed=q, rowmajor=rm)
    write_quant()
    write_layout_i8()
    print("golden fixtures written")


if __name__ == "__main__":
    main()
