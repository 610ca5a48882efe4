"""Pins the CPU checker: bit-identical to outputs of the reference's own CPU expert engine (tests/golden/cpuband_jobs.npz,
produced by tests/golden/make_golden.py from the reference source), and to the engine itself where its build is present."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
import make_golden as MG  # noqa: E402

G = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def experts():
    return MG.job_experts()


def test_checker_reproduces_reference_engine_outputs(oracle, experts):
    z = np.load(os.path.join(G, "cpuband_jobs.npz"))
    for j, spec in enumerate(MG.JOBS):
        x, sel, rw = MG.job_inputs(j, spec)
        chk = np.array([x.astype(np.float64).sum(), float(sel.sum()), rw.astype(np.float64).sum()])
        assert np.array_equal(chk, z[f"xsum{j}"]), "seeded inputs differ from the ones the fixture was made with"
        got = oracle.moe_forward(6144, 2048, 0, x, sel, rw, MG.JOB_LO, experts)
        assert np.array_equal(got.view(np.int32), z[f"out{j}"].view(np.int32)), f"job {j} not bit-identical"
        assert np.abs(got).max() > 0


def test_many_pick_job_equals_one_pick_jobs_in_order(oracle, experts):
    """The property the reference's own test checks (tools/dev/test_grace_picks.py): a job's partial is, bit for bit, the
    sum in pick order of the one-pick jobs of its picks."""
    x, sel, rw = MG.job_inputs(3, MG.JOBS[3])
    lo, n = MG.JOB_LO, MG.JOB_EXPERTS
    got = oracle.moe_forward(6144, 2048, 0, x, sel, rw, lo, experts)
    order = []
    for r in range(sel.shape[0]):
        for e in sel[r]:
            if lo <= e < lo + n and e not in order:
                order.append(int(e))
    assert len(order) >= 3
    ref = np.zeros_like(got)
    for e in order:
        s1 = np.full_like(sel, 0); w1 = np.zeros_like(rw)
        for r in range(sel.shape[0]):
            hit = np.nonzero(sel[r] == e)[0]
            if len(hit):
                s1[r, 0] = e; w1[r, 0] = rw[r, hit[0]]
        ref = ref + oracle.moe_forward(6144, 2048, 0, x, s1, w1, lo, experts)
    assert np.array_equal(ref.view(np.int32), got.view(np.int32))


def test_rows_are_independent_jobs_of_eight(oracle, experts):
    """16 rows are two independent 8-row jobs, like the reference's caller cuts them (tier_split.py:346-354)."""
    x = np.concatenate([MG.job_inputs(3, MG.JOBS[3])[0], MG.job_inputs(2, MG.JOBS[2])[0]])
    sel = np.concatenate([MG.job_inputs(3, MG.JOBS[3])[1], MG.job_inputs(2, MG.JOBS[2])[1]])
    rw = np.concatenate([MG.job_inputs(3, MG.JOBS[3])[2], MG.job_inputs(2, MG.JOBS[2])[2]])
    z = np.load(os.path.join(G, "cpuband_jobs.npz"))
    got = oracle.moe_forward(6144, 2048, 0, x, sel, rw, MG.JOB_LO, experts)
    assert np.array_equal(got[:8].view(np.int32), z["out3"].view(np.int32))
    assert np.array_equal(got[8:].view(np.int32), z["out2"].view(np.int32))


def test_exact_mode_close_to_int8_mode(oracle, experts):
    x, sel, rw = MG.job_inputs(1, MG.JOBS[1])
    a = oracle.moe_forward(6144, 2048, 0, x, sel, rw, MG.JOB_LO, experts, mode=0)
    b = oracle.moe_forward(6144, 2048, 0, x, sel, rw, MG.JOB_LO, experts, mode=1)
    rel = np.linalg.norm(a - b) / np.linalg.norm(b)
    assert 1e-3 < rel < 3e-2       # the int8 activation round trips cost about 1 % (the reason for the act_quant mode)


@pytest.mark.parametrize("variant", ["avx2", "vnni", "scalar"])
def test_against_reference_engine_live(oracle, experts, variant):
    """Every build of the reference engine (the shim's AVX2, AVX-512-VNNI and scalar inner loops) gives the restatement's
    result bit for bit, and therefore the stored golden outputs: the variants differ in speed only."""
    if not oracle.ref_available(variant):
        pytest.skip(f"reference engine build '{variant}' not present (or the host lacks its instructions)")
    eng = oracle.RefEngine(experts, MG.JOB_LO, threads=4, variant=variant)
    try:
        for j, spec in enumerate(MG.JOBS[:3]):
            x, sel, rw = MG.job_inputs(j + 10, spec)
            ref, _ = eng.job(x, sel, rw)
            got = oracle.moe_forward(6144, 2048, 0, x, sel, rw, MG.JOB_LO, experts)
            assert np.array_equal(ref.view(np.int32), got.view(np.int32))
        z = np.load(os.path.join(G, "cpuband_jobs.npz"))
        x, sel, rw = MG.job_inputs(0, MG.JOBS[0])
        ref, _ = eng.job(x, sel, rw)
        assert np.array_equal(ref.view(np.int32), z["out0"].view(np.int32))
    finally:
        eng.stop()


def test_q8_roundtrip_definition(oracle):
    v = np.linspace(-3, 5, 64).astype(np.float32)
    out = oracle.q8_roundtrip(v)
    for i in range(0, 64, 32):
        s = np.float32(np.abs(v[i:i + 32]).max()) / np.float32(127)
        q = np.rint(v[i:i + 32] * (np.float32(1) / s))
        assert np.array_equal(out[i:i + 32], (q * s).astype(np.float32))
    assert np.array_equal(oracle.q8_roundtrip(np.zeros(32, dtype=np.float32)), np.zeros(32, dtype=np.float32))
