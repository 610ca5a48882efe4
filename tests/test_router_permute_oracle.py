"""Router and permutation restatements: defining properties, and the reference's own pick_groups outputs."""
import json
import os

import numpy as np

from hecate_b200 import synth

G = os.path.join(os.path.dirname(__file__), "golden")


def _bits(a, bf16):
    return synth.to_bf16_bits(a) if bf16 else np.asarray(a, dtype=np.float16).view(np.uint16)


def test_router_semantics(oracle):
    R, H, E = 6, 512, 64
    x = synth.activations(3, 0, R, H)
    w = synth.bf16_bits_to_f32(synth.to_bf16_bits(synth.router_weight(3, 0, E, H) * 20)); bias = synth.router_bias(3, 0, E, 0.1)
    sel, rw, lg = oracle.router(_bits(x, True), 1, _bits(w, True), 1, bias, 8, 2.5, want_logits=True)
    ref = x.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(lg - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())
    act = 1.0 / (1.0 + np.exp(-lg.astype(np.float64)))
    key = act + bias
    for r in range(R):
        assert len(set(sel[r])) == 8
        ks = key[r, sel[r]]
        assert np.all(np.diff(ks) <= 1e-7)                                  # selection order = descending key
        assert ks.min() >= np.delete(key[r], sel[r]).max() - 1e-7           # nothing better left out
        wref = act[r, sel[r]] * 2.5 / act[r, sel[r]].sum()
        assert np.abs(rw[r].astype(np.float64) - wref).max() < 2e-3


def test_router_ties_go_to_lower_index(oracle):
    H, E = 256, 32
    x = np.ones((1, H), dtype=np.float32)
    w = np.zeros((E, H), dtype=np.float32)            # all logits 0 -> all keys equal
    sel, rw = oracle.router(_bits(x, False), 0, _bits(w, False), 0, None, 8, 1.0)
    assert list(sel[0]) == list(range(8))
    assert np.allclose(rw.astype(np.float32), 0.125)
    bias = np.zeros(E, dtype=np.float32); bias[20] = 0.5; bias[7] = 0.5
    sel, _ = oracle.router(_bits(x, False), 0, _bits(w, False), 0, bias, 4, 1.0)
    assert list(sel[0]) == [7, 20, 0, 1]


def test_det_exp_accuracy(oracle):
    xs = np.linspace(-30, 30, 2001).astype(np.float32)
    got = np.array([oracle.lib().orc_det_expf(float(v)) for v in xs])
    assert np.abs(got / np.exp(xs.astype(np.float64)) - 1).max() < 3e-7


def test_permute_is_stable_sort(oracle):
    R, E = 300, 64
    sel, rw = synth.zipf_routing(5, 0, R, E, 8, 1.1)
    order, tok, eid, wt, counts = oracle.permute(sel, rw, E)
    fs = sel.reshape(-1)
    ref = np.argsort(fs, kind="stable")
    assert np.array_equal(order, ref.astype(np.int32))
    assert np.array_equal(tok, (ref // 8).astype(np.int32))
    assert np.array_equal(eid, fs[ref].astype(np.int32))
    assert np.array_equal(wt, rw.reshape(-1)[ref].astype(np.float32))
    assert np.array_equal(counts, np.bincount(fs, minlength=E).astype(np.int32))


def test_row_blocks_match_reference_pick_groups(oracle):
    cases = json.load(open(os.path.join(G, "pick_groups.json")))
    assert len(cases) > 30
    for c in cases:
        rbt = oracle.row_blocks(c["counts"], c["bm"], c["balance"])
        want = np.array(c["rbt"], dtype=np.int32).reshape(-1, 4)
        assert np.array_equal(rbt, want), c
        # coverage: every pick in exactly one block, blocks within one expert, sizes <= bm
        cnt = np.zeros(len(c["counts"]), dtype=np.int64)
        for e, first, n, z in rbt:
            assert 0 < n <= c["bm"] and z == 0
            cnt[e] += n
        assert np.array_equal(cnt, np.array(c["counts"]))


def test_zipf_routing_shape():
    sel, rw = synth.zipf_routing(0, 0, 512, 256, 8, 1.1)
    assert sel.shape == (512, 8) and all(len(set(r)) == 8 for r in sel)
    assert np.allclose(rw.astype(np.float32).sum(1), 1.0, atol=2e-3)
    counts = np.bincount(sel.reshape(-1), minlength=256)
    assert counts[:8].sum() > 4 * counts[-8:].sum()        # popularity falls with the expert index
