"""Routing logs in the reference's record format and load-balanced expert placement over GPUs."""
import numpy as np
import pytest

from hecate_b200 import placement as P, synth


def test_route_log_round_trip(tmp_path):
    p = str(tmp_path / "route.bin")
    layers = [3, 4, 77]
    steps = [synth.rand_bytes(1, 5 + i, 3 * r * 8).reshape(3, r, 8).astype(np.int16) for i, r in enumerate((1, 8, 5))]
    P.write_route_log(p, layers, steps[:2])
    P.write_route_log(p, layers, steps[2:], append=True)
    got_layers, got = P.read_route_log(p)
    assert got_layers == layers and len(got) == 3 and all(np.array_equal(a, b) for a, b in zip(got, steps))
    open(p, "ab").write(b"\x01\x02\x03\x04")
    with pytest.raises(ValueError):
        P.read_route_log(p)


def test_step_counts_are_distinct_per_step():
    steps = [np.array([[[0, 0, 1, 2, 3, 4, 5, 6], [0, 9, 9, 9, 9, 9, 9, 9]]], dtype=np.int16)] * 3
    c = P.step_counts([12], steps, n_experts=16)[12]
    assert c[0] == 3 and c[9] == 3 and c[7] == 0
    perm = {12: list(range(15, -1, -1))}
    c2 = P.step_counts([12], steps, n_experts=16, perm_by_layer=perm)[12]
    assert c2[15] == 3 and c2[6] == 3 and c2[0] == 0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_balance_beats_contiguous_under_zipf(world):
    sel, _ = synth.zipf_routing(10, 0, 4096, 256, 8, 1.3)
    counts = P.pick_counts(sel, 256)
    base, plan = P.contiguous(counts, world), P.balance(counts, world)
    assert sorted(plan.perm) == list(range(256)) and plan.slots == 256 // world
    assert plan.imbalance() < base.imbalance() and plan.imbalance() < 1.0 + 0.6 * (base.imbalance() - 1.0)
    # the plan built on one sample holds on another sample of the same popularity
    sel2, _ = synth.zipf_routing(11, 0, 4096, 256, 8, 1.3)
    pos = P.positions(sel2, plan)
    load = np.array([((pos >= r * plan.slots) & (pos < (r + 1) * plan.slots)).sum() for r in range(world)])
    sel_load = np.array([((sel2 >= r * plan.slots) & (sel2 < (r + 1) * plan.slots)).sum() for r in range(world)])
    assert load.max() / load.mean() < sel_load.max() / sel_load.mean()


def test_copies_split_the_hottest_expert():
    sel, _ = synth.zipf_routing(10, 0, 4096, 256, 8, 1.3)
    counts = P.pick_counts(sel, 256)
    plain, rep = P.balance(counts, 8), P.balance(counts, 8, extra_slots=8)
    assert len(rep.perm) == 264 and rep.slots == 33
    hot = int(np.argmax(counts))
    assert len(rep.copies[hot]) >= 2 and len({p // rep.slots for p in rep.copies[hot]}) == len(rep.copies[hot])   # on different GPUs
    assert rep.imbalance() <= plain.imbalance() + 1e-9
    pos = P.positions(sel, rep)
    for e in (hot, 5, 200):
        assert set(np.unique(pos[sel == e])) <= set(rep.copies[e])
    share = np.bincount(pos[sel == hot], minlength=264)[rep.copies[hot]]
    assert share.max() <= 1.2 * share.mean()
    with pytest.raises(ValueError):
        P.balance(counts, 8, extra_slots=3)


def test_permute_router():
    counts = np.arange(16, dtype=np.float64)
    plan = P.balance(counts, 4)
    wt = np.arange(16 * 4).reshape(16, 4); bias = np.arange(16.0)
    w2, b2 = P.permute_router(wt, bias, plan)
    assert all(np.array_equal(w2[p], wt[e]) and b2[p] == bias[e] for p, e in enumerate(plan.perm))
    with pytest.raises(ValueError):
        P.permute_router(wt, bias, P.balance(counts, 4, extra_slots=4))
