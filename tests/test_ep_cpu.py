"""Expert-parallel host logic on CPU ranks (gloo, world size 2): the expert ranges and the shared-row split cover the layer
exactly once, and partials summed over ranks equal the single-rank result."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_plan_covers_everything_once():
    from hecate_b200.ep import shard_plan
    for world in (1, 2, 4, 8):
        seen = np.zeros(256, dtype=int)
        rows = np.zeros(16, dtype=int)
        for r in range(world):
            p = shard_plan(r, world, 256)
            seen[p["lo"]:p["lo"] + p["n_local"]] += 1
            rows[[i for i in range(16) if i % p["shared_mod"] == p["shared_rem"]]] += 1
        assert (seen == 1).all() and (rows == 1).all()
    with pytest.raises(ValueError):
        shard_plan(0, 3, 256)


def test_replica_owners_serve_every_pick_once_and_level_the_load():
    """Every expert on two ranks: each picked position gets one of its two holders, and the most loaded rank serves fewer experts
    than under the one-holder split (averaged over routings; never more than one above the mean at 2 ranks)."""
    from hecate_b200 import synth
    from hecate_b200.ep import replica_owners
    for world in (2, 4, 8):
        npr = 256 // world
        worst_one, worst_two = [], []
        for seed in range(20):
            sel, _ = synth.zipf_routing(seed, 0, 16, 256, 8, 0.0)
            own = replica_owners(sel, 256, world)
            ids = np.unique(sel)
            assert sorted(own) == list(ids)
            for e, r in own.items():
                assert r in (e // npr, (e // npr - 1) % world)
            load = np.bincount(list(own.values()), minlength=world)
            worst_two.append(load.max()); worst_one.append(np.bincount(ids // npr, minlength=world).max())
            if world == 2:
                assert load.max() - load.min() <= 1
        assert np.mean(worst_two) <= np.mean(worst_one) - (0 if world == 2 else 1.5)
    assert replica_owners(np.array([[300, -1]]), 256, 4) == {}


def test_prefill_destinations_mask():
    """The all-to-all-v's row routing: a row goes to the ranks that hold one of its experts; foreign ids go nowhere; the share of
    (row, rank) pairs skipped under uniform top-8 routing is (1 - 1/W)^8."""
    from hecate_b200 import synth
    from hecate_b200.ep import prefill_destinations
    sel = np.array([[0, 1, 2, 3, 4, 5, 6, 7], [0, 64, 128, 192, 1, 65, 129, 193], [255, 255, 255, 255, 255, 255, 255, 999], [-1, 300, 400, 500, 600, 700, 800, 900]])
    m = prefill_destinations(sel, 64, 4)
    assert m.tolist() == [[True, False, False, False], [True, True, True, True], [False, False, False, True], [False, False, False, False]]
    for world in (2, 4, 8):
        s, _ = synth.zipf_routing(5, 0, 4096, 256, 8, 0.0)
        frac = 1.0 - prefill_destinations(s, 256 // world, world).mean()
        assert abs(frac - (1 - 1 / world) ** 8) < 0.02, (world, frac)


def _rank_main(rank, world, port, out_path):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    from helpers import HostLayer
    from hecate_b200 import synth
    from hecate_b200.ep import shard_plan
    from oracle import oracle as O
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    H, I, E, R = 256, 128, 8, 6
    hl = HostLayer(0, 0, H, I, range(E), 128, True)
    ex, sh = hl.oracle_experts(O)
    x = synth.activations(1, 0, R, H).astype(np.float16)
    sel, rw = synth.zipf_routing(2, 0, R, E, 8, 0.0)
    p = shard_plan(rank, world, E)
    # this rank's partial: its experts for all rows, the shared expert for its rows only (as hmoe_decode_ep computes it)
    part = O.moe_forward(H, I, 128, x, sel, rw, p["lo"], ex[p["lo"]:p["lo"] + p["n_local"]], None, mode=1)
    mine = [r for r in range(R) if r % p["shared_mod"] == p["shared_rem"]]
    none = np.full((len(mine), 8), 10 ** 6, dtype=np.int64)
    part[mine] += O.moe_forward(H, I, 128, x[mine], none, rw[mine], 0, [], sh, mode=1)
    t = torch.from_numpy(part.astype(np.float64))
    dist.all_reduce(t)
    if rank == 0:
        full = O.moe_forward(H, I, 128, x, sel, rw, 0, ex, sh, mode=1)
        np.save(out_path, np.stack([t.numpy(), full.astype(np.float64)]))
    dist.barrier()
    dist.destroy_process_group()


def test_partials_over_two_gloo_ranks_equal_single_rank(tmp_path):
    import torch.multiprocessing as mp
    out = str(tmp_path / "ep.npy")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
    got, full = np.load(out)
    assert np.abs(got - full).max() <= 1e-5 * np.abs(full).max()
