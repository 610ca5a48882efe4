"""Expert-parallel decode on GPUs: the peer-memory combine against the single-GPU result (needs 2 GPUs, else skipped), and
the bounded wait of the combine kernel when a peer never signals (1 GPU, no fault: the kernel gives up and reports it)."""
import ctypes as C
import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_combine_wait_is_bounded_and_reported():
    """A 'peer' whose flag nobody ever raises: the combine kernel waits about two seconds, sets the status bit, adds
    nothing, and the context stays usable."""
    import torch
    from hecate_b200 import moe
    from hecate_b200._lib import lib, vp
    dev = torch.device("cuda:0")
    H, rows = 256, 4
    slot_floats = 16 * H
    own = torch.zeros(2 * slot_floats + 64, dtype=torch.float32, device=dev)
    dead = torch.zeros(2 * slot_floats + 64, dtype=torch.float32, device=dev)      # stands in for a peer that never arrives
    own[:rows * H] = 1.0
    slots = (C.c_void_p * 2)(own.data_ptr(), dead.data_ptr())
    flags = (C.c_void_p * 2)(own.data_ptr() + 2 * slot_floats * 4, dead.data_ptr() + 2 * slot_floats * 4)
    f = torch.zeros(rows, H, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    gen = torch.full((1,), 2, dtype=torch.int32, device=dev)               # the step counter lives in device memory
    rc = lib().hmoe_ep_combine(C.c_int(0), C.c_int(2), slots, flags, vp(gen), vp(f), C.c_int(rows), C.c_int(H), C.c_size_t(slot_floats),
                               vp(status), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == 0
    torch.cuda.synchronize()
    assert int(status.item()) & 1 == 1                       # the wait gave up
    assert float(f.abs().max()) == 0.0                       # and nothing was combined
    status.zero_()
    # the same call with the peer's flag raised completes and sums both slots (generation 2 -> slot 0)
    own_flags = own[2 * slot_floats:].view(torch.int32); own_flags[1] = 2
    dead[:rows * H] = 0.5
    rc = lib().hmoe_ep_combine(C.c_int(0), C.c_int(2), slots, flags, vp(gen), vp(f), C.c_int(rows), C.c_int(H), C.c_size_t(slot_floats),
                               vp(status), C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0 and int(status.item()) == 0
    assert torch.allclose(f, torch.full_like(f, 1.5))


def _rank_main(rank, world, port, out_path):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from helpers import HostLayer
    from hecate_b200 import moe, synth
    from hecate_b200.ep import EpDecoder, shard_plan
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    H, I, E, R = 512, 256, 16, 16
    p = shard_plan(rank, world, E)
    local = HostLayer(0, 0, H, I, range(p["lo"], p["lo"] + p["n_local"]), 128, True).upload(dev)
    x = torch.from_numpy(synth.activations(1, 0, R, H)).to(dev).half()
    res = {}
    for mode in (True, "separate", False):                  # peer combine as the down launch's tail, as its own kernel, NCCL all-reduce
        dec = EpDecoder(rank, world, local, E, dev, dist, use_peer=bool(mode), fused_tail=(mode is True))
        outs = []
        for stepi in range(4):                                # several steps: both slots and the generation logic get used
            sel, rw = synth.zipf_routing(10 + stepi, 0, R, E, 8, 0.0)
            f = torch.zeros(R, H, device=dev)
            dec.step(x, torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), f)
            outs.append(f)
        assert dec.status() == 0
        res[mode] = torch.stack(outs)
        if dec.peer is not None:
            dist.barrier(); dec.peer.close()
    # data-parallel tokens: every rank passes only its own rows (rank, rank + world, ...); dispatch and combine over peer memory
    dp_err = torch.zeros(1, device=dev)
    for fused in (True, False):
        dec = EpDecoder(rank, world, local, E, dev, dist, use_peer=True, fused_tail=fused)
        own = dec.own_rows(R)
        outs = []
        for stepi in range(4):
            sel, rw = synth.zipf_routing(10 + stepi, 0, R, E, 8, 0.0)
            f_own = torch.zeros(len(own), H, device=dev)
            dec.step_dp(x[own].contiguous(), torch.from_numpy(sel[own]).to(dev), torch.from_numpy(rw[own]).to(dev), f_own, R)
            outs.append(f_own)
        assert dec.status() == 0 and dec.dispatch_bytes(R) == (world - 1) * len(own) * (H * 2 + 80)
        dp = torch.stack(outs)
        dist.barrier(); dec.peer.close()
        dp_err = torch.maximum(dp_err, torch.tensor([float((dp - res[True][:, own]).abs().max() / res[True].abs().max())], device=dev))
    # the same in four launches: the router's launch is the dispatch and the set-up (every rank routes all rows itself)
    wt = torch.from_numpy(synth.router_weight(7, 0, 32, H)).to(dev).to(torch.float16)
    for fused in (False, True):
        dec = EpDecoder(rank, world, local, E, dev, dist, use_peer=True, fused_tail=fused)
        own = dec.own_rows(R)
        for stepi in range(3):
            xs = torch.from_numpy(synth.activations(30 + stepi, 0, R, H)).to(dev).half()
            sel_f = torch.empty(R, 8, dtype=torch.int64, device=dev); rw_f = torch.empty(R, 8, dtype=torch.float16, device=dev)
            f_own = torch.zeros(len(own), H, device=dev)
            dec.step_dp_fused(xs[own].contiguous(), wt, None, 1.0, sel_f, rw_f, f_own, R)      # 32 router rows, 16 experts: ids >= 16 are foreign to every rank
            # reference: the separate router on all rows, then the replicated-rows step
            sel_r = torch.empty(R, 8, dtype=torch.int64, device=dev); rw_r = torch.empty(R, 8, dtype=torch.float16, device=dev)
            moe.router_fused(xs, wt, None, None, None, sel_r, rw_r, 8, 1.0)
            f_all = torch.zeros(R, H, device=dev)
            dec.step(xs, sel_r, rw_r, f_all)
            assert torch.equal(sel_f, sel_r) and torch.equal(rw_f.view(torch.int16), rw_r.view(torch.int16))
            dp_err = torch.maximum(dp_err, torch.tensor([float((f_own - f_all[own]).abs().max() / f_all.abs().max())], device=dev))
        assert dec.status() == 0
        dist.barrier(); dec.peer.close()
    # Every expert on two ranks (at 2 ranks: both hold all of them, rank 1 in the order band 1, band 0): each step gives every
    # picked expert to one of its holders by the same rule on both ranks, so the combined result is the single-GPU one and the
    # two ranks' work lists together hold every picked expert exactly once.
    from hecate_b200.ep import replica_owners
    E2 = 32
    wt2 = torch.from_numpy(synth.router_weight(8, 0, E2, H)).to(dev).to(torch.float16)
    npr2 = E2 // world
    ids2 = [(rank * npr2 + i) % E2 for i in range(2 * npr2)]
    both = HostLayer(0, 0, H, I, ids2, 128, True).upload(dev)
    full2 = HostLayer(0, 0, H, I, range(E2), 128, True).upload(dev)
    dec = EpDecoder(rank, world, both, E2, dev, dist, use_peer=True, replicas=2)
    own = dec.own_rows(R)
    ws2 = moe.decode_workspace(H, I, dev)
    for stepi in range(3):
        xs = torch.from_numpy(synth.activations(40 + stepi, 0, R, H)).to(dev).half()
        sel_f = torch.empty(R, 8, dtype=torch.int64, device=dev); rw_f = torch.empty(R, 8, dtype=torch.float16, device=dev)
        f_own = torch.zeros(len(own), H, device=dev)
        dec.step_dp_fused(xs[own].contiguous(), wt2, None, 1.0, sel_f, rw_f, f_own, R)
        y_ref = torch.zeros(R, H, device=dev)
        moe.decode(full2, xs, sel_f, rw_f, y_ref, ws2)
        dp_err = torch.maximum(dp_err, torch.tensor([float((f_own - y_ref[own]).abs().max() / y_ref.abs().max())], device=dev))
        owners = replica_owners(sel_f.cpu().numpy(), E2, world)
        m_dev = torch.tensor([float(moe.route_distinct(dec.ws))], device=dev)
        m_all = [torch.zeros_like(m_dev) for _ in range(world)]
        dist.all_gather(m_all, m_dev)
        assert [int(t.item()) for t in m_all] == [sum(1 for o in owners.values() if o == r) for r in range(world)]
    assert dec.status() == 0
    dist.barrier(); dec.peer.close()
    dist.all_reduce(dp_err, op=dist.ReduceOp.MAX)
    sep_err = torch.tensor([float((res["separate"] - res[True]).abs().max() / res[True].abs().max())], device=dev)
    dist.all_reduce(sep_err, op=dist.ReduceOp.MAX)
    dp_err = torch.maximum(dp_err, sep_err)
    # The reference's int8 shared expert beside the int4 routed experts, at a shape whose two small kernels leave most blocks
    # without work: the programmatic launch chain must still order the step counter and the partial slot (every rank adds its
    # share of the shared expert's rows into the slot of THIS step).
    from hecate_b200 import layout as LY
    mk8 = lambda s_, N, K: (synth.rand_bytes(13, s_, N * K).reshape(N, K).astype(np.uint8), np.exp(synth.normal(13, s_ + 50, N) * 0.5 - 7.5).astype(np.float32))
    ex8 = (mk8(1, I, H), mk8(2, I, H), mk8(3, H, I))
    up = lambda a_: torch.from_numpy(np.ascontiguousarray(a_)).to(dev)
    sh8 = tuple(up(LY.pack_i8(c)) for c, _ in ex8) + tuple(up(s_) for _, s_ in ex8)
    base = HostLayer(0, 0, H, I, range(p["lo"], p["lo"] + p["n_local"]), 128, False).upload(dev)
    t8 = moe.ExpertTables(H, I, 8, *[base.keep[i] for i in range(6)], group=128, shared=sh8, device=dev, shared_i8=True)
    i8_err = torch.zeros(1, device=dev)
    dec = EpDecoder(rank, world, t8, E, dev, dist, use_peer=True)
    outs8 = []
    for stepi in range(4):
        sel, rw = synth.zipf_routing(10 + stepi, 0, R, E, 8, 0.0)
        f = torch.zeros(R, H, device=dev)
        dec.step(x, torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), f)
        outs8.append(f)
    assert dec.status() == 0
    dist.barrier(); dec.peer.close()
    if rank == 0:
        full8 = HostLayer(0, 0, H, I, range(E), 128, False).upload(dev)
        tf8 = moe.ExpertTables(H, I, 8, *[full8.keep[i] for i in range(6)], group=128, shared=sh8, device=dev, shared_i8=True)
        ws8 = moe.decode_workspace(H, I, dev)
        for stepi in range(4):
            sel, rw = synth.zipf_routing(10 + stepi, 0, R, E, 8, 0.0)
            y = torch.zeros(R, H, device=dev)
            moe.decode(tf8, x, torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws8)
            i8_err = torch.maximum(i8_err, ((outs8[stepi] - y).norm() / y.norm()).reshape(1))
    # all ranks hold the same bits after the peer combine (fixed rank order)
    mine = res[True].clone()
    others = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(others, mine)
    same = all(torch.equal(o, mine) for o in others)
    if rank == 0:
        full = HostLayer(0, 0, H, I, range(E), 128, True).upload(dev)
        ws = moe.decode_workspace(H, I, dev)
        refs = []
        for stepi in range(4):
            sel, rw = synth.zipf_routing(10 + stepi, 0, R, E, 8, 0.0)
            y = torch.zeros(R, H, device=dev)
            moe.decode(full, x, torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), y, ws)
            refs.append(y)
        ref = torch.stack(refs)
        np.save(out_path, np.array([float(same), float((res[True] - ref).norm() / ref.norm()), float((res[False] - ref).norm() / ref.norm()),
                                    float(dp_err.item()), float(i8_err.item())]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_peer_combine_matches_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "ep.npy")
    mp.spawn(_rank_main, args=(2, 29600 + os.getpid() % 2000, out), nprocs=2, join=True)
    same, err_peer, err_nccl, err_dp, err_i8 = np.load(out)
    assert same == 1.0
    assert err_peer < 1e-3 and err_nccl < 1e-3
    assert err_dp < 1e-3                 # dispatched rows give what replicated rows give (the sums differ only in their atomic order)
    assert err_i8 < 1e-3                 # int8 shared expert under expert parallelism = the single-GPU result


def _prefill_rank_main(rank, world, port, out_path):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    from helpers import HostLayer
    from hecate_b200 import moe, synth
    from hecate_b200.ep import EpPrefill, shard_plan
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    H, I, E, R = 256, 128, 8, 320
    rpr = R // world
    p = shard_plan(rank, world, E)
    local = HostLayer(0, 0, H, I, range(p["lo"], p["lo"] + p["n_local"]), 128, True).upload(dev)
    xa = synth.activations(1, 0, R, H); sel, rw = synth.zipf_routing(2, 0, R, E, 8, 1.1)
    sl = slice(rank * rpr, (rank + 1) * rpr)
    errs = []
    outs = {}
    for use_peer in (False, True, "short"):
        # 320 rows in total: few enough for the streaming kernels ("short": hmoe_short_prefill_ep + reduce-scatter); the other two arms
        # keep the grouped GEMMs
        ep = EpPrefill(rank, world, local, E, rpr, dev, dist, use_peer=use_peer is True, short=use_peer == "short")
        assert ep.short == (use_peer == "short")
        out = torch.empty(rpr, H, device=dev)
        for _ in range(2):                     # twice: the second step reuses the zeroed peer buffer and the next barrier generation
            ep.step(torch.from_numpy(xa[sl]).to(dev).to(torch.bfloat16), torch.from_numpy(sel[sl]).to(dev), torch.from_numpy(rw[sl]).to(dev), out)
        assert ep.status() == 0
        outs[use_peer] = out
    # A placement by load with copies of the hottest experts (hecate_b200.placement): rank r loads the experts at positions
    # [r * slots, (r + 1) * slots) of the plan, the selection is expressed in positions; the result must be the contiguous one.
    from hecate_b200 import placement as PL
    plan = PL.balance(PL.pick_counts(sel, E), world, extra_slots=2)
    ids = plan.perm[rank * plan.slots:(rank + 1) * plan.slots]
    placed = HostLayer(0, 0, H, I, ids, 128, True).upload(dev)
    selp = PL.positions(sel, plan)
    assert max(len(c) for c in plan.copies) > 1 and plan.imbalance() <= PL.contiguous(PL.pick_counts(sel, E), world).imbalance()
    ep = EpPrefill(rank, world, placed, len(plan.perm), rpr, dev, dist, use_peer=True)
    out_p = torch.empty(rpr, H, device=dev)
    ep.step(torch.from_numpy(xa[sl]).to(dev).to(torch.bfloat16), torch.from_numpy(selp[sl]).to(dev), torch.from_numpy(rw[sl]).to(dev), out_p)
    assert ep.status() == 0
    gathered_placed = [torch.empty_like(out_p) for _ in range(world)]
    dist.all_gather(gathered_placed, out_p)
    # Dispatch as an all-to-all-v over peer memory. A routing in which two rows of three select experts of their own rank only
    # (the other rank's picks replaced by ids no rank holds): those rows must not travel, and the rank that does not get them
    # must not read them. The first step sends every row everywhere with large values, which stay in the staging areas
    # where the second step stores nothing.
    sel_v = sel.copy()
    owner = np.arange(R) // rpr
    keep_home = (np.arange(R) % 3 != 0)[:, None] & (sel_v // p["n_local"] != owner[:, None])
    sel_v[keep_home] = 1000
    outs_v = {}
    sent_ok = True
    for use_peer in (False, True):
        ep = EpPrefill(rank, world, local, E, rpr, dev, dist, use_peer=use_peer, dispatch="peer", short=False)
        out_v = torch.empty(rpr, H, device=dev)
        ep.step(torch.from_numpy(xa[sl] * 50).to(dev).to(torch.bfloat16), torch.from_numpy(sel[sl]).to(dev), torch.from_numpy(rw[sl]).to(dev), out_v)
        s0 = int(ep.sent.item())
        ep.step(torch.from_numpy(xa[sl]).to(dev).to(torch.bfloat16), torch.from_numpy(sel_v[sl]).to(dev), torch.from_numpy(rw[sl]).to(dev), out_v)
        assert ep.status() == 0
        want = int(((sel_v[sl] < E) & (sel_v[sl] // p["n_local"] != rank)).any(axis=1).sum())
        sent_ok &= s0 == rpr * (world - 1) and int(ep.sent.item()) - s0 == want and want < rpr
        outs_v[use_peer] = out_v
    assert sent_ok
    gathered_v = {k: [torch.empty_like(v) for _ in range(world)] for k, v in outs_v.items()}
    for k in outs_v:
        dist.all_gather(gathered_v[k], outs_v[k])
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, outs[True])
    gathered_nccl = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered_nccl, outs[False])
    gathered_short = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered_short, outs["short"])
    if rank == 0:
        full = HostLayer(0, 0, H, I, range(E), 128, True).upload(dev)
        ws = moe.prefill_workspace(R, 8, E, H, I, dev)
        ref = torch.zeros(R, H, device=dev)
        moe.prefill(full, torch.from_numpy(xa).to(dev).to(torch.bfloat16), torch.from_numpy(sel).to(dev), torch.from_numpy(rw).to(dev), ref, ws)
        got = torch.cat(gathered); got_nccl = torch.cat(gathered_nccl); got_placed = torch.cat(gathered_placed)
        ref_v = torch.zeros(R, H, device=dev)
        moe.prefill(full, torch.from_numpy(xa).to(dev).to(torch.bfloat16), torch.from_numpy(sel_v).to(dev), torch.from_numpy(rw).to(dev), ref_v, ws)
        ev = [float((torch.cat(gathered_v[k]) - ref_v).norm() / ref_v.norm()) for k in (False, True)]
        np.save(out_path, np.array([float((got - ref).norm() / ref.norm()), float((got_nccl - ref).norm() / ref.norm()),
                                    float((got_placed - ref).norm() / ref.norm())] + ev + [float((torch.cat(gathered_short) - ref).norm() / ref.norm())]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_prefill_matches_single_gpu(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    out = str(tmp_path / "epp.npy")
    mp.spawn(_prefill_rank_main, args=(2, 29700 + os.getpid() % 2000, out), nprocs=2, join=True)
    e = np.load(out)
    assert e[0] < 1e-3 and e[1] < 1e-3, e        # peer-memory combine, NCCL reduce-scatter combine
    assert e[2] < 1e-3, e                         # experts placed by load with copies: same result as contiguous ids
    assert e[3] < 1e-3 and e[4] < 1e-3, e        # peer-memory all-to-all-v dispatch, with either combine
    assert e[5] < 1e-3, e                         # local experts through the streaming kernels (short prefill), reduce-scatter combine
