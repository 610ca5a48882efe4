"""Expert-parallel decode over the GPUs of one box: one process per GPU (torch.distributed for the set-up plumbing), experts
split by contiguous id ranges, the step's rows replicated on every rank, partial outputs combined over NVLink peer memory
by `hmoe_ep_combine` (or, as the baseline, by an NCCL all-reduce).

The reference has no expert parallelism; the shape kept from it is its band split: every band receives all rows with
(sel, rw), ignores foreign ids and returns an fp32 partial that is added in a fixed order (runtime/tier/tier_split.py:3-11,
runtime/tier/moe4/moe4.cu:93,702-717).
"""
import ctypes as C
import json
import os
import time

import numpy as np

from . import moe
from ._lib import check, lib, vp

MAX_ROWS = 16


def shard_plan(rank, world, n_experts):
    """Which part of a layer rank `rank` of `world` serves: experts [lo, lo + n_local) and, of the shared expert, the rows
    r with r % shared_mod == shared_rem."""
    if n_experts % world:
        raise ValueError("the number of experts must be a multiple of the world size")
    n_local = n_experts // world
    return dict(lo=rank * n_local, n_local=n_local, shared_mod=world, shared_rem=rank)


class PeerBuffers:
    """Symmetric buffers of the combine: per rank two fp32 partial slots [MAX_ROWS * H] and `world` generation flags,
    allocated with cudaMalloc by the library, exported with CUDA IPC and opened by every peer."""

    def __init__(self, rank, world, H, device, dist, slot_floats=None):
        import torch
        self.rank, self.world, self.H = rank, world, H
        self.slot_floats = MAX_ROWS * H if slot_floats is None else (slot_floats + 63) // 64 * 64
        self.bytes = 2 * self.slot_floats * 4 + 512          # two slots, `world` flags (256 B), the generation word (256 B)
        p = C.c_void_p()
        check(lib().hmoe_ep_alloc(C.c_size_t(self.bytes), C.byref(p)))
        self.own = p.value
        h = (C.c_ubyte * 64)()
        check(lib().hmoe_ep_export(C.c_void_p(self.own), h))
        handles = [None] * world
        dist.all_gather_object(handles, bytes(h))
        self.base = []
        for r in range(world):
            if r == rank:
                self.base.append(self.own)
            else:
                q = C.c_void_p()
                check(lib().hmoe_ep_open((C.c_ubyte * 64).from_buffer_copy(handles[r]), C.byref(q)))
                self.base.append(q.value)
        self.slots = (C.c_void_p * world)(*self.base)
        self.flags = (C.c_void_p * world)(*[b + 2 * self.slot_floats * 4 for b in self.base])
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.gen_ptr = self.own + 2 * self.slot_floats * 4 + 256
        dist.barrier()

    def close(self):
        for r, b in enumerate(self.base):
            if r != self.rank:
                lib().hmoe_ep_close(C.c_void_p(b))
        lib().hmoe_ep_free(C.c_void_p(self.own))


class EpDecoder:
    """One rank's side of an expert-parallel decode layer."""

    def __init__(self, rank, world, tables, n_experts, device, dist, use_peer=True):
        self.rank, self.world, self.tabs, self.dev, self.dist = rank, world, tables, device, dist
        self.plan = shard_plan(rank, world, n_experts)
        assert tables.n == self.plan["n_local"]
        self.ws = moe.decode_workspace(tables.H, tables.I, device)
        self.use_peer = use_peer and world > 1
        self.peer = PeerBuffers(rank, world, tables.H, device, dist) if self.use_peer else None
        import torch
        self.y = torch.zeros(MAX_ROWS, tables.H, dtype=torch.float32, device=device)
        self.struct = tables.struct()

    def step(self, x, sel, rw, f):
        """f[R][H] (fp32) += the layer's output for rows x with global routing (sel, rw); identical on every rank."""
        import torch
        R = x.shape[0]
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        pl = self.plan
        if self.use_peer:
            check(lib().hmoe_decode_ep(C.byref(self.struct), vp(x), C.c_int(moe._dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(pl["lo"]),
                                       C.c_int(pl["n_local"]), C.c_int(0), C.c_void_p(self.peer.own), vp(self.ws),
                                       C.c_size_t(self.ws.numel()), C.c_int(pl["shared_mod"]), C.c_int(pl["shared_rem"]),
                                       C.c_void_p(self.peer.gen_ptr), C.c_size_t(self.peer.slot_floats), st))
            check(lib().hmoe_ep_combine(C.c_int(self.rank), C.c_int(self.world), self.peer.slots, self.peer.flags, C.c_void_p(self.peer.gen_ptr),
                                        vp(f), C.c_int(R), C.c_int(self.tabs.H), C.c_size_t(self.peer.slot_floats), vp(self.peer.status), st))
        else:
            y = self.y[:R]
            check(lib().hmoe_decode_ep(C.byref(self.struct), vp(x), C.c_int(moe._dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(pl["lo"]),
                                       C.c_int(pl["n_local"]), C.c_int(0), vp(y), vp(self.ws), C.c_size_t(self.ws.numel()),
                                       C.c_int(pl["shared_mod"]), C.c_int(pl["shared_rem"]), None, C.c_size_t(0), st))
            if self.world > 1:
                self.dist.all_reduce(y)
            moe.moe4_combine(f, 0, y, R, 0)
        return f

    def status(self):
        import torch
        torch.cuda.synchronize(self.dev)
        s = moe.ws_status(self.ws)
        if self.peer is not None:
            s |= int(self.peer.status.item())
        return s


class EpPrefill:
    """Expert-parallel prefill. Dispatch: the ranks' token slices are all-gathered (NCCL); every rank runs the grouped GEMMs
    for its experts over all tokens (ids outside [lo, lo + n_local) are dropped by the permutation) plus the shared expert
    for its own tokens. Combine, use_peer = True: the down GEMM adds every row's sums straight into the output of the rank
    that owns the row, over NVLink peer memory, and a flag barrier ends the step. use_peer = False (the baseline): a local
    full-size partial and an NCCL reduce-scatter."""

    def __init__(self, rank, world, tables, n_experts, rows_per_rank, device, dist, use_peer=None):
        import torch
        if use_peer is None:
            # measured at 2 GPUs (32768 rows): the fused combine is 5 % slower than the reduce-scatter it replaces, because every
            # pick of a remote token crosses the link (up to 8 per token) where the reduce-scatter sends one sum per token; the
            # volumes meet at 8 GPUs (one pick per token and GPU on average)
            use_peer = world >= 8
        self.rank, self.world, self.tabs, self.dev, self.dist, self.rpr = rank, world, tables, device, dist, rows_per_rank
        self.plan = shard_plan(rank, world, n_experts)
        R = rows_per_rank * world
        self.R = R
        self.ws = moe.prefill_workspace(R, tables.topk, tables.n, tables.H, tables.I, device)
        self.x_all = torch.empty(R, tables.H, dtype=torch.bfloat16, device=device)
        self.sel_all = torch.empty(R, tables.topk, dtype=torch.int64, device=device)
        self.rw_all = torch.empty(R, tables.topk, dtype=torch.float16, device=device)
        self.use_peer = use_peer and world > 1
        self.struct = tables.struct()
        self.gen = 0
        if self.use_peer:
            # one slot of the symmetric buffer is this rank's output [rows_per_rank][H]; the flags serve the barrier
            self.peer = PeerBuffers(rank, world, tables.H, device, dist, slot_floats=rows_per_rank * tables.H)
            self.out_tab = (C.c_void_p * world)(*self.peer.base)
        else:
            self.peer = None
            self.partial = torch.empty(R, tables.H, dtype=torch.float32, device=device)

    def step(self, x, sel, rw, out):
        """x bf16 [R/W][H], sel, rw: this rank's tokens; out fp32 [R/W][H] receives their MoE output."""
        import torch
        d, pl = self.dist, self.plan
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        nbytes = self.rpr * self.tabs.H * 4
        if self.use_peer:
            # own output cleared before the step's first collective: when the all-gather returns on a peer, this rank has passed it
            check(lib().hmoe_ep_memset(C.c_void_p(self.peer.own), C.c_int(0), C.c_size_t(nbytes), st))
        if self.world > 1:
            d.all_gather_into_tensor(self.x_all, x); d.all_gather_into_tensor(self.sel_all, sel); d.all_gather_into_tensor(self.rw_all, rw)
        else:
            self.x_all.copy_(x); self.sel_all.copy_(sel); self.rw_all.copy_(rw)
        if self.use_peer:
            self.gen += 1
            check(lib().hmoe_prefill_ep_peer(C.byref(self.struct), vp(self.x_all), C.c_int(moe._dt(self.x_all)), vp(self.sel_all), vp(self.rw_all),
                                             C.c_int(self.R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), self.out_tab,
                                             C.c_int(self.world), C.c_int(self.rpr), vp(self.ws), C.c_size_t(self.ws.numel()),
                                             C.c_int(self.rank * self.rpr), C.c_int(self.rpr), st))
            check(lib().hmoe_ep_barrier(C.c_int(self.rank), C.c_int(self.world), self.peer.flags, C.c_uint32(self.gen), vp(self.peer.status), st))
            check(lib().hmoe_ep_copy(vp(out), C.c_void_p(self.peer.own), C.c_size_t(nbytes), st))
            return out
        self.partial.zero_()
        check(lib().hmoe_prefill_ep(C.byref(self.struct), vp(self.x_all), C.c_int(moe._dt(self.x_all)), vp(self.sel_all), vp(self.rw_all),
                                    C.c_int(self.R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), vp(self.partial), vp(self.ws),
                                    C.c_size_t(self.ws.numel()), C.c_int(self.rank * self.rpr), C.c_int(self.rpr), st))
        if self.world > 1:
            d.reduce_scatter_tensor(out, self.partial)
        else:
            out.copy_(self.partial)
        return out

    def status(self):
        import torch
        torch.cuda.synchronize(self.dev)
        s = moe.ws_status(self.ws)
        if self.peer is not None:
            s |= int(self.peer.status.item())
        return s


def bench_prefill(args, world, rank, dev):
    """bench.py --mode prefill for N > 1: args.rows tokens in total, split over the ranks; uniform or Zipf routing."""
    import torch
    import torch.distributed as dist
    import bench as B
    from . import synth
    E, H, I, TOPK = B.E, B.H, B.I, B.TOPK
    R = args.rows
    rpr = R // world
    steps, warmup = min(args.steps, 50), max(3, min(args.warmup, 5))
    sel_all, rw_all = synth.zipf_routing(10, 0, R, E, TOPK, args.zipf)
    # Placement: "contiguous" = expert e on GPU e // (E / world); "balanced" = experts dealt to the GPUs by load
    # (hecate_b200.placement.balance) from the pick counts of ANOTHER sample of the same popularity (the routing log of an
    # earlier chunk), optionally with extra slots for copies of the hottest experts. The selection is then expressed in router
    # positions, as a router with permuted weight rows would emit it.
    from . import placement as PL
    want = getattr(args, "placement", "auto")
    use_plan = want == "balanced" or (want == "auto" and args.zipf > 0)
    base_imb = PL.contiguous(PL.pick_counts(sel_all, E), world).imbalance()
    if use_plan:
        cal, _ = synth.zipf_routing(11, 0, R, E, TOPK, args.zipf)
        plan = PL.balance(PL.pick_counts(cal, E), world, extra_slots=getattr(args, "extra_slots", 0))
        sel_all = PL.positions(sel_all, plan)
        E = len(plan.perm)
    pl = shard_plan(rank, world, E)
    tabs = B.build_layer(dev, 100 + rank, list(range(pl["lo"], pl["lo"] + pl["n_local"])), torch, moe)
    x = torch.from_numpy(synth.activations(rank, 0, rpr, H)).to(torch.bfloat16).to(dev)
    sel = torch.from_numpy(sel_all[rank * rpr:(rank + 1) * rpr]).to(dev); rw = torch.from_numpy(rw_all[rank * rpr:(rank + 1) * rpr]).to(dev)
    out = torch.empty(rpr, H, dtype=torch.float32, device=dev)
    times = {}
    st_all = 0
    launches = 0
    for mode in ("nccl", "peer"):
        ep = EpPrefill(rank, world, tabs, E, rpr, dev, dist, use_peer=(mode == "peer"))
        for _ in range(warmup):
            ep.step(x, sel, rw, out)
        torch.cuda.synchronize(); dist.barrier()
        l0 = moe.launch_count()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with B.ClockSampler(dev.index) as cs:
            torch.cuda.synchronize(); dist.barrier()
            ev0.record()
            for _ in range(steps):
                ep.step(x, sel, rw, out)
            ev1.record()
            torch.cuda.synchronize(); dist.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        times[mode] = float(ms.item())
        launches = moe.launch_count() - l0
        st = torch.tensor([ep.status()], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
        st_all |= int(st.item())
        if ep.peer is not None:
            dist.barrier(); ep.peer.close()
        del ep
    best = min(times, key=times.get)               # both arms are timed; the line reports the faster one and names it
    ms = torch.tensor([times[best]], device=dev)
    st = torch.tensor([st_all], device=dev)
    picks = np.array([int(((sel_all >= r * pl["n_local"]) & (sel_all < (r + 1) * pl["n_local"])).sum()) for r in range(world)])
    if rank == 0:
        flop = 2.0 * (TOPK * R + R) * (3 * I * H)
        t = float(ms.item()) * 1e-3
        peaks = json.load(open(os.path.join(B.ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(B.ROOT, "MEASURED_PEAKS.json")) else {}
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0)) * world
        print(json.dumps({
            "metric": "moe_prefill_expert_gemm_tflops", "value": flop / t / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 -> fp16 x fp16 -> fp32 (tcgen05)", "data": "synthetic",
            "config": {"workload": f"prefill M={R} tokens over {world} GPUs ({rpr} each), Zipf({args.zipf}) top-8 over {E} experts + shared, "
                                   f"{pl['n_local']} expert slots per GPU ({'placed by load from a calibration sample' if use_plan else 'contiguous ids'}), "
                                   f"all-gather dispatch (NCCL), combine: " + ("fused into the down GEMM over NVLink peer memory" if best == "peer" else "NCCL reduce-scatter"),
                       "l2": "inputs larger than L2"},
            "tokens_per_s": R / t, "nccl_reduce_scatter_ms_per_step": times["nccl"], "peer_combine_ms_per_step": times["peer"],
            "dispatch_bytes_per_rank": (world - 1) * rpr * (H * 2 + TOPK * 10), "combine_bytes_per_rank": (world - 1) * rpr * H * 4,
            "picks_per_rank": picks.tolist(), "load_imbalance_max_over_mean": float(picks.max() / picks.mean()),
            "load_imbalance_contiguous_placement": base_imb,
            "roofline": {"bound": "tensor", "kernel": "whole step incl. collectives", "achieved": flop / t / 1e12, "peak": peak, "unit": "TFLOP/s",
                         "frac": flop / t / 1e12 / peak, "peak_kind": "measured (sustained) x n_gpus", "traffic": None},
            "gpu_launches": int(launches), "device_status": int(st.item()), "clocks": cs.summary()}))
    dist.barrier()
    dist.destroy_process_group()


def bench_decode(args, world, rank, dev):
    """bench.py's N > 1 arm: the decode configuration with the 256 experts split over `world` GPUs, the 16 rows replicated
    (strong scaling: the global batch is fixed), combine over peer memory; the NCCL all-reduce variant is timed beside it."""
    import torch
    import torch.distributed as dist
    import bench as B
    from . import synth
    E, H, I, TOPK, ROWS, NBATCH = B.E, B.H, B.I, B.TOPK, B.ROWS, B.NBATCH
    steps, warmup = args.steps, max(3, args.warmup)
    pl = shard_plan(rank, world, E)
    tabs = B.build_layer(dev, 100 + rank, list(range(pl["lo"], pl["lo"] + pl["n_local"])), torch, moe)
    wt = torch.from_numpy(synth.router_weight(0, 0, E, H)).to(dev).to(torch.bfloat16)
    bias = torch.zeros(E, dtype=torch.float32, device=dev)
    xs = [torch.from_numpy(synth.activations(b, 0, ROWS, H)).to(torch.bfloat16).to(dev) for b in range(NBATCH)]
    xs_host = [x.cpu().pin_memory() for x in xs]
    sel = torch.empty(ROWS, TOPK, dtype=torch.int64, device=dev)
    rw = torch.empty(ROWS, TOPK, dtype=torch.float16, device=dev)
    f = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    f_host = torch.empty(ROWS, H, dtype=torch.float32).pin_memory()
    x_in = torch.empty(ROWS, H, dtype=torch.bfloat16, device=dev)
    results = {}
    for mode in ("nccl", "peer"):
        dec = EpDecoder(rank, world, tabs, E, dev, dist, use_peer=(mode == "peer"))

        def step(x):
            moe.router_fused(x, wt, bias, None, None, sel, rw, TOPK, 1.0)
            dec.step(x, sel, rw, f)

        for i in range(warmup):
            step(xs[i % NBATCH])
        torch.cuda.synchronize(); dist.barrier()
        run_step, per_step = B.make_graphed(step, xs, torch, moe, (not args.no_graph) and mode == "peer")
        for i in range(warmup):
            run_step(i % NBATCH)
        torch.cuda.synchronize(); dist.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with B.ClockSampler(dev.index) as cs:
            torch.cuda.synchronize(); dist.barrier()
            ev0.record()
            for i in range(steps):
                run_step(i % NBATCH)
            ev1.record()
            torch.cuda.synchronize(); dist.barrier()
        ms = torch.tensor([ev0.elapsed_time(ev1) / steps], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        launches = per_step * steps
        t0 = time.perf_counter()
        n2 = min(steps, 200)
        for i in range(n2):
            x_in.copy_(xs_host[i % NBATCH], non_blocking=True); step(x_in); f_host.copy_(f, non_blocking=True); torch.cuda.synchronize()
        e2e = torch.tensor([(time.perf_counter() - t0) / n2], device=dev)
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
        st = torch.tensor([dec.status()], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
        results[mode] = dict(ms=float(ms.item()), e2e=float(e2e.item()), launches=int(launches), status=int(st.item()), clocks=cs.summary())
        if dec.peer is not None:
            dist.barrier(); dec.peer.close()
    # load balance of the last batch: distinct local experts per rank
    d_local = torch.tensor([float(((sel >= pl["lo"]) & (sel < pl["lo"] + pl["n_local"])).nonzero().shape[0] and
                                  torch.unique(sel[(sel >= pl["lo"]) & (sel < pl["lo"] + pl["n_local"])]).numel())], device=dev)
    d_all = [torch.zeros_like(d_local) for _ in range(world)]
    dist.all_gather(d_all, d_local)
    if rank == 0:
        r = results["peer"]
        dl = [float(t.item()) for t in d_all]
        peak, kind = B.measured_peaks()
        bytes_rank_max = (max(dl) + 1) * B.EXPERT_BYTES + E * H * 2
        print(json.dumps({
            "metric": B.METRIC, "value": ROWS / (r["ms"] * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int4 x fp16 -> fp32",
            "data": "synthetic",
            "config": {"workload": B.WORKLOAD + f"; experts split over {world} GPUs ({pl['n_local']} each), rows replicated, "
                                                "combine over NVLink peer memory",
                       "l2": "inputs larger than L2: 8 input batches in a ring, each step streams different experts"},
            "us_per_layer": r["ms"] * 1e3, "nccl_allreduce_us_per_layer": results["nccl"]["ms"] * 1e3,
            "distinct_local_experts_last_step": dl, "load_imbalance_max_over_mean": max(dl) / (sum(dl) / len(dl)),
            "combine_bytes_per_rank": (world - 1) * ROWS * H * 4, "dispatch_bytes_per_rank": 0,
            "roofline": {"bound": "hbm", "kernel": "decode kernels of the most loaded rank (whole call)", "achieved": bytes_rank_max / (r["ms"] * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s", "frac": bytes_rank_max / (r["ms"] * 1e-3) / 1e9 / peak, "peak_kind": kind, "traffic": None},
            "e2e": {"value": ROWS / r["e2e"], "unit": B.UNIT, "h2d_bytes_per_step": ROWS * H * 2, "d2h_bytes_per_step": ROWS * H * 4,
                    "us_per_layer": r["e2e"] * 1e6},
            "gpu_launches": r["launches"], "device_status": max(r["status"], results["nccl"]["status"]), "clocks": r["clocks"]}))
    dist.barrier()
    dist.destroy_process_group()
