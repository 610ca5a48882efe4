"""Expert parallelism over the GPUs of one box: one process per GPU (torch.distributed for the set-up plumbing), experts split
by contiguous id ranges. Decode: either the step's rows are replicated on every rank (`EpDecoder.step`, partial outputs combined
over NVLink peer memory by `hmoe_ep_combine`, or, as the baseline, by an NCCL all-reduce), or the tokens are data-parallel
(`EpDecoder.step_dp`): every rank routes its own rows, `hmoe_ep_dispatch` all-gathers rows, selections and weights through peer
memory, and `hmoe_ep_combine_own` brings back each rank's own rows: the two halves of the all-to-all. Prefill: `EpPrefill`.

The reference has no expert parallelism; the shape kept from it is its band split: every band receives all rows with
(sel, rw), ignores foreign ids and returns an fp32 partial that is added in a fixed order (runtime/tier/tier_split.py:3-11,
runtime/tier/moe4/moe4.cu:93,702-717).
"""
import ctypes as C

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


def replica_owners(sel, n_experts, world):
    """Host mirror of the device's choice with every expert on two ranks (EpDecoder(replicas=2)): rank r holds the bands r and r + 1
    (mod world) of n_experts / world router positions, so position e of band p is held by ranks p and p - 1; the bands walk their
    positions side by side and give each picked position to the holder with fewer experts so far (ties: rank p).
    Returns {position: rank} for the picked positions of `sel` (any integer array)."""
    import numpy as np
    npr = n_experts // world
    picked = np.zeros(n_experts, dtype=bool)
    ids = np.asarray(sel).reshape(-1)
    picked[ids[(ids >= 0) & (ids < n_experts)]] = True
    load = [0] * world
    owner = {}
    for i in range(npr):
        new = list(load)
        for p in range(world):
            if picked[p * npr + i]:
                q = (p - 1) % world
                o = q if load[q] < load[p] else p
                owner[p * npr + i] = o
                new[o] += 1
        load = new
    return owner


def prefill_destinations(sel, n_per_rank, world):
    """Host mirror of hmoe_prefill_ep_dispatch's routing of rows: a boolean array [rows][world], entry (i, p) set when rank p holds
    one of row i's selected router positions (position e belongs to rank e // n_per_rank; ids outside [0, world * n_per_rank)
    select no rank). The row's own rank always receives it as well; that is not included here."""
    import numpy as np
    sel = np.asarray(sel)
    valid = (sel >= 0) & (sel < world * n_per_rank)
    owner = np.where(valid, sel // n_per_rank, -1)
    return (owner[:, :, None] == np.arange(world)[None, None, :]).any(axis=1)


class PeerBuffers:
    """Symmetric buffers of the combine: per rank two fp32 partial slots [MAX_ROWS * H] and `world` generation flags,
    allocated with cudaMalloc by the library, exported with CUDA IPC and opened by every peer."""

    def __init__(self, rank, world, H, device, dist, slot_floats=None, stage_topk=0, prefill_stage=None):
        import torch
        self.rank, self.world, self.H = rank, world, H
        self.slot_floats = MAX_ROWS * H if slot_floats is None else (slot_floats + 63) // 64 * 64
        self.bytes = 2 * self.slot_floats * 4 + 512          # two slots, `world` flags (256 B), the generation word (256 B)
        self.stage_off = self.bytes                          # optional: the staging area of the decode dispatch
        if stage_topk:
            self.bytes += lib().hmoe_ep_stage_bytes(C.c_int(H), C.c_int(stage_topk))
        if prefill_stage:                                    # (rows of all ranks, topk): the staging area of the prefill dispatch
            self.bytes = (self.bytes + 255) // 256 * 256
            self.pstage_off = self.bytes
            self.bytes += lib().hmoe_prefill_ep_stage_bytes(C.c_int(prefill_stage[0]), C.c_int(H), C.c_int(prefill_stage[1]))
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
        if stage_topk:
            self.stage = (C.c_void_p * world)(*[b + self.stage_off for b in self.base])
            offs = [C.c_size_t() for _ in range(3)]
            check(lib().hmoe_ep_stage_offsets(C.c_int(H), C.c_int(stage_topk), *[C.byref(o) for o in offs]))
            self.stage_x, self.stage_sel, self.stage_rw = (self.own + self.stage_off + o.value for o in offs)
        if prefill_stage:
            self.pstage = (C.c_void_p * world)(*[b + self.pstage_off for b in self.base])
            so, ro = C.c_size_t(), C.c_size_t()
            check(lib().hmoe_prefill_ep_stage_offsets(C.c_int(prefill_stage[0]), C.c_int(H), C.c_int(prefill_stage[1]), C.byref(so), C.byref(ro)))
            self.pstage_x, self.pstage_sel, self.pstage_rw = self.own + self.pstage_off, self.own + self.pstage_off + so.value, self.own + self.pstage_off + ro.value
        dist.barrier()

    def close(self):
        for r, b in enumerate(self.base):
            if r != self.rank:
                lib().hmoe_ep_close(C.c_void_p(b))
        lib().hmoe_ep_free(C.c_void_p(self.own))


class EpDecoder:
    """One rank's side of an expert-parallel decode layer."""

    def __init__(self, rank, world, tables, n_experts, device, dist, use_peer=True, fused_tail=False, replicas=1):
        """replicas = 2: every expert is held by two ranks (the tables of rank r hold the bands r and r + 1 (mod world) of
        n_experts / world router positions each, in this order) and every step gives each picked expert to the less loaded of its
        two holders, the same choice on every rank (step_dp_fused only; twice the weight memory)."""
        self.rank, self.world, self.tabs, self.dev, self.dist = rank, world, tables, device, dist
        assert replicas in (1, 2) and (replicas == 1 or world > 1)
        self.replicas = replicas
        # fused_tail: the combine runs as the tail of the down launch (hmoe_decode_ep_combine) instead of as a kernel of its own;
        # it needs the register-resident decode kernels (H <= 6144, I <= 2048). Measured at 2 GPUs it is 2-3 us slower than the
        # separate kernel (148 blocks poll the flags instead of one thread), so it is off by default.
        self.fused_tail = fused_tail and tables.H <= 6144 and tables.I <= 2048
        self.plan = shard_plan(rank, world, n_experts)
        if replicas == 2:
            self.plan["n_local"] *= 2
        assert tables.n == self.plan["n_local"]
        self.ws = moe.decode_workspace(tables.H, tables.I, device)
        self.use_peer = use_peer and world > 1
        self.peer = PeerBuffers(rank, world, tables.H, device, dist, stage_topk=tables.topk) if self.use_peer else None
        import torch
        self.y = torch.zeros(MAX_ROWS, tables.H, dtype=torch.float32, device=device)
        self.struct = tables.struct()

    def step(self, x, sel, rw, f, tables=None):
        """f[R][H] (fp32) += the layer's output for rows x with global routing (sel, rw); identical on every rank. The rows are
        replicated (every rank passes all of them)."""
        import torch
        if self.replicas != 1:
            raise RuntimeError("experts held by two ranks are served by step_dp_fused only")
        R = x.shape[0]
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        pl = self.plan
        struct = self.struct if tables is None else tables.struct()
        if self.use_peer and self.fused_tail:
            self._decode_combine(struct, vp(x), moe._dt(x), vp(sel), vp(rw), R, f, 0, st)
        elif self.use_peer:
            check(lib().hmoe_decode_ep(C.byref(struct), vp(x), C.c_int(moe._dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(pl["lo"]),
                                       C.c_int(pl["n_local"]), C.c_int(0), C.c_void_p(self.peer.own), vp(self.ws),
                                       C.c_size_t(self.ws.numel()), C.c_int(pl["shared_mod"]), C.c_int(pl["shared_rem"]),
                                       C.c_void_p(self.peer.gen_ptr), C.c_size_t(self.peer.slot_floats), st))
            check(lib().hmoe_ep_combine(C.c_int(self.rank), C.c_int(self.world), self.peer.slots, self.peer.flags, C.c_void_p(self.peer.gen_ptr),
                                        vp(f), C.c_int(R), C.c_int(self.tabs.H), C.c_size_t(self.peer.slot_floats), vp(self.peer.status), st))
        else:
            y = self.y[:R]
            check(lib().hmoe_decode_ep(C.byref(struct), vp(x), C.c_int(moe._dt(x)), vp(sel), vp(rw), C.c_int(R), C.c_int(pl["lo"]),
                                       C.c_int(pl["n_local"]), C.c_int(0), vp(y), vp(self.ws), C.c_size_t(self.ws.numel()),
                                       C.c_int(pl["shared_mod"]), C.c_int(pl["shared_rem"]), None, C.c_size_t(0), st))
            if self.world > 1:
                self.dist.all_reduce(y)
            moe.moe4_combine(f, 0, y, R, 0)
        return f

    def _decode_combine(self, struct, x, x_dt, sel, rw, R, f, own_rows, st):
        pl, pb = self.plan, self.peer
        check(lib().hmoe_decode_ep_combine(C.byref(struct), x, C.c_int(x_dt), sel, rw, C.c_int(R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]),
                                           C.c_int(0), vp(self.ws), C.c_size_t(self.ws.numel()), C.c_int(pl["shared_mod"]),
                                           C.c_int(pl["shared_rem"]), C.c_void_p(pb.gen_ptr), C.c_size_t(pb.slot_floats), C.c_int(self.rank),
                                           C.c_int(self.world), pb.slots, pb.flags, vp(f), C.c_int(own_rows), vp(pb.status), st))

    def own_rows(self, R):
        """Rows of a step that this rank holds when the tokens are data-parallel: rank, rank + world, ..."""
        return list(range(self.rank, R, self.world))

    def step_dp(self, x_own, sel_own, rw_own, f_own, R, tables=None):
        """Data-parallel tokens: x_own [n][H], sel_own, rw_own are this rank's rows (rows rank, rank + world, ... of the step's R
        rows) with the routing its own router call produced; f_own [n][H] (fp32) += their layer output. Dispatch and combine are
        the two halves of an all-to-all over NVLink peer memory (hmoe_ep_dispatch, hmoe_ep_combine_own). `tables`: another layer's
        experts through the same buffers (a stack of layers shares one set)."""
        import torch
        if not self.use_peer or self.replicas != 1:
            raise RuntimeError("step_dp needs the peer-memory buffers and one holder per expert")
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        pl, pb = self.plan, self.peer
        struct = self.struct if tables is None else tables.struct()
        H, topk = self.tabs.H, self.tabs.topk
        check(lib().hmoe_ep_dispatch(C.c_int(self.rank), C.c_int(self.world), pb.stage, vp(x_own), vp(sel_own), vp(rw_own), C.c_int(R), C.c_int(H),
                                     C.c_int(topk), vp(pb.status), st))
        if self.fused_tail:
            self._decode_combine(struct, C.c_void_p(pb.stage_x), moe._dt(x_own), C.c_void_p(pb.stage_sel), C.c_void_p(pb.stage_rw), R, f_own, 1, st)
            return f_own
        check(lib().hmoe_decode_ep(C.byref(struct), C.c_void_p(pb.stage_x), C.c_int(moe._dt(x_own)), C.c_void_p(pb.stage_sel), C.c_void_p(pb.stage_rw),
                                   C.c_int(R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), C.c_void_p(pb.own), vp(self.ws),
                                   C.c_size_t(self.ws.numel()), C.c_int(pl["shared_mod"]), C.c_int(pl["shared_rem"]), C.c_void_p(pb.gen_ptr),
                                   C.c_size_t(pb.slot_floats), st))
        check(lib().hmoe_ep_combine_own(C.c_int(self.rank), C.c_int(self.world), pb.slots, pb.flags, C.c_void_p(pb.gen_ptr), vp(f_own), C.c_int(R),
                                        C.c_int(H), C.c_size_t(pb.slot_floats), vp(pb.status), st))
        return f_own

    def step_dp_fused(self, x_own, wt, bias, scale, sel, rw, f_own, R, tables=None):
        """Data-parallel tokens in four launches (hmoe_decode_ep_dp): the router's launch is also the dispatch of the rows and the
        expert kernels' set-up; every rank routes all R rows (sel, rw [R][topk] are outputs). x_own [n][H]: this rank's rows;
        f_own [n][H] (fp32) += their layer output."""
        import torch
        if not self.use_peer:
            raise RuntimeError("step_dp_fused needs the peer-memory buffers")
        st = C.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
        pl, pb = self.plan, self.peer
        struct = self.struct if tables is None else tables.struct()
        E = wt.shape[0]
        need = lib().hmoe_router_ws_bytes(C.c_int(R), C.c_int(E))
        if getattr(self, "_rws", None) is None or self._rws.numel() < need:
            self._rws = torch.zeros(max(need, 1 << 16), dtype=torch.uint8, device=self.dev)
        check(lib().hmoe_decode_ep_dp(C.byref(struct), vp(x_own), C.c_int(moe._dt(x_own)), vp(wt), C.c_int(moe._dt(wt)), vp(bias), C.c_int(R),
                                      C.c_int(E), C.c_float(float(scale)), vp(sel), vp(rw), vp(self._rws), C.c_size_t(self._rws.numel()),
                                      C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), vp(self.ws), C.c_size_t(self.ws.numel()),
                                      C.c_int(self.rank), C.c_int(self.world), pb.stage, pb.slots, pb.flags, C.c_void_p(pb.gen_ptr),
                                      C.c_size_t(pb.slot_floats), vp(f_own), vp(pb.status), C.c_int(int(self.fused_tail)), st))
        return f_own

    def dispatch_bytes(self, R, itemsize=2, with_routing=True):
        """Bytes this rank sends to other ranks per step: its rows and (step_dp) their selections and weights."""
        return (self.world - 1) * len(self.own_rows(R)) * (self.tabs.H * itemsize + (self.tabs.topk * 10 if with_routing else 0))

    def status(self):
        import torch
        torch.cuda.synchronize(self.dev)
        s = moe.ws_status(self.ws)
        if self.peer is not None:
            s |= int(self.peer.status.item())
        return s


class EpPrefill:
    """Expert-parallel prefill. Dispatch: the ranks' token slices are all-gathered (NCCL), or, dispatch="peer", sent as an
    all-to-all-v over NVLink peer memory (hmoe_prefill_ep_dispatch: a row goes only to the ranks that hold one of its experts);
    every rank runs the grouped GEMMs for its experts over all tokens (ids outside [lo, lo + n_local) are dropped by the
    permutation) plus the shared expert for its own tokens. Combine, use_peer = True: the down GEMM adds every row's sums straight into the output of the rank
    that owns the row, over NVLink peer memory, and a flag barrier ends the step. use_peer = False (the baseline): a local
    full-size partial and an NCCL reduce-scatter. short: with the reduce-scatter combine, steps of few rows in total (up to
    moe.forward_short_rows(), e.g. a decode step of many sequences) run the local experts through the streaming kernels
    (hmoe_short_prefill_ep) instead of the grouped GEMMs; None = whenever the layer allows it."""

    def __init__(self, rank, world, tables, n_experts, rows_per_rank, device, dist, use_peer=None, dispatch="nccl", short=None):
        import torch
        assert dispatch in ("nccl", "peer")
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
        sh8 = tables.shared is not None and tables.shared_i8          # the int8 shared expert hands over to the grouped GEMMs earlier (see hmoe_forward)
        can_short = R <= (min(256, moe.forward_short_rows()) if sh8 else moe.forward_short_rows()) and tables.H <= 6144 and tables.I <= 2048 and not (use_peer and world > 1)
        if short and not can_short:
            raise moe.HmoeError("EpPrefill: short needs <= forward_short_rows() rows in total, H <= 6144, I <= 2048 and the reduce-scatter combine")
        self.short = can_short if short is None else bool(short)
        if self.short:
            self.ws_short = moe.short_prefill_workspace(R, tables.H, tables.I, tables.topk, device)
        if not (dispatch == "peer" and world > 1):
            self.x_all = torch.empty(R, tables.H, dtype=torch.bfloat16, device=device)
            self.sel_all = torch.empty(R, tables.topk, dtype=torch.int64, device=device)
            self.rw_all = torch.empty(R, tables.topk, dtype=torch.float16, device=device)
        self.use_peer = use_peer and world > 1
        self.peer_dispatch = dispatch == "peer" and world > 1
        self.struct = tables.struct()
        self.gen = 0
        self.peer = None
        if self.use_peer or self.peer_dispatch:
            # one slot of the symmetric buffer is this rank's output [rows_per_rank][H]; the flags serve the barriers
            self.peer = PeerBuffers(rank, world, tables.H, device, dist, slot_floats=rows_per_rank * tables.H if self.use_peer else 64,
                                    prefill_stage=(R, tables.topk) if self.peer_dispatch else None)
            self.out_tab = (C.c_void_p * world)(*self.peer.base)
        if self.peer_dispatch:
            self.sent = torch.zeros(1, dtype=torch.int64, device=device)       # (row, remote rank) pairs stored so far
        if not self.use_peer:
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
        if self.peer_dispatch:
            # the previous step's readers are done: every rank passed the barrier / reduce-scatter that ended it
            self.gen += 1
            check(lib().hmoe_prefill_ep_dispatch(C.c_int(self.rank), C.c_int(self.world), self.peer.pstage, vp(x), vp(sel), vp(rw), C.c_int(self.rpr),
                                                 C.c_int(self.tabs.H), C.c_int(self.tabs.topk), C.c_int(pl["n_local"]), vp(self.sent), st))
            check(lib().hmoe_ep_barrier(C.c_int(self.rank), C.c_int(self.world), self.peer.flags, C.c_uint32(self.gen), vp(self.peer.status), st))
            xa, sa, ra = C.c_void_p(self.peer.pstage_x), C.c_void_p(self.peer.pstage_sel), C.c_void_p(self.peer.pstage_rw)
        else:
            if self.world > 1:
                d.all_gather_into_tensor(self.x_all, x); d.all_gather_into_tensor(self.sel_all, sel); d.all_gather_into_tensor(self.rw_all, rw)
            else:
                self.x_all.copy_(x); self.sel_all.copy_(sel); self.rw_all.copy_(rw)
            xa, sa, ra = vp(self.x_all), vp(self.sel_all), vp(self.rw_all)
        if self.use_peer:
            self.gen += 1
            check(lib().hmoe_prefill_ep_peer(C.byref(self.struct), xa, C.c_int(moe._dt(x)), sa, ra,
                                             C.c_int(self.R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), self.out_tab,
                                             C.c_int(self.world), C.c_int(self.rpr), vp(self.ws), C.c_size_t(self.ws.numel()),
                                             C.c_int(self.rank * self.rpr), C.c_int(self.rpr), st))
            check(lib().hmoe_ep_barrier(C.c_int(self.rank), C.c_int(self.world), self.peer.flags, C.c_uint32(self.gen), vp(self.peer.status), st))
            check(lib().hmoe_ep_copy(vp(out), C.c_void_p(self.peer.own), C.c_size_t(nbytes), st))
            return out
        self.partial.zero_()
        fn, ws = (lib().hmoe_short_prefill_ep, self.ws_short) if self.short else (lib().hmoe_prefill_ep, self.ws)
        check(fn(C.byref(self.struct), xa, C.c_int(moe._dt(x)), sa, ra,
                 C.c_int(self.R), C.c_int(pl["lo"]), C.c_int(pl["n_local"]), C.c_int(0), vp(self.partial), vp(ws),
                 C.c_size_t(ws.numel()), C.c_int(self.rank * self.rpr), C.c_int(self.rpr), st))
        if self.world > 1:
            d.reduce_scatter_tensor(out, self.partial)
        else:
            out.copy_(self.partial)
        return out

    def status(self):
        import torch
        torch.cuda.synchronize(self.dev)
        s = moe.ws_status(self.ws)
        if self.short:
            s |= moe.ws_status(self.ws_short)
        if self.peer is not None:
            s |= int(self.peer.status.item())
        return s
