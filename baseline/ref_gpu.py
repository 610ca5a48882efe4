"""BASELINE INFRASTRUCTURE: drives the reference's own GPU kernels (built unchanged for sm_100a by build_ref_gpu.py) through
their stock entry points, the way the reference's dispatcher does. Used by tests (second parity reference) and by bench.py
(same-box GPU baseline). Nothing under hecate_b200/ imports this module.

Call sequences followed (paths relative to the reference project):
  decode    runtime/tier/tier_split.py:341-354  (moe4.forward per chunk of <= 8 rows, scratch from moe4.scratch, grid sizes
            2 x and 3 x the SM count, tier_split.py:166); done_ptr is never passed (its wait is unbounded, moe4.cu:707)
  prefill   runtime/tier/tier_split.py:427-462  (_prefill_gb300, int4 branch: stable argsort of the flattened selection, one host
            sync for the per-expert counts, pick groups of <= 16384 picks with balanced row blocks of <= 256 picks uploaded
            from pinned memory, moe4t.forward per group)
  router    runtime/core/exl3_router.py:176-184 (zeroed logits [8][256] + counter, router_fused for 2..8 rows)
  combine   runtime/tier/cn.cu:190-210          (combine_norm, no done flag)
The reference's formats apply: fp16 activations, one fp32 scale per weight row, routed experts only (its shared expert is int8
and runs as separate GEMVs by default).
"""
import numpy as np

from . import build_ref_gpu as B

NPOS4 = 16384            # picks per moe4t call (EXL3_TIER_P4_NPOS default, runtime/tier/tier_split.py:61)
H, I = 6144, 2048        # compiled into the reference kernels


def available(*names):
    import os
    return all(os.path.exists(B.module_path(n)) for n in names)


def pick_groups(counts, npos=NPOS4, bm=256, balance=True):
    """Expert groups of <= npos picks with their row-block tables, as the reference's pick_groups yields them
    (runtime/tier/rtx_split.py:236-255): (first pick, end pick, int32 [n][4] {expert, first pick relative to the group,
    picks <= bm, 0}). The row blocks of a group come from the CPU checker's row_blocks, which is pinned against outputs of the
    reference function (tests/golden/pick_groups.json)."""
    from oracle import oracle as O
    c = np.asarray(counts, dtype=np.int64)
    ends = np.cumsum(c)
    e0 = 0
    while e0 < len(c):
        p0 = int(ends[e0] - c[e0])
        e1 = e0
        while e1 < len(c) and ends[e1] <= p0 + npos:
            e1 += 1
        if e1 == e0:
            raise ValueError("an expert has more picks than a group holds")
        rbt = O.row_blocks(c[e0:e1].astype(np.int32), bm, balance)
        rbt[:, 0] += e0
        yield p0, int(ends[e1 - 1]), rbt
        e0 = e1


class RefGpu:
    """The reference kernels on one device. tables: hecate_b200.moe.ExpertTables with group = 0 (per-row fp32 scales)."""

    def __init__(self, device):
        import torch
        self.torch, self.dev = torch, device
        self.moe4, self.moe4t, self.cn, self.rt = (B.load(n) for n in ("moe4", "moe4t", "cn", "router"))
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        self.blocks, self.blocks_a = sms * 2, sms * 3
        self.scr = None
        self.p4scr = None
        self.rbuf = None

    # -- decode -------------------------------------------------------------------------------------------------------
    def decode(self, tabs, x, sel, rw, out):
        """out fp32 [R][H] = routed experts of rows x (fp16), R <= 64, in chunks of 8 rows."""
        t = tabs.tabs
        if self.scr is None:
            self.scr = self.moe4.scratch(self.dev)
        R = x.shape[0]
        for c in range(0, R, 8):
            n = min(8, R - c)
            yh = out[c:c + n]
            yh.zero_()
            self.moe4.forward(x[c:c + n], sel[c:c + n], rw[c:c + n], tabs.n, t["gate_w"], t["up_w"], t["down_w"], t["gate_s"], t["up_s"],
                              t["down_s"], *self.scr, yh, self.blocks, self.blocks_a, 0)
        return out

    # -- prefill ------------------------------------------------------------------------------------------------------
    def prefill(self, tabs, x, sel, rw):
        torch = self.torch
        K8 = sel.shape[-1]
        fs = sel.reshape(-1)
        order = torch.argsort(fs, stable=True)
        counts = torch.bincount(fs, minlength=tabs.n).tolist()          # the reference's host sync
        out = torch.zeros(x.shape[0], H, dtype=torch.float, device=x.device)
        if self.p4scr is None:
            self.p4scr = self.moe4t.scratch(self.dev, NPOS4)
        gu, ar, d = self.p4scr
        n4 = sum(counts)
        if n4:
            seg = order[:n4]
            tok = (seg // K8).int(); eid = fs[seg].int(); wt = rw.reshape(-1)[seg].float()
            t = tabs.tabs
            for p0, p1, rbt in pick_groups(counts, NPOS4, 256, True):
                rb = torch.from_numpy(rbt).pin_memory().to(x.device, non_blocking=True)
                self.moe4t.forward(x, tok[p0:p1], eid[p0:p1], wt[p0:p1], rb, t["gate_w"], t["up_w"], t["down_w"], t["gate_s"], t["up_s"],
                                   t["down_s"], gu, ar, d.view(1, NPOS4, H), out)
        return out

    # -- router -------------------------------------------------------------------------------------------------------
    def router(self, x, wt, bias, topk, scale):
        """x fp16 [R][H] with 1 <= R <= 8, wt fp16 [E][H], bias fp32 [E] or None -> (sel int64 [R][topk], rw fp16)."""
        torch = self.torch
        if self.rbuf is None:
            self.rbuf = (torch.zeros(8, 256, dtype=torch.float, device=self.dev), torch.zeros(1, dtype=torch.int, device=self.dev))
        R = x.shape[0]
        sel = torch.empty(R, topk, dtype=torch.int64, device=self.dev)
        rw = torch.empty(R, topk, dtype=torch.float16, device=self.dev)
        self.rt.router_fused(x.contiguous(), wt, bias, self.rbuf[0], self.rbuf[1], sel, rw, topk, float(scale))
        return sel, rw

    # -- combine + next input norm ------------------------------------------------------------------------------------
    def combine_norm(self, f, o, y, o2, r, w, xn, eps, cbias=0.0, cscale=1.0):
        self.cn.combine_norm(f, o.data_ptr() if o is not None else 0, y, f.shape[0], o2.data_ptr() if o2 is not None else 0, 0, r, w, xn,
                             eps, cbias, cscale)
