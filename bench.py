#!/usr/bin/env python
"""Benchmark of the MoE expert hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One MoE layer of the benchmark definition: hidden 6144, 256 routed experts, top-8 sigmoid/bias router, one shared expert,
SwiGLU experts gate/up [2048 x 6144] and down [6144 x 2048] in packed int4 with a bf16 scale per 128 input columns. Inputs are
synthetic (seeded): codes uniform, scales lognormal(-4, 0.5), activations N(0, 1) in bf16, router weight N(0, 0.02) in bf16.

The headline line is the DECODE configuration (8 tokens x (1 + 1 MTP draft) = 16 rows): a step = router (whose launch also does the
expert kernels' set-up) -> gate_up (+ SiLU * up * weight) -> down -> combine into the fp32 layer output. `value` is rows/s with inputs resident in HBM, `e2e` the
same call chain fed from pinned host memory with the host<->device copies inside the timed region. Consecutive steps use
different input batches (8 in a ring), so each step streams a different ~2 GB of the 4.85 GB layer, far more than the L2.

The same JSON line carries, as further objects:
  prefill        N = 1: M = 8192 tokens, Zipf(1.1) expert popularity (permute -> gather -> grouped gate_up GEMM -> grouped down
                 GEMM on tcgen05); N > 1: M = 32768 tokens expert-parallel with uniform routing, and `prefill_zipf` with Zipf(1.3)
  parity_check   outputs of THIS layer (a few decode rows, a few prefill tokens, both activation modes) against the CPU checker,
                 computed outside the timed regions; N > 1: the peer-memory combine against the NCCL arm
  act_quant      the same steps timed in the mode that reproduces the CPU engine's int8 activation round trips
  reference_gpu  the reference's own GPU kernels (baseline/_ref, built unchanged for sm_100a) on the same device and inputs, in
                 their format (fp16 activations, one fp32 scale per row, routed experts only), beside this library in that format
  cpu_baseline   the reference CPU engine on the host cores (config 2 as two 8-row jobs + the shared expert, and config 1)

`--impl reference` times the reference's own CPU expert engine (oracle/_ref, built from the reference source) on the host
cores, on a bounded sample of the same workload. `--mode decode|prefill` runs one arm alone (profiling).
"""
import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H, I, E, TOPK, ROWS = 6144, 2048, 256, 8, 16
GROUP = 128
PER_MATRIX = I * H // 2                                  # packed bytes of one matrix
SCALE_BYTES = (2 * I * (H // GROUP) + H * (I // GROUP)) * 2
EXPERT_BYTES = 3 * PER_MATRIX + SCALE_BYTES              # 19,464,192
GATE_UP_BYTES = 2 * PER_MATRIX + 2 * I * (H // GROUP) * 2
PICK_FLOP = 2.0 * 3 * I * H                              # 75,497,472 per (token, expert) pair
NBATCH = 8
METRIC = "moe_layer_decode_rows_per_s"
UNIT = "rows/s"
WORKLOAD = "decode M=8 tokens x (1 + 1 MTP draft) = 16 rows, H=6144, 256 experts top-8 + shared, int4 g128 bf16 scales"
# DRAM traffic of one gate_up launch relative to its algorithmic bytes (dram__bytes_read + write of an ncu capture of the reduced
# case --experts 64; traffic grows in proportion to the experts streamed). Re-derive when the capture is refreshed.
GATE_UP_TRAFFIC_RATIO = 0.982
# bars: the benchmark definition's against the CPU engine (int8 activation mode; errors normalised as max|a-b| / max|b| and
# mean|a-b| / mean|b|) and the reference GPU kernels' own gate (norm-relative, tools/quant/test_moe4_rtx.py:70) otherwise
MAX_REL, MEAN_ABS, NORM_REL = 1e-2, 1e-3, 2e-3


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return {"hbm": float(d["hbm_gbs"]), "bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d["bf16_tflops_sustained"]),
                    "kind": "measured"}
        except Exception:
            pass
    return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the timed region runs."""

    def __init__(self, index, period=0.02):
        self.samples, self.reasons, self.stop_flag, self.period = [], set(), False, period
        self.max_mhz = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            self.nv, self.h = nv, nv.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = None
        self.t = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self.t.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        if self.nv is not None:
            self.t.join()

    def summary(self):
        s = self.samples
        return {"sm_mhz": float(np.median(s)) if s else None, "sm_max_mhz": self.max_mhz, "samples": len(s),
                "reasons": sorted(self.reasons)}


def errors(got, ref):
    """(max-rel, mean-abs, norm-rel), the first two normalised: max|a-b| / max|b| and mean|a-b| / mean|b|."""
    got = np.asarray(got, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    d = np.abs(got - ref)
    return (float(d.max() / max(np.abs(ref).max(), 1e-30)), float(d.mean() / max(np.abs(ref).mean(), 1e-30)),
            float(np.linalg.norm(got - ref) / max(np.linalg.norm(ref), 1e-30)))


# ----------------------------------------------------------------------------------------------------------------------
# the reference CPU engine on the host cores
def cpu_reference_arm(jobs, warmup, seed=0, variants=("avx2", "vnni")):
    """Times the reference CPU engine (oracle/_ref; without it, this repository's restatement) on the decode workload in the
    engine's own format (row-major int4, one fp32 scale per row, 8 rows and 8 picks per row and job):
      config 2  the 16 rows as two 8-row jobs of the routed experts plus, for each, one job that applies the shared expert to the
                same 8 rows (one pick of weight 1: the engine reads 8 picks per row, so the 9th pick is a job of its own);
                value = 16 rows / (sum of the four median job times)
      config 1  one row: a job of its 8 picks plus a one-pick job of the shared expert
    Routing is uniform random top-8 of 256 (what the seeded router produces); the weights are seeded random bytes."""
    from oracle import oracle as O
    from hecate_b200 import synth
    cores = os.cpu_count() or 1
    threads = max(1, min(60, cores - 2))
    sel, rw = synth.zipf_routing(seed, 0, ROWS, E, TOPK, 0.0)
    x = synth.activations(seed, 0, ROWS, H).astype(np.float16)
    ids = sorted(set(int(e) for e in sel.reshape(-1)))
    remap = {e: i for i, e in enumerate(ids)}
    sel_local = np.vectorize(remap.get)(sel).astype(np.int64)
    S = len(ids)                                          # local id of the shared expert
    rng = np.random.default_rng(seed)
    experts = []
    for _ in range(S + 1):
        q = lambda N, K: rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
        sc = lambda N: np.exp(-4.0 + 0.5 * rng.standard_normal(N)).astype(np.float32).reshape(1, N)
        experts.append(O.Expert(q(I, H), q(I, H), q(H, I), sc(I), sc(I), sc(H), H, I, packed=False))
    sh_sel = np.full((8, TOPK), -1, dtype=np.int64); sh_sel[:, 0] = S
    sh_rw = np.zeros((8, TOPK), dtype=np.float16); sh_rw[:, 0] = 1.0
    jobs_c2 = [(x[0:8], sel_local[0:8], rw[0:8]), (x[0:8], sh_sel, sh_rw), (x[8:16], sel_local[8:16], rw[8:16]), (x[8:16], sh_sel, sh_rw)]
    jobs_c1 = [(x[0:1], sel_local[0:1], rw[0:1]), (x[0:1], sh_sel[0:1], sh_rw[0:1])]
    out = {"cores": threads, "unit": UNIT, "distinct_routed_experts": S,
           "sample": f"{jobs} timed repetitions of every job (median ISSUE->DONE time per job, summed): config 2 = two 8-row jobs of the routed "
                     f"experts ({S} distinct) + two 8-row one-pick jobs of the shared expert; config 1 = one row, 8 picks + the shared expert; "
                     f"engine format (row-major int4, fp32 scale per row)"}

    def run_engine(variant):
        eng = O.RefEngine(experts, 0, threads=threads, core0=0, variant=variant)
        try:
            med = lambda job: float(np.median([eng.job(*job)[1] for _ in range(warmup + jobs)][warmup:]))
            t2 = [med(j) for j in jobs_c2]
            t1 = [med(j) for j in jobs_c1]
        finally:
            eng.stop()
        return {"value": ROWS / sum(t2), "ms_16_rows": sum(t2) * 1e3, "ms_per_job": [t * 1e3 for t in t2],
                "config1_us_per_token": sum(t1) * 1e6, "config1_rows_per_s": 1.0 / sum(t1)}

    done = {}
    for v in variants:
        if O.ref_available(v):
            done[v] = run_engine(v)
    if done:
        best = max(done, key=lambda v: done[v]["value"])
        out.update(kind="reference", value=done[best]["value"], ms_16_rows=done[best]["ms_16_rows"], variant=best, variants=done,
                   variant_note="avx2 / vnni / scalar: the AArch64 SDOT and FMLA of the engine's inner loop mapped to AVX2 widening multiply-adds, "
                                "to one AVX-512-VNNI instruction, or to scalar loops; results are bit-identical")
    else:
        t0 = time.perf_counter()
        for _ in range(max(1, jobs // 4)):
            O.moe_forward(H, I, 0, x, sel_local, rw, 0, experts[:S], experts[S])
        t = (time.perf_counter() - t0) / max(1, jobs // 4)
        out.update(kind="port", value=ROWS / t, cores=O.threads(), ms_16_rows=t * 1e3)
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 50))
    cb = cpu_reference_arm(steps, max(1, min(args.warmup, 5)), variants=("avx2", "vnni", "scalar") if args.all_variants else ("avx2", "vnni"))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": cb["ms_16_rows"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 x int8 -> fp32", "data": "synthetic",
            "config": {"workload": WORKLOAD + " [reference CPU engine: two 8-row jobs + the shared expert, fp32 scale per row]"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------------
# the layer
class Layer:
    """Seeded synthetic experts resident in HBM: n routed experts + one shared expert, in the benchmark's format (bf16 scale per
    128 columns) and, over the same packed codes, in the reference's format (one fp32 scale per row; routed experts only)."""

    def __init__(self, dev, seed, n, rowscale=False):
        import torch
        from hecate_b200 import moe, synth
        self.n, self.dev = n, dev
        self.pool = torch.empty((n + 1) * 3 * PER_MATRIX, dtype=torch.uint8, device=dev)
        moe.fill_bytes(self.pool, seed, synth.stream_id(0, "gate_q", 0))
        view = self.view
        g = torch.Generator(device=dev); g.manual_seed(seed + 1)
        sc = lambda N, K: (torch.randn(n + 1, N // 64, K // GROUP, 64, device=dev, generator=g) * 0.5 - 4.0).exp().to(torch.bfloat16)
        self.gs, self.us, self.ds = sc(I, H), sc(I, H), sc(H, I)          # device order [N/64][K/128][64] per expert
        shared = (view(n, 0), view(n, 1), view(n, 2), self.gs[n], self.us[n], self.ds[n])
        self.tabs = moe.ExpertTables(H, I, TOPK, [view(e, 0) for e in range(n)], [view(e, 1) for e in range(n)],
                                     [view(e, 2) for e in range(n)], list(self.gs[:n]), list(self.us[:n]), list(self.ds[:n]), group=GROUP,
                                     shared=shared, device=dev)
        self.tabs.keep.append(self.pool)
        self.tabs0 = None
        if rowscale:
            rs = lambda N: (torch.randn(n, N, device=dev, generator=g) * 0.5 - 4.0).exp()
            self.rs = (rs(I), rs(I), rs(H))
            self.tabs0 = moe.ExpertTables(H, I, TOPK, [view(e, 0) for e in range(n)], [view(e, 1) for e in range(n)],
                                          [view(e, 2) for e in range(n)], list(self.rs[0]), list(self.rs[1]), list(self.rs[2]), group=0,
                                          shared=None, device=dev)
            self.tabs0.keep.append(self.pool)

    def view(self, e, k):
        return self.pool[(e * 3 + k) * PER_MATRIX:(e * 3 + k + 1) * PER_MATRIX]

    def host_experts(self, O, ids):
        """Host copies of experts `ids` (n = the shared expert) for the CPU checker, from the device tensors."""
        from hecate_b200 import layout
        out = []
        for e in ids:
            q = [self.view(e, k).cpu().numpy() for k in range(3)]
            s = [layout.group_scales_logical(t[e].float().cpu().numpy(), N) for t, N in ((self.gs, I), (self.us, I), (self.ds, H))]
            out.append(O.Expert(q[0], q[1], q[2], s[0], s[1], s[2], H, I))
        return out


def make_graphed(step, xs, torch, moe, use_graph):
    """Returns (run(batch_index), kernels launched per step). With graphs: one captured graph per input batch."""
    l0 = moe.launch_count()
    step(xs[0])
    per_step = moe.launch_count() - l0
    if not use_graph:
        return (lambda b: step(xs[b])), per_step
    graphs = []
    try:
        for x in xs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                step(x)
            graphs.append(g)
    except Exception as e:                      # capture refused: run eagerly, say so
        print(f"graph capture failed ({e}); running eagerly", file=sys.stderr)
        return (lambda b: step(xs[b])), per_step
    return (lambda b: graphs[b].replay()), per_step


def timed(torch, run, steps, nb, lead=0):
    """ms per step over `steps` calls of run(i % nb), CUDA events on the current stream, synchronised on both sides. lead: that
    many further warm-up steps are queued directly in front of the start event (multi-GPU arms: the ranks leave the host-side
    barrier tens of microseconds apart, and without them the first timed step would measure that skew, not the step)."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    for i in range(lead):
        run((nb - lead + i) % nb)
    ev0.record()
    for i in range(steps):
        run(i % nb)
    ev1.record()
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1) / steps


def wait_probe(moe, steps):
    """With the diagnostic build of the library: steps = None clears the prefill GEMMs' wait counters and returns {} (None with the
    normal build); otherwise returns, per kernel, the share of the blocks' lifetime each role spent in each of its waits."""
    import ctypes as C
    from hecate_b200 import _lib
    L = _lib.lib()
    if not hasattr(L, "hmoe_probe_read"):
        return None
    buf = (C.c_ulonglong * 64)()
    L.hmoe_probe_read(buf, 1)
    if steps is None:
        return {}
    names = {0: "mma_thread_waits_for_weights", 1: "mma_thread_waits_for_inputs", 2: "mma_thread_waits_for_free_accumulators",
             4: "dequant_warp0_waits_for_ring_slot", 10: "dequant_warp15_waits_for_ring_slot", 9: "dequant_warp0_store_fence_arrive",
             6: "tma_thread_waits_for_ring_slot", 7: "readout_warp_waits_for_tile", 8: "readout_warp_reads_out"}
    out = {}
    for k, kernel in ((1, "gate_up"), (0, "down")):
        tot = buf[32 * k + 15]
        out[kernel] = dict({"block_lifetime_cycles_all_sms_per_step": tot / steps}, **{n: buf[32 * k + i] / max(tot, 1) for i, n in names.items()})
    return out


def decode_timeline(torch, run_step, nbatch, reps=24):
    """With the diagnostic build of the library: the decode chain's kernels stamp the global timer (earliest / latest over their
    blocks); returns the median time of every stamp after the router's entry, in microseconds, over single replayed steps."""
    import ctypes as C
    from hecate_b200 import _lib
    L = _lib.lib()
    if not hasattr(L, "hmoe_tl_router"):
        return None
    bufs = {n: (C.c_ulonglong * 16)() for n in ("router", "decode", "combine")}

    def read(clear):
        for n, b in bufs.items():
            getattr(L, "hmoe_tl_" + n)(b, clear)
    rows = []
    for it in range(reps):
        run_step(it % nbatch); torch.cuda.synchronize(); read(1)        # a step before keeps the caches and clocks as in a run
        run_step((it + 1) % nbatch); torch.cuda.synchronize(); read(0)
        r, d, c = bufs["router"], bufs["decode"], bufs["combine"]
        ev = {"router_logits_done": r[1], "selection_done": r[3], "work_list_done": r[5], "gate_up_first_block_resident": d[0],
              "gate_up_wait_returned": d[2], "gate_up_first_weights_in": d[4], "gate_up_end": d[1], "down_first_block_resident": d[8],
              "down_wait_returned": d[10], "down_first_weights_in": d[12], "down_end": d[9], "combine_wait_returned": c[0]}
        rows.append([(v - r[0]) / 1e3 for v in ev.values()])
    med = np.median(np.array(rows), axis=0)
    return {k: float(v) for k, v in zip(ev.keys(), med)}


def oracle_rows(O, layer, x_rows, sel_rows, rw_rows, mode):
    """The CPU checker's output for a few rows of THIS layer (weights copied back from the device). x_rows float32 (bf16 values)."""
    ids = sorted(set(int(e) for e in sel_rows.reshape(-1)))
    remap = {e: i for i, e in enumerate(ids)}
    loc = np.vectorize(remap.get)(sel_rows).astype(np.int64)
    hx = layer.host_experts(O, ids + [layer.n])
    return O.moe_forward(H, I, GROUP, x_rows.astype(np.float16), loc, rw_rows, 0, hx[:-1], hx[-1], mode=mode)


# ----------------------------------------------------------------------------------------------------------------------
# N = 1
def decode_arm(args, dev, layer, torch, moe, synth, O):
    steps, warmup = args.steps, max(3, args.warmup)
    n_exp = layer.n
    tabs = layer.tabs
    wt = torch.from_numpy(synth.router_weight(0, 0, n_exp, H)).to(dev).to(torch.bfloat16)
    bias = torch.zeros(n_exp, dtype=torch.float32, device=dev)
    xs_np = [synth.activations(b, 0, ROWS, H) for b in range(NBATCH)]
    xs_host = [torch.from_numpy(x).to(torch.bfloat16).pin_memory() for x in xs_np]
    xs = [x.to(dev) for x in xs_host]
    sel = torch.empty(ROWS, TOPK, dtype=torch.int64, device=dev)
    rw = torch.empty(ROWS, TOPK, dtype=torch.float16, device=dev)
    ws = moe.decode_workspace(H, I, dev)
    y = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    f = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    x_in = torch.empty(ROWS, H, dtype=torch.bfloat16, device=dev)
    f_host = torch.empty(ROWS, H, dtype=torch.float32).pin_memory()
    aq = [False]

    def step(x):
        moe.router_decode(tabs, x, wt, bias, sel, rw, 1.0, y, ws, act_quant=aq[0])      # router (+ set-up) -> gate_up -> down
        moe.moe4_combine(f, 0, y, ROWS, 0)

    distinct, routes = [], []
    for b in range(NBATCH):                  # distinct experts per batch (for the algorithmic byte count) and the routing itself
        moe.router_fused(xs[b], wt, bias, None, None, sel, rw, TOPK, 1.0)
        distinct.append(int(torch.unique(sel).numel()))
        routes.append((sel.cpu().numpy().copy(), rw.cpu().numpy().copy()))
    for i in range(warmup):
        step(xs[i % NBATCH])
    torch.cuda.synchronize()
    # One CUDA graph per input batch (the reference runs its decode forward as captured graphs too, runtime/core/exl3_vgraph.py):
    # a step allocates nothing, does not synchronise and its launch shapes do not depend on the routing.
    run_step, launches_per_step = make_graphed(step, xs, torch, moe, not args.no_graph)
    for i in range(warmup):
        run_step(i % NBATCH)
    with ClockSampler(dev.index) as cs:
        ms_per_step = timed(torch, run_step, steps, NBATCH)
        if len(cs.samples) < 5:           # very short runs: keep the same load going so the clock record is not empty
            t_end = time.time() + 0.4
            while time.time() < t_end:
                run_step(0); torch.cuda.synchronize()
    launches = launches_per_step * steps
    timeline = decode_timeline(torch, run_step, NBATCH)              # diagnostic library only
    # kernel durations: a second pass over the same steps launched eagerly back to back, CUDA events around each kernel on
    # its stream (recorded by the library into a ring); read after the pass
    moe.set_profiling(True)
    for i in range(min(steps, 32)):
        step(xs[i % NBATCH])
    torch.cuda.synchronize()
    phase = np.array(moe.decode_phase_times())
    moe.set_profiling(False)
    mean_d = float(np.mean([distinct[i % NBATCH] for i in range(steps)]))
    gate_up_bytes = (mean_d + 1) * GATE_UP_BYTES
    layer_bytes = (mean_d + 1) * EXPERT_BYTES + n_exp * H * 2 + ROWS * H * 6
    pk = peaks()
    achieved = gate_up_bytes / (phase[1] * 1e-3) / 1e9

    # end to end: host buffers in, host buffer out, every step. The host->device copy of the step's rows, the layer call and
    # the device->host copy of its result are captured as one graph per input batch (the same public calls, replayed), and the
    # host waits for the result before the next step.
    def e2e_step(b):
        x_in.copy_(xs_host[b], non_blocking=True); step(x_in); f_host.copy_(f, non_blocking=True)
    run_e2e, _ = make_graphed(e2e_step, list(range(NBATCH)), torch, moe, not args.no_graph)
    for i in range(3):
        run_e2e(i % NBATCH)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(steps):
        run_e2e(i % NBATCH)
        torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / steps

    # the parity mode (the CPU engine's int8 activation round trips), timed the same way
    aq[0] = True
    run_q, _ = make_graphed(step, xs, torch, moe, not args.no_graph)
    for i in range(3):
        run_q(i % NBATCH)
    ms_q = timed(torch, run_q, steps, NBATCH)
    aq[0] = False

    # smaller batches through the same call (1 row = the reference's single-token decode step): latency per layer call and the
    # share of the HBM rate its algorithmic bytes reach
    small = {}
    for r in (1, 2, 4, 8):
        xr = [x[:r].contiguous() for x in xs]
        sel_r, rw_r = sel[:r].clone(), rw[:r].clone()
        y_r, f_r = torch.zeros(r, H, dtype=torch.float32, device=dev), torch.zeros(r, H, dtype=torch.float32, device=dev)

        def step_r(x):
            moe.router_decode(tabs, x, wt, bias, sel_r, rw_r, 1.0, y_r, ws)
            moe.moe4_combine(f_r, 0, y_r, r, 0)
        d_r = []
        for b in range(NBATCH):
            step_r(xr[b]); d_r.append(int(torch.unique(sel_r).numel()))
        run_r, _ = make_graphed(step_r, xr, torch, moe, not args.no_graph)
        for i in range(3):
            run_r(i % NBATCH)
        ms_r = timed(torch, run_r, max(8, min(steps, 64)), NBATCH)
        tl_r = decode_timeline(torch, run_r, NBATCH) if r == 1 else None
        bytes_r = (float(np.mean(d_r)) + 1) * EXPERT_BYTES + n_exp * H * 2 + r * H * 6
        small[str(r)] = {"us_per_layer": ms_r * 1e3, "distinct_experts": float(np.mean(d_r)),
                         "layer_hbm_frac": bytes_r / (ms_r * 1e-3) / 1e9 / peaks()["hbm"], **({"timeline_us": tl_r} if tl_r else {})}

    # larger batches than a decode call takes (the range the reference serves with 8-row chunks of its decode kernels,
    # tier_split.py:341-355): the short-prefill call (routing given) next to the grouped GEMMs on the same inputs, and the share
    # of the HBM rate the distinct experts' bytes reach
    short = {}
    for r in (32, 64, 128):
        xm = [torch.from_numpy(synth.activations(40 + b, 0, r, H)).to(torch.bfloat16).to(dev) for b in range(2)]
        rm = [synth.zipf_routing(50 + b, 0, r, n_exp, TOPK, 0.0) for b in range(2)]
        sm = [torch.from_numpy(q[0]).to(dev) for q in rm]; wm = [torch.from_numpy(q[1]).to(dev) for q in rm]
        o_s, o_g = torch.zeros(r, H, dtype=torch.float32, device=dev), torch.zeros(r, H, dtype=torch.float32, device=dev)
        ws_s, ws_g = moe.short_prefill_workspace(r, H, I, TOPK, dev), moe.prefill_workspace(r, TOPK, n_exp, H, I, dev)

        def step_s(b):
            o_s.zero_(); moe.short_prefill(tabs, xm[b], sm[b], wm[b], o_s, ws_s)

        def step_g(b):
            o_g.zero_(); moe.prefill(tabs, xm[b], sm[b], wm[b], o_g, ws_g)
        step_s(0); step_g(0)
        agree = float(((o_s - o_g).norm() / o_g.norm().clamp_min(1e-30)).item())
        run_s, _ = make_graphed(step_s, [0, 1], torch, moe, not args.no_graph)
        run_g, _ = make_graphed(step_g, [0, 1], torch, moe, not args.no_graph)
        for i in range(3):
            run_s(i % 2); run_g(i % 2)
        ms_s, ms_g = timed(torch, run_s, 8, 2), timed(torch, run_g, 8, 2)
        d_m = float(np.mean([len(np.unique(q[0])) for q in rm]))
        short[str(r)] = {"us_per_layer": ms_s * 1e3, "grouped_gemms_us_per_layer": ms_g * 1e3, "distinct_experts": d_m,
                         "layer_hbm_frac": (d_m + 1) * EXPERT_BYTES / (ms_s * 1e-3) / 1e9 / peaks()["hbm"],
                         "norm_rel_short_vs_grouped_gemms": agree, "device_status": int(moe.ws_status(ws_s))}
        del ws_s, ws_g

    # parity on this very layer, outside the timed regions: the router's selection bit for bit, two rows of batch 0 in both modes
    parity = {}
    if O is not None:
        bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)
        osel, orw = O.router(bits(xs[0]), 1, bits(wt), 1, None, TOPK, 1.0)
        s0, w0 = routes[0]
        parity["router_bit_exact"] = bool(np.array_equal(osel, s0) and np.array_equal(orw.view(np.uint16), w0.view(np.uint16)))
        rows = [0, 9]
        for mode_name, q in (("act_quant1_vs_cpu_engine", True), ("act_quant0_vs_exact", False)):
            y.zero_()
            moe.decode(tabs, xs[0], torch.from_numpy(s0).to(dev), torch.from_numpy(w0).to(dev), y, ws, act_quant=q)
            got = y[rows].cpu().numpy(); y.zero_()
            ref = oracle_rows(O, layer, xs_np[0][rows], s0[rows], w0[rows], 0 if q else 1)
            e = errors(got, ref)
            parity[mode_name] = {"max_rel": e[0], "mean_abs": e[1], "norm_rel": e[2], "rows": rows,
                                 "ok": bool(e[0] < MAX_REL and e[1] < MEAN_ABS) if q else bool(e[2] < NORM_REL)}
    status = moe.ws_status(ws)
    line = {
        "metric": METRIC, "value": ROWS / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int4 x fp16 -> fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD if n_exp == 256 else WORKLOAD + f" [reduced to {n_exp} experts]",
                   "launch": "eager" if args.no_graph else "cuda graph per input batch",
                   "l2": "inputs larger than L2: ~2 GB of weights streamed per step, 8 input batches in a ring",
                   "distinct_experts_per_step": mean_d},
        "us_per_layer": ms_per_step * 1e3,
        "layer_hbm_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_hbm_frac": layer_bytes / (ms_per_step * 1e-3) / 1e9 / pk["hbm"],
        "phase_us": {"prepare": phase[0] * 1e3, "gate_up": phase[1] * 1e3, "down": phase[2] * 1e3},
        "roofline": {"bound": "hbm", "kernel": "decode_stream_kernel (gate_up)", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                     "frac": achieved / pk["hbm"], "peak_kind": pk["kind"], "traffic": GATE_UP_TRAFFIC_RATIO * gate_up_bytes,
                     "algorithmic_bytes_per_launch": gate_up_bytes},
        "e2e": {"value": ROWS / e2e_s, "unit": UNIT, "h2d_bytes_per_step": ROWS * H * 2, "d2h_bytes_per_step": ROWS * H * 4,
                "us_per_layer": e2e_s * 1e6},
        "act_quant": {"decode_us_per_layer": ms_q * 1e3, "decode_vs_default": ms_q / ms_per_step},
        "small_batches": small, "short_prefill": short, **({"timeline_us": timeline} if timeline else {}),
        "parity_check": {"decode": parity},
        "gpu_launches": int(launches), "device_status": int(status), "clocks": cs.summary(),
    }
    return line, dict(wt=wt, bias=bias, xs=xs, routes=routes)


def prefill_arm(args, dev, layer, torch, moe, synth, O, R=8192, zipf=1.1):
    """Prefill configuration: M = 8192 tokens, Zipf(1.1) expert popularity, top-8 without replacement, + shared expert.
    A step = permute -> gather -> grouped gate_up GEMM (+ SiLU epilogue) -> grouped down GEMM (+ scatter-add epilogue).
    value = TFLOP/s over the algorithmic flops 2 * (8 R + R) * 37,748,736 (padding columns not counted)."""
    n_exp, tabs = layer.n, layer.tabs
    steps, warmup = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))
    NB = 2
    xs_np = [synth.activations(20 + b, 0, R, H) for b in range(NB)]
    xs = [torch.from_numpy(x).to(torch.bfloat16).to(dev) for x in xs_np]
    routes = [synth.zipf_routing(10 + b, 0, R, n_exp, TOPK, zipf) for b in range(NB)]
    sels = [torch.from_numpy(r[0]).to(dev) for r in routes]; rws = [torch.from_numpy(r[1]).to(dev) for r in routes]
    ws = moe.prefill_workspace(R, TOPK, n_exp, H, I, dev)
    out = torch.zeros(R, H, dtype=torch.float32, device=dev)
    x_host = xs[0].cpu().pin_memory(); out_host = torch.empty(R, H, dtype=torch.float32).pin_memory()
    x_in = torch.empty_like(xs[0])
    aq = [False]
    wsq = [ws]

    def step(i):
        out.zero_()
        moe.prefill(tabs, xs[i % NB], sels[i % NB], rws[i % NB], out, wsq[0], act_quant=aq[0])

    for i in range(warmup):
        step(i)
    probe = wait_probe(moe, None)                # diagnostic library only (python -m hecate_b200.csrc.build --probe-waits): clears its counters
    l0 = moe.launch_count()
    with ClockSampler(dev.index) as cs:
        ms = timed(torch, step, steps, NB)
    launches = moe.launch_count() - l0
    probe = wait_probe(moe, steps) if probe is not None else None
    n2 = max(1, min(steps, 10))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(n2):
        x_in.copy_(x_host, non_blocking=True); out.zero_()
        moe.prefill(tabs, x_in, sels[0], rws[0], out, ws)
        out_host.copy_(out, non_blocking=True); torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / n2
    flop = (TOPK * R + R) * PICK_FLOP
    counts = np.bincount(routes[0][0].reshape(-1), minlength=n_exp)
    pk = peaks()
    tf = flop / (ms * 1e-3) / 1e12
    res = {
        "metric": "moe_prefill_expert_gemm_tflops", "value": tf, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps, "warmup": warmup,
        "tokens_per_s": R / (ms * 1e-3), "dtype": "int4 -> fp16 x fp16 -> fp32 (tcgen05)", **({"wait_shares": probe} if probe else {}),
        "config": {"workload": f"prefill M={R} tokens, Zipf({zipf}) top-8 over {n_exp} experts + shared, H=6144, int4 g128 bf16 scales",
                   "l2": "inputs larger than L2 (4.85 GB of weights, 0.9 GB gathered inputs)", "max_picks_per_expert": int(counts.max()),
                   "min_picks_per_expert": int(counts.min())},
        "roofline": {"bound": "tensor", "kernel": "prefill_gemm_kernel<2> + <1> (whole step: permute, gather, both grouped GEMMs)",
                     "achieved": tf, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": tf / pk["bf16"], "peak_kind": pk["kind"] + " burst (bf16_tflops)",
                     "peak_sustained": pk["bf16_sustained"], "frac_sustained": tf / pk["bf16_sustained"], "traffic": None,
                     "algorithmic_flop_per_step": flop},
        "e2e": {"value": flop / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": R * H * 2, "d2h_bytes_per_step": R * H * 4,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches), "clocks": cs.summary()}
    parity = {}
    if O is not None:
        rows = [0, R // 2 + 1, R - 1]
        for mode_name, q in (("act_quant0_vs_exact", False), ("act_quant1_vs_cpu_engine", True)):
            if q:
                wsq[0] = moe.prefill_workspace(R, TOPK, n_exp, H, I, dev, act_quant=True)
                aq[0] = True
                step(0); step(0)
                res["act_quant_ms_per_step"] = timed(torch, step, max(1, min(steps, 5)), NB)
            step(0)
            got = out[rows].cpu().numpy()
            ref = oracle_rows(O, layer, xs_np[0][rows], routes[0][0][rows], routes[0][1][rows], 0 if q else 1)
            e = errors(got, ref)
            parity[mode_name] = {"max_rel": e[0], "mean_abs": e[1], "norm_rel": e[2], "rows": rows,
                                 "ok": bool(e[0] < MAX_REL and e[1] < MEAN_ABS) if q else bool(e[2] < NORM_REL)}
        res["device_status_act_quant"] = int(moe.ws_status(wsq[0]))
        aq[0] = False; wsq[0] = ws
    res["device_status"] = int(moe.ws_status(ws))
    return res, parity


def reference_gpu_arm(args, dev, layer, torch, moe, synth, dec):
    """The reference's own GPU kernels on this device, through their stock entry points (baseline/ref_gpu.py), and this library
    on the same inputs in the same format (fp16 activations, one fp32 scale per row, routed experts only)."""
    from baseline import ref_gpu
    if not ref_gpu.available("moe4", "moe4t"):
        return {"unavailable": "baseline/_ref holds no build of the reference GPU kernels"}
    rg = ref_gpu.RefGpu(dev)
    tabs0 = layer.tabs0
    steps = max(3, min(args.steps, 20))
    res = {"format": "fp16 activations, fp32 scale per row, routed experts only (the reference kernels' format); "
                     "16 rows = two 8-row moe4 calls (its kernels take <= 8 rows)"}
    xs16 = [x.to(torch.float16) for x in dec["xs"]]
    sels = [torch.from_numpy(r[0]).to(dev) for r in dec["routes"]]; rws = [torch.from_numpy(r[1]).to(dev) for r in dec["routes"]]
    ws = moe.decode_workspace(H, I, dev)
    y = torch.zeros(ROWS, H, dtype=torch.float32, device=dev); yr = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    for rows in (8, 16):
        def ours(b):
            y.zero_(); moe.decode(tabs0, xs16[b][:rows], sels[b][:rows], rws[b][:rows], y[:rows], ws)
        def theirs(b):
            rg.decode(tabs0, xs16[b][:rows], sels[b][:rows], rws[b][:rows], yr[:rows])
        ours(0); theirs(0); torch.cuda.synchronize()
        e = errors(y[:rows].cpu().numpy(), yr[:rows].cpu().numpy())
        run_o, _ = make_graphed(ours, list(range(NBATCH)), torch, moe, not args.no_graph)
        run_t, _ = make_graphed(theirs, list(range(NBATCH)), torch, moe, not args.no_graph)
        for i in range(3):
            run_o(i); run_t(i)
        res[f"decode_{rows}_rows"] = {"reference_us": timed(torch, run_t, steps, NBATCH) * 1e3, "ours_us": timed(torch, run_o, steps, NBATCH) * 1e3,
                                      "norm_rel_ours_vs_reference": e[2], "ok": bool(e[2] < NORM_REL)}
    del run_o, run_t
    R = 8192
    x = torch.from_numpy(synth.activations(20, 0, R, H)).to(torch.float16).to(dev)
    s_np, w_np = synth.zipf_routing(10, 0, R, layer.n, TOPK, 1.1)
    sel, rw = torch.from_numpy(s_np).to(dev), torch.from_numpy(w_np).to(dev)
    wsp = moe.prefill_workspace(R, TOPK, layer.n, H, I, dev)
    out = torch.zeros(R, H, dtype=torch.float32, device=dev)
    keep = [None]
    def ours_p(i):
        out.zero_(); moe.prefill(tabs0, x, sel, rw, out, wsp)
    def theirs_p(i):
        keep[0] = rg.prefill(tabs0, x, sel, rw)
    ours_p(0); theirs_p(0); torch.cuda.synchronize()
    e = errors(out[::64].cpu().numpy(), keep[0][::64].cpu().numpy())
    for i in range(2):
        ours_p(i); theirs_p(i)
    n = max(3, min(steps, 10))
    t_ref, t_ours = timed(torch, theirs_p, n, 1), timed(torch, ours_p, n, 1)
    flop = TOPK * R * PICK_FLOP
    res["prefill_8192_rows"] = {"reference_ms": t_ref, "ours_ms": t_ours, "reference_tflops": flop / (t_ref * 1e-3) / 1e12,
                                "ours_tflops": flop / (t_ours * 1e-3) / 1e12, "norm_rel_ours_vs_reference": e[2], "ok": bool(e[2] < NORM_REL),
                                "note": "routed experts only (8 picks per token); the reference arm includes its host-side argsort / bincount "
                                        "sync and row-block upload, ours its device permutation"}
    res["device_status"] = int(moe.ws_status(ws)) | int(moe.ws_status(wsp))
    return res


def run_ours(args):
    import torch
    from hecate_b200 import moe, synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        return run_ep(args, world, rank, dev)
    O = None
    if not args.no_check:
        from oracle import oracle as O
    layer = Layer(dev, 0, args.experts, rowscale=not args.no_ref_gpu)
    line = None
    if args.mode in ("all", "decode"):
        line, dec = decode_arm(args, dev, layer, torch, moe, synth, O)
    if args.mode in ("all", "prefill"):
        pre, par = prefill_arm(args, dev, layer, torch, moe, synth, O, R=args.rows, zipf=args.zipf)
        if line is None:
            line = dict(pre, n_gpus=1, higher_is_better=True, scaling="weak", vs_baseline=None, data="synthetic", parity_check={"prefill": par})
        else:
            line["prefill"] = pre
            line["parity_check"]["prefill"] = par
            line["gpu_launches"] += pre["gpu_launches"]
            line["device_status"] |= pre["device_status"]
    if args.mode == "all" and not args.no_ref_gpu:
        try:
            line["reference_gpu"] = reference_gpu_arm(args, dev, layer, torch, moe, synth, dec)
        except Exception as e:                   # the baseline must never take the product's numbers down with it
            line["reference_gpu"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    if args.mode in ("all", "decode") and not args.no_cpu:
        del layer
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_reference_arm(20, 3)
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------------
# N > 1: expert parallel
def run_ep(args, world, rank, dev):
    """The decode configuration with the 256 experts split over `world` GPUs (strong scaling: the 16-row batch is fixed), and the
    long-prefill configuration (32768 tokens over the ranks) with uniform and with Zipf(1.3) routing."""
    import torch
    import torch.distributed as dist
    from hecate_b200 import ep, moe, synth
    from hecate_b200 import placement as PL
    dist.init_process_group("nccl", device_id=dev)
    pl = ep.shard_plan(rank, world, E)
    layer = Layer(dev, 100 + rank, pl["n_local"])
    tabs = layer.tabs
    line = None
    if args.mode in ("all", "decode"):
        line = ep_decode_arm(args, world, rank, dev, tabs, pl, torch, dist, ep, moe, synth, layer=layer)
    if args.mode in ("all", "prefill"):
        R = 32768 if args.mode == "all" else args.rows
        runs = (("prefill", 0.0), ("prefill_zipf", 1.3)) if args.mode == "all" else (("prefill", args.zipf),)
        for key, z in runs:
            res = ep_prefill_arm(args, world, rank, dev, tabs, R, z, torch, dist, ep, moe, synth, PL)
            if rank == 0:
                if line is None:
                    line = dict(res, n_gpus=world, higher_is_better=True, scaling="strong", vs_baseline=None, data="synthetic")
                else:
                    line[key] = res
                    line["gpu_launches"] += res["gpu_launches"]
                    line["device_status"] |= res["device_status"]
    L = args.layers if args.layers > 0 else (75 if (world == 8 and args.mode == "all") else 0)
    if L > 0:
        del layer, tabs
        torch.cuda.empty_cache()
        try:
            res = stack_arm(args, world, rank, dev, L, torch, dist, ep, moe, synth)
        except Exception as exc:                    # the headline arms above are measured already: report the failure, keep the line
            res = {"metric": "moe_stack_decode_us_per_layer", "error": f"{type(exc).__name__}: {exc}"[:300], "layers": L}
        if rank == 0:
            if line is None:
                line = dict(res, n_gpus=world, higher_is_better=True, scaling="strong", vs_baseline=None, data="synthetic")
            else:
                line["stack"] = res
    if rank == 0:
        print(json.dumps(line))
    dist.barrier()
    dist.destroy_process_group()


def stack_arm(args, world, rank, dev, L, torch, dist, ep, moe, synth):
    """The expert stack of a whole model: L MoE layers with per-layer weights and router (layer index in the seed), the experts
    of every layer split over the GPUs, decode batch of 8 tokens x (1 + 1 draft) = 16 rows that are data-parallel (rank r holds
    rows r, r + world, ...). Per layer and rank: dispatch of the rank's rows over peer memory + router + set-up (one launch) ->
    expert kernels -> combine of the rank's rows over peer memory. One CUDA graph replays all L layers of a step.
    Successive layers use different input batches, so every layer routes differently."""
    pl = ep.shard_plan(rank, world, E)
    layers = [Layer(dev, 1000 + 16 * l + rank, pl["n_local"]) for l in range(L)]
    g = torch.Generator(device=dev); g.manual_seed(7)
    wts = [(torch.randn(E, H, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(L)]
    bias = torch.zeros(E, dtype=torch.float32, device=dev)
    dec = ep.EpDecoder(rank, world, layers[0].tabs, E, dev, dist, use_peer=world > 1)
    own = list(range(rank, ROWS, world))
    n_own = len(own)
    NB = 4
    xs = [torch.from_numpy(synth.activations(b, 0, ROWS, H)).to(torch.bfloat16).to(dev) for b in range(NB + 1)]
    xo = [x[own].contiguous() for x in xs]
    sel = torch.empty(max(n_own, 1), TOPK, dtype=torch.int64, device=dev); rw = torch.empty(max(n_own, 1), TOPK, dtype=torch.float16, device=dev)
    sel16 = torch.empty(ROWS, TOPK, dtype=torch.int64, device=dev); rw16 = torch.empty(ROWS, TOPK, dtype=torch.float16, device=dev)
    f_own = torch.zeros(max(n_own, 1), H, dtype=torch.float32, device=dev)
    f = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)

    def step(b):
        for l in range(L):
            if world > 1:
                dec.step_dp_fused(xo[(b + l) % (NB + 1)], wts[l], bias, 1.0, sel16, rw16, f_own, ROWS, tables=layers[l].tabs)
            else:
                x = xs[(b + l) % (NB + 1)]
                moe.router_fused(x, wts[l], bias, None, None, sel16, rw16, TOPK, 1.0)
                dec.step(x, sel16, rw16, f, tables=layers[l].tabs)

    steps, warmup = max(1, min(args.steps, 20)), 3
    for i in range(2):
        step(i)
    torch.cuda.synchronize(); dist.barrier()
    run_step, per_step = make_graphed(step, list(range(NB)), torch, moe, not args.no_graph)
    for i in range(warmup):
        run_step(i % NB)
    torch.cuda.synchronize(); dist.barrier()
    with ClockSampler(dev.index) as cs:
        dist.barrier()
        t = timed(torch, run_step, steps, NB, lead=1)
        dist.barrier()
    ms = torch.tensor([t], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    st = torch.tensor([dec.status()], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
    resident = sum(lay.pool.numel() + 2 * (lay.gs.numel() + lay.us.numel() + lay.ds.numel()) for lay in layers)
    del run_step
    if dec.peer is not None:
        dist.barrier(); dec.peer.close()
    if rank != 0:
        return None
    t = float(ms.item())
    return {"metric": "moe_stack_decode_us_per_layer", "value": t * 1e3 / L, "unit": "us/layer", "layers": L, "ms_per_step": t, "steps": steps,
            "warmup": warmup, "tokens_per_s": 8 / (t * 1e-3), "rows_per_s": ROWS / (t * 1e-3), "experts_per_gpu_per_layer": pl["n_local"],
            "resident_gb_per_gpu": resident / 1e9, "launch": "eager" if args.no_graph else "one cuda graph per step over all layers",
            "dispatch_bytes_per_rank_per_layer": (world - 1) * n_own * H * 2 if world > 1 else 0,
            "combine_bytes_per_rank_per_layer": (world - 1) * n_own * H * 4 if world > 1 else 0,
            "config": {"workload": f"{L} MoE layers (per-layer random weights and routing from seed), decode M=8 tokens x 2 rows, experts "
                                   f"split over {world} GPUs, data-parallel tokens with dispatch + combine over NVLink peer memory every layer"},
            "gpu_launches": int(per_step * steps), "device_status": int(st.item()), "clocks": cs.summary()}


def ep_decode_arm(args, world, rank, dev, tabs, pl, torch, dist, ep, moe, synth, layer=None):
    """Two arms. "peer" (the headline): the 16 rows are data-parallel (rank r holds rows r, r + world, ...); per step every rank
    dispatches its rows (an all-gather over NVLink peer memory, done by the router's own launch), routes all rows, runs its experts
    on them and brings its own rows' sums back over peer memory: four launches (hmoe_decode_ep_dp). "nccl" (the baseline): rows
    replicated, router replicated, NCCL all-reduce of the fp32 partials."""
    steps, warmup = args.steps, max(3, args.warmup)
    wt = torch.from_numpy(synth.router_weight(0, 0, E, H)).to(dev).to(torch.bfloat16)
    bias = torch.zeros(E, dtype=torch.float32, device=dev)
    xs = [torch.from_numpy(synth.activations(b, 0, ROWS, H)).to(torch.bfloat16).to(dev) for b in range(NBATCH)]
    own = list(range(rank, ROWS, world))
    n_own = len(own)
    xo = [x[own].contiguous() for x in xs]
    xo_host = [x.cpu().pin_memory() for x in xo]
    xs_host = [x.cpu().pin_memory() for x in xs]
    sel = torch.empty(ROWS, TOPK, dtype=torch.int64, device=dev)
    rw = torch.empty(ROWS, TOPK, dtype=torch.float16, device=dev)
    sel_o = torch.empty(max(n_own, 1), TOPK, dtype=torch.int64, device=dev); rw_o = torch.empty(max(n_own, 1), TOPK, dtype=torch.float16, device=dev)
    f = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    f_o = torch.zeros(max(n_own, 1), H, dtype=torch.float32, device=dev)
    f_host = torch.empty(ROWS, H, dtype=torch.float32).pin_memory()
    x_in = torch.empty(ROWS, H, dtype=torch.bfloat16, device=dev)
    xo_in = torch.empty(max(n_own, 1), H, dtype=torch.bfloat16, device=dev)
    results, outs = {}, {}
    disp_bytes = 0
    # "peer2": every expert on two GPUs (this rank also holds the next rank's experts, generated from that rank's seed, so the
    # copies are identical); each step gives a picked expert to the less loaded of its two holders
    modes = ("nccl", "peer", "peer2") if layer is not None and world > 1 else ("nccl", "peer")
    for mode in modes:
        if mode == "peer2":
            nxt = Layer(dev, 100 + (rank + 1) % world, layer.n)
            n1 = layer.n
            both = [[L.view(e, k) for L in (layer, nxt) for e in range(n1)] for k in range(3)] + \
                   [[t[e] for L in (layer, nxt) for t in (getattr(L, a),) for e in range(n1)] for a in ("gs", "us", "ds")]
            tabs2 = moe.ExpertTables(H, I, TOPK, *both, group=GROUP,
                                     shared=(layer.view(n1, 0), layer.view(n1, 1), layer.view(n1, 2), layer.gs[n1], layer.us[n1], layer.ds[n1]), device=dev)
            tabs2.keep += [layer.pool, nxt.pool, nxt.gs, nxt.us, nxt.ds]
            dec = ep.EpDecoder(rank, world, tabs2, E, dev, dist, use_peer=True, replicas=2)
        else:
            dec = ep.EpDecoder(rank, world, tabs, E, dev, dist, use_peer=(mode == "peer"))
        if mode != "nccl":
            disp_bytes = dec.dispatch_bytes(ROWS, with_routing=False)

            def step(x):                        # x: this rank's rows; one launch dispatches them, routes all rows and sets up
                dec.step_dp_fused(x, wt, bias, 1.0, sel, rw, f_o, ROWS)
            inputs, hosts, x_dev, out_dev = xo, xo_host, xo_in, f_o
        else:
            def step(x):                        # x: all rows
                moe.router_fused(x, wt, bias, None, None, sel, rw, TOPK, 1.0)
                dec.step(x, sel, rw, f)
            inputs, hosts, x_dev, out_dev = xs, xs_host, x_in, f

        for i in range(warmup):
            step(inputs[i % NBATCH])
        torch.cuda.synchronize(); dist.barrier()
        out_dev.zero_(); step(inputs[0]); torch.cuda.synchronize()
        outs[mode] = (f[own] if mode == "nccl" else f_o[:n_own]).clone(); out_dev.zero_()     # this rank's rows of one step, for the cross-check
        if mode == "peer2":
            dm = torch.tensor([float(moe.route_distinct(dec.ws))], device=dev)
            dm_all = [torch.zeros_like(dm) for _ in range(world)]
            dist.all_gather(dm_all, dm)
            d_bal = [float(t.item()) for t in dm_all]
        dist.barrier()
        graph = (not args.no_graph) and mode != "nccl"      # NCCL calls are left eager
        run_step, per_step = make_graphed(step, inputs, torch, moe, graph)
        for i in range(warmup):
            run_step(i % NBATCH)
        torch.cuda.synchronize(); dist.barrier()
        with ClockSampler(dev.index) as cs:
            dist.barrier()
            t = timed(torch, run_step, steps, NBATCH, lead=3)
            dist.barrier()
        ms = torch.tensor([t], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        launches = per_step * steps
        if mode == "peer":
            # for comparison: the same buffers with the rows already replicated on every rank (no dispatch; e.g. behind a
            # tensor-parallel attention), combine of all rows over peer memory
            def step_rep(x):
                moe.router_fused(x, wt, bias, None, None, sel, rw, TOPK, 1.0)
                dec.step(x, sel, rw, f)
            for i in range(3):
                step_rep(xs[i])
            torch.cuda.synchronize(); dist.barrier()
            run_rep, _ = make_graphed(step_rep, xs, torch, moe, graph)
            for i in range(3):
                run_rep(i)
            torch.cuda.synchronize(); dist.barrier()
            t_rep = torch.tensor([timed(torch, run_rep, steps, NBATCH, lead=3)], device=dev)
            dist.all_reduce(t_rep, op=dist.ReduceOp.MAX)
            rep_us = float(t_rep.item()) * 1e3
            del run_rep
            dist.barrier()

        def e2e_step(b):
            x_dev.copy_(hosts[b], non_blocking=True); step(x_dev); f_host[:out_dev.shape[0]].copy_(out_dev, non_blocking=True)
        run_e2e, _ = make_graphed(e2e_step, list(range(NBATCH)), torch, moe, graph)
        for i in range(3):
            run_e2e(i % NBATCH)
        torch.cuda.synchronize(); dist.barrier()
        n2 = min(steps, 200)
        t0 = time.perf_counter()
        for i in range(n2):
            run_e2e(i % NBATCH); torch.cuda.synchronize()
        e2e = torch.tensor([(time.perf_counter() - t0) / n2], device=dev)
        dist.all_reduce(e2e, op=dist.ReduceOp.MAX)
        st = torch.tensor([dec.status()], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
        results[mode] = dict(ms=float(ms.item()), e2e=float(e2e.item()), launches=int(launches), status=int(st.item()), clocks=cs.summary())
        del run_step, run_e2e
        if dec.peer is not None:
            dist.barrier(); dec.peer.close()
        if mode == "peer2":
            del dec, tabs2, nxt, both
            torch.cuda.empty_cache()
    # load balance of the last batch: distinct local experts per rank (sel holds the replicated routing of the nccl arm's last step)
    mine = (sel >= pl["lo"]) & (sel < pl["lo"] + pl["n_local"])
    d_local = torch.tensor([float(torch.unique(sel[mine]).numel()) if bool(mine.any()) else 0.0], device=dev)
    d_all = [torch.zeros_like(d_local) for _ in range(world)]
    dist.all_gather(d_all, d_local)
    e = torch.tensor(list(errors(outs["peer"].cpu().numpy(), outs["nccl"].cpu().numpy())) if n_own else [0.0, 0.0, 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    e2 = None
    if "peer2" in outs:
        e2 = torch.tensor(list(errors(outs["peer2"].cpu().numpy(), outs["nccl"].cpu().numpy())) if n_own else [0.0, 0.0, 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(e2, op=dist.ReduceOp.MAX)
    if rank != 0:
        return None
    dl = [float(t.item()) for t in d_all]
    two = "peer2" in results and results["peer2"]["ms"] < results["peer"]["ms"]       # the faster arm is the headline, named in config
    r = results["peer2"] if two else results["peer"]
    pk = peaks()
    bytes_rank_max = (max(d_bal if two else dl) + 1) * EXPERT_BYTES + E * H * 2
    extra = {}
    if "peer2" in results:
        extra = {"one_holder_us_per_layer": results["peer"]["ms"] * 1e3, "two_holders_us_per_layer": results["peer2"]["ms"] * 1e3,
                 "distinct_local_experts_two_holders": d_bal, "load_imbalance_two_holders": max(d_bal) / (sum(d_bal) / len(d_bal))}
    return {
        "metric": METRIC, "value": ROWS / (r["ms"] * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": r["ms"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int4 x fp16 -> fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD + f"; experts split over {world} GPUs ({pl['n_local']} each), tokens data-parallel ({n_own} rows per GPU), "
                                          "dispatch and combine as an all-to-all over NVLink peer memory"
                                          + ("; every expert held by two GPUs (twice the weight memory), each step served by the less loaded holder" if two else ""),
                   "l2": "inputs larger than L2: 8 input batches in a ring, each step streams different experts"},
        "us_per_layer": r["ms"] * 1e3, "nccl_allreduce_us_per_layer": results["nccl"]["ms"] * 1e3,
        "replicated_rows_us_per_layer": rep_us, **extra,
        "distinct_local_experts_last_step": dl, "load_imbalance_max_over_mean": max(dl) / (sum(dl) / len(dl)),
        "combine_bytes_per_rank": (world - 1) * n_own * H * 4, "dispatch_bytes_per_rank": disp_bytes,
        "roofline": {"bound": "hbm", "kernel": "decode kernels of the most loaded rank (whole call)", "achieved": bytes_rank_max / (r["ms"] * 1e-3) / 1e9,
                     "peak": pk["hbm"], "unit": "GB/s", "frac": bytes_rank_max / (r["ms"] * 1e-3) / 1e9 / pk["hbm"], "peak_kind": pk["kind"], "traffic": None},
        "e2e": {"value": ROWS / r["e2e"], "unit": UNIT, "h2d_bytes_per_step": n_own * H * 2, "d2h_bytes_per_step": n_own * H * 4,
                "us_per_layer": r["e2e"] * 1e6, "note": "per rank: its own rows in, its own rows' result out"},
        "parity_check": {"decode": dict({"peer_all_to_all_vs_nccl_allreduce": {"max_rel": float(e[0]), "mean_abs": float(e[1]), "norm_rel": float(e[2]),
                                                                               "ok": bool(float(e[2]) < 1e-3)}},
                                        **({"two_holders_vs_nccl_allreduce": {"max_rel": float(e2[0]), "mean_abs": float(e2[1]), "norm_rel": float(e2[2]),
                                                                              "ok": bool(float(e2[2]) < 1e-3)}} if e2 is not None else {}))},
        "gpu_launches": r["launches"], "device_status": max(x["status"] for x in results.values()), "clocks": r["clocks"]}


def ep_prefill_arm(args, world, rank, dev, tabs, R, zipf, torch, dist, ep, moe, synth, PL):
    """R tokens in total, split over the ranks; uniform or Zipf routing. Placement: contiguous ids for uniform routing; under
    skew the experts are dealt to the GPUs by load (hecate_b200.placement.balance) from the pick counts of ANOTHER sample of the
    same popularity (the routing log of an earlier chunk), and the selection is expressed in router positions, as a router with
    permuted weight rows would emit it. Both dispatches (NCCL all-gather; all-to-all-v over NVLink peer memory, a row only to the
    ranks that hold one of its experts) and both combines (NCCL reduce-scatter; fused into the down GEMM over peer memory) are
    timed and cross-checked; the line reports the fastest pair and names it."""
    rpr = R // world
    steps, warmup = max(1, min(args.steps, 20)), max(3, min(args.warmup, 5))
    sel_all, rw_all = synth.zipf_routing(10, 0, R, E, TOPK, zipf)
    want = getattr(args, "placement", "auto")
    use_plan = want == "balanced" or (want == "auto" and zipf > 0)
    base_imb = PL.contiguous(PL.pick_counts(sel_all, E), world).imbalance()
    if use_plan:
        cal, _ = synth.zipf_routing(11, 0, R, E, TOPK, zipf)
        plan = PL.balance(PL.pick_counts(cal, E), world, extra_slots=0)
        sel_all = PL.positions(sel_all, plan)
    pl = ep.shard_plan(rank, world, E)
    x = torch.from_numpy(synth.activations(rank, 0, rpr, H)).to(torch.bfloat16).to(dev)
    sel = torch.from_numpy(sel_all[rank * rpr:(rank + 1) * rpr]).to(dev); rw = torch.from_numpy(rw_all[rank * rpr:(rank + 1) * rpr]).to(dev)
    out = torch.empty(rpr, H, dtype=torch.float32, device=dev)
    times, outs = {}, {}
    st_all = launches = 0
    sent_rows = 0
    # [dispatch +] combine through the grouped GEMMs; steps of few rows in total also through the streaming kernels ("short": the
    # local experts via hmoe_short_prefill_ep, NCCL all-gather and reduce-scatter around them)
    modes = ("nccl", "peer", "a2a+nccl", "a2a+peer") + (("short",) if R <= moe.forward_short_rows() else ())
    for mode in modes:
        a2a = mode.startswith("a2a")
        p = ep.EpPrefill(rank, world, tabs, E, rpr, dev, dist, use_peer=mode.endswith("peer"), dispatch="peer" if a2a else "nccl", short=mode == "short")
        for _ in range(warmup):
            p.step(x, sel, rw, out)
        torch.cuda.synchronize(); dist.barrier()
        outs[mode] = out[::256].clone()
        if a2a:
            sent_rows = int(p.sent.item()) // warmup
        l0 = moe.launch_count()
        with ClockSampler(dev.index) as cs:
            dist.barrier()
            t = timed(torch, lambda i: p.step(x, sel, rw, out), steps, 1, lead=1)
            dist.barrier()
        ms = torch.tensor([t], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        times[mode] = float(ms.item())
        launches = moe.launch_count() - l0
        st = torch.tensor([p.status()], device=dev); dist.all_reduce(st, op=dist.ReduceOp.MAX)
        st_all |= int(st.item())
        if p.peer is not None:
            dist.barrier(); p.peer.close()
        del p
    best = min(times, key=times.get)               # all arms are timed; the line reports the fastest one and names it
    e3 = None
    if "short" in outs:
        e3 = torch.tensor(list(errors(outs["short"].cpu().numpy(), outs["nccl"].cpu().numpy())), device=dev, dtype=torch.float64)
        dist.all_reduce(e3, op=dist.ReduceOp.MAX)
    e = torch.tensor(list(errors(outs["peer"].cpu().numpy(), outs["nccl"].cpu().numpy())), device=dev, dtype=torch.float64)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    e2 = torch.tensor(list(errors(outs["a2a+peer"].cpu().numpy(), outs["nccl"].cpu().numpy())), device=dev, dtype=torch.float64)
    dist.all_reduce(e2, op=dist.ReduceOp.MAX)
    sr = torch.tensor([sent_rows], device=dev); dist.all_reduce(sr, op=dist.ReduceOp.MAX)
    sent_rows = int(sr.item())
    picks = np.array([int(((sel_all >= r * pl["n_local"]) & (sel_all < (r + 1) * pl["n_local"])).sum()) for r in range(world)])
    if rank != 0:
        return None
    flop = (TOPK * R + R) * PICK_FLOP
    t = times[best] * 1e-3
    pk = peaks()
    return {
        "metric": "moe_prefill_expert_gemm_tflops", "value": flop / t / 1e12, "unit": "TFLOP/s", "steps": steps, "warmup": warmup,
        "ms_per_step": t * 1e3, "dtype": "int4 -> fp16 x fp16 -> fp32 (tcgen05)",
        "config": {"workload": f"prefill M={R} tokens over {world} GPUs ({rpr} each), Zipf({zipf}) top-8 over {E} experts + shared, "
                               f"{pl['n_local']} experts per GPU ({'placed by load from a calibration sample' if use_plan else 'contiguous ids'}), "
                               + ("dispatch: all-to-all-v over NVLink peer memory" if best.startswith("a2a") else "dispatch: all-gather (NCCL)")
                               + ", combine: " + ("fused into the down GEMM over NVLink peer memory" if best.endswith("peer") else "NCCL reduce-scatter")
                               + (", local experts through the streaming kernels (short prefill)" if best == "short" else ""),
                   "l2": "inputs larger than L2"},
        "tokens_per_s": R / t, "nccl_reduce_scatter_ms_per_step": times["nccl"], "peer_combine_ms_per_step": times["peer"],
        "peer_dispatch_nccl_combine_ms_per_step": times["a2a+nccl"], "peer_dispatch_peer_combine_ms_per_step": times["a2a+peer"],
        **({"short_prefill_ms_per_step": times["short"]} if "short" in times else {}),
        "dispatch_bytes_per_rank": (world - 1) * rpr * (H * 2 + TOPK * 10) if not best.startswith("a2a") else sent_rows * H * 2 + (world - 1) * rpr * TOPK * 10,
        "dispatch_bytes_per_rank_all_gather": (world - 1) * rpr * (H * 2 + TOPK * 10),
        "dispatch_bytes_per_rank_all_to_all_v": sent_rows * H * 2 + (world - 1) * rpr * TOPK * 10,
        "combine_bytes_per_rank": (world - 1) * rpr * H * 4,
        "picks_per_rank": picks.tolist(), "load_imbalance_max_over_mean": float(picks.max() / picks.mean()),
        "load_imbalance_contiguous_placement": base_imb,
        "roofline": {"bound": "tensor", "kernel": "whole step incl. collectives", "achieved": flop / t / 1e12, "peak": pk["bf16"] * world, "unit": "TFLOP/s",
                     "frac": flop / t / 1e12 / (pk["bf16"] * world), "peak_kind": pk["kind"] + " burst (bf16_tflops) x n_gpus",
                     "frac_sustained": flop / t / 1e12 / (pk["bf16_sustained"] * world), "traffic": None},
        "parity_check": {"peer_combine_vs_nccl_reduce_scatter": {"max_rel": float(e[0]), "mean_abs": float(e[1]), "norm_rel": float(e[2]),
                                                                 "ok": bool(float(e[2]) < 1e-5)},
                         "peer_dispatch_and_combine_vs_nccl": {"max_rel": float(e2[0]), "mean_abs": float(e2[1]), "norm_rel": float(e2[2]),
                                                               "ok": bool(float(e2[2]) < 1e-5)},
                         **({"short_prefill_vs_grouped_gemms": {"max_rel": float(e3[0]), "mean_abs": float(e3[1]), "norm_rel": float(e3[2]),
                                                                "ok": bool(float(e3[2]) < 1e-3)}} if e3 is not None else {})},
        "gpu_launches": int(launches), "device_status": int(st_all), "clocks": cs.summary()}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="all", choices=["all", "decode", "prefill"], help="all (default): the decode headline plus the prefill, "
                    "parity and baseline objects; decode / prefill: that arm alone")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-check", action="store_true", help="skip the parity checks against the CPU checker")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip the reference GPU kernels")
    ap.add_argument("--all-variants", action="store_true", help="--impl reference: also time the scalar build of the engine")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels eagerly instead of replaying CUDA graphs")
    ap.add_argument("--rows", type=int, default=8192, help="prefill rows (N = 1, or --mode prefill)")
    ap.add_argument("--zipf", type=float, default=1.1, help="prefill expert popularity exponent (0 = uniform)")
    ap.add_argument("--placement", default="auto", choices=["auto", "contiguous", "balanced"],
                    help="N > 1 prefill: expert -> GPU map; auto = balanced by load when the routing is skewed")
    ap.add_argument("--layers", type=int, default=0, help="N > 1: also run a stack of this many MoE layers (default: 75 at 8 GPUs, else none)")
    ap.add_argument("--experts", type=int, default=E, help="routed experts resident (256 = the benchmark; fewer only for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
