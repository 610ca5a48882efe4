#!/usr/bin/env python
"""Benchmark of the MoE expert hot path on B200: one decode MoE layer call per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the decode configuration of the benchmark definition): hidden 6144, 256 routed experts, top-8 sigmoid/bias router,
one shared expert, SwiGLU experts gate/up [2048 x 6144] and down [6144 x 2048] in packed int4 with a bf16 scale per 128
input columns, decode batch of 8 tokens each with one MTP draft = 16 rows. Inputs are synthetic (seeded): codes uniform,
scales lognormal(-4, 0.5), activations N(0, 1) in bf16, router weight N(0, 0.02) in bf16.

A step = router -> prepare -> gate_up (+ SiLU * up * weight) -> down -> combine into the fp32 layer output. `value` is rows/s
with inputs resident in HBM; `e2e` is the same call chain fed from pinned host memory with the host<->device copies inside
the timed region. Consecutive steps use different input batches (8 in a ring), so each step selects a different ~100 of the
256 experts: about 2 GB of the 4.85 GB layer is streamed per step, far more than the 126 MB L2.

`--impl reference` times the reference's own CPU expert engine (oracle/_ref, built from the reference source) on the host
cores, on a bounded sample of the same workload.
"""
import argparse
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
NBATCH = 8
METRIC = "moe_layer_decode_rows_per_s"
UNIT = "rows/s"
WORKLOAD = "decode M=8 tokens x (1 + 1 MTP draft) = 16 rows, H=6144, 256 experts top-8 + shared, int4 g128 bf16 scales"


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


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


# ----------------------------------------------------------------------------------------------------------------------
def cpu_reference_arm(steps, warmup, seed=0):
    """Times the reference CPU engine (or, without it, this repository's restatement) on 8-row jobs of the workload."""
    from oracle import oracle as O
    from hecate_b200 import synth
    cores = os.cpu_count() or 1
    threads = max(1, min(60, cores - 2))
    sel, rw = synth.zipf_routing(seed, 0, 8, E, TOPK, 0.0)
    x = synth.activations(seed, 0, 8, H).astype(np.float16)
    ids = sorted(set(int(e) for e in sel.reshape(-1)))
    remap = {e: i for i, e in enumerate(ids)}
    sel_local = np.vectorize(remap.get)(sel).astype(np.int64)
    experts = []
    for e in ids:                       # row-major int4 + one fp32 scale per row: the engine's own format
        mk = lambda kind, n: synth.rand_bytes(seed, synth.stream_id(0, kind, e), n).reshape(-1)
        sc = lambda kind, N, K: synth.scales(seed, 0, kind, e, N, K, K)
        experts.append(O.Expert(mk("gate_q", I * H // 2).reshape(I, H // 2), mk("up_q", I * H // 2).reshape(I, H // 2),
                                mk("down_q", H * I // 2).reshape(H, I // 2), sc("gate_s", I, H), sc("up_s", I, H),
                                sc("down_s", H, I), H, I, packed=False))
    times = []
    if O.ref_available():
        kind = "reference"
        eng = O.RefEngine(experts, 0, threads=threads, core0=0)
        try:
            for i in range(warmup + steps):
                _, dt = eng.job(x, sel_local, rw)
                if i >= warmup:
                    times.append(dt)
        finally:
            eng.stop()
    else:
        kind = "port"
        threads = O.threads()
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            O.moe_forward(H, I, 0, x, sel_local, rw, 0, experts)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
    t = float(np.median(times))
    return {"value": 8.0 / t, "unit": UNIT, "cores": threads, "kind": kind, "ms_per_job": t * 1e3,
            "sample": f"{len(times)} jobs of 8 rows ({len(ids)} distinct routed experts, per-row fp32 scales, no shared expert), "
                      f"median ISSUE->DONE time"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 50))
    cb = cpu_reference_arm(steps, max(1, min(args.warmup, 5)))
    line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": args.warmup, "ms_per_step": cb["ms_per_job"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "int4 x int8 -> fp32", "data": "synthetic",
            "config": {"workload": WORKLOAD + " [CPU sample: one 8-row job per step]"},
            "cpu_baseline": cb, "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------------------------------------
def build_layer(dev, seed, experts, torch, moe):
    """Seeded synthetic experts resident in HBM: `experts` routed experts + one shared expert."""
    from hecate_b200 import synth
    n = len(experts)
    pool = torch.empty((n + 1) * 3 * PER_MATRIX, dtype=torch.uint8, device=dev)
    moe.fill_bytes(pool, seed, synth.stream_id(0, "gate_q", 0))
    view = lambda e, k: pool[(e * 3 + k) * PER_MATRIX:(e * 3 + k + 1) * PER_MATRIX]
    g = torch.Generator(device=dev); g.manual_seed(seed + 1)
    sc = lambda N, K: (torch.randn(n + 1, N // 64, K // GROUP, 64, device=dev, generator=g) * 0.5 - 4.0).exp().to(torch.bfloat16)
    gs, us, ds = sc(I, H), sc(I, H), sc(H, I)          # device order [N/64][K/128][64] per expert
    shared = (view(n, 0), view(n, 1), view(n, 2), gs[n], us[n], ds[n])
    tabs = moe.ExpertTables(H, I, TOPK, [view(e, 0) for e in range(n)], [view(e, 1) for e in range(n)],
                            [view(e, 2) for e in range(n)], list(gs[:n]), list(us[:n]), list(ds[:n]), group=GROUP, shared=shared, device=dev)
    tabs.keep.append(pool)
    return tabs


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


def run_ours(args):
    import torch
    import torch.distributed as dist
    from hecate_b200 import moe, synth
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from hecate_b200 import ep
        return ep.bench_decode(args, world, rank, dev)
    steps, warmup = args.steps, max(3, args.warmup)
    E = args.experts
    tabs = build_layer(dev, 0, list(range(E)), torch, moe)
    wt = torch.from_numpy(synth.router_weight(0, 0, E, H)).to(dev).to(torch.bfloat16)
    bias = torch.zeros(E, dtype=torch.float32, device=dev)
    xs_host = [torch.from_numpy(synth.activations(b, 0, ROWS, H)).to(torch.bfloat16).pin_memory() for b in range(NBATCH)]
    xs = [x.to(dev) for x in xs_host]
    sel = torch.empty(ROWS, TOPK, dtype=torch.int64, device=dev)
    rw = torch.empty(ROWS, TOPK, dtype=torch.float16, device=dev)
    ws = moe.decode_workspace(H, I, dev)
    y = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    f = torch.zeros(ROWS, H, dtype=torch.float32, device=dev)
    x_in = torch.empty(ROWS, H, dtype=torch.bfloat16, device=dev)
    f_host = torch.empty(ROWS, H, dtype=torch.float32).pin_memory()

    def step(x):
        moe.router_fused(x, wt, bias, None, None, sel, rw, TOPK, 1.0)
        moe.decode(tabs, x, sel, rw, y, ws)
        moe.moe4_combine(f, 0, y, ROWS, 0)

    # distinct experts per batch (for the algorithmic byte count)
    distinct = []
    for b in range(NBATCH):
        moe.router_fused(xs[b], wt, bias, None, None, sel, rw, TOPK, 1.0)
        distinct.append(int(torch.unique(sel).numel()))
    for i in range(warmup):
        step(xs[i % NBATCH])
    torch.cuda.synchronize()
    # One CUDA graph per input batch (the reference runs its decode forward as captured graphs too, runtime/core/exl3_vgraph.py):
    # a step allocates nothing, does not synchronise and its launch shapes do not depend on the routing.
    run_step, launches_per_step = make_graphed(step, xs, torch, moe, not args.no_graph)
    for i in range(warmup):
        run_step(i % NBATCH)
    torch.cuda.synchronize()
    phase = np.zeros(3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        torch.cuda.synchronize()
        ev0.record()
        for i in range(steps):
            run_step(i % NBATCH)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1)
        if len(cs.samples) < 5:           # very short runs: keep the same load going so the clock record is not empty
            t_end = time.time() + 0.4
            while time.time() < t_end:
                run_step(0); torch.cuda.synchronize()
    launches = launches_per_step * steps
    moe.set_profiling(True)
    # kernel durations: a second pass over the same steps launched eagerly back to back, CUDA events around each kernel on
    # its stream (recorded by the library into a ring); read after the pass
    for i in range(min(steps, 32)):
        step(xs[i % NBATCH])
    torch.cuda.synchronize()
    phase = np.array(moe.decode_phase_times())
    moe.set_profiling(False)
    status = moe.ws_status(ws)
    mean_d = float(np.mean([distinct[i % NBATCH] for i in range(steps)]))
    gate_up_bytes = (mean_d + 1) * GATE_UP_BYTES
    layer_bytes = (mean_d + 1) * EXPERT_BYTES + E * H * 2 + ROWS * H * 6
    peak, peak_kind = measured_peaks()
    achieved = gate_up_bytes / (phase[1] * 1e-3) / 1e9
    # DRAM traffic of one gate_up launch: dram__bytes_read + write of an ncu capture of the reduced case (--experts 64: 709.4 MB
    # for 722.3 MB of algorithmic bytes, profiles/decode_stream_kernels_experts64.md), scaled to this launch by the experts it streams
    traffic = 0.982 * gate_up_bytes
    ms_per_step = ms / steps

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

    cb = cpu_reference_arm(20, 3) if not args.no_cpu else None
    line = {
        "metric": METRIC, "value": ROWS / (ms_per_step * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int4 x fp16 -> fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD if E == 256 else WORKLOAD + f" [reduced to {E} experts]", "launch": "eager" if args.no_graph else "cuda graph per input batch", "l2": "inputs larger than L2: ~2 GB of weights streamed per step, 8 input batches in a ring",
                   "distinct_experts_per_step": mean_d},
        "us_per_layer": ms_per_step * 1e3,
        "layer_hbm_gbs": layer_bytes / (ms_per_step * 1e-3) / 1e9,
        "layer_hbm_frac": layer_bytes / (ms_per_step * 1e-3) / 1e9 / peak,
        "phase_us": {"prepare": phase[0] * 1e3, "gate_up": phase[1] * 1e3, "down": phase[2] * 1e3},
        "roofline": {"bound": "hbm", "kernel": "decode_stream_kernel (gate_up)", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                     "algorithmic_bytes_per_launch": gate_up_bytes},
        "e2e": {"value": ROWS / e2e_s, "unit": UNIT, "h2d_bytes_per_step": ROWS * H * 2, "d2h_bytes_per_step": ROWS * H * 4,
                "us_per_layer": e2e_s * 1e6},
        "gpu_launches": int(launches), "device_status": int(status), "clocks": cs.summary(),
    }
    if cb:
        line["cpu_baseline"] = cb
    print(json.dumps(line))


def run_prefill(args):
    """Prefill configuration: M = 8192 tokens, Zipf(1.1) expert popularity, top-8 without replacement, + shared expert.
    A step = permute -> gather -> grouped gate_up GEMM (+ SiLU epilogue) -> grouped down GEMM (+ scatter-add epilogue).
    value = TFLOP/s over the algorithmic flops 2 * (8 R + R) * 37,748,736 (padding columns not counted)."""
    import torch
    from hecate_b200 import moe, synth
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        from hecate_b200 import ep
        return ep.bench_prefill(args, world, int(os.environ.get("RANK", "0")), dev)
    E, R = args.experts, args.rows
    steps, warmup = min(args.steps, 200), max(3, min(args.warmup, 10))
    tabs = build_layer(dev, 0, list(range(E)), torch, moe)
    NB = 2
    xs = [torch.from_numpy(synth.activations(b, 0, R, H)).to(torch.bfloat16).to(dev) for b in range(NB)]
    routes = [synth.zipf_routing(10 + b, 0, R, E, TOPK, args.zipf) for b in range(NB)]
    sels = [torch.from_numpy(r[0]).to(dev) for r in routes]; rws = [torch.from_numpy(r[1]).to(dev) for r in routes]
    ws = moe.prefill_workspace(R, TOPK, E, H, I, dev)
    out = torch.zeros(R, H, dtype=torch.float32, device=dev)
    x_host = xs[0].cpu().pin_memory(); out_host = torch.empty(R, H, dtype=torch.float32).pin_memory()
    x_in = torch.empty_like(xs[0])

    def step(i):
        out.zero_()
        moe.prefill(tabs, xs[i % NB], sels[i % NB], rws[i % NB], out, ws)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    l0 = moe.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as cs:
        ev0.record()
        for i in range(steps):
            step(i)
        ev1.record()
        torch.cuda.synchronize()
        ms = ev0.elapsed_time(ev1) / steps
    launches = moe.launch_count() - l0
    status = moe.ws_status(ws)
    t0 = time.perf_counter()
    for i in range(min(steps, 20)):
        x_in.copy_(x_host, non_blocking=True); out.zero_()
        moe.prefill(tabs, x_in, sels[0], rws[0], out, ws)
        out_host.copy_(out, non_blocking=True); torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / min(steps, 20)
    flop = 2.0 * (TOPK * R + R) * (3 * I * H)
    counts = np.bincount(routes[0][0].reshape(-1), minlength=E)
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0)); kind = "measured (sustained)" if peaks else "fallback"
    tf = flop / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "moe_prefill_expert_gemm_tflops", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 -> fp16 x fp16 -> fp32 (tcgen05)",
        "data": "synthetic",
        "config": {"workload": f"prefill M={R} tokens, Zipf({args.zipf}) top-8 over {E} experts + shared, H=6144, int4 g128 bf16 scales",
                   "l2": "inputs larger than L2 (4.85 GB of weights, 0.9 GB gathered inputs)", "max_picks_per_expert": int(counts.max()),
                   "min_picks_per_expert": int(counts.min())},
        "tokens_per_s": R / (ms * 1e-3),
        "roofline": {"bound": "tensor", "kernel": "prefill_gemm_kernel<2> + <1> (whole step)", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                     "frac": tf / peak, "peak_kind": kind, "traffic": None},
        "e2e": {"value": flop / e2e_s / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": R * H * 2, "d2h_bytes_per_step": R * H * 4,
                "ms_per_step": e2e_s * 1e3},
        "gpu_launches": int(launches), "device_status": int(status), "clocks": cs.summary()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-graph", action="store_true", help="launch the step's kernels eagerly instead of replaying CUDA graphs")
    ap.add_argument("--mode", default="decode", choices=["decode", "prefill"], help="decode (default, the headline) or prefill")
    ap.add_argument("--rows", type=int, default=8192, help="prefill rows")
    ap.add_argument("--zipf", type=float, default=1.1, help="prefill expert popularity exponent (0 = uniform)")
    ap.add_argument("--placement", default="auto", choices=["auto", "contiguous", "balanced"],
                    help="N > 1 prefill: expert -> GPU map; auto = balanced by load when --zipf > 0")
    ap.add_argument("--extra-slots", type=int, default=0, help="N > 1 prefill, balanced placement: slots for copies of the hottest experts")
    ap.add_argument("--experts", type=int, default=E, help="routed experts resident (256 = the benchmark; fewer only for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.mode == "prefill":
        run_prefill(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
