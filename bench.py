"""MoE layer forward+backward throughput on B200 (tokens/s), one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mixtral|olmoe|dsv3|cfg1|routing]
                    [--impl reference] [--ep peer|nccl] [--cuda-graph] [--no-cpu-baseline]

A step is one forward+backward of the MoE layer on one batch of synthetic tokens. The default
workload is the Mixtral-shape configuration (T=16384, H=4096, I=14336, E=8, top-2, router logits
~N(0,1) injected): it is the configuration the metric's "at 1/2/4/8 B200" clause and the
expert-parallel scaling target are stated on, and it fits one GPU. With N > 1 the experts are
sharded over the ranks (8/N per GPU), the global batch stays fixed (strong scaling, T/N tokens per
rank) and rows travel by the fused peer-memory kernels (`--ep peer`, default) or NCCL all-to-all
(`--ep nccl`). `--cuda-graph` (one GPU) times the step as one CUDA graph replay.

Rank 0 prints one JSON line. `value` is timed with every input resident in HBM; `e2e` repeats the
measurement through the public `MoE` API with pinned-host inputs copied in and results copied out
inside the timed region; `roofline` is the dominant kernel (CUDA events around each of its
launches inside the timed region); `cpu_baseline` is the CPU oracle (a port of the reference's
torch path) on a bounded sample of the same workload. `--impl reference` times that CPU path alone.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

_ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(_ROOT, "flash-model-architectures_b200"), _ROOT):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch
import torch.distributed as dist

WORKLOADS = {
    # name: T, H, I, E, k, seed, router
    "cfg1": dict(T=512, H=256, I=512, E=8, k=2, seed=0, router="gate"),
    "olmoe": dict(T=8192, H=2048, I=1024, E=64, k=8, seed=1, router="gate"),
    "mixtral": dict(T=16384, H=4096, I=14336, E=8, k=2, seed=2, router="logits"),
    "dsv3": dict(T=32768, H=7168, I=2048, E=256, k=8, seed=3, router="zipf"),
}
CPU_SAMPLE_TOKENS = {"cfg1": 512, "olmoe": 512, "mixtral": 256, "dsv3": 256}
# The DeepSeek-V3 shape holds 42 GiB of float32 expert weights (and as much again for their gradients):
# its CPU sample runs on 8 of the 256 experts with top-8 routing among those (the same FLOPs per token).
CPU_SAMPLE_EXPERTS = {"dsv3": 8}
METRIC = "moe_layer_fwd_bwd_tokens_per_s"
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each GEMM at N = 1 from
# an ncu capture of this same command (profiles/grouped_gemm_mixtral_dram_traffic.md). grouped_wgrad
# is the mean of its two launches per step.
NCU_TRAFFIC_BYTES = {
    "mixtral": {
        "grouped_wgrad": 4.89e9, "grouped_gemm[NT,swiglu]": 11.05e9, "grouped_gemm[NN,store]": 17.45e9,
        "grouped_gemm[NT,store]": 7.24e9, "grouped_gemm[NN,swiglu_bwd]": 9.03e9,
    },
}


def step_flops(w: dict, tokens: int) -> float:
    """18*T*k*H*I for the expert MLPs (forward 6, input gradients 6, weight gradients 6 per M*H*I)
    plus 6*T*H*E for the router GEMM when the workload has one."""
    f = 18.0 * tokens * w["k"] * w["H"] * w["I"]
    if w["router"] == "gate":
        f += 6.0 * tokens * w["H"] * w["E"]
    return f


def kernel_flops(label: str, w: dict, rows: float) -> float | None:
    mhi = rows * w["H"] * w["I"]
    return {
        "grouped_gemm[NT,swiglu]": 4 * mhi,
        "grouped_gemm[NT,store]": 2 * mhi,
        "grouped_gemm[NN,swiglu_bwd]": 2 * mhi,
        "grouped_gemm[NN,store]": 4 * mhi,
        "grouped_wgrad": 3 * mhi,  # two launches per step: 2*MHI (down) and 4*MHI (up); this is their mean
    }.get(label)


def measured_peaks() -> tuple[float, str]:
    path = os.path.join(_ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            peaks = json.load(fh)
        return float(peaks["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained)"
    except Exception:
        return 1590.0, "fallback (1.59 PFLOP/s)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None

    def _run(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def report(self) -> dict:
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def routing_microbench(args, device) -> None:
    """Integer routing work and row movement as HBM GB/s (the routing microbenchmark configuration): continuous_count
    and the stable index construction over int32 ids uniform in [0, E), E in {8, 64, 256},
    N in {2^16, 2^20, 2^24}; gather into expert order and top-8 combine of bf16 rows of width 4096
    at N in {2^16, 2^20} (at 2^24 the expanded buffer alone would be 128 GiB). Algorithmic bytes:
    count 4N + 4E; index build 4N read + 8N written; gather 2*T*H + 4N read + 2*N*H written;
    combine 2*N*H + 6N read + 2*T*H written. L2 is flushed (a 256 MB write) before every timed launch,
    and a short device-side spin lets the host enqueue the launch before the timed region starts, so
    Python dispatch time is not counted as kernel time."""
    import xma
    from xma import ops
    from xma.layers.moe.routing import build_expert_index

    peak = 6554.6
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as fh:
            peak = float(json.load(fh)["hbm_gbs"])
    except Exception:
        pass
    flush = torch.empty(64 << 20, dtype=torch.int32, device=device)

    def timed(fn, reps: int = 10) -> float:
        fn()
        best = []
        for _ in range(reps):
            flush.zero_()
            torch.cuda._sleep(600_000)  # ~0.3 ms of device spin: the host queues the launches meanwhile
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize(device)
            best.append(start.elapsed_time(end))
        return statistics.median(best)

    gen = torch.Generator(device=device).manual_seed(5)
    table = []
    k, H = 8, 4096
    for E in (8, 64, 256):
        for logn in (16, 20, 24):
            n = 1 << logn
            ids = torch.randint(0, E, (n,), device=device, dtype=torch.int32, generator=gen)
            ms = timed(lambda: xma.continuous_count(ids, E))
            table.append({"kernel": "continuous_count", "E": E, "N": n, "ms": round(ms, 4),
                          "GB/s": round((4 * n + 4 * E) / ms / 1e6, 1)})
            sorted_ids = ids.sort().values
            ms = timed(lambda: xma.continuous_count(sorted_ids, E))
            table.append({"kernel": "continuous_count(sorted ids)", "E": E, "N": n, "ms": round(ms, 4),
                          "GB/s": round((4 * n + 4 * E) / ms / 1e6, 1)})
            ms = timed(lambda: build_expert_index(ids, E, top_k=k))
            table.append({"kernel": "moe_index_build", "E": E, "N": n, "ms": round(ms, 4),
                          "GB/s": round(12 * n / ms / 1e6, 1)})
            if logn <= 20:
                T = n // k
                index = build_expert_index(ids, E, top_k=k)
                x = torch.randn(T, H, device=device, generator=gen).to(torch.bfloat16)
                rows = torch.empty(index.cap, H, device=device, dtype=torch.bfloat16)
                ms = timed(lambda: ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, rows, k, index.inv_row))
                table.append({"kernel": "permute_rows", "E": E, "N": n, "ms": round(ms, 4),
                              "GB/s": round((2 * T * H + 4 * n + 2 * n * H) / ms / 1e6, 1)})
                ms = timed(lambda: ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, rows, k))
                table.append({"kernel": "permute_rows(destination-major)", "E": E, "N": n, "ms": round(ms, 4),
                              "GB/s": round((2 * T * H + 4 * n + 2 * n * H) / ms / 1e6, 1)})
                w = torch.rand(T, k, device=device, generator=gen).to(torch.bfloat16)
                y = torch.empty(T, H, device=device, dtype=torch.bfloat16)
                ms = timed(lambda: ops.combine_rows_cuda(rows, index.inv_row, w.view(-1), y, k))
                table.append({"kernel": "combine_rows", "E": E, "N": n, "ms": round(ms, 4),
                              "GB/s": round((2 * n * H + 6 * n + 2 * T * H) / ms / 1e6, 1)})
                del x, rows, w, y, index
    # Router front end (gate GEMM + top-k + softmax in one launch) on the three layer shapes; the
    # library GEMM followed by the stand-alone top-k kernel is timed beside it. Algorithmic bytes:
    # x and the gate weight read once, logits and the three routing outputs written once.
    from xma.layers.moe.routing import router_topk_softmax
    for T, hidden, E, top_k in ((16384, 4096, 8, 2), (8192, 2048, 64, 8), (32768, 7168, 256, 8)):
        x = torch.randn(T, hidden, device=device, generator=gen).to(torch.bfloat16)
        wg = (torch.randn(E, hidden, device=device, generator=gen) * 0.02).to(torch.bfloat16)
        logits = torch.empty(T, E, device=device, dtype=torch.bfloat16)
        wts = torch.empty(T, top_k, device=device, dtype=torch.bfloat16)
        probs = torch.empty(T, top_k, device=device, dtype=torch.float32)
        sel = torch.empty(T, top_k, device=device, dtype=torch.int64)
        nbytes = 2 * T * hidden + 2 * E * hidden + 2 * T * E + T * top_k * 14
        ms = timed(lambda: ops.router_gate_topk_cuda(x, wg, logits, wts, probs, sel, top_k))
        table.append({"kernel": "router_gate_topk", "E": E, "N": T * top_k, "ms": round(ms, 4),
                      "GB/s": round(nbytes / ms / 1e6, 1)})
        ms = timed(lambda: router_topk_softmax(x @ wg.t(), top_k))
        table.append({"kernel": "library GEMM + router_topk_softmax", "E": E, "N": T * top_k, "ms": round(ms, 4),
                      "GB/s": round(nbytes / ms / 1e6, 1)})
        del x, wg, logits, wts, probs, sel
    for row in table:
        row["frac_of_measured_hbm"] = round(row["GB/s"] / peak, 3)
    # CPU baseline: torch's bincount + stable sort on the host for the middle size
    n, E = 1 << 20, 64
    ids = torch.randint(0, E, (n,), dtype=torch.int32)
    t0 = time.perf_counter()
    for _ in range(5):
        ids.long().bincount(minlength=E)
        ids.sort(stable=True)
    cpu_ms = (time.perf_counter() - t0) / 5 * 1e3
    best = max(table, key=lambda r: r["GB/s"])
    print(json.dumps({
        "metric": "routing_hbm_gbs", "unit": "GB/s", "value": best["GB/s"], "n_gpus": 1, "higher_is_better": True,
        "dtype": "int32/bf16", "data": "synthetic", "config": {"workload": "routing microbench (ids uniform in [0,E), seed 5)"},
        "hbm_peak_gbs": peak, "rows": table,
        "cpu_baseline": {"value": round(16 * n / cpu_ms / 1e6, 2), "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "bincount + stable sort of 2^20 int32 ids, E=64 (4N+12N bytes)"},
    }), flush=True)


def make_logits(w: dict, tokens: int, device, generator) -> torch.Tensor | None:
    if w["router"] == "gate":
        return None
    logits = torch.randn(tokens, w["E"], device=device, generator=generator)
    if w["router"] == "zipf":
        # Per-expert bias = log-frequency of a Zipf(s = 1.1) law, ln(rank^-1.1), over a seeded random
        # permutation of the experts. With T = 32768, top-8 of 256 this leaves ~25 experts without a
        # single token and sends ~60 % of the rows to the 8 most popular experts.
        cpu = torch.Generator().manual_seed(w["seed"])
        ranks = torch.randperm(w["E"], generator=cpu).float() + 1.0
        logits = logits + (-1.1 * ranks.log()).to(device)
    return logits


def run_cpu_oracle(w: dict, tokens: int, steps: int, warmup: int, weights=None, experts: int | None = None) -> tuple[float, int]:
    """Times the CPU oracle (float32) on `tokens` tokens of the workload, on the first `experts`
    experts when given. Returns (tokens/s, threads)."""
    from oracle import moe_oracle as O

    g = torch.Generator().manual_seed(w["seed"])
    H, I, k = w["H"], w["I"], w["k"]
    E = experts or w["E"]
    if weights is None:
        w_fc = torch.empty(E, 2 * I, H).normal_(0, 0.02, generator=g)
        w_proj = torch.empty(E, H, I).normal_(0, 0.02, generator=g)
        gate = torch.empty(E, H).normal_(0, 0.02, generator=g)
    else:
        gate, w_fc, w_proj = (t[:E] for t in weights)
    x = torch.randn(tokens, H, generator=g)
    gy = torch.randn(tokens, H, generator=g)
    selected = None
    if w["router"] != "gate":
        logits = make_logits(w, tokens, torch.device("cpu"), g)[:, :E]
        selected = logits.topk(k, -1).indices
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.moe_forward_backward(x, gate, w_fc, w_proj, k, gy, O.swiglu_packed, selected)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    return tokens / (sum(times) / len(times)), torch.get_num_threads()


def reference_arm(args, w: dict, rank: int) -> None:
    if rank != 0:
        return
    tokens = CPU_SAMPLE_TOKENS[args.workload]
    experts = CPU_SAMPLE_EXPERTS.get(args.workload)
    value, cores = run_cpu_oracle(w, tokens, args.steps, args.warmup, experts=experts)
    sample = f"{tokens} tokens of the {args.workload} workload per step, float32, CPU oracle (port of the reference torch path)"
    if experts:
        sample += f", on {experts} of the {w['E']} experts"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tokens / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, w, 1),
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(args, w: dict, world: int) -> dict:
    return {
        "workload": f"{args.workload}: MoE fwd+bwd, T={w['T']} tokens (global), hidden {w['H']}, intermediate {w['I']}, "
                    f"E={w['E']}, top-{w['k']}, swiglu, router={w['router']}, seed {w['seed']}",
        "global_batch_tokens": w["T"], "tokens_per_gpu": w["T"] // world, "experts_per_gpu": w["E"] // world,
        "parallelism": f"ep{world} ({args.ep})" if world > 1 else "single",
        "l2": "inputs larger than L2 (weights + activations per step exceed 126 MB); no flush between steps",
    }


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="mixtral", choices=sorted(WORKLOADS) + ["routing"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"], help="expert-parallel data movement for N > 1")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="N=1: time the step as one CUDA graph replay (the per-kernel table still comes from an eager pass)")
    args = ap.parse_args()
    if args.workload == "routing":
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        torch.cuda.set_device(device)
        routing_microbench(args, device)
        return
    w = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, w, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")

    import xma
    from xma import _native as N
    from xma.layers.moe.routing import router_topk_softmax

    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD

    T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
    tokens_local = T // world
    gen = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + rank)
    torch.manual_seed(w["seed"])
    with torch.device(device):
        moe = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02, expert_parallel_group=group,
                      expert_parallel_mode=args.ep).to(torch.bfloat16)
    with torch.no_grad():
        moe.gate.weight.normal_(0, 0.02)
        if world > 1:  # every rank holds its own block of experts: re-seed per rank
            moe.c_fc.weight.normal_(0, 0.02, generator=gen)
            moe.c_proj.weight.normal_(0, 0.02, generator=gen)
    params = [p for p in moe.parameters()]

    def new_batch():
        x = torch.randn(tokens_local, H, device=device, generator=gen).to(torch.bfloat16)
        gy = torch.randn(tokens_local, H, device=device, generator=gen).to(torch.bfloat16)
        return x, gy, make_logits(w, tokens_local, device, gen)

    def step(x: torch.Tensor, gy: torch.Tensor, logits: torch.Tensor | None):
        for p in params:
            p.grad = None
        x.requires_grad_(True)
        x.grad = None
        if logits is None:
            y, _ = moe(x)
        else:
            logits.requires_grad_(True)
            logits.grad = None
            weights, selected = router_topk_softmax(logits, k)
            y = moe._compute_experts(x, weights.to(x.dtype), selected)
        y.backward(gy)
        return y, x.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def timed(fn, steps: int, sampler=None) -> float:
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx = sampler if sampler is not None else ClockSampler(local_rank)
        with ctx:
            start.record()
            for _ in range(steps):
                fn()
            end.record()
            torch.cuda.synchronize(device)
        barrier()
        ms = torch.tensor([start.elapsed_time(end) / steps], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # ---- device-resident measurement ----
    x, gy, logits = new_batch()
    for _ in range(args.warmup):
        step(x, gy, logits)
    N.check_status(device)
    sampler = ClockSampler(local_rank)
    # Per-launch CUDA events (on the launching stream) are recorded inside the timed region: they give
    # the kernel table, the roofline's launch duration and the launch count of exactly the timed steps.
    N.profiler.start(timing=True)
    ms = timed(lambda: step(x, gy, logits), args.steps, sampler)
    N.profiler.stop()
    N.check_status(device)
    launches = N.profiler.launches
    kernels = N.profiler.summary()
    profiled_ms = eager_ms = ms
    if args.cuda_graph:
        eager_ms = timed(lambda: step(x, gy, logits), args.steps)  # eager without the per-launch events
        if world > 1:
            raise SystemExit("--cuda-graph is a single-GPU option")
        # The step makes no host synchronisation and no launch that depends on device data, so the
        # whole forward + backward records into one graph; replaying it removes the per-launch host
        # cost, which is what bounds the small workloads.
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(3):
                step(x, gy, logits)
        torch.cuda.current_stream(device).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(x, gy, logits)
        for _ in range(3):
            graph.replay()
        ms = timed(graph.replay, args.steps, ClockSampler(local_rank))
        N.check_status(device)
    value = T / (ms / 1e3)

    # ---- end to end: pinned host buffers in, results out, inside the timed region ----
    # Every step copies its inputs from pinned host memory and its results (y and dx) back. Copies
    # run on their own streams with two sets of device input buffers, so the upload of step i+1 and
    # the download of step i overlap the compute of their neighbours, as an input pipeline would.
    hx = x.detach().cpu().pin_memory()
    hgy = gy.cpu().pin_memory()
    hlogits = logits.detach().cpu().pin_memory() if logits is not None else None
    hy = torch.empty_like(hx).pin_memory()
    hdx = torch.empty_like(hx).pin_memory()
    main = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    slots = []
    for _ in range(2):
        slots.append({
            "x": torch.empty_like(x), "gy": torch.empty_like(gy),
            "logits": torch.empty_like(logits) if logits is not None else None,
            "free": None,  # event: the compute that last read this slot has finished
        })
    e2e_state = {"i": 0, "out_done": None}

    def e2e_step():
        slot = slots[e2e_state["i"] % 2]
        e2e_state["i"] += 1
        with torch.cuda.stream(s_in):
            if slot["free"] is not None:
                s_in.wait_event(slot["free"])
            slot["x"].copy_(hx, non_blocking=True)
            if hlogits is not None:
                slot["logits"].copy_(hlogits, non_blocking=True)
            ev_x = s_in.record_event()
            slot["gy"].copy_(hgy, non_blocking=True)
            ev_gy = s_in.record_event()
        main.wait_event(ev_x)
        main.wait_event(ev_gy)
        xin = slot["x"].detach()
        lin = slot["logits"].detach() if slot["logits"] is not None else None
        y, dx = step(xin, slot["gy"], lin)
        ev_done = main.record_event()
        slot["free"] = ev_done
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done)
            hy.copy_(y.detach(), non_blocking=True)
            hdx.copy_(dx, non_blocking=True)
            y.record_stream(s_out)
            dx.record_stream(s_out)
            e2e_state["out_done"] = s_out.record_event()

    def e2e_timed(steps: int) -> float:
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(main)
        for _ in range(steps):
            e2e_step()
        main.wait_event(e2e_state["out_done"])  # the last download is inside the timed region
        end.record(main)
        torch.cuda.synchronize(device)
        barrier()
        t = torch.tensor([start.elapsed_time(end) / steps], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(2):
        e2e_step()
    torch.cuda.synchronize(device)
    e2e_ms = e2e_timed(args.steps)
    h2d = hx.numel() * 2 + hgy.numel() * 2 + (hlogits.numel() * 4 if hlogits is not None else 0)
    d2h = hy.numel() * 2 + hdx.numel() * 2

    if rank == 0:
        peak, peak_src = measured_peaks()
        rows_local = tokens_local * k  # near-uniform load: rows a rank's experts receive ~ rows it sends
        table = {}
        best = None
        for label, (calls, total_ms) in sorted(kernels.items(), key=lambda kv: -kv[1][1]):
            avg = total_ms / calls
            flops = kernel_flops(label, w, rows_local)
            entry = {"launches": calls, "avg_ms": round(avg, 4), "share": round(total_ms / (profiled_ms * args.steps), 4)}
            if flops is not None:
                entry["tflops"] = round(flops / avg / 1e9, 1)
                if best is None:
                    best = (label, flops, avg)
            table[label] = entry
        roofline = None
        if best is not None:
            label, flops, avg = best
            achieved = flops / avg / 1e9
            roofline = {
                "bound": "tensor", "kernel": label, "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                "frac": round(achieved / peak, 4), "frac_of_nominal_2250": round(achieved / 2250.0, 4),
                "peak_source": peak_src,
                "traffic": NCU_TRAFFIC_BYTES.get(args.workload, {}).get(label) if world == 1 else None,
                "flops_per_launch": flops, "avg_launch_ms": round(avg, 4),
            }
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(args, w, world),
            "clocks": sampler.report(),
            "e2e": {"value": T / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "cuda_graph": {"ms_per_step": ms, "eager_ms_per_step": eager_ms} if args.cuda_graph else None,
            "roofline": roofline,
            "step_tflops": round(step_flops(w, T) / ms / 1e9 / world, 1),
            "step_frac_of_peak": round(step_flops(w, T) / ms / 1e9 / world / peak, 4),
            "kernels": table,
        }
        if world == 1 and not args.no_cpu_baseline:
            tokens = CPU_SAMPLE_TOKENS[args.workload]
            experts = CPU_SAMPLE_EXPERTS.get(args.workload)
            ne = experts or E
            weights = (moe.gate.weight.detach()[:ne].float().cpu(), moe.c_fc.weight.detach()[:ne].float().cpu(),
                       moe.c_proj.weight.detach()[:ne].float().cpu())
            cpu_value, cores = run_cpu_oracle(w, tokens, 1, 1, weights, experts)
            line["cpu_baseline"] = {
                "value": cpu_value, "unit": "tokens/s", "cores": cores, "kind": "port",
                "sample": f"{tokens} tokens of the same workload, float32, 1 warm-up + 1 timed fwd+bwd of the CPU oracle"
                          + (f", on {experts} of the {E} experts" if experts else ""),
            }
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
