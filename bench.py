"""MoE layer forward+backward throughput on B200 (tokens/s), one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload mixtral|olmoe|dsv3|cfg1|routing|gemm]
                    [--impl reference] [--ep peer|nccl] [--cuda-graph] [--no-cpu-baseline] [--no-extras]

A step is one forward+backward of the MoE layer on one batch of synthetic tokens. The default
workload is the Mixtral-shape configuration (T=16384, H=4096, I=14336, E=8, top-2, router logits
~N(0,1) injected): it is the configuration the metric's "at 1/2/4/8 B200" clause and the
expert-parallel scaling target are stated on, and it fits one GPU. With N > 1 the experts are
sharded over the ranks (8/N per GPU), the global batch stays fixed (strong scaling, T/N tokens per
rank) and rows travel by the fused peer-memory kernels (`--ep peer`, default) or NCCL all-to-all
(`--ep nccl`). `--cuda-graph` (one GPU) times the step as one CUDA graph replay.

Rank 0 prints one JSON line. `value` is timed with every input resident in HBM, after `preheat_s`
seconds of untimed back-to-back steps so that every N is measured in the same steady power regime;
`e2e` repeats the measurement through the public `MoE` API with pinned-host inputs copied in and
results copied out inside the timed region; `roofline` is the dominant kernel (CUDA events around
each of its launches inside the timed region); `ep_check` compares the last step's outputs, input
gradients, a slice of the weight gradients and the routing integers with a float32 oracle, at every
N; `cpu_baseline` is the reference's own torch path (or, when its copy is absent, the CPU oracle) on a
bounded sample of the same workload. At N = 1 the line also carries `workloads` (the OLMoE-like and
DeepSeek-V3-like layer shapes and the routing microbenchmark) and `reference_triton` (the
reference's Triton kernels on the same GPU, when they run). `--impl reference` times the reference's
CPU path alone.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
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
PREHEAT_S = 2.0
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of each GEMM at N = 1, from a
# one-off profiler capture of this command; not re-measured by the run that prints them.
NCU_TRAFFIC_BYTES = {
    "mixtral": {
        "grouped_wgrad": 6.31e9, "grouped_gemm[NT,swiglu]": 12.50e9, "grouped_gemm[NN,store]": 14.87e9,
        "grouped_gemm[NT,store]": 6.40e9, "grouped_gemm[NN,swiglu_bwd]": 9.99e9,
    },
}
N1_CLOCK_FILE = os.path.join(tempfile.gettempdir(), "xma_b200_bench_n1_clock.json")


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


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


_SAMPLER_CODE = r"""
import sys, time
import pynvml as nv
nv.nvmlInit()
h = nv.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
period = float(sys.argv[2])
print("max", nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM), flush=True)
while True:
    t = time.time()
    try:
        print(t, nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), nv.nvmlDeviceGetCurrentClocksThrottleReasons(h), flush=True)
    except Exception:
        pass
    time.sleep(max(0.0, period - (time.time() - t)))
"""


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) from a process of its own, so the
    sampling does not compete with the launch loop for the interpreter; `window()` selects the samples
    taken between two host time stamps."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, physical_index: int, period_s: float = 0.002) -> None:
        self.path = os.path.join(tempfile.gettempdir(), f"xma_b200_clocks_{os.getpid()}_{physical_index}.txt")
        self.proc = None
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen([sys.executable, "-c", _SAMPLER_CODE, str(physical_index), str(period_s)],
                                         stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def close(self) -> None:
        if self.proc is not None:
            self.proc.terminate()  # this exact child, by its handle
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
            self.proc = None
            self.out.close()

    def window(self, t0: float, t1: float) -> dict:
        samples, mask, max_mhz = [], 0, None
        try:
            with open(self.path) as fh:
                for line in fh:
                    parts = line.split()
                    if parts and parts[0] == "max":
                        max_mhz = int(parts[1])
                    elif len(parts) == 3 and t0 <= float(parts[0]) <= t1:
                        samples.append(int(parts[1]))
                        mask |= int(parts[2])
        except Exception:
            pass
        return {
            "sm_mhz": statistics.median(samples) if samples else None,
            "sm_max_mhz": max_mhz,
            "reasons": sorted(name for bit, name in self.REASONS.items() if mask & bit),
            "samples": len(samples),
        }


def physical_gpu_index(local_rank: int) -> int:
    visible = os.environ.get("CUDA_VISIBLE_DEVICES")
    if visible:
        try:
            return int(visible.split(",")[local_rank])
        except Exception:
            pass
    return local_rank


def routing_microbench(device, log2n: tuple[int, ...] = (16, 18, 20, 24), router: bool = True) -> dict:
    """Integer routing work and row movement as HBM GB/s (the routing microbenchmark configuration):
    continuous_count and the stable index construction over int32 ids uniform in [0, E), E in {8, 64, 256},
    N in {2^16, 2^20, 2^24}; gather into expert order and top-8 combine of bf16 rows of width 4096
    at N in {2^16, 2^20} (at 2^24 the expanded buffer alone would be 128 GiB). Algorithmic bytes:
    count 4N + 4E; index build 4N read + 8N written; gather 2*T*H + 4N read + 2*N*H written;
    combine 2*N*H + 6N read + 2*T*H written. L2 is flushed (a 256 MB write) before every timed launch,
    and a short device-side spin lets the host enqueue the launch before the timed region starts, so
    Python dispatch time is not counted as kernel time."""
    import xma
    from xma import ops
    from xma.layers.moe.routing import build_expert_index, router_topk_softmax

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
        for logn in log2n:
            n = 1 << logn
            ids = torch.randint(0, E, (n,), device=device, dtype=torch.int32, generator=gen)
            if logn != 18:
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
            if logn in (16, 20):
                T = n // k
                index = build_expert_index(ids, E, top_k=k)
                x = torch.randn(T, H, device=device, generator=gen).to(torch.bfloat16)
                rows = torch.empty(index.cap, H, device=device, dtype=torch.bfloat16)
                ms = timed(lambda: ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, rows, k, index.inv_row))
                table.append({"kernel": "permute_rows", "E": E, "N": n, "ms": round(ms, 4),
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
    for T, hidden, E, top_k in ((16384, 4096, 8, 2), (8192, 2048, 64, 8), (32768, 7168, 256, 8)) if router else ():
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
    del flush
    return {
        "hbm_peak_gbs": peak, "rows": table,
        "cpu_baseline": {"value": round(16 * n / cpu_ms / 1e6, 2), "unit": "GB/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": "bincount + stable sort of 2^20 int32 ids, E=64 (4N+12N bytes)"},
    }


def gemm_microbench(device, seconds: float = 1.0) -> dict:
    """The grouped GEMM kernels alone at a mid-size shape (8 experts x 2048 rows, K = 8192, N = 4096: 1 GB on
    the device, small enough for a full profiler capture), each looped for `seconds` so that it is
    measured under the board power limit, with the library's batched GEMM (torch.bmm on the same shapes)
    timed the same way beside it."""
    from xma import _native as N
    from xma import ops
    from xma.layers.moe.routing import build_expert_index

    E, rows, K, Nn = 8, 2048, 8192, 4096
    g = torch.Generator(device=device).manual_seed(9)
    ids = torch.arange(E, device=device).repeat_interleave(rows).view(-1, 1)
    index = build_expert_index(ids, E)
    M = E * rows
    bf = torch.bfloat16
    a = torch.randn(index.cap, K, device=device, generator=g).to(bf)
    w_nt = (torch.randn(E, Nn, K, device=device, generator=g) * 0.02).to(bf)
    w_nn = w_nt.transpose(1, 2).contiguous()
    c = torch.empty(index.cap, Nn, device=device, dtype=bf)
    y = torch.randn(index.cap, Nn, device=device, generator=g).to(bf)
    dw = torch.empty(E, K, Nn, device=device, dtype=bf)
    pre = torch.empty(index.cap, Nn, device=device, dtype=bf)
    act = torch.empty(index.cap, Nn // 2, device=device, dtype=bf)
    a3, c3 = a[:M].view(E, rows, K), torch.empty(E, rows, Nn, device=device, dtype=bf)
    flops = 2.0 * M * K * Nn
    # the swiglu-backward kernel at the Mixtral layer's reduction length (K = H = 4096), I = 4096
    dy = torch.randn(index.cap, 4096, device=device, generator=g).to(bf)
    w_proj = (torch.randn(E, 4096, Nn, device=device, generator=g) * 0.02).to(bf)
    pre2 = torch.randn(index.cap, 2 * Nn, device=device, generator=g).to(bf)
    d_pre2 = torch.empty(index.cap, 2 * Nn, device=device, dtype=bf)
    partials = torch.empty(N.gemm_n_tiles(Nn), index.cap, device=device)
    scale = torch.rand(M, device=device, generator=g).to(bf)
    half_flops = 2.0 * M * 4096 * Nn
    cases = {
        "grouped_gemm[NT,store] (256x512 tile)": lambda: ops.grouped_gemm_cuda(a, w_nt, index.padded_offsets, c, None, None, None, None, N.GEMM_NT, N.EPI_STORE),
        "grouped_gemm[NN,store] (256x512 tile)": lambda: ops.grouped_gemm_cuda(a, w_nn, index.padded_offsets, c, None, None, None, None, N.GEMM_NN, N.EPI_STORE),
        "grouped_gemm[NT,swiglu]": lambda: ops.grouped_gemm_cuda(a, w_nt, index.padded_offsets, pre, act, index.row_src, None, None, N.GEMM_NT, N.EPI_SWIGLU),
        "grouped_wgrad (256x512 tile)": lambda: ops.grouped_wgrad_cuda(a, y, index.padded_offsets, dw),
        "grouped_gemm[NN,swiglu_bwd] K=4096": lambda: ops.grouped_gemm_cuda(dy, w_proj, index.padded_offsets, d_pre2, pre2, index.row_src, scale, partials, N.GEMM_NN, N.EPI_SWIGLU_BWD),
        "torch.bmm NT (library)": lambda: torch.bmm(a3, w_nt.transpose(1, 2), out=c3),
        "torch.bmm NN (library)": lambda: torch.bmm(a3, w_nn, out=c3),
    }
    out = {}
    for name, fn in cases.items():
        for _ in range(3):
            fn()
        torch.cuda.synchronize(device)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize(device)
        reps = max(3, int(seconds * 1e3 / max(start.elapsed_time(end), 1e-3)))
        for _ in range(reps // 2):  # bring the clocks to their steady level first
            fn()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize(device)
        ms = start.elapsed_time(end) / reps
        out[name] = {"ms": round(ms, 4), "tflops": round((half_flops if "K=4096" in name else flops) / ms / 1e9, 1),
                     "launches_timed": reps}
    N.check_status(device)
    return {"shape": {"experts": E, "rows_per_expert": rows, "K": K, "N": Nn}, "kernels": out}


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


def run_cpu_port(w: dict, tokens: int, steps: int, warmup: int, experts: int | None = None) -> tuple[float, int]:
    """Times the CPU oracle (float32, a port of the reference's torch path) on `tokens` tokens of the
    workload, on the first `experts` experts when given. Returns (tokens/s, threads)."""
    from oracle import moe_oracle as O

    torch.set_num_threads(host_threads())
    g = torch.Generator().manual_seed(w["seed"])
    H, I, k = w["H"], w["I"], w["k"]
    E = experts or w["E"]
    w_fc = torch.empty(E, 2 * I, H).normal_(0, 0.02, generator=g)
    w_proj = torch.empty(E, H, I).normal_(0, 0.02, generator=g)
    gate = torch.empty(E, H).normal_(0, 0.02, generator=g)
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


def run_reference_subprocess(w: dict, tokens: int, steps: int, warmup: int, experts: int | None, backend: str, device: str,
                             dtype: str, timeout_s: float) -> dict:
    """The unmodified reference (oracle/_ref) in a process of its own; returns its JSON line as a dict."""
    runner = os.path.join(_ROOT, "oracle", "ref_runner.py")
    cmd = [sys.executable, runner, "--spec", json.dumps(w), "--tokens", str(tokens), "--steps", str(steps), "--warmup",
           str(warmup), "--backend", backend, "--device", device, "--dtype", dtype, "--threads", str(host_threads())]
    if experts:
        cmd += ["--experts", str(experts)]
    env = dict(os.environ)
    for name in ("OMP_NUM_THREADS", "MKL_NUM_THREADS"):  # a launcher's one-thread default must not reach the CPU arm
        env.pop(name, None)
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(name, None)
    try:
        done = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=env)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no result within {timeout_s:.0f} s"}
    for line in reversed(done.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except Exception:
                break
    tail = (done.stderr or done.stdout or "").strip().splitlines()[-1:] or ["no output"]
    return {"unavailable": f"exit code {done.returncode}: {tail[0][:300]}"}


def cpu_reference(w: dict, workload: str, steps: int, warmup: int) -> dict:
    """The reference's own CPU implementation of the path on the host cores (its torch path from
    oracle/_ref); the CPU oracle, a port of it, when the copy is absent or does not run."""
    tokens = CPU_SAMPLE_TOKENS[workload]
    experts = CPU_SAMPLE_EXPERTS.get(workload)
    sample = f"{tokens} tokens of the {workload} workload per step, float32"
    if experts:
        sample += f", on {experts} of the {w['E']} experts"
    got = run_reference_subprocess(w, tokens, steps, warmup, experts, "torch", "cpu", "float32", 1500.0)
    if "tokens_per_s" in got:
        return {"value": got["tokens_per_s"], "unit": "tokens/s", "cores": got["threads"], "kind": "reference",
                "sample": sample + ", the reference's torch path (kernel_backend=torch) from its unmodified sources"}
    value, cores = run_cpu_port(w, tokens, steps, warmup, experts)
    return {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": sample + f", CPU oracle (port of the reference torch path; the reference itself: {got.get('unavailable')})"}


def reference_arm(args, w: dict, rank: int) -> None:
    if rank != 0:
        return
    base = cpu_reference(w, args.workload, args.steps, args.warmup)
    tokens = CPU_SAMPLE_TOKENS[args.workload]
    value = base["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * tokens / value, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w, 1, args.ep),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name: str, w: dict, world: int, ep: str) -> dict:
    return {
        "workload": f"{name}: MoE fwd+bwd, T={w['T']} tokens (global), hidden {w['H']}, intermediate {w['I']}, "
                    f"E={w['E']}, top-{w['k']}, swiglu, router={w['router']}, seed {w['seed']}",
        "global_batch_tokens": w["T"], "tokens_per_gpu": w["T"] // world, "experts_per_gpu": w["E"] // world,
        "parallelism": f"ep{world} ({ep})" if world > 1 else "single",
        "l2": "inputs larger than L2 (weights + activations per step exceed 126 MB); no flush between steps",
    }


class Bench:
    """One workload on this rank: the layer, a batch, the step, and the measurements on it."""

    def __init__(self, name: str, ep: str, world: int, rank: int, device, group, sampler: ClockSampler | None) -> None:
        import xma

        self.name, self.w, self.world, self.rank, self.device, self.group = name, WORKLOADS[name], world, rank, device, group
        self.sampler = sampler
        w = self.w
        T, H, I, E, k = w["T"], w["H"], w["I"], w["E"], w["k"]
        self.tokens_local = T // world
        self.gen = torch.Generator(device=device).manual_seed(w["seed"] * 1000 + rank)
        torch.manual_seed(w["seed"])
        # Parameters are created in bf16 on the device (the DeepSeek-V3 shape holds 21 GiB of them).
        with torch.device(device):
            prev = torch.get_default_dtype()
            torch.set_default_dtype(torch.bfloat16)
            try:
                self.moe = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02, expert_parallel_group=group,
                                   expert_parallel_mode=ep)
            finally:
                torch.set_default_dtype(prev)
        with torch.no_grad():
            self.moe.gate.weight.normal_(0, 0.02)
            if world > 1:  # every rank holds its own block of experts: re-seed per rank
                self.moe.c_fc.weight.normal_(0, 0.02, generator=self.gen)
                self.moe.c_proj.weight.normal_(0, 0.02, generator=self.gen)
        self.params = list(self.moe.parameters())
        self.x = torch.randn(self.tokens_local, H, device=device, generator=self.gen).to(torch.bfloat16)
        self.gy = torch.randn(self.tokens_local, H, device=device, generator=self.gen).to(torch.bfloat16)
        self.logits = make_logits(w, self.tokens_local, device, self.gen)

    def step(self, x: torch.Tensor, gy: torch.Tensor, logits: torch.Tensor | None):
        from xma.layers.moe.routing import router_topk_softmax

        for p in self.params:
            p.grad = None
        x.requires_grad_(True)
        x.grad = None
        if logits is None:
            y, _ = self.moe(x)
        else:
            logits.requires_grad_(True)
            logits.grad = None
            weights, selected = router_topk_softmax(logits, self.w["k"])
            y = self.moe._compute_experts(x, weights.to(x.dtype), selected)
        y.backward(gy)
        return y, x.grad

    def barrier(self) -> None:
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize(self.device)

    def max_over_ranks(self, value: float) -> float:
        t = torch.tensor([value], device=self.device)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps: int) -> tuple[float, dict]:
        """EXACTLY `steps` calls between two events, barrier + synchronize on both sides, max over ranks."""
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.time()
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        # How long the host took to queue a step (below the device time: the device is the slower side).
        self.host_ms_per_step = (time.time() - t0) * 1e3 / steps
        torch.cuda.synchronize(self.device)
        t1 = time.time()
        self.barrier()
        ms = self.max_over_ranks(start.elapsed_time(end) / steps)
        clocks = self.sampler.window(t0, t1) if self.sampler is not None else {}
        return ms, clocks

    def preheat(self, fn, seconds: float, est_ms: float) -> int:
        """Untimed back-to-back steps for about `seconds` (the same count on every rank)."""
        n = max(1, int(math.ceil(seconds * 1e3 / max(est_ms, 1e-3))))
        for _ in range(n):
            fn()
        return n

    def measure(self, steps: int, warmup: int, preheat_s: float, cuda_graph: bool = False) -> dict:
        from xma import _native as N

        x, gy, logits = self.x, self.gy, self.logits
        run = lambda: self.step(x, gy, logits)
        for _ in range(warmup):
            run()
        N.check_status(self.device)
        est_ms, _ = self.timed(run, 2)
        pre_steps = self.preheat(run, preheat_s, est_ms)
        # The headline time is taken without any instrumentation; a second pass of the same K steps with
        # CUDA events around every launch gives the kernel table and the launch count.
        ms, clocks = self.timed(run, steps)
        host_ms = self.max_over_ranks(self.host_ms_per_step)
        N.profiler.start(timing=True)
        profiled_ms, _ = self.timed(run, steps)
        N.profiler.stop()
        N.check_status(self.device)
        out = {"ms": ms, "profiled_ms": profiled_ms, "clocks": clocks, "launches": N.profiler.launches,
               "kernels": N.profiler.summary(), "preheat_steps": pre_steps, "eager_ms": ms, "graph": False,
               "host_queue_ms_per_step": round(host_ms, 3)}
        if cuda_graph:
            if self.world > 1:
                raise SystemExit("--cuda-graph is a single-GPU option")
            # The step makes no host synchronisation and no launch whose arguments depend on device data, so
            # the whole forward + backward records into one graph; replaying it removes the per-launch host
            # cost, which is what bounds the small workloads.
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(3):
                    run()
            torch.cuda.current_stream(self.device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                run()
            for _ in range(3):
                graph.replay()
            out["ms"], out["clocks"] = self.timed(graph.replay, steps)
            out["graph"] = True
            N.check_status(self.device)
        return out

    def measure_e2e(self, steps: int, upload_inputs: bool = True, download_results: bool = True, depth: int = 2,
                    link: bool = True) -> dict:
        """Every step copies its inputs from pinned host memory and its results (y and dx) back, inside the
        timed region. Copies run on their own streams with `depth` sets of device input buffers, and the
        upload of step i+depth-1 is queued BEFORE the kernels of step i, so it overlaps them even when the
        host is the slower side (short steps at N = 8), as an input pipeline with prefetch would. The two
        switches leave one direction out: they exist for `--e2e-breakdown`, which tells the directions'
        costs apart; the `e2e` figure of the bench line always has both."""
        x, gy, logits, device = self.x, self.gy, self.logits, self.device
        hx = x.detach().cpu().pin_memory()
        hgy = gy.cpu().pin_memory()
        hlogits = logits.detach().cpu().pin_memory() if logits is not None else None
        hy = torch.empty_like(hx).pin_memory()
        hdx = torch.empty_like(hx).pin_memory()
        main = torch.cuda.current_stream(device)
        s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        slots = [{"x": torch.empty_like(x), "gy": torch.empty_like(gy),
                  "logits": torch.empty_like(logits) if logits is not None else None,
                  "free": None, "ready": None} for _ in range(depth)]
        state = {"i": 0, "out_done": None}

        def upload(slot: dict, always: bool = False) -> None:
            if not (upload_inputs or always):
                return
            with torch.cuda.stream(s_in):
                if slot["free"] is not None:
                    s_in.wait_event(slot["free"])  # the compute that last read this slot has finished
                slot["x"].copy_(hx, non_blocking=True)
                if hlogits is not None:
                    slot["logits"].copy_(hlogits, non_blocking=True)
                slot["gy"].copy_(hgy, non_blocking=True)
                slot["ready"] = s_in.record_event()

        def e2e_step() -> None:
            slot = slots[state["i"] % depth]
            upload(slots[(state["i"] + depth - 1) % depth])  # a later step's inputs, queued ahead of this step's kernels
            state["i"] += 1
            if upload_inputs:
                main.wait_event(slot["ready"])
            xin = slot["x"].detach()
            lin = slot["logits"].detach() if slot["logits"] is not None else None
            y, dx = self.step(xin, slot["gy"], lin)
            slot["free"] = main.record_event()
            if not download_results:
                return
            with torch.cuda.stream(s_out):
                s_out.wait_event(slot["free"])
                hy.copy_(y.detach(), non_blocking=True)
                hdx.copy_(dx, non_blocking=True)
                y.record_stream(s_out)
                dx.record_stream(s_out)
                state["out_done"] = s_out.record_event()

        for slot in slots[:depth - 1]:
            upload(slot, always=True)
        if not upload_inputs:
            upload(slots[depth - 1], always=True)  # every slot holds the inputs; nothing is uploaded from here on
        for _ in range(depth):
            e2e_step()
        torch.cuda.synchronize(device)
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(main)
        t0 = time.time()
        for _ in range(steps):
            e2e_step()
        host_ms = (time.time() - t0) * 1e3 / steps
        if state["out_done"] is not None:
            main.wait_event(state["out_done"])  # the last download is inside the timed region
        end.record(main)
        torch.cuda.synchronize(device)
        self.barrier()
        ms = self.max_over_ranks(start.elapsed_time(end) / steps)
        host_ms = self.max_over_ranks(host_ms)
        h2d = hx.numel() * 2 + hgy.numel() * 2 + (hlogits.numel() * 4 if hlogits is not None else 0)
        d2h = hy.numel() * 2 + hdx.numel() * 2
        link = self.host_link(hx, hy, slots[0]["x"], s_in, s_out, h2d, d2h) if link else None
        return {"value": self.w["T"] / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "host_queue_ms_per_step": round(host_ms, 3), "host_link": link}

    def host_link(self, hx, hy, dx, s_in, s_out, h2d_bytes: int, d2h_bytes: int) -> dict:
        """What the box's host links give when every rank copies at once, both directions together, with
        nothing else running: the floor they set for an end-to-end step (all ranks' bytes over the summed
        rates). Outside every timed region."""
        reps = max(2, int(math.ceil((1 << 28) / (hx.numel() * 2))))
        torch.cuda.synchronize(self.device)
        self.barrier()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        marks[0].record(s_in)
        marks[2].record(s_out)
        for _ in range(reps):
            with torch.cuda.stream(s_in):
                dx.copy_(hx, non_blocking=True)
            with torch.cuda.stream(s_out):
                hy.copy_(dx, non_blocking=True)  # the values are irrelevant here
        marks[1].record(s_in)
        marks[3].record(s_out)
        torch.cuda.synchronize(self.device)
        self.barrier()
        moved = reps * hx.numel() * 2
        rates = torch.tensor([moved / marks[0].elapsed_time(marks[1]) / 1e6, moved / marks[2].elapsed_time(marks[3]) / 1e6],
                             device=self.device)
        if self.world > 1:
            dist.all_reduce(rates, op=dist.ReduceOp.SUM)
        up, down = float(rates[0].item()), float(rates[1].item())
        return {"h2d_gbs_all_ranks": round(up, 1), "d2h_gbs_all_ranks": round(down, 1),
                "floor_ms_per_step": round(max(h2d_bytes * self.world / up, d2h_bytes * self.world / down) / 1e6, 3)}

    # ------------------------------------------------------------------------------------------
    # Correctness of the measured configuration, outside every timed region
    # ------------------------------------------------------------------------------------------
    def _gather(self, t: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return t
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts, dim=0)

    def ep_check(self) -> dict:
        """One more (untimed) step, then: `tokens` sampled local tokens against the float32 oracle (the
        reference's torch path restated) with the expert weights gathered from their owners; 256 x 256
        corner slices of both weight gradients of this rank's first expert against float32 X_e^T Y_e
        over that expert's rows gathered from every rank; the routing integers against torch's stable
        sort. Errors are max |got - ref| / max |ref|; every figure is the worst over the ranks."""
        import torch.nn.functional as F

        from oracle import moe_oracle as O
        from xma.layers.moe.routing import build_expert_index, router_topk_softmax

        w, dev, world, rank = self.w, self.device, self.world, self.rank
        H, I, E, k = w["H"], w["I"], w["E"], w["k"]
        epr = E // world
        rel = lambda a, b: float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-30))

        x = self.x.detach().clone()
        y, dx = self.step(x, self.gy, self.logits)
        y, dx = y.detach(), dx.detach()
        dw_fc, dw_proj = self.moe.c_fc.weight.grad, self.moe.c_proj.weight.grad
        gate = self.moe.gate.weight.detach()
        with torch.no_grad():
            if self.logits is not None:
                weights, selected = router_topk_softmax(self.logits.detach(), k)
            else:  # the layer's own router, so that the selection is the one the step used
                _, weights, selected = self.moe._compute_routing_weights(self.x.detach())
            weights = weights.to(torch.bfloat16)

        # ---- sampled tokens against the oracle ----
        n_s = 48 if E <= 64 else 8
        pick = torch.randperm(self.tokens_local, generator=torch.Generator().manual_seed(17 + rank))[:n_s].to(dev)
        w_fc_all = self._gather(self.moe.c_fc.weight.detach())
        w_proj_all = self._gather(self.moe.c_proj.weight.detach())
        used = selected[pick].unique()
        remap = torch.full((E,), -1, dtype=torch.long, device=dev)
        remap[used] = torch.arange(used.numel(), device=dev)
        xs = self.x.detach()[pick].float().requires_grad_(True)
        if self.logits is None:
            picked = F.linear(xs, gate.float()).gather(1, selected[pick])
            wts = torch.softmax(picked, dim=-1)  # the router path carries gradient into dx, as in the layer
        else:
            wts = weights[pick].float()
        ref = O.compute_experts(xs, wts, remap[selected[pick]], w_fc_all[used].float(), w_proj_all[used].float())
        ref.backward(self.gy[pick].float())
        err_y, err_dx = rel(y[pick], ref.detach()), rel(dx[pick], xs.grad)
        del w_fc_all, w_proj_all, ref

        # ---- weight-gradient slices of this rank's first expert ----
        x_all, gy_all = self._gather(self.x.detach()), self._gather(self.gy)
        sel_all, wts_all = self._gather(selected), self._gather(weights)
        counts_all = torch.bincount(sel_all.flatten(), minlength=E)
        local = counts_all[rank * epr:(rank + 1) * epr]
        el = int(local.argmax())
        e = rank * epr + el
        tok, slot = torch.nonzero(sel_all == e, as_tuple=True)
        err_dw = 0.0
        if tok.numel() > 0:
            xe, ge = x_all[tok].float(), gy_all[tok].float()
            pe = wts_all[tok, slot].float().unsqueeze(1)
            w1, w2 = self.moe.c_fc.weight.detach()[el].float(), self.moe.c_proj.weight.detach()[el].float()
            for c0 in (0, I - 256) if I >= 256 else (0,):
                cw = min(256, I)
                pre_u = (xe @ w1[c0:c0 + cw].t()).to(torch.bfloat16).float()
                pre_g = (xe @ w1[I + c0:I + c0 + cw].t()).to(torch.bfloat16).float()
                sig = torch.sigmoid(pre_g)
                h = pre_u * pre_g * sig
                dh = ((ge * pe) @ w2[:, c0:c0 + cw])
                du, dg = dh * pre_g * sig, dh * pre_u * (sig + pre_g * sig * (1 - sig))
                r0 = 0 if c0 == 0 else H - min(256, H)
                rw = min(256, H)
                err_dw = max(err_dw, rel(dw_proj[el, r0:r0 + rw, c0:c0 + cw], (ge[:, r0:r0 + rw] * pe).t() @ h))
                err_dw = max(err_dw, rel(dw_fc[el, c0:c0 + cw, r0:r0 + rw], du.t() @ xe[:, r0:r0 + rw]))
                err_dw = max(err_dw, rel(dw_fc[el, I + c0:I + c0 + cw, r0:r0 + rw], dg.t() @ xe[:, r0:r0 + rw]))
        del x_all, gy_all

        # ---- routing integers ----
        flat = selected.flatten()
        order = flat.sort(stable=True)
        routing_exact = True
        home = build_expert_index(selected, E, block_m=1)
        routing_exact &= torch.equal(home.sorted_expert_idxs.long(), order.values)
        routing_exact &= torch.equal(home.sorted_scattered_idxs.long(), order.indices)
        routing_exact &= torch.equal(home.expert_frequency.long(), torch.bincount(flat, minlength=E))
        state = getattr(self.moe, "_peer_state", None)
        if world > 1 and state is not None and getattr(state, "last_routing", None) is not None:
            dest_rank, dest_row, lpo = state.last_routing
            counts = torch.stack([torch.bincount(s.flatten(), minlength=E) for s in sel_all.view(world, -1, k)])  # [world, E]
            padded = (counts.sum(0) + 127) // 128 * 128
            off = torch.zeros(E, dtype=torch.long, device=dev)
            for d in range(world):
                blk = padded[d * epr:(d + 1) * epr]
                off[d * epr:(d + 1) * epr] = blk.cumsum(0) - blk
            base = off + counts[:rank].sum(0)
            first = torch.bincount(flat, minlength=E).cumsum(0) - torch.bincount(flat, minlength=E)
            inv = torch.empty_like(order.indices)
            inv[order.indices] = torch.arange(flat.numel(), device=dev)
            want_row = base[flat] + (inv - first[flat])
            routing_exact &= torch.equal(dest_row.long(), want_row)
            routing_exact &= torch.equal(dest_rank.long(), flat // epr)
            mine = padded[rank * epr:(rank + 1) * epr]
            routing_exact &= torch.equal(lpo.long(), torch.cat([mine.new_zeros(1), mine.cumsum(0)]))
        worst = torch.tensor([err_y, err_dx, err_dw, 0.0 if routing_exact else 1.0], device=dev)
        if world > 1:
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return {"y": round(float(worst[0]), 6), "dx": round(float(worst[1]), 6), "dw_slice": round(float(worst[2]), 6),
                "routing_exact": bool(worst[3] == 0), "n_ranks": world, "tokens_per_rank": n_s,
                "tolerance": 2e-2}

    def report(self, m: dict, peak: float, peak_src: str) -> dict:
        """The per-workload part of the JSON line (rank 0)."""
        w, world = self.w, self.world
        rows_local = self.tokens_local * w["k"]  # near-uniform load: rows a rank's experts receive ~ rows it sends
        steps_ms = m["profiled_ms"]
        table, best, in_kernels = {}, None, 0.0
        calls_per_step = None
        for label, (calls, total_ms) in sorted(m["kernels"].items(), key=lambda kv: -kv[1][1]):
            avg = total_ms / calls
            flops = kernel_flops(label, w, rows_local)
            entry = {"launches": calls, "avg_ms": round(avg, 4), "share": round(total_ms / (steps_ms * m["steps"]), 4)}
            in_kernels += total_ms
            if flops is not None:
                entry["tflops"] = round(flops / avg / 1e9, 1)
                if best is None:
                    best = (label, flops, avg)
            table[label] = entry
        roofline = None
        if best is not None:
            label, flops, avg = best
            achieved = flops / avg / 1e9
            traffic = NCU_TRAFFIC_BYTES.get(self.name, {}).get(label) if world == 1 else None
            roofline = {
                "bound": "tensor", "kernel": label, "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
                "frac": round(achieved / peak, 4), "frac_of_nominal_2250": round(achieved / 2250.0, 4),
                "peak_source": peak_src, "traffic": traffic,
                "traffic_source": "constant from a one-off capture" if traffic is not None else None,
                "flops_per_launch": flops, "avg_launch_ms": round(avg, 4),
            }
        ms = m["ms"]
        return {
            "ms_per_step": ms, "tokens_per_s": w["T"] / (ms / 1e3), "clocks": m["clocks"], "preheat_s": m["preheat_s"],
            "preheat_steps": m["preheat_steps"], "gpu_launches": m["launches"], "roofline": roofline,
            "step_tflops": round(step_flops(w, w["T"]) / ms / 1e9 / world, 1),
            "step_frac_of_peak": round(step_flops(w, w["T"]) / ms / 1e9 / world / peak, 4),
            "kernel_share": round(in_kernels / (steps_ms * m["steps"]), 4),
            "kernels": table,
        }


def ep_overheads(table: dict, steps: int, ms: float) -> dict:
    """Where an expert-parallel step's time goes besides the GEMMs (CUDA events around every launch of
    this library inside the timed region; a barrier's time includes waiting for the slowest rank)."""
    def per_step(*labels):
        return round(sum(table[l]["avg_ms"] * table[l]["launches"] for l in labels if l in table) / steps, 4)

    gemm = per_step("grouped_wgrad", "grouped_gemm[NT,swiglu]", "grouped_gemm[NT,store]", "grouped_gemm[NN,swiglu_bwd]",
                    "grouped_gemm[NN,store]")
    sync = per_step("ep_barrier", "ep_exchange_counts")
    rows = per_step("ep_dispatch_rows", "ep_combine_pull", "ep_prepare_rows", "ep_pull_scalars", "permute_rows")
    # Launches the layer puts on its second stream, beside work of the first (the backward pass's last
    # meeting and its pulls under the weight-gradient GEMMs, the copy of the received rows under the first
    # GEMM, the zeroing of padding rows under the dispatch): no time of their own unless they outlast it.
    hidden = per_step(*(l for l in table if l.startswith("overlapped_")))
    other = round(sum(v["avg_ms"] * v["launches"] for v in table.values()) / steps - gemm - sync - rows - hidden, 4)
    return {"gemm_ms": gemm, "barrier_and_count_exchange_ms": sync, "row_movement_ms": rows, "other_kernels_ms": other,
            "second_stream_ms": hidden,
            "outside_kernels_ms": round(ms - gemm - sync - rows - other, 4),
            "launches_per_step": round(sum(v["launches"] for v in table.values()) / steps, 1)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="mixtral", choices=sorted(WORKLOADS) + ["routing", "gemm"])
    ap.add_argument("--seconds", type=float, default=1.0, help="--workload gemm: how long every kernel is looped")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="N=1: skip the other layer shapes, the routing microbenchmark and the reference's Triton arm")
    ap.add_argument("--routing-log2n", default="16,18,20,24",
                    help="--workload routing: id counts as powers of two (a short list keeps a profiler capture small)")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"], help="expert-parallel data movement for N > 1")
    ap.add_argument("--e2e-breakdown", action="store_true",
                    help="also time the end-to-end loop without uploads, without downloads, without both, and with deeper prefetch")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="N=1: time the step as one CUDA graph replay (the per-kernel table still comes from an eager pass)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "routing":
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        sizes = tuple(int(v) for v in args.routing_log2n.split(","))
        result = routing_microbench(device, sizes, router=sizes == (16, 18, 20, 24))
        best = max(result["rows"], key=lambda r: r["GB/s"])
        print(json.dumps({
            "metric": "routing_hbm_gbs", "unit": "GB/s", "value": best["GB/s"], "n_gpus": 1, "higher_is_better": True,
            "dtype": "int32/bf16", "data": "synthetic",
            "config": {"workload": "routing microbench (ids uniform in [0,E), seed 5)"}, **result,
        }), flush=True)
        return
    if args.workload == "gemm":
        device = torch.device("cuda", local_rank)
        torch.cuda.set_device(device)
        result = gemm_microbench(device, args.seconds)
        best = max(v["tflops"] for k, v in result["kernels"].items() if k.startswith("grouped"))
        print(json.dumps({"metric": "grouped_gemm_tflops", "unit": "TFLOP/s", "value": best, "n_gpus": 1,
                          "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
                          "config": {"workload": "grouped GEMM kernels alone, 8 experts x 2048 rows, K=8192, N=4096"}, **result}),
              flush=True)
        return
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        reference_arm(args, w, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1")

    from xma import _native as N  # fails loudly when the CUDA library is missing: there is no other path

    N.lib()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        group = dist.group.WORLD
    sampler = ClockSampler(physical_gpu_index(local_rank))  # every rank samples its own GPU
    peak, peak_src = measured_peaks()

    bench = Bench(args.workload, args.ep, world, rank, device, group, sampler)
    m = bench.measure(args.steps, args.warmup, PREHEAT_S, args.cuda_graph)
    m["steps"], m["preheat_s"] = args.steps, PREHEAT_S
    e2e = bench.measure_e2e(args.steps)
    if args.e2e_breakdown:
        # The same loop with one or both directions of the host copies left out, and with one more batch
        # of prefetch: ms per step each (every rank runs every variant; they contain meetings).
        variants = (("no_copies", dict(upload_inputs=False, download_results=False)),
                    ("upload_only", dict(download_results=False)), ("download_only", dict(upload_inputs=False)),
                    ("both_prefetch_2", dict(depth=3)))
        e2e["breakdown_ms"] = {name: round(bench.measure_e2e(args.steps, link=False, **kw)["ms_per_step"], 4)
                               for name, kw in variants}
    check = bench.ep_check()
    # Median SM clock of every rank's GPU inside the timed region. A rank that waits at the meetings for a
    # slower GPU draws less power and clocks higher, so rank 0's clock alone says little at N > 1.
    mine = torch.tensor([float(m["clocks"].get("sm_mhz") or 0.0)], device=device)
    by_rank = [mine.clone() for _ in range(world)]
    if world > 1:
        dist.all_gather(by_rank, mine)
    mhz_by_rank = [float(t.item()) for t in by_rank]

    line = None
    if rank == 0:
        rep = bench.report(m, peak, peak_src)
        seen = [v for v in mhz_by_rank if v > 0]
        mhz = sum(seen) / len(seen) if seen else None   # mean over the ranks of their median clocks
        rep["clocks"]["sm_mhz_by_rank"] = mhz_by_rank
        reference_mhz = None
        if world == 1 and mhz:
            try:
                with open(N1_CLOCK_FILE, "w") as fh:
                    json.dump({"sm_mhz": mhz, "workload": args.workload}, fh)
            except Exception:
                pass
            reference_mhz = mhz
        elif mhz:
            try:
                with open(N1_CLOCK_FILE) as fh:
                    rec = json.load(fh)
                if rec.get("workload") == args.workload:
                    reference_mhz = rec["sm_mhz"]
            except Exception:
                pass
        value = rep["tokens_per_s"]
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": rep["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(args.workload, w, world, args.ep),
            "clocks": rep["clocks"], "preheat_s": PREHEAT_S, "preheat_steps": rep["preheat_steps"],
            # tokens/s scaled to the SM clock the N=1 run of the same workload saw on this box (the file the
            # N=1 run leaves in the temporary directory), with this run's clock taken as the mean over the
            # ranks of their median clocks; null when no such run came before
            "value_clock_normalised": round(value * reference_mhz / mhz, 1) if (mhz and reference_mhz) else None,
            "clock_reference_mhz": reference_mhz,
            "e2e": e2e, "gpu_launches": rep["gpu_launches"],
            # the slowest rank's host time to queue one step (it runs ahead of the device while it is below ms_per_step)
            "host_queue_ms_per_step": m["host_queue_ms_per_step"],
            "cuda_graph": {"ms_per_step": m["ms"], "eager_ms_per_step": m["eager_ms"]} if args.cuda_graph else None,
            "roofline": rep["roofline"], "step_tflops": rep["step_tflops"], "step_frac_of_peak": rep["step_frac_of_peak"],
            "kernel_share": rep["kernel_share"], "ep_check": check, "kernels": rep["kernels"],
        }
        if world > 1:
            line["ep_overheads"] = ep_overheads(rep["kernels"], args.steps, m["profiled_ms"])

    # ---- N = 1 extras: the other configurations, in the same steady regime, after the headline ----
    if world == 1:
        del bench
        torch.cuda.empty_cache()
        if not args.no_extras:
            extras = {}
            for name in ("olmoe", "dsv3"):
                if name == args.workload:
                    continue
                try:
                    other = Bench(name, args.ep, 1, 0, device, None, sampler)
                    om = other.measure(min(args.steps, 10), 3, 1.0)
                    om["steps"], om["preheat_s"] = min(args.steps, 10), 1.0
                    rep = other.report(om, peak, peak_src)
                    rep["config"] = workload_config(name, WORKLOADS[name], 1, args.ep)["workload"]
                    rep["step_frac_of_sustained_peak"] = rep.pop("step_frac_of_peak")
                    extras[name] = rep
                    del other
                except Exception as error:  # e.g. not enough free memory for the 21 GiB shape
                    extras[name] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}
                torch.cuda.empty_cache()
            try:
                extras["routing"] = routing_microbench(device)["rows"]
            except Exception as error:
                extras["routing"] = {"unavailable": f"{type(error).__name__}: {str(error)[:200]}"}
            torch.cuda.empty_cache()
            line["workloads"] = extras
            # The reference's own GPU path (its Triton kernels, kernel_backend=triton) on this GPU, same
            # workload, bf16, in a process of its own; never this library's kernels.
            got = run_reference_subprocess(w, w["T"], 3, 2, None, "triton", "cuda", "bfloat16", 600.0)
            if "tokens_per_s" in got:
                line["reference_triton"] = {"value": got["tokens_per_s"], "unit": "tokens/s", "ms_per_step": got["ms_per_step"],
                                            "sample": "the reference's MoE with kernel_backend=triton, bf16, same workload, 2 warm-up + 3 timed steps"}
            else:
                line["reference_triton"] = "unavailable: " + str(got.get("unavailable"))
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_reference(w, args.workload, 1, 1)
    if sampler is not None:
        sampler.close()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        state = getattr(bench.moe, "_peer_state", None)
        if state is not None:
            state.release()  # unmap the peers' buffers before any rank's process goes away
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
