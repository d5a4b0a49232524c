"""Times the REFERENCE's own MoE layer (the unmodified copy under oracle/_ref) in a process of its
own. TEST / MEASUREMENT INFRASTRUCTURE ONLY: `bench.py` runs this file as a subprocess for its
`--impl reference` arm, its `cpu_baseline` key and its `reference_triton` key. Nothing of this
repository's package is imported here (both packages are called `xma` and both register `xma::` ops,
so they cannot share a process).

    python oracle/ref_runner.py --spec '{"T":..,"H":..,"I":..,"E":..,"k":..,"seed":..,"router":..}'
        --tokens N [--experts M] --backend torch|triton --device cpu|cuda --steps K --warmup W [--threads C]

Prints one JSON line: {"tokens_per_s", "ms_per_step", "threads", "backend", "device", "tokens"} or
{"unavailable": "<reason>"}.

The reference is driven exactly as its own test drives it (tests/layers/moe_test.py:92-121): the
`MoE` module with `swiglu_packed` as activation, `kernel_backend` passed to the call. One rebinding,
no edit: `xma.layers.moe.continuous_count` is bound to the torch backend, because
xma/layers/moe/__init__.py:219 does not forward `kernel_backend` and the default would JIT-build the
CUDA extension, whose CUTLASS headers are not part of the checkout (.gitmodules:1-3).
"""

from __future__ import annotations

import argparse
import functools
import json
import os
import sys
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--spec", required=True)
    ap.add_argument("--tokens", type=int, required=True)
    ap.add_argument("--experts", type=int, default=0)
    ap.add_argument("--backend", default="torch", choices=["torch", "triton"])
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--dtype", default="float32", choices=["float32", "bfloat16"])
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--threads", type=int, default=0)
    args = ap.parse_args()

    here = os.path.dirname(os.path.abspath(__file__))
    ref_dir = os.path.join(here, "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "xma")):
        print(json.dumps({"unavailable": "oracle/_ref/xma is missing (run oracle/make_ref.py where the reference checkout is)"}))
        return
    # Only the reference's package may be importable as `xma` in this process.
    sys.path[:] = [ref_dir] + [p for p in sys.path if "flash-model-architectures_b200" not in p]
    try:
        import torch

        if args.threads > 0:
            torch.set_num_threads(args.threads)
        import xma  # the reference
        import xma.layers.moe as ref_moe
        from xma import KernelBackend

        ref_moe.continuous_count = functools.partial(xma.continuous_count, kernel_backend=KernelBackend.torch)
        spec = json.loads(args.spec)
        H, I, k = spec["H"], spec["I"], spec["k"]
        E = args.experts or spec["E"]
        tokens = args.tokens
        dtype = getattr(torch, args.dtype)
        device = torch.device(args.device)
        backend = KernelBackend.torch if args.backend == "torch" else KernelBackend.triton
        act = lambda t: xma.swiglu_packed(t, kernel_backend=backend)

        g = torch.Generator().manual_seed(spec["seed"])
        with torch.device(device):
            moe = xma.MoE(num_experts=E, num_experts_per_tok=k, hidden_size=H, intermediate_size=I,
                          activation_function=act, is_glu=True, add_bias=False, std=0.02).to(dtype)
        with torch.no_grad():
            moe.gate.weight.normal_(0, 0.02)
        x = torch.randn(tokens, H, generator=g).to(dtype).to(device).requires_grad_(True)
        gy = torch.randn(tokens, H, generator=g).to(dtype).to(device)
        logits = None
        if spec["router"] != "gate":
            logits = torch.randn(tokens, spec["E"], generator=g)[:, :E]
            if spec["router"] == "zipf":
                ranks = torch.randperm(spec["E"], generator=torch.Generator().manual_seed(spec["seed"])).float() + 1.0
                logits = logits + (-1.1 * ranks.log())[:E]
            logits = logits.to(device)

        def step() -> None:
            moe.zero_grad(set_to_none=True)
            x.grad = None
            if logits is None:
                y = moe(x, kernel_backend=backend)[0]
            else:
                values, selected = logits.topk(k, dim=-1)
                weights = torch.softmax(values.float(), dim=-1).to(dtype)
                y = moe._compute_experts(x, weights, selected, kernel_backend=backend)
            y.backward(gy)

        sync = (lambda: torch.cuda.synchronize(device)) if device.type == "cuda" else (lambda: None)
        for _ in range(args.warmup):
            step()
        sync()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step()
        sync()
        seconds = (time.perf_counter() - t0) / max(args.steps, 1)
        print(json.dumps({"tokens_per_s": tokens / seconds, "ms_per_step": seconds * 1e3, "threads": torch.get_num_threads(),
                          "backend": args.backend, "device": args.device, "tokens": tokens, "experts": E}))
    except Exception as error:  # the reason goes into the benchmark line
        print(json.dumps({"unavailable": f"{type(error).__name__}: {str(error)[:300]}"}))


if __name__ == "__main__":
    main()
