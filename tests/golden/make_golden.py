"""Generates tests/golden/*.npz by running the REFERENCE implementation's torch path on CPU.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <path to the reference checkout>

The reference package is imported from that path (nothing is copied). Inputs come from numpy's
PCG64 generator so that the tests can regenerate them bit-exactly from the seed; the files hold
the reference's outputs (and the small inputs, for convenience). The reference's torch MoE path
calls `continuous_count` without forwarding `kernel_backend` (xma/layers/moe/__init__.py:219), which
on a CPU-only host reaches the CUDA JIT build; the documented workaround is applied here:
rebinding `xma.layers.moe.continuous_count` to the torch backend. No reference file is modified.
"""

from __future__ import annotations

import functools
import os
import sys

import numpy as np
import torch


def inputs(seed: int, T: int, H: int, I: int, E: int, glu: bool = True) -> dict[str, np.ndarray]:
    """Deterministic inputs shared by this script and tests/golden_inputs.py (keep in sync)."""
    rng = np.random.default_rng(seed)
    f = lambda *s: rng.standard_normal(s, dtype=np.float32)
    return {
        "x": f(T, H),
        "gate": f(E, H) * np.float32(0.02),
        "w_fc": f(E, (2 if glu else 1) * I, H) * np.float32(0.02),
        "w_proj": f(E, H, I) * np.float32(0.02),
        "grad_y": f(T, H),
    }


def sample(a: np.ndarray, step: int = 37) -> np.ndarray:
    return a.reshape(-1)[::step].copy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import xma  # the reference
    import xma.layers.moe as ref_moe
    from xma import KernelBackend, MoE, continuous_count, swiglu_packed

    assert os.path.realpath(os.path.dirname(xma.__file__)).startswith(os.path.realpath(ref_root))
    ref_moe.continuous_count = functools.partial(continuous_count, kernel_backend=KernelBackend.torch)
    out_dir = os.path.dirname(os.path.abspath(__file__))
    torch.set_num_threads(8)

    def run_layer(name, seed, T, H, I, E, k, dtype, activation, glu, full):
        inp = inputs(seed, T, H, I, E, glu)
        moe = MoE(E, k, H, I, activation, glu, False, 0.02)
        with torch.no_grad():
            moe.gate.weight.copy_(torch.from_numpy(inp["gate"]))
            moe.c_fc.weight.copy_(torch.from_numpy(inp["w_fc"]))
            moe.c_proj.weight.copy_(torch.from_numpy(inp["w_proj"]))
        moe = moe.to(dtype)
        x = torch.from_numpy(inp["x"]).to(dtype).requires_grad_(True)
        y, logits = moe(x, kernel_backend=KernelBackend.torch)
        y.backward(torch.from_numpy(inp["grad_y"]).to(dtype))
        with torch.no_grad():
            _, weights, selected = moe._compute_routing_weights(x)
        f32 = lambda t: t.detach().float().numpy()
        rec = {
            "meta": np.array([seed, T, H, I, E, k, int(glu)], dtype=np.int64),
            "y": f32(y), "router_logits": f32(logits), "router_weights": f32(weights),
            "selected_experts": selected.numpy().astype(np.int64),
            "dx": f32(x.grad), "dgate": f32(moe.gate.weight.grad),
        }
        dw_fc, dw_proj = f32(moe.c_fc.weight.grad), f32(moe.c_proj.weight.grad)
        if full:
            rec["dw_fc"], rec["dw_proj"] = dw_fc, dw_proj
        else:
            rec["dw_fc_sample"], rec["dw_proj_sample"] = sample(dw_fc), sample(dw_proj)
            rec["dw_fc_abs_sum"] = np.array(np.abs(dw_fc, dtype=np.float64).sum())
            rec["dw_proj_abs_sum"] = np.array(np.abs(dw_proj, dtype=np.float64).sum())
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **rec)
        print(name, {k_: v.shape for k_, v in rec.items()})

    swiglu = lambda t: swiglu_packed(t, kernel_backend=KernelBackend.torch)
    # small float32 case, every tensor kept
    run_layer("moe_small_fp32", 0, 64, 64, 128, 4, 2, torch.float32, swiglu, True, True)
    # the reference's CPU-runnable benchmark configuration (T=512, H=256, I=512, E=8, k=2, float32)
    run_layer("moe_cfg1_fp32", 0, 512, 256, 512, 8, 2, torch.float32, swiglu, True, False)
    # bfloat16 on the torch path
    run_layer("moe_small_bf16", 1, 64, 64, 128, 4, 2, torch.bfloat16, swiglu, True, True)
    # the activations of the reference's own test (tests/test_commons.py:93-94) at its token count
    run_layer("moe_glu_fp32", 42, 7, 64, 128, 6, 2, torch.float32, torch.nn.GLU(), True, True)
    run_layer("moe_gelu_fp32", 42, 7, 64, 128, 6, 4, torch.float32, torch.nn.GELU(approximate="tanh"), False, True)
    # many experts, top-8, some experts empty
    run_layer("moe_e128_fp32", 3, 7, 64, 128, 128, 8, torch.float32, swiglu, True, False)

    # continuous_count (reference torch backend) on the sizes its test uses around powers of two
    rng = np.random.default_rng(7)
    rec = {}
    for n in (1, 2, 9, 17, 1033, 4105, 3000):
        ids = rng.integers(0, 72, size=n, dtype=np.int64)
        rec[f"ids_{n}"] = ids
        rec[f"count_{n}"] = continuous_count(torch.from_numpy(ids), 72, kernel_backend=KernelBackend.torch).numpy().astype(np.int64)
    rec["count_bins1"] = continuous_count(torch.from_numpy(rec["ids_9"]), 1, kernel_backend=KernelBackend.torch).numpy().astype(np.int64)
    np.savez_compressed(os.path.join(out_dir, "continuous_count.npz"), **rec)

    # swiglu_packed forward/backward (reference torch backend)
    x = torch.from_numpy(np.random.default_rng(9).standard_normal((33, 96), dtype=np.float32)).requires_grad_(True)
    dy = torch.from_numpy(np.random.default_rng(10).standard_normal((33, 48), dtype=np.float32))
    y = swiglu(x)
    y.backward(dy)
    np.savez_compressed(os.path.join(out_dir, "swiglu_packed.npz"), x=x.detach().numpy(), dy=dy.numpy(), y=y.detach().numpy(), dx=x.grad.numpy())
    # unpacked swiglu forward/backward (reference torch backend)
    from xma import swiglu as ref_swiglu

    g = torch.from_numpy(np.random.default_rng(12).standard_normal((37, 40), dtype=np.float32)).requires_grad_(True)
    u = torch.from_numpy(np.random.default_rng(13).standard_normal((37, 40), dtype=np.float32)).requires_grad_(True)
    dy = torch.from_numpy(np.random.default_rng(14).standard_normal((37, 40), dtype=np.float32))
    y = ref_swiglu(g, u, kernel_backend=KernelBackend.torch)
    y.backward(dy)
    np.savez_compressed(os.path.join(out_dir, "swiglu.npz"), gate=g.detach().numpy(), up=u.detach().numpy(), dy=dy.numpy(),
                        y=y.detach().numpy(), dgate=g.grad.numpy(), dup=u.grad.numpy())
    # pack_sequence / unpack_sequence (reference torch backend), both padding sides
    from xma import pack_sequence, unpack_sequence

    rng = np.random.default_rng(11)
    seqlens = np.array([5, 0, 9, 1, 7], dtype=np.int64)
    cu = torch.from_numpy(np.concatenate([[0], np.cumsum(seqlens)]))
    padded = torch.from_numpy(rng.standard_normal((5, 9, 3, 4), dtype=np.float32))
    packed = torch.from_numpy(rng.standard_normal((int(seqlens.sum()), 6), dtype=np.float32))
    rec = {"cu_seqlens": cu.numpy(), "padded": padded.numpy(), "packed": packed.numpy()}
    for side in ("left", "right"):
        rec[f"pack_{side}"] = pack_sequence([padded], cu, int(seqlens.sum()), side, kernel_backend=KernelBackend.torch)[0].numpy()
        rec[f"unpack_{side}"] = unpack_sequence([packed], cu, 5, 9, side, kernel_backend=KernelBackend.torch)[0].numpy()
    np.savez_compressed(os.path.join(out_dir, "sequence_packing.npz"), **rec)
    print("done")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    main(sys.argv[1])
