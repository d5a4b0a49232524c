"""Host-side behaviour of the drop-in surface that needs no GPU."""

import pytest
import torch

import xma
from xma import KernelBackend, MoE, continuous_count, swiglu_packed
from xma.accelerator import require_cuda_backend


def test_kernel_backend_enum_matches_reference_values():
    assert {b.value for b in KernelBackend} == {"cuda", "nki", "pallas", "rocm", "torch", "triton"}


@pytest.mark.parametrize("backend", [KernelBackend.torch, KernelBackend.triton, KernelBackend.rocm])
def test_other_backends_raise(backend):
    with pytest.raises(ValueError, match="not available"):
        require_cuda_backend(backend)
    require_cuda_backend(None)
    require_cuda_backend(KernelBackend.cuda)


def test_state_dict_matches_reference_layout():
    moe = MoE(num_experts=4, num_experts_per_tok=2, hidden_size=64, intermediate_size=128,
              activation_function=swiglu_packed, is_glu=True, add_bias=False, std=0.02)
    sd = moe.state_dict()
    assert list(sd) == ["gate.weight", "c_fc.weight", "c_fc.N_array", "c_fc.K_array", "c_proj.weight",
                        "c_proj.N_array", "c_proj.K_array"]
    assert sd["c_fc.weight"].shape == (4, 256, 64) and sd["c_proj.weight"].shape == (4, 64, 128)
    assert sd["c_fc.N_array"].dtype == torch.uint32 and sd["c_fc.N_array"].tolist() == [256] * 4
    assert sd["c_fc.K_array"].tolist() == [64] * 4 and sd["c_proj.N_array"].tolist() == [64] * 4
    assert sd["gate.weight"].shape == (4, 64)
    non_glu = MoE(4, 2, 64, 128, torch.nn.GELU(), False, False, 0.02)
    assert non_glu.c_fc.weight.shape == (4, 128, 64)
    assert abs(moe.c_fc.weight.std().item() - 0.02) < 2e-3


def test_continuous_count_bins_one_shortcut():
    out = continuous_count(torch.arange(5), 1)
    assert out.dtype == torch.uint32 and out.tolist() == [5]


def test_continuous_count_checks_its_input():
    with pytest.raises(AssertionError):
        continuous_count(torch.zeros(2, 2, dtype=torch.int64), 4)
    with pytest.raises(AssertionError):
        continuous_count(torch.zeros(4), 4)


def test_no_cpu_fallback():
    """CPU tensors never take a silent slow path: the ops refuse them."""
    with pytest.raises(Exception):
        continuous_count(torch.zeros(8, dtype=torch.int64), 4)
    moe = MoE(4, 2, 64, 128, swiglu_packed, True, False, 0.02)
    with pytest.raises(Exception):
        moe(torch.randn(3, 64))
    with pytest.raises(ValueError):
        moe(torch.randn(3, 64), kernel_backend=KernelBackend.torch)


def test_missing_library_fails_loudly(monkeypatch):
    from xma import _native as N

    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", "/nonexistent/libxma_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        N.lib()


def test_set_seed():
    xma.set_seed(3)
    a = torch.rand(2)
    xma.set_seed(3)
    assert torch.equal(a, torch.rand(2))


def test_path_selection_policy():
    """Which kernels a layer takes is decided on the host from dtypes and sizes alone."""
    from xma.layers.moe.routing import FUSED_ROUTER_MAX_EXPERTS, fused_router_supported

    def layer(E, k, H, I, act, dtype):
        return xma.MoE(num_experts=E, num_experts_per_tok=k, hidden_size=H, intermediate_size=I, activation_function=act,
                       is_glu=True, add_bias=False, std=0.02).to(dtype)

    assert layer(8, 2, 64, 128, xma.swiglu_packed, torch.bfloat16)._fused_path()
    assert layer(8, 2, 64, 128, xma.swiglu_packed, torch.float16)._fused_path()
    assert not layer(8, 2, 64, 128, xma.swiglu_packed, torch.float32)._fused_path()  # split-bf16 unfused products
    assert not layer(8, 2, 64, 96, xma.swiglu_packed, torch.bfloat16)._fused_path()   # I not a multiple of 128
    assert not layer(8, 2, 64, 128, torch.nn.GLU(), torch.bfloat16)._fused_path()     # any other callable

    x = torch.empty(4, 64, dtype=torch.bfloat16)
    w = lambda E, dtype=torch.bfloat16: torch.empty(E, 64, dtype=dtype)
    assert FUSED_ROUTER_MAX_EXPERTS == 256
    assert fused_router_supported(x, w(128), 8) and fused_router_supported(x, w(256), 8)
    assert fused_router_supported(x, w(64), 8) and fused_router_supported(x, w(8), 2)
    assert not fused_router_supported(x, w(6), 2)       # logits rows of 12 bytes cannot leave through bulk tensor stores
    assert not fused_router_supported(x, w(264), 8)     # more experts than one accumulator tile holds
    assert not fused_router_supported(x, w(136 - 4), 8)  # E % 8
    assert not fused_router_supported(x, w(128), 9)
    assert not fused_router_supported(x.float(), w(128, torch.float32), 8)
    assert not fused_router_supported(x, w(128, torch.float16), 8)  # mixed dtypes


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on the host alone (the reference's torch path from its unmodified
    copy when that exists, else the CPU oracle) and prints one JSON line with the contract's keys."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    done = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--workload", "cfg1",
                           "--steps", "1", "--warmup", "1"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-500:]
    lines = [l for l in done.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["config"]["workload"].startswith("cfg1")


def test_bench_accounting_helpers(tmp_path):
    """The benchmark's arithmetic that needs no GPU: FLOP model, per-kernel FLOPs, the expert-parallel
    time split and the clock-sample window."""
    import importlib.util
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("xma_bench", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    w = bench.WORKLOADS["mixtral"]
    assert bench.step_flops(w, w["T"]) == 18.0 * 16384 * 2 * 4096 * 14336          # no gate GEMM: logits are injected
    o = bench.WORKLOADS["olmoe"]
    assert bench.step_flops(o, o["T"]) == 18.0 * 8192 * 8 * 2048 * 1024 + 6.0 * 8192 * 2048 * 64
    rows = 32768
    parts = [bench.kernel_flops(k, w, rows) for k in ("grouped_gemm[NT,swiglu]", "grouped_gemm[NT,store]",
                                                       "grouped_gemm[NN,swiglu_bwd]", "grouped_gemm[NN,store]")]
    assert sum(parts) + 2 * bench.kernel_flops("grouped_wgrad", w, rows) == bench.step_flops(w, w["T"])
    assert bench.kernel_flops("combine_rows", w, rows) is None

    table = {
        "grouped_wgrad": {"launches": 4, "avg_ms": 1.0}, "grouped_gemm[NT,swiglu]": {"launches": 2, "avg_ms": 2.0},
        "ep_barrier": {"launches": 10, "avg_ms": 0.02}, "ep_exchange_counts": {"launches": 2, "avg_ms": 0.03},
        "ep_dispatch_rows": {"launches": 4, "avg_ms": 0.1}, "moe_index_build": {"launches": 2, "avg_ms": 0.05},
        "overlapped_ep_barrier": {"launches": 2, "avg_ms": 0.3}, "overlapped_ep_combine_pull": {"launches": 2, "avg_ms": 0.1},
    }
    split = bench.ep_overheads(table, steps=2, ms=5.0)
    assert split["gemm_ms"] == 4.0 and split["barrier_and_count_exchange_ms"] == 0.13
    assert split["row_movement_ms"] == 0.2 and split["other_kernels_ms"] == 0.05
    assert abs(split["outside_kernels_ms"] - 0.62) < 1e-9 and split["launches_per_step"] == 14.0
    assert split["second_stream_ms"] == 0.4  # second-stream launches: reported, not charged to the step

    sampler = bench.ClockSampler.__new__(bench.ClockSampler)
    sampler.path = str(tmp_path / "clocks.txt")
    with open(sampler.path, "w") as fh:
        fh.write("max 1965\n10.0 1900 0\n11.0 1200 4\n12.0 1300 4\n13.0 1250 4\n20.0 600 8\n")
    got = sampler.window(10.5, 13.5)
    assert got == {"sm_mhz": 1250, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"], "samples": 3}
