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
