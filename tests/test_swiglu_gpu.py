"""Stand-alone swiglu (unpacked) on the GPU: the reference's golden vectors, its test matrix
(tests/functional/swiglu_test.py:19-65: 2-d sizes, three dtypes, eager and torch.compile) and the
tolerances it states (float32: 5.4e-5 forward, 5e-6 gradients; 16-bit types: one rounding)."""

import numpy as np
import pytest
import torch

import xma
from golden_inputs import GOLDEN_DIR
from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def test_swiglu_reference_goldens(device):
    rec = np.load(f"{GOLDEN_DIR}/swiglu.npz")
    g = torch.from_numpy(rec["gate"]).to(device).requires_grad_(True)
    u = torch.from_numpy(rec["up"]).to(device).requires_grad_(True)
    y = xma.swiglu(g, u)
    y.backward(torch.from_numpy(rec["dy"]).to(device))
    torch.testing.assert_close(y.detach().cpu(), torch.from_numpy(rec["y"]), rtol=0, atol=5.4e-5)
    torch.testing.assert_close(g.grad.cpu(), torch.from_numpy(rec["dgate"]), rtol=0, atol=5e-6)
    torch.testing.assert_close(u.grad.cpu(), torch.from_numpy(rec["dup"]), rtol=0, atol=5e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("size", [(1, 1), (7, 5), (33, 40), (1024, 1024), (4100, 3700), (3, 7, 16)])
def test_swiglu_matches_oracle(device, dtype, size):
    """Odd sizes take the scalar kernel, sizes that are a multiple of 16 bytes the vector kernel."""
    g = torch.randn(*size, device=device).to(dtype).requires_grad_(True)
    u = torch.randn(*size, device=device).to(dtype).requires_grad_(True)
    y = xma.swiglu(g, u, kernel_backend=xma.KernelBackend.cuda)
    y.mean().backward()
    g2, u2 = g.detach().clone().requires_grad_(True), u.detach().clone().requires_grad_(True)
    ref = O.swiglu(g2, u2)
    ref.mean().backward()
    if dtype == torch.float32:
        torch.testing.assert_close(y, ref, rtol=0, atol=5.4e-5)
        torch.testing.assert_close(g.grad, g2.grad, rtol=0, atol=5e-6)
        torch.testing.assert_close(u.grad, u2.grad, rtol=0, atol=5e-6)
    else:
        torch.testing.assert_close(y, ref, rtol=1.6e-2, atol=1e-3)
        torch.testing.assert_close(g.grad.float(), g2.grad.float(), rtol=1.6e-2, atol=1e-6)
        torch.testing.assert_close(u.grad.float(), u2.grad.float(), rtol=1.6e-2, atol=1e-6)


def test_swiglu_under_torch_compile(device):
    g = torch.randn(64, 256, device=device, dtype=torch.bfloat16)
    u = torch.randn(64, 256, device=device, dtype=torch.bfloat16)
    compiled = torch.compile(xma.swiglu, fullgraph=True)(g, u)
    assert torch.equal(compiled, xma.swiglu(g, u))


def test_swiglu_rejects_mismatched_inputs(device):
    g = torch.randn(4, 8, device=device)
    with pytest.raises(AssertionError):
        xma.swiglu(g, torch.randn(4, 9, device=device))
    with pytest.raises(AssertionError):
        xma.swiglu(g, torch.randn(4, 8, device=device, dtype=torch.bfloat16))
