"""Gather into padded expert order, top-k combine and its weight gradient (HBM-bound row kernels)."""

import pytest
import torch

from gpu_helpers import make_selection, rows_in_use
from xma import ops
from xma.layers.moe.routing import build_expert_index

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
# The last four shapes have fewer 16-byte vectors per row (or in the last 32-vector step of a row) than
# copies per token: lanes that hold a copy's destination then have no column of their own.
@pytest.mark.parametrize("T,E,k,H", [(7, 8, 2, 64), (512, 8, 2, 256), (2048, 64, 8, 2048), (300, 6, 4, 576), (129, 2, 1, 8),
                                     (1500, 40, 8, 48), (333, 16, 8, 8), (400, 64, 8, 288), (200, 32, 6, 264)])
def test_permute_and_combine(device, dtype, T, E, k, H):
    index = build_expert_index(make_selection(T, E, k, device), E)
    used = rows_in_use(index)
    x = torch.randn(T, H, device=device, dtype=dtype)
    w = torch.rand(T, k, device=device, dtype=dtype)
    rs = index.row_src[:used].long()
    valid = (rs >= 0)[:, None]
    src = rs.clamp(min=0)
    zero = torch.zeros((), device=device, dtype=dtype)

    want_scaled = torch.where(valid, (x[src // k].float() * w.view(-1)[src].float()[:, None]).to(dtype), zero)
    for inv_row in (None, index.inv_row):  # destination-major gather, then the source-major form
        out = torch.full((index.cap, H), float("nan"), device=device, dtype=dtype)
        ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, out, k, inv_row)
        assert torch.equal(out[:used], torch.where(valid, x[src // k], zero))  # a copy: bit-exact
        ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, w.view(-1), out, k, inv_row)
        assert torch.equal(out[:used], want_scaled)  # one float32 multiply, one rounding: bit-exact

    rows = torch.randn(index.cap, H, device=device, dtype=dtype)
    y = torch.empty(T, H, device=device, dtype=dtype)
    picked = rows[index.inv_row.long()].view(T, k, H).float()
    tol = dict(rtol=0, atol=1e-5 * k) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1e-2)
    ops.combine_rows_cuda(rows, index.inv_row, w.view(-1), y, k)
    torch.testing.assert_close(y.float(), (picked * w.float()[:, :, None]).sum(1), **tol)
    ops.combine_rows_cuda(rows, index.inv_row, None, y, k)
    torch.testing.assert_close(y.float(), picked.sum(1), **tol)

    dy = torch.randn(T, H, device=device, dtype=dtype)
    dw = torch.empty(T, k, device=device, dtype=dtype)
    ops.combine_rows_backward_weights_cuda(rows, index.inv_row, dy, dw.view(-1), k)
    want = (picked * dy.float()[:, None, :]).sum(-1)
    tol = dict(rtol=1e-4, atol=1e-3) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=0.5)
    torch.testing.assert_close(dw.float(), want, **tol)


def test_gather_then_sum_is_k_times_identity(device):
    """Size-independent property at full benchmark size: combine(permute(x)) == k * x exactly for
    k a power of two (every addend is the same bf16 value)."""
    T, E, k, H = 8192, 64, 8, 2048
    index = build_expert_index(make_selection(T, E, k, device, seed=1), E)
    x = torch.randn(T, H, device=device, dtype=torch.bfloat16)
    rows = torch.empty(index.cap, H, device=device, dtype=torch.bfloat16)
    ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, rows, k, index.inv_row)
    y = torch.empty_like(x)
    ops.combine_rows_cuda(rows, index.inv_row, None, y, k)
    assert torch.equal(y, x * k)
