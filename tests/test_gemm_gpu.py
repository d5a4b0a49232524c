"""tcgen05 grouped GEMMs against float32 per-expert products (tolerance: max rel err 1e-2, bf16 inputs,
float32 accumulation, one bf16 rounding of the result)."""

import pytest
import torch
import torch.nn.functional as F

from gpu_helpers import (assert_status_clean, grouped_reference, make_selection, max_rel_err, padded_rows, row_experts,
                         rows_in_use)
from xma import _native as N
from xma import ops
from xma.layers.moe.routing import build_expert_index

pytestmark = pytest.mark.gpu
TOL = 1e-2

SHAPES = [  # T, E, k, K, N
    (64, 1, 1, 64, 256), (64, 1, 1, 128, 256), (64, 1, 1, 256, 256), (64, 1, 1, 1024, 256), (128, 2, 1, 320, 512),
    (512, 8, 2, 256, 1024), (300, 6, 2, 576, 320), (2048, 64, 8, 512, 768), (1024, 8, 2, 4096, 2048), (7, 128, 8, 576, 256),
    (33, 4, 2, 72, 8),
    # reductions of 4096 and more with a plain store take the 256 x 512 tile: N a multiple of 512, N with a
    # partial last tile, N below 512 (narrow tile again), odd tile counts per expert, a single row
    (300, 6, 2, 8192, 1024), (700, 3, 2, 8192, 640), (64, 2, 1, 8256, 1536), (300, 6, 2, 8192, 256), (1, 1, 1, 16384, 512),
]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("layout", [N.GEMM_NT, N.GEMM_NN])
@pytest.mark.parametrize("T,E,k,K,Nn", SHAPES)
def test_grouped_gemm_store(device, layout, dtype, T, E, k, K, Nn):
    index = build_expert_index(make_selection(T, E, k, device, skew=E >= 64), E)
    used = rows_in_use(index)
    a = padded_rows(index, K, dtype)
    shape = (E, Nn, K) if layout == N.GEMM_NT else (E, K, Nn)
    w = (torch.randn(*shape, device=device) * 0.1).to(dtype)
    c = torch.full((index.cap, Nn), float("nan"), device=device, dtype=dtype)
    ops.grouped_gemm_cuda(a, w, index.padded_offsets, c, None, None, None, None, layout, N.EPI_STORE)
    assert_status_clean(device)
    ref = grouped_reference(a, w, index, used, transpose_w=layout == N.GEMM_NT)
    assert max_rel_err(c[:used], ref) < TOL
    assert torch.all(c[:used][index.row_src[:used] < 0] == 0)  # padding rows stay zero


@pytest.mark.parametrize("T,E,k,M,Nn,skew", [(64, 1, 1, 128, 256, False), (300, 2, 1, 128, 256, False), (512, 8, 2, 256, 512, False),
                                             (300, 6, 2, 320, 576, False), (2048, 64, 8, 512, 256, True), (4096, 8, 2, 1024, 2048, False),
                                             (7, 128, 8, 256, 576, False), (50, 3, 1, 8, 8, False),
                                             # a mean of 2048 rows per expert and more takes the 256 x 512 tile
                                             (5000, 2, 1, 320, 1024, False), (9000, 4, 1, 256, 640, True), (2500, 1, 1, 128, 512, False),
                                             # ... and so does a weight matrix of 2^23 elements, however few the rows
                                             (300, 3, 1, 2048, 4096, True)])
def test_grouped_wgrad(device, T, E, k, M, Nn, skew):
    index = build_expert_index(make_selection(T, E, k, device, skew), E)
    used = rows_in_use(index)
    x = padded_rows(index, M, seed=1)
    y = padded_rows(index, Nn, seed=2)
    dw = torch.full((E, M, Nn), float("nan"), device=device, dtype=torch.bfloat16)
    ops.grouped_wgrad_cuda(x, y, index.padded_offsets, dw)
    assert_status_clean(device)
    experts = row_experts(index, used)
    ref = torch.zeros(E, M, Nn, device=device)
    for e in range(E):
        m = experts == e
        if m.any():
            ref[e] = x[:used][m].float().t() @ y[:used][m].float()
    assert max_rel_err(dw, ref) < TOL
    empty = index.expert_frequency.cpu().long() == 0
    if empty.any():  # experts without rows get exact zeros (the reference pre-zeroes, __init__.py:121)
        assert torch.all(dw[empty.to(device)] == 0)


@pytest.mark.parametrize("T,E,k,H,I", [(64, 1, 1, 64, 128), (512, 8, 2, 256, 512), (300, 6, 2, 576, 256), (2048, 64, 8, 512, 1024),
                                       (7, 128, 8, 576, 256)])
def test_swiglu_epilogues(device, T, E, k, H, I):
    index = build_expert_index(make_selection(T, E, k, device), E)
    used = rows_in_use(index)
    xg = padded_rows(index, H)
    w1 = (torch.randn(E, 2 * I, H, device=device) * 0.05).to(torch.bfloat16)
    p = torch.rand(T * k, device=device).to(torch.bfloat16)
    pre = torch.empty(index.cap, 2 * I, device=device, dtype=torch.bfloat16)
    act = torch.empty(index.cap, I, device=device, dtype=torch.bfloat16)
    ops.grouped_gemm_cuda(xg, w1, index.padded_offsets, pre, act, index.row_src, p, None, N.GEMM_NT, N.EPI_SWIGLU)
    assert_status_clean(device)
    assert max_rel_err(pre[:used], grouped_reference(xg, w1, index, used, True)) < TOL
    rp = pre[:used].float()
    rs = index.row_src[:used].long()
    scale = torch.where(rs >= 0, p.float()[rs.clamp(min=0)], torch.zeros((), device=device))
    # the activation is computed from the ROUNDED pre-activation, as the reference does
    assert max_rel_err(act[:used], rp[:, :I] * F.silu(rp[:, I:]) * scale[:, None]) < TOL

    w2 = (torch.randn(E, H, I, device=device) * 0.05).to(torch.bfloat16)
    dyg = padded_rows(index, H, seed=3)
    dpre = torch.empty(index.cap, 2 * I, device=device, dtype=torch.bfloat16)
    # d(row scale): per-column-tile partial sums [tiles, cap], added up in tile order by a second kernel
    partials = torch.full((N.gemm_n_tiles(I), index.cap), float("nan"), device=device)
    ops.grouped_gemm_cuda(dyg, w2, index.padded_offsets, dpre, pre, index.row_src, p, partials, N.GEMM_NN, N.EPI_SWIGLU_BWD)
    dscale = torch.zeros(T * k, device=device)
    ops.reduce_row_partials_cuda(partials, index.row_src, index.rows_in_use, dscale)
    assert_status_clean(device)
    acc = grouped_reference(dyg, w2, index, used, False)
    u, g = rp[:, :I], rp[:, I:]
    s = torch.sigmoid(g)
    dh = acc * scale[:, None]
    assert max_rel_err(dpre[:used], torch.cat([dh * g * s, dh * u * (s + g * s * (1 - s))], 1)) < TOL
    want = torch.zeros(T * k, device=device)
    want[rs[rs >= 0]] = (acc * u * g * s).sum(1)[rs >= 0]
    assert max_rel_err(dscale, want) < 1e-4  # float32 accumulation, only the summation order differs


def test_linearity_at_benchmark_size(device):
    """Size-independent property on the OLMoE-like shape (M=65536, K=2048, N=2048):
    gemm(a, w) + gemm(b, w) == gemm(a + b, w) up to bf16 rounding of the three results."""
    T, E, k, K, Nn = 8192, 64, 8, 2048, 2048
    index = build_expert_index(make_selection(T, E, k, device, seed=1), E)
    used = rows_in_use(index)
    a = padded_rows(index, K, seed=1)
    b = padded_rows(index, K, seed=2)
    w = (torch.randn(E, Nn, K, device=device) * 0.02).to(torch.bfloat16)
    outs = []
    for inp in (a, b, a + b):
        c = torch.empty(index.cap, Nn, device=device, dtype=torch.bfloat16)
        ops.grouped_gemm_cuda(inp, w, index.padded_offsets, c, None, None, None, None, N.GEMM_NT, N.EPI_STORE)
        outs.append(c[:used].float())
    assert_status_clean(device)
    # a + b is rounded to bf16 before the product: allow 3 roundings of relative size 2^-8
    assert max_rel_err(outs[0] + outs[1], outs[2]) < 1.5e-2


def test_split_f32_is_an_exact_hi_lo_pair(device):
    """hi = bf16(src) bit-exactly, lo = bf16(src - hi) bit-exactly, hi + lo within 2^-16 of src; odd
    counts exercise the scalar tail."""
    for count in (1, 3, 4, 1001, 1 << 20):
        src = torch.randn(count, device=device) * 3
        hi = torch.empty(count, device=device, dtype=torch.bfloat16)
        lo = torch.empty_like(hi)
        ops.split_f32_cuda(src, hi, lo)
        assert torch.equal(hi, src.to(torch.bfloat16))
        assert torch.equal(lo, (src - hi.float()).to(torch.bfloat16))
        assert torch.all((hi.float() + lo.float() - src).abs() <= src.abs() * 2.0 ** -16)


@pytest.mark.parametrize("layout", [N.GEMM_NT, N.GEMM_NN])
@pytest.mark.parametrize("T,E,k,K,Nn", [(64, 1, 1, 64, 256), (300, 6, 2, 576, 320), (2048, 64, 8, 512, 768), (7, 128, 8, 576, 256),
                                        (33, 4, 2, 72, 8)])
def test_grouped_gemm_float32_output(device, layout, T, E, k, K, Nn):
    """EPI_STORE_F32 writes the float32 accumulator unrounded; EPI_ADD_F32 adds to what is there.
    bf16 products are exact in float32, so the only difference to the float32 reference is the order
    of the additions: tolerance 1e-5 relative."""
    index = build_expert_index(make_selection(T, E, k, device, skew=E >= 64), E)
    used = rows_in_use(index)
    a = padded_rows(index, K, torch.bfloat16)
    shape = (E, Nn, K) if layout == N.GEMM_NT else (E, K, Nn)
    w = (torch.randn(*shape, device=device) * 0.1).to(torch.bfloat16)
    c = torch.full((index.cap, Nn), float("nan"), device=device, dtype=torch.float32)
    ops.grouped_gemm_cuda(a, w, index.padded_offsets, c, None, None, None, None, layout, N.EPI_STORE_F32)
    ref = grouped_reference(a, w, index, used, transpose_w=layout == N.GEMM_NT)
    assert max_rel_err(c[:used], ref) < 1e-5
    first = c.clone()
    ops.grouped_gemm_cuda(a, w, index.padded_offsets, c, None, None, None, None, layout, N.EPI_ADD_F32)
    assert_status_clean(device)
    assert torch.equal(c[:used], 2 * first[:used])


@pytest.mark.parametrize("T,E,k,M,Nn,skew", [(64, 1, 1, 128, 256, False), (300, 6, 2, 320, 576, False), (2048, 64, 8, 512, 256, True),
                                             (50, 3, 1, 8, 8, False)])
def test_grouped_wgrad_float32_output(device, T, E, k, M, Nn, skew):
    index = build_expert_index(make_selection(T, E, k, device, skew), E)
    used = rows_in_use(index)
    x = padded_rows(index, M, seed=1)
    y = padded_rows(index, Nn, seed=2)
    dw = torch.full((E, M, Nn), float("nan"), device=device, dtype=torch.float32)
    ops.grouped_wgrad_f32_cuda(x, y, index.padded_offsets, dw, False)
    experts = row_experts(index, used)
    ref = torch.zeros(E, M, Nn, device=device)
    for e in range(E):
        m = experts == e
        if m.any():
            ref[e] = x[:used][m].float().t() @ y[:used][m].float()
    assert max_rel_err(dw, ref) < 1e-5
    empty = (index.expert_frequency.cpu().long() == 0).to(device)
    if empty.any():
        assert torch.all(dw[empty] == 0)
    first = dw.clone()
    ops.grouped_wgrad_f32_cuda(x, y, index.padded_offsets, dw, True)
    assert_status_clean(device)
    assert torch.equal(dw, 2 * first)
