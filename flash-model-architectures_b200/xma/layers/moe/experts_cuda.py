"""Autograd functions that run the expert MLPs on the sm_100a grouped GEMMs.

`fused_swiglu_experts` is the hot path: gather -> up projection with the swiglu and the router
weight fused in the epilogue -> down projection -> k-way sum, and the matching backward
(dX, per-expert dW, swiglu backward and router-probability gradient). It stands in for
_ScatteredExperts (xma/layers/moe/triton_implementation/__init__.py:12-161) used twice with
swiglu_packed between.

`grouped_linear`, `gather_rows` and `combine_rows` are the unfused pieces for arbitrary
activation callables.
"""

from __future__ import annotations

import torch

from ... import _native as N
from ... import ops
from .routing import ExpertIndex


def _check_dtype(*tensors: torch.Tensor) -> None:
    dtype = tensors[0].dtype
    if dtype not in (torch.bfloat16, torch.float16):
        raise RuntimeError(f"the sm_100a grouped GEMM runs in bf16 or fp16, got {dtype}")
    for t in tensors:
        if t.dtype != dtype:
            raise RuntimeError(f"mixed dtypes: {dtype} and {t.dtype}")


class _FusedSwigluExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, index: ExpertIndex):
        scaled = router_weights is not None
        _check_dtype(x, w_fc, w_proj, *([router_weights] if scaled else []))
        x = x.contiguous()
        w_fc = w_fc.contiguous()
        w_proj = w_proj.contiguous()
        scale = router_weights.contiguous().view(-1) if scaled else None
        T, H = x.shape
        E, two_i, _ = w_fc.shape
        inter = two_i // 2
        k = index.top_k
        cap = index.cap
        opts = dict(dtype=x.dtype, device=x.device)

        xg = torch.empty(cap, H, **opts)
        ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, xg, k, index.inv_row)
        pre = torch.empty(cap, two_i, **opts)
        act = torch.empty(cap, inter, **opts)  # router_weight * swiglu(pre)
        ops.grouped_gemm_cuda(
            xg, w_fc, index.padded_offsets, pre, act, index.row_src, scale, None, N.GEMM_NT, N.EPI_SWIGLU
        )
        out_rows = torch.empty(cap, H, **opts)
        ops.grouped_gemm_cuda(
            act, w_proj, index.padded_offsets, out_rows, None, None, None, None, N.GEMM_NT, N.EPI_STORE
        )
        y = torch.empty(T, H, **opts)
        ops.combine_rows_cuda(out_rows, index.inv_row, None, y, k)

        ctx.save_for_backward(xg, pre, act, w_fc, w_proj, scale)
        ctx.index = index
        ctx.num_tokens = T
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, pre, act, w_fc, w_proj, scale = ctx.saved_tensors
        index: ExpertIndex = ctx.index
        dy = dy.contiguous()
        T, H = dy.shape
        E, two_i, _ = w_fc.shape
        inter = two_i // 2
        k = index.top_k
        cap = index.cap
        opts = dict(dtype=dy.dtype, device=dy.device)

        dyg = torch.empty(cap, H, **opts)
        ops.permute_rows_cuda(dy, index.row_src, index.rows_in_use, None, dyg, k, index.inv_row)

        # d(pre) = swiglu'(pre) * router_weight * (dy W_proj); the same epilogue accumulates
        # d(router_weight) = <dy W_proj, swiglu(pre)>.
        d_pre = torch.empty(cap, two_i, **opts)
        d_router = torch.zeros(T * k, dtype=torch.float32, device=dy.device) if scale is not None else None
        ops.grouped_gemm_cuda(
            dyg, w_proj, index.padded_offsets, d_pre, pre, index.row_src, scale, d_router, N.GEMM_NN,
            N.EPI_SWIGLU_BWD,
        )
        dw_proj = torch.empty_like(w_proj)
        ops.grouped_wgrad_cuda(dyg, act, index.padded_offsets, dw_proj)
        dw_fc = torch.empty_like(w_fc)
        ops.grouped_wgrad_cuda(d_pre, xg, index.padded_offsets, dw_fc)

        dxg = dyg  # dyg is dead after the two products above; reuse its storage
        ops.grouped_gemm_cuda(
            d_pre, w_fc, index.padded_offsets, dxg, None, None, None, None, N.GEMM_NN, N.EPI_STORE
        )
        dx = torch.empty(T, H, **opts)
        ops.combine_rows_cuda(dxg, index.inv_row, None, dx, k)
        d_weights = d_router.view(T, k).to(dy.dtype) if d_router is not None else None
        return dx, dw_fc, dw_proj, d_weights, None


def fused_swiglu_experts(x, w_fc, w_proj, router_weights, index: ExpertIndex) -> torch.Tensor:
    """y[t] = sum_j p[t,j] * W_proj[e] swiglu(W_fc[e] x[t]) for e = selected[t,j]; p = 1 when
    `router_weights` is None (expert-parallel ranks scale on the token's home rank instead)."""
    return _FusedSwigluExperts.apply(x, w_fc, w_proj, router_weights, index)


class _GatherRows(torch.autograd.Function):
    """rows[p] = x[row_src[p] // k] (the `group` kernel, group_kernel.py:12-100)."""

    @staticmethod
    def forward(ctx, x, index: ExpertIndex, rows: int | None):
        x = x.contiguous()
        out = torch.empty(index.cap if rows is None else rows, x.size(1), dtype=x.dtype, device=x.device)
        ops.permute_rows_cuda(x, index.row_src, index.rows_in_use, None, out, index.top_k, index.inv_row)
        ctx.index = index
        ctx.num_tokens = x.size(0)
        return out

    @staticmethod
    def backward(ctx, d_rows):
        index: ExpertIndex = ctx.index
        d_rows = d_rows.contiguous()
        dx = torch.empty(ctx.num_tokens, d_rows.size(1), dtype=d_rows.dtype, device=d_rows.device)
        ops.combine_rows_cuda(d_rows, index.inv_row, None, dx, index.top_k)
        return dx, None, None


class _CombineRows(torch.autograd.Function):
    """y[t] = sum_j w[t,j] * rows[inv_row[t*k+j]] (bmm at triton_implementation/__init__.py:39-43)."""

    @staticmethod
    def forward(ctx, rows, weights, index: ExpertIndex):
        rows = rows.contiguous()
        weights = weights.contiguous()
        T = weights.size(0)
        y = torch.empty(T, rows.size(1), dtype=rows.dtype, device=rows.device)
        ops.combine_rows_cuda(rows, index.inv_row, weights.view(-1), y, index.top_k)
        ctx.save_for_backward(rows, weights)
        ctx.index = index
        return y

    @staticmethod
    def backward(ctx, dy):
        rows, weights = ctx.saved_tensors
        index: ExpertIndex = ctx.index
        dy = dy.contiguous()
        d_rows = torch.empty_like(rows)
        ops.permute_rows_cuda(
            dy, index.row_src, index.rows_in_use, weights.view(-1), d_rows, index.top_k, index.inv_row
        )
        d_weights = torch.empty_like(weights)
        ops.combine_rows_backward_weights_cuda(rows, index.inv_row, dy, d_weights.view(-1), index.top_k)
        return d_rows, d_weights, None


class _GroupedLinear(torch.autograd.Function):
    """rows_out[p] = rows_in[p] @ W[e(p)]^T over rows in padded expert order."""

    @staticmethod
    def forward(ctx, rows, weight, index: ExpertIndex):
        _check_dtype(rows, weight)
        rows = rows.contiguous()
        weight = weight.contiguous()
        out = torch.empty(index.cap, weight.size(1), dtype=rows.dtype, device=rows.device)
        ops.grouped_gemm_cuda(
            rows, weight, index.padded_offsets, out, None, None, None, None, N.GEMM_NT,
            N.EPI_STORE,
        )
        ctx.save_for_backward(rows, weight)
        ctx.index = index
        return out

    @staticmethod
    def backward(ctx, d_out):
        rows, weight = ctx.saved_tensors
        index: ExpertIndex = ctx.index
        d_out = d_out.contiguous()
        d_rows = torch.empty_like(rows)
        ops.grouped_gemm_cuda(
            d_out, weight, index.padded_offsets, d_rows, None, None, None, None, N.GEMM_NN, N.EPI_STORE
        )
        d_weight = torch.empty_like(weight)
        ops.grouped_wgrad_cuda(d_out, rows, index.padded_offsets, d_weight)
        return d_rows, d_weight, None


def _split(t: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    hi = torch.empty(t.shape, dtype=torch.bfloat16, device=t.device)
    lo = torch.empty_like(hi)
    ops.split_f32_cuda(t.contiguous(), hi, lo)
    return hi, lo


def _product_f32(a, w, padded_offsets, out, layout: int) -> None:
    """out (float32) = a @ w[e] from split operands: hi*hi, then hi*lo and lo*hi added in place."""
    (a_hi, a_lo), (w_hi, w_lo) = a, w
    for i, (x, y) in enumerate(((a_hi, w_hi), (a_hi, w_lo), (a_lo, w_hi))):
        ops.grouped_gemm_cuda(x, y, padded_offsets, out, None, None, None, None, layout,
                              N.EPI_STORE_F32 if i == 0 else N.EPI_ADD_F32)


class _GroupedLinearF32(torch.autograd.Function):
    """`_GroupedLinear` for float32 rows and weights. The tensor cores take bf16: every operand is
    split into a bf16 pair (value = hi + lo to 2^-16 relative) and a product is three bf16 passes
    accumulated in float32, which is tighter than the TF32 products the reference's Triton kernels
    make of float32 inputs (scatter_kernel.py:49)."""

    @staticmethod
    def forward(ctx, rows, weight, index: ExpertIndex):
        rows_s, weight_s = _split(rows), _split(weight)
        out = torch.empty(index.cap, weight.size(1), dtype=torch.float32, device=rows.device)
        _product_f32(rows_s, weight_s, index.padded_offsets, out, N.GEMM_NT)
        ctx.save_for_backward(*rows_s, *weight_s)
        ctx.index = index
        return out

    @staticmethod
    def backward(ctx, d_out):
        r_hi, r_lo, w_hi, w_lo = ctx.saved_tensors
        index: ExpertIndex = ctx.index
        d_hi, d_lo = _split(d_out)
        d_rows = torch.empty(r_hi.shape, dtype=torch.float32, device=d_out.device)
        _product_f32((d_hi, d_lo), (w_hi, w_lo), index.padded_offsets, d_rows, N.GEMM_NN)
        d_weight = torch.empty(w_hi.shape, dtype=torch.float32, device=d_out.device)
        for i, (x, y) in enumerate(((d_hi, r_hi), (d_hi, r_lo), (d_lo, r_hi))):
            ops.grouped_wgrad_f32_cuda(x, y, index.padded_offsets, d_weight, i > 0)
        return d_rows, d_weight, None


def gather_rows(x, index: ExpertIndex, rows: int | None = None) -> torch.Tensor:
    """`rows` limits the output to its first rows (the unpadded order needs exactly T*k of them)."""
    return _GatherRows.apply(x, index, rows)


def combine_rows(rows, weights, index: ExpertIndex) -> torch.Tensor:
    return _CombineRows.apply(rows, weights, index)


def grouped_linear(rows, weight, index: ExpertIndex) -> torch.Tensor:
    if rows.dtype == torch.float32 and weight.dtype == torch.float32:
        return _GroupedLinearF32.apply(rows, weight, index)
    return _GroupedLinear.apply(rows, weight, index)
