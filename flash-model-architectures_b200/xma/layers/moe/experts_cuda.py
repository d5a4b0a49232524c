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
    """Index tensors come in as plain arguments and are kept with save_for_backward (no tensor hangs
    on `ctx` as an attribute), so torch.compile can trace forward and backward of the function."""

    @staticmethod
    def forward(ctx, x, w_fc, w_proj, router_weights, padded_offsets, row_src, inv_row, rows_in_use, cap: int, k: int):
        scaled = router_weights is not None
        _check_dtype(x, w_fc, w_proj, *([router_weights] if scaled else []))
        x = x.contiguous()
        w_fc = w_fc.contiguous()
        w_proj = w_proj.contiguous()
        scale = router_weights.contiguous().view(-1) if scaled else None
        T, H = x.shape
        E, two_i, _ = w_fc.shape
        inter = two_i // 2
        opts = dict(dtype=x.dtype, device=x.device)

        xg = torch.empty(cap, H, **opts)
        ops.permute_rows_cuda(x, row_src, rows_in_use, None, xg, k, inv_row)
        pre = torch.empty(cap, two_i, **opts)
        act = torch.empty(cap, inter, **opts)  # router_weight * swiglu(pre)
        ops.grouped_gemm_cuda(xg, w_fc, padded_offsets, pre, act, row_src, scale, None, N.GEMM_NT, N.EPI_SWIGLU)
        out_rows = torch.empty(cap, H, **opts)
        ops.grouped_gemm_cuda(act, w_proj, padded_offsets, out_rows, None, None, None, None, N.GEMM_NT, N.EPI_STORE)
        y = torch.empty(T, H, **opts)
        ops.combine_rows_cuda(out_rows, inv_row, None, y, k)

        ctx.save_for_backward(xg, pre, act, w_fc, w_proj, scale, padded_offsets, row_src, inv_row, rows_in_use)
        ctx.cap = cap
        ctx.top_k = k
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, pre, act, w_fc, w_proj, scale, padded_offsets, row_src, inv_row, rows_in_use = ctx.saved_tensors
        cap, k = ctx.cap, ctx.top_k
        dy = dy.contiguous()
        T, H = dy.shape
        E, two_i, _ = w_fc.shape
        inter = two_i // 2
        opts = dict(dtype=dy.dtype, device=dy.device)

        dyg = torch.empty(cap, H, **opts)
        ops.permute_rows_cuda(dy, row_src, rows_in_use, None, dyg, k, inv_row)

        # d(pre) = swiglu'(pre) * router_weight * (dy W_proj); the same epilogue writes, per column
        # tile, the partial sums of d(router_weight) = <dy W_proj, swiglu(pre)>, added up in tile
        # order afterwards (deterministic, like the reference's bmm).
        d_pre = torch.empty(cap, two_i, **opts)
        partials = None
        if scale is not None:
            partials = torch.empty(N.gemm_n_tiles(inter), cap, dtype=torch.float32, device=dy.device)
        ops.grouped_gemm_cuda(dyg, w_proj, padded_offsets, d_pre, pre, row_src, scale, partials, N.GEMM_NN, N.EPI_SWIGLU_BWD)
        d_weights = None
        if scale is not None:
            d_router = torch.empty(T * k, dtype=torch.float32, device=dy.device)
            if T * k > 0:
                ops.reduce_row_partials_cuda(partials, row_src, rows_in_use, d_router)
            d_weights = d_router.view(T, k).to(dy.dtype)
        dw_proj = torch.empty_like(w_proj)
        ops.grouped_wgrad_cuda(dyg, act, padded_offsets, dw_proj)
        dw_fc = torch.empty_like(w_fc)
        ops.grouped_wgrad_cuda(d_pre, xg, padded_offsets, dw_fc)

        dxg = dyg  # dyg is dead after the two products above; reuse its storage
        ops.grouped_gemm_cuda(d_pre, w_fc, padded_offsets, dxg, None, None, None, None, N.GEMM_NN, N.EPI_STORE)
        dx = torch.empty(T, H, **opts)
        ops.combine_rows_cuda(dxg, inv_row, None, dx, k)
        return dx, dw_fc, dw_proj, d_weights, None, None, None, None, None, None


def fused_swiglu_experts(x, w_fc, w_proj, router_weights, index: ExpertIndex) -> torch.Tensor:
    """y[t] = sum_j p[t,j] * W_proj[e] swiglu(W_fc[e] x[t]) for e = selected[t,j]; p = 1 when
    `router_weights` is None (expert-parallel ranks scale on the token's home rank instead)."""
    return _FusedSwigluExperts.apply(x, w_fc, w_proj, router_weights, index.padded_offsets, index.row_src,
                                     index.inv_row, index.rows_in_use, index.cap, index.top_k)


class _GatherRows(torch.autograd.Function):
    """rows[p] = x[row_src[p] // k] (the `group` kernel, group_kernel.py:12-100)."""

    @staticmethod
    def forward(ctx, x, row_src, inv_row, rows_in_use, rows: int, k: int):
        x = x.contiguous()
        out = torch.empty(rows, x.size(1), dtype=x.dtype, device=x.device)
        ops.permute_rows_cuda(x, row_src, rows_in_use, None, out, k, inv_row)
        ctx.save_for_backward(inv_row)
        ctx.top_k = k
        ctx.num_tokens = x.size(0)
        return out

    @staticmethod
    def backward(ctx, d_rows):
        (inv_row,) = ctx.saved_tensors
        d_rows = d_rows.contiguous()
        dx = torch.empty(ctx.num_tokens, d_rows.size(1), dtype=d_rows.dtype, device=d_rows.device)
        ops.combine_rows_cuda(d_rows, inv_row, None, dx, ctx.top_k)
        return dx, None, None, None, None, None


class _CombineRows(torch.autograd.Function):
    """y[t] = sum_j w[t,j] * rows[inv_row[t*k+j]] (bmm at triton_implementation/__init__.py:39-43)."""

    @staticmethod
    def forward(ctx, rows, weights, row_src, inv_row, rows_in_use, k: int):
        rows = rows.contiguous()
        weights = weights.contiguous()
        T = weights.size(0)
        y = torch.empty(T, rows.size(1), dtype=rows.dtype, device=rows.device)
        ops.combine_rows_cuda(rows, inv_row, weights.view(-1), y, k)
        ctx.save_for_backward(rows, weights, row_src, inv_row, rows_in_use)
        ctx.top_k = k
        return y

    @staticmethod
    def backward(ctx, dy):
        rows, weights, row_src, inv_row, rows_in_use = ctx.saved_tensors
        k = ctx.top_k
        dy = dy.contiguous()
        d_rows = torch.empty_like(rows)
        ops.permute_rows_cuda(dy, row_src, rows_in_use, weights.view(-1), d_rows, k, inv_row)
        d_weights = torch.empty_like(weights)
        ops.combine_rows_backward_weights_cuda(rows, inv_row, dy, d_weights.view(-1), k)
        return d_rows, d_weights, None, None, None, None


class _GroupedLinear(torch.autograd.Function):
    """rows_out[p] = rows_in[p] @ W[e(p)]^T over rows in padded expert order."""

    @staticmethod
    def forward(ctx, rows, weight, padded_offsets, cap: int):
        _check_dtype(rows, weight)
        rows = rows.contiguous()
        weight = weight.contiguous()
        out = torch.empty(cap, weight.size(1), dtype=rows.dtype, device=rows.device)
        ops.grouped_gemm_cuda(rows, weight, padded_offsets, out, None, None, None, None, N.GEMM_NT, N.EPI_STORE)
        ctx.save_for_backward(rows, weight, padded_offsets)
        return out

    @staticmethod
    def backward(ctx, d_out):
        rows, weight, padded_offsets = ctx.saved_tensors
        d_out = d_out.contiguous()
        d_rows = torch.empty_like(rows)
        ops.grouped_gemm_cuda(d_out, weight, padded_offsets, d_rows, None, None, None, None, N.GEMM_NN, N.EPI_STORE)
        d_weight = torch.empty_like(weight)
        ops.grouped_wgrad_cuda(d_out, rows, padded_offsets, d_weight)
        return d_rows, d_weight, None, None


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
    def forward(ctx, rows, weight, padded_offsets, cap: int):
        rows_s, weight_s = _split(rows), _split(weight)
        out = torch.empty(cap, weight.size(1), dtype=torch.float32, device=rows.device)
        _product_f32(rows_s, weight_s, padded_offsets, out, N.GEMM_NT)
        ctx.save_for_backward(*rows_s, *weight_s, padded_offsets)
        return out

    @staticmethod
    def backward(ctx, d_out):
        r_hi, r_lo, w_hi, w_lo, padded_offsets = ctx.saved_tensors
        d_hi, d_lo = _split(d_out)
        d_rows = torch.empty(r_hi.shape, dtype=torch.float32, device=d_out.device)
        _product_f32((d_hi, d_lo), (w_hi, w_lo), padded_offsets, d_rows, N.GEMM_NN)
        d_weight = torch.empty(w_hi.shape, dtype=torch.float32, device=d_out.device)
        for i, (x, y) in enumerate(((d_hi, r_hi), (d_hi, r_lo), (d_lo, r_hi))):
            ops.grouped_wgrad_f32_cuda(x, y, padded_offsets, d_weight, i > 0)
        return d_rows, d_weight, None, None


def gather_rows(x, index: ExpertIndex, rows: int | None = None) -> torch.Tensor:
    """`rows` limits the output to its first rows (the unpadded order needs exactly T*k of them)."""
    return _GatherRows.apply(x, index.row_src, index.inv_row, index.rows_in_use, index.cap if rows is None else rows,
                             index.top_k)


def combine_rows(rows, weights, index: ExpertIndex) -> torch.Tensor:
    return _CombineRows.apply(rows, weights, index.row_src, index.inv_row, index.rows_in_use, index.top_k)


def grouped_linear(rows, weight, index: ExpertIndex) -> torch.Tensor:
    if rows.dtype == torch.float32 and weight.dtype == torch.float32:
        return _GroupedLinearF32.apply(rows, weight, index.padded_offsets, index.cap)
    return _GroupedLinear.apply(rows, weight, index.padded_offsets, index.cap)
