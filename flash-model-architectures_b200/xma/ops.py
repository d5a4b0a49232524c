"""`xma::` custom ops over the C ABI of libxma_b200.so.

Each op mirrors how the reference registers its kernels (xma/custom_op.py:64-90): the caller
allocates outputs, the op mutates them and returns None. The ops pass raw device pointers, sizes
and the current CUDA stream to the library; nothing is computed in Python.
"""

from __future__ import annotations

import torch

from . import _native as N
from .custom_op import xma_op


def _on_device(t: torch.Tensor):
    return torch.cuda.device(t.device)


@xma_op(mutates_args={"output"})
def continuous_count_cuda(x: torch.Tensor, output: torch.Tensor, E: int) -> None:
    assert x.is_cuda and x.is_contiguous() and output.is_contiguous()
    with _on_device(x):
        N.check(
            N.lib().xma_continuous_count(
                N.ptr(x), int(x.dtype == torch.int64), x.numel(), N.ptr(output), E, N.stream_ptr(x.device)
            ),
            "xma_continuous_count",
        )


@xma_op(mutates_args={"topk_weights", "topk_probs", "selected"})
def router_topk_softmax_cuda(
    logits: torch.Tensor, topk_weights: torch.Tensor, topk_probs: torch.Tensor, selected: torch.Tensor, top_k: int
) -> None:
    assert logits.is_cuda and logits.is_contiguous()
    T, E = logits.shape
    with _on_device(logits):
        N.check(
            N.lib().xma_router_topk_softmax(
                N.ptr(logits), N.dtype_code(logits.dtype), T, E, top_k, N.ptr(topk_weights), N.ptr(topk_probs),
                N.ptr(selected), N.stream_ptr(logits.device),
            ),
            "xma_router_topk_softmax",
        )


@xma_op(mutates_args={"d_logits"})
def router_topk_softmax_backward_cuda(
    d_weights: torch.Tensor, topk_probs: torch.Tensor, selected: torch.Tensor, d_logits: torch.Tensor, top_k: int
) -> None:
    T, E = d_logits.shape
    with _on_device(d_logits):
        N.check(
            N.lib().xma_router_topk_softmax_backward(
                N.ptr(d_weights), N.dtype_code(d_logits.dtype), N.ptr(topk_probs), N.ptr(selected), T, E, top_k,
                N.ptr(d_logits), N.stream_ptr(d_logits.device),
            ),
            "xma_router_topk_softmax_backward",
        )


@xma_op(
    mutates_args={
        "expert_frequency", "expert_offsets", "sorted_expert_idxs", "sorted_scattered_idxs", "padded_offsets",
        "row_src", "inv_row", "tile_expert", "workspace",
    }
)
def moe_index_build_cuda(
    ids: torch.Tensor,
    expert_frequency: torch.Tensor,
    expert_offsets: torch.Tensor,
    sorted_expert_idxs: torch.Tensor,
    sorted_scattered_idxs: torch.Tensor,
    padded_offsets: torch.Tensor,
    row_src: torch.Tensor,
    inv_row: torch.Tensor,
    tile_expert: torch.Tensor,
    workspace: torch.Tensor,
    num_experts: int,
) -> None:
    assert ids.is_cuda and ids.is_contiguous() and ids.dtype in (torch.int32, torch.int64)
    with _on_device(ids):
        N.check(
            N.lib().xma_moe_index_build(
                N.ptr(ids), int(ids.dtype == torch.int64), ids.numel(), num_experts, N.ptr(expert_frequency),
                N.ptr(expert_offsets), N.ptr(sorted_expert_idxs), N.ptr(sorted_scattered_idxs), N.ptr(padded_offsets),
                N.ptr(row_src), N.ptr(inv_row), N.ptr(tile_expert), N.ptr(workspace), N.stream_ptr(ids.device),
            ),
            "xma_moe_index_build",
        )


@xma_op(mutates_args={"dst"})
def permute_rows_cuda(
    src: torch.Tensor,
    row_src: torch.Tensor,
    tile_expert: torch.Tensor,
    coeff: torch.Tensor | None,
    dst: torch.Tensor,
    fan_out: int,
) -> None:
    assert src.is_contiguous() and dst.is_contiguous()
    with _on_device(src):
        N.check(
            N.lib().xma_permute_rows(
                N.ptr(src), N.dtype_code(src.dtype), src.size(-1), N.ptr(row_src), N.ptr(tile_expert), dst.size(0),
                fan_out, N.ptr(coeff), N.ptr(dst), N.stream_ptr(src.device),
            ),
            "xma_permute_rows",
        )


@xma_op(mutates_args={"out"})
def combine_rows_cuda(
    rows: torch.Tensor, inv_row: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor, top_k: int
) -> None:
    assert rows.is_contiguous() and out.is_contiguous()
    with _on_device(rows):
        N.check(
            N.lib().xma_combine_rows(
                N.ptr(rows), N.dtype_code(rows.dtype), rows.size(-1), N.ptr(inv_row), N.ptr(weights), out.size(0),
                top_k, N.ptr(out), N.stream_ptr(rows.device),
            ),
            "xma_combine_rows",
        )


@xma_op(mutates_args={"d_weights"})
def combine_rows_backward_weights_cuda(
    rows: torch.Tensor, inv_row: torch.Tensor, d_out: torch.Tensor, d_weights: torch.Tensor, top_k: int
) -> None:
    assert rows.is_contiguous() and d_out.is_contiguous()
    with _on_device(rows):
        N.check(
            N.lib().xma_combine_rows_backward_weights(
                N.ptr(rows), N.dtype_code(rows.dtype), rows.size(-1), N.ptr(inv_row), N.ptr(d_out), d_out.size(0),
                top_k, N.ptr(d_weights), N.stream_ptr(rows.device),
            ),
            "xma_combine_rows_backward_weights",
        )


@xma_op(mutates_args={"c", "aux", "d_row_scale", "status"})
def grouped_gemm_cuda(
    a: torch.Tensor,
    w: torch.Tensor,
    tile_expert: torch.Tensor,
    c: torch.Tensor,
    aux: torch.Tensor | None,
    row_src: torch.Tensor | None,
    row_scale: torch.Tensor | None,
    d_row_scale: torch.Tensor | None,
    status: torch.Tensor,
    layout: int,
    epilogue: int,
) -> None:
    """c = grouped a @ w[e] with the epilogue fused; see xma_grouped_gemm in include/xma_b200.h."""
    assert a.is_contiguous() and w.is_contiguous() and c.is_contiguous() and w.dim() == 3
    cap, k = a.shape
    num_experts = w.size(0)
    n = w.size(1) if layout == N.GEMM_NT else w.size(2)
    assert (w.size(2) if layout == N.GEMM_NT else w.size(1)) == k
    with _on_device(a):
        N.check(
            N.lib().xma_grouped_gemm(
                layout, epilogue, N.dtype_code(a.dtype), N.ptr(a), N.ptr(w), N.ptr(tile_expert), cap, num_experts, n,
                k, N.ptr(c), N.ptr(aux), N.ptr(row_src), N.ptr(row_scale), N.ptr(d_row_scale), N.ptr(status),
                N.stream_ptr(a.device),
            ),
            "xma_grouped_gemm",
        )


@xma_op(mutates_args={"dw", "status"})
def grouped_wgrad_cuda(
    x: torch.Tensor, y: torch.Tensor, padded_offsets: torch.Tensor, dw: torch.Tensor, status: torch.Tensor
) -> None:
    """dw[e] = x_e^T @ y_e over the rows of expert e; see xma_grouped_wgrad in include/xma_b200.h."""
    assert x.is_contiguous() and y.is_contiguous() and dw.is_contiguous()
    cap, m = x.shape
    n = y.size(1)
    with _on_device(x):
        N.check(
            N.lib().xma_grouped_wgrad(
                N.dtype_code(x.dtype), N.ptr(x), N.ptr(y), N.ptr(padded_offsets), cap, dw.size(0), m, n, N.ptr(dw),
                N.ptr(status), N.stream_ptr(x.device),
            ),
            "xma_grouped_wgrad",
        )


@xma_op(mutates_args={"y"})
def swiglu_packed_forward_cuda(x: torch.Tensor, y: torch.Tensor) -> None:
    rows, half = y.numel() // y.size(-1), y.size(-1)
    with _on_device(x):
        N.check(
            N.lib().xma_swiglu_packed_forward(
                N.ptr(x), N.dtype_code(x.dtype), rows, half, N.ptr(y), N.stream_ptr(x.device)
            ),
            "xma_swiglu_packed_forward",
        )


@xma_op(mutates_args={"dx"})
def swiglu_packed_backward_cuda(x: torch.Tensor, dy: torch.Tensor, dx: torch.Tensor) -> None:
    rows, half = dy.numel() // dy.size(-1), dy.size(-1)
    with _on_device(x):
        N.check(
            N.lib().xma_swiglu_packed_backward(
                N.ptr(x), N.ptr(dy), N.dtype_code(x.dtype), rows, half, N.ptr(dx), N.stream_ptr(x.device)
            ),
            "xma_swiglu_packed_backward",
        )
