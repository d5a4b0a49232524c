"""`xma::` custom ops over the C ABI of libxma_b200.so.

Each op mirrors how the reference registers its kernels (xma/custom_op.py:64-90): the caller
allocates outputs, the op mutates them and returns None. The ops pass raw device pointers, sizes
and the current CUDA stream to the library; nothing is computed in Python.
"""

from __future__ import annotations

import torch

from . import _native as N
from .custom_op import xma_op


_index_small_limit: int | None = None


def _kernels_per_call(name: str, args: tuple) -> int:
    """CUDA kernels an entry point launches (memsets are not counted): the index build is one cluster
    launch up to the size the library reports (xma_moe_index_small_limit, at most 256 experts) and
    five launches beyond (csrc/routing.cu:launch_index_build)."""
    global _index_small_limit
    if name == "xma_moe_index_build":
        if _index_small_limit is None:
            _index_small_limit = int(N.lib().xma_moe_index_small_limit())
        n, num_experts = args[2], args[3]
        return 1 if 0 < n <= _index_small_limit and num_experts <= 256 else 5
    return 1


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_entry_points: dict = {}


def _launch(name: str, anchor: torch.Tensor, *args) -> None:
    """Calls one C-ABI entry point on `anchor`'s device and current stream; raises on a non-zero status."""
    if not anchor.is_cuda:
        raise RuntimeError("libxma_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")
    fn = _entry_points.get(name)
    if fn is None:
        fn = _entry_points[name] = getattr(N.lib(), name)
    profiler = N.profiler
    index = anchor.device.index
    if not profiler.enabled and _raw_stream is not None and index == torch.cuda.current_device():
        # The usual case (tensor on the current device, no profiling): no device guard and no stream
        # object, which keeps the host cost of a launch to the ctypes call itself.
        status = fn(*args, _raw_stream(index))
        if status != 0:
            N.check(status, name)
        return
    with torch.cuda.device(anchor.device):
        stream = torch.cuda.current_stream(anchor.device)
        if profiler.enabled:
            profiler.launches += _kernels_per_call(name, args)
            start = torch.cuda.Event(enable_timing=True) if profiler.timing else None
            if start is not None:
                start.record(stream)
            status = fn(*args, stream.cuda_stream)
            if start is not None:
                end = torch.cuda.Event(enable_timing=True)
                end.record(stream)
                profiler.records.append((profiler.label(name, args), start, end))
        else:
            status = fn(*args, stream.cuda_stream)
    N.check(status, name)


@xma_op(mutates_args={"output"})
def continuous_count_cuda(x: torch.Tensor, output: torch.Tensor, E: int) -> None:
    assert x.is_contiguous() and output.is_contiguous()
    _launch("xma_continuous_count", x,
        N.ptr(x), int(x.dtype == torch.int64), x.numel(), N.ptr(output), E,
    )


@xma_op(mutates_args={"topk_weights", "topk_probs", "selected"})
def router_topk_softmax_cuda(
    logits: torch.Tensor, topk_weights: torch.Tensor, topk_probs: torch.Tensor, selected: torch.Tensor, top_k: int
) -> None:
    assert logits.is_contiguous()
    T, E = logits.shape
    _launch("xma_router_topk_softmax", logits,
        N.ptr(logits), N.dtype_code(logits.dtype), T, E, top_k, N.ptr(topk_weights), N.ptr(topk_probs),
        N.ptr(selected),
    )


@xma_op(mutates_args={"logits", "topk_weights", "topk_probs", "selected"})
def router_gate_topk_cuda(
    x: torch.Tensor, w_gate: torch.Tensor, logits: torch.Tensor, topk_weights: torch.Tensor, topk_probs: torch.Tensor,
    selected: torch.Tensor, top_k: int
) -> None:
    """logits = x @ w_gate^T with top-k and softmax in the epilogue; see xma_router_gate_topk in include/xma_b200.h."""
    assert x.is_contiguous() and w_gate.is_contiguous() and x.dtype == w_gate.dtype
    T, H = x.shape
    _launch("xma_router_gate_topk", x,
        N.dtype_code(x.dtype), N.ptr(x), N.ptr(w_gate), T, H, w_gate.size(0), top_k, N.ptr(logits), N.ptr(topk_weights),
        N.ptr(topk_probs), N.ptr(selected), N.ptr(N.status_word(x.device)),
    )


@xma_op(mutates_args={"d_logits"})
def router_topk_softmax_backward_cuda(
    d_weights: torch.Tensor, topk_probs: torch.Tensor, selected: torch.Tensor, d_logits: torch.Tensor, top_k: int
) -> None:
    T, E = d_logits.shape
    _launch("xma_router_topk_softmax_backward", d_logits,
        N.ptr(d_weights), N.dtype_code(d_logits.dtype), N.ptr(topk_probs), N.ptr(selected), T, E, top_k,
        N.ptr(d_logits),
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
    tile_expert: torch.Tensor | None,
    workspace: torch.Tensor,
    num_experts: int,
    block_m: int,
) -> None:
    assert ids.is_contiguous() and ids.dtype in (torch.int32, torch.int64)
    _launch("xma_moe_index_build", ids,
        N.ptr(ids), int(ids.dtype == torch.int64), ids.numel(), num_experts, N.ptr(expert_frequency),
        N.ptr(expert_offsets), N.ptr(sorted_expert_idxs), N.ptr(sorted_scattered_idxs), N.ptr(padded_offsets),
        N.ptr(row_src), N.ptr(inv_row), N.ptr(tile_expert), block_m, N.ptr(workspace),
    )


@xma_op(mutates_args={"dst"})
def permute_rows_cuda(
    src: torch.Tensor,
    row_src: torch.Tensor,
    rows_in_use: torch.Tensor | None,
    coeff: torch.Tensor | None,
    dst: torch.Tensor,
    fan_out: int,
    inv_row: torch.Tensor | None = None,
) -> None:
    assert src.is_contiguous() and dst.is_contiguous()
    _launch("xma_permute_rows", src,
        N.ptr(src), N.dtype_code(src.dtype), src.size(-1), N.ptr(row_src), N.ptr(inv_row), N.ptr(rows_in_use),
        dst.size(0), src.size(0),
        fan_out, N.ptr(coeff), N.ptr(dst),
    )


@xma_op(mutates_args={"out"})
def combine_rows_cuda(
    rows: torch.Tensor, inv_row: torch.Tensor, weights: torch.Tensor | None, out: torch.Tensor, top_k: int
) -> None:
    assert rows.is_contiguous() and out.is_contiguous()
    _launch("xma_combine_rows", rows,
        N.ptr(rows), N.dtype_code(rows.dtype), rows.size(-1), N.ptr(inv_row), N.ptr(weights), out.size(0),
        top_k, N.ptr(out),
    )


@xma_op(mutates_args={"d_weights"})
def combine_rows_backward_weights_cuda(
    rows: torch.Tensor, inv_row: torch.Tensor, d_out: torch.Tensor, d_weights: torch.Tensor, top_k: int
) -> None:
    assert rows.is_contiguous() and d_out.is_contiguous()
    _launch("xma_combine_rows_backward_weights", rows,
        N.ptr(rows), N.dtype_code(rows.dtype), rows.size(-1), N.ptr(inv_row), N.ptr(d_out), d_out.size(0),
        top_k, N.ptr(d_weights),
    )


@xma_op(mutates_args={"c", "aux", "d_row_scale"})
def grouped_gemm_cuda(
    a: torch.Tensor,
    w: torch.Tensor,
    padded_offsets: torch.Tensor,
    c: torch.Tensor,
    aux: torch.Tensor | None,
    row_src: torch.Tensor | None,
    row_scale: torch.Tensor | None,
    d_row_scale: torch.Tensor | None,
    layout: int,
    epilogue: int,
) -> None:
    """c = grouped a @ w[e] with the epilogue fused; see xma_grouped_gemm in include/xma_b200.h."""
    assert a.is_contiguous() and w.is_contiguous() and c.is_contiguous() and w.dim() == 3
    cap, k = a.shape
    num_experts = w.size(0)
    n = w.size(1) if layout == N.GEMM_NT else w.size(2)
    assert (w.size(2) if layout == N.GEMM_NT else w.size(1)) == k
    _launch("xma_grouped_gemm", a,
        layout, epilogue, N.dtype_code(a.dtype), N.ptr(a), N.ptr(w), N.ptr(padded_offsets), cap, num_experts, n,
        k, N.ptr(c), N.ptr(aux), N.ptr(row_src), N.ptr(row_scale), N.ptr(d_row_scale), N.ptr(N.status_word(a.device)),
    )


@xma_op(mutates_args={"out"})
def reduce_row_partials_cuda(
    partials: torch.Tensor, row_src: torch.Tensor, rows_in_use: torch.Tensor | None, out: torch.Tensor
) -> None:
    """out[row_src[r]] = sum_j partials[j, r], j ascending; see xma_reduce_row_partials in include/xma_b200.h."""
    assert partials.is_contiguous() and partials.dtype == torch.float32 and out.dtype == torch.float32
    _launch("xma_reduce_row_partials", partials,
        N.ptr(partials), partials.size(0), partials.size(1), N.ptr(row_src), N.ptr(rows_in_use), N.ptr(out),
    )


@xma_op(mutates_args={"dw"})
def grouped_wgrad_cuda(
    x: torch.Tensor, y: torch.Tensor, padded_offsets: torch.Tensor, dw: torch.Tensor
) -> None:
    """dw[e] = x_e^T @ y_e over the rows of expert e; see xma_grouped_wgrad in include/xma_b200.h."""
    assert x.is_contiguous() and y.is_contiguous() and dw.is_contiguous()
    cap, m = x.shape
    n = y.size(1)
    _launch("xma_grouped_wgrad", x,
        N.dtype_code(x.dtype), N.ptr(x), N.ptr(y), N.ptr(padded_offsets), cap, dw.size(0), m, n, N.ptr(dw),
        N.ptr(N.status_word(x.device)),
    )


@xma_op(mutates_args={"dw"})
def grouped_wgrad_f32_cuda(
    x: torch.Tensor, y: torch.Tensor, padded_offsets: torch.Tensor, dw: torch.Tensor, accumulate: bool
) -> None:
    """float32 dw[e] (+)= x_e^T @ y_e; see xma_grouped_wgrad_f32 in include/xma_b200.h."""
    assert x.is_contiguous() and y.is_contiguous() and dw.is_contiguous() and dw.dtype == torch.float32
    cap, m = x.shape
    n = y.size(1)
    _launch("xma_grouped_wgrad_f32", x,
        N.dtype_code(x.dtype), N.ptr(x), N.ptr(y), N.ptr(padded_offsets), cap, dw.size(0), m, n, N.ptr(dw),
        int(accumulate), N.ptr(N.status_word(x.device)),
    )


@xma_op(mutates_args={"out"})
def sum_partials_cuda(partials: torch.Tensor, out: torch.Tensor) -> None:
    """out = partials.sum(0) in float32, rounded to out.dtype; see xma_sum_partials in include/xma_b200.h."""
    assert partials.is_contiguous() and out.is_contiguous() and partials.dtype == torch.float32
    _launch("xma_sum_partials", partials, N.ptr(partials), partials.size(0), out.numel(), N.dtype_code(out.dtype), N.ptr(out))


@xma_op(mutates_args={"hi", "lo"})
def split_f32_cuda(src: torch.Tensor, hi: torch.Tensor, lo: torch.Tensor) -> None:
    """hi = bf16(src), lo = bf16(src - hi); see xma_split_f32 in include/xma_b200.h."""
    assert src.is_contiguous() and src.dtype == torch.float32 and hi.dtype == torch.bfloat16 and lo.dtype == torch.bfloat16
    _launch("xma_split_f32", src, N.ptr(src), src.numel(), N.ptr(hi), N.ptr(lo))


@xma_op(mutates_args={"y"})
def swiglu_packed_forward_cuda(x: torch.Tensor, y: torch.Tensor) -> None:
    rows, half = y.numel() // y.size(-1), y.size(-1)
    _launch("xma_swiglu_packed_forward", x,
        N.ptr(x), N.dtype_code(x.dtype), rows, half, N.ptr(y),
    )


@xma_op(mutates_args={"dx"})
def swiglu_packed_backward_cuda(x: torch.Tensor, dy: torch.Tensor, dx: torch.Tensor) -> None:
    rows, half = dy.numel() // dy.size(-1), dy.size(-1)
    _launch("xma_swiglu_packed_backward", x,
        N.ptr(x), N.ptr(dy), N.dtype_code(x.dtype), rows, half, N.ptr(dx),
    )


@xma_op(mutates_args={"y"})
def swiglu_forward_cuda(gate: torch.Tensor, up: torch.Tensor, y: torch.Tensor) -> None:
    _launch("xma_swiglu_forward", gate, N.ptr(gate), N.ptr(up), N.dtype_code(gate.dtype), gate.numel(), N.ptr(y))


@xma_op(mutates_args={"dgate", "dup"})
def swiglu_backward_cuda(
    gate: torch.Tensor, up: torch.Tensor, dy: torch.Tensor, dgate: torch.Tensor, dup: torch.Tensor
) -> None:
    _launch("xma_swiglu_backward", gate, N.ptr(gate), N.ptr(up), N.ptr(dy), N.dtype_code(gate.dtype), gate.numel(),
            N.ptr(dgate), N.ptr(dup))


@xma_op(mutates_args={"output"})
def pack_unpack_sequence_cuda(
    x: torch.Tensor, output: torch.Tensor, cu_seqlens: torch.Tensor, padding_side: str, pack: bool
) -> None:
    """pack: output[token] = x[b, s]; unpack: output[b, s] = x[token], zeros on padding (same argument
    order as the reference's pack_unpack_sequence_cuda, kernel.cu:67-132)."""
    assert x.is_contiguous() and output.is_contiguous() and cu_seqlens.is_contiguous()
    assert cu_seqlens.dtype in (torch.int32, torch.int64, torch.uint32)
    padded = x if pack else output
    batch, seq = padded.size(0), padded.size(1)
    row_bytes = padded[0, 0].numel() * padded.element_size()
    _launch(
        "xma_pack_sequence" if pack else "xma_unpack_sequence", output,
        N.ptr(x), N.ptr(cu_seqlens), int(cu_seqlens.dtype == torch.int64), batch, seq, row_bytes,
        int(padding_side == "left"), N.ptr(output),
    )
