"""ctypes binding of libxma_b200.so (C ABI declared in include/xma_b200.h).

There is no fallback: if the library is missing or a call returns a non-zero status, a
RuntimeError is raised.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_int32, c_int64, c_void_p

import torch

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# XMA_B200_LIB points at another build of the same library (profiling and experiments).
LIB_PATH = os.environ.get("XMA_B200_LIB") or os.path.join(_PKG_ROOT, "libxma_b200.so")

XMA_BLOCK_M = 128
XMA_BLOCK_N = 256
EPI_STORE, EPI_SWIGLU, EPI_SWIGLU_BWD, EPI_STORE_F32, EPI_ADD_F32 = 0, 1, 2, 3, 4
GEMM_NT, GEMM_NN = 0, 1

_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}

# name -> (restype, argtypes); must list every symbol include/xma_b200.h declares.
_SIGNATURES = {
    "xma_status_string": (ctypes.c_char_p, [c_int32]),
    "xma_abi_version": (c_int32, []),
    "xma_padded_capacity": (c_int64, [c_int64, c_int32, c_int32]),
    "xma_moe_index_workspace_bytes": (c_int64, [c_int64, c_int32]),
    "xma_moe_index_small_limit": (c_int64, []),
    "xma_continuous_count": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_int32, c_void_p]),
    "xma_router_topk_softmax": (
        c_int32, [c_void_p, c_int32, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p]),
    "xma_router_topk_softmax_backward": (
        c_int32, [c_void_p, c_int32, c_void_p, c_void_p, c_int64, c_int32, c_int32, c_void_p, c_void_p]),
    "xma_moe_index_build": (
        c_int32, [c_void_p, c_int32, c_int64, c_int32] + [c_void_p] * 8 + [c_int32, c_void_p, c_void_p]),
    "xma_moe_index_build_static": (
        c_int32, [c_void_p, c_int32, c_int64, c_int32] + [c_void_p] * 8 + [c_int32, c_void_p]),
    "xma_moe_index_static_scratch_bytes": (c_int64, []),
    "xma_permute_rows": (
        c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_void_p,
                  c_void_p, c_void_p]),
    "xma_combine_rows": (
        c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "xma_combine_rows_backward_weights": (
        c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_void_p]),
    "xma_grouped_gemm": (
        c_int32, [c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int64]
        + [c_void_p] * 7),
    "xma_swiglu_packed_forward": (c_int32, [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_void_p]),
    "xma_swiglu_packed_backward": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_void_p, c_void_p]),
    "xma_swiglu_forward": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p]),
    "xma_swiglu_backward": (c_int32, [c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p]),
    "xma_pack_sequence": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p]),
    "xma_unpack_sequence": (c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int64, c_int64, c_int32, c_void_p, c_void_p]),
    "xma_ipc_get_handle": (c_int32, [c_void_p, ctypes.c_char_p]),
    "xma_ipc_open_handle": (c_int32, [ctypes.c_char_p, ctypes.POINTER(c_void_p)]),
    "xma_ipc_close_handle": (c_int32, [c_void_p]),
    "xma_ep_barrier": (c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int64, c_void_p, c_void_p]),
    "xma_ep_exchange_counts": (
        c_int32, [c_void_p, c_int32, c_int32, c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int64, c_void_p, c_void_p]),
    "xma_ep_plan": (
        c_int32, [c_void_p, c_int32, c_int32, c_int32, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "xma_ep_prepare_rows": (
        c_int32, [c_void_p, c_void_p, c_int32, c_int64, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "xma_ep_dispatch_rows": (
        c_int32, [c_void_p, c_int32, c_int64, c_int64, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int32, c_int64, c_void_p, c_void_p]),
    "xma_ep_combine_pull": (
        c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_int64, c_int32, c_void_p, c_int64, c_void_p]),
    "xma_ep_pull_scalars": (c_int32, [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_int64, c_void_p]),
    "xma_reduce_row_partials": (c_int32, [c_void_p, c_int32, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "xma_selftest_bounded_wait": (c_int32, [c_void_p, c_int64, c_void_p]),
    "xma_sum_partials": (c_int32, [c_void_p, c_int32, c_int64, c_int32, c_void_p, c_void_p]),
    "xma_grouped_wgrad": (
        c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "xma_grouped_wgrad_f32": (
        c_int32, [c_int32, c_void_p, c_void_p, c_void_p, c_int64, c_int32, c_int64, c_int64, c_void_p, c_int32, c_void_p,
                  c_void_p]),
    "xma_split_f32": (c_int32, [c_void_p, c_int64, c_void_p, c_void_p, c_void_p]),
    "xma_router_gate_topk": (
        c_int32, [c_int32, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p,
                  c_void_p, c_void_p]),
}

_lib = None


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python flash-model-architectures_b200/build.py` "
                "(there is no fallback path)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        message = lib().xma_status_string(status).decode()
        raise RuntimeError(f"{what} failed: {message} (xma_status {status})")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise RuntimeError(f"dtype {dtype} is not supported by libxma_b200") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def padded_capacity(n: int, num_experts: int, block_m: int = XMA_BLOCK_M) -> int:
    return (-(-max(n, 0) // block_m) + num_experts) * block_m


def gemm_n_tiles(n: int) -> int:
    """Column tiles of the grouped GEMM over n output columns (rows of the d_row_scale partials)."""
    return -(-n // XMA_BLOCK_N)


def index_workspace_elems(n: int, num_experts: int) -> int:
    """int32 elements of workspace xma_moe_index_build needs; the same arithmetic as
    xma_moe_index_workspace_bytes (csrc/routing.cu:index_plan), kept in Python so that building an
    index does not call into ctypes while torch.compile traces the layer."""
    segs = min(max(-(-n // 1024), 1), 8192)
    seg_len = -(-(-(-max(n, 1) // segs)) // 32) * 32
    segs = -(-n // seg_len) if n > 0 else 1
    return 2 * segs * num_experts + 64


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """int32 word the GEMM kernels write when one of their bounded waits runs out."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _status_words.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _status_words[index] = word
    return word


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if a kernel reported a device-side timeout since the last check."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = status_word(device)
    code = int(word.item())
    if code != 0:
        word.zero_()
        raise RuntimeError(f"libxma_b200: bounded device-side wait ran out (code {code})")


class _Profiler:
    """Opt-in launch counter and per-call CUDA-event timer used by bench.py.

    While `enabled`, every C-ABI call adds the number of kernels it launches to `launches`; with
    `timing` it is also bracketed by two events on the launching stream."""

    def __init__(self) -> None:
        self.enabled = False
        self.timing = False
        self.launches = 0
        self.records: list = []
        self.prefix = ""  # prepended to the labels of calls made while a caller sets it (e.g. "router_")

    def start(self, timing: bool = False) -> None:
        self.enabled, self.timing, self.launches, self.records = True, timing, 0, []

    def stop(self) -> None:
        self.enabled = False

    def label(self, name: str, args: tuple) -> str:
        if name == "xma_grouped_gemm":
            layout, epilogue = args[0], args[1]
            return f"{self.prefix}grouped_gemm[{'NT' if layout == GEMM_NT else 'NN'},{('store', 'swiglu', 'swiglu_bwd', 'store_f32', 'add_f32')[epilogue]}]"
        return self.prefix + name[4:]

    def summary(self) -> dict[str, tuple[int, float]]:
        """label -> (calls, total milliseconds); call after a device synchronize."""
        out: dict[str, list] = {}
        for label, start, end in self.records:
            rec = out.setdefault(label, [0, 0.0])
            rec[0] += 1
            rec[1] += start.elapsed_time(end)
        return {k: (v[0], v[1]) for k, v in out.items()}


profiler = _Profiler()
