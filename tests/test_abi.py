"""The C-ABI library loads without a GPU and exports every symbol include/xma_b200.h declares."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xma_b200.h")


def declared_symbols() -> list[str]:
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(xma_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    for must in ("xma_continuous_count", "xma_moe_index_build", "xma_grouped_gemm", "xma_grouped_wgrad",
                 "xma_permute_rows", "xma_combine_rows", "xma_router_topk_softmax"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from xma import _native as N

    handle = ctypes.CDLL(N.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(handle, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header():
    from xma import _native as N

    assert sorted(N.exported_symbols()) == declared_symbols()


def test_host_only_entry_points():
    from xma import _native as N

    lib = N.lib()
    assert lib.xma_abi_version() >= 1
    assert lib.xma_status_string(0) == b"ok"
    assert b"unknown" in lib.xma_status_string(77)
    assert b"CUDA runtime error 2" in lib.xma_status_string(1002)
    for n, e in ((0, 1), (1, 8), (128, 8), (129, 8), (65536, 64), (262144, 256)):
        cap = lib.xma_padded_capacity(n, e, N.XMA_BLOCK_M)
        assert cap == N.padded_capacity(n, e)
        assert lib.xma_padded_capacity(n, e, 1) == N.padded_capacity(n, e, 1) == max(n, 0) + e
        assert cap % N.XMA_BLOCK_M == 0 and cap >= n + e * (N.XMA_BLOCK_M - 1) - (N.XMA_BLOCK_M - 1)
    for n in (0, 1, 31, 1024, 1025, 65536, 262144, (1 << 20) + 7, 1 << 24):
        for e in (1, 8, 256):
            assert lib.xma_moe_index_workspace_bytes(n, e) == 4 * N.index_workspace_elems(n, e)


def test_bad_arguments_are_rejected_without_touching_a_gpu():
    from xma import _native as N

    lib = N.lib()
    assert lib.xma_continuous_count(None, 0, 10, None, 8, None) == 1  # XMA_ERR_BAD_ARG
    assert lib.xma_continuous_count(None, 0, 0, None, 0, None) == 1
    assert lib.xma_router_topk_softmax(None, 0, 4, 8, 9, None, None, None, None) == 2  # k > E: unsupported
    assert lib.xma_router_topk_softmax(None, 0, 4, 4096, 2, None, None, None, None) == 2
    assert lib.xma_grouped_gemm(0, 0, 0, None, None, None, 128, 1, 256, 64, None, None, None, None, None, None, None) == 1
    assert lib.xma_permute_rows(None, 0, 64, None, None, None, 128, 16, 1, None, None, None) == 1
    assert lib.xma_permute_rows(None, 0, 64, None, None, None, 0, 0, 1, None, None, None) == 0  # nothing to do
    with pytest.raises(RuntimeError, match="bad argument"):
        N.check(1, "probe")


def test_new_entry_points_reject_bad_arguments_on_the_host():
    """Argument checks of the router front end, the float32 products, the split, the unpacked swiglu:
    all answered before anything is launched (no GPU needed)."""
    from xma import _native as N

    lib = N.lib()
    BAD, UNSUPPORTED = 1, 2
    # router front end: E must be a multiple of 8 and at most 256, k at most 8 and at most E, H % 8 == 0
    args = lambda T, H, E, k, dt=0: (dt, None, None, T, H, E, k, None, None, None, None, None, None)
    assert lib.xma_router_gate_topk(*args(16, 64, 12, 2)) == UNSUPPORTED
    assert lib.xma_router_gate_topk(*args(16, 64, 264, 2)) == UNSUPPORTED
    assert lib.xma_router_gate_topk(*args(16, 64, 64, 9)) == UNSUPPORTED
    assert lib.xma_router_gate_topk(*args(16, 60, 64, 2)) == UNSUPPORTED
    assert lib.xma_router_gate_topk(*args(16, 64, 64, 2, 2)) == UNSUPPORTED  # float32 operands
    assert lib.xma_router_gate_topk(*args(-1, 64, 64, 2)) == BAD
    assert lib.xma_router_gate_topk(*args(0, 64, 64, 2)) == 0  # no tokens: nothing to do
    assert lib.xma_router_gate_topk(*args(16, 64, 64, 2)) == BAD  # null pointers
    # float32 epilogues are accepted codes; anything else is not
    gemm = lambda epi: lib.xma_grouped_gemm(0, epi, 0, None, None, None, 128, 1, 256, 64, None, None, None, None, None,
                                            None, None)
    assert gemm(3) == BAD and gemm(4) == BAD  # null pointers, but a known epilogue
    assert lib.xma_grouped_wgrad_f32(0, None, None, None, 128, 1, 64, 64, None, 0, None, None) == BAD
    assert lib.xma_split_f32(None, 0, None, None, None) == 0
    assert lib.xma_split_f32(None, 16, None, None, None) == BAD
    assert lib.xma_swiglu_forward(None, None, 0, 0, None, None) == 0
    assert lib.xma_swiglu_forward(None, None, 0, 8, None, None) == BAD
    assert lib.xma_swiglu_backward(None, None, None, 0, -1, None, None, None) == BAD
    # index build: sizes whose padded capacity would not fit 32-bit row numbers are refused
    assert lib.xma_moe_index_build(None, 0, (1 << 31) - 64, 8, None, None, None, None, None, None, None, None, 128, None,
                                   None) == UNSUPPORTED
