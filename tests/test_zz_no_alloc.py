"""The allocation-free index build (`xma_moe_index_build_static`) against the regular entry point.

Some hosts of the library cannot allocate device memory when they call it (a frozen memory pool, a
call site where the allocator must not be entered). For them the counting sort's scratch lives in
a fixed array inside the library. This test calls the entry point straight through the C ABI, twice
in a row with different problems, and requires bit-identical outputs to `xma_moe_index_build`
(integer work: no tolerance). Both problems are large enough to take the multi-kernel path that uses
the built-in array, and the second is smaller than the first, so stale scratch left by the first call
would show if it mattered. The file name makes pytest collect it last.
"""

import pytest
import torch

from xma import _native as N

pytestmark = pytest.mark.gpu

OUTPUTS = ("expert_frequency", "expert_offsets", "sorted_expert_idxs", "sorted_scattered_idxs", "padded_offsets",
           "row_src", "inv_row", "tile_expert")


def _buffers(n: int, num_experts: int, block_m: int, device) -> dict[str, torch.Tensor]:
    cap = N.padded_capacity(n, num_experts, block_m)
    i32 = dict(dtype=torch.int32, device=device)
    return {
        "expert_frequency": torch.full((num_experts,), -7, **i32),
        "expert_offsets": torch.full((num_experts,), -7, **i32),
        "sorted_expert_idxs": torch.full((n,), -7, **i32),
        "sorted_scattered_idxs": torch.full((n,), -7, **i32),
        "padded_offsets": torch.full((num_experts + 1,), -7, **i32),
        "row_src": torch.full((cap,), -7, **i32),
        "inv_row": torch.full((n,), -7, **i32),
        "tile_expert": torch.full((cap // block_m + 1,), -7, **i32),
    }


def _run(static: bool, ids: torch.Tensor, num_experts: int, block_m: int) -> dict[str, torch.Tensor]:
    lib = N.lib()
    out = _buffers(ids.numel(), num_experts, block_m, ids.device)
    stream = torch.cuda.current_stream(ids.device).cuda_stream
    head = (ids.data_ptr(), int(ids.dtype == torch.int64), ids.numel(), num_experts)
    ptrs = tuple(out[name].data_ptr() for name in OUTPUTS)
    if static:
        status = lib.xma_moe_index_build_static(*head, *ptrs, block_m, stream)
    else:
        workspace = torch.empty(N.index_workspace_elems(ids.numel(), num_experts), dtype=torch.int32, device=ids.device)
        status = lib.xma_moe_index_build(*head, *ptrs, block_m, workspace.data_ptr(), stream)
    N.check(status, "index build")
    torch.cuda.synchronize(ids.device)
    return out


def test_static_scratch_index_build_matches_regular_entry_point(device):
    assert N.lib().xma_moe_index_static_scratch_bytes() == 4 << 20
    g = torch.Generator().manual_seed(11)
    problems = [  # two calls in a row; the second is smaller and uses other ids, dtype and expert count
        (torch.randint(0, 64, (700000,), generator=g, dtype=torch.int64), 64, N.XMA_BLOCK_M),
        (torch.randint(0, 6, (560000,), generator=g, dtype=torch.int32), 6, N.XMA_BLOCK_M),
    ]
    side = torch.cuda.Stream(device)
    for i, (ids, num_experts, block_m) in enumerate(problems):
        ids = ids.to(device)
        assert ids.numel() > N.lib().xma_moe_index_small_limit()  # beyond the one-block form, which needs no scratch
        if i == 1:  # the second call on another stream, ordered after the first
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                got = _run(True, ids, num_experts, block_m)
            torch.cuda.current_stream(device).wait_stream(side)
        else:
            got = _run(True, ids, num_experts, block_m)
        want = _run(False, ids, num_experts, block_m)
        for name in OUTPUTS:
            assert torch.equal(got[name], want[name]), name
        assert int(got["expert_frequency"].sum()) == ids.numel()


def test_static_scratch_rejects_oversized_problems(device):
    lib = N.lib()
    n, num_experts = 1 << 24, 1024  # needs 2 * 8192 * 1024 counters = 64 MiB of scratch
    assert lib.xma_moe_index_workspace_bytes(n, num_experts) > lib.xma_moe_index_static_scratch_bytes()
    status = lib.xma_moe_index_build_static(None, 0, n, num_experts, *([None] * 8), N.XMA_BLOCK_M, None)
    assert status == 6  # XMA_ERR_SCRATCH_TOO_SMALL, decided from the sizes before anything is launched
    with pytest.raises(RuntimeError, match="built-in buffer"):
        N.check(status, "xma_moe_index_build_static")
