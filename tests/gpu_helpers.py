"""Shared helpers of the GPU parity tests."""

from __future__ import annotations

import torch

from oracle import moe_oracle as O
from xma import _native as N
from xma.layers.moe.routing import ExpertIndex


def make_selection(T: int, E: int, k: int, device, skew: bool = False, dtype=torch.int64, seed: int = 0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits = logits + torch.linspace(4, -8, E)  # the last experts receive no rows
    return logits.topk(k, -1).indices.to(dtype).to(device)


def expected_padded_order(selected: torch.Tensor, E: int, cap: int, block_m: int = N.XMA_BLOCK_M):
    """The padded expert order derived from the oracle's stable sort, all int64 on the device."""
    dev = selected.device
    k = selected.size(1)
    se, ss, freq, off = O.sort_experts(selected.long(), E)
    f = freq.long()
    padded = (f + block_m - 1) // block_m * block_m
    po = torch.cat([torch.zeros(1, dtype=torch.long, device=dev), padded.cumsum(0)])
    row_src = torch.full((cap,), -1, dtype=torch.long, device=dev)
    start = off - f
    for e in range(E):
        row_src[po[e]: po[e] + f[e]] = ss[start[e]: start[e] + f[e]]
    valid = row_src >= 0
    inv = torch.empty(selected.numel(), dtype=torch.long, device=dev)
    inv[row_src[valid]] = torch.nonzero(valid).flatten()
    tiles = torch.full((cap // block_m + 1,), -1, dtype=torch.long, device=dev)
    for e in range(E):
        tiles[po[e] // block_m: po[e + 1] // block_m] = e
    tiles[-1] = po[-1] // block_m
    return dict(sorted_expert_idxs=se, sorted_scattered_idxs=ss, expert_frequency=freq, expert_offsets=off,
                padded_offsets=po, row_src=row_src, inv_row=inv, tile_expert=tiles)


def rows_in_use(index: ExpertIndex) -> int:
    return int(index.tile_expert[-1].item()) * N.XMA_BLOCK_M


def row_experts(index: ExpertIndex, used: int) -> torch.Tensor:
    return index.tile_expert[:-1].long().repeat_interleave(N.XMA_BLOCK_M)[:used]


def padded_rows(index: ExpertIndex, cols: int, dtype=torch.bfloat16, seed: int = 0, scale: float = 1.0) -> torch.Tensor:
    """Random rows in padded expert order with zero padding rows."""
    g = torch.Generator(device=index.row_src.device).manual_seed(seed)
    rows = (torch.randn(index.cap, cols, device=index.row_src.device, generator=g) * scale).to(dtype)
    rows[index.row_src < 0] = 0
    return rows


def grouped_reference(a: torch.Tensor, w: torch.Tensor, index: ExpertIndex, used: int, transpose_w: bool) -> torch.Tensor:
    """float32 per-expert products: a_e @ w[e]^T (forward layout) or a_e @ w[e] (input-gradient layout)."""
    experts = row_experts(index, used)
    out = torch.zeros(used, w.size(1) if transpose_w else w.size(2), device=a.device)
    for e in range(w.size(0)):
        m = experts == e
        if m.any():
            we = w[e].float()
            out[m] = a[:used][m].float() @ (we.t() if transpose_w else we)
    return out


def max_rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """max |got - ref| / max |ref| : the bf16 parity measure (tolerance 2e-2)."""
    return ((got.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-12)).item()


def assert_status_clean(device) -> None:
    torch.cuda.synchronize(device)
    assert int(N.status_word(device).item()) == 0, "a bounded device-side wait ran out"
