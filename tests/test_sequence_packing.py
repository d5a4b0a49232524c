"""pack_sequence / unpack_sequence: the oracle against the reference's golden vectors (CPU) and the
sm_100a kernels against the oracle (GPU, copies: bit-exact), forward and backward."""

import numpy as np
import pytest
import torch

from golden_inputs import GOLDEN_DIR
from oracle import moe_oracle as O


def _golden():
    rec = np.load(f"{GOLDEN_DIR}/sequence_packing.npz")
    return {k: torch.from_numpy(rec[k]) for k in rec.files}


@pytest.mark.parametrize("side", ["left", "right"])
def test_oracle_matches_reference_goldens(side):
    g = _golden()
    assert torch.equal(O.pack_sequence(g["padded"], g["cu_seqlens"], side), g[f"pack_{side}"])
    assert torch.equal(O.unpack_sequence(g["packed"], g["cu_seqlens"], 5, 9, side), g[f"unpack_{side}"])


@pytest.mark.gpu
@pytest.mark.parametrize("side", ["left", "right"])
def test_kernels_match_goldens(device, side):
    import xma

    g = _golden()
    cu = g["cu_seqlens"].to(device)
    got = xma.pack_sequence([g["padded"].to(device)], cu, int(cu[-1]), side)[0]
    assert torch.equal(got.cpu(), g[f"pack_{side}"])
    got = xma.unpack_sequence([g["packed"].to(device)], cu, 5, 9, side)[0]
    assert torch.equal(got.cpu(), g[f"unpack_{side}"])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("cu_dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("side", ["left", "right"])
@pytest.mark.parametrize("B,S,tail", [(4, 2048, (2048,)), (7, 33, (5,)), (3, 17, (2, 3)), (1, 1, (8,)), (16, 128, (576,))])
def test_kernels_match_oracle_forward_and_backward(device, dtype, cu_dtype, side, B, S, tail):
    import xma

    g = torch.Generator().manual_seed(B * 1000 + S)
    seqlens = torch.randint(0, S + 1, (B,), generator=g)
    seqlens[0] = S  # one full row, and (often) an empty one
    if B > 1:
        seqlens[1] = 0
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), seqlens.cumsum(0)]).to(cu_dtype).to(device)
    total = int(seqlens.sum())
    padded = torch.randn(B, S, *tail, generator=g).to(dtype).to(device).requires_grad_(True)
    packed = xma.pack_sequence([padded], cu, total, side)[0]
    assert torch.equal(packed, O.pack_sequence(padded.detach(), cu.long(), side))
    gp = torch.randn(total, *tail, generator=g).to(dtype).to(device)
    packed.backward(gp)
    # the gradient of a gather is the scatter into zeros, which is exactly unpack
    assert torch.equal(padded.grad, O.unpack_sequence(gp, cu.long(), B, S, side))

    stream = torch.randn(total, *tail, generator=g).to(dtype).to(device).requires_grad_(True)
    out = xma.unpack_sequence([stream], cu, B, S, side)[0]
    assert torch.equal(out, O.unpack_sequence(stream.detach(), cu.long(), B, S, side))
    go = torch.randn(B, S, *tail, generator=g).to(dtype).to(device)
    out.backward(go)
    assert torch.equal(stream.grad, O.pack_sequence(go, cu.long(), side))
    # round trip: pack(unpack(x)) == x
    assert torch.equal(xma.pack_sequence([out.detach()], cu, total, side)[0], stream.detach())
