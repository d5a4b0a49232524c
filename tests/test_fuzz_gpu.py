"""Seeded random shapes per kernel against the oracle / float32 torch: the sizes the hand-picked
cases do not hit (dimensions that are multiples of 8 but of nothing larger, expert counts that are not
a multiple of the warp size, more copies per token than 16-byte vectors per row, single rows)."""

import random

import pytest
import torch

import xma
from gpu_helpers import (assert_status_clean, expected_padded_order, grouped_reference, make_selection, max_rel_err,
                         padded_rows, row_experts, rows_in_use)
from xma import _native as N
from xma import ops
from xma.layers.moe.routing import build_expert_index, router_topk_softmax

pytestmark = pytest.mark.gpu


def _cases(seed, count, make):
    rng = random.Random(seed)
    return [make(rng) for _ in range(count)]


@pytest.mark.parametrize("n,E,dtype", _cases(1, 24, lambda r: (r.choice([1, 5, 31, 32, 33, 1000, 4097, 70000, 300001]),
                                                               r.choice([1, 2, 7, 33, 40, 100, 255, 257, 1000, 1024]),
                                                               r.choice([torch.int32, torch.int64]))))
def test_fuzz_index_build_and_count(device, n, E, dtype):
    g = torch.Generator(device=device).manual_seed(n + E)
    ids = torch.randint(0, E, (n,), device=device, dtype=dtype, generator=g)
    assert torch.equal(xma.continuous_count(ids, E).cpu().long(), torch.bincount(ids.cpu().long(), minlength=E))
    index = build_expert_index(ids, E, top_k=1)
    exp = expected_padded_order(ids.view(-1, 1), E, index.cap)
    for key, want in exp.items():
        assert torch.equal(getattr(index, key).long(), want.long()), key


@pytest.mark.parametrize("T,E,k,dtype", _cases(2, 24, lambda r: (r.choice([1, 3, 64, 257, 1001]), r.choice([1, 2, 5, 31, 33, 72, 129, 500, 1024]),
                                                                 r.randint(1, 32), r.choice([torch.float32, torch.bfloat16, torch.float16]))))
def test_fuzz_router_topk(device, T, E, k, dtype):
    k = min(k, E)
    g = torch.Generator(device=device).manual_seed(T * 7 + E)
    logits = torch.randn(T, E, device=device, generator=g).to(dtype).requires_grad_(True)
    w, sel = router_topk_softmax(logits, k)
    stable = torch.sort(logits.detach().float(), dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(sel, stable)
    ref = torch.softmax(logits.detach().float().gather(1, sel), -1)
    torch.testing.assert_close(w.float(), ref, rtol=0, atol=2e-7 if dtype == torch.float32 else 4e-3)
    gw = torch.randn(T, k, device=device, generator=g).to(dtype)
    w.backward(gw)
    lin = logits.detach().float().requires_grad_(True)
    torch.softmax(lin.gather(1, sel), -1).backward(gw.float())
    torch.testing.assert_close(logits.grad.float(), lin.grad, rtol=0, atol=1e-6 if dtype == torch.float32 else 4e-3)


@pytest.mark.parametrize("T,E,k,K,Nn,layout", _cases(3, 24, lambda r: (r.choice([1, 50, 129, 700, 3000]), r.choice([1, 3, 8, 40, 130]),
                                                                       r.randint(1, 4), 8 * r.randint(1, 70), 8 * r.randint(1, 70),
                                                                       r.choice([N.GEMM_NT, N.GEMM_NN]))))
def test_fuzz_grouped_gemm(device, T, E, k, K, Nn, layout):
    k = min(k, E)
    index = build_expert_index(make_selection(T, E, k, device, seed=T + E), E)
    used = rows_in_use(index)
    a = padded_rows(index, K, torch.bfloat16, seed=K)
    shape = (E, Nn, K) if layout == N.GEMM_NT else (E, K, Nn)
    w = (torch.randn(*shape, device=device) * 0.1).to(torch.bfloat16)
    c = torch.full((index.cap, Nn), float("nan"), device=device, dtype=torch.bfloat16)
    ops.grouped_gemm_cuda(a, w, index.padded_offsets, c, None, None, None, None, layout, N.EPI_STORE)
    assert_status_clean(device)
    ref = grouped_reference(a, w, index, used, transpose_w=layout == N.GEMM_NT)
    assert max_rel_err(c[:used], ref) < 1e-2


@pytest.mark.parametrize("T,E,k,M,Nn", _cases(4, 16, lambda r: (r.choice([1, 50, 129, 700, 3000]), r.choice([1, 3, 8, 40, 130]),
                                                                r.randint(1, 4), 8 * r.randint(1, 70), 8 * r.randint(1, 70))))
def test_fuzz_grouped_wgrad(device, T, E, k, M, Nn):
    k = min(k, E)
    index = build_expert_index(make_selection(T, E, k, device, seed=T + E), E)
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
    assert max_rel_err(dw, ref) < 1e-2
    assert not torch.isnan(dw).any()
