"""Integer routing work on the GPU: bit-exact against the oracle (and the reference's goldens)."""

import numpy as np
import pytest
import torch

import xma
from golden_inputs import GOLDEN_DIR, load
from gpu_helpers import expected_padded_order, make_selection
from oracle import moe_oracle as O
from xma.layers.moe.routing import build_expert_index, router_topk_softmax

pytestmark = pytest.mark.gpu


def reference_sizes():
    # tests/test_commons.py:34-46 of the reference: 2^i + j for i < 15, j < 10, plus sizes around 3000
    sizes = {2**i + j for i in range(15) for j in range(10)}
    rng = np.random.default_rng(0)
    sizes |= {int(3000 + v) for v in rng.integers(-1000, 1000, size=50)}
    return sorted(sizes)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
def test_continuous_count_reference_matrix(device, dtype):
    """tests/functional/continuous_count_test.py:19-44: E=72, exact equality with bincount."""
    g = torch.Generator().manual_seed(42)
    for n in reference_sizes():
        x = torch.randint(0, 72, (n,), generator=g, dtype=dtype).to(device)
        got = xma.continuous_count(x=x, bins=72, kernel_backend=xma.KernelBackend.cuda)
        assert got.dtype == torch.uint32 and got.device == x.device
        assert torch.equal(got.cpu(), O.continuous_count(x.cpu(), 72)), n


@pytest.mark.parametrize("bins", [2, 8, 64, 256, 1024, 5000, 16384])
@pytest.mark.parametrize("n", [0, 1, 31, 4099, 70001, 1 << 18, (1 << 20) + 5, (1 << 22) + 3])
def test_continuous_count_bins_and_layouts(device, bins, n):
    """Every counting scheme (packed registers up to 8 bins, [bin][lane] counters up to 1024, replicated
    copies beyond) in both launch forms (one cluster up to 2^18 ids, a grid of blocks beyond), on
    unsorted, sorted and misaligned inputs of both id types."""
    g = torch.Generator().manual_seed(bins * 7 + n)
    base = torch.randint(0, bins, (n + 3,), generator=g, dtype=torch.int64).to(device)
    for x in (base[:n], base[:n].sort().values, base[1: n + 1], base[3: n + 3].to(torch.int32)[1:] if n > 1 else base[:n]):
        x = x.contiguous() if not x.is_contiguous() else x  # offset views stay misaligned on purpose
        got = xma.continuous_count(x, bins)
        assert torch.equal(got.cpu(), O.continuous_count(x.cpu(), bins)[:bins])


def test_continuous_count_ignores_out_of_range(device):
    x = torch.tensor([0, 1, 5, -1, 9, 1, 4, 4], device=device)
    assert xma.continuous_count(x, 5).tolist() == [1, 2, 0, 0, 2]


def test_continuous_count_goldens(device):
    rec = np.load(f"{GOLDEN_DIR}/continuous_count.npz")
    for key in rec.files:
        if key.startswith("ids_"):
            n = key.split("_")[1]
            got = xma.continuous_count(torch.from_numpy(rec[key]).to(device), 72)
            assert np.array_equal(got.cpu().numpy().astype(np.int64), rec[f"count_{n}"])
    assert xma.continuous_count(torch.from_numpy(rec["ids_9"]).to(device), 1).tolist() == rec["count_bins1"].tolist()


def test_continuous_count_under_torch_compile(device):
    fn = torch.compile(xma.continuous_count, fullgraph=True)
    x = torch.randint(0, 72, (4097,), device=device)
    assert torch.equal(fn(x, 72).cpu(), O.continuous_count(x.cpu(), 72))


@pytest.mark.parametrize("T,E,k", [(7, 8, 2), (512, 8, 2), (1000, 64, 8), (333, 256, 8), (64, 6, 4), (50, 128, 8), (9, 4, 1),
                                   (17, 1024, 32), (8192, 64, 8)])
def test_router_topk_fp32_matches_torch_exactly(device, T, E, k):
    """float32 logits have no ties here: indices equal torch.topk's, values bit-exact."""
    g = torch.Generator().manual_seed(T + E + k)
    logits = torch.randn(T, E, generator=g).to(device)
    w, sel = router_topk_softmax(logits, k)
    v_ref, i_ref = O.get_topk(logits, k)
    assert sel.dtype == torch.int64 and torch.equal(sel, i_ref)
    assert torch.equal(logits.gather(1, sel), v_ref)
    torch.testing.assert_close(w, torch.softmax(v_ref.float(), -1), rtol=0, atol=2e-7)


@pytest.mark.parametrize("T,E,k", [(4096, 256, 8), (4096, 8, 2), (1000, 64, 8)])
def test_router_topk_bf16_ties_go_to_lowest_expert(device, T, E, k):
    """bf16 logits tie often: values must equal torch.topk's bit-exactly, the index set must be a
    valid top-k set, and ties are broken towards the lowest expert id (stable descending sort)."""
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(T, E, generator=g).to(torch.bfloat16).to(device)
    w, sel = router_topk_softmax(logits, k)
    v_ref, _ = logits.topk(k, -1)
    assert torch.equal(logits.gather(1, sel), v_ref)
    stable = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :k]
    assert torch.equal(sel, stable)
    torch.testing.assert_close(w.float(), torch.softmax(v_ref.float(), -1), rtol=0, atol=4e-3)


def test_router_topk_goldens(device):
    """Routing of the reference's own torch path on the golden inputs."""
    for name in ("moe_small_fp32", "moe_cfg1_fp32", "moe_e128_fp32"):
        _, ref, meta = load(name)
        w, sel = router_topk_softmax(ref["router_logits"].to(device), meta["k"])
        assert torch.equal(sel.cpu(), ref["selected_experts"])
        torch.testing.assert_close(w.cpu(), ref["router_weights"], rtol=0, atol=2e-7)


def test_router_backward_matches_autograd(device):
    T, E, k = 300, 64, 8
    logits = torch.randn(T, E, device=device, requires_grad=True)
    w, _ = router_topk_softmax(logits, k)
    g = torch.randn_like(w)
    w.backward(g)
    ref_in = logits.detach().clone().requires_grad_(True)
    torch.softmax(ref_in.topk(k, -1).values.float(), -1).backward(g)
    torch.testing.assert_close(logits.grad, ref_in.grad, rtol=0, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32])
@pytest.mark.parametrize("T,E,k,skew", [(7, 8, 2, False), (512, 8, 2, False), (8192, 64, 8, False), (4096, 256, 8, True),
                                        (7, 128, 8, False), (100000, 8, 2, False), (1 << 20, 64, 8, False),
                                        (333, 6, 4, True), (1, 1, 1, False), (129, 2, 1, False)])
def test_index_build_is_bit_exact(device, T, E, k, skew, dtype):
    sel = make_selection(T, E, k, device, skew, dtype)
    index = build_expert_index(sel, E)
    exp = expected_padded_order(sel, E, index.cap)
    for key, want in exp.items():
        got = getattr(index, key)
        assert torch.equal(got.cpu().long(), want.cpu().long()), key
    if skew:
        assert int((index.expert_frequency.cpu().long() == 0).sum()) > 0  # empty experts are covered


def test_continuous_count_packed_counters_do_not_overflow(device):
    """One bin takes every id: the 8-bit fields of the packed per-thread counters must spill in time."""
    for n in (255 * 512 * 16 + 17, (1 << 23) + 1):
        x = torch.full((n,), 3, dtype=torch.int32, device=device)
        assert xma.continuous_count(x, 8).tolist() == [0, 0, 0, n, 0, 0, 0, 0]
        assert xma.continuous_count(x.long(), 5).tolist() == [0, 0, 0, n, 0]


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("n,E", [(8193, 8), (12000, 64), (30000, 6), (65536, 64), (100001, 256), (262144, 256),
                                 (524288, 8), (524289, 64)])
def test_index_build_cluster_sizes(device, n, E, dtype):
    """The one-launch form at every cluster size (1, 2, 4, 8, 16 CTAs), at its largest input and one id
    beyond it (five launches). Bit-exact against the stable sort, skewed so that some experts are empty."""
    g = torch.Generator(device=device).manual_seed(n % 977)
    ids = torch.randint(0, max(E - 2, 1), (n,), device=device, dtype=dtype, generator=g)
    index = build_expert_index(ids, E, top_k=1)
    exp = expected_padded_order(ids.view(-1, 1), E, index.cap)
    for key, want in exp.items():
        assert torch.equal(getattr(index, key).long(), want.long()), key


@pytest.mark.parametrize("n,E", [((1 << 24) + 77, 8), (3 * (1 << 22) + 5, 256), ((1 << 21) + 3, 1000), (5000, 1024)])
def test_index_build_large_flat_inputs(device, n, E):
    """Flat id vectors at the sizes where the segment length changes: 1536-id segments (staged
    scatter, groups that end inside a step), more than 2048 ids per segment (direct scatter), and
    expert counts up to the supported maximum. Bit-exact against the stable sort."""
    g = torch.Generator(device=device).manual_seed(n % 1000)
    ids = torch.randint(0, E, (n,), device=device, dtype=torch.int32, generator=g)
    index = build_expert_index(ids, E, top_k=1)
    exp = expected_padded_order(ids.view(-1, 1), E, index.cap)
    for key, want in exp.items():
        assert torch.equal(getattr(index, key).long(), want.long()), key


@pytest.mark.parametrize("block_m", [1, 2, 4, 12, 96, 128, 256])
def test_index_build_other_block_sizes(device, block_m):
    """xma_moe_index_build pads segments to any block_m (the expert-parallel plan uses 1; powers of two
    take a shift path, other values a division path)."""
    from xma import _native as N
    from xma import ops

    E, n = 24, 5003
    ids = make_selection(n, E, 1, device, skew=True, dtype=torch.int32).view(-1)
    cap = N.padded_capacity(n, E, block_m)
    i32 = dict(dtype=torch.int32, device=device)
    freq = torch.empty(E, dtype=torch.uint32, device=device)
    off, se, ss = torch.empty(E, **i32), torch.empty(n, **i32), torch.empty(n, **i32)
    po, row_src, inv = torch.empty(E + 1, **i32), torch.full((cap,), 7, **i32), torch.empty(n, **i32)
    tiles = torch.full((cap // block_m + 1,), 7, **i32)
    ws = torch.empty(N.index_workspace_elems(n, E), **i32)
    ops.moe_index_build_cuda(ids, freq, off, se, ss, po, row_src, inv, tiles, ws, E, block_m)
    exp = expected_padded_order(ids.view(-1, 1), E, cap, block_m)
    got = dict(sorted_expert_idxs=se, sorted_scattered_idxs=ss, expert_frequency=freq, expert_offsets=off,
               padded_offsets=po, row_src=row_src, inv_row=inv, tile_expert=tiles)
    for key, want in exp.items():
        assert torch.equal(got[key].long(), want.long()), key


def test_index_build_reference_unstable_sort_agrees_per_expert(device):
    """Against the reference's own `sort()` (not stable): same sorted ids, same counts, and the same
    multiset of flat indices inside every expert segment."""
    sel = make_selection(2048, 64, 8, device)
    index = build_expert_index(sel, 64)
    se, ss = sel.flatten().sort()
    assert torch.equal(index.sorted_expert_idxs.long(), se)
    off = index.expert_offsets.long().cpu()
    start = 0
    mine, theirs = index.sorted_scattered_idxs.long().cpu(), ss.cpu()
    for e in range(64):
        end = int(off[e])
        assert torch.equal(mine[start:end].sort().values, theirs[start:end].sort().values)
        start = end


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("T,H,E,k", [(1, 64, 8, 1), (7, 64, 8, 2), (129, 576, 128, 8), (1000, 256, 64, 8), (300, 72, 16, 3),
                                     (8192, 2048, 64, 8), (16384, 4096, 8, 2), (4096, 7168, 256, 8), (255, 2048, 248, 8)])
def test_fused_router_gate_topk(device, dtype, T, H, E, k):
    """xma_router_gate_topk: (1) logits against the float32 product, max rel err 1e-2 (one rounding to
    the storage type); (2) weights, float32 probabilities and selected experts bit-identical to the
    stand-alone top-k/softmax kernel run on the logits this kernel wrote, so the tie rule and the
    softmax are the same code path in effect; (3) rows past T untouched."""
    from gpu_helpers import assert_status_clean, max_rel_err
    from xma import ops

    g = torch.Generator(device=device).manual_seed(T + E)
    x = torch.randn(T, H, device=device, generator=g).to(dtype)
    w = (torch.randn(E, H, device=device, generator=g) * 0.05).to(dtype)
    logits = torch.full((T + 3, E), 7.0, device=device, dtype=dtype)
    weights = torch.empty(T, k, device=device, dtype=dtype)
    probs = torch.empty(T, k, device=device, dtype=torch.float32)
    selected = torch.full((T, k), -1, device=device, dtype=torch.int64)
    ops.router_gate_topk_cuda(x, w, logits, weights, probs, selected, k)
    assert_status_clean(device)
    assert torch.all(logits[T:] == 7.0)
    logits = logits[:T].contiguous()
    assert max_rel_err(logits, x.float() @ w.float().t()) <= 1e-2

    w2 = torch.empty_like(weights)
    p2 = torch.empty_like(probs)
    s2 = torch.empty_like(selected)
    ops.router_topk_softmax_cuda(logits, w2, p2, s2, k)
    assert torch.equal(selected, s2)
    assert torch.equal(probs, p2)
    assert torch.equal(weights, w2)


@pytest.mark.parametrize("T,H,E,k", [(777, 256, 64, 8), (7, 576, 128, 8), (5000, 2048, 8, 2), (1, 64, 16, 1),
                                     (9000, 1024, 256, 8)])
def test_fused_router_backward_matches_autograd(device, T, H, E, k):
    """Gradients of the fused router (x and gate weight) against autograd through linear + topk +
    softmax on the same bf16 values; an extra gradient on the logits (auxiliary loss) is added in.
    Both products run on this library's kernels (the grouped GEMM with every token in one group, the
    weight-gradient GEMM split over row segments): token counts that are not multiples of 64 or 128,
    one and several segments, 8 to 256 experts."""
    from gpu_helpers import assert_status_clean, max_rel_err
    from xma.layers.moe.routing import fused_router, fused_router_supported

    g = torch.Generator(device=device).manual_seed(3)
    x = torch.randn(T, H, device=device, generator=g).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(E, H, device=device, generator=g) * 0.05).to(torch.bfloat16).requires_grad_(True)
    gw = torch.randn(T, k, device=device, generator=g).to(torch.bfloat16)
    gl = (torch.randn(T, E, device=device, generator=g) * 0.1).to(torch.bfloat16)
    assert fused_router_supported(x, w, k)
    logits, weights, selected = fused_router(x, w, k)
    torch.autograd.backward([weights, logits], [gw, gl])
    assert_status_clean(device)

    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().float().requires_grad_(True)
    ref_logits = xr @ wr.t()
    ref_weights = torch.softmax(ref_logits.gather(1, selected), dim=-1)
    torch.autograd.backward([ref_weights, ref_logits], [gw.float(), gl.float()])
    assert max_rel_err(x.grad, xr.grad) <= 2e-2
    assert max_rel_err(w.grad, wr.grad) <= 2e-2


@pytest.mark.parametrize("k", [1, 2, 8])
def test_get_topk_matches_torch(device, k):
    """MoE._get_topk (xma/layers/moe/__init__.py:268-274): float32 logits have no ties, so values and
    indices equal torch.topk's (torch.max's for k = 1) exactly."""
    moe = xma.MoE(num_experts=64, num_experts_per_tok=k, hidden_size=64, intermediate_size=128,
                  activation_function=xma.swiglu_packed, is_glu=True, add_bias=False, std=0.02).to(device)
    logits = torch.randn(300, 64, device=device)
    values, indices = moe._get_topk(logits)
    ref_v, ref_i = logits.topk(k, dim=-1)
    assert torch.equal(values, ref_v) and torch.equal(indices, ref_i)
