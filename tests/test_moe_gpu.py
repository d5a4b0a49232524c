"""The MoE layer on the GPU against the float32 oracle and the reference's golden vectors.

Tolerance (bf16, stated by the target): max |got - ref| / max |ref| <= 2e-2 for outputs and all
gradients, with the oracle run in float32 on the same bf16-rounded inputs and with the kernel run's
`selected_experts` injected so that routing cannot diverge. The reference's own absolute tolerances
(tests/layers/moe_test.py:112-156) are checked as well where its test applies.
"""

import pytest
import torch
import torch.nn.functional as F

import xma
from golden_inputs import load, sample
from gpu_helpers import assert_status_clean, max_rel_err
from oracle import moe_oracle as O
from xma.layers.moe.routing import router_topk_softmax

pytestmark = pytest.mark.gpu
TOL = 2e-2


def build(device, E, k, H, I, act, glu, dtype, seed):
    torch.manual_seed(seed)
    with torch.device(device):
        moe = xma.MoE(num_experts=E, num_experts_per_tok=k, hidden_size=H, intermediate_size=I, activation_function=act,
                      is_glu=glu, add_bias=False, std=0.02).to(dtype)
    with torch.no_grad():
        moe.gate.weight.normal_(0, 0.02)
    return moe


def run_and_compare(moe, x, gy, oracle_act, tol=TOL):
    device = x.device
    y, logits = moe(x)
    y.backward(gy)
    assert_status_clean(device)
    selected = router_topk_softmax(logits.detach(), moe.top_k)[1]
    ref = O.moe_forward_backward(x.detach().float(), moe.gate.weight.detach().float(), moe.c_fc.weight.detach().float(),
                                 moe.c_proj.weight.detach().float(), moe.top_k, gy.float(), oracle_act, selected)
    errs = {
        "y": max_rel_err(y, ref["y"]),
        "dx": max_rel_err(x.grad, ref["dx"]),
        "dw_fc": max_rel_err(moe.c_fc.weight.grad, ref["dw_fc"]),
        "dw_proj": max_rel_err(moe.c_proj.weight.grad, ref["dw_proj"]),
        "dgate": max_rel_err(moe.gate.weight.grad, ref["dgate"]),
    }
    assert all(v <= tol for v in errs.values()), errs
    return y, ref


@pytest.mark.parametrize("T,H,I,E,k,seed", [
    (512, 256, 512, 8, 2, 0),       # the reference's CPU-runnable benchmark shape
    (7, 2048, 8192, 2, 2, 42), (7, 2048, 8192, 4, 2, 42), (7, 2048, 8192, 6, 4, 42), (7, 2048, 8192, 8, 4, 42),
    (7, 576, 256, 128, 8, 42),      # shapes of tests/layers/moe_test.py:18-57 at its T=7
    (2048, 1024, 512, 64, 8, 1), (1, 64, 128, 4, 1, 5), (129, 64, 128, 3, 3, 6),
])
def test_fused_swiglu_layer_matches_oracle(device, T, H, I, E, k, seed):
    moe = build(device, E, k, H, I, xma.swiglu_packed, True, torch.bfloat16, seed)
    assert moe._fused_path()
    x = torch.randn(T, H, device=device, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(T, H, device=device, dtype=torch.bfloat16)
    run_and_compare(moe, x, gy, O.swiglu_packed)


def test_olmoe_like_shape_matches_oracle(device):
    """The OLMoE-like benchmark configuration at full size: T=8192, H=2048, I=1024, E=64, top-8, seed 1."""
    moe = build(device, 64, 8, 2048, 1024, xma.swiglu_packed, True, torch.bfloat16, 1)
    x = torch.randn(4, 2048, 2048, device=device, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.randn(4, 2048, 2048, device=device, dtype=torch.bfloat16)
    y, logits = moe(x)
    assert y.shape == x.shape and logits.shape == (8192, 64)
    y.backward(gy)
    assert_status_clean(device)
    selected = router_topk_softmax(logits.detach(), 8)[1]
    ref = O.moe_forward_backward(x.detach().float().view(-1, 2048), moe.gate.weight.detach().float(),
                                 moe.c_fc.weight.detach().float(), moe.c_proj.weight.detach().float(), 8,
                                 gy.float().view(-1, 2048), O.swiglu_packed, selected)
    assert max_rel_err(y.view(-1, 2048), ref["y"]) <= TOL
    assert max_rel_err(x.grad.view(-1, 2048), ref["dx"]) <= TOL
    assert max_rel_err(moe.c_fc.weight.grad, ref["dw_fc"]) <= TOL
    assert max_rel_err(moe.c_proj.weight.grad, ref["dw_proj"]) <= TOL
    assert max_rel_err(moe.gate.weight.grad, ref["dgate"]) <= TOL


@pytest.mark.parametrize("glu", [True, False])
@pytest.mark.parametrize("T,H,I,E,k", [(7, 2048, 8192, 4, 2), (7, 576, 256, 128, 8), (300, 256, 512, 8, 2)])
def test_unfused_path_with_reference_test_activations(device, glu, T, H, I, E, k):
    """nn.GLU / nn.GELU(tanh) as in tests/test_commons.py:93-94: arbitrary callables run between two
    unfused grouped GEMMs. Two checks: max rel err <= 2e-2 against the float32 oracle, and the
    reference's own bf16 absolute tolerances (tests/layers/moe_test.py:112-156) against the oracle
    run in bf16, which is what the reference's test compares (kernel path vs torch path, same dtype)."""
    act = torch.nn.GLU() if glu else torch.nn.GELU(approximate="tanh")
    oracle_act = (lambda t: F.glu(t, dim=-1)) if glu else (lambda t: F.gelu(t, approximate="tanh"))
    moe = build(device, E, k, H, I, act, glu, torch.bfloat16, 42)
    assert not moe._fused_path()
    x = torch.randn(T, H, device=device, dtype=torch.bfloat16, requires_grad=True)
    gy = torch.ones(T, H, device=device, dtype=torch.bfloat16)  # the reference test uses y.sum().backward()
    y, _ = run_and_compare(moe, x, gy, oracle_act)
    selected = router_topk_softmax(moe.gate(x.detach()), k)[1]
    ref = O.moe_forward_backward(x.detach(), moe.gate.weight.detach(), moe.c_fc.weight.detach(), moe.c_proj.weight.detach(),
                                 k, gy, oracle_act, selected)
    torch.testing.assert_close(y, ref["y"], rtol=0, atol=2.35e-2)
    torch.testing.assert_close(x.grad, ref["dx"], rtol=0, atol=4e-2)
    torch.testing.assert_close(moe.c_fc.weight.grad, ref["dw_fc"], rtol=0, atol=4e-2)
    torch.testing.assert_close(moe.c_proj.weight.grad, ref["dw_proj"], rtol=0, atol=4e-2)


@pytest.mark.parametrize("name", ["moe_small_fp32", "moe_cfg1_fp32", "moe_small_bf16"])
def test_layer_against_reference_goldens(device, name):
    """bf16 kernels on the golden inputs against the reference's own outputs (float32 or bf16 torch
    path). bf16 router logits can flip a near-tie, so the layer's own routing is only required to agree
    on most rows; every value comparison runs with the REFERENCE's selected_experts injected through
    `_compute_experts` (router weights recomputed from the bf16 logits at those experts), so the output
    and every gradient are always compared."""
    inp, ref, meta = load(name)
    k = meta["k"]
    moe = build(device, meta["E"], k, meta["H"], meta["I"], xma.swiglu_packed, True, torch.bfloat16, 0)
    with torch.no_grad():
        moe.gate.weight.copy_(inp["gate"])
        moe.c_fc.weight.copy_(inp["w_fc"])
        moe.c_proj.weight.copy_(inp["w_proj"])
    x = inp["x"].to(device).to(torch.bfloat16).requires_grad_(True)
    gy = inp["grad_y"].to(device).to(torch.bfloat16)
    with torch.no_grad():
        own = router_topk_softmax(moe.gate(x.detach()), k)[1].cpu()
    assert (own.sort(-1).values == ref["selected_experts"].long().sort(-1).values).all(1).float().mean() > 0.9

    selected = ref["selected_experts"].long().to(device)
    logits = moe.gate(x)
    weights = torch.softmax(logits.gather(-1, selected).float(), dim=-1).to(torch.bfloat16)
    y = moe._compute_experts(x, weights, selected)
    y.backward(gy)
    assert_status_clean(device)
    assert max_rel_err(y.detach().cpu(), ref["y"]) <= 3e-2
    assert max_rel_err(x.grad.cpu(), ref["dx"]) <= 3e-2
    assert max_rel_err(moe.gate.weight.grad.cpu(), ref["dgate"]) <= 3e-2
    if "dw_fc" in ref:
        assert max_rel_err(moe.c_fc.weight.grad.cpu(), ref["dw_fc"]) <= 3e-2
        assert max_rel_err(moe.c_proj.weight.grad.cpu(), ref["dw_proj"]) <= 3e-2
    else:  # large cases keep every 37th element of the weight gradients
        assert max_rel_err(sample(moe.c_fc.weight.grad.cpu()), ref["dw_fc_sample"]) <= 3e-2
        assert max_rel_err(sample(moe.c_proj.weight.grad.cpu()), ref["dw_proj_sample"]) <= 3e-2


def test_compute_experts_entry_with_injected_routing(device):
    """`_compute_experts` is the entry for configurations that give router logits directly
    (Mixtral-like: fp32 logits, E=8, top-2); skewed logits leave some experts empty."""
    T, H, I, E, k = 1024, 512, 1024, 8, 2
    moe = build(device, E, k, H, I, xma.swiglu_packed, True, torch.bfloat16, 2)
    logits = torch.randn(T, E, device=device) + torch.tensor([3.0, 2, 1, 0, -1, -30, -30, -30], device=device)
    w, sel = router_topk_softmax(logits, k)
    x = torch.randn(T, H, device=device, dtype=torch.bfloat16, requires_grad=True)
    y = moe._compute_experts(x, w.to(torch.bfloat16), sel)
    gy = torch.randn_like(y)
    y.backward(gy)
    assert_status_clean(device)
    xr = x.detach().float().requires_grad_(True)
    w1 = moe.c_fc.weight.detach().float().requires_grad_(True)
    w2 = moe.c_proj.weight.detach().float().requires_grad_(True)
    yr = O.compute_experts(xr, w.to(torch.bfloat16).float(), sel, w1, w2)
    yr.backward(gy.float())
    assert max_rel_err(y, yr) <= TOL and max_rel_err(x.grad, xr.grad) <= TOL
    assert max_rel_err(moe.c_fc.weight.grad, w1.grad) <= TOL and max_rel_err(moe.c_proj.weight.grad, w2.grad) <= TOL
    assert torch.all(moe.c_fc.weight.grad[5:] == 0) and torch.all(moe.c_proj.weight.grad[5:] == 0)


def test_swiglu_packed_standalone(device):
    """tests/functional/swiglu_packed_test.py:55-61: float32 atol 4.9e-5 forward, 5e-6 gradient."""
    import numpy as np
    from golden_inputs import GOLDEN_DIR

    rec = np.load(f"{GOLDEN_DIR}/swiglu_packed.npz")
    x = torch.from_numpy(rec["x"]).to(device).requires_grad_(True)
    y = xma.swiglu_packed(x)
    y.backward(torch.from_numpy(rec["dy"]).to(device))
    torch.testing.assert_close(y.detach().cpu(), torch.from_numpy(rec["y"]), rtol=0, atol=4.9e-5)
    torch.testing.assert_close(x.grad.cpu(), torch.from_numpy(rec["dx"]), rtol=0, atol=5e-6)
    for shape in ((5, 7, 64), (4096, 2048), (33, 6)):
        xb = torch.randn(*shape, device=device, dtype=torch.bfloat16, requires_grad=True)
        yb = xma.swiglu_packed(xb)
        torch.testing.assert_close(yb, O.swiglu_packed(xb.detach()), rtol=1.6e-2, atol=1e-3)


@pytest.mark.parametrize("fused,glu,dtype,E,k,H,I", [
    (True, True, torch.bfloat16, 8, 2, 256, 512),
    (True, True, torch.bfloat16, 6, 4, 2048, 8192),     # shapes of tests/layers/moe_test.py:18-57
    (False, True, torch.bfloat16, 4, 2, 2048, 8192),    # nn.GLU between two unfused grouped GEMMs
    (False, False, torch.bfloat16, 128, 8, 576, 256),   # nn.GELU(tanh), one-launch router front end
    (False, True, torch.float32, 4, 2, 2048, 8192),     # float32 parameters (split-bf16 products)
])
def test_torch_compile_fullgraph_forward_and_backward(device, fused, glu, dtype, E, k, H, I):
    """tests/layers/moe_test.py:103-156: the module is compiled with fullgraph=True, run on T=7 tokens,
    back-propagated through with y.sum().backward(), and output, input gradient and expert weight
    gradients are compared. Here the compiled module is compared with the eager module (same kernels:
    equal up to the library GEMM the compiler may pick for the router) and with the float32 oracle
    at the reference's tolerances for the dtype."""
    if fused:
        act, oracle_act = xma.swiglu_packed, O.swiglu_packed
    elif glu:
        act, oracle_act = torch.nn.GLU(), (lambda t: F.glu(t, dim=-1))
    else:
        act, oracle_act = torch.nn.GELU(approximate="tanh"), (lambda t: F.gelu(t, approximate="tanh"))
    moe = build(device, E, k, H, I, act, glu, dtype, 42)
    assert moe._fused_path() == fused
    x = torch.randn(7, H, device=device, dtype=dtype)

    def run(module):
        moe.zero_grad(set_to_none=True)
        xin = x.clone().requires_grad_(True)
        y, logits = module(xin)
        y.sum().backward()
        return (y.detach(), xin.grad, moe.c_fc.weight.grad.clone(), moe.c_proj.weight.grad.clone(),
                moe.gate.weight.grad.clone(), logits.detach())

    eager = run(moe)
    torch._dynamo.reset()
    compiled = run(torch.compile(moe, fullgraph=True))
    assert_status_clean(device)
    # The compiled router may reach its logits through another library GEMM than the eager one; where a
    # token's k-th and (k+1)-th logits lie within one rounding step of each other (they do in the second
    # case: 0.009 apart at a bf16 step of 0.008) that can change the token's experts. The two runs are
    # compared with each other when they routed alike, and the compiled run always with the oracle on its
    # own routing.
    selected = router_topk_softmax(compiled[5], k)[1]
    if torch.equal(selected, router_topk_softmax(eager[5], k)[1]):
        names = ("y", "dx", "dw_fc", "dw_proj", "dgate")
        loose = 1e-2 if dtype != torch.float32 else 1e-4
        for name, got, want in zip(names, compiled, eager):
            assert max_rel_err(got, want) <= loose, (name, max_rel_err(got, want))

    ref = O.moe_forward_backward(x.float(), moe.gate.weight.detach().float(), moe.c_fc.weight.detach().float(),
                                 moe.c_proj.weight.detach().float(), k, torch.ones(7, H, device=device), oracle_act, selected)
    tol = F32_TOL if dtype == torch.float32 else TOL
    # The reference's absolute tolerances (moe_test.py:112-156) are between two runs in the same dtype; here
    # the other side is the float32 oracle, so a bf16 result additionally gets two units in the last place
    # (the few gradient elements of magnitude > 2.5, where one rounding step already exceeds the bound).
    atols = {torch.bfloat16: (2.35e-2, 4e-2, 4e-2), torch.float32: (6e-3, 6.5e-3, 3e-2)}[dtype]
    for name, got, atol in zip(("y", "dx", "dw_fc", "dw_proj"), compiled, (atols[0], atols[1], atols[2], atols[2])):
        assert max_rel_err(got, ref[name]) <= tol, (name, max_rel_err(got, ref[name]))
        torch.testing.assert_close(got.float(), ref[name], rtol=0 if dtype == torch.float32 else 1.6e-2, atol=atol)


def test_empty_batch(device):
    """No tokens at all: every kernel sees zero rows; outputs are empty, weight gradients are zeros."""
    moe = build(device, 8, 2, 256, 512, xma.swiglu_packed, True, torch.bfloat16, 0)
    x = torch.zeros(0, 256, device=device, dtype=torch.bfloat16, requires_grad=True)
    y, logits = moe(x)
    assert y.shape == (0, 256) and logits.shape == (0, 8)
    y.sum().backward()
    assert_status_clean(device)
    assert x.grad.shape == (0, 256)
    assert torch.all(moe.c_fc.weight.grad == 0) and torch.all(moe.c_proj.weight.grad == 0)


def _full_size_case(device, T, H, I, E, k, seed, skew):
    """Builds bf16 weights directly on the device (no float32 copies) and a routing for a full-size
    benchmark configuration."""
    g = torch.Generator(device=device).manual_seed(seed)
    moe = xma.MoE.__new__(xma.MoE)
    torch.nn.Module.__init__(moe)
    moe.num_experts, moe.top_k, moe.hidden_size, moe.intermediate_size, moe.is_glu = E, k, H, I, True
    moe.expert_parallel_group, moe.expert_parallel_mode, moe._peer_state, moe.num_local_experts = None, "nccl", None, E
    moe.act = xma.swiglu_packed

    class _W(torch.nn.Module):
        def __init__(self, shape):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.empty(*shape, device=device, dtype=torch.bfloat16).normal_(0, 0.02, generator=g))
            self.bias = None

    moe.c_fc, moe.c_proj = _W((E, 2 * I, H)), _W((E, H, I))
    logits = torch.randn(T, E, device=device, generator=g)
    if skew:
        ranks = torch.randperm(E, generator=torch.Generator().manual_seed(seed)).float() + 1.0
        logits = logits + (-1.1 * ranks.log()).to(device)
    weights, selected = router_topk_softmax(logits, k)
    x = torch.randn(T, H, device=device, generator=g).to(torch.bfloat16)
    return moe, x, weights.to(torch.bfloat16), selected


@pytest.mark.parametrize("name,T,H,I,E,k,seed,skew", [
    ("mixtral", 16384, 4096, 14336, 8, 2, 2, False),
    ("deepseek-v3", 32768, 7168, 2048, 256, 8, 3, True),
])
def test_full_size_shapes_by_properties_and_sampled_tokens(device, name, T, H, I, E, k, seed, skew):
    """The two large benchmark configurations at full size.
    (1) Size-independent property: halving every router weight halves the output bit-exactly (a
        power-of-two scale commutes with every bf16 rounding on the path).
    (2) 48 sampled tokens against the float32 oracle run on those tokens alone (a token's output does
        not depend on the other tokens), tolerance max rel err 2e-2; the input gradient of the same
        tokens against the oracle's.
    (3) Experts that received no token get an exactly zero weight gradient.
    (4) 256 x 256 slices of both weight gradients of two experts, the one with the most rows and the
        non-empty one with the fewest, against float32 X_e^T Y_e built from the oracle's formulas on
        that expert's rows (d(activation input) and the activation restricted to the slice's columns)."""
    moe, x, weights, selected = _full_size_case(device, T, H, I, E, k, seed, skew)
    x.requires_grad_(True)
    y = moe._compute_experts(x, weights, selected)
    with torch.no_grad():
        y_half = moe._compute_experts(x.detach(), weights * 0.5, selected)
    assert torch.equal(y_half, y.detach() * 0.5)

    gy = torch.randn(T, H, device=device, generator=torch.Generator(device=device).manual_seed(7)).to(torch.bfloat16)
    y.backward(gy)
    assert_status_clean(device)

    pick = torch.randperm(T, generator=torch.Generator().manual_seed(1))[:48].to(device)
    xs = x.detach()[pick].float().requires_grad_(True)
    ref = O.compute_experts(xs, weights[pick].float(), selected[pick], moe.c_fc.weight.detach().float(),
                            moe.c_proj.weight.detach().float()) if E <= 8 else None
    if ref is None:
        # 256 experts x 117 MB of float32 weights do not fit a second copy: run the oracle expert by expert
        used = selected[pick].unique()
        remap = torch.full((E,), -1, dtype=torch.long, device=device)
        remap[used] = torch.arange(used.numel(), device=device)
        ref = O.compute_experts(xs, weights[pick].float(), remap[selected[pick]],
                                moe.c_fc.weight.detach()[used].float(), moe.c_proj.weight.detach()[used].float())
    ref.backward(gy[pick].float())
    assert max_rel_err(y.detach()[pick], ref.detach()) <= TOL
    assert max_rel_err(x.grad[pick], xs.grad) <= TOL

    counts = torch.bincount(selected.flatten(), minlength=E)
    empty = counts == 0
    if skew:
        assert int(empty.sum()) > 0
    if empty.any():
        assert torch.all(moe.c_fc.weight.grad[empty] == 0) and torch.all(moe.c_proj.weight.grad[empty] == 0)

    busy = int(counts.argmax())
    sparse = int(torch.where(counts > 0, counts, counts.max() + 1).argmin())
    for e in {busy, sparse}:
        tok, slot = torch.nonzero(selected == e, as_tuple=True)
        xe = x.detach()[tok].float()                     # [m_e, H]
        pe = weights[tok, slot].float().unsqueeze(1)      # router weight of every row
        ge = gy[tok].float()
        w1, w2 = moe.c_fc.weight.detach()[e].float(), moe.c_proj.weight.detach()[e].float()
        pre = (xe @ w1.t()).to(torch.bfloat16).float()   # the reference rounds the up projection (Appendix step 2)
        u, g = pre[:, :I], pre[:, I:]
        sig = torch.sigmoid(g)
        h = u * g * sig                                   # swiglu, unscaled
        dh = (ge @ w2) * pe                               # d(h) = p * dy W2
        du, dg = dh * g * sig, dh * u * (sig + g * sig * (1 - sig))
        for (r0, c0) in ((0, 0), (H - 256, I - 256)):
            # dW_proj[e][r0:r0+256, c0:c0+256] = (p dy)[:, rows]^T h[:, cols]
            want = (ge[:, r0:r0 + 256] * pe).t() @ h[:, c0:c0 + 256]
            assert max_rel_err(moe.c_proj.weight.grad[e, r0:r0 + 256, c0:c0 + 256], want) <= TOL, (name, e, "dw_proj")
        for (r0, c0) in ((0, 0), (2 * I - 256, H - 256)):
            # dW_fc[e][r0:r0+256, c0:c0+256] = d(pre)[:, rows]^T x[:, cols]; rows < I are the up half
            d_pre = du if r0 < I else dg
            rr = r0 if r0 < I else r0 - I
            want = d_pre[:, rr:rr + 256].t() @ xe[:, c0:c0 + 256]
            assert max_rel_err(moe.c_fc.weight.grad[e, r0:r0 + 256, c0:c0 + 256], want) <= TOL, (name, e, "dw_fc")
        del xe, ge, w1, w2, pre, u, g, sig, h, dh, du, dg
    del moe, x, y, y_half, gy
    torch.cuda.empty_cache()


F32_TOL = 2e-4  # hi/lo bf16 split: ~2^-16 per operand; TF32 (the reference's Triton products) would be ~1e-3


@pytest.mark.parametrize("name,act,glu", [
    ("moe_small_fp32", "swiglu", True), ("moe_cfg1_fp32", "swiglu", True), ("moe_glu_fp32", "glu", True),
    ("moe_gelu_fp32", "gelu", False), ("moe_e128_fp32", "swiglu", True),
])
def test_float32_layer_against_reference_goldens(device, name, act, glu):
    """float32 parameters and inputs (tests/layers/moe_test.py:65 runs float32 too) against the
    reference's own float32 outputs, at the reference's float32 tolerances (moe_test.py:112-156:
    output 6e-3, input gradient 6.5e-3, weight gradients 3e-2 absolute) and at the much tighter
    relative bound the split-bf16 products allow. Routing must equal the reference's exactly."""
    inp, ref, meta = load(name)
    fn = {"swiglu": xma.swiglu_packed, "glu": torch.nn.GLU(), "gelu": torch.nn.GELU(approximate="tanh")}[act]
    moe = build(device, meta["E"], meta["k"], meta["H"], meta["I"], fn, glu, torch.float32, 0)
    assert not moe._fused_path()
    with torch.no_grad():
        moe.gate.weight.copy_(inp["gate"])
        moe.c_fc.weight.copy_(inp["w_fc"])
        moe.c_proj.weight.copy_(inp["w_proj"])
    x = inp["x"].to(device).requires_grad_(True)
    y, logits = moe(x)
    y.backward(inp["grad_y"].to(device))
    assert_status_clean(device)
    assert y.dtype == torch.float32 and moe.c_fc.weight.grad.dtype == torch.float32
    sel = router_topk_softmax(logits.detach(), meta["k"])[1].cpu()
    assert torch.equal(sel.sort(-1).values, ref["selected_experts"].long().sort(-1).values)
    torch.testing.assert_close(y.detach().cpu(), ref["y"], rtol=0, atol=6e-3)
    torch.testing.assert_close(x.grad.cpu(), ref["dx"], rtol=0, atol=6.5e-3)
    assert max_rel_err(y.detach().cpu(), ref["y"]) <= F32_TOL
    assert max_rel_err(x.grad.cpu(), ref["dx"]) <= F32_TOL
    assert max_rel_err(moe.gate.weight.grad.cpu(), ref["dgate"]) <= F32_TOL
    if "dw_fc" in ref:
        torch.testing.assert_close(moe.c_fc.weight.grad.cpu(), ref["dw_fc"], rtol=0, atol=3e-2)
        torch.testing.assert_close(moe.c_proj.weight.grad.cpu(), ref["dw_proj"], rtol=0, atol=3e-2)
        assert max_rel_err(moe.c_fc.weight.grad.cpu(), ref["dw_fc"]) <= F32_TOL
        assert max_rel_err(moe.c_proj.weight.grad.cpu(), ref["dw_proj"]) <= F32_TOL


@pytest.mark.parametrize("T,H,I,E,k", [(7, 2048, 8192, 4, 2), (7, 576, 256, 128, 8), (1000, 256, 512, 8, 2)])
def test_float32_layer_matches_oracle(device, T, H, I, E, k):
    """Shapes of tests/layers/moe_test.py:18-57 in float32 against the float32 oracle."""
    moe = build(device, E, k, H, I, xma.swiglu_packed, True, torch.float32, 42)
    x = torch.randn(T, H, device=device, requires_grad=True)
    gy = torch.randn(T, H, device=device)
    run_and_compare(moe, x, gy, O.swiglu_packed, tol=F32_TOL)


@pytest.mark.parametrize("fused", [True, False])
def test_float16_layer_matches_oracle(device, fused):
    """float16 (tests/layers/moe_test.py:65): the 2e-2 relative bound against the float32 oracle, and the
    reference's float16 absolute tolerances (moe_test.py:112-156: 4e-3 output and input gradient,
    2.5e-2 weight gradients) against the oracle run in float32."""
    act = xma.swiglu_packed if fused else torch.nn.GLU()
    oracle_act = O.swiglu_packed if fused else (lambda t: F.glu(t, dim=-1))
    moe = build(device, 6, 4, 2048, 8192, act, True, torch.float16, 42)
    assert moe._fused_path() == fused
    x = torch.randn(7, 2048, device=device, dtype=torch.float16, requires_grad=True)
    gy = torch.ones(7, 2048, device=device, dtype=torch.float16)
    y, ref = run_and_compare(moe, x, gy, oracle_act)
    torch.testing.assert_close(y.float(), ref["y"], rtol=0, atol=4e-3)
    torch.testing.assert_close(x.grad.float(), ref["dx"], rtol=0, atol=4e-3)
    torch.testing.assert_close(moe.c_fc.weight.grad.float(), ref["dw_fc"], rtol=0, atol=2.5e-2)
    torch.testing.assert_close(moe.c_proj.weight.grad.float(), ref["dw_proj"], rtol=0, atol=2.5e-2)


def test_layer_step_is_cuda_graph_capturable(device):
    """Forward and backward make no host synchronisation and no launch whose arguments depend on device
    data: a whole step is recorded into one CUDA graph and replayed on new inputs, with results equal
    bit for bit to the eager step (every kernel is deterministic: the router-weight gradient is summed
    in a fixed order; the gate's own gradient GEMMs are the library's)."""
    moe = build(device, 16, 4, 256, 512, xma.swiglu_packed, True, torch.bfloat16, 9)
    T = 1024
    static_x = torch.randn(T, 256, device=device, dtype=torch.bfloat16, requires_grad=True)
    static_gy = torch.randn(T, 256, device=device, dtype=torch.bfloat16)

    def step():
        for p in moe.parameters():
            p.grad = None
        static_x.grad = None
        y, _ = moe(static_x)
        y.backward(static_gy)
        return y

    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream(device).wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = step()
    dx_static, dw_static = static_x.grad, moe.c_fc.weight.grad

    new_x = torch.randn(T, 256, device=device, dtype=torch.bfloat16)
    new_gy = torch.randn(T, 256, device=device, dtype=torch.bfloat16)
    with torch.no_grad():
        static_x.copy_(new_x)
        static_gy.copy_(new_gy)
    graph.replay()
    torch.cuda.synchronize(device)
    got = (y_static.clone(), dx_static.clone(), dw_static.clone(), moe.gate.weight.grad.clone())
    assert_status_clean(device)

    y_eager = step()  # eager, same static inputs
    assert torch.equal(got[0], y_eager)
    assert torch.equal(got[2], moe.c_fc.weight.grad)
    assert torch.equal(got[1], static_x.grad)
    assert torch.equal(got[3], moe.gate.weight.grad)


def _fuzz_cases():
    import random

    rng = random.Random(1234)
    cases = []
    for i in range(36):
        E = rng.choice([1, 2, 3, 5, 8, 16, 24, 40, 64, 128, 136, 200, 256])
        k = rng.randint(1, min(8, E))
        H = 8 * rng.randint(1, 96)
        I = 128 * rng.randint(1, 6) if i % 3 else 8 * rng.randint(1, 80)  # every third case: not a multiple of 128
        T = rng.choice([1, 2, 7, 31, 128, 129, 255, 300, 777, 1500])
        dtype = [torch.bfloat16, torch.float16, torch.float32][i % 3 if i % 7 else 0]
        cases.append((T, H, I, E, k, dtype, 100 + i))
    return cases


@pytest.mark.parametrize("T,H,I,E,k,dtype,seed", _fuzz_cases())
def test_layer_fuzz_against_oracle(device, T, H, I, E, k, dtype, seed):
    """Seeded random shapes over every path the layer can take: fused swiglu (I a multiple of 128,
    bf16/fp16), unfused (other I), float32 (split-bf16 products), routers with and without the
    one-launch front end (E >= 128), single tokens, single experts, k = 1. Forward and every
    gradient against the float32 oracle: 2e-2 relative for 16-bit types, 2e-4 for float32."""
    moe = build(device, E, k, H, I, xma.swiglu_packed, True, dtype, seed)
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(T, H, device=device, generator=g).to(dtype).requires_grad_(True)
    gy = torch.randn(T, H, device=device, generator=g).to(dtype)
    run_and_compare(moe, x, gy, O.swiglu_packed, tol=F32_TOL if dtype == torch.float32 else TOL)


def test_make_graphed_callables(device):
    """torch.cuda.make_graphed_callables records the layer's forward and backward as CUDA graphs with
    autograd kept: the graphed layer trains like the eager one (same outputs and gradients bit for bit)."""
    moe = build(device, 8, 2, 256, 512, xma.swiglu_packed, True, torch.bfloat16, 3)
    T = 512
    sample = torch.randn(T, 256, device=device, dtype=torch.bfloat16, requires_grad=True)
    graphed = torch.cuda.make_graphed_callables(moe, (sample,))
    x = torch.randn(T, 256, device=device, dtype=torch.bfloat16)
    gy = torch.randn(T, 256, device=device, dtype=torch.bfloat16)

    xe = x.clone().requires_grad_(True)
    moe.zero_grad(set_to_none=True)
    ye, _ = moe(xe)
    ye.backward(gy)
    eager = (ye.detach().clone(), xe.grad.clone(), moe.c_fc.weight.grad.clone(), moe.gate.weight.grad.clone())

    xg = x.clone().requires_grad_(True)
    moe.zero_grad(set_to_none=True)
    yg, logits = graphed(xg)
    yg.backward(gy)
    assert_status_clean(device)
    assert logits.shape == (T, 8)
    assert torch.equal(yg, eager[0])
    assert torch.equal(moe.c_fc.weight.grad, eager[2])
    assert torch.equal(xg.grad, eager[1])
    assert torch.equal(moe.gate.weight.grad, eager[3])


def test_router_weight_gradient_is_deterministic(device):
    """d(router weight) is the sum of per-column-tile partials taken in tile order (the reference gets it
    from one bmm, triton_implementation/__init__.py:83): two runs give the same bits, for the gate
    gradient and for the router's share of the input gradient."""
    moe = build(device, 8, 2, 512, 2048, xma.swiglu_packed, True, torch.bfloat16, 4)
    x = torch.randn(2048, 512, device=device, dtype=torch.bfloat16)
    gy = torch.randn(2048, 512, device=device, dtype=torch.bfloat16)
    runs = []
    for _ in range(3):
        moe.zero_grad(set_to_none=True)
        xin = x.clone().requires_grad_(True)
        moe(xin)[0].backward(gy)
        runs.append((xin.grad.clone(), moe.gate.weight.grad.clone()))
    for dx, dgate in runs[1:]:
        assert torch.equal(dx, runs[0][0]) and torch.equal(dgate, runs[0][1])


def test_bounded_wait_runs_out_and_reports(device):
    """The wait every role of the GEMM kernels uses, on a barrier nothing arrives at, with a 1 ms limit:
    the kernel returns, the status word holds the code and the host-side check raises (then clears)."""
    from xma import _native as N

    word = N.status_word(device)
    word.zero_()
    N.check(N.lib().xma_selftest_bounded_wait(word.data_ptr(), 1_000_000, torch.cuda.current_stream(device).cuda_stream),
            "xma_selftest_bounded_wait")
    torch.cuda.synchronize(device)
    assert int(word.item()) == 199
    with pytest.raises(RuntimeError, match="code 199"):
        xma._native.check_status(device)
    assert_status_clean(device)
