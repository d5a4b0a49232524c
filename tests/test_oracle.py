"""The CPU oracle against golden vectors produced by the reference's own torch path."""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from golden_inputs import GOLDEN_DIR, load, sample
from oracle import moe_oracle as O

ACTS = {
    "moe_small_fp32": O.swiglu_packed,
    "moe_cfg1_fp32": O.swiglu_packed,
    "moe_small_bf16": O.swiglu_packed,
    "moe_glu_fp32": lambda t: F.glu(t, dim=-1),
    "moe_gelu_fp32": lambda t: F.gelu(t, approximate="tanh"),
    "moe_e128_fp32": O.swiglu_packed,
}


@pytest.mark.parametrize("name", list(ACTS))
def test_oracle_matches_reference_goldens(name):
    inp, ref, meta = load(name)
    dtype = torch.bfloat16 if name.endswith("bf16") else torch.float32
    cast = lambda t: t.to(dtype)
    got = O.moe_forward_backward(
        cast(inp["x"]), cast(inp["gate"]), cast(inp["w_fc"]), cast(inp["w_proj"]), meta["k"], cast(inp["grad_y"]), ACTS[name]
    )
    # routing is integer work: exact
    assert torch.equal(got["selected_experts"], ref["selected_experts"])
    # the oracle repeats the reference's operations in the reference's order: float32 results agree to
    # rounding noise of differently-ordered sums only where the stable sort reorders rows inside one
    # expert (index_add order). atol is in units of the tensors' own scale.
    tol = dict(rtol=0, atol=2e-6) if dtype == torch.float32 else dict(rtol=0, atol=2e-2)
    for key in ("y", "router_logits", "router_weights", "dx", "dgate"):
        torch.testing.assert_close(got[key].float(), ref[key], **tol, msg=lambda m, key=key: f"{key}: {m}")
    for key in ("dw_fc", "dw_proj"):
        if key in ref:
            torch.testing.assert_close(got[key].float(), ref[key], **tol)
        else:
            torch.testing.assert_close(sample(got[key].float()), ref[key + "_sample"], **tol)
            assert abs(got[key].double().abs().sum().item() - float(ref[key + "_abs_sum"])) <= 1e-4 * float(ref[key + "_abs_sum"])


def test_continuous_count_goldens():
    rec = np.load(f"{GOLDEN_DIR}/continuous_count.npz")
    for key in rec.files:
        if key.startswith("ids_"):
            n = key.split("_")[1]
            got = O.continuous_count(torch.from_numpy(rec[key]), 72)
            assert got.dtype == torch.uint32
            assert np.array_equal(got.numpy().astype(np.int64), rec[f"count_{n}"])
    got = O.continuous_count(torch.from_numpy(rec["ids_9"]), 1)
    assert np.array_equal(got.numpy().astype(np.int64), rec["count_bins1"])


def test_swiglu_packed_goldens():
    rec = np.load(f"{GOLDEN_DIR}/swiglu_packed.npz")
    x = torch.from_numpy(rec["x"]).requires_grad_(True)
    y = O.swiglu_packed(x)
    y.backward(torch.from_numpy(rec["dy"]))
    # the reference's own float32 tolerances (tests/functional/swiglu_packed_test.py:55-61)
    torch.testing.assert_close(y.detach(), torch.from_numpy(rec["y"]), rtol=0, atol=4.9e-5)
    torch.testing.assert_close(x.grad, torch.from_numpy(rec["dx"]), rtol=0, atol=5e-6)


def test_swiglu_goldens():
    rec = np.load(f"{GOLDEN_DIR}/swiglu.npz")
    g = torch.from_numpy(rec["gate"]).requires_grad_(True)
    u = torch.from_numpy(rec["up"]).requires_grad_(True)
    y = O.swiglu(g, u)
    y.backward(torch.from_numpy(rec["dy"]))
    # the reference's own float32 tolerances (tests/functional/swiglu_test.py:58-65)
    torch.testing.assert_close(y.detach(), torch.from_numpy(rec["y"]), rtol=0, atol=5.4e-5)
    torch.testing.assert_close(g.grad, torch.from_numpy(rec["dgate"]), rtol=0, atol=5e-6)
    torch.testing.assert_close(u.grad, torch.from_numpy(rec["dup"]), rtol=0, atol=5e-6)


def test_sort_is_stable_and_consistent():
    torch.manual_seed(0)
    sel = torch.randint(0, 6, (37, 3))
    se, ss, freq, off = O.sort_experts(sel, 6)
    assert torch.equal(se, sel.flatten()[ss])
    assert torch.all(se[1:] >= se[:-1])
    same = se[1:] == se[:-1]
    assert torch.all(ss[1:][same] > ss[:-1][same])  # ascending flat index inside one expert
    assert int(off[-1]) == sel.numel() and torch.equal(off, freq.long().cumsum(0))
