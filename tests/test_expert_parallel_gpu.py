"""Expert parallelism on GPUs: the sharded layer must reproduce the single-GPU layer on the same
global batch, with rows moved by NCCL all-to-all ("nccl") or by the fused peer-memory kernels ("peer").
The multi-GPU cases run at world size 2 and at min(visible GPUs, 4) and are skipped when fewer GPUs
are visible; the 1-rank case, the plan checks and the barrier time-limit check run the peer-memory
kernels on a single GPU."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, mode: str) -> None:
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path[:0] = [os.path.join(root, "flash-model-architectures_b200"), root]
    import xma
    from xma import _native as N

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        T, H, I, E, k = 1024, 512, 1024, 8, 2
        torch.manual_seed(0)
        with torch.device(device):
            full = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02).to(torch.bfloat16)
            part = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02, expert_parallel_group=dist.group.WORLD,
                           expert_parallel_mode=mode).to(torch.bfloat16)
        e_local = E // world
        mine = slice(rank * e_local, (rank + 1) * e_local)
        with torch.no_grad():
            full.gate.weight.normal_(0, 0.02)
            part.gate.weight.copy_(full.gate.weight)
            part.c_fc.weight.copy_(full.c_fc.weight[mine])
            part.c_proj.weight.copy_(full.c_proj.weight[mine])
        x = torch.randn(T, H, device=device, dtype=torch.bfloat16)
        gy = torch.randn(T, H, device=device, dtype=torch.bfloat16)
        xf = x.clone().requires_grad_(True)
        yf, logits_f = full(xf)
        yf.backward(gy)
        sl = slice(rank * T // world, (rank + 1) * T // world)
        xp = x[sl].clone().requires_grad_(True)
        for _ in range(2):  # twice: the second pass re-uses the shared buffers of the first
            xp.grad = None
            part.zero_grad(set_to_none=True)
            yp, logits_p = part(xp)
            yp.backward(gy[sl])
        N.check_status(device)
        assert part.expert_parallel_mode == mode  # no silent change of the data path

        rel = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()
        assert torch.equal(logits_p, logits_f[sl])  # same GEMM rows -> same routing
        errs = {
            "y": rel(yp, yf[sl]), "dx": rel(xp.grad, xf.grad[sl]),
            "dw_fc": rel(part.c_fc.weight.grad, full.c_fc.weight.grad[mine]),
            "dw_proj": rel(part.c_proj.weight.grad, full.c_proj.weight.grad[mine]),
        }
        assert all(v <= 2e-2 for v in errs.values()), errs
        # the gate gradient of a rank covers its own tokens; the sum over ranks is the full gradient
        part.all_reduce_router_gradient()
        assert rel(part.gate.weight.grad, full.gate.weight.grad) <= 2e-2

        # Two forward passes, then their two backward passes in reverse order (a layer used twice in
        # one graph, or pipelining): the second backward starts right after the first one's pulls.
        xa = x[sl].clone().requires_grad_(True)
        xb = (x[sl] * 0.5).clone().requires_grad_(True)
        part.zero_grad(set_to_none=True)
        meetings = part._peer_state.seq if mode == "peer" else 0
        ya, _ = part(xa)
        yb, _ = part(xb)
        yb.backward(gy[sl])
        ya.backward(gy[sl])
        N.check_status(device)
        if mode == "peer":
            # forward: count exchange + 2 barriers; backward: 1 barrier + 1 on the second stream, and one
            # more in front of a backward pass that follows another one directly
            assert part._peer_state.seq - meetings == 3 + 3 + 2 + 3
        full.zero_grad(set_to_none=True)
        xfa = x.clone().requires_grad_(True)
        xfb = (x * 0.5).clone().requires_grad_(True)
        yfa, _ = full(xfa)
        yfb, _ = full(xfb)
        (yfa * 1).backward(gy)
        (yfb * 1).backward(gy)
        errs = {
            "ya": rel(ya, yfa[sl]), "yb": rel(yb, yfb[sl]), "dxa": rel(xa.grad, xfa.grad[sl]), "dxb": rel(xb.grad, xfb.grad[sl]),
            "dw_fc": rel(part.c_fc.weight.grad, full.c_fc.weight.grad[mine]),
            "dw_proj": rel(part.c_proj.weight.grad, full.c_proj.weight.grad[mine]),
        }
        assert all(v <= 2e-2 for v in errs.values()), ("two forwards then two backwards", errs)

        # Narrow rows: fewer 16-byte vectors per row (3) than copies per token (4), token counts that
        # are not a multiple of the tile, routing injected so both layers see the same experts.
        T, H, I, E, k = 604, 24, 128, 16, 4
        with torch.device(device):
            full = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02).to(torch.bfloat16)
            part = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02, expert_parallel_group=dist.group.WORLD,
                           expert_parallel_mode=mode).to(torch.bfloat16)
        e_local = E // world
        mine = slice(rank * e_local, (rank + 1) * e_local)
        with torch.no_grad():
            part.c_fc.weight.copy_(full.c_fc.weight[mine])
            part.c_proj.weight.copy_(full.c_proj.weight[mine])
        g = torch.Generator(device=device).manual_seed(11)
        x = torch.randn(T, H, device=device, generator=g).to(torch.bfloat16)
        gy = torch.randn(T, H, device=device, generator=g).to(torch.bfloat16)
        from xma.layers.moe.routing import router_topk_softmax

        sl = slice(rank * T // world, (rank + 1) * T // world)
        logits = torch.randn(T, E, device=device, generator=g)
        one_sided = logits.clone()
        one_sided[:, e_local:] -= 100.0  # every token picks experts of rank 0 only: the other ranks receive no rows
        for case, lg in (("spread", logits), ("all rows to rank 0", one_sided)):
            weights, selected = router_topk_softmax(lg, k)
            weights = weights.to(torch.bfloat16)
            if case != "spread":
                assert int(selected.max()) < e_local
            for m in (full, part):
                m.zero_grad(set_to_none=True)
            xf = x.clone().requires_grad_(True)
            yf = full._compute_experts(xf, weights, selected)
            yf.backward(gy)
            xp = x[sl].clone().requires_grad_(True)
            yp = part._compute_experts(xp, weights[sl], selected[sl])
            yp.backward(gy[sl])
            N.check_status(device)
            errs = {
                "y": rel(yp, yf[sl]), "dx": rel(xp.grad, xf.grad[sl]),
                "dw_proj": rel(part.c_proj.weight.grad, full.c_proj.weight.grad[mine]) if rank == 0 or case == "spread" else 0.0,
                "dw_fc": rel(part.c_fc.weight.grad, full.c_fc.weight.grad[mine]) if rank == 0 or case == "spread" else 0.0,
            }
            assert all(v <= 2e-2 for v in errs.values()), (case, errs)
            if case != "spread" and rank != 0:  # experts without rows: exact zeros
                assert torch.all(part.c_fc.weight.grad == 0) and torch.all(part.c_proj.weight.grad == 0)
    finally:
        dist.destroy_process_group()


def _worlds() -> list[int]:
    """2, and the largest power of two up to 4 that the visible GPUs allow."""
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    return sorted({2, 4 if n >= 4 else 2})


@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_matches_single_gpu(mode, world):
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mp.spawn(_worker, args=(world, _free_port(), mode), nprocs=world, join=True)


def test_peer_path_with_one_rank():
    """World size 1: the fused dispatch / pull kernels, the device-side plan and the GEMMs on the
    shared buffers, without any peer mapping."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    mp.spawn(_worker, args=(1, _free_port(), "peer"), nprocs=1, join=True)


def test_peer_plan_matches_host_arithmetic():
    """xma_ep_plan for every rank of a 4-rank group against the same arithmetic in numpy."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import numpy as np

    from xma import _native as N
    from xma.ops import _launch

    dev = torch.device("cuda", 0)
    world, E = 4, 24
    epr = E // world
    rng = np.random.default_rng(0)
    counts = rng.integers(0, 700, size=(world, E)).astype(np.int32)
    counts[:, 5] = 0  # an expert nobody routes to
    counts_dev = torch.from_numpy(counts).to(dev)
    totals = counts.sum(0)
    padded = (totals + 127) // 128 * 128
    for rank in range(world):
        lpo = torch.empty(epr + 1, dtype=torch.int32, device=dev)
        ltot = torch.empty(epr, dtype=torch.int32, device=dev)
        base = torch.empty(E, dtype=torch.int32, device=dev)
        _launch("xma_ep_plan", counts_dev, N.ptr(counts_dev), E, world, rank, E, 1 << 20, N.ptr(lpo), N.ptr(ltot),
                N.ptr(base), N.ptr(N.status_word(dev)))
        want_base = np.zeros(E, dtype=np.int64)
        for e in range(E):
            owner = e // epr
            want_base[e] = padded[owner * epr:e].sum() + counts[:rank, e].sum()
        mine = slice(rank * epr, (rank + 1) * epr)
        want_lpo = np.concatenate([[0], np.cumsum(padded[mine])])
        assert base.cpu().numpy().tolist() == want_base.tolist()
        assert lpo.cpu().numpy().tolist() == want_lpo.tolist()
        assert ltot.cpu().numpy().tolist() == totals[mine].tolist()


def test_peer_plan_refuses_what_does_not_fit():
    """A rank that would receive more rows than its buffers hold, or ranks whose buffers come from
    different sizing calls: the plan writes a status code, hands out negative rows and no local work,
    and the dispatch kernel then stores nothing (bounds check, no trap)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from xma import _native as N
    from xma.ops import _launch

    dev = torch.device("cuda", 0)
    world, E = 2, 4
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    for case, cap, tags, code in (("overflow", 256, (1, 1), 302), ("generation", 1 << 20, (1, 2), 301)):
        counts = torch.tensor([[200, 100, 7, 9, tags[0]], [300, 50, 1, 2, tags[1]]], dtype=torch.int32, device=dev)
        lpo = torch.full((E // world + 1,), 77, dtype=torch.int32, device=dev)
        ltot = torch.full((E // world,), 77, dtype=torch.int32, device=dev)
        base = torch.full((E,), 77, dtype=torch.int32, device=dev)
        status.zero_()
        _launch("xma_ep_plan", counts, N.ptr(counts), E + 1, world, 0, E, cap, N.ptr(lpo), N.ptr(ltot), N.ptr(base),
                N.ptr(status))
        assert int(status.item()) == code, case
        assert bool((base < 0).all()) and lpo.tolist() == [0, 0, 0] and ltot.tolist() == [0, 0], case

        # the dispatch that follows a refused plan leaves the destination untouched
        T, H, k = 8, 64, 2
        x = torch.randn(T, H, device=dev).to(torch.bfloat16)
        selected = torch.randint(0, E, (T, k), device=dev)
        from xma.layers.moe.routing import build_expert_index

        home = build_expert_index(selected, E, block_m=1)
        dst = torch.full((cap if cap < 4096 else 4096, H), 3.0, device=dev, dtype=torch.bfloat16)
        table = torch.tensor([dst.data_ptr(), dst.data_ptr()], dtype=torch.int64, device=dev)
        dest_rank = torch.empty(T * k, dtype=torch.int32, device=dev)
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        status.zero_()
        _launch("xma_ep_dispatch_rows", x, N.ptr(x), N.dtype_code(x.dtype), H, T, k, N.ptr(selected), N.ptr(home.inv_row),
                N.ptr(home.expert_offsets), N.ptr(home.expert_frequency), N.ptr(base), E // world, N.ptr(table), None,
                None, N.ptr(dest_rank), N.ptr(dest_row), 1, dst.size(0), N.ptr(status))
        assert int(status.item()) == 303, case
        assert bool((dst == 3.0).all()), case


def test_barrier_gives_up_after_its_time_limit():
    """A barrier with a rank that never arrives (a flag word nothing writes): after the limit the
    kernel records code 304 and returns; the context stays usable and the host-side check raises."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from xma import _native as N
    from xma.ops import _launch

    dev = torch.device("cuda", 0)
    mine = torch.zeros(2, dtype=torch.int32, device=dev)      # this rank's flag words; word 1 is never written
    absent = torch.zeros(2, dtype=torch.int32, device=dev)    # stands in for the absent rank's flag words
    table = torch.tensor([mine.data_ptr(), absent.data_ptr()], dtype=torch.int64, device=dev)
    word = N.status_word(dev)
    word.zero_()
    _launch("xma_ep_barrier", table, N.ptr(table), 0, 2, 1, 2_000_000, N.ptr(word))  # 2 ms
    torch.cuda.synchronize(dev)
    assert mine.tolist() == [1, 0] and absent.tolist() == [1, 0]
    with pytest.raises(RuntimeError, match="code 304"):
        N.check_status(dev)
    N.check_status(dev)  # cleared by the failed check
    assert float(torch.ones(4, device=dev).sum()) == 4.0


@pytest.mark.parametrize("world", [4, 8])
def test_peer_kernels_with_emulated_ranks_on_one_gpu(world):
    """The data path of the peer mode for 4 and 8 ranks on ONE GPU: every "rank" is a set of buffers on
    the same device and the ranks' kernels run one after the other (the count exchange with its flag words
    already satisfied, since kernels of different ranks must not wait for each other on one GPU; no
    barrier kernel). Count exchange, plan, prepare, dispatch, the fused GEMMs on every rank's received
    rows and the pull are compared with the single-GPU layer's forward output and with host arithmetic."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import xma
    from xma import _native as N
    from xma import ops
    from xma.layers.moe.routing import build_expert_index, router_topk_softmax
    from xma.ops import _launch

    dev = torch.device("cuda", 0)
    # hidden 1024 with ~130 tokens per rank makes the row movers put four warps on a token (8 ranks);
    # hidden 256 keeps one warp per token (4 ranks)
    T_all, H, I, E, k = 128 * world + 24, (1024 if world == 8 else 256), 128, 16, 2
    epr = E // world
    torch.manual_seed(world)
    with torch.device(dev):
        full = xma.MoE(E, k, H, I, xma.swiglu_packed, True, False, 0.02).to(torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(5)
    x_all = torch.randn(T_all, H, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(T_all, E, device=dev, generator=g)
    weights_all, selected_all = router_topk_softmax(logits, k)
    weights_all = weights_all.to(torch.bfloat16)
    with torch.no_grad():
        want = full._compute_experts(x_all, weights_all, selected_all)

    bounds = [T_all * r // world for r in range(world + 1)]
    cap = N.padded_capacity((bounds[1] - bounds[0] + 1) * world * k, epr)
    i32 = dict(dtype=torch.int32, device=dev)
    rows_in = [torch.full((cap, H), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(world)]
    scale = [torch.zeros(cap, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    rows_out = [torch.empty(cap, H, device=dev, dtype=torch.bfloat16) for _ in range(world)]
    tables = [torch.zeros(world, E + 1, **i32) for _ in range(world)]
    flags = [torch.full((world,), 1, **i32) for _ in range(world)]   # every peer "has arrived" at sequence number 1
    ptrs = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device=dev)
    p_rows_in, p_scale, p_rows_out, p_tables, p_flags = ptrs(rows_in), ptrs(scale), ptrs(rows_out), ptrs(tables), ptrs(flags)
    status = N.status_word(dev)
    status.zero_()

    homes = []
    for r in range(world):   # count exchange, rank by rank
        sel = selected_all[bounds[r]:bounds[r + 1]].contiguous()
        home = build_expert_index(sel, E, block_m=1)
        homes.append((sel, home))
        _launch("xma_ep_exchange_counts", sel, N.ptr(home.expert_frequency.view(torch.int32)), E, 7, N.ptr(p_tables),
                N.ptr(p_flags), r, world, 1, 1_000_000_000, N.ptr(status))
    counts = torch.stack([torch.bincount(s.flatten(), minlength=E) for s, _ in homes]).to(torch.int32)
    for r in range(world):
        assert torch.equal(tables[r][:, :E], counts) and bool((tables[r][:, E] == 7).all())

    plans, dests = [], []
    for r in range(world):   # plan, prepare, dispatch
        sel, home = homes[r]
        lpo, totals, base = torch.empty(epr + 1, **i32), torch.empty(epr, **i32), torch.empty(E, **i32)
        _launch("xma_ep_plan", tables[r], N.ptr(tables[r]), E + 1, world, r, E, cap, N.ptr(lpo), N.ptr(totals), N.ptr(base),
                N.ptr(status))
        row_src = torch.empty(cap, **i32)
        _launch("xma_ep_prepare_rows", rows_in[r], N.ptr(lpo), N.ptr(totals), epr, cap, N.dtype_code(torch.bfloat16), H,
                N.ptr(row_src), N.ptr(rows_in[r]), None)
        plans.append((lpo, totals, row_src))
        xr = x_all[bounds[r]:bounds[r + 1]].contiguous()
        wr = weights_all[bounds[r]:bounds[r + 1]].contiguous()
        t = xr.size(0)
        dest_rank, dest_row = torch.empty(t * k, **i32), torch.empty(t * k, **i32)
        _launch("xma_ep_dispatch_rows", xr, N.ptr(xr), N.dtype_code(xr.dtype), H, t, k, N.ptr(sel), N.ptr(home.inv_row),
                N.ptr(home.expert_offsets), N.ptr(home.expert_frequency), N.ptr(base), epr, N.ptr(p_rows_in), N.ptr(wr),
                N.ptr(p_scale), N.ptr(dest_rank), N.ptr(dest_row), 1, cap, N.ptr(status))
        dests.append((dest_rank, dest_row))
    padded = (counts.sum(0) + 127) // 128 * 128
    for r in range(world):   # the owner's offsets against host arithmetic; every row in use was delivered
        mine = padded[r * epr:(r + 1) * epr].long()
        assert plans[r][0].tolist() == [0] + mine.cumsum(0).tolist()
        used = int(plans[r][0][-1])
        assert not torch.isnan(rows_in[r][:used].float()).any()

    for r in range(world):   # the experts of every rank on the rows it received
        lpo, totals, row_src = plans[r]
        mine = slice(r * epr, (r + 1) * epr)
        pre = torch.empty(cap, 2 * I, device=dev, dtype=torch.bfloat16)
        act = torch.empty(cap, I, device=dev, dtype=torch.bfloat16)
        ops.grouped_gemm_cuda(rows_in[r], full.c_fc.weight.detach()[mine].contiguous(), lpo, pre, act, row_src, scale[r], None,
                              N.GEMM_NT, N.EPI_SWIGLU)
        ops.grouped_gemm_cuda(act, full.c_proj.weight.detach()[mine].contiguous(), lpo, rows_out[r], None, None, None, None,
                              N.GEMM_NT, N.EPI_STORE)
    for r in range(world):   # pull and compare with the single-GPU layer
        t = bounds[r + 1] - bounds[r]
        y = torch.empty(t, H, device=dev, dtype=torch.bfloat16)
        _launch("xma_ep_combine_pull", y, N.ptr(p_rows_out), N.dtype_code(y.dtype), H, N.ptr(dests[r][0]), N.ptr(dests[r][1]),
                t, k, N.ptr(y), cap)
        ref = want[bounds[r]:bounds[r + 1]]
        assert ((y.float() - ref.float()).abs().max() / ref.float().abs().max()).item() <= 2e-2, r
    torch.cuda.synchronize(dev)
    assert int(status.item()) == 0
