"""Expert parallelism on 2 GPUs (NCCL): the sharded layer must reproduce the single-GPU layer on the
same global batch. Skipped when fewer than 2 GPUs are visible."""

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

        rel = lambda a, b: ((a.float() - b.float()).abs().max() / b.float().abs().max()).item()
        assert torch.equal(logits_p, logits_f[sl])  # same GEMM rows -> same routing
        errs = {
            "y": rel(yp, yf[sl]), "dx": rel(xp.grad, xf.grad[sl]),
            "dw_fc": rel(part.c_fc.weight.grad, full.c_fc.weight.grad[mine]),
            "dw_proj": rel(part.c_proj.weight.grad, full.c_proj.weight.grad[mine]),
        }
        assert all(v <= 2e-2 for v in errs.values()), errs
        # the gate gradient of a rank covers its own tokens; the sum over ranks is the full gradient
        g = part.gate.weight.grad.float().clone()
        dist.all_reduce(g)
        assert rel(g, full.gate.weight.grad) <= 2e-2
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_matches_single_gpu(mode):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port(), mode), nprocs=2, join=True)
