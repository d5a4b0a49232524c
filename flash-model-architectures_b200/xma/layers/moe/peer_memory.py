"""Device buffers of every rank of a process group mapped into this process (CUDA IPC).

One process per GPU on one node: each rank allocates its buffer with the ordinary allocator, shares
the allocation's IPC handle through the group's object all-gather, and opens the other ranks'
handles. Kernels then reach a peer's buffer with plain loads and stores over NVLink. The table of
base addresses lives on the device as int64[world]."""

from __future__ import annotations

import torch
import torch.distributed as dist


_opened: dict[bytes, list] = {}  # IPC handle -> [base address in this process, users] (an allocation is opened once)


def _open(handle: bytes) -> int:
    entry = _opened.get(handle)
    if entry is None:
        import ctypes

        from ... import _native as N

        out = ctypes.c_void_p()
        N.check(N.lib().xma_ipc_open_handle(handle, ctypes.byref(out)), "xma_ipc_open_handle")
        entry = _opened[handle] = [int(out.value), 0]
    entry[1] += 1
    return entry[0]


def _close(handle: bytes) -> None:
    """Drops one user of a mapping; the last one unmaps it (the owner can then return the memory)."""
    entry = _opened.get(handle)
    if entry is None:
        return
    entry[1] -= 1
    if entry[1] <= 0:
        from ... import _native as N

        del _opened[handle]
        N.check(N.lib().xma_ipc_close_handle(entry[0]), "xma_ipc_close_handle")


class PeerBuffer:
    """`local` is this rank's buffer; `table` is an int64[world] device tensor of every rank's base
    address as mapped here (entry `rank` is `local` itself)."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group, zero: bool = False) -> None:
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = device
        self._handles: list[bytes] = []
        # `zero`: cleared before any peer can reach it (the collective at the end of this constructor
        # synchronises the stream on every rank).
        self.local = (torch.zeros if zero else torch.empty)(numel, dtype=dtype, device=device)
        # torch's exporter tells where the storage sits inside its cudaMalloc allocation (and keeps
        # that allocation alive while it is shared); the IPC handle itself comes from the library.
        failure = None
        mine = None
        try:
            shared = self.local.untyped_storage()._share_cuda_()
            offset = int(shared[3]) + self.local.storage_offset() * self.local.element_size()
            import ctypes

            from ... import _native as N

            raw = ctypes.create_string_buffer(64)
            with torch.cuda.device(device):
                N.check(N.lib().xma_ipc_get_handle(self.local.data_ptr() - offset, raw), "xma_ipc_get_handle")
            mine = (raw.raw, offset)
        except RuntimeError as error:
            failure = error
        handles: list = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        addresses = []
        try:
            if failure is None and any(h is None for h in handles):
                raise RuntimeError("a rank could not export its buffer")
            if failure is not None:
                raise failure
            with torch.cuda.device(device):
                for r in range(self.world):
                    if r == self.rank:
                        addresses.append(self.local.data_ptr())
                    else:
                        addresses.append(_open(handles[r][0]) + handles[r][1])
                        self._handles.append(handles[r][0])
        except RuntimeError as error:  # e.g. the ranks are not on one node, or IPC is not permitted here
            failure = error
        # Every rank learns whether every rank could map every buffer (also the barrier after the mapping).
        ok = torch.tensor([0 if failure is not None else 1], dtype=torch.int32, device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer mapping of device buffers failed on at least one rank ({failure})")
        self.table = torch.tensor(addresses, dtype=torch.int64, device=device)

    def close(self) -> None:
        """Unmaps the peers' buffers. The caller makes sure no kernel of any rank still uses them."""
        with torch.cuda.device(self.device):
            for handle in self._handles:
                _close(handle)
        self._handles = []
        self.table = None

    def view(self, *shape: int) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        return self.local[:n].view(*shape)
