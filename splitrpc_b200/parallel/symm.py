"""Process-group bootstrap and symmetric (peer-mapped) device memory.

Every rank allocates the same arena; after the rendezvous each rank knows the
address of every peer's arena in its own address space (NVLink peer mapping), so
kernels can load from and store to a peer with plain instructions.  NVLink
multicast binding is left off: the kernels here only use unicast peer access.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def init_distributed(backend: str = "nccl") -> tuple[int, int, int]:
    """Initialises ``torch.distributed`` from the torchrun environment; returns (rank, world, local_rank)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))
    elif not dist.is_initialized():
        dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world, local_rank


class SymmetricArena:
    """A byte arena that exists at the same offsets on every rank, carved into named tensors.

    ``ptr(name, rank)`` is the address of ``name`` on ``rank`` as seen from this process.
    """

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.group = group or dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, self.group)
        self.base_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self._off = 0
        self._tensors: dict[str, tuple[int, torch.Tensor]] = {}
        torch.cuda.synchronize()
        dist.barrier(self.group)

    def alloc(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._off + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric arena exhausted allocating {name}")
        t = self.buf[off:off + nbytes].view(dtype).view(*shape)
        self._tensors[name] = (off, t)
        self._off = off + nbytes
        return t

    def tensor(self, name: str) -> torch.Tensor:
        return self._tensors[name][1]

    def ptr(self, name: str, rank: int, byte_offset: int = 0) -> int:
        return self.base_ptrs[rank] + self._tensors[name][0] + byte_offset

    def barrier(self) -> None:
        torch.cuda.synchronize()
        dist.barrier(self.group)
