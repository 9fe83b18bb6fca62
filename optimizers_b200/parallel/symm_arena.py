"""Peer-addressable device memory for the fused compute+collective kernels.

One ``SymmetricArena`` is a byte buffer allocated identically on every rank of a process group
on one NVLink/NVSwitch domain.  After the rendezvous every rank knows the device address of
every peer's buffer, so kernels can load from and store to peer memory directly
(plain ``ld``/``st`` over NVLink; no TMA multicast is ever pointed at this memory).
``torch.distributed`` (NCCL) is used only for the one-time handle exchange.

The arena is carved into named regions at fixed offsets, identical on every rank, so that an
offset computed locally addresses the same logical object on any peer.  Every region is followed
by a guard of ``_GUARD`` bytes holding a fixed pattern; ``overrun_regions()`` names the regions whose
guard a local or a peer kernel has overwritten (checked on the host by the multi-GPU tests).
"""

from __future__ import annotations

import torch
from torch import distributed as dist, Tensor


_GUARD = 256
_PATTERN = 0xA5


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class SymmetricArena:
    def __init__(self, regions: dict[str, int], device: torch.device, group: dist.ProcessGroup) -> None:
        """``regions`` maps a name to its size in bytes; regions are laid out in dict order."""
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.offsets: dict[str, int] = {}
        self._guards: dict[str, int] = {}
        cursor = 0
        for name, nbytes in regions.items():
            self.offsets[name] = cursor
            cursor += _align(max(nbytes, 1))
            self._guards[name] = cursor
            cursor += _GUARD
        self.nbytes = cursor
        self.local: Tensor = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.local.zero_()
        for start in self._guards.values():
            self.local[start : start + _GUARD].fill_(_PATTERN)
        self._handle = symm_mem.rendezvous(self.local, group=group)
        self.peer_ptrs: list[int] = [int(p) for p in self._handle.buffer_ptrs]
        assert len(self.peer_ptrs) == self.world
        assert self.peer_ptrs[self.rank] == self.local.data_ptr()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def region(self, name: str, nbytes: int | None = None) -> Tensor:
        """Local uint8 view of a region."""
        start = self.offsets[name]
        end = self._guards[name]
        if nbytes is not None:
            end = start + nbytes
        return self.local[start:end]

    def peer_addresses(self, name: str) -> list[int]:
        """Device address of a region on every rank of the group (index = group rank)."""
        off = self.offsets[name]
        return [p + off for p in self.peer_ptrs]

    def overrun_regions(self) -> list[str]:
        """Names of the regions whose trailing guard no longer holds its pattern (host check; waits
        for the device)."""
        return [
            name for name, start in self._guards.items()
            if not bool((self.local[start : start + _GUARD] == _PATTERN).all())
        ]
