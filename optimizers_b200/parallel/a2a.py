"""Single-collective shard exchange between FSDP2 dim-0 shards and whole-parameter owners.

Under the lossless ROUND_ROBIN strategy each full parameter has one owner rank in the shard
group.  Two exchanges per step, each one ``all_to_all`` over persistent flat buffers:

* gather   every rank sends its local dim-0 shard of parameter i (its gradient, or its value) to
           the owner of i, which concatenates the shards into the full tensor;
* scatter  every owner cuts its updated full parameters into dim-0 chunks and sends chunk r to
           rank r, which copies it into its local shard.

Chunk sizes reproduce ``torch.chunk`` exactly (ceil-sized leading chunks, possibly empty trailing
ones), because that is how ``fully_shard`` lays out dim-0 shards.  Buffer layout, identical on
both sides of a transfer: the section exchanged with peer r lists the parameters concerned in
ascending parameter index.  Peak memory of a gather is O(total_params / group_size) per rank
instead of O(total_params) for per-parameter ``full_tensor()`` calls.

Reference counterparts: ``distributed_shampoo/utils/shampoo_fully_shard_utils.py``
(chunk math :111-186, ``AllToAllContext`` :254-373, ``RedistributeParamsContext`` :376-588,
``GatherGradientsContext`` :591-858, legacy multi-round helpers :26-108).
"""

from __future__ import annotations

import abc
import contextlib
import logging
import math
from collections.abc import Callable
from itertools import accumulate

import torch
from torch import distributed as dist, Tensor
from torch.distributed.tensor import DTensor

logger: logging.Logger = logging.getLogger(__name__)


def _compute_chunk_sizes(numel: int, num_chunks: int) -> list[int]:
    """Sizes ``torch.chunk`` gives when cutting ``numel`` rows into ``num_chunks`` chunks, padded
    with zeros to exactly ``num_chunks`` entries."""
    if numel == 0:
        return [0] * num_chunks
    step = -(-numel // num_chunks)
    sizes = []
    left = numel
    for _ in range(num_chunks):
        take = min(step, left)
        sizes.append(take)
        left -= take
    return sizes


def _compute_param_chunk_sizes(params: tuple[DTensor, ...], group_size: int) -> list[list[int]]:
    """Per parameter: number of elements of its dim-0 chunk on every rank (a 0-d parameter lives
    entirely on rank 0)."""
    out = []
    for p in params:
        shape = tuple(p.shape)
        if not shape:
            out.append([1] + [0] * (group_size - 1))
            continue
        row = math.prod(shape[1:])
        out.append([c * row for c in _compute_chunk_sizes(shape[0], group_size)])
    return out


_default_comm_path = "nccl"
# Device types whose memory the peer exchange can address from every rank.  Tests that stand in
# shared host memory for NVLink peers add "cpu".
_PEER_DEVICE_TYPES: tuple[str, ...] = ("cuda",)


@contextlib.contextmanager
def exchange_comm_path(comm_path: str):
    """Contexts created inside use ``comm_path`` ("nccl": all_to_all collective; "p2p": stores
    into peer memory from inside one kernel) unless they are given one explicitly."""
    global _default_comm_path
    previous, _default_comm_path = _default_comm_path, comm_path
    try:
        yield
    finally:
        _default_comm_path = previous


def _views(buffer: Tensor, sizes: list[int]) -> list[Tensor]:
    ends = list(accumulate(sizes))
    return [buffer[e - s : e] for s, e in zip(sizes, ends, strict=True)]


class AllToAllContext(abc.ABC):
    """Metadata and persistent buffers of one direction of the exchange."""

    @torch.no_grad()
    def __init__(
        self,
        params: tuple[DTensor, ...],
        assigned_params_mask: tuple[bool, ...],
        dist_group: dist.ProcessGroup,
        owner_ranks: list[int] | None = None,
        comm_path: str | None = None,
    ) -> None:
        if not params:
            raise ValueError("params cannot be empty")
        if len(params) != len(assigned_params_mask):
            raise ValueError(
                f"len(params) ({len(params)}) != len(assigned_params_mask) ({len(assigned_params_mask)})"
            )
        self._params = tuple(params)
        self._assigned_params_mask = tuple(assigned_params_mask)
        self._dist_group = dist_group
        self._group_size = dist_group.size()
        self._rank = dist.get_rank(group=dist_group)
        n = self._group_size
        self._owner_ranks = list(owner_ranks) if owner_ranks is not None else [i % n for i in range(len(params))]
        if len(self._owner_ranks) != len(params):
            raise ValueError(f"len(owner_ranks) ({len(self._owner_ranks)}) != len(params) ({len(params)})")
        first = params[0].to_local()
        self._dtype, self._device = first.dtype, first.device
        if any(p.to_local().dtype != self._dtype for p in params):
            raise NotImplementedError("Parameters of different dtypes are not currently supported.")

        self._local_param_indices = [i for i, mine in enumerate(self._assigned_params_mask) if mine]
        self._param_chunk_sizes = _compute_param_chunk_sizes(self._params, n)
        self._params_owned_by = [[i for i, o in enumerate(self._owner_ranks) if o == r] for r in range(n)]
        self._send_sizes, self._recv_sizes = self._compute_send_recv_sizes()
        self._total_send_size, self._total_recv_size = sum(self._send_sizes), sum(self._recv_sizes)
        self._send_buffer = torch.empty(self._total_send_size, dtype=self._dtype, device=self._device)
        self._recv_buffer = torch.empty(self._total_recv_size, dtype=self._dtype, device=self._device)
        self._p2p = (comm_path or _default_comm_path) == "p2p" and self._device.type in _PEER_DEVICE_TYPES and n > 1
        if self._p2p:
            self._setup_peer_exchange()
        self._send_list = _views(self._send_buffer, self._send_sizes)
        self._recv_list = _views(self._recv_buffer, self._recv_sizes)
        self._precompute_subclass_metadata()

    @abc.abstractmethod
    def _compute_send_recv_sizes(self) -> tuple[list[int], list[int]]: ...

    @abc.abstractmethod
    def _precompute_subclass_metadata(self) -> None: ...

    # ------------------------------------------------------------------------------------------
    # Peer-memory exchange (comm_path="p2p"): the receive buffer lives in memory every rank of the
    # group can address; senders store their sections straight into it from the source tensors.
    # ------------------------------------------------------------------------------------------
    def _section_sizes(self, sender: int, receiver: int) -> int:
        """Elements ``sender`` delivers to ``receiver`` (known to every rank from the shared metadata)."""
        raise NotImplementedError

    def _setup_peer_exchange(self) -> None:
        from optimizers_b200.ops import build
        from optimizers_b200.parallel.symm_arena import SymmetricArena

        n, es = self._group_size, torch.empty(0, dtype=self._dtype).element_size()
        if es != 4:
            raise NotImplementedError("comm_path='p2p' of the lossless exchange supports 4-byte parameter dtypes")
        if n > 8:
            raise RuntimeError("comm_path='p2p' needs all ranks of the shard group on one NVLink domain (at most 8)")
        self._ext = build.load()
        sizes = [[self._section_sizes(q, r) for r in range(n)] for q in range(n)]
        assert [sizes[q][self._rank] for q in range(n)] == self._recv_sizes
        assert sizes[self._rank] == self._send_sizes
        recv_total = max(sum(sizes[q][r] for q in range(n)) for r in range(n))
        self._arena = SymmetricArena({"recv": recv_total * es, "flags": 2 * 32 * 4}, self._device, self._dist_group)
        self._recv_buffer = self._arena.region("recv", self._total_recv_size * es).view(self._dtype)
        # byte address of this rank's section inside every receiver's buffer
        bases = self._arena.peer_addresses("recv")
        self._dest_base = [bases[r] + sum(sizes[q][r] for q in range(self._rank)) * es for r in range(n)]
        self._flags = self._arena.region("flags").view(torch.int32)
        self._flag_bases = [
            torch.tensor([a + k * 128 for a in self._arena.peer_addresses("flags")], dtype=torch.int64, device=self._device)
            for k in range(2)
        ]
        self._status = torch.zeros(1, dtype=torch.int32, device=self._device)
        self._barrier_seq = 0
        self._zeros = torch.zeros(0, dtype=self._dtype, device=self._device)

    def _peer_barrier(self, which: int) -> None:
        self._ext.peer_barrier(
            self._flags[which * 32 : which * 32 + 32], self._flag_bases[which], self._rank, self._group_size,
            self._barrier_seq, self._status,
        )

    def _execute_peer_push(self, sections: list[list[Tensor | int]]) -> None:
        """``sections[r]``: the tensors (or, for an absent source, the element count to zero-fill)
        that make up this rank's section for receiver ``r``, in section order."""
        es = 4
        self._barrier_seq += 1
        self._peer_barrier(0)  # every receiver has consumed the previous exchange
        specs = []
        need_zero = max((x for sec in sections for x in sec if isinstance(x, int)), default=0)
        if need_zero > self._zeros.numel():
            self._zeros = torch.zeros(need_zero, dtype=self._dtype, device=self._device)
        keep = []
        for r, sec in enumerate(sections):
            at = self._dest_base[r]
            for x in sec:
                if isinstance(x, int):
                    src, count = self._zeros, x
                else:
                    src = x if x.is_contiguous() else x.contiguous()
                    count = src.numel()
                    keep.append(src)
                specs.append((src.data_ptr(), at, count * es))
                at += count * es
        table = self._ext.build_copy_table(specs, self._device.index)
        self._ext.peer_copy(*table)
        self._peer_barrier(1)  # every sender's stores have landed
        self._keep_alive = (keep, table)

    def check_status(self) -> None:
        if self._p2p and int(self._status.item()) & 4:
            raise RuntimeError("a peer rank did not reach the exchange barrier in time (bounded device-side wait expired)")

    def _execute_all_to_all(self) -> None:
        # The sections are contiguous in the flat buffers, so the single-tensor form applies; it
        # also exists on every backend (gloo has no list all_to_all).
        dist.all_to_all_single(
            self._recv_buffer,
            self._send_buffer,
            output_split_sizes=self._recv_sizes,
            input_split_sizes=self._send_sizes,
            group=self._dist_group,
        )

    # sizes of the two kinds of section: what owners exchange with shard holders
    def _shards_for_owner(self, owner: int) -> int:
        """Elements this rank's shards contribute to the parameters owned by ``owner``."""
        return sum(self._param_chunk_sizes[i][self._rank] for i in self._params_owned_by[owner])

    def _chunks_of_mine_on(self, peer: int) -> int:
        """Elements of this rank's own parameters that live on ``peer``."""
        return sum(self._param_chunk_sizes[i][peer] for i in self._local_param_indices)


class GatherGradientsContext(AllToAllContext):
    """Shards -> owners (gradients every step, parameter values at set-up and after a load)."""

    def _compute_send_recv_sizes(self) -> tuple[list[int], list[int]]:
        n = self._group_size
        return [self._shards_for_owner(r) for r in range(n)], [self._chunks_of_mine_on(r) for r in range(n)]

    def _precompute_subclass_metadata(self) -> None:
        n = self._group_size
        self._param_global_shapes = [tuple(p.shape) for p in self._params]
        # send side: for peer r, my shard of every parameter r owns
        self._send_plan: list[tuple[int, int, Tensor]] = []  # (param index, chunk numel, destination view)
        cursor = 0
        for r in range(n):
            for i in self._params_owned_by[r]:
                size = self._param_chunk_sizes[i][self._rank]
                if size > 0:
                    self._send_plan.append((i, size, self._send_buffer[cursor : cursor + size]))
                    cursor += size
        # receive side: section r holds chunk r of each of my parameters; assemble per parameter
        section_start = [0, *accumulate(self._recv_sizes)][:-1]
        self._full_buffers: list[Tensor] = []
        self._unpack_src: list[Tensor] = []
        self._unpack_dst: list[Tensor] = []
        offsets = list(section_start)
        pieces: dict[int, list[tuple[int, int]]] = {i: [] for i in self._local_param_indices}
        for r in range(n):
            for i in self._local_param_indices:
                size = self._param_chunk_sizes[i][r]
                pieces[i].append((offsets[r], size))
                offsets[r] += size
        for i in self._local_param_indices:
            full = torch.empty(sum(s for _, s in pieces[i]), dtype=self._dtype, device=self._device)
            self._full_buffers.append(full)
            at = 0
            for start, size in pieces[i]:
                if size > 0:
                    self._unpack_src.append(self._recv_buffer[start : start + size])
                    self._unpack_dst.append(full[at : at + size])
                    at += size
        logger.info(
            f"GatherGradientsContext initialized: rank={self._rank}, group_size={n}, num_params={len(self._params)}, "
            f"local_params={len(self._local_param_indices)}, send_sizes={self._send_sizes}, recv_sizes={self._recv_sizes}"
        )

    def _pack_send_buffer(self, data_source: Callable[[int], Tensor | None]) -> None:
        src, dst = [], []
        for i, size, view in self._send_plan:
            data = data_source(i)
            if data is None:
                view.zero_()
            else:
                src.append(data[:size])
                dst.append(view)
        if dst:
            torch._foreach_copy_(dst, src)

    def _unpack_recv_buffer(self, has_grad: list[bool]) -> list[Tensor | None]:
        if self._unpack_dst:
            torch._foreach_copy_(self._unpack_dst, self._unpack_src)
        out: list[Tensor | None] = [None] * len(self._params)
        for full, i in zip(self._full_buffers, self._local_param_indices, strict=True):
            if has_grad[i]:
                shape = self._param_global_shapes[i]
                out[i] = full.squeeze() if not shape else full.view(shape)
        return out

    def _section_sizes(self, sender: int, receiver: int) -> int:
        return sum(self._param_chunk_sizes[i][sender] for i in self._params_owned_by[receiver])

    def _exchange(self, source: Callable[[int], Tensor | None], present: list[bool]) -> list[Tensor | None]:
        if self._p2p:
            sections: list[list[Tensor | int]] = [[] for _ in range(self._group_size)]
            for r in range(self._group_size):
                for i in self._params_owned_by[r]:
                    size = self._param_chunk_sizes[i][self._rank]
                    if size > 0:
                        data = source(i)
                        sections[r].append(size if data is None else data[:size])
            self._execute_peer_push(sections)
        else:
            self._pack_send_buffer(source)
            self._execute_all_to_all()
        # Clones: the persistent buffers are overwritten by the next exchange.
        return [t.clone() if t is not None else None for t in self._unpack_recv_buffer(present)]

    @torch.no_grad()
    def gather_gradients(self) -> list[Tensor | None]:
        """Full gradients of this rank's parameters (``None`` elsewhere and where no gradient exists)."""
        has_grad = [p.grad is not None for p in self._params]

        def source(i: int) -> Tensor | None:
            return self._params[i].grad.to_local().flatten() if has_grad[i] else None

        return self._exchange(source, has_grad)

    @torch.no_grad()
    def gather_params(self) -> list[Tensor | None]:
        """Full values of this rank's parameters (``None`` for the others)."""
        return self._exchange(lambda i: self._params[i].to_local().flatten(), [True] * len(self._params))


class RedistributeParamsContext(AllToAllContext):
    """Owners -> shards: the mirror image of the gather."""

    def _compute_send_recv_sizes(self) -> tuple[list[int], list[int]]:
        n = self._group_size
        return [self._chunks_of_mine_on(r) for r in range(n)], [self._shards_for_owner(r) for r in range(n)]

    def _section_sizes(self, sender: int, receiver: int) -> int:
        return sum(self._param_chunk_sizes[i][receiver] for i in self._params_owned_by[sender])

    def _precompute_subclass_metadata(self) -> None:
        n = self._group_size
        self._param_local_numels = [p.to_local().numel() for p in self._params]
        self._param_global_numels = [p.numel() for p in self._params]
        self._local_position = {i: k for k, i in enumerate(self._local_param_indices)}
        self._local_param_global_shapes = [tuple(self._params[i].shape) for i in self._local_param_indices]
        # send side: section r holds chunk r of each of my parameters
        self._send_plan: list[tuple[int, int, Tensor]] = []  # (param index, peer, destination view)
        cursor = 0
        for r in range(n):
            for i in self._local_param_indices:
                size = self._param_chunk_sizes[i][r]
                if size > 0:
                    self._send_plan.append((i, r, self._send_buffer[cursor : cursor + size]))
                    cursor += size
        # receive side: section r holds my shard of every parameter r owns
        self._recv_src: list[Tensor] = []
        self._recv_dst: list[Tensor] = []
        cursor = 0
        for r in range(n):
            for i in self._params_owned_by[r]:
                size = self._param_chunk_sizes[i][self._rank]
                if size > 0:
                    local = self._params[i].to_local()
                    assert size == local.numel(), f"chunk_size ({size}) != local_numel ({local.numel()}) for param {i}"
                    self._recv_src.append(self._recv_buffer[cursor : cursor + size])
                    self._recv_dst.append(local.flatten())
                cursor += size
        logger.info(
            f"RedistributeParamsContext initialized: rank={self._rank}, group_size={n}, num_params={len(self._params)}, "
            f"local_params={len(self._local_param_indices)}, send_sizes={self._send_sizes}, recv_sizes={self._recv_sizes}"
        )

    @torch.no_grad()
    def redistribute_and_update_params(self, local_full_params: list[Tensor]) -> None:
        """Send every owned, updated full parameter back to the ranks holding its shards and copy
        what arrives into the local shards."""
        assert len(local_full_params) == len(self._local_param_indices), (
            f"Expected {len(self._local_param_indices)} local params, got {len(local_full_params)}"
        )
        n = self._group_size
        chunks: list[list[Tensor]] = []
        for full, shape in zip(local_full_params, self._local_param_global_shapes, strict=True):
            parts = [full.flatten()] if not shape else [c.flatten() for c in torch.chunk(full.view(shape), n, dim=0)]
            parts += [full.new_empty(0)] * (n - len(parts))
            chunks.append(parts)
        src = [chunks[self._local_position[i]][r] for i, r, _ in self._send_plan]
        if self._p2p:
            sections: list[list[Tensor | int]] = [[] for _ in range(n)]
            for (_, r, _), piece in zip(self._send_plan, src, strict=True):
                sections[r].append(piece)
            self._execute_peer_push(sections)
        else:
            dst = [view for _, _, view in self._send_plan]
            if dst:
                torch._foreach_copy_(dst, src)
            self._execute_all_to_all()
        if self._recv_dst:
            torch._foreach_copy_(self._recv_dst, self._recv_src)


# ----------------------------------------------------------------------------------------------
# Legacy multi-round exchange (one all_to_all per parameter); kept for API parity.
# ----------------------------------------------------------------------------------------------
def prepare_update_param_buffers(params: tuple[DTensor, ...], group_size: int) -> list[Tensor]:
    """One flat receive buffer cut at the local-shard boundaries, padded with empty views to a
    multiple of ``group_size`` entries (one entry per all_to_all slot)."""
    if any(p.dtype != params[0].dtype for p in params):
        raise NotImplementedError(
            "When using round-robin assignment in FSDP Shampoo, parameters of different dtypes are not currently supported."
        )
    sizes = [p.to_local().numel() for p in params]
    total = sum(sizes)
    buffer = params[0].to_local().new_zeros(total)
    cuts = list(accumulate(sizes))
    cuts += [total] * (-len(cuts) % group_size)
    return list(torch.tensor_split(buffer, cuts[:-1]))


def redistribute_and_update_params(
    params: tuple[DTensor, ...], local_full_params: list[Tensor], update_param_buffers: list[Tensor], dist_group: dist.ProcessGroup
) -> None:
    """Round k: the rank owning parameter ``k*group_size + rank`` sends its dim-0 chunks to
    everyone; ranks without a parameter in that round send empties."""
    n = dist_group.size()
    rounds = len(update_param_buffers) // n
    logger.info(f"Running {rounds} rounds of a2a ops.")
    for k in range(rounds):
        full = local_full_params[k] if k < len(local_full_params) else params[0].to_local().new_zeros(0)
        send = [t.flatten() for t in torch.chunk(full, n, dim=0)]
        send += [send[-1][send[-1].shape[0] :]] * (n - len(send))
        dist.all_to_all(update_param_buffers[k * n : (k + 1) * n], send, dist_group)
    torch._foreach_copy_([p.to_local().flatten() for p in params], update_param_buffers[: len(params)])
