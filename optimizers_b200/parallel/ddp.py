"""DDP distributor: ZeRO-1 style sharing of the optimizer work under data parallelism.

Parameters and gradients are replicated (the data-parallel wrapper all-reduces the gradients).
Ranks are cut into groups of ``num_trainers_per_group``; inside a group every block has one
owner, chosen by longest-processing-time-first balancing on the block's aligned size in the
communication dtype.  Only the owner keeps state for a block and computes its search direction;
one all-gather per step then hands every rank all directions (or, with ``communicate_params``,
the updated parameters themselves).

Buffer layout (part of the behaviour other ranks and the fused kernels rely on): one int8 buffer
of ``group_size`` equal chunks; chunk r holds rank r's blocks back to back in global block
order, each block starting at a multiple of 64 bytes; a block's slot is viewed in the
communication dtype with the block's shape.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_ddp_distributor.py:131-589``.
"""

from __future__ import annotations

import logging
from collections.abc import Iterable
from functools import partial
from typing import Any

import torch
from torch import distributed as dist, Tensor
from torch.distributed.tensor import DTensor

from optimizers_b200.config import DDPDistributedConfig, DISTRIBUTED_CONFIG, PARAMS, ShampooRuntimeConfig
from optimizers_b200.parallel.base import DistributorInterface
from optimizers_b200.parallel.block_info import DTensorBlockInfo
from optimizers_b200.parallel.dist_utils import allocate_zeros_on_owner, batched, get_device_mesh, shampoo_comm_profiler
from optimizers_b200.utils.blocking import (
    compress_list,
    distribute_buffer_sizes,
    generate_pairwise_indices,
    get_dtype_size,
)

logger: logging.Logger = logging.getLogger(__name__)


def carve_block_buffers(
    global_buffer: Tensor,
    buffer_size_ranks: tuple[tuple[int, int], ...],
    blocks: tuple[Tensor, ...],
    group_size: int,
    communication_dtype: torch.dtype,
) -> tuple[Tensor, tuple[Tensor, ...], tuple[int, ...]]:
    """Split ``global_buffer`` into per-rank chunks and per-block typed views.

    Returns ``(chunks, per-block views in global block order, per-block byte offsets inside the
    global buffer)``."""
    chunk = global_buffer.numel() // group_size
    cursor = [0] * group_size
    views: list[Tensor] = []
    offsets: list[int] = []
    elem = get_dtype_size(communication_dtype)
    for (aligned_bytes, rank), block in zip(buffer_size_ranks, blocks, strict=True):
        start = rank * chunk + cursor[rank]
        cursor[rank] += aligned_bytes
        assert cursor[rank] <= chunk, "per-rank chunk is too small for its blocks"
        raw = global_buffer[start : start + block.numel() * elem]
        views.append(raw.view(communication_dtype).view(block.shape))
        offsets.append(start)
    return tuple(torch.split(global_buffer, chunk)) if chunk else (), tuple(views), tuple(offsets)


class DDPDistributor(DistributorInterface):
    def __init__(
        self,
        param_group: dict[str, Any],
        runtime_config: ShampooRuntimeConfig | None = None,
        dist_group: dist.ProcessGroup | None = dist.distributed_c10d.GroupMember.WORLD,
    ) -> None:
        super().__init__(param_group, runtime_config)
        cfg: DDPDistributedConfig = param_group[DISTRIBUTED_CONFIG]
        self._global_masked_blocked_params: tuple[Tensor, ...] = self._global_blocked_params
        self._communicate_params: bool = cfg.communicate_params
        self._communication_dtype: torch.dtype = cfg.communication_dtype
        self._block_id_rank: int | None = None
        self._resolve_group(cfg, dist_group)
        self._group_rank: int = dist.get_rank(group=self._dist_group)

        # Ownership is decided on meta tensors in the communication dtype: no memory, exact sizes.
        meta_blocks = tuple(b.to(device="meta", dtype=cfg.communication_dtype) for b in self._global_blocked_params)
        self._buffer_size_ranks = distribute_buffer_sizes(meta_blocks, self._group_size, cfg.load_balancing_config)
        owners = tuple(rank for _, rank in self._buffer_size_ranks)
        self._block_owner_ranks: tuple[int, ...] = owners
        self._distributor_selector = tuple(r == self._group_rank for r in owners)
        self._local_block_info_list = self._construct_local_block_info_list(owners, self._group_rank)
        self._local_blocked_params = compress_list(self._global_blocked_params, self._distributor_selector)
        self._local_masked_blocked_params = self._local_blocked_params
        self._local_grad_selector = (True,) * len(self._local_blocked_params)
        self._construct_distributed_buffers(self._buffer_size_ranks, cfg.communication_dtype, self._group_rank)

    def _resolve_group(self, cfg: DDPDistributedConfig, dist_group: dist.ProcessGroup | None) -> None:
        """Decide which ranks share the work of this parameter group.  Sets ``_dist_group`` (the
        all-gather group), ``_group_size``, ``_global_size`` and ``_owner_mesh_rows`` (the
        replicate x shard arrangement used to place state DTensors on their owners)."""
        self._global_size: int = dist.get_world_size(group=dist_group)
        if cfg.num_trainers_per_group == -1:
            logger.info(
                f"Note that distributed_config.num_trainers_per_group={cfg.num_trainers_per_group}! Defaulting to world size {self._global_size}."
            )
        self._group_size: int = cfg.num_trainers_per_group if cfg.num_trainers_per_group != -1 else self._global_size
        # Collective: every rank creates every sub-group and keeps its own.
        self._dist_group: dist.ProcessGroup = dist.new_subgroups(group_size=self._group_size, group=dist_group)[0]
        # The mesh must be the same object request on every rank (its creation is collective): all
        # ranks of the parent group, one row per sub-group.  Column j then is the set of ranks that
        # hold identical copies of the state owned by the j-th member of each sub-group.
        parent = dist_group if dist_group is not None else dist.group.WORLD
        all_ranks = dist.get_process_group_ranks(group=parent)
        self._owner_mesh_rows: tuple[tuple[int, ...], ...] = tuple(batched(all_ranks, self._group_size))
        # Made here, on every rank, and not when the first state tensor is allocated: a rank that owns
        # no block allocates no state, and a mesh (its process groups) created by the other ranks
        # only never completes under NCCL with communicators bound at start-up
        # (init_process_group(device_id=...)): measured as a hang of every rank.
        device_type = self._param_group[PARAMS][0].device.type
        mesh = get_device_mesh(device_type=device_type, mesh=self._owner_mesh_rows, mesh_dim_names=("replicate", "shard"))
        mesh._get_all_submeshes(mesh_dim_name="replicate")  # type: ignore[attr-defined]

    # -- parameters may be DTensors (composable replicate()) ------------------------------------
    @torch.no_grad()
    def _get_params_or_grads(self, get_grad: bool = False) -> Iterable[Tensor | None]:
        def local(t: Tensor | None) -> Tensor | None:
            return t.to_local() if isinstance(t, DTensor) else t

        params = self._param_group[PARAMS]
        return (local(p.grad) for p in params) if get_grad else (local(p) for p in params)

    # -- construction ----------------------------------------------------------------------------
    def _allocate_zeros_distributed_tensor(
        self, size: tuple[int, ...], dtype: torch.dtype, device: torch.device, group_source_rank: int
    ) -> Tensor:
        return allocate_zeros_on_owner(size, dtype, device, self._owner_mesh_rows, group_source_rank)

    @torch.no_grad()
    def _construct_local_block_info_list(
        self, group_source_ranks: tuple[int, ...], group_rank: int
    ) -> tuple[DTensorBlockInfo, ...]:
        infos = []
        for (param_index, p), (lo, hi) in zip(
            enumerate(self._param_group[PARAMS]),
            generate_pairwise_indices(self._global_num_blocks_per_param),
            strict=True,
        ):
            for block_index, owner in enumerate(group_source_ranks[lo:hi]):
                if owner != group_rank:
                    continue
                infos.append(
                    DTensorBlockInfo(
                        param=p,
                        composable_block_ids=self._construct_composable_block_ids(
                            param_index, block_index, self._block_id_rank
                        ),
                        allocate_zeros_tensor=partial(
                            self._allocate_zeros_distributed_tensor, group_source_rank=owner
                        ),
                    )
                )
        return tuple(infos)

    def _construct_distributed_buffers(
        self, buffer_size_ranks: tuple[tuple[int, int], ...], communication_dtype: torch.dtype, group_rank: int
    ) -> None:
        per_rank = [sum(size for size, r in buffer_size_ranks if r == i) for i in range(self._group_size)]
        chunk = max(per_rank) if per_rank else 0
        self._global_dist_buffer = self._allocate_global_buffer(chunk * self._group_size)
        chunks, views, offsets = carve_block_buffers(
            self._global_dist_buffer, buffer_size_ranks, self._global_blocked_params, self._group_size, communication_dtype
        )
        self._local_dist_buffer = chunks[group_rank] if chunks else self._global_dist_buffer
        self._global_dist_blocked_buffers: tuple[Tensor, ...] = views
        self._global_block_byte_offsets: tuple[int, ...] = offsets
        self._local_dist_blocked_buffers = compress_list(views, self._distributor_selector)
        self._global_masked_dist_blocked_buffers = self._global_dist_blocked_buffers
        self._local_masked_dist_blocked_buffers = self._local_dist_blocked_buffers

    def _allocate_global_buffer(self, nbytes: int) -> Tensor:
        """The all-gather buffer.  Overridden by the peer-to-peer variant, which places it in
        memory every rank of the group can address."""
        return torch.zeros(nbytes, dtype=torch.int8, device=self._global_blocked_params[0].device)

    # -- step ------------------------------------------------------------------------------------
    @torch.compiler.disable
    def _all_gather(self) -> None:
        with shampoo_comm_profiler(f"{self.__class__.__name__}::all_gather_into_tensor"):
            dist.all_gather_into_tensor(
                output_tensor=self._global_dist_buffer, input_tensor=self._local_dist_buffer, group=self._dist_group
            )

    @torch.no_grad()
    def update_params(self, blocked_search_directions: tuple[Tensor, ...], use_masked_tensors: bool = True) -> None:
        if use_masked_tensors:
            local_params, local_bufs = self._local_masked_blocked_params, self._local_masked_dist_blocked_buffers
            global_params, global_bufs = self._global_masked_blocked_params, self._global_masked_dist_blocked_buffers
        else:
            local_params, local_bufs = self._local_blocked_params, self._local_dist_blocked_buffers
            global_params, global_bufs = self._global_blocked_params, self._global_dist_blocked_buffers

        if self._communicate_params:
            assert len(local_params) == len(blocked_search_directions), (
                f"Expected len(local_params)={len(local_params)} to be equal to len(blocked_search_directions)={len(blocked_search_directions)}."
            )
            if blocked_search_directions:
                torch._foreach_add_(local_params, blocked_search_directions)
                torch._foreach_copy_(local_bufs, local_params)
            self._all_gather()  # issued even with nothing to send: ranks stay in lock-step
            if global_params:
                torch._foreach_copy_(global_params, global_bufs)
        else:
            assert len(local_bufs) == len(blocked_search_directions), (
                f"Expected len(local_buffers)={len(local_bufs)} to be equal to len(blocked_search_directions)={len(blocked_search_directions)}."
            )
            if blocked_search_directions:
                torch._foreach_copy_(local_bufs, blocked_search_directions)
            self._all_gather()
            if global_params:
                torch._foreach_add_(global_params, global_bufs)

    def _refresh_local_selection(self) -> None:
        if self._previous_global_grad_selector == self._global_grad_selector:
            return
        super()._refresh_local_selection()
        sel = self._global_grad_selector
        self._global_masked_blocked_params = compress_list(self._global_blocked_params, sel)
        self._global_masked_dist_blocked_buffers = compress_list(self._global_dist_blocked_buffers, sel)
        self._local_masked_dist_blocked_buffers = compress_list(
            self._local_dist_blocked_buffers, self._local_grad_selector
        )

    def merge_and_block_gradients(self) -> tuple[Tensor, ...]:
        grads = self._merge_and_block_gradients()
        self._refresh_local_selection()
        return grads
