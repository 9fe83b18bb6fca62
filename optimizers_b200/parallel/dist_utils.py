"""Small helpers shared by the distributed distributors: profiler ranges around collectives,
a stream context that orders a side stream after the current one, a cached ``DeviceMesh``
factory, the owner-sub-mesh DTensor allocator, and the process groups of the hybrid-shard
distributors.

Reference counterpart: ``distributed_shampoo/distributor/shampoo_dist_utils.py:20-119``.
"""

from __future__ import annotations

from collections.abc import Generator
from contextlib import contextmanager
from functools import cache
from itertools import islice

import torch
from torch import distributed as dist
from torch.autograd import profiler
from torch.distributed import tensor as dtensor
from torch.distributed.device_mesh import DeviceMesh


@contextmanager
def shampoo_comm_profiler(name: str) -> Generator[None, None, None]:
    """Profiler range (and NVTX range on CUDA builds) around one collective."""
    pushed = False
    if torch.cuda.is_available():
        try:
            torch.cuda.nvtx.range_push(name)
            pushed = True
        except Exception:
            pushed = False
    try:
        with profiler.record_function(name):
            yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()


@contextmanager
def cuda_stream_context(stream: torch.cuda.Stream) -> Generator[None, None, None]:
    """Run the body on ``stream`` after everything already queued on the current stream."""
    stream.wait_stream(torch.cuda.current_stream(stream.device))
    with torch.cuda.stream(stream):
        yield


@cache
def get_device_mesh(
    device_type: str,
    mesh: tuple[tuple[int, ...], ...] | tuple[int, ...],
    mesh_dim_names: tuple[str, ...] | None = None,
) -> DeviceMesh:
    """``DeviceMesh`` construction creates process groups, so identical requests share one mesh."""
    return DeviceMesh(device_type=device_type, mesh=mesh, mesh_dim_names=mesh_dim_names)


def batched(iterable, n: int):
    if n < 1:
        raise ValueError(f"n={n} must be at least one")
    it = iter(iterable)
    while chunk := tuple(islice(it, n)):
        yield chunk


def allocate_zeros_on_owner(
    size: tuple[int, ...],
    dtype: torch.dtype,
    device: torch.device,
    mesh_rows: tuple[tuple[int, ...], ...],
    group_source_rank: int,
) -> torch.Tensor:
    """Zeros as a DTensor replicated over the sub-mesh of ranks that own the same blocks.

    ``mesh_rows`` is the (replicate x shard) arrangement of the ranks that share the work of one
    group; column ``group_source_rank`` is the set of ranks holding identical copies of the
    owner's state.  Checkpoint tools use the placement to know which ranks hold which state."""
    mesh_2d = get_device_mesh(device_type=device.type, mesh=mesh_rows, mesh_dim_names=("replicate", "shard"))
    submesh = mesh_2d._get_all_submeshes(mesh_dim_name="replicate")[group_source_rank]  # type: ignore[attr-defined]
    return dtensor.zeros(size, dtype=dtype, device_mesh=submesh, placements=[dtensor.Replicate()])


def create_hybrid_shard_process_groups(device_mesh: DeviceMesh, dist_group_size: int) -> dist.ProcessGroup:
    """Communication group of the hybrid-shard distributors: the replicate dim of ``device_mesh``
    (all ranks holding the same shard) cut into consecutive groups of ``dist_group_size``.

    Process-group creation is collective, so every rank builds the (replicate x shard) mesh of
    every shard position, in the same order, and keeps the group of its own.  The meshes are
    cached under exactly the arguments ``allocate_zeros_on_owner`` uses later, which therefore
    never creates a group on a subset of ranks."""
    assert device_mesh.mesh_dim_names is not None, "DeviceMesh must have mesh_dim_names"
    mine: dist.ProcessGroup | None = None
    for same_shard_ranks in device_mesh.mesh.T:
        sub = get_device_mesh(
            device_type=device_mesh.device_type,
            mesh=tuple(map(tuple, same_shard_ranks.view(-1, dist_group_size).tolist())),
            mesh_dim_names=("replicate", "shard"),
        )
        if dist.get_rank() in same_shard_ranks:
            mine = sub.get_group("shard")
    assert mine is not None
    return mine
