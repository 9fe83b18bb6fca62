"""Spawn helper for multi-process CPU (gloo) tests."""

import io
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, store_path, fn, args, queue):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        # File-store rendezvous: no TCP port to collide on.
        dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=world)
        result = fn(rank, world, *args)
        blob = io.BytesIO()
        torch.save(result, blob)  # plain bytes: no shared-memory handles outlive the child
        queue.put((rank, "ok", blob.getvalue()))
    except Exception:
        queue.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn, world: int, *args):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the per-rank results."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    handle, store_path = tempfile.mkstemp(prefix="ob200_store_")
    os.close(handle)
    os.unlink(store_path)
    procs = [ctx.Process(target=_entry, args=(r, world, store_path, fn, args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, status, payload = queue.get(timeout=300)
        if status == "error":
            for p in procs:
                p.terminate()
            raise AssertionError(f"rank {rank} failed:\n{payload}")
        results[rank] = torch.load(io.BytesIO(payload), weights_only=False)
    for p in procs:
        p.join(timeout=60)
    if os.path.exists(store_path):
        os.unlink(store_path)
    return [results[r] for r in range(world)]
