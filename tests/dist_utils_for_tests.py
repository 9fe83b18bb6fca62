"""Spawn helper for multi-process CPU (gloo) tests."""

import io
import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _entry(rank, world, store_path, fn, args, queue):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), GLOO_SOCKET_IFNAME="lo")
    torch.set_num_threads(1)
    if os.environ.get("OB200_TEST_STALL_DUMP"):
        # Debug aid: OB200_TEST_STALL_DUMP=/some/prefix makes every rank write its Python stack to
        # <prefix>.<rank> if it is still running after 60 s (shows which collective a rank sits in).
        import faulthandler

        faulthandler.dump_traceback_later(60, file=open(f"{os.environ['OB200_TEST_STALL_DUMP']}.{rank}", "w"))
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


class _TransientRendezvousError(RuntimeError):
    pass


def _run_once(fn, world: int, args):
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    handle, store_path = tempfile.mkstemp(prefix="ob200_store_")
    os.close(handle)
    os.unlink(store_path)
    procs = [ctx.Process(target=_entry, args=(r, world, store_path, fn, args, queue)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        waited = 0
        while len(results) < world:
            try:
                rank, status, payload = queue.get(timeout=5)
            except Exception:
                waited += 5
                if waited >= 120 or all(not p.is_alive() for p in procs):
                    raise _TransientRendezvousError("a rank exited or stalled without reporting")
                continue
            if status == "error":
                if "connectFullMesh" in payload or "Connection refused" in payload or "timed out connecting" in payload:
                    raise _TransientRendezvousError(payload)
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            results[rank] = torch.load(io.BytesIO(payload), weights_only=False)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        if os.path.exists(store_path):
            os.unlink(store_path)
    return [results[r] for r in range(world)]


def run_distributed(fn, world: int, *args):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the per-rank results.
    Loopback rendezvous of several gloo ranks occasionally fails to connect under load; such a
    set-up failure (never a failure inside ``fn``) is retried."""
    last = None
    for _ in range(5):
        try:
            return _run_once(fn, world, args)
        except _TransientRendezvousError as e:
            last = e
    raise AssertionError(f"gloo rendezvous failed five times: {last}")
