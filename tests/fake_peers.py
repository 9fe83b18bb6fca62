"""Peer memory among gloo ranks on one host, for CPU tests of the fused compute + collective paths.

The engine's peer-to-peer mode needs three things from the platform: memory that every rank of a
group can address (``torch.distributed._symmetric_memory``), kernels that load from and store to
it, and a barrier between ranks.  Here the memory is POSIX shared memory mapped into every rank,
"device addresses" are the addresses of those mappings in the calling process, the kernels are the
torch stand-ins of ``fake_block_ext`` extended by the peer forms (gradients summed from every rank's
arena, directions stored into every rank's gather buffer), and the barrier is a gloo barrier.  The
real ``SymmetricArena`` (layout, guard regions, peer address tables) and the engine's own barrier
placement run unchanged.
"""

import atexit
import ctypes
from multiprocessing import shared_memory

import torch
import torch.distributed as dist

from fake_block_ext import FakeBlockExt, _at, _DTYPES

_own = {}      # data_ptr of a local arena tensor -> its SharedMemory
_mapped = []   # peers' segments: kept mapped for the life of the process


def _address(shm):
    return ctypes.addressof(ctypes.c_char.from_buffer(shm.buf))


def _cleanup():
    for shm in _own.values():
        try:
            shm.close()
            shm.unlink()
        except Exception:  # noqa: BLE001
            pass


atexit.register(_cleanup)


def symm_empty(nbytes, dtype=torch.uint8, device=None):
    assert dtype == torch.uint8
    shm = shared_memory.SharedMemory(create=True, size=max(int(nbytes), 1))
    tensor = torch.frombuffer(shm.buf, dtype=torch.uint8)[: int(nbytes)]
    _own[tensor.data_ptr()] = shm
    return tensor


class _Handle:
    def __init__(self, buffer_ptrs):
        self.buffer_ptrs = buffer_ptrs


def symm_rendezvous(tensor, group=None):
    mine = _own[tensor.data_ptr()]
    world = dist.get_world_size(group)
    names = [None] * world
    dist.all_gather_object(names, mine.name, group=group)
    pointers = []
    for rank, name in enumerate(names):
        if rank == dist.get_rank(group):
            pointers.append(tensor.data_ptr())
            continue
        peer = shared_memory.SharedMemory(name=name)
        _mapped.append(peer)
        pointers.append(_address(peer))
    return _Handle(pointers)


class FakePeerExt(FakeBlockExt):
    barrier_timeout = 30.0  # seconds a rank waits for the others before it reports the peer timeout

    def peer_barrier(self, local_flags, peer_flag_bases, my_rank, world, seq, status):
        """The kernel's protocol: announce ``seq`` in slot ``my_rank`` of every member's flag array, then
        wait until every slot of the local array has reached ``seq``; a wait that runs out sets the
        peer-timeout bit of the status word instead of blocking for ever."""
        import time

        for base in peer_flag_bases.tolist():
            _at(base + 4 * my_rank, 1, torch.int32)[0] = seq
        deadline = time.monotonic() + self.barrier_timeout
        while bool((local_flags[:world] < seq).any()):
            if time.monotonic() > deadline:
                status[0] |= 4
                return
            time.sleep(0.0005)

    def build_copy_table(self, specs, device_index):
        return (list(specs), None, len(specs))

    def peer_copy(self, specs, _chunks, _n):
        for source, destination, nbytes in specs:
            ctypes.memmove(destination, source, nbytes)

    def grad_prologue(self, blocks, tiles, n, grad_ptrs, l2, beta1, beta3, bc1, graft_kind, g_beta2, g_weight, g_bc2, g_eps,
                      write_split, status, num_grad_peers, grad_scale):
        if num_grad_peers == 0:
            return super().grad_prologue(blocks, tiles, n, grad_ptrs, l2, beta1, beta3, bc1, graft_kind, g_beta2, g_weight,
                                         g_bc2, g_eps, write_split, status, 0, grad_scale)
        # The owner sums the peers' gradients in rank order and scales the sum: build that gradient
        # in a scratch tensor per slot and hand the local form a table pointing at the scratch.
        pointers = grad_ptrs.tolist()
        slots = sorted({b.grad_slot for b in blocks})
        scratch, table = {}, [0] * (max(slots) + 1)
        for slot in slots:
            extent = max((b.grad_offset + (b.m - 1) * b.w().stride(0) + b.n) for b in blocks if b.grad_slot == slot)
            total = torch.zeros(extent)
            for r in range(num_grad_peers):
                total += _at(pointers[slot * num_grad_peers + r], extent)
            scratch[slot] = total * grad_scale
            table[slot] = scratch[slot].data_ptr()
        return super().grad_prologue(blocks, tiles, n, torch.tensor(table, dtype=torch.int64), l2, beta1, beta3, bc1, graft_kind,
                                     g_beta2, g_weight, g_bc2, g_eps, write_split, status, 0, 1.0)

    def direction_epilogue(self, blocks, tiles, n, lr, graft_only, graft_kind, g_bc2, g_eps, wd_alpha, primal, mu_y, mu_x,
                           classic, momentum, dampening, nesterov, send_dtype, split_input, peer_bases, send_params):
        if not peer_bases:
            return super().direction_epilogue(blocks, tiles, n, lr, graft_only, graft_kind, g_bc2, g_eps, wd_alpha, primal, mu_y,
                                              mu_x, classic, momentum, dampening, nesterov, send_dtype, split_input, [], send_params)
        # Compute every block's direction into a private slot, then store it into every rank's buffer.
        private = {}
        for b in blocks:
            if b.aux == 1:
                continue
            private[id(b)] = torch.zeros(b.m * b.n, dtype=_DTYPES[send_dtype])
            b.send = private[id(b)].data_ptr()
        super().direction_epilogue(blocks, tiles, n, lr, graft_only, graft_kind, g_bc2, g_eps, wd_alpha, primal, mu_y, mu_x,
                                   classic, momentum, dampening, nesterov, send_dtype, split_input, [], send_params)
        for b in blocks:
            if b.aux == 1:
                continue
            for base in peer_bases:
                _at(base + b.slot_offset, b.m * b.n, _DTYPES[send_dtype]).copy_(private[id(b)])
            b.send = 0

    def run_gemm_plan_push(self, specs, _tiles, _n, alpha, beta, split, status, peer_bases, send_dtype):
        """The last preconditioner product with the all-gather in its epilogue: the result, cast to
        the communication dtype, goes to the block's slot in every rank's gather buffer (and its
        squared norm to ``sumsq``); nothing is written locally."""
        for spec in specs:
            a_hi, a_lo, b_hi, b_lo, _c, _d_hi, _d_lo, sumsq, _ldc, _ldd, flags, _upper, push_offset = spec[:13]
            assert flags & self.FLAG_PEER_PUSH and flags & self.FLAG_NO_C
            A = a_hi + (a_lo if a_lo is not None else 0)
            B = b_hi + (b_lo if b_lo is not None else 0)
            out = alpha * (A.double() @ B.double().T).float()
            if flags & self.FLAG_SUMSQ:
                sumsq[0] += (out.double() ** 2).sum().float()
            flat = out.reshape(-1).to(_DTYPES[send_dtype])
            for base in peer_bases:
                _at(base + push_offset, flat.numel(), _DTYPES[send_dtype]).copy_(flat)
