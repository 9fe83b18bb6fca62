"""Failure detection without faulting a device.

Host side: a rank that leaves between steps is noticed by its peer as an error of the next
collective (gloo ranks on CPU).  Device side: a bounded wait on a peer flag that nothing sets
expires, reports through the status word and leaves the context usable (single GPU, the absent
peer emulated by a flag array that is never written)."""

import pytest
import torch

from dist_utils_for_tests import run_distributed


def _leaving_rank(rank: int, world: int):
    import torch.distributed as dist

    from optimizers_b200 import AdaGradPreconditionerConfig, DDPDistributedConfig, DistributedShampoo

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(12, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    opt = DistributedShampoo(
        model.parameters(), lr=1e-2, max_preconditioner_dim=8, precondition_frequency=2, start_preconditioning_step=2,
        grafting_config=AdaGradPreconditionerConfig(epsilon=1e-8),
        distributed_config=DDPDistributedConfig(num_trainers_per_group=world),
    )
    g = torch.Generator().manual_seed(1)
    for step in range(4):
        if rank == 1 and step == 2:
            # Leaves between steps: no collective of its own is in flight.
            dist.destroy_process_group()
            return "left"
        x = torch.randn(8, 12, generator=g)
        opt.zero_grad()
        model(x).square().mean().backward()
        try:
            opt.step()
        except Exception as e:  # the all-gather with the departed rank fails instead of hanging
            return f"detected:{type(e).__name__}"
    return "finished"


def test_departed_rank_is_detected_at_the_next_collective():
    results = run_distributed(_leaving_rank, 2)
    assert results[1] == "left"
    assert results[0].startswith("detected:"), results


@pytest.mark.gpu
def test_peer_wait_expires_with_status_and_context_survives():
    from optimizers_b200.ops import build

    ext = build.load()
    dev = torch.device("cuda")
    mine = torch.zeros(32, dtype=torch.int32, device=dev)    # slot 1 would be written by the peer
    absent = torch.zeros(32, dtype=torch.int32, device=dev)  # stands in for the peer's flag array
    bases = torch.tensor([mine.data_ptr(), absent.data_ptr()], dtype=torch.int64, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ext.peer_barrier(mine, bases, 0, 2, 1, status)
    torch.cuda.synchronize()
    assert int(status.item()) & 4, "the expired wait must set the peer-timeout bit"
    assert int(absent[0].item()) == 1  # this rank's own announcement did go out
    # the context is intact: ordinary work still runs
    assert torch.ones(1024, device=dev).sum().item() == 1024


@pytest.mark.gpu
def test_engine_turns_status_bits_into_exceptions():
    from optimizers_b200 import DistributedShampoo, NativeRuntimeConfig

    model = torch.nn.Linear(32, 16).cuda()
    opt = DistributedShampoo(model.parameters(), lr=1e-3, max_preconditioner_dim=32,
                             native_runtime_config=NativeRuntimeConfig(backend="native"))
    eng = opt._per_group_state_lists[0]["native_engine"]
    for bit, text in ((1, "pipeline"), (4, "peer rank")):
        eng._status.fill_(bit)
        with pytest.raises(RuntimeError, match=text):
            eng.check_status()
    eng._status.zero_()
    eng.check_status()
