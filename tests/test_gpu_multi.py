"""Multi-GPU tests of the native DDP engine: NCCL all-gather path and the peer-to-peer paths
(reduce-scatter fused into the prologue, all-gather fused into the epilogue of the last
preconditioner GEMM or into the pointwise epilogue) against the torch step."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(mode: str, nproc: int, out: str, port: int, timeout: int = 300) -> None:
    """Launch the worker on ``nproc`` GPUs.  The launcher gets its own process group so that a run
    that exceeds the limit is ended together with its ranks (none survives to hold a GPU)."""
    import signal

    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
        "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_multi_gpu_worker.py"), mode, out,
    ]
    proc = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, start_new_session=True)
    try:
        stdout, stderr = proc.communicate(timeout=timeout)
    except subprocess.TimeoutExpired:
        os.killpg(proc.pid, signal.SIGKILL)
        stdout, stderr = proc.communicate()
        raise AssertionError(f"worker {mode!r} exceeded {timeout} s\n" + stdout[-2000:] + stderr[-2000:]) from None
    assert proc.returncode == 0, stdout[-3000:] + stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["native_nccl", "p2p_push", "p2p_pull", "p2p_gemm"])
def test_native_ddp_matches_torch_ddp(tmp_path, mode):
    n = min(torch.cuda.device_count(), 4)
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run("torch", n, ref, 29541)
    _run(mode, n, got, 29542)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["native_nccl+tiny", "p2p_push+tiny", "p2p_pull+tiny", "native_nccl+dead", "p2p_push+dead"])
def test_native_ddp_with_idle_ranks_and_unused_parameters(tmp_path, mode):
    """A model of one block leaves every rank but its owner without work (they still take part in the
    barriers and receive the direction); a registered layer that never gets a gradient is skipped,
    as in the reference (distributor/gpu_tests/shampoo_ddp_distributor_test.py:318-362)."""
    n = min(torch.cuda.device_count(), 4)
    suffix = mode[mode.index("+"):]
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run("torch" + suffix, n, ref, 29561)
    _run(mode, n, got, 29562)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["native_nccl", "p2p_push"])
def test_native_ddp_communicate_params_matches_torch(tmp_path, mode):
    """communicate_params=True: owners apply their blocks' updates and the updated parameters
    are gathered (NCCL, or stored into the peers' buffers by the epilogue)."""
    n = min(torch.cuda.device_count(), 4)
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run("torch+params", n, ref, 29547)
    _run(f"{mode}+params", n, got, 29548)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode", ["native_nccl", "p2p_push", "p2p_pull", "p2p_gemm"])
def test_native_ddp_bf16_communication_matches_torch(tmp_path, mode):
    """The communication dtype of the benchmarks: directions are cast to bf16 by the kernel that
    stores them into the gather buffers, as the torch step casts them before its all-gather."""
    n = min(torch.cuda.device_count(), 4)
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run("torch+bf16", n, ref, 29551)
    _run(f"{mode}+bf16", n, got, 29552)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("strategy", ["fully_shard_rr", "fully_shard_rep"])
def test_lossless_primal_averaging_eval_parameters_match_torch(tmp_path, strategy):
    """Lossless distributors block gathered full copies; optimizer.eval() under the native engine
    has to reach the model's own shards (the grouped switch kernel plus the distributor's
    write-back), so the eval-mode parameters equal those of the torch step."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run(f"torch:{strategy}:gpa", n, ref, 29553)
    _run(f"native:{strategy}:gpa", n, got, 29554)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


SHARDED = ["fsdp", "hsdp", "fully_shard", "fully_shard_rr", "fully_shard_rep", "hybrid_shard", "hybrid_shard_rr"]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("strategy", SHARDED)
def test_native_sharded_matches_torch(tmp_path, strategy):
    """Every sharded distributor runs the native step on the tensors it blocks (flat shards,
    dim-0 shards, gathered full copies) and lands where the torch step lands."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run(f"torch:{strategy}", n, ref, 29543)
    _run(f"native:{strategy}", n, got, 29544)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("strategy", ["fully_shard_rr", "hybrid_shard_rr"])
def test_lossless_peer_memory_exchange_matches_all_to_all(tmp_path, strategy):
    """ROUND_ROBIN lossless distributors with the exchange done by one kernel that stores into
    the receivers' memory over NVLink (comm_path="p2p") against the all_to_all collective."""
    n = 4 if torch.cuda.device_count() >= 4 else 2
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run(f"native:{strategy}", n, ref, 29545)
    _run(f"native:{strategy}:p2p", n, got, 29546)
    # The exchange moves bits; the engine's norm reductions use atomics, so two runs agree to an ulp.
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (a - b).abs().max()


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs (replicate groups of two)")
@pytest.mark.parametrize("strategy", ["hsdp", "hybrid_shard"])
def test_replicate_group_peer_push_matches_nccl_all_gather(tmp_path, strategy):
    """HSDP / hybrid shard: the owners of a replicate group store their search directions straight
    into the other members' gather buffers (comm_path="p2p") instead of the NCCL all-gather."""
    ref, got = str(tmp_path / "ref.pt"), str(tmp_path / "got.pt")
    _run(f"torch:{strategy}", 4, ref, 29555)
    _run(f"native:{strategy}:p2p", 4, got, 29556)
    for a, b in zip(torch.load(ref), torch.load(got)):
        assert torch.allclose(a, b, rtol=5e-3, atol=5e-4), (a - b).abs().max()
