"""Smoke tests of the example entry points on CPU."""

import pytest
import torch

from optimizers_b200.examples import gpa_example, train
from optimizers_b200.examples.loss_metrics import LossMetrics
from optimizers_b200.examples.parallelism import STRATEGIES, SingleGPUStrategy
from optimizers_b200.examples.resolvers import resolve_fsdp_param_strategy, resolve_torch_dtype, resolve_weight_decay_type


@pytest.mark.parametrize(
    "argv",
    [
        ["--model", "convnet", "--optimizer", "shampoo"],
        ["--model", "mlp", "--optimizer", "muon"],
        ["--model", "gpt2", "--small", "--optimizer", "soap", "--seq-len", "16"],
        ["--model", "llama", "--small", "--optimizer", "gpa_adamw", "--seq-len", "16"],
        ["--model", "convnet", "--optimizer", "adamw"],
    ],
)
def test_train_cli_runs(argv):
    loss = train.main(argv + ["--steps", "2", "--batch-size", "4", "--device", "cpu"])
    assert loss == loss and loss > 0


def test_gpa_example_improves_eval_loss():
    first, last = gpa_example.main(["--steps", "40", "--device", "cpu", "--eval-interp-coeff", "0.9"])
    assert last < first


def test_loss_metrics_window_and_lifetime():
    m = LossMetrics(window_size=2)
    for v in (1.0, 2.0, 6.0):
        m.update(torch.tensor(v))
    assert float(m.window_loss) == pytest.approx(4.0) and float(m.lifetime_loss) == pytest.approx(3.0)
    m.log(); m.update_global_metrics(); m.log_global_metrics(); m.flush()
    # a long stream against the plain definitions, across several turns of the ring
    gen = torch.Generator().manual_seed(0)
    values = (torch.rand(57, generator=gen) * 10).tolist()
    for window in (1, 5, 100):
        m = LossMetrics(window_size=window)
        for i, v in enumerate(values, 1):
            m.update(torch.tensor(v))
            tail = values[max(0, i - window) : i]
            assert float(m.window_loss) == pytest.approx(sum(tail) / len(tail), rel=1e-5)
            assert float(m.lifetime_loss) == pytest.approx(sum(values[:i]) / i, rel=1e-5)


def test_resolvers_and_strategies():
    assert resolve_torch_dtype("bfloat16") is torch.bfloat16 and resolve_torch_dtype("torch.float32") is torch.float32
    assert resolve_fsdp_param_strategy("round_robin").name == "ROUND_ROBIN"
    assert resolve_weight_decay_type("l2").name == "L2"
    for bad in (resolve_torch_dtype, resolve_fsdp_param_strategy, resolve_weight_decay_type):
        with pytest.raises(ValueError):
            bad("nope")
    assert set(STRATEGIES) == {"none", "ddp", "ddp_fused", "fsdp", "hsdp", "fully_shard", "hybrid_shard"}
    model = torch.nn.Linear(2, 2)
    wrapped = SingleGPUStrategy().wrap_model(model, 0, "gloo")
    assert wrapped.model is model and wrapped.distributed_config is None
    assert STRATEGIES["hsdp"]().requires_device_mesh and STRATEGIES["ddp"]().requires_distributed


def test_yaml_presets_parse_and_command_line_wins(tmp_path):
    import glob
    import os

    folder = os.path.join(os.path.dirname(train.__file__), "configs")
    presets = sorted(glob.glob(os.path.join(folder, "*.yaml")))
    assert len(presets) >= 4
    for path in presets:
        args = train.parse_args(["--config", path])
        assert args.steps > 0
    args = train.parse_args(["--config", "resnet18_ddp", "--steps", "3"])
    assert (args.model, args.parallelism, args.steps, args.max_preconditioner_dim) == ("resnet18", "ddp", 3, 1024)
    bad = tmp_path / "bad.yaml"
    bad.write_text("no_such_option: 1\n")
    with pytest.raises(SystemExit):
        train.parse_args(["--config", str(bad)])


def test_exchange_comm_path_is_scoped():
    from optimizers_b200.parallel import a2a

    assert a2a._default_comm_path == "nccl"
    with a2a.exchange_comm_path("p2p"):
        assert a2a._default_comm_path == "p2p"
    assert a2a._default_comm_path == "nccl"


def test_fused_ops_fall_back_to_the_same_formulas_on_cpu():
    from optimizers_b200.models import fused_ops

    torch.manual_seed(0)
    x = torch.randn(5, 12, requires_grad=True)
    w = torch.randn(7, 12, requires_grad=True)
    b = torch.randn(7)
    t = torch.randint(0, 7, (5,))
    assert torch.equal(fused_ops.linear(x, w, b), torch.nn.functional.linear(x, w, b))
    want = torch.nn.functional.cross_entropy(torch.nn.functional.linear(x, w), t)
    assert torch.allclose(fused_ops.lm_head_cross_entropy(x, w, t), want)
    g = torch.ones(12)
    assert torch.allclose(fused_ops.layer_norm(x, g, torch.zeros(12)), torch.nn.functional.layer_norm(x, (12,), g, torch.zeros(12)))
    rms = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(fused_ops.rms_norm(x, g), rms, atol=1e-6)
