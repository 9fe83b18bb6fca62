"""Example trainer: any example model x optimizer x parallelism strategy on synthetic data.

    python -m optimizers_b200.examples.train --model convnet --optimizer shampoo --steps 20
    torchrun --nproc-per-node 2 -m optimizers_b200.examples.train --parallelism ddp --backend gloo --device cpu
    torchrun --nproc-per-node 8 -m optimizers_b200.examples.train --model gpt2 --parallelism ddp_fused

Checkpoints are written with ``torch.distributed.checkpoint`` in eval mode (the averaged
parameters) and training continues in train mode afterwards.

Reference counterparts: ``distributed_shampoo/examples/cifar10_example.py:74-134`` and
``distributed_shampoo/examples/utils.py:38-307`` (environment, seeding, optimizer
instantiation, checkpoint save/load, training loop).
"""

from __future__ import annotations

import argparse
import logging
import os
import random

import numpy as np
import torch
import torch.distributed as dist

import optimizers_b200 as ob
from optimizers_b200.examples.loss_metrics import LossMetrics
from optimizers_b200.examples.parallelism import STRATEGIES
from optimizers_b200.examples.resolvers import resolve_fsdp_param_strategy, resolve_torch_dtype, resolve_weight_decay_type

logger = logging.getLogger(__name__)


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", choices=["mlp", "convnet", "resnet18", "gpt2", "llama"], default="convnet")
    ap.add_argument("--optimizer", choices=["shampoo", "soap", "muon", "adam", "adamw", "sgd", "gpa_adamw"], default="shampoo")
    ap.add_argument("--parallelism", choices=list(STRATEGIES), default="none")
    ap.add_argument("--backend", default="nccl")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch-size", type=int, default=128, help="per-rank batch size")
    ap.add_argument("--seq-len", type=int, default=256)
    ap.add_argument("--small", action="store_true", help="shrink the language models for smoke runs")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--weight-decay-type", default="DECOUPLED")
    ap.add_argument("--max-preconditioner-dim", type=int, default=1024)
    ap.add_argument("--precondition-frequency", type=int, default=10)
    ap.add_argument("--grafting", choices=["none", "sgd", "adagrad", "rmsprop", "adam"], default="adam")
    ap.add_argument("--momentum", type=float, default=0.0)
    ap.add_argument("--communication-dtype", default="float32")
    ap.add_argument("--param-assignment-strategy", default="DEFAULT")
    ap.add_argument("--num-sub-groups", type=int, default=1)
    ap.add_argument("--dp-replicate-degree", type=int, default=2)
    ap.add_argument("--native-backend", choices=["auto", "native", "torch"], default="auto")
    ap.add_argument("--seed", type=int, default=2022)
    ap.add_argument("--window-size", type=int, default=10)
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--metrics-dir", default=None)
    ap.add_argument("--config", default=None, metavar="YAML",
                    help="YAML file of option defaults (keys are the option names with underscores, e.g. "
                    "max_preconditioner_dim: 2048); a bare name is looked up under examples/configs/. "
                    "Options given on the command line win.")
    args = ap.parse_args(argv)
    if args.config is not None:
        import os

        import yaml

        path = args.config
        if not os.path.exists(path):
            path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "configs", f"{args.config}.yaml")
        with open(path) as fh:
            preset = yaml.safe_load(fh) or {}
        unknown = set(preset) - set(vars(args))
        if unknown:
            raise SystemExit(f"unknown keys in {path}: {sorted(unknown)}")
        ap.set_defaults(**preset)
        args = ap.parse_args(argv)
    return args


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)


def build_model(args: argparse.Namespace) -> tuple[torch.nn.Module, str]:
    """Returns the model and the kind of batch it consumes (``image`` or ``tokens``)."""
    from optimizers_b200 import models as M

    if args.model == "mlp":
        return M.MLP(), "flat"
    if args.model == "convnet":
        return M.ConvNet(32, 32), "image"
    if args.model == "resnet18":
        return M.ResNet18(), "image"
    if args.model == "gpt2":
        cfg = M.GPT2Config(vocab_size=1024, n_ctx=args.seq_len, n_layer=2, n_head=4, d_model=128, d_mlp=512) if args.small else M.GPT2Config()
        return M.GPT2(cfg), "tokens"
    cfg = M.LlamaConfig(vocab_size=1024, n_layer=2, n_head=4, d_model=128, d_ffn=256) if args.small else M.LlamaConfig()
    return M.Llama(cfg), "tokens"


def synthetic_batch(kind: str, args: argparse.Namespace, model: torch.nn.Module, device: torch.device, gen: torch.Generator):
    b = args.batch_size
    if kind == "tokens":
        vocab = getattr(model, "cfg").vocab_size
        tokens = torch.randint(0, vocab, (b, args.seq_len + 1), generator=gen).to(device)
        return tokens[:, :-1], tokens[:, 1:]
    shape = (b, 784) if kind == "flat" else (b, 3, 32, 32)
    return torch.randn(*shape, generator=gen).to(device), torch.randint(0, 10, (b,), generator=gen).to(device)


def distributed_config_factory(args: argparse.Namespace):
    """A callable the parallelism strategy completes with what only it knows (metadata, mesh)."""
    comm = resolve_torch_dtype(args.communication_dtype)
    strategy = resolve_fsdp_param_strategy(args.param_assignment_strategy)
    return {
        "none": None,
        "ddp": lambda **kw: ob.DDPDistributedConfig(communication_dtype=comm, **kw),
        "ddp_fused": lambda **kw: ob.DDPDistributedConfig(communication_dtype=comm, **kw),
        "fsdp": lambda **kw: ob.FSDPDistributedConfig(**kw),
        "hsdp": lambda **kw: ob.HSDPDistributedConfig(communication_dtype=comm, **kw),
        "fully_shard": lambda **kw: ob.FullyShardDistributedConfig(
            param_assignment_strategy=strategy, num_sub_groups=args.num_sub_groups, **kw
        ),
        "hybrid_shard": lambda **kw: ob.HybridShardDistributedConfig(
            communication_dtype=comm, param_assignment_strategy=strategy, num_sub_groups=args.num_sub_groups, **kw
        ),
    }[args.parallelism]


def build_optimizer(args: argparse.Namespace, model: torch.nn.Module, distributed_config) -> torch.optim.Optimizer:
    params = list(model.parameters())
    if args.optimizer == "sgd":
        return torch.optim.SGD(params, lr=args.lr, momentum=args.momentum, weight_decay=args.weight_decay)
    if args.optimizer == "adam":
        return torch.optim.Adam(params, lr=args.lr, weight_decay=args.weight_decay)
    if args.optimizer == "adamw":
        return torch.optim.AdamW(params, lr=args.lr, weight_decay=args.weight_decay)
    if args.optimizer == "gpa_adamw":
        return ob.GPAAdamW(params, lr=args.lr, weight_decay=args.weight_decay)
    grafting = {
        "none": None,
        "sgd": ob.SGDPreconditionerConfig(),
        "adagrad": ob.AdaGradPreconditionerConfig(),
        "rmsprop": ob.RMSpropPreconditionerConfig(),
        "adam": ob.AdamPreconditionerConfig(),
    }[args.grafting]
    fused = args.parallelism == "ddp_fused"
    common = dict(
        lr=args.lr,
        betas=(0.9, 0.999),
        epsilon=1e-12,
        weight_decay=args.weight_decay,
        weight_decay_type=resolve_weight_decay_type(args.weight_decay_type),
        max_preconditioner_dim=args.max_preconditioner_dim,
        precondition_frequency=args.precondition_frequency,
        grafting_config=grafting,
        iterate_averaging_config=ob.ClassicMomentumConfig(momentum=args.momentum) if args.momentum > 0 else None,
        native_runtime_config=ob.NativeRuntimeConfig(
            backend=args.native_backend, comm_path="p2p" if fused else "nccl", fuse_gradient_reduction=fused
        ),
    )
    if distributed_config is not None:
        common["distributed_config"] = distributed_config
    if args.optimizer == "soap":
        common["preconditioner_config"] = ob.DefaultSOAPConfig
    elif args.optimizer == "muon":
        # Spectral descent for matrices, sign descent for vectors and scalars.
        matrices = [p for p in params if p.dim() >= 2]
        others = [p for p in params if p.dim() < 2]
        groups = [
            {
                "params": matrices,
                "preconditioner_config": ob.DefaultSpectralDescentPreconditionerConfig,
                "grafting_config": None,
                "max_preconditioner_dim": float("inf"),
                "distributed_config": ob.SingleDeviceDistributedConfig(target_parameter_dimensionality=2),
            }
        ]
        if others:
            groups.append({"params": others, "preconditioner_config": ob.DefaultSignDescentPreconditionerConfig, "grafting_config": None})
        return ob.DistributedShampoo(groups, **common)
    return ob.DistributedShampoo(params, **common)


def save_checkpoint(path: str, model: torch.nn.Module, optimizer: torch.optim.Optimizer) -> None:
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_state_dict

    if hasattr(optimizer, "eval"):
        optimizer.eval()
    model_sd, optim_sd = get_state_dict(model, optimizer)
    dcp.save({"model": model_sd, "optim": optim_sd}, checkpoint_id=path)
    if hasattr(optimizer, "train"):
        optimizer.train()


def load_checkpoint(path: str, model: torch.nn.Module, optimizer: torch.optim.Optimizer) -> None:
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint.state_dict import get_state_dict, set_state_dict

    if not os.path.isdir(path):
        return
    if hasattr(optimizer, "eval"):
        optimizer.eval()
    model_sd, optim_sd = get_state_dict(model, optimizer)
    state = {"model": model_sd, "optim": optim_sd}
    dcp.load(state, checkpoint_id=path)
    set_state_dict(model, optimizer, model_state_dict=state["model"], optim_state_dict=state["optim"])
    if hasattr(optimizer, "train"):
        optimizer.train()


def main(argv=None) -> float:
    args = parse_args(argv)
    logging.basicConfig(level=logging.INFO, format=f"[rank {os.environ.get('RANK', 0)}] %(message)s")
    set_seed(args.seed)
    strategy = STRATEGIES[args.parallelism](distributed_config_factory(args))
    world, rank, local_rank = 1, 0, int(os.environ.get("LOCAL_RANK", 0))
    if strategy.requires_distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(backend=args.backend)
        world, rank = dist.get_world_size(), dist.get_rank()
    device = torch.device(args.device, local_rank) if args.device == "cuda" else torch.device("cpu")
    if device.type == "cuda":
        torch.cuda.set_device(device)

    model, kind = build_model(args)
    model = model.to(device)
    mesh = None
    if strategy.requires_device_mesh:
        from torch.distributed.device_mesh import init_device_mesh

        r = args.dp_replicate_degree
        mesh = init_device_mesh(device.type, (r, world // r), mesh_dim_names=("replicate", "shard"))
    wrapped = strategy.wrap_model(model, local_rank, args.backend, mesh)
    model = wrapped.model
    optimizer = build_optimizer(args, model, wrapped.distributed_config)
    if args.checkpoint_dir:
        load_checkpoint(args.checkpoint_dir, model, optimizer)
    if hasattr(optimizer, "train"):
        optimizer.train()

    metrics = LossMetrics(window_size=args.window_size, device=device, world_size=world, metrics_dir=args.metrics_dir)
    gen = torch.Generator().manual_seed(args.seed + rank)
    keep_grads = args.parallelism == "ddp_fused"
    for _ in range(args.steps):
        x, y = synthetic_batch(kind, args, getattr(model, "module", model), device, gen)
        optimizer.zero_grad(set_to_none=not keep_grads)
        loss = model(x, y) if kind == "tokens" else torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        optimizer.step()
        metrics.update(loss)
        metrics.log()
        metrics.update_global_metrics()
        if rank == 0:
            metrics.log_global_metrics()
    metrics.flush()
    if args.checkpoint_dir:
        save_checkpoint(args.checkpoint_dir, model, optimizer)
    final = float(metrics.lifetime_loss)
    if strategy.requires_distributed:
        dist.barrier()
        dist.destroy_process_group()
    return final


if __name__ == "__main__":
    main()
