"""Loss curves of a small GPT-2 trained with Distributed Shampoo by three implementations of the
same step: this framework's native engine, this framework's torch step, and the unmodified
reference (``baseline/_ref``).  The data is a learnable synthetic language (each token is a fixed
function of the two tokens before it, with 10 % noise), so the loss falls from ln(vocab) towards
the noise floor and differences between the implementations show up as diverging curves.

    python benchmarks/convergence_check.py --steps 300

Prints one JSON line per implementation with the loss every ``--every`` steps.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def make_batches(vocab: int, batch: int, seq: int, count: int, device):
    import torch

    g = torch.Generator().manual_seed(7)
    table = torch.randint(0, vocab, (vocab, vocab), generator=g)
    out = []
    for _ in range(count):
        t = torch.empty(batch, seq + 1, dtype=torch.long)
        t[:, :2] = torch.randint(0, vocab, (batch, 2), generator=g)
        for i in range(2, seq + 1):
            nxt = table[t[:, i - 2], t[:, i - 1]]
            noise = torch.randint(0, vocab, (batch,), generator=g)
            t[:, i] = torch.where(torch.rand(batch, generator=g) < 0.1, noise, nxt)
        out.append(t.to(device))
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--every", type=int, default=25)
    ap.add_argument("--impls", default="native,torch,reference")
    ap.add_argument("--precondition-frequency", type=int, default=20)
    ap.add_argument("--epsilon", type=float, default=1e-10)
    ap.add_argument("--gemm-mode", default="tf32x3")
    args = ap.parse_args()

    import torch

    from optimizers_b200.models import GPT2, GPT2Config

    dev = torch.device("cuda", 0)
    torch.backends.cuda.matmul.allow_tf32 = False
    vocab, seq, batch = 512, 64, 32
    data = make_batches(vocab, batch, seq, 16, dev)
    for impl in args.impls.split(","):
        if impl == "reference":
            sys.path.insert(0, os.path.join(REPO, "baseline", "_ref"))
            import distributed_shampoo as lib

            extra = {}
        else:
            import optimizers_b200 as lib

            extra = {"native_runtime_config": lib.NativeRuntimeConfig(backend=impl, gemm_mode=args.gemm_mode)}
        torch.manual_seed(0)
        model = GPT2(GPT2Config(vocab_size=vocab, n_ctx=seq, n_layer=4, n_head=4, d_model=256, d_mlp=1024, fused=False)).to(dev)
        opt = lib.DistributedShampoo(
            model.parameters(), lr=3e-3, betas=(0.9, 0.999), epsilon=args.epsilon, weight_decay=1e-4,
            max_preconditioner_dim=512, precondition_frequency=args.precondition_frequency,
            start_preconditioning_step=args.precondition_frequency,
            grafting_config=lib.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8), **extra,
        )
        losses = []
        for step in range(args.steps):
            t = data[step % len(data)]
            loss = model(t[:, :-1], t[:, 1:])
            loss.backward()
            opt.step()
            opt.zero_grad(set_to_none=True)
            if step % args.every == 0 or step == args.steps - 1:
                losses.append(round(float(loss.item()), 4))
        print(json.dumps({"impl": impl, "epsilon": args.epsilon, "gemm_mode": args.gemm_mode if impl == "native" else None, "ln_vocab": round(math.log(vocab), 4), "every": args.every, "losses": losses}))


if __name__ == "__main__":
    main()
