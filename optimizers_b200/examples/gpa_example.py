"""Single-device example for GPA-AdamW: the one-convolution ConvNet on synthetic 32x32 images,
showing the ``train()`` / ``eval()`` protocol (gradients are taken at the y sequence, the model
is evaluated at the averaged x sequence).

    python -m optimizers_b200.examples.gpa_example --steps 50 --eval-interp-coeff 0.9

Reference counterpart: ``gpa/examples/cifar10_example.py:36-133``.
"""

from __future__ import annotations

import argparse

import torch

from optimizers_b200.gpa_adamw import GPAAdamW, IterateAveragingType
from optimizers_b200.models import ConvNet


def main(argv=None) -> tuple[float, float]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--weight-decay", type=float, default=0.0)
    ap.add_argument("--train-interp-coeff", type=float, default=0.7)
    ap.add_argument("--eval-interp-coeff", type=float, default=0.9967)
    ap.add_argument("--schedule-free", action="store_true")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)

    torch.manual_seed(args.seed)
    device = torch.device(args.device)
    model = ConvNet(32, 32).to(device)
    opt = GPAAdamW(
        model.parameters(), lr=args.lr, weight_decay=args.weight_decay,
        iterate_averaging_type=IterateAveragingType.SCHEDULE_FREE if args.schedule_free else IterateAveragingType.GPA,
        train_interp_coeff=args.train_interp_coeff, eval_interp_coeff=args.eval_interp_coeff,
    )
    # A fixed synthetic "dataset" so that the loss can actually go down.
    gen = torch.Generator().manual_seed(args.seed)
    data = torch.randn(512, 3, 32, 32, generator=gen).to(device)
    labels = torch.randint(0, 10, (512,), generator=gen).to(device)

    def evaluate() -> float:
        opt.eval()  # parameters <- averaged iterate x
        with torch.no_grad():
            value = torch.nn.functional.cross_entropy(model(data), labels).item()
        opt.train()  # back to the gradient sequence y
        return value

    opt.train()
    first = evaluate()
    for step in range(args.steps):
        idx = torch.randint(0, 512, (args.batch_size,), generator=gen).to(device)
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(data[idx]), labels[idx])
        loss.backward()
        opt.step()
        if step % 10 == 0:
            print(f"step {step:4d}  train loss {loss.item():.4f}")
    last = evaluate()
    print(f"eval loss at the averaged iterate: {first:.4f} -> {last:.4f}")
    return first, last


if __name__ == "__main__":
    main()
