"""Microbenchmark of the fused model kernels against the stock PyTorch formulation.

  lm_head_xent   x[T, C] @ W[V, C]^T -> mean cross-entropy, forward + backward (dx, dW)
  layer_norm     fp32 [T, C] -> bf16, forward + backward
  rms_norm       same without mean / bias
  colsum         column sums of a [T, C] bf16 matrix (bias gradient)

Timed with CUDA events, L2 flushed between iterations.  Bandwidth figures count the algorithmic
bytes of the fused kernels only (cross-entropy: one read and one write of the bf16 logits).

    python benchmarks/model_ops_microbench.py --tokens 16384 --vocab 50257 --dim 768
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def timed(fn, iters: int, flush: torch.Tensor) -> float:
    times = []
    for i in range(iters + 3):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=16384)
    ap.add_argument("--vocab", type=int, default=50257)
    ap.add_argument("--dim", type=int, default=768)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-torch", action="store_true")
    args = ap.parse_args()

    from optimizers_b200.models import fused_ops
    from optimizers_b200.ops import build

    ext = build.load()
    dev = torch.device("cuda")
    T, V, C = args.tokens, args.vocab, args.dim
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.manual_seed(0)
    x = torch.randn(T, C, device=dev, requires_grad=True)
    W = (torch.randn(V, C, device=dev) * 0.02).requires_grad_()
    tgt = torch.randint(0, V, (T,), device=dev)
    gamma, beta = torch.ones(C, device=dev, requires_grad=True), torch.zeros(C, device=dev, requires_grad=True)
    out = {"tokens": T, "vocab": V, "dim": C}

    def head(fused: bool):
        def run():
            x.grad = W.grad = None
            with torch.autocast("cuda", dtype=torch.bfloat16):
                if fused:
                    loss = fused_ops.lm_head_cross_entropy(x, W, tgt)
                else:
                    loss = F.cross_entropy(F.linear(x, W).float(), tgt)
            loss.backward()
        return run

    out["lm_head_xent_fused_ms"] = timed(head(True), args.iters, flush)
    if not args.skip_torch:
        out["lm_head_xent_torch_ms"] = timed(head(False), args.iters, flush)

    ld = (V + 63) // 64 * 64
    logits = torch.randn(T, ld, device=dev).to(torch.bfloat16)
    ms = timed(lambda: ext.xent_fwd_bwd(logits, V, tgt, -100), args.iters, flush)
    out["xent_kernel_ms"] = ms
    out["xent_kernel_gbs"] = 2 * T * ld * 2 / ms / 1e6

    def norm(fused: bool, rms: bool):
        def run():
            x.grad = gamma.grad = beta.grad = None
            with torch.autocast("cuda", dtype=torch.bfloat16):
                if fused:
                    y = fused_ops.rms_norm(x, gamma) if rms else fused_ops.layer_norm(x, gamma, beta)
                elif rms:
                    y = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * gamma).to(torch.bfloat16)
                else:
                    y = F.layer_norm(x, (C,), gamma, beta).to(torch.bfloat16)
            y.backward(dy)
        return run

    dy = torch.randn(T, C, device=dev).to(torch.bfloat16)
    ms = timed(lambda: ext.colsum(dy), args.iters, flush)
    out["colsum_kernel_ms"] = ms
    out["colsum_kernel_gbs"] = T * C * 2 / ms / 1e6
    if not args.skip_torch:
        out["colsum_torch_ms"] = timed(lambda: dy.sum(0, dtype=torch.float32), args.iters, flush)
    if ext.norm_supported(C):
        for rms in (False, True):
            name = "rms_norm" if rms else "layer_norm"
            out[f"{name}_fused_ms"] = timed(norm(True, rms), args.iters, flush)
            if not args.skip_torch:
                out[f"{name}_torch_ms"] = timed(norm(False, rms), args.iters, flush)
        g32, b32 = gamma.detach(), beta.detach()
        xd = x.detach()
        ms = timed(lambda: ext.norm_fwd(xd, g32, b32, 1e-5, False, True), args.iters, flush)
        out["layer_norm_fwd_kernel_ms"] = ms
        out["layer_norm_fwd_kernel_gbs"] = T * C * (4 + 2) / ms / 1e6
        _, mean, rstd = ext.norm_fwd(xd, g32, b32, 1e-5, False, True)
        ms = timed(lambda: ext.norm_bwd(dy, xd, g32, mean, rstd, False), args.iters, flush)
        out["layer_norm_bwd_kernel_ms"] = ms
        out["layer_norm_bwd_kernel_gbs"] = T * C * (2 + 4 + 4) / ms / 1e6
    print(json.dumps({k: (round(v, 4) if isinstance(v, float) else v) for k, v in out.items()}))


if __name__ == "__main__":
    main()
