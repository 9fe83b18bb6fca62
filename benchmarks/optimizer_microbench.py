"""Optimizer-only microbenchmark: 64 (or --blocks) square blocks of size d x d, fp32.

Timed separately with CUDA events (L2 flushed between iterations by writing a 256 MB buffer):

  factor   the factor update  L <- b2 L + w G G^T, R <- b2 R + w G^T G  (grouped tcgen05 SYRK
           with the EMA and the packed-triangle store fused in the epilogue)
  apply    the preconditioner application  P = L^(-1/4) G R^(-1/4)  (two grouped GEMMs)
  both are also run through the torch/cuBLAS formulation the reference uses
  (tensordot + pack + foreach EMA; unpack + two tensordot), for comparison on the same GPU.

Achieved TFLOP/s counts the algorithmic flops (triangle only for the factor update:
2 * d^2(d+1)/2 * d per factor; 4 d^3 for the application) and, for --mode tf32x3, is the
fp32-equivalent rate (three tensor-core products are issued per algorithmic product).

    python benchmarks/optimizer_microbench.py --d 2048 --blocks 16 --mode tf32x3
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def timed(fn, iters: int, flush: torch.Tensor) -> float:
    """Median milliseconds per call."""
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
    ap.add_argument("--d", type=int, default=2048)
    ap.add_argument("--blocks", type=int, default=64)
    ap.add_argument("--mode", choices=["tf32x3", "tf32"], default="tf32x3")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--skip-torch", action="store_true")
    args = ap.parse_args()

    from optimizers_b200.ops import build
    from optimizers_b200.utils.blocking import pack_upper_triangular, unpack_upper_triangular

    ext = build.load()
    dev = torch.device("cuda")
    d, nb, split = args.d, args.blocks, args.mode == "tf32x3"
    torch.manual_seed(0)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    ld = _pad4(d)

    G = [torch.randn(d, d, device=dev) * 1e-2 for _ in range(nb)]
    packed = d * (d + 1) // 2
    L = [torch.zeros(packed, device=dev) for _ in range(nb)]
    R = [torch.zeros(packed, device=dev) for _ in range(nb)]
    inv = []
    for _ in range(2):
        A = torch.randn(d, d, device=dev)
        inv.append(A @ A.T / d + 1e-6 * torch.eye(d, device=dev))

    def split_of(x):
        hi = torch.zeros(x.shape[0], ld, device=dev)
        lo = torch.zeros_like(hi) if split else None
        if split:
            ext.tf32_split(x, hi[:, :d], lo[:, :d])
        else:
            hi[:, :d].copy_(x)
        return hi[:, :d], (lo[:, :d] if split else None)

    g = [split_of(x) for x in G]
    gt = [split_of(x.T.contiguous()) for x in G]
    li, ri = split_of(inv[0]), split_of(inv[1])
    tt = [(torch.zeros(d, ld, device=dev), torch.zeros(d, ld, device=dev) if split else None) for _ in range(nb)]
    P = [torch.zeros(d, d, device=dev) for _ in range(nb)]

    syrk = []
    for i in range(nb):
        syrk.append((g[i][0], g[i][1], g[i][0], g[i][1], L[i], None, None, None, d, 0, ext.FLAG_PACKED_C, True))
        syrk.append((gt[i][0], gt[i][1], gt[i][0], gt[i][1], R[i], None, None, None, d, 0, ext.FLAG_PACKED_C, True))
    syrk_plan = ext.build_gemm_plan(syrk)
    g1, g2 = [], []
    for i in range(nb):
        if split:
            g1.append((ri[0], ri[1], g[i][0], g[i][1], None, tt[i][0], tt[i][1], None, 0, ld, ext.FLAG_NO_C | ext.FLAG_SPLIT_OUT, False))
        else:
            g1.append((ri[0], None, g[i][0], None, tt[i][0], None, None, None, ld, 0, 0, False))
        g2.append((li[0], li[1], tt[i][0][:, :d], tt[i][1][:, :d] if split else None, P[i], None, None, None, d, 0, 0, False))
    p1, p2 = ext.build_gemm_plan(g1), ext.build_gemm_plan(g2)

    def run_factor():
        ext.run_gemm_plan(*syrk_plan, 0.001, 0.999, split, status)

    def run_apply():
        ext.run_gemm_plan(*p1, 1.0, 0.0, split, status)
        ext.run_gemm_plan(*p2, 1.0, 0.0, split, status)

    def torch_factor():
        for i in range(nb):
            outer = (pack_upper_triangular(torch.tensordot(G[i], G[i], dims=[[1], [1]])),
                     pack_upper_triangular(torch.tensordot(G[i], G[i], dims=[[0], [0]])))
            torch._foreach_mul_([L[i], R[i]], 0.999)
            torch._foreach_add_([L[i], R[i]], outer, alpha=0.001)

    Lp, Rp = pack_upper_triangular(inv[0]), pack_upper_triangular(inv[1])

    def torch_apply():
        for i in range(nb):
            l, r = unpack_upper_triangular(Lp, d), unpack_upper_triangular(Rp, d)
            t = torch.tensordot(G[i], l, dims=([0], [0]))
            P[i] = torch.tensordot(t, r, dims=([0], [0]))

    peaks = {}
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except OSError:
        pass
    out = {"d": d, "blocks": nb, "mode": args.mode}
    factor_flops = 2 * nb * (2.0 * d * packed)
    apply_flops = nb * 4.0 * d**3
    for name, fn, flops in (("factor", run_factor, factor_flops), ("apply", run_apply, apply_flops)):
        ms = timed(fn, args.iters, flush)
        out[f"{name}_ms"] = ms
        out[f"{name}_tflops_fp32_equiv"] = flops / ms / 1e9
        mma = flops * (3 if split else 1) / ms / 1e9
        out[f"{name}_tensor_tflops_issued"] = mma
    torch.cuda.synchronize()
    assert status.item() == 0, "kernel reported an error status"
    if not args.skip_torch:
        torch.backends.cuda.matmul.allow_tf32 = False
        out["torch_factor_ms"] = timed(torch_factor, max(args.iters // 2, 2), flush)
        out["torch_apply_ms"] = timed(torch_apply, max(args.iters // 2, 2), flush)
    if peaks:
        out["measured_bf16_tflops_burst"] = peaks.get("bf16_tflops")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
