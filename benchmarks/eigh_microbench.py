"""Batched symmetric eigensolver: the divide-and-conquer solver of this framework against
torch.linalg.eigh (cuSOLVER syevd, what the reference calls per factor) on a list of factor sizes.

    python benchmarks/eigh_microbench.py --sizes 2048:16,768:32 --spectrum gram
    python benchmarks/eigh_microbench.py --preset gpt2      # the factor sizes of GPT-2 124M at block 2048
    python benchmarks/eigh_microbench.py --factors-from-bench 26 --skip-library --profile --host-profile
                                                             # the factors of bench.py's model after 26 steps

Prints one JSON line per arm: milliseconds (CUDA events, after one warm-up run, inputs larger than
the L2), accuracy against fp64, and the work counters of the divide-and-conquer driver.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def gpt2_sizes() -> list[tuple[int, int]]:
    """(d, count) of the Kronecker factors of GPT-2 124M with max_preconditioner_dim 2048."""
    counts: dict[int, int] = {}

    def add(rows: int, cols: int) -> None:
        for r0 in range(0, rows, 2048):
            for c0 in range(0, cols, 2048):
                for d in (min(2048, rows - r0), min(2048, cols - c0)):
                    counts[d] = counts.get(d, 0) + 1

    add(50257, 768)
    add(1024, 768)
    for _ in range(12):
        add(2304, 768), add(768, 768), add(3072, 768), add(768, 3072)
    return sorted(counts.items(), reverse=True)


def factors_of_the_bench_model(steps: int, dev: torch.device) -> list[torch.Tensor]:
    """Train the model of ``bench.py`` (GPT-2 124M, this framework's optimizer, one GPU) for ``steps``
    steps on synthetic tokens and return its unpacked Kronecker factors larger than 128."""
    import bench
    from optimizers_b200.models import GPT2, GPT2Config

    torch.manual_seed(1234)
    model = GPT2(GPT2Config(n_layer=12)).to(dev)
    opt = bench.build_optimizer("ours", model, 1, argparse.Namespace(backend="native", gemm_mode="tf32x3", comm="p2p", layers=12), None)
    for _ in range(steps):
        tokens = torch.randint(0, bench.VOCAB, (16, 1025), device=dev)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model(tokens[:, :-1], tokens[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
    mats = []
    for rec in opt._per_group_state_lists:
        for kf in rec["shampoo_preconditioner_list"]._local_kronecker_factors_unwrapped:
            for f in kf.factor_matrices:
                A = kf.unpack(f)
                if A.shape[0] > 128:
                    mats.append(A.clone())
    del opt, model
    torch.cuda.empty_cache()
    return mats


def make(d: int, spectrum: str, gen: torch.Generator, dev: torch.device) -> torch.Tensor:
    if spectrum == "gram":  # a few hundred accumulated gradient outer products with decaying column scales
        G = torch.randn(d, 2 * d, device=dev, generator=gen) * torch.rand(2 * d, device=dev, generator=gen) ** 4
        return G @ G.T / d
    if spectrum == "lowrank":  # first refresh: one gradient of a d x d/3 block
        G = torch.randn(d, max(d // 3, 1), device=dev, generator=gen)
        return G @ G.T / d
    q, _ = torch.linalg.qr(torch.randn(d, d, device=dev, generator=gen))
    lam = 1.0 / torch.arange(1, d + 1, device=dev) ** (2.0 if spectrum == "power2" else 1.0)
    return (q * lam) @ q.T


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="2048:8,768:16")
    ap.add_argument("--preset", choices=["", "gpt2"], default="")
    ap.add_argument("--spectrum", choices=["gram", "lowrank", "power1", "power2"], default="gram")
    ap.add_argument("--passes", type=int, default=2)
    ap.add_argument("--polish", choices=["householder", "newton_schulz"], default="householder")
    ap.add_argument("--skip-library", action="store_true")
    ap.add_argument("--profile", action="store_true", help="also print the time per phase of the driver")
    ap.add_argument("--check", action="store_true", help="accuracy against fp64 eigh (slow)")
    ap.add_argument("--factors-from-bench", type=int, default=0, metavar="STEPS",
                    help="use the factors of bench.py's model after STEPS training steps instead of synthetic spectra")
    ap.add_argument("--host-profile", action="store_true", help="also print a cProfile of the host side of one run")
    args = ap.parse_args()
    from optimizers_b200.matrix.eigh_dc import NativeBackend, eigh_divide_and_conquer
    from optimizers_b200.ops import build

    ext = build.load()
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(0)
    sizes = gpt2_sizes() if args.preset == "gpt2" else [tuple(int(x) for x in s.split(":")) for s in args.sizes.split(",")]
    if args.factors_from_bench > 0:
        sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        mats = factors_of_the_bench_model(args.factors_from_bench, dev)
        by_size: dict[int, int] = {}
        for m in mats:
            by_size[m.shape[0]] = by_size.get(m.shape[0], 0) + 1
        sizes = sorted(by_size.items(), reverse=True)
        args.spectrum = f"bench.py model after {args.factors_from_bench} steps"
    else:
        mats = [make(d, args.spectrum, gen, dev) for d, count in sizes for _ in range(count)]
    big = [m for m in mats if m.shape[0] > 128]
    total_bytes = sum(m.numel() * 4 for m in big)

    def timed(fn):
        fn()  # warm-up
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop), out

    backend = NativeBackend(ext, dev, range_passes=args.passes, polish=args.polish)
    ms, (lams, vecs, info) = timed(lambda: eigh_divide_and_conquer(backend, big))
    line = {
        "arm": "divide_and_conquer", "ms": ms, "matrices": len(big), "sizes": sizes, "input_bytes": total_bytes,
        "spectrum": args.spectrum, "rounds": info["rounds"], "sign_computations": info["sign_computations"], "sign_stages": info["sign_stages"],
        "work_over_sum_d3": info["sign_cubes"] / sum(float(m.shape[0]) ** 3 for m in big),
        "failed": info["failed"] + backend.failed_in_finish, "status": int(backend.status.item()),
    }
    if args.check:
        worst = {"eig": 0.0, "orth": 0.0, "recon": 0.0}
        for m, lam, Q in list(zip(big, lams, vecs))[:: max(1, len(big) // 6)]:
            if lam is None:
                continue
            A = m.double()
            ref = torch.linalg.eigvalsh(A)
            Qd, ld = Q.double(), lam.double()
            worst["eig"] = max(worst["eig"], float((ld - ref).abs().max() / ref.abs().max()))
            worst["orth"] = max(worst["orth"], float(torch.linalg.norm(Qd.T @ Qd - torch.eye(A.shape[0], device=dev, dtype=torch.float64))))
            worst["recon"] = max(worst["recon"], float(torch.linalg.norm((Qd * ld) @ Qd.T - A) / torch.linalg.norm(A)))
        line["worst_vs_fp64"] = worst
    print(json.dumps(line), flush=True)
    if args.profile:
        backend.profile = {}
        _, (_, _, info) = timed(lambda: (backend.profile.clear(), eigh_divide_and_conquer(backend, big))[1])
        calls = backend.profile.pop("calls", [])
        print(json.dumps({"arm": "divide_and_conquer phases (ms, serialised)", **{k: round(v, 2) for k, v in backend.profile.items()}}), flush=True)
        print(json.dumps({"arm": "divide_and_conquer calls (phase, subproblems, mean size, ms)", "calls": calls}), flush=True)
    if args.host_profile:
        import cProfile
        import io
        import pstats

        backend.profile = None
        profiler = cProfile.Profile()
        profiler.enable()
        eigh_divide_and_conquer(backend, big)
        torch.cuda.synchronize()
        profiler.disable()
        text = io.StringIO()
        pstats.Stats(profiler, stream=text).sort_stats("tottime").print_stats(16)
        print(text.getvalue(), flush=True)
    if not args.skip_library:
        ms_lib, _ = timed(lambda: [torch.linalg.eigh(m) for m in big])
        print(json.dumps({"arm": "torch.linalg.eigh loop", "ms": ms_lib, "matrices": len(big)}), flush=True)


if __name__ == "__main__":
    main()
