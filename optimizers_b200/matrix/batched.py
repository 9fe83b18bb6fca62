"""Batched refresh of inverse roots for the native engine.

The torch refresh walks blocks and factors one at a time and synchronises with the host twice
per factor.  Here all factors of a refresh are processed together:

1. one pass prepares the bias-corrected (optionally trace-scaled) factor matrices and a single
   device->host read checks all of them for NaN/Inf;
2. the symmetric eigendecompositions run batched on this framework's own kernels: factors up to
   128 x 128 in one launch of the shared-memory Jacobi kernel, larger ones by the spectral
   divide-and-conquer solver of ``eigh_dc`` (tensor-core products, Householder panels, Jacobi
   leaves); a matrix either gives up on goes to ``torch.linalg.eigh`` on a pool of CUDA streams,
   one Python thread per stream, which is also where the double-precision retry lives; the
   eigenvalue stabilisation and the scaling ``Q·diag(λ^(-1/p))`` need no host synchronisation;
3. the reconstruction ``X = (Q·λ^(-1/p)) Qᵀ`` of every factor is one grouped tcgen05 launch;
4. the packed checkpoint state is refreshed from the result, a second single read checks it, and
   the caller rebuilds the (hi, lo) operand mirrors from the state.

Semantics follow the reference's eigen path (``distributed_shampoo/preconditioner/
matrix_functions.py:179-279, 306-366, 725-770`` and the failure handling of
``shampoo_preconditioner_list.py:314-443``): ε-perturbation before or after the decomposition,
double-precision retry, a failed factor keeps its previous inverse root and counts towards the
block's tolerated consecutive failures.
"""

from __future__ import annotations

import logging
import threading
from concurrent.futures import ThreadPoolExecutor
from types import SimpleNamespace
from fractions import Fraction
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import EigenConfig, EighEigendecompositionConfig, PerturbationConfig, PreconditionerValueError
from optimizers_b200.matrix import functions as mf

logger: logging.Logger = logging.getLogger(__name__)

import os as _os

# Streams / host threads of the refresh pool (OB200_REFRESH_POOL overrides; the library eigensolver
# gains little beyond a handful of concurrent problems).
_POOL_SIZE = max(1, int(_os.environ.get("OB200_REFRESH_POOL", "8")))
_JACOBI_MAX_SWEEPS = 24
_JACOBI_TOLERANCE = 2e-6  # relative size of a column pair's inner product below which it is left alone

_pools: dict[int, tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]] = {}
_tls = threading.local()


def _pool(device: torch.device) -> tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _pools:
        # torch initialises its linear-algebra back-end lazily and not thread-safely: the first
        # eigh / qr must happen on one thread before the pool's threads call them concurrently.
        warm = torch.eye(2, device=device)
        torch.linalg.eigh(warm)
        torch.linalg.qr(warm)
        streams = [torch.cuda.Stream(device=device) for _ in range(_POOL_SIZE)]
        _pools[key] = (ThreadPoolExecutor(max_workers=_POOL_SIZE, thread_name_prefix="ob200-eigh"), streams)
    return _pools[key]


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


def _prepared_factors(ext: Any, blocks: list[Any], bias_correction2: Tensor | float) -> list[tuple[Any, int, Tensor]]:
    """``(block, k, A)`` for every factor of ``blocks`` with ``A`` the full, bias-corrected (and,
    if configured, trace-scaled) factor matrix.  fp32 state is unpacked by one grouped launch and
    divided by one multi-tensor launch; other dtypes take the per-factor tensor path."""
    out: list[tuple[Any, int, Tensor]] = []
    specs, native = [], []
    for b in blocks:
        kf = b.factors
        for k, factor in enumerate(kf.factor_matrices):
            if ext is not None and factor.is_cuda and factor.dtype == torch.float32 and (factor.dim() == 1 or factor.stride(-1) == 1):
                d = kf._packed_dim(factor) if factor.dim() == 1 else factor.shape[0]
                A = torch.empty(d, d, dtype=torch.float32, device=factor.device)
                specs.append((factor, d, A, None))
                native.append(A)
            else:
                A = kf.unpack(factor / bias_correction2)
            out.append((b, k, A))
    if specs:
        ext.unpack_split(*ext.build_unpack_table(specs))
        torch._foreach_div_(native, float(bias_correction2))
    for n, (b, k, A) in enumerate(out):
        kf = b.factors
        if kf.use_trace_scaling:
            out[n] = (b, k, A * torch.pow(torch.clamp(torch.trace(A), min=kf.epsilon), -kf.trace_scaling_exponent))
    return out


class _PhaseClock:
    """OB200_REFRESH_TIMING=1: log the wall time of the phases of a refresh, each bracketed by a
    device synchronisation (diagnostics; the synchronisations cost a little themselves)."""

    enabled = _os.environ.get("OB200_REFRESH_TIMING", "0") == "1"

    def __init__(self, what: str) -> None:
        self.what, self.marks = what, []
        self.tick("start")

    def tick(self, name: str) -> None:
        if not self.enabled:
            return
        import time

        torch.cuda.synchronize()
        self.marks.append((name, time.perf_counter()))

    def report(self) -> None:
        if self.enabled:
            parts = [f"{b[0]} {1e3 * (b[1] - a[1]):.1f}" for a, b in zip(self.marks, self.marks[1:])]
            logger.warning("%s phases (ms): %s", self.what, ", ".join(parts))


def _all_finite(tensors: list[Tensor]) -> list[bool]:
    """Per-tensor finiteness with one multi-tensor launch and one host read: a norm is finite
    exactly when every element is (the max norm cannot overflow)."""
    if not tensors:
        return []
    return torch.isfinite(torch.stack(torch._foreach_norm(tensors, float("inf")))).cpu().tolist()


# Upper bound on the sum of d^2 over the factors advanced together by the divide-and-conquer
# eigensolver (OB200_EIGH_CHUNK_ELEMS overrides).  Its workspace is about 25 fp32 arrays of that
# size; the bound actually used is further limited to a third of the memory free at the refresh.
# The more factors advance together, the fuller the grouped launches of the deep levels are.
_DC_CHUNK_ELEMS = int(_os.environ.get("OB200_EIGH_CHUNK_ELEMS", str(512 * 1024 * 1024)))
_DC_WORKSPACE_ARRAYS = 25
# OB200_EIGH=library sends every factor larger than the Jacobi kernel's limit to the library eigensolver.
_DC_ENABLED = _os.environ.get("OB200_EIGH", "native") != "library"
# Host threads (each with its own stream) that drive the eigensolver on disjoint halves of the factors
# (OB200_EIGH_LANES=2).  Off by default: measured on the factors of GPT-2 124M the refresh is bound by
# the device once the scratch matrices are allocated per batch (1235 ms with two lanes, 1243 ms with
# one), and a second stream doubles the allocator's cached pools.
_DC_LANES = int(_os.environ.get("OB200_EIGH_LANES", "1"))
_lane_pools: dict[int, tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]] = {}


def _lane_pool(device: torch.device) -> tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _lane_pools:
        _lane_pools[key] = (
            ThreadPoolExecutor(max_workers=2, thread_name_prefix="ob200-eigh-lane"),
            [torch.cuda.Stream(device=device) for _ in range(2)],
        )
    return _lane_pools[key]


def native_eigh(
    ext: Any, mats: list[Tensor], status: Tensor, hints: list[Tensor | None] | None = None
) -> list[tuple[Tensor, Tensor] | None]:
    """Eigendecompositions of symmetric fp32 matrices larger than the Jacobi kernel's limit with the
    divide-and-conquer solver on the tensor cores, in chunks of bounded workspace, largest first.
    An entry is ``None`` where the solver gave the matrix up (the caller falls back to the library).
    ``hints``: per matrix, eigenvalues of the same factor from its previous refresh (CPU tensor) or
    ``None``; they steer the solver's split points only."""
    from optimizers_b200.matrix.eigh_dc import NativeBackend, eigh_divide_and_conquer

    out: list[tuple[Tensor, Tensor] | None] = [None] * len(mats)
    if not mats or not _DC_ENABLED:
        return out
    order = sorted(range(len(mats)), key=lambda i: -mats[i].shape[0])
    free_bytes, _ = torch.cuda.mem_get_info(mats[0].device)
    free_bytes += torch.cuda.memory_reserved(mats[0].device) - torch.cuda.memory_allocated(mats[0].device)  # cached blocks are reusable
    limit = max(min(_DC_CHUNK_ELEMS, free_bytes // (3 * 4 * _DC_WORKSPACE_ARRAYS)), 1)
    chunks: list[list[int]] = [[]]
    size = 0
    for i in order:
        d2 = mats[i].shape[0] ** 2
        if chunks[-1] and size + d2 > limit:
            chunks.append([])
            size = 0
        chunks[-1].append(i)
        size += d2
    device = mats[0].device
    main = torch.cuda.current_stream(device)

    def solve(group: list[int], stream: torch.cuda.Stream | None):
        backend = NativeBackend(ext, device, status)
        group_hints = [hints[i] for i in group] if hints is not None else None
        if stream is None:
            return backend, eigh_divide_and_conquer(backend, [mats[i] for i in group], hints=group_hints)
        with torch.cuda.stream(stream):
            lams, vecs, info = eigh_divide_and_conquer(backend, [mats[i] for i in group], hints=group_hints)
            for t in (*lams, *vecs):
                if t is not None:
                    t.record_stream(main)  # allocated from this lane's pool, consumed on the caller's stream
        return backend, (lams, vecs, info)

    for chunk in chunks:
        # Two lanes: the host work of a round (launch tables, thousands of scratch views) is about
        # a third of a refresh and the device idles meanwhile.  Each lane is a thread with its own
        # stream driving half of the matrices; a lane blocked in a device read has released the
        # interpreter lock, so the other lane's host work runs while this lane's kernels do.
        lanes = [chunk[0::2], chunk[1::2]] if _DC_LANES > 1 and len(chunk) >= 8 else [chunk]
        if len(lanes) == 1:
            results = [solve(chunk, None)]
        else:
            from optimizers_b200.matrix.eigh_dc import prepare_test_matrix

            prepare_test_matrix(ext, device, max(mats[i].shape[0] for i in chunk))  # shared by the lanes: made once
            executor, streams = _lane_pool(device)
            for st in streams:
                st.wait_stream(main)
            futures = [executor.submit(solve, lane, st) for lane, st in zip(lanes, streams)]
            results = [f.result() for f in futures]
            for st in streams:
                main.wait_stream(st)
        lams, vecs = [None] * len(chunk), [None] * len(chunk)
        info = {"rounds": 0, "sign_computations": 0, "sign_cubes": 0.0, "one_sided_splits": 0, "failed": [], "reasons": {}}
        leaves_retried, failed_in_finish = 0, []
        position = {i: n for n, i in enumerate(chunk)}
        for lane, (lane_backend, (lane_lams, lane_vecs, lane_info)) in zip(lanes, results, strict=True):
            for r, i in enumerate(lane):
                lams[position[i]], vecs[position[i]] = lane_lams[r], lane_vecs[r]
            info["rounds"] = max(info["rounds"], lane_info["rounds"])
            for key in ("sign_computations", "sign_cubes", "one_sided_splits"):
                info[key] += lane_info[key]
            info["failed"] += [position[lane[r]] for r in lane_info["failed"]]
            info["reasons"].update({position[lane[r]]: why for r, why in lane_info["reasons"].items()})
            leaves_retried += lane_backend.leaves_retried
            failed_in_finish += [position[lane[r]] for r in lane_backend.failed_in_finish]
        backend = SimpleNamespace(leaves_retried=leaves_retried, failed_in_finish=failed_in_finish)
        for i, lam, Q in zip(chunk, lams, vecs, strict=True):
            if lam is not None:
                out[i] = (lam, Q)
        logger.info(
            "divide-and-conquer eigh: %d matrices (largest %d), %d rounds, %d sign computations, work %.2f x sum d^3, "
            "%d one-sided splits, %d leaves retried",
            len(chunk), mats[chunk[0]].shape[0], info["rounds"], info["sign_computations"],
            info["sign_cubes"] / sum(float(mats[i].shape[0]) ** 3 for i in chunk), info["one_sided_splits"],
            backend.leaves_retried,
        )
        given_up = sorted(set(info["failed"]) | set(backend.failed_in_finish))
        if given_up:
            logger.warning(
                "The divide-and-conquer eigensolver gave up on %d of %d matrices; the library eigensolver takes them. %s",
                len(given_up), len(chunk), "; ".join(f"[{chunk[r]}] {why}" for r, why in info["reasons"].items()) or "(leaf Jacobi sweeps exhausted)",
            )
    return out


# OB200_EIGH_HINTS=1: plan the eigensolver's split points from the eigenvalues of the previous refresh.
# Measured on the factors of GPT-2 124M (342 matrices, 256 to 2048): 15 % fewer sign-iteration flops, but the
# better balanced splits have larger QR factorisations and the refresh as a whole was 15 % slower, so
# the default is the mean / geometric rule.
_USE_HINTS = _os.environ.get("OB200_EIGH_HINTS", "0") == "1"


def _hints_of(items: list[Any], indices: list[int]) -> list[Tensor | None] | None:
    """Eigenvalues each factor had at its previous refresh (kept on the engine's block record, on
    the host; not part of the checkpoint: after a resume the first refresh plans without them)."""
    if not _USE_HINTS:
        return None
    out = []
    for i in indices:
        store = getattr(items[i].block, "eig_hints", None)
        out.append(store.get(items[i].k) if store is not None else None)
    return out


def _remember_eigenvalues(items: list[Any], indices: list[int], solved: list[tuple[Tensor, Tensor] | None]) -> None:
    good = [(i, pair[0]) for i, pair in zip(indices, solved, strict=True) if pair is not None]
    if not good or not _USE_HINTS:
        return
    flat = torch.cat([lam for _, lam in good]).cpu()  # one device -> host copy for all factors
    cursor = 0
    for i, lam in good:
        n = lam.numel()
        block = items[i].block
        try:
            if getattr(block, "eig_hints", None) is None:
                block.eig_hints = {}
            block.eig_hints[items[i].k] = flat[cursor : cursor + n].clone()
        except AttributeError:  # a block record without the slot (foreign caller): no hints
            pass
        cursor += n


class _Item:
    __slots__ = ("block", "k", "A", "root", "qs_hi", "qs_lo", "q_hi", "q_lo", "error", "done", "lam", "Q")

    def __init__(self, block: Any, k: int, A: Tensor, root: float) -> None:
        self.block, self.k, self.A, self.root = block, k, A, root
        self.error: Exception | None = None
        self.done: torch.cuda.Event | None = None


def eigen_refresh_supported(cfg: Any) -> bool:
    return isinstance(cfg, EigenConfig) and cfg.eigendecomposition_offload_device == ""


def eigdec_refresh_supported(cfg: Any) -> bool:
    """Eigendecomposed Shampoo: plain eigh (no adaptive skipping, no offload) runs batched."""
    return (
        isinstance(cfg, EighEigendecompositionConfig) and cfg.eigendecomposition_offload_device == "" and cfg.tolerance == 0.0
    )


def batched_eigen_refresh(ext: Any, blocks: list[Any], bias_correction2: Tensor | float, split: bool, status: Tensor) -> None:
    """Refresh ``inv_factor_matrices`` (state) and the ``inv_hi/inv_lo`` mirrors of ``blocks``.
    For eigendecomposed Shampoo (``factors.kind == "eigendecomposed"``) the state refreshed is the
    pair (eigenvalues, eigenvectors) and the mirrors receive the reconstruction, split in place.

    ``blocks`` are the native engine's block records (``.factors`` is the ``BlockFactors`` of the
    block, ``.inv_hi/.inv_lo`` the mirrors).  Raises ``PreconditionerValueError`` on non-finite
    factors or results and ``ValueError`` once a block exceeds its tolerated failures."""
    if not blocks:
        return
    device = blocks[0].inv_hi[0].device
    main = torch.cuda.current_stream(device)

    clock = _PhaseClock("eigen refresh")
    # 1. prepare + one finiteness read
    items: list[_Item] = [_Item(b, k, A, b.factors.roots[k]) for b, k, A in _prepared_factors(ext, blocks, bias_correction2)]
    finite = _all_finite([it.A for it in items])
    for it, ok in zip(items, finite):
        if not ok:
            index = it.block.factors.factor_matrix_indices[it.k]
            raise PreconditionerValueError(
                f"Encountered nan/inf values in factor matrix {index}! "
                "To mitigate, check if nan inputs are being passed into the network or nan gradients are being passed to the optimizer. "
                "Otherwise, in some cases, this may be due to divergence of the algorithm. To mitigate, try decreasing the learning rate or increasing grafting epsilon."
            )

    clock.tick("prepare")
    # 2. eigendecompositions on the stream pool (largest first for balance)
    ready = torch.cuda.Event()
    ready.record(main)
    lazy_pool: list = []  # the stream pool is only set up when a factor falls back to the library

    def pool():
        if not lazy_pool:
            lazy_pool.extend(_pool(device))
        return lazy_pool

    def finish(it: _Item, lam: Tensor, Q: Tensor) -> None:
        """Eigenpairs -> the two GEMM operands of the reconstruction, (Q s) and Q, as (hi, lo) pairs."""
        kf = it.block.factors
        cfg = kf.amortized_computation_config
        it.lam = lam
        scale = mf.stabilized_inverse_power(lam, Fraction(it.root), kf.epsilon, cfg.rank_deficient_stability_config)
        Q = Q.contiguous()
        it.Q = Q
        Qs = (Q * scale.unsqueeze(0)).contiguous()
        d = Q.shape[0]
        ld = _pad4(d)
        if split:
            it.qs_hi, it.qs_lo = torch.zeros(d, ld, device=device), torch.zeros(d, ld, device=device)
            it.q_hi, it.q_lo = torch.zeros(d, ld, device=device), torch.zeros(d, ld, device=device)
            ext.tf32_split(Qs, it.qs_hi[:, :d], it.qs_lo[:, :d])
            ext.tf32_split(Q, it.q_hi[:, :d], it.q_lo[:, :d])
        else:
            it.qs_hi = torch.zeros(d, ld, device=device)
            it.q_hi = torch.zeros(d, ld, device=device)
            it.qs_hi[:, :d].copy_(Qs)
            it.q_hi[:, :d].copy_(Q)
            it.qs_lo = it.q_lo = None

    def work(it: _Item, slot: int) -> None:
        kf = it.block.factors
        cfg = kf.amortized_computation_config  # EigenConfig, or EighEigendecompositionConfig (eigendecomposed)
        stream = pool()[1][slot]
        with torch.cuda.device(device), torch.cuda.stream(stream):
            stream.wait_event(ready)
            try:
                lam, Q = mf.matrix_eigendecomposition(
                    it.A,
                    epsilon=kf.epsilon,
                    eigendecomposition_config=EighEigendecompositionConfig(
                        rank_deficient_stability_config=cfg.rank_deficient_stability_config,
                        retry_double_precision=cfg.retry_double_precision,
                        tolerance=0.0,
                    ),
                )
                finish(it, lam, Q)
            except Exception as exception:  # keep the previous inverse root of this factor
                it.error = exception
            it.done = torch.cuda.Event()
            it.done.record(stream)

    # Small factors: one launch of the shared-memory Jacobi eigensolver for all of them; the
    # library eigensolver (stream pool) takes the rest and any matrix Jacobi did not converge on.
    pooled = list(range(len(items)))
    small = [i for i in pooled if items[i].A.shape[0] <= ext.JACOBI_MAX_N]
    if small:
        ridged = []
        for i in small:
            kf = items[i].block.factors
            stability = kf.amortized_computation_config.rank_deficient_stability_config
            ridged.append(mf._ridge(items[i].A, kf.epsilon * getattr(stability, "perturb_before_computation", 0)).contiguous())
        lams, qs, sweeps = ext.jacobi_eigh(ridged, _JACOBI_MAX_SWEEPS, _JACOBI_TOLERANCE)
        used = sweeps.cpu().tolist()
        done_here = set()
        # Converged matrices of one size and root share their follow-up work: a handful of
        # launches per group instead of a dozen per matrix.
        groups: dict[tuple[int, float], list[tuple[int, Tensor, Tensor]]] = {}
        for i, lam, Q, n_sweeps in zip(small, lams, qs, used, strict=True):
            if n_sweeps > _JACOBI_MAX_SWEEPS:
                continue  # not converged: let the library solver handle it
            kf = items[i].block.factors
            if not isinstance(kf.amortized_computation_config.rank_deficient_stability_config, PerturbationConfig):
                # the pseudo-inverse cut-off is per matrix: no shared follow-up
                try:
                    finish(items[i], lam, Q)
                except Exception as exception:
                    items[i].error = exception
                items[i].done = torch.cuda.Event()
                items[i].done.record(main)
                done_here.add(i)
                continue
            groups.setdefault((lam.shape[0], float(items[i].root)), []).append((i, lam, Q))
        for (d, root), members in groups.items():
            kf0 = items[members[0][0]].block.factors
            stability = kf0.amortized_computation_config.rank_deficient_stability_config
            try:
                lam_b = torch.stack([m[1] for m in members])  # [B, d]
                q_b = torch.stack([m[2] for m in members])  # [B, d, d]
                scale_b = mf.stabilized_inverse_power(
                    lam_b, Fraction(root), kf0.epsilon, stability, lambda_min=lam_b.min(dim=-1, keepdim=True).values
                )
                qs_b = q_b * scale_b.unsqueeze(-2)
                n_b, ld = len(members), _pad4(d)
                bufs = [torch.zeros(n_b, d, ld, device=device) for _ in range(4 if split else 2)]
                if split:
                    ext.tf32_split(qs_b.view(n_b * d, d), bufs[0].view(n_b * d, ld)[:, :d], bufs[1].view(n_b * d, ld)[:, :d])
                    ext.tf32_split(q_b.view(n_b * d, d), bufs[2].view(n_b * d, ld)[:, :d], bufs[3].view(n_b * d, ld)[:, :d])
                else:
                    bufs[0][:, :, :d].copy_(qs_b)
                    bufs[1][:, :, :d].copy_(q_b)
                for n, (i, lam, Q) in enumerate(members):
                    it = items[i]
                    it.lam, it.Q = lam, Q
                    if split:
                        it.qs_hi, it.qs_lo, it.q_hi, it.q_lo = bufs[0][n], bufs[1][n], bufs[2][n], bufs[3][n]
                    else:
                        it.qs_hi, it.q_hi, it.qs_lo, it.q_lo = bufs[0][n], bufs[1][n], None, None
            except Exception as exception:
                for i, _, _ in members:
                    items[i].error = exception
            for i, _, _ in members:
                items[i].done = torch.cuda.Event()
                items[i].done.record(main)
                done_here.add(i)
        pooled = [i for i in pooled if i not in done_here]
        ready.record(main)

    clock.tick("small factors (jacobi + scaling)")
    # Larger factors: the batched divide-and-conquer eigensolver; the library takes what it gives up.
    large = [i for i in pooled if items[i].A.shape[0] > ext.JACOBI_MAX_N and items[i].A.dtype == torch.float32]
    if large:
        ridged = []
        for i in large:
            kf = items[i].block.factors
            stability = kf.amortized_computation_config.rank_deficient_stability_config
            ridged.append(mf._ridge(items[i].A, kf.epsilon * getattr(stability, "perturb_before_computation", 0)))
        solved = native_eigh(ext, ridged, status, _hints_of(items, large))
        clock.tick("large factors: eigensolver")
        _remember_eigenvalues(items, large, solved)
        done_here = set()
        for i, pair in zip(large, solved, strict=True):
            if pair is None:
                continue
            try:
                finish(items[i], *pair)
            except Exception as exception:
                items[i].error = exception
            items[i].done = torch.cuda.Event()
            items[i].done.record(main)
            done_here.add(i)
        pooled = [i for i in pooled if i not in done_here]
        ready.record(main)

    order = sorted(pooled, key=lambda i: -items[i].A.shape[0])
    futures = [pool()[0].submit(work, items[i], n % _POOL_SIZE) for n, i in enumerate(order)]
    for f in futures:
        f.result()
    for it in items:
        assert it.done is not None
        main.wait_event(it.done)

    clock.tick("scaling + operand split, library fallback")
    # 3. grouped reconstruction X = (Q s) Q^T, written as plain fp32 into the hi mirror
    specs = []
    good = [it for it in items if it.error is None]
    for it in good:
        d = it.A.shape[0]
        out = it.block.inv_hi[it.k]
        specs.append(
            (it.qs_hi[:, :d], it.qs_lo[:, :d] if split else None, it.q_hi[:, :d], it.q_lo[:, :d] if split else None,
             out, None, None, None, out.stride(0), 0, 0, False)
        )
    if specs:
        plan = ext.build_gemm_plan(specs)
        ext.run_gemm_plan(*plan, 1.0, 0.0, split, status)

    clock.tick("reconstruction")
    # 4. checkpoint state (packed upper triangle) from the result + one finiteness read; the
    #    operand mirrors are then rebuilt from the state so that both always agree exactly
    checked: list[Tensor] = []
    pack_specs: list[tuple[Tensor, Tensor]] = []  # fp32 state: one grouped launch writes every packed triangle
    for it in good:
        d = it.A.shape[0]
        kf = it.block.factors
        if kf.kind == "eigendecomposed":
            kf.factor_matrices_eigenvalues[it.k].copy_(it.lam)
            kf.factor_matrices_eigenvectors[it.k].copy_(it.Q)
            mirror = it.block.inv_hi[it.k][:, :d]
            checked.append(mirror)  # finite only if the eigenvalues it was built from are
            if split:  # the reconstruction becomes the (hi, lo) operand pair in place
                ext.tf32_split(mirror, mirror, it.block.inv_lo[it.k][:, :d])
            continue
        state = kf.inv_factor_matrices[it.k]
        if state.dtype == torch.float32 and (state.dim() == 1 or state.stride(-1) == 1):
            pack_specs.append((it.block.inv_hi[it.k][:, :d], state))
        else:
            state.copy_(kf.pack(it.block.inv_hi[it.k][:, :d]).to(dtype=state.dtype))
        checked.append(state)
    if pack_specs:
        ext.pack_upper(*ext.build_pack_table(pack_specs))
    for it, ok in zip(good, _all_finite(checked)):
        if not ok:
            index = it.block.factors.factor_matrix_indices[it.k]
            raise PreconditionerValueError(
                f"Encountered nan or inf values in matrices of factor matrix {index}! "
                "To mitigate, check factor matrix before the matrix computation."
            )
    main.synchronize()  # scratch allocated on the pool streams may now be reused
    clock.tick("state packing + finiteness")
    clock.report()

    # failure bookkeeping per block
    last_error: dict[int, Exception | None] = {}
    for it in items:
        if it.error is not None:
            index = it.block.factors.factor_matrix_indices[it.k]
            logger.warning(
                f"Matrix computation failed for factor matrix {index} with exception={it.error!r}. Using previous preconditioner and continuing..."
            )
            last_error[id(it.block)] = it.error
        else:
            last_error.setdefault(id(it.block), None)
    for b in blocks:
        b.factors.note_refresh_outcome(last_error.get(id(b)))


# ----------------------------------------------------------------------------------------------
# Coupled Newton inverse root, all factors at once, on the grouped tensor-core GEMM
# ----------------------------------------------------------------------------------------------
def newton_refresh_supported(cfg: Any) -> bool:
    from optimizers_b200.config import CoupledHigherOrderConfig, CoupledNewtonConfig

    return isinstance(cfg, (CoupledNewtonConfig, CoupledHigherOrderConfig))


def _taylor_coefficients(p: int, order: int) -> list[float]:
    """Coefficients of 1, x, ..., x^(order-1) in the Taylor series of (1 - x)^(-1/p)."""
    coeff = [1.0]
    num = den = 1
    for i in range(1, order):
        num *= 1 + (i - 1) * p
        den *= i * p
        coeff.append(num / den)
    return coeff


class _NewtonItem:
    """Iteration buffers of one factor.  Every matrix is kept as a (hi, lo) tf32 pair in padded
    storage so that it can be an operand of the next grouped GEMM; ``X`` and ``M`` ping-pong."""

    __slots__ = (
        "block", "k", "d", "root", "power", "A", "Ar", "X", "M", "Mp", "R", "T", "pw", "err", "converged", "last_err", "iters",
    )


def _pair(d: int, device: torch.device, split: bool) -> tuple[Tensor, Tensor | None]:
    ld = _pad4(d)
    hi = torch.zeros(d, ld, device=device)
    return hi, (torch.zeros(d, ld, device=device) if split else None)


def _v(p: tuple[Tensor, Tensor | None], d: int) -> tuple[Tensor, Tensor | None]:
    return p[0][:, :d], (p[1][:, :d] if p[1] is not None else None)


def _power_chain(p: int) -> list[tuple[int, int, int]]:
    """Multiplication schedule for M_p^p as ``(result exponent, left exponent, right exponent)``
    triples: repeated squaring, then products of the squares that make up ``p``."""
    steps: list[tuple[int, int, int]] = []
    e = 1
    squares = [1]
    while e * 2 <= p:
        steps.append((e * 2, e, e))
        e *= 2
        squares.append(e)
    acc = None
    for s in reversed(squares):
        if p & s:
            if acc is None:
                acc = s
            else:
                steps.append((acc + s, acc, s))
                acc += s
    return steps


def batched_newton_refresh(
    ext: Any, blocks: list[Any], bias_correction2: Tensor | float, split: bool, status: Tensor, check_every: int = 4
) -> None:
    """Coupled Newton iteration for ``(F/bc2 + eps I)^(-1/p)`` of every factor of ``blocks``.

    Per iteration and factor: ``M_p = (1-a) I + a M`` (a = -1/p; grouped pointwise kernel that also
    splits the operand), ``X <- X M_p``, ``M <- M_p^p M`` (grouped tcgen05 GEMMs whose epilogues
    write the split result).  All matrices are polynomials in the same symmetric matrix, hence
    symmetric and commuting, which is what lets the K-major "TN" kernel compute plain products.
    ``max|M - I|`` is reduced on the device; the host reads the error vector every
    ``check_every`` iterations and drops converged factors from the launch tables.  A factor stops
    when its error is below the configured tolerance, when the iteration limit is reached
    (warning, as in the reference), or when the error stalls above the tolerance at the
    rounding floor of the tensor-core accumulation (error below 1e-3 and not improved by 10 %
    between two checks).

    ``CoupledHigherOrderConfig`` runs through the same loop (reference:
    distributed_shampoo/preconditioner/matrix_functions.py:439-661): the ridge is
    ``max(rel_epsilon * ||A||_inf, abs_epsilon)``, the start is ``z = 1 / trace``, the first step is a
    Newton step and every later one builds ``M_p = sum_i c_i (I - M)^i`` (Taylor coefficients of
    ``(1 - x)^(-1/p)``) by Horner products whose ``+ c_i I`` is the GEMM epilogue's diagonal term;
    the error is read every iteration, an increase by 20 % stops the factor, and at the end
    ``max |A_r X^p - I| <= 0.1`` is verified on the device and ``X^q`` formed for a fractional
    root ``p / q``."""
    from optimizers_b200.config import CoupledHigherOrderConfig

    if not blocks:
        return
    # The iteration amplifies operand rounding: a single tf32 product per multiply does not
    # converge (error stalls near 1e-1), so the split products are used whatever the engine's
    # GEMM mode for the per-step kernels is.
    split = True
    device = blocks[0].inv_hi[0].device
    cfg = blocks[0].factors.amortized_computation_config
    max_iterations, tolerance = cfg.max_iterations, cfg.tolerance
    higher = cfg if isinstance(cfg, CoupledHigherOrderConfig) else None

    items: list[_NewtonItem] = []
    for b, k, A in _prepared_factors(ext, blocks, bias_correction2):
        kf = b.factors
        root = Fraction(kf.roots[k])
        if higher is None and root.denominator != 1:
            raise ValueError(f"root.denominator={root.denominator} must be equal to 1 to use coupled inverse Newton iteration!")
        if higher is not None and min(abs(root.numerator), abs(root.denominator)) >= 10:
            logger.warning(
                f"abs(root.numerator)={abs(root.numerator)} and abs(root.denominator)={abs(root.denominator)} are probably too big for best performance."
            )
        it = _NewtonItem()
        it.block, it.k, it.d, it.root, it.power, it.A = b, k, A.shape[0], root.numerator, root.denominator, A
        it.converged, it.last_err, it.iters = False, float("inf"), 0
        it.Ar = None
        items.append(it)
    finite = _all_finite([it.A for it in items])
    for it, ok in zip(items, finite):
        if not ok:
            index = it.block.factors.factor_matrix_indices[it.k]
            raise PreconditionerValueError(f"Encountered nan/inf values in factor matrix {index}!")

    # Initial iterates: z = (p+1) / (2 ||A||_F), X = z^(1/p) I, M = z A  (no host synchronisation).
    errs = torch.zeros(len(items), device=device)
    for n, it in enumerate(items):
        d, p = it.d, it.root
        A_r = it.A.clone()
        if higher is None:
            A_r.diagonal().add_(it.block.factors.epsilon)
            z = (p + 1) / (2 * torch.linalg.norm(A_r))
        else:
            lam = torch.linalg.matrix_norm(it.A, torch.inf)
            A_r.diagonal().add_(torch.clamp(lam * higher.rel_epsilon, min=higher.abs_epsilon))
            z = torch.reciprocal(torch.trace(A_r))
            it.Ar = _pair(d, device, split)  # the verification at the end multiplies X^p by it
            ext.tf32_split(A_r, *_v(it.Ar, d))
        it.X = [_pair(d, device, split), _pair(d, device, split)]
        it.M = [_pair(d, device, split), _pair(d, device, split)]
        it.Mp = _pair(d, device, split)
        it.pw = {}
        x0 = torch.zeros(d, d, device=device)
        x0.diagonal().fill_(1.0)
        x0 *= z ** (1.0 / p)
        m0 = A_r * z
        for src, dst in ((x0, it.X[0]), (m0, it.M[0])):
            hi, lo = _v(dst, d)
            if split:
                ext.tf32_split(src, hi, lo)
            else:
                hi.copy_(src)
        it.err = errs[n : n + 1]
    order = higher.order if higher is not None else 0
    return _newton_iterate(ext, items, errs, split, status, max_iterations, tolerance, check_every, blocks, order)


_NEWTON_CHUNK_ELEMS = 64 * 1024 * 1024  # sum of d^2 iterated together (16 arrays of that size are live)


def _newton_iterate(ext, items, errs, split, status, max_iterations, tolerance, check_every, blocks, order=0) -> None:
    failures: dict[int, Exception] = {}
    by_root: dict[int, list[_NewtonItem]] = {}
    for it in items:
        by_root.setdefault(it.root, []).append(it)  # grouped by the numerator p; q only matters at the end
    for p, group in by_root.items():
        chunk: list[_NewtonItem] = []
        size = 0
        for it in sorted(group, key=lambda x: -x.d):
            if chunk and size + it.d * it.d > _NEWTON_CHUNK_ELEMS:
                _newton_run_chunk(ext, chunk, p, errs, split, status, max_iterations, tolerance, check_every, failures, order)
                chunk, size = [], 0
            chunk.append(it)
            size += it.d * it.d
        if chunk:
            _newton_run_chunk(ext, chunk, p, errs, split, status, max_iterations, tolerance, check_every, failures, order)

    # results -> packed checkpoint state; one finiteness read
    good = [it for it in items if id(it) not in failures]
    flags = []
    for it in good:
        kf = it.block.factors
        hi, lo = _v(it.X, it.d)
        full = hi + lo if lo is not None else hi
        state = kf.inv_factor_matrices[it.k]
        state.copy_(kf.pack(full).to(dtype=state.dtype))
        flags.append(torch.isfinite(state).all())
    if flags:
        for it, ok in zip(good, torch.stack(flags).cpu().tolist()):
            if not ok:
                index = it.block.factors.factor_matrix_indices[it.k]
                raise PreconditionerValueError(f"Encountered nan or inf values in matrices of factor matrix {index}!")
    last_error: dict[int, Exception | None] = {}
    for it in items:
        err = failures.get(id(it))
        if err is not None:
            logger.warning(
                f"Matrix computation failed for factor matrix {it.block.factors.factor_matrix_indices[it.k]} with exception={err!r}. Using previous preconditioner and continuing..."
            )
            last_error[id(it.block)] = err
        else:
            last_error.setdefault(id(it.block), None)
    for b in blocks:
        b.factors.note_refresh_outcome(last_error.get(id(b)))


def _newton_run_chunk(ext, chunk, p, errs, split, status, max_iterations, tolerance, check_every, failures, order=0) -> None:
    device = errs.device
    alpha = -1.0 / p
    chain = _power_chain(p)
    coeff = _taylor_coefficients(p, order) if order else None
    horner = max(order - 2, 0)  # products per higher-order step that build M_p
    if order:
        check_every = 1  # the stopping rule compares consecutive errors
    for it in chunk:
        d = it.d
        it.pw = {e: _pair(d, device, split) for e, _, _ in chain}
        # full-precision copies of M (source of the affine step and of the error measure)
        it.A = [torch.zeros(d, _pad4(d), device=device), torch.zeros(d, _pad4(d), device=device)]
        hi, lo = _v(it.M[0], d)
        it.A[0][:, :d].copy_(hi + lo if lo is not None else hi)
        if horner:
            it.R = _pair(d, device, split)
            it.T = [_pair(d, device, split) for _ in range(min(horner, 2))]

    def gemm(a, b, out, d, c_full=None, flags=0):
        # Every product here is a polynomial in one symmetric matrix, hence symmetric: only the
        # upper tiles are computed and mirrored bit for bit.  Without that, the antisymmetric part
        # of the rounding errors is amplified from step to step (the kernel multiplies by B^T) and
        # the error of an ill-conditioned factor stalls near 1e-3.
        a_hi, a_lo = _v(a, d)
        b_hi, b_lo = _v(b, d)
        flags |= ext.FLAG_MIRROR
        if split:
            flags |= ext.FLAG_SPLIT_OUT | (0 if c_full is not None else ext.FLAG_NO_C)
            return (a_hi, a_lo, b_hi, b_lo, c_full, out[0], out[1], None, out[0].stride(0), out[0].stride(0), flags, True)
        # single-pass mode: the plain result is the operand of the next product
        return (a_hi, None, b_hi, None, out[0], None, None, None, out[0].stride(0), 0, flags, True)

    def build(active, cur, newton_step):
        nxt = cur ^ 1
        full_m = lambda it, which: it.A[which][:, : it.d] if split else it.M[which][0][:, : it.d]  # noqa: E731
        pre = []  # (table, a, b) pointwise passes, then (plan, gamma) products that end in M_p
        if newton_step or not horner:
            # Newton: (1 - a) I + a M;  order 2: c0 I + c1 (I - M)
            lin = (alpha, 1.0 - alpha) if (newton_step or not order) else (-coeff[1], coeff[0] + coeff[1])
            pre.append((ext.build_mat_table([(full_m(it, cur), *_v(it.Mp, it.d), None) for it in active]), *lin))
            products = []
        else:
            # R = I - M;  T = c_{o-1} R + c_{o-2} I;  T <- c_i I + T R for i = o-3 .. 0, the last one into M_p
            pre.append((ext.build_mat_table([(full_m(it, cur), *_v(it.R, it.d), None) for it in active]), -1.0, 1.0))
            pre.append((
                ext.build_mat_table([(full_m(it, cur), *_v(it.T[0], it.d), None) for it in active]),
                -coeff[order - 1], coeff[order - 1] + coeff[order - 2],
            ))
            products = []
            for n, i in enumerate(reversed(range(order - 2))):
                src = lambda it: it.T[n % 2]  # noqa: E731
                dst = (lambda it: it.Mp) if i == 0 else (lambda it: it.T[(n + 1) % 2])  # noqa: E731
                specs = [gemm(src(it), it.R, dst(it), it.d, flags=ext.FLAG_ADD_DIAG) for it in active]
                products.append((ext.build_gemm_plan(specs), coeff[i]))
        stages = [[gemm(it.X[cur], it.Mp, it.X[nxt], it.d) for it in active]]
        for n, (e, l, r) in enumerate(chain):
            specs = [gemm(it.Mp if l == 1 else it.pw[l], it.Mp if r == 1 else it.pw[r], it.pw[e], it.d) for it in active]
            if n == 0:
                stages[0] = stages[0] + specs  # independent of X <- X M_p: same launch
            else:
                stages.append(specs)
        last = []
        for it in active:
            top = it.Mp if p == 1 else it.pw[p]
            c_full = it.A[nxt] if split else None
            last.append(gemm(top, it.M[cur], it.M[nxt], it.d, c_full=c_full))
        stages.append(last)
        plans = [ext.build_gemm_plan(s) for s in stages]
        err_src = [(full_m(it, nxt), None, None, it.err) for it in active]
        return pre, products, plans, ext.build_mat_table(err_src)

    active = list(chunk)
    cur = 0
    tables = {}
    iteration = 0
    while active:
        key = (cur, bool(order) and iteration == 0)
        if key not in tables:
            tables[key] = build(active, cur, key[1])
        pre, products, plans, err_table = tables[key]
        for table, a, b in pre:
            ext.affine_identity_split(*table, a, b)
        for plan, gamma in products:
            ext.run_gemm_plan(*plan, 1.0, 0.0, split, status, gamma)
        for plan in plans:
            ext.run_gemm_plan(*plan, 1.0, 0.0, split, status)
        iteration += 1
        cur ^= 1
        if iteration % check_every and iteration < max_iterations:
            continue
        errs.zero_()
        ext.identity_error(*err_table)
        values = torch.stack([it.err[0] for it in active]).cpu().tolist()  # the only host read of the loop
        still = []
        for it, e in zip(active, values):
            it.iters = iteration
            stalled = e < 1e-3 and e > 0.9 * it.last_err
            grew = bool(order) and e > 1.2 * it.last_err  # the reference's early stop of the higher-order iteration
            if e != e or e == float("inf"):
                failures[id(it)] = ArithmeticError("coupled Newton iteration produced NaN/Inf")
            elif e <= tolerance or stalled or grew or iteration >= max_iterations:
                if e > tolerance and iteration >= max_iterations:
                    logger.warning(
                        "Higher order method did not converge and reached maximum number of iterations!"
                        if order else "Newton did not converge and reached maximum number of iterations!"
                    )
            else:
                it.last_err = e
                still.append(it)
                continue
            it.X = it.X[cur]  # the iterate that was current when the factor stopped
        if len(still) != len(active):
            tables = {}
        active = still
    if order:
        _verify_and_power(ext, [it for it in chunk if id(it) not in failures], p, chain, gemm, errs, split, status, failures)
    for it in chunk:  # release iteration buffers
        it.M = it.Mp = it.pw = it.A = it.R = it.T = it.Ar = None


def _verify_and_power(ext, items, p, chain, gemm, errs, split, status, failures) -> None:
    """End of the higher-order iteration: fail the factors with ``max |A_r X^p - I| > 0.1``
    (reference: matrix_functions.py:628-640) and raise X to the denominator of a fractional root."""
    if not items:
        return
    device = errs.device

    def run(specs):
        if specs:
            ext.run_gemm_plan(*ext.build_gemm_plan(specs), 1.0, 0.0, split, status)

    for e, l, r in chain:  # X^p through the buffers of the power chain
        run([gemm(it.X if l == 1 else it.pw[l], it.X if r == 1 else it.pw[r], it.pw[e], it.d) for it in items])
    specs = []
    for it in items:
        top = it.X if p == 1 else it.pw[p]
        a_hi, a_lo = _v(top, it.d)
        b_hi, b_lo = _v(it.Ar, it.d)
        specs.append((a_hi, a_lo if split else None, b_hi, b_lo if split else None, it.A[0][:, : it.d], None, None, None,
                      it.A[0].stride(0), 0, ext.FLAG_MIRROR, True))
    run(specs)
    errs.zero_()
    ext.identity_error(*ext.build_mat_table([(it.A[0][:, : it.d], None, None, it.err) for it in items]))
    values = torch.stack([it.err[0] for it in items]).cpu().tolist()
    for it, e in zip(items, values):
        if not e <= 1e-1:
            failures[id(it)] = ArithmeticError(
                f"Error in matrix inverse root (before powering for fractions) {e} exceeds threshold 1e-1, raising an exception!"
            )
    by_power: dict[int, list] = {}
    for it in items:
        if it.power > 1 and id(it) not in failures:
            by_power.setdefault(it.power, []).append(it)
    for q, group in by_power.items():
        steps = _power_chain(q)
        for it in group:
            it.pw = {e: _pair(it.d, device, split) for e, _, _ in steps}
        for e, l, r in steps:
            run([gemm(it.X if l == 1 else it.pw[l], it.X if r == 1 else it.pw[r], it.pw[e], it.d) for it in group])
        for it in group:
            it.X = it.pw[q]


# --------------------------------------------------------------------------------------------------
# Batched quintic Newton-Schulz orthogonalisation on the grouped tensor-core GEMM
# --------------------------------------------------------------------------------------------------
class BatchedNewtonSchulz:
    """Orthogonalises a fixed list of matrix shapes, all matrices advancing together: every
    iteration is three grouped GEMM launches over the whole list instead of three library GEMMs
    per matrix (reference: ``matrix_functions.py:956-1008``, called per block from
    ``spectral_descent_preconditioner_list.py``).

    With X tall (wide inputs are iterated transposed) and B = X^T X an iteration is
        B      = Xt Xt^T                      (Xt = X^T as a K-major operand)
        D      = b B + c B B                  (in place on the plain copy of B: beta = b, alpha = c)
        X      = a X + X D,   Xt = a Xt + D Xt
    where the last two products are one launch; the transposed iterate is advanced alongside because
    the GEMM takes both operands K-major.  Operand (hi, lo) pairs of the iterate are double
    buffered: a launch never writes operands that other tiles of the same launch still read."""

    def __init__(self, ext: Any, shapes: list[tuple[int, int]], device: torch.device, split: bool = True) -> None:
        self._ext = ext
        self._split = split
        self._device = device
        self.shapes = list(shapes)
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        z = lambda r, c: torch.zeros(r, _pad4(c), device=device)  # noqa: E731
        pair = lambda r, c: (z(r, c), z(r, c) if split else None)  # noqa: E731
        self._items = []
        for m, n in self.shapes:
            wide = m < n
            M, N = (n, m) if wide else (m, n)
            it = {
                "wide": wide, "M": M, "N": N,
                "X": z(M, N), "Xt": z(N, M), "B": z(N, N),
                "Xs": [pair(M, N), pair(M, N)], "Xts": [pair(N, M), pair(N, M)],
                "Bs": pair(N, N), "Ds": pair(N, N),
            }
            self._items.append(it)
        self._plans = [self._build(cur) for cur in (0, 1)]

    def _build(self, cur: int):
        ext, split = self._ext, self._split
        nxt = cur ^ 1
        SO = ext.FLAG_SPLIT_OUT

        def v(p, k):
            return p[0][:, :k], (p[1][:, :k] if p[1] is not None else None)

        def spec(a, b, k, c, out):
            a_hi, a_lo = v(a, k)
            b_hi, b_lo = v(b, k)
            if split:
                return (a_hi, a_lo, b_hi, b_lo, c, out[0], out[1], None, c.stride(0), out[0].stride(0), SO, False)
            # single-pass mode: operands are the plain arrays themselves
            return (a_hi, None, b_hi, None, c, None, None, None, c.stride(0), 0, 0, False)

        g1, g2, g3 = [], [], []
        for it in self._items:
            M, N = it["M"], it["N"]
            if split:
                xs, xts, bs, ds = it["Xs"][cur], it["Xts"][cur], it["Bs"], it["Ds"]
                xs_n, xts_n = it["Xs"][nxt], it["Xts"][nxt]
            else:
                # plain arrays double as operands; ping-pong the iterate itself
                xs, xts = (it["Xs"][cur][0], None), (it["Xts"][cur][0], None)
                xs_n, xts_n = (it["Xs"][nxt][0], None), (it["Xts"][nxt][0], None)
                bs, ds = (it["B"], None), (it["Ds"][0], None)
            if split:
                g1.append(spec(xts, xts, M, it["B"], bs))
                g2.append(spec(bs, bs, N, it["B"], ds))
                g3.append(spec(xs, ds, N, it["X"], xs_n))
                g3.append(spec(ds, xs, N, it["Xt"], xts_n))
            else:
                g1.append(spec(xts, xts, M, it["B"], None))
                g2.append(spec(bs, bs, N, ds[0], None))
                g3.append(spec(xs, ds, N, xs_n[0], None))
                g3.append(spec(ds, xs, N, xts_n[0], None))
        return tuple(ext.build_gemm_plan(s) for s in (g1, g2, g3))

    @torch.no_grad()
    def __call__(self, mats: list[Tensor], num_iterations: int, coefficients: tuple[float, float, float]) -> list[Tensor]:
        ext, split = self._ext, self._split
        a, b, c = coefficients
        norms = torch._foreach_norm(mats)
        for it, A, nrm in zip(self._items, mats, norms, strict=True):
            X = A / torch.clamp(nrm, min=1e-8)
            if it["wide"]:
                X = X.T
            M, N = it["M"], it["N"]
            it["X"][:, :N].copy_(X)
            it["Xt"][:, :M].copy_(X.T)
            if split:
                ext.tf32_split(it["X"][:, :N], it["Xs"][0][0][:, :N], it["Xs"][0][1][:, :N])
                ext.tf32_split(it["Xt"][:, :M], it["Xts"][0][0][:, :M], it["Xts"][0][1][:, :M])
            else:
                it["Xs"][0][0].copy_(it["X"])
                it["Xts"][0][0].copy_(it["Xt"])
        cur = 0
        for _ in range(num_iterations):
            p1, p2, p3 = self._plans[cur]
            ext.run_gemm_plan(*p1, 1.0, 0.0, split, self._status)
            if split:
                ext.run_gemm_plan(*p2, c, b, split, self._status)
                ext.run_gemm_plan(*p3, 1.0, a, split, self._status)
            else:
                # D = b B + c B B into its own array (B is an operand of this launch), X_next = a X + X D
                for it in self._items:
                    it["Ds"][0].copy_(it["B"])
                ext.run_gemm_plan(*p2, c, b, split, self._status)
                for it in self._items:
                    it["Xs"][cur ^ 1][0].copy_(it["Xs"][cur][0])
                    it["Xts"][cur ^ 1][0].copy_(it["Xts"][cur][0])
                ext.run_gemm_plan(*p3, 1.0, a, split, self._status)
            cur ^= 1
        out = []
        for it in self._items:
            M, N = it["M"], it["N"]
            X = it["X"][:, :N] if split else it["Xs"][cur][0][:, :N]
            out.append((X.T if it["wide"] else X).clone())
        return out

    def check_status(self) -> None:
        if int(self._status.item()) & 1:
            raise RuntimeError("grouped GEMM pipeline wait timed out (device-side bounded wait expired)")


# --------------------------------------------------------------------------------------------------
# Eigenbasis refresh of the eigenvalue-corrected variant: all factors of a group concurrently
# --------------------------------------------------------------------------------------------------
def eigenbasis_refresh_supported(cfg: Any) -> bool:
    from optimizers_b200.config import QREigendecompositionConfig

    if isinstance(cfg, QREigendecompositionConfig):
        return True
    return isinstance(cfg, EighEigendecompositionConfig) and cfg.eigendecomposition_offload_device == ""


def native_qr_iteration(
    ext: Any, mats: list[Tensor], estimates: list[Tensor], max_iterations: int, tolerance: float, status: Tensor
) -> list[Tensor]:
    """The reference's warm-started QR iteration (``matrix_functions.py:799-852``) for all factors
    of a refresh at once, on this framework's kernels only.

    With V the previous eigenvectors of A:  B = V^T A V;  while the off-diagonal criterion
    ``||B - diag B||_F <= tolerance ||B||_F`` fails (and iterations remain):  Q R = B,  B <- Q^T B Q
    (= R Q),  V <- V Q;  finally the columns are ordered by ascending diag(B).  The products are
    grouped tensor-core launches over all factors (symmetric ones compute the upper tiles only), the
    QR factorisations one call of the batched Householder driver (panel kernel + block-reflector
    kernel), the criterion one reduction launch whose results the host reads once per iteration for
    all factors together.  Returns the new eigenvector matrices (columns)."""
    from optimizers_b200.matrix.eigh_dc import _Mat

    device = mats[0].device
    F = ext
    n_all = [m.shape[0] for m in mats]

    def pair_of(x: Tensor) -> _Mat:
        n0, n1 = x.shape
        m = _Mat(n0, n1, device)
        m.plain.copy_(x)
        ext.tf32_split(m.plain, m.hi, m.lo)
        return m

    A = [pair_of(a) for a in mats]
    V = [pair_of(v) for v in estimates]  # columns are eigenvectors; K-major operand over the eigenvector index
    Vt = [_Mat(n, n, device, plain=False) for n in n_all]
    table = ext.build_transpose_table([(v.hi, vt.hi, None, None) for v, vt in zip(V, Vt)] + [(v.lo, vt.lo, None, None) for v, vt in zip(V, Vt)])
    ext.transpose_split(*table)

    def run(specs: list[tuple], alpha: float = 1.0, beta: float = 0.0) -> None:
        if specs:
            ext.run_gemm_plan(*ext.build_gemm_plan(specs), alpha, beta, True, status)

    def product(a: _Mat, b: _Mat, out: _Mat, sym: bool = False, plain: bool = True) -> tuple:
        """out = a b^T as plain array and (hi, lo) pair."""
        flags = F.FLAG_SPLIT_OUT | (F.FLAG_MIRROR if sym else 0) | (0 if plain else F.FLAG_NO_C)
        c = out.plain if plain else None
        return (a.hi, a.lo, b.hi, b.lo, c, out.hi, out.lo, None, out.hi.stride(0), out.hi.stride(0), flags, sym)

    def congruence(Wt: list[_Mat], M: list[_Mat], idx: list[int]) -> list[_Mat]:
        """W^T M W for symmetric M, W given by its transpose (rows = columns of W)."""
        T = {i: _Mat(n_all[i], n_all[i], device, plain=False) for i in idx}
        out = {i: _Mat(n_all[i], n_all[i], device) for i in idx}
        run([product(Wt[i], M[i], T[i], plain=False) for i in idx])
        run([product(T[i], Wt[i], out[i], sym=True) for i in idx])
        return out

    everyone = list(range(len(mats)))
    B = congruence(Vt, A, everyone)
    active = everyone
    for _ in range(max_iterations):
        if not active:
            break
        stats = torch.zeros(len(active), 2, device=device)
        ops = ext.build_sym_table([(B[i].plain, None, None, stats[k], 0.0, 0.0) for k, i in enumerate(active)])
        ext.sq_offdiag(ops[0], len(active))
        still = []
        for i, (total2, diag2) in zip(active, stats.cpu().tolist(), strict=True):  # the host read of this iteration
            off = max(total2 - diag2, 0.0) ** 0.5
            if not off <= tolerance * total2**0.5:  # also true for NaN: let the QR run, the caller's finiteness check reports it
                still.append(i)
        active = still
        if not active:
            break
        # Q R = B on the batched Householder driver; B is symmetric, so it is its own transposed storage.
        Zt = {i: _Mat(n_all[i], n_all[i], device) for i in active}
        work = {i: B[i].plain.clone() for i in active}
        ext.householder_qr([(work[i], n_all[i], n_all[i], Zt[i].plain, Zt[i].hi, Zt[i].lo) for i in active])
        newB = congruence(Zt, B, active)
        newV = {i: _Mat(n_all[i], n_all[i], device) for i in active}
        newVt = {i: _Mat(n_all[i], n_all[i], device, plain=False) for i in active}
        run([product(V[i], Zt[i], newV[i]) for i in active] + [product(Zt[i], V[i], newVt[i], plain=False) for i in active])
        for i in active:
            B[i], V[i], Vt[i] = newB[i], newV[i], newVt[i]
    out = []
    for i in everyone:
        _, order = torch.diagonal(B[i].plain).sort(stable=True)
        out.append(V[i].plain.index_select(1, order))
    return out


def batched_eigenbasis_refresh(blocks: list[Any], bias_correction2: Tensor | float, ext: Any = None) -> None:
    """Recompute ``factor_matrices_eigenvectors`` of every block (eigh, or the warm-started QR
    iteration of ``matrix_functions.py:799-852``) with the factors spread over a pool of streams,
    each driven by its own host thread, so that the library factorisations and the convergence
    reads of different factors overlap; the main thread reads the device twice in total
    (finiteness of the inputs, finiteness of the results) instead of three times per factor.
    The mathematics per factor is that of ``matrix_eigendecomposition``."""
    if not blocks:
        return
    device = blocks[0].factors.factor_matrices[0].device
    main = torch.cuda.current_stream(device)
    items: list[_Item] = [_Item(b, k, A, 0.0) for b, k, A in _prepared_factors(ext, blocks, bias_correction2)]
    finite = _all_finite([it.A for it in items])
    for it, ok in zip(items, finite):
        if not ok:
            index = it.block.factors.factor_matrix_indices[it.k]
            raise PreconditionerValueError(
                f"Encountered nan/inf values in factor matrix {index}! "
                "To mitigate, check if nan inputs are being passed into the network or nan gradients are being passed to the optimizer. "
                "Otherwise, in some cases, this may be due to divergence of the algorithm. To mitigate, try decreasing the learning rate or increasing grafting epsilon."
            )
    ready = torch.cuda.Event()
    ready.record(main)
    lazy_pool: list = []  # the stream pool is only set up when a factor falls back to the library

    def pool():
        if not lazy_pool:
            lazy_pool.extend(_pool(device))
        return lazy_pool

    def work(it: _Item, slot: int) -> None:
        kf = it.block.factors
        stream = pool()[1][slot]
        with torch.cuda.device(device), torch.cuda.stream(stream):
            stream.wait_event(ready)
            old_q = kf.factor_matrices_eigenvectors[it.k]
            try:
                _, Q = mf.matrix_eigendecomposition(
                    A=it.A,
                    eigendecomposition_config=kf.amortized_computation_config,
                    eigenvectors_estimate=old_q.to(dtype=it.A.dtype),
                    epsilon=kf.epsilon,
                )
                it.q_hi = Q.to(dtype=old_q.dtype)
            except Exception as exception:  # keep the previous eigenbasis of this factor
                it.error = exception
            it.done = torch.cuda.Event()
            it.done.record(stream)

    pooled = list(range(len(items)))
    cfg0 = blocks[0].factors.amortized_computation_config
    from optimizers_b200.config import QREigendecompositionConfig

    if ext is not None and isinstance(cfg0, QREigendecompositionConfig) and _DC_ENABLED:
        native = [
            i for i in pooled
            if items[i].A.dtype == torch.float32 and items[i].A.shape[0] >= 2
            and items[i].block.factors.factor_matrices_eigenvectors[items[i].k].dtype == torch.float32
        ]
        if native:
            stability = cfg0.rank_deficient_stability_config
            ridged = [
                mf._ridge(items[i].A, items[i].block.factors.epsilon * getattr(stability, "perturb_before_computation", 0))
                for i in native
            ]
            old = [items[i].block.factors.factor_matrices_eigenvectors[items[i].k] for i in native]
            status = torch.zeros(1, dtype=torch.int32, device=device)
            results = native_qr_iteration(ext, ridged, old, cfg0.max_iterations, cfg0.tolerance, status)
            for i, Q in zip(native, results, strict=True):
                items[i].q_hi = Q
                items[i].done = torch.cuda.Event()
                items[i].done.record(main)
            if int(status.item()) & 1:
                raise RuntimeError("grouped GEMM pipeline wait timed out (device-side bounded wait expired)")
            done = set(native)
            pooled = [i for i in pooled if i not in done]
            ready.record(main)
    if ext is not None and isinstance(cfg0, EighEigendecompositionConfig) and cfg0.tolerance == 0.0:
        # Small factors: one launch of the shared-memory Jacobi eigensolver for all of them.
        small = [i for i in pooled if items[i].A.shape[0] <= ext.JACOBI_MAX_N]
        if small:
            stability = cfg0.rank_deficient_stability_config
            ridged = [
                mf._ridge(items[i].A, items[i].block.factors.epsilon * getattr(stability, "perturb_before_computation", 0)).contiguous()
                for i in small
            ]
            _, qs, sweeps = ext.jacobi_eigh(ridged, _JACOBI_MAX_SWEEPS, _JACOBI_TOLERANCE)
            done_here = set()
            for i, Q, n_sweeps in zip(small, qs, sweeps.cpu().tolist(), strict=True):
                if n_sweeps > _JACOBI_MAX_SWEEPS:
                    continue
                it = items[i]
                it.q_hi = Q.to(dtype=it.block.factors.factor_matrices_eigenvectors[it.k].dtype)
                it.done = torch.cuda.Event()
                it.done.record(main)
                done_here.add(i)
            pooled = [i for i in pooled if i not in done_here]
            ready.record(main)
        large = [i for i in pooled if items[i].A.shape[0] > ext.JACOBI_MAX_N and items[i].A.dtype == torch.float32]
        if large:
            stability = cfg0.rank_deficient_stability_config
            ridged = [
                mf._ridge(items[i].A, items[i].block.factors.epsilon * getattr(stability, "perturb_before_computation", 0))
                for i in large
            ]
            status = torch.zeros(1, dtype=torch.int32, device=device)
            solved = native_eigh(ext, ridged, status, _hints_of(items, large))
            _remember_eigenvalues(items, large, solved)
            done_here = set()
            for i, pair in zip(large, solved, strict=True):
                if pair is None:
                    continue
                it = items[i]
                it.q_hi = pair[1].to(dtype=it.block.factors.factor_matrices_eigenvectors[it.k].dtype)
                it.done = torch.cuda.Event()
                it.done.record(main)
                done_here.add(i)
            pooled = [i for i in pooled if i not in done_here]
            ready.record(main)
            if int(status.item()) & 1:
                raise RuntimeError("grouped GEMM pipeline wait timed out (device-side bounded wait expired)")
    order = sorted(pooled, key=lambda i: -items[i].A.shape[0])
    futures = [pool()[0].submit(work, items[i], n % _POOL_SIZE) for n, i in enumerate(order)]
    for f in futures:
        f.result()
    for it in items:
        assert it.done is not None
        main.wait_event(it.done)
    good = [it for it in items if it.error is None]
    if good:
        ok_list = _all_finite([it.q_hi for it in good])
        for it, ok in zip(good, ok_list):
            if not ok:
                index = it.block.factors.factor_matrix_indices[it.k]
                raise PreconditionerValueError(
                    f"Encountered nan or inf values in eigenvectors of factor matrix {index}! "
                    "To mitigate, check factor matrix before the matrix computation."
                )
            it.block.factors.factor_matrices_eigenvectors[it.k].copy_(it.q_hi)
    main.synchronize()  # scratch allocated on the pool streams may now be reused
    last_error: dict[int, Exception | None] = {}
    for it in items:
        if it.error is not None:
            index = it.block.factors.factor_matrix_indices[it.k]
            logger.warning(
                f"Matrix computation failed for factor matrix {index} with exception={it.error!r}. Using previous preconditioner and continuing..."
            )
            last_error[id(it.block)] = it.error
        else:
            last_error.setdefault(id(it.block), None)
    for b in blocks:
        b.factors.note_refresh_outcome(last_error.get(id(b)))
