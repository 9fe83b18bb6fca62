"""Batched refresh of inverse roots for the native engine.

The torch refresh walks blocks and factors one at a time and synchronises with the host twice
per factor.  Here all factors of a refresh are processed together:

1. one pass prepares the bias-corrected (optionally trace-scaled) factor matrices and a single
   device->host read checks all of them for NaN/Inf;
2. the symmetric eigendecompositions run concurrently on a pool of CUDA streams, one Python
   thread per stream (``torch.linalg.eigh`` blocks its calling thread on an error code, so
   threads, not just streams, are needed for overlap); the eigenvalue stabilisation and the
   scaling ``Q·diag(λ^(-1/p))`` run on the same stream without host synchronisation;
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
from fractions import Fraction
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import EigenConfig, EighEigendecompositionConfig, PreconditionerValueError
from optimizers_b200.matrix import functions as mf

logger: logging.Logger = logging.getLogger(__name__)

_POOL_SIZE = 8
_pools: dict[int, tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]] = {}
_tls = threading.local()


def _pool(device: torch.device) -> tuple[ThreadPoolExecutor, list[torch.cuda.Stream]]:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _pools:
        streams = [torch.cuda.Stream(device=device) for _ in range(_POOL_SIZE)]
        _pools[key] = (ThreadPoolExecutor(max_workers=_POOL_SIZE, thread_name_prefix="ob200-eigh"), streams)
    return _pools[key]


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


class _Item:
    __slots__ = ("block", "k", "A", "root", "qs_hi", "qs_lo", "q_hi", "q_lo", "error", "done")

    def __init__(self, block: Any, k: int, A: Tensor, root: float) -> None:
        self.block, self.k, self.A, self.root = block, k, A, root
        self.error: Exception | None = None
        self.done: torch.cuda.Event | None = None


def eigen_refresh_supported(cfg: Any) -> bool:
    return isinstance(cfg, EigenConfig) and cfg.eigendecomposition_offload_device == ""


def batched_eigen_refresh(ext: Any, blocks: list[Any], bias_correction2: Tensor | float, split: bool, status: Tensor) -> None:
    """Refresh ``inv_factor_matrices`` (state) and the ``inv_hi/inv_lo`` mirrors of ``blocks``.

    ``blocks`` are the native engine's block records (``.factors`` is the ``BlockFactors`` of the
    block, ``.inv_hi/.inv_lo`` the mirrors).  Raises ``PreconditionerValueError`` on non-finite
    factors or results and ``ValueError`` once a block exceeds its tolerated failures."""
    if not blocks:
        return
    device = blocks[0].inv_hi[0].device
    main = torch.cuda.current_stream(device)

    # 1. prepare + one finiteness read
    items: list[_Item] = []
    for b in blocks:
        kf = b.factors
        for k, factor in enumerate(kf.factor_matrices):
            A = kf.unpack(factor / bias_correction2)
            if kf.use_trace_scaling:
                A = A * torch.pow(torch.clamp(torch.trace(A), min=kf.epsilon), -kf.trace_scaling_exponent)
            items.append(_Item(b, k, A, kf.roots[k]))
    finite = torch.stack([torch.isfinite(it.A).all() for it in items]).cpu()
    for it, ok in zip(items, finite.tolist()):
        if not ok:
            index = it.block.factors.factor_matrix_indices[it.k]
            raise PreconditionerValueError(
                f"Encountered nan/inf values in factor matrix {index}! "
                "To mitigate, check if nan inputs are being passed into the network or nan gradients are being passed to the optimizer. "
                "Otherwise, in some cases, this may be due to divergence of the algorithm. To mitigate, try decreasing the learning rate or increasing grafting epsilon."
            )

    # 2. eigendecompositions on the stream pool (largest first for balance)
    ready = torch.cuda.Event()
    ready.record(main)
    executor, streams = _pool(device)

    def work(it: _Item, slot: int) -> None:
        kf = it.block.factors
        cfg: EigenConfig = kf.amortized_computation_config
        stream = streams[slot]
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
                scale = mf.stabilized_inverse_power(
                    lam, Fraction(it.root), kf.epsilon, cfg.rank_deficient_stability_config
                )
                Q = Q.contiguous()
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
            except Exception as exception:  # keep the previous inverse root of this factor
                it.error = exception
            it.done = torch.cuda.Event()
            it.done.record(stream)

    order = sorted(range(len(items)), key=lambda i: -items[i].A.shape[0])
    futures = [executor.submit(work, items[i], n % _POOL_SIZE) for n, i in enumerate(order)]
    for f in futures:
        f.result()
    for it in items:
        assert it.done is not None
        main.wait_event(it.done)

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

    # 4. checkpoint state (packed upper triangle) from the result + one finiteness read; the
    #    operand mirrors are then rebuilt from the state so that both always agree exactly
    flags = []
    for it in good:
        d = it.A.shape[0]
        kf = it.block.factors
        state = kf.inv_factor_matrices[it.k]
        state.copy_(kf.pack(it.block.inv_hi[it.k][:, :d]).to(dtype=state.dtype))
        flags.append(torch.isfinite(state).all())
    if flags:
        ok_list = torch.stack(flags).cpu().tolist()
        for it, ok in zip(good, ok_list):
            if not ok:
                index = it.block.factors.factor_matrix_indices[it.k]
                raise PreconditionerValueError(
                    f"Encountered nan or inf values in matrices of factor matrix {index}! "
                    "To mitigate, check factor matrix before the matrix computation."
                )
    main.synchronize()  # scratch allocated on the pool streams may now be reused

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
