"""Native sm_100a execution of one parameter group's optimizer step.

The torch step walks Python lists of per-block tensors and launches several kernels per block.
The native engine instead keeps a *device block table* for the group and runs the whole step as
a fixed, short sequence of grouped launches:

    grad_prologue        one pass over the gradients (L2, tf32 operand splits in both
                         orientations, filtered-gradient EMA, grafting second moment and norm)
    grouped SYRK         every factor of every block:  F <- beta2 F + w X X^T, written straight
                         into the (packed) factor state by the tensor-core kernel's epilogue
    [refresh]            at amortised steps: inverse roots, then their operand mirrors
    grouped GEMM x2      T^T = R^(-1/p) G^T and P = L^(-1/p) T with the Frobenius norm of P
                         accumulated in the epilogue
    direction_epilogue   grafting rescale, weight decay, momentum, -lr, primal averaging, update

The checkpointed state tensors are exactly those the preconditioner lists allocated; the engine
adds scratch operands and full (unpacked, split) mirrors of the inverse roots, which are rebuilt
from the state after every refresh and after ``load_state_dict``.

The eigenvalue-corrected variant (SOAP) replaces the two apply GEMMs by project -> scale ->
unproject (``_soap_step``) and updates its second moment in the epilogue of the projection GEMM.

Coverage: fp32 parameters on CUDA, blocks of order 1 or 2 (and contiguous order-3 blocks for
root-inverse Shampoo) with every dim preconditioned,
root-inverse, eigendecomposed, KL or eigenvalue-corrected Shampoo with no / SGD / AdaGrad / RMSprop / Adam grafting,
any weight decay type,
classic momentum, GPA / Schedule-Free, every distributor; the DDP family (DDP, and the replicate
groups of HSDP and hybrid shard) gathers the search directions with NCCL or, with
``comm_path="p2p"``, by stores into the peers' buffers over NVLink.  Anything else makes
``build_native_engine`` return ``None`` (torch step) or raise with ``backend="native"``.
"""

from __future__ import annotations

import logging
from typing import Any

import torch
from torch import Tensor

from optimizers_b200.config import (
    AdaGradPreconditionerConfig,
    DDPDistributedConfig,
    DISTRIBUTED_CONFIG,
    DISTRIBUTOR,
    EigendecomposedKLShampooPreconditionerConfig,
    EigendecomposedShampooPreconditionerConfig,
    EigenvalueCorrectedShampooPreconditionerConfig,
    FILTERED_GRAD_LIST,
    GRAFTING_CONFIG,
    GRAFTING_PRECONDITIONER_LIST,
    LR_CPU_PINNED,
    MASKED_BLOCKED_GRADS,
    MOMENTUM_BUFFER_LIST,
    NativeRuntimeConfig,
    PARAMS,
    PRECONDITIONER_CONFIG,
    PreconditionerValueError,
    RootInvKLShampooPreconditionerConfig,
    RootInvShampooPreconditionerConfig,
    SGDPreconditionerConfig,
    SHAMPOO_PRECONDITIONER_LIST,
    TRAIN_MODE,
    WEIGHT_BUFFER_LIST,
    WeightDecayType,
)
from optimizers_b200.utils import tracing
from optimizers_b200.utils.blocking import compress_list

logger: logging.Logger = logging.getLogger(__name__)

_GRAFT_NONE, _GRAFT_SGD, _GRAFT_ADAGRAD = 0, 1, 2


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


# Configurations whose 2-D blocks may carry a factor on one dim only (the other switched off by an
# exponent of 0): one-sided products.  Under KL-Shampoo such a block has no other dim to precondition
# its Gram along, so its statistics are the plain ones.
_ONE_SIDED_CONFIGS = (
    RootInvShampooPreconditionerConfig, EigendecomposedShampooPreconditionerConfig,
    RootInvKLShampooPreconditionerConfig, EigendecomposedKLShampooPreconditionerConfig,
)


def _why_not_covered(rec: dict[str, Any], group: dict[str, Any]) -> str | None:
    pc = group[PRECONDITIONER_CONFIG]
    if type(pc) in (RootInvShampooPreconditionerConfig, RootInvKLShampooPreconditionerConfig):
        if pc.factor_matrix_dtype != torch.float32 or pc.inv_factor_matrix_dtype != torch.float32:
            return "factor matrices must be fp32"
    elif type(pc) in (EigendecomposedShampooPreconditionerConfig, EigendecomposedKLShampooPreconditionerConfig):
        dtypes = (pc.factor_matrix_dtype, pc.factor_matrix_eigenvectors_dtype, pc.factor_matrix_eigenvalues_dtype)
        if any(d != torch.float32 for d in dtypes):
            return "factor matrices, eigenvectors and eigenvalues must be fp32"
    elif type(pc) is EigenvalueCorrectedShampooPreconditionerConfig:
        dtypes = (pc.factor_matrix_dtype, pc.factor_matrix_eigenvectors_dtype, pc.corrected_eigenvalues_dtype)
        if any(d != torch.float32 for d in dtypes):
            return "factor matrices, eigenvectors and corrected eigenvalues must be fp32"
    else:
        return f"preconditioner config {type(pc).__name__} has no native step yet"
    gc = group[GRAFTING_CONFIG]
    if gc is not None and not isinstance(gc, (SGDPreconditionerConfig, AdaGradPreconditionerConfig)):
        return f"grafting config {type(gc).__name__} has no native step"
    dc = group[DISTRIBUTED_CONFIG]
    if isinstance(dc, DDPDistributedConfig):
        if dc.communication_dtype not in (torch.float32, torch.bfloat16, torch.float16):
            return f"communication dtype {dc.communication_dtype} has no native step"
    # What the distributor blocks: the parameters themselves, their local shards, or (lossless
    # variants) this rank's gathered full copies.
    for p in rec[DISTRIBUTOR]._get_params_or_grads():
        if p.dtype != torch.float32 or not p.is_contiguous() or type(p.detach()) is not Tensor:
            return "parameters (or their local shards) must be plain contiguous fp32 tensors"
    # Dims switched off by an exponent of 0: decided from the configuration and the global block list,
    # so that every rank of a group reaches the same verdict.
    overrides = getattr(pc, "inverse_exponent_override", {}).values()
    if any(0.0 in (o.values() if isinstance(o, dict) else (o,)) for o in overrides):
        if type(pc) not in _ONE_SIDED_CONFIGS:
            return "dims switched off by an exponent of 0 have no native step under eigenvalue-corrected Shampoo"
        if any(b.dim() > 2 for b in rec[DISTRIBUTOR]._global_blocked_params):
            return "dims switched off by an exponent of 0 have no native step next to blocks of order 3"
    plist = rec[SHAMPOO_PRECONDITIONER_LIST]
    for block, sel in zip(
        rec[DISTRIBUTOR].local_blocked_params, plist._local_preconditioned_dims_selector_list, strict=True
    ):
        if block.dim() > 3 or (block.dim() == 3 and not _order3_ok(block, pc)):
            return f"block of order {block.dim()} and shape {tuple(block.shape)} has no native step yet"
        if not all(sel) and (block.dim() > 2 or type(pc) not in _ONE_SIDED_CONFIGS):
            return "blocks with unpreconditioned dims have a native step only for 1-D / 2-D blocks of root-inverse, eigendecomposed and KL Shampoo"
        if block.numel() == 0:
            return "empty blocks"
    # The same verdict on every rank: ranks that disagreed would meet in different collectives.
    if any(b.dim() > 3 or b.numel() == 0 or (b.dim() == 3 and not _order3_ok(b, pc)) for b in rec[DISTRIBUTOR]._global_blocked_params):
        return "a block of another rank has no native step"
    return None


def _order3_ok(block: Tensor, pc: Any) -> bool:
    """Order-3 blocks (a, b, c) run natively for root-inverse, eigendecomposed and eigenvalue-corrected
    Shampoo when they are contiguous and a, b are multiples of 4, so that every mode unfolding is an
    exact, 16-byte aligned 2-D view."""
    a, b, _ = block.shape
    covered = type(pc) in (  # not KL
        RootInvShampooPreconditionerConfig, EigendecomposedShampooPreconditionerConfig, EigenvalueCorrectedShampooPreconditionerConfig
    )
    return covered and block.is_contiguous() and a % 4 == 0 and b % 4 == 0


_FALLBACK_REASON = "native_engine_fallback_reason"  # key of the per-group record: why the group runs the torch step


def maybe_build_native_engine(optimizer: Any, rec: dict[str, Any], group: dict[str, Any], cfg: NativeRuntimeConfig):
    """Return a native engine for the group, or ``None`` to use the torch step.

    ``backend="torch"`` and non-CUDA groups always get ``None``.  ``backend="native"`` raises when
    the group cannot be covered; ``"auto"`` falls back silently."""
    if cfg.backend == "torch" or group[PARAMS][0].device.type != "cuda":
        if cfg.backend == "native":
            raise RuntimeError("native backend requested for a parameter group that is not on a CUDA device")
        rec[_FALLBACK_REASON] = 'backend="torch" was requested' if cfg.backend == "torch" else "the parameters are not on a CUDA device"
        return None
    return build_native_engine(optimizer, rec, group, cfg)


def build_native_engine(optimizer: Any, rec: dict[str, Any], group: dict[str, Any], cfg: NativeRuntimeConfig):
    reason = _why_not_covered(rec, group)
    if reason is None and torch.cuda.get_device_capability(group[PARAMS][0].device)[0] != 10:
        reason = "device is not sm_100"
    if reason is not None:
        if cfg.backend == "native":
            raise RuntimeError(f"native backend requested but {reason}")
        logger.info("Parameter group uses the torch step: %s.", reason)
        rec[_FALLBACK_REASON] = reason
        return None
    return NativeGroupEngine(optimizer, rec, group, cfg)


class _ZeroPool:
    """Zero-initialised fp32 scratch carved out of a few large allocations: the operand arrays of a
    group are hundreds of tensors, and one fill launch per tensor made engine construction the
    bulk of a short run's kernel launches.  Every array starts on a 256-byte boundary."""

    CHUNK_ELEMS = 64 * 1024 * 1024  # 256 MB

    def __init__(self, device: torch.device) -> None:
        self._device = device
        self._chunk: Tensor | None = None
        self._cursor = 0

    def zeros(self, *shape: int) -> Tensor:
        numel = 1
        for n in shape:
            numel *= n
        padded = (numel + 63) // 64 * 64
        if padded > self.CHUNK_ELEMS // 4:  # large arrays get their own allocation
            return torch.zeros(*shape, dtype=torch.float32, device=self._device)
        if self._chunk is None or self._cursor + padded > self._chunk.numel():
            self._chunk = torch.zeros(self.CHUNK_ELEMS, dtype=torch.float32, device=self._device)
            self._cursor = 0
        out = self._chunk[self._cursor : self._cursor + numel].view(*shape)
        self._cursor += padded
        return out


class _Block:
    """Host-side record of one local block: views, state, scratch operands."""

    __slots__ = (
        "index", "param_view", "grad_slot", "grad_offset", "m", "n", "n_pad", "m_pad", "order", "factors",
        "m1", "v", "mom", "z", "g_hi", "g_lo", "gt_hi", "gt_lo", "f_hi", "f_lo", "tt_hi", "tt_lo", "p",
        "inv_hi", "inv_lo", "ev", "qt_hi", "qt_lo", "t2_hi", "t2_lo",
        "dims3", "view2d", "y_hi", "y_lo", "zt_hi", "zt_lo", "aux_g_hi", "aux_g_lo", "aux_gt_hi", "aux_gt_lo", "d1_hi", "d1_lo", "d2_hi", "d2_lo",
        "e1_hi", "e1_lo", "e2_hi", "e2_lo",  # second set of chain intermediates (eigenvalue-corrected order-3: two chains per stage)
        "sel",  # per dim of the block: has a Kronecker factor (inverse_exponent_override 0 switches a dim off)
        "eig_hints",  # factor index -> eigenvalues found at the previous refresh (host tensor; steers the eigensolver)
    )


class NativeGroupEngine:
    def __init__(self, optimizer: Any, rec: dict[str, Any], group: dict[str, Any], cfg: NativeRuntimeConfig) -> None:
        from optimizers_b200.ops import build

        self._ext = build.load()
        self._optimizer = optimizer
        self._rec = rec
        self._group = group
        self._cfg = cfg
        self._split = cfg.gemm_mode == "tf32x3"
        self._dist = rec[DISTRIBUTOR]
        self._device = group[PARAMS][0].device
        self._plist = rec[SHAMPOO_PRECONDITIONER_LIST]
        self._glist = rec[GRAFTING_PRECONDITIONER_LIST]
        self._packing = group[PRECONDITIONER_CONFIG].use_symmetric_packing
        self._soap = type(group[PRECONDITIONER_CONFIG]) is EigenvalueCorrectedShampooPreconditionerConfig
        # Eigendecomposed Shampoo checkpoints (eigenvalues, eigenvectors); its inverse roots
        # Q f(lambda) Q^T only change at a refresh, so the step is the root-inverse step on mirrors
        # rebuilt then (the torch formulation rebuilds them from the eigendecomposition every step).
        self._eigdec = type(group[PRECONDITIONER_CONFIG]) in (
            EigendecomposedShampooPreconditionerConfig, EigendecomposedKLShampooPreconditionerConfig
        )
        # KL-Shampoo: the Gram of a dim is taken of the gradient preconditioned along the other dim,
        # two extra GEMMs per 2-D block in front of the factor SYRK.
        self._kl = type(group[PRECONDITIONER_CONFIG]) in (
            RootInvKLShampooPreconditionerConfig, EigendecomposedKLShampooPreconditionerConfig
        )
        self.launches_per_step = 0
        # Diagnostics: assign a list to ``phase_events`` and every step appends (name, CUDA event)
        # pairs at the boundaries of its phases (benchmarks/engine_microbench.py --phases).
        self.phase_events: list[tuple[str, torch.cuda.Event]] | None = None

        gc = group[GRAFTING_CONFIG]
        if gc is None:
            self._graft_kind = _GRAFT_NONE
        elif isinstance(gc, SGDPreconditionerConfig):
            self._graft_kind = _GRAFT_SGD
        else:
            self._graft_kind = _GRAFT_ADAGRAD

        self._status = torch.zeros(1, dtype=torch.int32, device=self._device)
        # Host mirror of the status word: every step ends with an asynchronous copy into pinned
        # memory and begins by looking at the copy of the step before (no synchronisation), so a
        # device-side timeout or a non-finite gradient surfaces one step late at the latest.
        self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_event: torch.cuda.Event | None = None
        self._ddp = isinstance(group[DISTRIBUTED_CONFIG], DDPDistributedConfig)
        # Every distributor of the DDP family (DDP itself, and the replicate groups of the HSDP and
        # hybrid-shard distributors) can deliver its search directions by peer stores instead of an
        # all-gather.  The fused gradient reduction only exists where the optimizer sees replicated,
        # unreduced gradients: plain DDP (the sharded wrappers reduce-scatter their own).
        self._p2p = self._ddp and cfg.comm_path == "p2p"
        self._pull = self._p2p and cfg.fuse_gradient_reduction and type(group[DISTRIBUTED_CONFIG]) is DDPDistributedConfig
        self._comm_params = bool(getattr(group[DISTRIBUTED_CONFIG], "communicate_params", False)) and self._ddp
        # Every rank must take the same decision, so the rule looks at the configuration only: a dim
        # switched off by an exponent of 0 leaves blocks without a final product to push from.
        overrides = getattr(group[PRECONDITIONER_CONFIG], "inverse_exponent_override", {}).values()
        some_dim_off = any(
            0.0 in (o.values() if isinstance(o, dict) else (o,)) for o in overrides
        )
        self._gemm_push = (
            self._p2p and cfg.fuse_direction_push and not self._soap and not self._comm_params and not some_dim_off
        )
        self.gemm_push_steps = 0  # steps whose all-gather ran from the GEMM epilogue
        self._comm_dtype_code = 0
        self._gather_table = None
        self._gather_for: tuple[bool, ...] | None = None
        self._barrier_seq = 0
        if self._ddp:
            cd = group[DISTRIBUTED_CONFIG].communication_dtype
            self._comm_dtype_code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[cd]
            sel = self._dist._distributor_selector
            self._local_slot_offsets = compress_list(self._dist._global_block_byte_offsets, sel)
        if self._p2p:
            self._setup_peer_memory()
        self._build_blocks()
        n_ptrs = max(len(self._local_params), 1)
        # Pinned staging buffers for the gradient pointer table, used in turn; each carries the
        # event of its last upload, and the host waits for that event before rewriting the buffer,
        # so a copy still queued on the device never sees another step's pointers however far the
        # host runs ahead.
        self._grad_ptrs_host = [torch.zeros(n_ptrs, dtype=torch.int64).pin_memory() for _ in range(2)]
        self._grad_ptrs_uploaded: list[torch.cuda.Event | None] = [None, None]
        self._grad_ptrs_flip = 0
        if not self._pull:
            self._grad_ptrs_dev = torch.zeros(n_ptrs, dtype=torch.int64, device=self._device)
        self._last_ptrs: list[int] | None = None
        self._active: tuple[bool, ...] | None = None
        self._plans_for: tuple[bool, ...] | None = None
        self.refresh_inverse_mirrors()

    # ------------------------------------------------------------------------------------------
    # Set-up
    # ------------------------------------------------------------------------------------------
    def _build_blocks(self) -> None:
        rec, dist = self._rec, self._dist
        dev = self._device
        # Local tensors the blocks are views of, aligned with dist._global_num_blocks_per_param.
        self._local_params = [p.detach() for p in dist._get_params_or_grads()]
        owner_of_block = [
            i for i, count in enumerate(dist._global_num_blocks_per_param) for _ in range(count)
        ]
        local_owner = compress_list(owner_of_block, dist._distributor_selector)
        blocks: list[_Block] = []
        factors_list = self._plist._local_kronecker_factors_unwrapped
        m1s = rec.get(FILTERED_GRAD_LIST)
        moms = rec.get(MOMENTUM_BUFFER_LIST)
        zs = rec.get(WEIGHT_BUFFER_LIST)
        vs = self._glist._local_preconditioner_list if self._graft_kind == _GRAFT_ADAGRAD else None
        self._norms = torch.zeros(max(len(dist.local_blocked_params), 1), 2, dtype=torch.float32, device=dev)

        pool = _ZeroPool(dev)
        zeros = pool.zeros

        selectors = self._plist._local_preconditioned_dims_selector_list
        for i, (view, info) in enumerate(zip(dist.local_blocked_params, dist.local_block_info_list, strict=True)):
            b = _Block()
            b.sel = tuple(selectors[i])
            b.eig_hints = None
            b.index = i
            b.param_view = view
            b.grad_slot = local_owner[i]
            b.grad_offset = (view.data_ptr() - self._local_params[b.grad_slot].data_ptr()) // 4
            b.order = view.dim()
            b.dims3 = None
            b.view2d = view
            if view.dim() == 1:
                b.m, b.n = 1, view.shape[0]
            elif view.dim() == 3:
                # (a, b, c) is presented to the pointwise kernels as (a*b) x c.
                b.dims3 = tuple(view.shape)
                b.m, b.n = view.shape[0] * view.shape[1], view.shape[2]
                b.view2d = view.view(b.m, b.n)
            else:
                b.m, b.n = view.shape
            b.n_pad, b.m_pad = _pad4(b.n), _pad4(b.m)
            b.factors = factors_list[i]
            b.m1 = m1s[i] if m1s is not None else None
            b.v = vs[i] if vs is not None else None
            b.mom = moms[i] if moms is not None else None
            b.z = zs[i] if zs is not None else None
            two_d = b.order == 2
            left = two_d and b.sel[0]  # a factor on the rows
            right = b.sel[-1]  # a factor on the columns (the only dim of a 1-D block)
            need_g = left or self._soap
            if b.dims3 is not None:
                self._alloc_order3(b, zeros)
                blocks.append(b)
                continue
            b.aux_g_hi = b.aux_g_lo = b.aux_gt_hi = b.aux_gt_lo = b.d1_hi = b.d1_lo = b.d2_hi = b.d2_lo = None
            b.e1_hi = b.e1_lo = b.e2_hi = b.e2_lo = None
            b.g_hi = zeros(b.m, b.n_pad) if need_g else None
            b.g_lo = zeros(b.m, b.n_pad) if need_g and self._split else None
            need_gt = right or self._soap
            b.gt_hi = zeros(b.n, b.m_pad) if need_gt else None
            b.gt_lo = zeros(b.n, b.m_pad) if need_gt and self._split else None
            b.f_hi = zeros(b.m, b.n_pad)
            b.f_lo = zeros(b.m, b.n_pad) if self._split else None
            # The chain intermediate T^T [n, m_pad] takes over the memory of G^T, whose last reader
            # (the factor SYRK) has run before the first chain GEMM writes.
            b.y_hi = b.y_lo = b.zt_hi = b.zt_lo = None
            if self._kl and left and right:
                # Y = G R^(-1/p) [m, n] and Z^T = G^T L^(-1/p) [n, m]: operands of the KL factor Grams.
                b.y_hi, b.zt_hi = zeros(b.m, b.n_pad), zeros(b.n, b.m_pad)
                if self._split:
                    b.y_lo, b.zt_lo = zeros(b.m, b.n_pad), zeros(b.n, b.m_pad)
            if left and not right:  # (F I)^T = F^T has no G^T to reuse
                b.tt_hi = zeros(b.n, b.m_pad)
                b.tt_lo = zeros(b.n, b.m_pad) if self._split else None
            else:
                b.tt_hi = b.gt_hi if left else None
                b.tt_lo = b.gt_lo if left and self._split else None
            # Likewise the search direction P [m, n] reuses G (hi part) when the pitches agree.
            b.p = b.g_hi if (b.g_hi is not None and b.n_pad == b.n) else zeros(b.m, b.n)
            dims = tuple(d for d, on in zip((b.m, b.n) if two_d else (b.n,), b.sel, strict=True) if on)
            b.inv_hi = [zeros(d, _pad4(d)) for d in dims]
            b.inv_lo = [zeros(d, _pad4(d)) if self._split else None for d in dims]
            b.ev = b.qt_hi = b.qt_lo = b.t2_hi = b.t2_lo = None
            if self._soap:
                # inv_hi/inv_lo hold the eigenvector matrices Q_k, qt_* their transposes.
                b.ev = b.factors.corrected_eigenvalues
                b.qt_hi = [zeros(d, _pad4(d)) for d in dims]
                b.qt_lo = [zeros(d, _pad4(d)) if self._split else None for d in dims]
                b.t2_hi = zeros(b.n, b.m_pad) if two_d else None
                b.t2_lo = zeros(b.n, b.m_pad) if two_d and self._split else None
            blocks.append(b)
        self._blocks = blocks

    def _alloc_order3(self, b: _Block, zeros) -> None:
        """Operand buffers of an order-3 block (a, b, c).  Mode unfoldings, all K-major:
        X_a = [a, b*c] (``aux_g``), X_b = [b, c*a] (``aux_gt``, the transpose of X_a, re-viewed),
        X_c = [c, a*b] (``gt``, the transpose of the (a*b) x c view).  The preconditioner chain
        contracts the fastest index of the current layout and emits the new index slowest, so three
        GEMMs walk (a,b,c) -> (c,a,b) -> (b,c,a) -> (a,b,c) without any transposition pass."""
        a, bb, c = b.dims3
        sp = self._split
        b.y_hi = b.y_lo = b.zt_hi = b.zt_lo = None
        pair = lambda r, cols: (zeros(r, cols), zeros(r, cols) if sp else None)  # noqa: E731
        b.g_hi = b.g_lo = None
        b.gt_hi, b.gt_lo = pair(c, a * bb)
        b.f_hi, b.f_lo = pair(a * bb, _pad4(c))
        b.aux_g_hi, b.aux_g_lo = pair(a, bb * c)
        b.aux_gt_hi, b.aux_gt_lo = pair(bb * c, a)
        # Chain intermediates and the result reuse operand arrays whose last reader (the factor
        # SYRK) precedes the chain: (c, ab) <- X_c, (b, ca) <- X_b, P (a, bc) <- X_a (hi part).
        b.d1_hi, b.d1_lo = b.gt_hi, b.gt_lo
        b.d2_hi = b.aux_gt_hi.view(bb, c * a)
        b.d2_lo = b.aux_gt_lo.view(bb, c * a) if sp else None
        b.tt_hi = b.tt_lo = None
        b.p = b.aux_g_hi
        b.inv_hi = [zeros(d, _pad4(d)) for d in b.dims3]
        b.inv_lo = [zeros(d, _pad4(d)) if sp else None for d in b.dims3]
        b.ev = b.qt_hi = b.qt_lo = b.t2_hi = b.t2_lo = None
        b.e1_hi = b.e1_lo = b.e2_hi = b.e2_lo = None
        if self._soap:
            # The raw gradient is projected as well (second moment in the eigenbasis): it needs the
            # (ab, c) operand form of G, the transposed eigenvector mirrors, and chain intermediates
            # of its own, since it runs in the same launches as the chain of the filtered gradient.
            b.g_hi, b.g_lo = pair(a * bb, _pad4(c))
            b.ev = b.factors.corrected_eigenvalues
            b.qt_hi = [zeros(d, _pad4(d)) for d in b.dims3]
            b.qt_lo = [zeros(d, _pad4(d)) if sp else None for d in b.dims3]
            b.e1_hi, b.e1_lo = pair(c, a * bb)
            b.e2_hi, b.e2_lo = pair(bb, c * a)

    def _send_ptr(self, b: _Block) -> int:
        if not self._ddp or self._p2p:
            return 0
        return self._dist._local_dist_blocked_buffers[b.index].data_ptr()

    def _slot_offset(self, b: _Block) -> int:
        return int(self._local_slot_offsets[b.index]) if self._ddp else 0

    def _setup_peer_memory(self) -> None:
        """Allocate the peer-addressable arena: gather buffer (same layout as the distributor's),
        two flag arrays for the cross-rank barriers, and, when the gradient reduction is fused,
        one fp32 gradient arena that autograd accumulates into."""
        from optimizers_b200.parallel.symm_arena import SymmetricArena

        dist_ = self._dist
        world = dist_._group_size
        if world > 8:
            raise RuntimeError("comm_path='p2p' needs all ranks of a group on one NVLink domain (at most 8)")
        regions = {"gather": dist_._global_dist_buffer.numel(), "flags": 2 * 32 * 4,
                   "scales": 4 * max(len(dist_._global_blocked_params), 1)}
        params = self._group[PARAMS]
        if self._pull:
            if dist_._group_size != dist_._global_size:
                raise RuntimeError("fuse_gradient_reduction needs num_trainers_per_group == world size")
            regions["grads"] = sum(p.numel() for p in params) * 4
        self._arena = SymmetricArena(regions, self._device, dist_._dist_group)
        self._flags = self._arena.region("flags").view(torch.int32)
        self._flag_bases = [
            torch.tensor([a + k * 128 for a in self._arena.peer_addresses("flags")], dtype=torch.int64, device=self._device)
            for k in range(2)
        ]
        self._gather_local = self._arena.region("gather", dist_._global_dist_buffer.numel())
        self._gather_bases = self._arena.peer_addresses("gather")
        # Per-block grafting scales of the GEMM-epilogue push path, indexed by global block.
        self._scales_local = self._arena.region("scales").view(torch.float32)
        self._scale_bases = self._arena.peer_addresses("scales")
        self._scale_copy_for: tuple[bool, ...] | None = None
        if self._pull:
            flat = self._arena.region("grads", regions["grads"]).view(torch.float32)
            bases = self._arena.peer_addresses("grads")
            table, cursor = [], 0
            self._grad_views = []
            for p in params:
                view = flat[cursor : cursor + p.numel()].view(p.shape)
                p.grad = view
                self._grad_views.append(view)
                table.extend(b + cursor * 4 for b in bases)
                cursor += p.numel()
            self._grad_ptrs_dev = torch.tensor(table, dtype=torch.int64, device=self._device)

    def _mark(self, name: str) -> None:
        if tracing.nvtx_enabled():
            torch.cuda.nvtx.mark(f"ob200::phase::{name}")
        if self.phase_events is not None:
            event = torch.cuda.Event(enable_timing=True)
            event.record()
            self.phase_events.append((name, event))

    def _peer_barrier(self, which: int) -> None:
        self._barrier_seq += 1
        self._ext.peer_barrier(
            self._flags[which * 32 : which * 32 + 32], self._flag_bases[which], self._arena.rank, self._arena.world,
            self._barrier_seq, self._status,
        )

    def _build_plans(self, active: tuple[bool, ...]) -> None:
        """(Re)build the block table and the three GEMM plans for the active blocks."""
        ext = self._ext
        blocks = [b for b, on in zip(self._blocks, active, strict=True) if on]
        self._active_blocks = blocks
        if not blocks:
            self._table = None
            return
        F = ext
        specs = []
        for b in blocks:
            specs.append(
                (
                    b.view2d, b.grad_offset, b.grad_slot, b.m, b.n, b.n_pad, b.m_pad, b.m1, b.v, b.mom, b.z,
                    b.g_hi, b.g_lo, b.gt_hi, b.gt_lo, b.f_hi, b.f_lo, b.p, self._norms[b.index], self._send_ptr(b),
                    self._slot_offset(b), b.ev, 0 if (self._soap or any(b.sel)) else 2,
                )
            )
        for b in blocks:
            if b.dims3 is None:
                continue
            # Auxiliary a x (b*c) view: only the (hi, lo) operands of the mode-a and mode-b unfoldings.
            a, bb, c = b.dims3
            specs.append(
                (b.param_view.view(a, bb * c), b.grad_offset, b.grad_slot, a, bb * c, bb * c, a)
                + (None,) * 4 + (b.aux_g_hi, b.aux_g_lo, b.aux_gt_hi, b.aux_gt_lo) + (None,) * 4 + (0, 0, None, 1)
            )
        self._table = ext.build_block_table(specs)
        if self._soap:
            # The scaling between projection and unprojection takes one exponent per launch: blocks
            # whose tensor order carries its own exponent override get a table of their own.
            by_root: dict[float, list] = {}
            for b, spec in zip(blocks, specs):
                by_root.setdefault(float(b.factors.roots[0]), []).append(spec)
            if len(by_root) == 1:
                self._eig_tables = [(self._table, next(iter(by_root)))]
            else:
                self._eig_tables = [(ext.build_block_table(group), root) for root, group in by_root.items()]
            self._build_soap_plans(blocks)
            return

        def op(t: Tensor, rows: int, k: int) -> Tensor:
            return t[:, :k] if t.shape[1] != k else t

        syrk, gemm0, gemm1, gemm2, kl = [], [], [], [], []
        f_transposes = []  # (F hi|lo -> T^T hi|lo) of the blocks preconditioned on the rows only
        pack_flag = F.FLAG_PACKED_C if self._packing else 0
        sp = self._split

        def chained(a_hi, a_lo, b_hi, b_lo, out_hi, out_lo):
            """Product whose result is only the operand of the next product of the chain."""
            if sp:
                return (a_hi, a_lo, b_hi, b_lo, None, out_hi, out_lo, None, 0, out_hi.stride(0), F.FLAG_NO_C | F.FLAG_SPLIT_OUT, False)
            return (a_hi, None, b_hi, None, out_hi, None, None, None, out_hi.stride(0), 0, 0, False)

        for b in blocks:
            fm = b.factors.factor_matrices
            if b.dims3 is not None:
                a, bb, c = b.dims3
                lo = lambda t: t if sp else None  # noqa: E731
                xa = (b.aux_g_hi, lo(b.aux_g_lo))
                xb = (b.aux_gt_hi.view(bb, c * a), lo(b.aux_gt_lo.view(bb, c * a) if sp else None))
                xc = (b.gt_hi, lo(b.gt_lo))
                for (x_hi, x_lo), factor, d in ((xa, fm[0], a), (xb, fm[1], bb), (xc, fm[2], c)):
                    syrk.append((x_hi, x_lo, x_hi, x_lo, factor, None, None, None, d, 0, pack_flag, self._packing))
                inv = [(b.inv_hi[k][:, :d], lo(b.inv_lo[k][:, :d] if sp else None)) for k, d in enumerate(b.dims3)]
                f = (b.f_hi[:, :c], lo(b.f_lo[:, :c] if sp else None))
                gemm0.append(chained(*inv[2], *f, b.d1_hi, b.d1_lo))
                d1 = (b.d1_hi.view(c * a, bb), lo(b.d1_lo.view(c * a, bb) if sp else None))
                gemm1.append(chained(*inv[1], *d1, b.d2_hi, b.d2_lo))
                d2 = (b.d2_hi.view(bb * c, a), lo(b.d2_lo.view(bb * c, a) if sp else None))
                gemm2.append((*inv[0], *d2, b.p, None, None, self._norms[b.index, 1:2], bb * c, 0, F.FLAG_SUMSQ, False))
                continue
            two_d = b.order == 2
            left, right = two_d and b.sel[0], b.sel[-1]
            if not (left or right):
                continue  # the prologue itself delivers P = filtered gradient and ||P||^2
            t_hi = t_lo = None
            if right:
                t_hi, t_lo = op(b.gt_hi, b.n, b.m), (op(b.gt_lo, b.n, b.m) if self._split else None)
            if self._kl and left and right:
                # (a block with a single factor has no other dim to precondition along: plain Gram)
                # KL-Shampoo statistics: L <- Gram of G R^(-1/p), R <- Gram of L^(-1/p) G, with the
                # current inverse roots (reference: shampoo_preconditioner_list.py:1945-2046).
                a_hi, a_lo = op(b.g_hi, b.m, b.n), (op(b.g_lo, b.m, b.n) if sp else None)
                ri = (op(b.inv_hi[1], b.n, b.n), op(b.inv_lo[1], b.n, b.n) if sp else None)
                li = (op(b.inv_hi[0], b.m, b.m), op(b.inv_lo[0], b.m, b.m) if sp else None)
                kl.append(chained(a_hi, a_lo, *ri, b.y_hi, b.y_lo))
                kl.append(chained(t_hi, t_lo, *li, b.zt_hi, b.zt_lo))
                y = (op(b.y_hi, b.m, b.n), op(b.y_lo, b.m, b.n) if sp else None)
                zt = (op(b.zt_hi, b.n, b.m), op(b.zt_lo, b.n, b.m) if sp else None)
                syrk.append((*y, *y, fm[0], None, None, None, b.m, 0, pack_flag, self._packing))
                syrk.append((*zt, *zt, fm[-1], None, None, None, b.n, 0, pack_flag, self._packing))
            else:
                if left:
                    a_hi, a_lo = op(b.g_hi, b.m, b.n), (op(b.g_lo, b.m, b.n) if self._split else None)
                    syrk.append((a_hi, a_lo, a_hi, a_lo, fm[0], None, None, None, b.m, 0, pack_flag, self._packing))
                if right:
                    syrk.append((t_hi, t_lo, t_hi, t_lo, fm[-1], None, None, None, b.n, 0, pack_flag, self._packing))

            f_hi, f_lo = op(b.f_hi, b.m, b.n), (op(b.f_lo, b.m, b.n) if self._split else None)
            sumsq = self._norms[b.index, 1:2]
            if left and not right:
                # P = L F: the chain's second product with T^T = F^T, made by a transposing copy
                l_hi, l_lo = op(b.inv_hi[0], b.m, b.m), (op(b.inv_lo[0], b.m, b.m) if self._split else None)
                tt_hi, tt_lo = op(b.tt_hi, b.n, b.m), (op(b.tt_lo, b.n, b.m) if self._split else None)
                f_transposes.append((f_hi, tt_hi, None, None))
                if self._split:  # tf32 rounding is elementwise: the transposed pair is the pair of the transpose
                    f_transposes.append((f_lo, tt_lo, None, None))
                gemm2.append((l_hi, l_lo, tt_hi, tt_lo, b.p, None, None, sumsq, b.n, 0, F.FLAG_SUMSQ, False))
            elif left:
                r_hi, r_lo = op(b.inv_hi[1], b.n, b.n), (op(b.inv_lo[1], b.n, b.n) if self._split else None)
                l_hi, l_lo = op(b.inv_hi[0], b.m, b.m), (op(b.inv_lo[0], b.m, b.m) if self._split else None)
                if self._split:
                    gemm1.append(
                        (r_hi, r_lo, f_hi, f_lo, None, b.tt_hi, b.tt_lo, None, 0, b.m_pad, F.FLAG_NO_C | F.FLAG_SPLIT_OUT, False)
                    )
                else:
                    gemm1.append((r_hi, None, f_hi, None, b.tt_hi, None, None, None, b.m_pad, 0, 0, False))
                tt_hi, tt_lo = op(b.tt_hi, b.n, b.m), (op(b.tt_lo, b.n, b.m) if self._split else None)
                gemm2.append((l_hi, l_lo, tt_hi, tt_lo, b.p, None, None, sumsq, b.n, 0, F.FLAG_SUMSQ, False))
            else:  # columns only: a 1-D block, or a 2-D block whose rows are not preconditioned
                r_hi, r_lo = op(b.inv_hi[-1], b.n, b.n), (op(b.inv_lo[-1], b.n, b.n) if self._split else None)
                gemm2.append((f_hi, f_lo, r_hi, r_lo, b.p, None, None, sumsq, b.n, 0, F.FLAG_SUMSQ, False))
        self._f_transpose_table = ext.build_transpose_table(f_transposes) if f_transposes else None
        # the pushing plan pairs one final product with every block (see the rule at _gemm_push)
        assert not self._gemm_push or len(gemm2) == len(blocks)
        self._syrk_plan = ext.build_gemm_plan(syrk) if syrk else None
        self._kl_plan = ext.build_gemm_plan(kl) if kl else None
        self._gemm0_plan = ext.build_gemm_plan(gemm0) if gemm0 else None
        self._gemm1_plan = ext.build_gemm_plan(gemm1) if gemm1 else None
        self._gemm2_plan = ext.build_gemm_plan(gemm2) if gemm2 else None
        if self._gemm_push:
            # Same products; the result goes to the block's slot of every gather buffer instead of b.p.
            flags = F.FLAG_SUMSQ | F.FLAG_NO_C | F.FLAG_PEER_PUSH
            push = [
                (s[0], s[1], s[2], s[3], None, None, None, s[7], s[8], 0, flags, False, self._slot_offset(b))
                for s, b in zip(gemm2, blocks, strict=True)
            ]
            self._gemm2_push_plan = ext.build_gemm_plan(push)

    def _build_soap_plans(self, blocks: list[_Block]) -> None:
        """GEMM plans of the eigenvalue-corrected step.  With Qt the transposed eigenvector
        mirrors, a 2-D block is projected as T^T = Q_R^T X^T, X~ = Q_L^T T and unprojected as
        U^T = Q_R S^T, P = Q_L U; a 1-D block (1 x n) uses the column side only.

        ``_soap_plans``: ``a`` first projection stage of the raw and of the filtered gradient,
        ``v`` second stage of the raw gradient with the squared-EMA epilogue into the corrected
        eigenvalues, ``f`` second stage of the filtered gradient into ``p``, ``u1``/``u2`` the
        unprojection of the scaled direction (``u2`` accumulates the norm)."""
        ext, split = self._ext, self._split
        F = ext

        def pair(hi: Tensor, lo: Tensor | None, k: int) -> tuple[Tensor, Tensor | None]:
            return hi[:, :k], (lo[:, :k] if lo is not None else None)

        def chained(a, b, out_hi, out_lo):
            """Product whose result is only an operand of the next product."""
            if split:
                return (*_ab(a, b), None, out_hi, out_lo, None, 0, out_hi.stride(0), F.FLAG_NO_C | F.FLAG_SPLIT_OUT, False)
            return (*_ab(a, b), out_hi, None, None, None, out_hi.stride(0), 0, 0, False)

        def _ab(a, b):
            return (a[0], a[1], b[0], b[1])

        syrk, st_a0, st_a, st_v, st_f, st_u0, st_u1, st_u2 = [], [], [], [], [], [], [], []
        pack_flag = F.FLAG_PACKED_C if self._packing else 0
        for b in blocks:
            fm = b.factors.factor_matrices
            if b.dims3 is not None:
                # Order-3 block (a, b, c): every product contracts the fastest index of the current
                # layout and emits the new one slowest, (a,b,c) -> (c,a,b) -> (b,c,a) -> (a,b,c); the
                # raw and the filtered gradient go through Q_c^T, Q_b^T, Q_a^T side by side, the
                # scaled direction back through Q_c, Q_b, Q_a.
                a, bb, c = b.dims3
                lo = lambda t: t if split else None  # noqa: E731
                xa = (b.aux_g_hi, lo(b.aux_g_lo))
                xb = (b.aux_gt_hi.view(bb, c * a), lo(b.aux_gt_lo.view(bb, c * a) if split else None))
                xc = (b.gt_hi, lo(b.gt_lo))
                for x, factor, d in ((xa, fm[0], a), (xb, fm[1], bb), (xc, fm[2], c)):
                    syrk.append((*_ab(x, x), factor, None, None, None, d, 0, pack_flag, self._packing))
                q = [pair(b.inv_hi[k], b.inv_lo[k], d) for k, d in enumerate(b.dims3)]
                qt = [pair(b.qt_hi[k], b.qt_lo[k], d) for k, d in enumerate(b.dims3)]
                g3, f3 = pair(b.g_hi, b.g_lo, c), pair(b.f_hi, b.f_lo, c)

                def as_rows(hi, lo_, rows, cols):
                    return (hi.view(rows, cols), lo_.view(rows, cols) if lo_ is not None else None)

                st_a0.append(chained(qt[2], g3, b.e1_hi, b.e1_lo))
                st_a0.append(chained(qt[2], f3, b.d1_hi, b.d1_lo))
                st_a.append(chained(qt[1], as_rows(b.e1_hi, b.e1_lo, c * a, bb), b.e2_hi, b.e2_lo))
                st_a.append(chained(qt[1], as_rows(b.d1_hi, b.d1_lo, c * a, bb), b.d2_hi, b.d2_lo))
                ev = b.ev.view(a, bb * c)
                st_v.append((*_ab(qt[0], as_rows(b.e2_hi, b.e2_lo, bb * c, a)), ev, None, None, None, bb * c, 0, F.FLAG_SQUARE_ACC, False))
                st_f.append((*_ab(qt[0], as_rows(b.d2_hi, b.d2_lo, bb * c, a)), b.p, None, None, None, bb * c, 0, 0, False))
                st_u0.append(chained(q[2], f3, b.d1_hi, b.d1_lo))
                st_u1.append(chained(q[1], as_rows(b.d1_hi, b.d1_lo, c * a, bb), b.d2_hi, b.d2_lo))
                st_u2.append((*_ab(q[0], as_rows(b.d2_hi, b.d2_lo, bb * c, a)), b.p, None, None, self._norms[b.index, 1:2], bb * c, 0, F.FLAG_SUMSQ, False))
                continue
            two_d = b.order == 2
            g = pair(b.g_hi, b.g_lo, b.n)
            gt = pair(b.gt_hi, b.gt_lo, b.m)
            f = pair(b.f_hi, b.f_lo, b.n)
            sumsq = self._norms[b.index, 1:2]
            if two_d:
                syrk.append((*_ab(g, g), fm[0], None, None, None, b.m, 0, pack_flag, self._packing))
            syrk.append((*_ab(gt, gt), fm[-1], None, None, None, b.n, 0, pack_flag, self._packing))
            r = 1 if two_d else 0
            qr, qrt = pair(b.inv_hi[r], b.inv_lo[r], b.n), pair(b.qt_hi[r], b.qt_lo[r], b.n)
            if two_d:
                ql, qlt = pair(b.inv_hi[0], b.inv_lo[0], b.m), pair(b.qt_hi[0], b.qt_lo[0], b.m)
                t2, tt = pair(b.t2_hi, b.t2_lo, b.m), pair(b.tt_hi, b.tt_lo, b.m)
                st_a.append(chained(qrt, g, b.t2_hi, b.t2_lo))
                st_a.append(chained(qrt, f, b.tt_hi, b.tt_lo))
                st_v.append((*_ab(qlt, t2), b.ev, None, None, None, b.n, 0, F.FLAG_SQUARE_ACC, False))
                st_f.append((*_ab(qlt, tt), b.p, None, None, None, b.n, 0, 0, False))
                st_u1.append(chained(qr, f, b.tt_hi, b.tt_lo))
                st_u2.append((*_ab(ql, tt), b.p, None, None, sumsq, b.n, 0, F.FLAG_SUMSQ, False))
            else:
                st_v.append((*_ab(g, qrt), b.ev, None, None, None, b.n, 0, F.FLAG_SQUARE_ACC, False))
                st_f.append((*_ab(f, qrt), b.p, None, None, None, b.n, 0, 0, False))
                st_u2.append((*_ab(f, qr), b.p, None, None, sumsq, b.n, 0, F.FLAG_SUMSQ, False))
        self._syrk_plan = ext.build_gemm_plan(syrk)
        mk = lambda specs: ext.build_gemm_plan(specs) if specs else None  # noqa: E731
        self._soap_plans = {
            "a0": mk(st_a0), "a": mk(st_a), "v": mk(st_v), "f": mk(st_f), "u0": mk(st_u0), "u1": mk(st_u1), "u2": mk(st_u2),
        }

    def refresh_inverse_mirrors(self, blocks: list[_Block] | None = None) -> None:
        """Rebuild the full (hi, lo) operand copies of the inverse roots (or, for the
        eigenvalue-corrected variant, of the eigenvector matrices and their transposes) from the
        state tensors: one grouped launch over every factor of every block (two for the
        eigenvalue-corrected variant)."""
        ext, sp = self._ext, self._split
        todo = self._blocks if blocks is None else blocks
        if not todo:
            return
        if self._soap:
            plain, transposed = [], []
            for b in todo:
                for k, Q in enumerate(b.factors.factor_matrices_eigenvectors):
                    d = Q.shape[0]
                    Q = Q if Q.stride(-1) == 1 else Q.contiguous()
                    plain.append((Q, d, b.inv_hi[k][:, :d], b.inv_lo[k][:, :d] if sp else None))
                    if sp:
                        transposed.append((Q, None, b.qt_hi[k][:, :d], b.qt_lo[k][:, :d]))
                    else:
                        transposed.append((Q, b.qt_hi[k][:, :d], None, None))
            ext.unpack_split(*ext.build_unpack_table(plain))
            ext.transpose_split(*ext.build_transpose_table(transposed))
            return
        specs = []
        for b in todo:
            if self._eigdec:
                from fractions import Fraction

                from optimizers_b200.matrix import functions as mf

                kf = b.factors
                stability = kf.amortized_computation_config.rank_deficient_stability_config
                sources = [
                    mf.matrix_inverse_root_from_eigendecomposition(
                        L=lam, Q=Q, root=Fraction(root), epsilon=kf.epsilon, rank_deficient_stability_config=stability
                    ).contiguous()
                    for Q, lam, root in zip(kf.factor_matrices_eigenvectors, kf.factor_matrices_eigenvalues, kf.roots, strict=True)
                ]
            else:
                # the state itself: the packed upper triangle or the full matrix
                sources = [m if m.dim() == 1 or m.stride(-1) == 1 else m.contiguous() for m in b.factors.inv_factor_matrices]
            for k, src in enumerate(sources):
                d = b.inv_hi[k].shape[0]
                specs.append((src, d, b.inv_hi[k][:, :d], b.inv_lo[k][:, :d] if sp else None))
        if specs:
            ext.unpack_split(*ext.build_unpack_table(specs))

    # ------------------------------------------------------------------------------------------
    # Hooks called by the optimizer
    # ------------------------------------------------------------------------------------------
    def on_selector_change(self, selector: tuple[bool, ...]) -> None:
        self._active = tuple(selector)

    def on_state_loaded(self) -> None:
        if hasattr(self._dist, "refresh_assigned_full_params"):
            # The lossless distributors re-gathered their full copies: block views moved.
            self._build_blocks()
            self._plans_for = None
            self._gather_for = None
            self._full_table = None
        self.refresh_inverse_mirrors()

    def mode_switch(self, coeff: float) -> bool:
        """W <- W + coeff (Z - W) on every local block in one grouped launch (train()/eval() of the
        primal-averaging schemes).  Returns False when the switch has to travel through the
        distributor's collective instead (DDP)."""
        if self._ddp:
            return False
        if getattr(self, "_full_table", None) is None:
            specs = [
                (b.view2d, 0, 0, b.m, b.n, b.n_pad, b.m_pad, None, None, None, b.z) + (None,) * 8 + (0, 0, None, 0)
                for b in self._blocks
            ]
            self._full_table = self._ext.build_block_table(specs) if specs else ()
        if self._full_table:
            self._ext.mode_switch(*self._full_table, coeff, 0)
        if hasattr(self._dist, "_write_back"):
            # Lossless sharded distributors block this rank's gathered full copies; the model reads
            # its dim-0 shards, so the switched values travel back through the distributor's
            # (collective) write-back on every rank.
            self._dist._write_back()
        return True

    def collect_gradients(self) -> tuple[int, ...]:
        """Native twin of ``merge_and_block_gradients``: records which parameters have a usable
        gradient, refreshes the distributor's selectors, and stages the gradient base pointers.
        No per-block views are created.  Returns the pointers (empty when nothing has a gradient)."""
        dist = self._dist
        if self._pull:
            # Gradients live in the peer-addressable arena; every parameter takes part every step.
            for p, view in zip(self._group[PARAMS], self._grad_views, strict=True):
                if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                    raise RuntimeError(
                        "fuse_gradient_reduction=True: a parameter's .grad no longer is its view of the shared "
                        "gradient arena; call optimizer.zero_grad(set_to_none=False) (never set grads to None)."
                    )
            dist._global_grad_selector = (True,) * len(dist._global_blocked_params)
            dist._refresh_local_selection()
            return (1,)
        ptrs: list[int] = []
        selector: list[bool] = []
        any_grad = False
        # Held until the next step: some distributors hand out freshly gathered gradients whose
        # memory must outlive the kernels that read it through the pointer table.
        self._grads_alive = list(dist._get_params_or_grads(get_grad=True))
        for g, count in zip(self._grads_alive, dist._global_num_blocks_per_param, strict=True):
            usable = g is not None and g.numel() > 0
            if usable:
                if g.dtype != torch.float32 or not g.is_contiguous():
                    raise RuntimeError("the native step needs contiguous fp32 gradients")
                if self._optimizer._runtime_config.eager_nan_check:
                    assert torch.isfinite(g).all(), (
                        f"Encountered gradient containing NaN/Inf in parameter with shape {g.shape}. Check your model for numerical instability or consider gradient clipping."
                    )
                ptrs.append(g.data_ptr())
                any_grad = True
            else:
                ptrs.append(0)
            selector.extend([usable] * count)
        dist._global_grad_selector = tuple(selector)
        dist._refresh_local_selection()
        if ptrs != self._last_ptrs:
            self._grad_ptrs_flip ^= 1
            staging = self._grad_ptrs_host[self._grad_ptrs_flip]
            uploaded = self._grad_ptrs_uploaded[self._grad_ptrs_flip]
            if uploaded is not None:
                uploaded.synchronize()
            staging[: len(ptrs)] = torch.tensor(ptrs, dtype=torch.int64)
            self._grad_ptrs_dev.copy_(staging, non_blocking=True)
            if self._device.type == "cuda":
                event = torch.cuda.Event()
                event.record()
                self._grad_ptrs_uploaded[self._grad_ptrs_flip] = event
            self._last_ptrs = ptrs
        local_any = any_grad and any(dist.local_grad_selector)
        return tuple(ptrs) if local_any else ()

    def zero_grad(self) -> None:
        """Zero the shared gradient arena in one memset (fused-reduction mode)."""
        if self._pull:
            self._arena.region("grads").zero_()

    # ------------------------------------------------------------------------------------------
    # Observability
    # ------------------------------------------------------------------------------------------
    def memory_report(self) -> dict[str, int]:
        """Bytes this group keeps on the device, by purpose; arrays that share storage (the search
        direction in the place of G, chain intermediates in the place of G^T) are counted once.

        ``state``: what a checkpoint holds (factors, inverse roots / eigenvectors, corrected
        eigenvalues, filtered gradient, grafting and momentum buffers).  ``operands``: the tf32
        (hi, lo) operand arrays of the gradient, its transpose, the filtered gradient and the chain
        intermediates.  ``mirrors``: unpacked (hi, lo) copies of the inverse roots / eigenvectors
        and their transposes.  ``exchange``: all-gather buffers or the peer-addressable arena."""
        seen: set[tuple[int, int]] = set()

        def total(tensors) -> int:
            count = 0
            for t in tensors:
                if t is None:
                    continue
                key = (t.data_ptr(), t.numel() * t.element_size())
                if key not in seen:
                    seen.add(key)
                    count += key[1]
            return count

        def tensors_of(obj) -> list[Tensor]:
            found = []
            for value in vars(obj).values():
                for item in value if isinstance(value, (tuple, list)) else (value,):
                    if isinstance(item, Tensor):
                        found.append(item)
            return found

        report = {"state": 0, "operands": 0, "mirrors": 0, "exchange": 0}
        operand_fields = [f for f in _Block.__slots__ if f.endswith(("_hi", "_lo")) and not f.startswith(("inv_", "qt_"))]
        for b in self._blocks:
            report["state"] += total([b.m1, b.v, b.mom, b.z, *tensors_of(b.factors)])
            report["operands"] += total([getattr(b, f) for f in operand_fields] + [b.p])
            for field in ("inv_hi", "inv_lo", "qt_hi", "qt_lo"):
                report["mirrors"] += total(getattr(b, field) or [])
        if self._p2p:
            report["exchange"] = int(self._arena.nbytes)
        elif self._ddp:
            buffer = self._dist._global_dist_buffer
            report["exchange"] = buffer.numel() * buffer.element_size()
        report["total"] = sum(report.values())
        return report

    # ------------------------------------------------------------------------------------------
    # The step
    # ------------------------------------------------------------------------------------------
    def _raise_for(self, code: int) -> None:
        if code & 1:
            raise RuntimeError("grouped GEMM pipeline wait timed out (device-side bounded wait expired)")
        if code & 4:
            raise RuntimeError("a peer rank did not reach the cross-rank barrier in time (bounded device-side wait expired)")
        if code & 2:
            self._status.zero_()
            self._status_host.zero_()
            raise PreconditionerValueError("Encountered NaN/Inf in a gradient passed to the optimizer.")

    def check_status(self) -> None:
        """Read the device status word (one synchronisation) and raise on kernel-reported errors."""
        self._raise_for(int(self._status.item()))

    def _poll_status(self) -> None:
        """Non-blocking twin of ``check_status``: inspects the pinned copy made at the end of the
        previous step once that copy has completed (it has, unless the host runs more than a step
        ahead of the device, in which case the look is deferred to the next step)."""
        event = self._status_event
        if event is not None and event.query():
            self._status_event = None
            code = int(self._status_host[0])
            if code:
                self._raise_for(code)

    def _post_status(self) -> None:
        if self._status_event is None:  # the previous copy has been consumed: the buffer is free
            self._status_host.copy_(self._status, non_blocking=True)
            self._status_event = torch.cuda.Event()
            self._status_event.record()

    def step(
        self, group, step, lr, beta1, beta3, weight_decay, peak_lr, weight_decay_type, has_grafting, refresh,
        use_bias_correction, graft_only, primal, classic, mu_y, mu_x, momentum, dampening, nesterov,
    ) -> None:
        rec, ext = self._rec, self._ext
        self._poll_status()
        active = self._active if self._active is not None else (True,) * len(self._blocks)
        if self._plans_for != active:
            self._build_plans(active)
            self._plans_for = active
        alpha = 0.0
        if weight_decay != 0.0 and weight_decay_type != WeightDecayType.L2:
            if weight_decay_type == WeightDecayType.DECOUPLED:
                alpha = weight_decay
            elif weight_decay_type == WeightDecayType.CORRECTED:
                alpha = weight_decay * rec[LR_CPU_PINNED].item() / peak_lr
            else:
                alpha = weight_decay / peak_lr
        # All ranks take the same decision: it depends on the step and the configuration only.
        use_push = self._gemm_push and not graft_only and not classic and not primal
        scaled = (lr, alpha) if use_push else None
        if not rec[MASKED_BLOCKED_GRADS] or self._table is None:
            # Nothing to compute here; other ranks may still need this rank in their collective.
            self.launches_per_step = 0
            self._finish_update(scaled)
            return
        self._mark("start")
        if self._p2p:
            # Every rank has finished its backward pass (its gradients are complete) and has applied
            # the previous step's directions (its gather buffer may be overwritten).
            self._peer_barrier(0)
            self._mark("barrier_entry")
        t = int(step.item())
        launches = 0

        plist, glist = self._plist, self._glist
        plist._refresh_bias_correction(step)
        bc1 = 1.0 - beta3 * beta1 ** (t - 1) if (beta1 != 0.0 and use_bias_correction) else 1.0
        g_beta2 = g_weight = 1.0
        g_bc2, g_eps = 1.0, 0.0
        if self._graft_kind == _GRAFT_ADAGRAD:
            g_beta2, g_weight, g_eps = glist._beta2, glist._weighting_factor, glist._epsilon
            if glist._use_bias_correction and g_beta2 < 1.0:
                glist._bias_correction2 = torch.tensor(1.0) - g_beta2**step
            g_bc2 = float(glist._bias_correction2)
        l2 = weight_decay if (weight_decay_type == WeightDecayType.L2) else 0.0

        self._norms.zero_()
        blocks_t, tiles_t, n_tiles = self._table
        ext.grad_prologue(
            blocks_t, tiles_t, n_tiles, self._grad_ptrs_dev, l2, beta1, beta3, bc1, self._graft_kind,
            g_beta2, g_weight, g_bc2, g_eps, self._split, self._status,
            self._arena.world if self._pull else 0, 1.0 / self._arena.world if self._pull else 1.0,
        )
        launches += 2
        self._mark("grad_prologue")
        if not self._soap and self._kl_plan is not None:
            ext.run_gemm_plan(*self._kl_plan, 1.0, 0.0, self._split, self._status)
            launches += 1
        if self._syrk_plan is not None:
            ext.run_gemm_plan(*self._syrk_plan, plist._weighting_factor, plist._beta2, self._split, self._status)
            launches += 1
        self._mark("factor_syrk")

        if refresh:
            self._refresh(self._active_blocks)
            self._mark("refresh")

        if self._soap:
            launches += self._soap_step(plist, graft_only)
        elif not graft_only:
            if self._gemm0_plan is not None:
                ext.run_gemm_plan(*self._gemm0_plan, 1.0, 0.0, self._split, self._status)
                launches += 1
            if self._gemm1_plan is not None:
                ext.run_gemm_plan(*self._gemm1_plan, 1.0, 0.0, self._split, self._status)
                launches += 1
            if self._f_transpose_table is not None:
                ext.transpose_split(*self._f_transpose_table)
                launches += 1
            if use_push:
                # The last preconditioner GEMM stores its tiles into every rank's gather buffer.
                ext.run_gemm_plan_push(
                    *self._gemm2_push_plan, 1.0, 0.0, self._split, self._status, self._gather_bases, self._comm_dtype_code
                )
            elif self._gemm2_plan is not None:
                ext.run_gemm_plan(*self._gemm2_plan, 1.0, 0.0, self._split, self._status)
            launches += 1

        self._mark("preconditioner_gemms")
        if use_push:
            launches += self._push_scales(has_grafting)
            self.gemm_push_steps += 1
            self.launches_per_step = launches
            self._finish_update(scaled)
            return
        if primal and not rec[TRAIN_MODE]:
            raise RuntimeError(
                "Called _apply_in_place_primal_averaging when not in train mode. Call optimizer.train() before calling optimizer.step()!"
            )
        ext.direction_epilogue(
            blocks_t, tiles_t, n_tiles, lr, graft_only, self._graft_kind if has_grafting else _GRAFT_NONE, g_bc2,
            g_eps, alpha, primal, mu_y, mu_x, classic, momentum, dampening, nesterov, self._comm_dtype_code, self._split,
            self._gather_bases if self._p2p else [], self._comm_params,
        )
        launches += 1
        self._mark("direction_epilogue")
        self.launches_per_step = launches
        self._finish_update()

    def _soap_step(self, plist: Any, graft_only: bool) -> int:
        """Second-moment update in the eigenbasis (every step) and, unless only the grafting
        direction is needed, project -> scale -> unproject of the filtered gradient."""
        ext, plans, split = self._ext, self._soap_plans, self._split
        run = lambda key, alpha=1.0, beta=0.0: ext.run_gemm_plan(*plans[key], alpha, beta, split, self._status)  # noqa: E731
        launches = 0
        for stage in ("a0", "a"):  # first stages of the projections: order-3 blocks only, then 2-D and order-3
            if plans[stage] is not None:
                run(stage)
                launches += 1
        run("v", plist._weighting_factor, plist._beta2)
        launches += 1
        if graft_only:
            return launches
        run("f")
        for (blocks_t, tiles_t, n_tiles), root in self._eig_tables:
            ext.eig_scale(blocks_t, tiles_t, n_tiles, float(plist._bias_correction2), 1.0 / root, plist._epsilon, split)
        for stage in ("u0", "u1"):
            if plans[stage] is not None:
                run(stage)
                launches += 1
        run("u2")
        return launches + 2 + len(self._eig_tables)

    def _refresh(self, blocks: list[_Block]) -> None:
        """Amortised computation for the given blocks: batched native path for the eigen root
        inverse, the per-factor torch path for every other matrix-function config."""
        from optimizers_b200.matrix import batched

        plist = self._plist
        cfg = self._group[PRECONDITIONER_CONFIG].amortized_computation_config
        blocks = [b for b in blocks if len(b.factors.factor_matrices) > 0]  # a block may have no preconditioned dim
        if not blocks:
            return
        if self._soap:
            if batched.eigenbasis_refresh_supported(cfg):
                batched.batched_eigenbasis_refresh(blocks, plist._bias_correction2, self._ext)
            else:
                for b in blocks:
                    b.factors.amortized_computation(bias_correction2=plist._bias_correction2)
        elif self._eigdec:
            if batched.eigdec_refresh_supported(cfg):
                batched.batched_eigen_refresh(self._ext, blocks, plist._bias_correction2, self._split, self._status)
                self.check_status()
                return  # the mirrors were written by the refresh itself
            for b in blocks:
                b.factors.amortized_computation(bias_correction2=plist._bias_correction2)
        elif batched.eigen_refresh_supported(cfg):
            batched.batched_eigen_refresh(self._ext, blocks, plist._bias_correction2, self._split, self._status)
        elif batched.newton_refresh_supported(cfg):
            batched.batched_newton_refresh(self._ext, blocks, plist._bias_correction2, self._split, self._status)
        else:
            for b in blocks:
                b.factors.amortized_computation(bias_correction2=plist._bias_correction2)
        from optimizers_b200.matrix.batched import _PhaseClock

        clock = _PhaseClock("engine refresh tail")
        self.refresh_inverse_mirrors(blocks)
        clock.tick("operand mirrors from the state")
        clock.report()
        self.check_status()

    def _push_scales(self, has_grafting: bool) -> int:
        """Send each local block's grafting scale ||graft direction|| / ||P|| to slot [global block]
        of every rank's scale table (one grouped peer copy of 4-byte entries)."""
        ext, dist_ = self._ext, self._dist
        if getattr(self, "_scales_src", None) is None:
            self._scales_src = torch.ones(max(len(self._blocks), 1), dtype=torch.float32, device=self._device)
            self._global_index = [i for i, mine in enumerate(dist_._distributor_selector) if mine]
        if has_grafting and self._graft_kind != _GRAFT_NONE:
            torch.div(self._norms[:, 0].sqrt(), self._norms[:, 1].sqrt().add_(1e-16), out=self._scales_src)
        else:
            self._scales_src.fill_(1.0)
        if self._scale_copy_for != self._plans_for:
            base = self._scales_src.data_ptr()
            specs = [
                (base + 4 * b.index, peer + 4 * self._global_index[b.index], 4)
                for b in self._active_blocks
                for peer in self._scale_bases
            ]
            self._scale_copy = ext.build_copy_table(specs, self._device.index)
            self._scale_copy_for = self._plans_for
        ext.peer_copy(*self._scale_copy)
        return 4

    def _finish_update(self, scaled: tuple[Tensor, float] | None = None) -> None:
        self._deliver(scaled)
        self._post_status()

    def _deliver(self, scaled: tuple[Tensor, float] | None = None) -> None:
        """Deliver the search directions.  Single device: the epilogue already updated the
        parameters.  DDP: all-gather (NCCL), or a cross-rank barrier after the epilogue's peer
        stores (p2p); then one grouped kernel adds every block's direction to the parameters."""
        if not self._ddp:
            if hasattr(self._dist, "_write_back"):
                self._dist._write_back()  # lossless variants: full copies -> local shards
            return
        dist_ = self._dist
        if self._p2p:
            if self.launches_per_step == 0:
                self._peer_barrier(0)
            self._peer_barrier(1)
            self._mark("barrier_exit")
            self.launches_per_step += 1
            recv = self._gather_local
        else:
            dist_._all_gather()
            self._mark("all_gather")
            recv = dist_._global_dist_buffer
        sel = dist_._global_grad_selector
        if self._gather_for != sel:
            specs = []
            base = recv.data_ptr()
            for index, (view, off, on) in enumerate(
                zip(dist_._global_blocked_params, dist_._global_block_byte_offsets, sel, strict=True)
            ):
                if not on:
                    continue
                if view.dim() == 3:
                    view = view.view(view.shape[0] * view.shape[1], view.shape[2])
                m, n = (1, view.shape[0]) if view.dim() == 1 else view.shape
                scale = self._scales_local[index : index + 1] if self._p2p else None
                specs.append((view, 0, 0, m, n, _pad4(n), _pad4(m)) + (None,) * 11 + (scale, base + off, off, None, 0))
            self._gather_table = self._ext.build_block_table(specs) if specs else None
            self._gather_for = sel
        # p2p: the slots were filled by this rank's and the peers' kernels; after a device-side
        # timeout they may be partial, so the apply kernel checks the status word itself.
        guard = self._status if self._p2p else None
        if self._gather_table is not None:
            if scaled is not None:
                self._ext.gathered_apply_scaled(*self._gather_table, self._comm_dtype_code, scaled[0], scaled[1], guard)
            else:
                self._ext.gathered_apply(*self._gather_table, self._comm_dtype_code, self._comm_params, guard)
            self._mark("gathered_apply")
            self.launches_per_step += 1
        if hasattr(dist_, "_write_back"):
            dist_._write_back()
