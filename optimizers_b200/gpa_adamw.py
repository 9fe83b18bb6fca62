"""GPA-AdamW: AdamW with Generalized Primal Averaging or Schedule-Free averaging.

Three sequences are kept: ``y`` (where gradients are taken; stored in the parameters while
training), ``z`` (the base AdamW iterate, in state ``"z"``) and ``x`` (the averaged iterate the
model should be evaluated at; the parameters hold it after ``eval()``).  One step, with
``c`` the z-weight of the averaging (``1 - eval_interp_coeff`` for GPA, the polynomial
Schedule-Free weight otherwise) and ``ĝ`` the bias-corrected Adam direction:

    m ← lerp(m, g, 1-β1);  v ← β2 v + (1-β2) g²;  ĝ = (m / bc1) / (sqrt(v / bc2) + ε)
    weight decay shrinks y or z by (1 - lr·wd)
    y ← lerp(y, z, c) + lr·(μy(1-c) - 1)·ĝ
    z ← z - lr·ĝ

``train()``/``eval()`` move the parameters between y and x by ``p ← lerp(p, z, 1-μy)`` and
``p ← lerp(p, z, 1-1/μy)``.  The optimizer starts in eval mode and ``step()`` raises until
``train()`` has been called.

On a B200 the whole update of a parameter group is one multi-tensor kernel
(``ops/csrc/flat_kernels.cu``) instead of a Python loop of pointwise launches per parameter.

Reference counterpart: ``gpa/gpa_adamw.py:42-540`` and ``gpa/gpa_types.py:14-50``.
"""

from __future__ import annotations

import enum
import logging
from collections.abc import Callable
from typing import Any

import torch
from torch.optim.optimizer import Optimizer, ParamsT

logger: logging.Logger = logging.getLogger(__name__)

# Group keys
LR = "lr"
EPS = "eps"
BETA1 = "beta1"
BETA2 = "beta2"
PARAMS = "params"
TRAIN_INTERP_COEFF = "train_interp_coeff"
WEIGHT_POW_COEFF = "weight_pow_coeff"
WEIGHT_LR_POWER = "weight_lr_power"
WEIGHT_DECAY = "weight_decay"
USE_WD_ON_Y = "use_wd_on_y"
EVAL_INTERP_COEFF = "eval_interp_coeff"
ITERATE_AVERAGING_TYPE = "iterate_averaging_type"
# Per-parameter state keys
Z_BUFFER = "z"
EXP_AVG = "exp_avg"
EXP_AVG_SQ = "exp_avg_sq"
# Group-shared state, stored on the first parameter of the group
TRAIN_MODE = "train_mode"
LR_MAX = "lr_max"
WEIGHT_SUM = "weight_sum"
STEP = "step"


class IterateAveragingType(enum.Enum):
    """GPA: fixed ``eval_interp_coeff``.  SCHEDULE_FREE: polynomially weighted running average."""

    GPA = "gpa"
    SCHEDULE_FREE = "schedule_free"


class GPAAdamW(Optimizer):
    def __init__(
        self,
        params: ParamsT,
        lr: float | torch.Tensor = 1.0,
        eps: float = 1e-8,
        beta1: float = 0.9,
        beta2: float = 0.999,
        weight_decay: float = 0,
        use_wd_on_y: bool = False,
        iterate_averaging_type: IterateAveragingType = IterateAveragingType.GPA,
        train_interp_coeff: float = 0.7,
        eval_interp_coeff: float = 0.9967,
        weight_pow_coeff: float = 0.0,
        weight_lr_power: float = 2,
        use_native_kernels: bool | None = None,
    ) -> None:
        if not lr >= 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not eps >= 0.0:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= beta1 < 1.0:
            raise ValueError(f"Invalid beta1 value: {beta1}")
        if not 0.0 <= beta2 < 1.0:
            raise ValueError(f"Invalid beta2 value: {beta2}")
        if not weight_decay >= 0.0:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        if not isinstance(iterate_averaging_type, IterateAveragingType):
            raise ValueError(
                f"iterate_averaging_type must be an IterateAveragingType enum, got {type(iterate_averaging_type)}"
            )
        if not 0.0 < train_interp_coeff <= 1.0:
            raise ValueError(f"train_interp_coeff must be in range (0, 1]: {train_interp_coeff}")
        if not 0.0 <= eval_interp_coeff <= 1.0:
            raise ValueError(f"eval_interp_coeff must be in range [0, 1]: {eval_interp_coeff}")
        if not weight_pow_coeff >= 0.0:
            raise ValueError(f"Invalid weight_pow_coeff value: {weight_pow_coeff}")
        if not weight_lr_power >= 0.0:
            raise ValueError(f"Invalid weight_lr_power value: {weight_lr_power}")
        super().__init__(
            params,
            {
                LR: lr,
                EPS: eps,
                TRAIN_INTERP_COEFF: train_interp_coeff,
                BETA1: beta1,
                BETA2: beta2,
                WEIGHT_POW_COEFF: weight_pow_coeff,
                WEIGHT_LR_POWER: weight_lr_power,
                WEIGHT_DECAY: weight_decay,
                USE_WD_ON_Y: use_wd_on_y,
                EVAL_INTERP_COEFF: eval_interp_coeff,
                ITERATE_AVERAGING_TYPE: iterate_averaging_type,
            },
        )
        self._use_native = use_native_kernels
        self._tables: dict[int, Any] = {}
        self.native_launches = 0

    # -- shared / per-parameter state ----------------------------------------------------------
    def _ensure_shared_state(self, group: dict[str, Any]):
        """Create the group-level scalars on the group's first parameter; returns that parameter."""
        if not group[PARAMS]:
            return None
        first = group[PARAMS][0]
        state = self.state[first]
        state.setdefault(TRAIN_MODE, torch.tensor(False, dtype=torch.bool))
        state.setdefault(LR_MAX, torch.tensor(-1.0, dtype=torch.float32))
        state.setdefault(WEIGHT_SUM, torch.tensor(0.0, dtype=torch.float32))
        state.setdefault(STEP, torch.tensor(0, dtype=torch.int64))
        return first

    def _init_group(self, group, params_with_grad, grads, exp_avgs, exp_avg_sqs, z_buffer_list) -> bool:
        """Create missing per-parameter buffers and collect those of parameters with a gradient."""
        self._ensure_shared_state(group)
        sparse = False
        for p in group[PARAMS]:
            if p.grad is None:
                continue
            sparse |= p.grad.is_sparse
            state = self.state[p]
            if Z_BUFFER not in state:
                state[Z_BUFFER] = torch.clone(p, memory_format=torch.preserve_format)
            if EXP_AVG not in state:
                state[EXP_AVG] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
            if EXP_AVG_SQ not in state:
                state[EXP_AVG_SQ] = torch.zeros_like(p, dtype=torch.float32, memory_format=torch.preserve_format)
            params_with_grad.append(p)
            grads.append(p.grad)
            exp_avgs.append(state[EXP_AVG])
            exp_avg_sqs.append(state[EXP_AVG_SQ])
            z_buffer_list.append(state[Z_BUFFER])
        return sparse

    # -- native path ---------------------------------------------------------------------------
    def _native_ok(self, params: list[torch.Tensor], zs: list[torch.Tensor]) -> bool:
        if self._use_native is False or not params:
            return False
        ok = all(
            p.is_cuda and p.is_contiguous() and p.grad.is_contiguous() and not p.grad.is_sparse
            and p.grad.dtype == p.dtype and p.dtype in (torch.float32, torch.bfloat16, torch.float16)
            and z.dtype == torch.float32 and type(p.data) is torch.Tensor
            for p, z in zip(params, zs, strict=True)
        ) and torch.cuda.get_device_capability(params[0].device)[0] == 10
        if not ok and self._use_native is True:
            raise RuntimeError("use_native_kernels=True needs contiguous CUDA parameters with fp32 z buffers on sm_100")
        return ok

    def _table(self, gi: int, params, grads, zs, ms, vs):
        """Pointer table of a group, rebuilt only when any tensor address changed."""
        from optimizers_b200.ops import build

        ext = build.load()
        key = tuple(t.data_ptr() for ts in (params, grads, zs, ms, vs) for t in ts)
        cached = self._tables.get(gi)
        if cached is None or cached[0] != key:
            table = ext.build_gpa_table(list(zip(params, grads, zs, ms, vs)))
            cached = (key, table)
            self._tables[gi] = cached
        return ext, cached[1]

    # -- mode switches ---------------------------------------------------------------------------
    def _switch(self, to_train: bool) -> None:
        for gi, group in enumerate(self.param_groups):
            first = self._ensure_shared_state(group)
            if first is None:
                continue
            mode = self.state[first][TRAIN_MODE]
            if bool(mode.item()) == to_train:
                continue
            mu_y = group[TRAIN_INTERP_COEFF]
            weight = (1 - mu_y) if to_train else (1 - 1 / mu_y)
            with_z = [p for p in group[PARAMS] if p in self.state and Z_BUFFER in self.state[p]]
            zs = [self.state[p][Z_BUFFER] for p in with_z]
            if with_z and self._use_native is not False and all(
                p.is_cuda and p.is_contiguous() and z.dtype == torch.float32 and z.is_contiguous() and type(p.data) is torch.Tensor
                and p.dtype in (torch.float32, torch.bfloat16, torch.float16)
                for p, z in zip(with_z, zs)
            ) and torch.cuda.get_device_capability(with_z[0].device)[0] == 10:
                # One grouped launch: p <- lerp(p, z, weight) for every parameter of the group.
                from optimizers_b200.ops import build

                ext = build.load()
                table, chunks, n_chunks = ext.build_gpa_table([(p, None, z, z, z) for p, z in zip(with_z, zs)])
                ext.gpa_lerp(table, n_chunks, chunks, weight)
                self.native_launches += 1
                mode.fill_(to_train)
                continue
            for p in group[PARAMS]:
                state = self.state.get(p) if p in self.state else None
                if state and Z_BUFFER in state:
                    p.lerp_(end=state[Z_BUFFER].to(p.device), weight=weight)
            mode.fill_(to_train)

    @torch.no_grad()
    def eval(self) -> None:
        """Parameters become the averaged x sequence."""
        logger.info("Toggling GPAAdamW eval mode!")
        self._switch(False)

    @torch.no_grad()
    def train(self) -> None:
        """Parameters become the y sequence gradients are taken at."""
        logger.info("Toggling GPAAdamW train mode!")
        self._switch(True)

    # -- step --------------------------------------------------------------------------------------
    @staticmethod
    def compute_avg_coeff(
        iterate_averaging_type: IterateAveragingType,
        eval_interp_coeff: float,
        k: int,
        weight_pow_coeff: float,
        lr_max: float,
        weight_lr_power: float,
        weight_sum_ref: torch.Tensor,
    ) -> float:
        """The z-weight of the averaging step.  Schedule-Free: w_k / Σ w_i with
        w_k = k^r · lr_max^power (``weight_sum_ref`` is advanced in place); GPA: 1 - μx."""
        if iterate_averaging_type == IterateAveragingType.SCHEDULE_FREE:
            weight = (k**weight_pow_coeff) * (lr_max**weight_lr_power)
            weight_sum_ref += weight
            return weight / weight_sum_ref
        return 1 - eval_interp_coeff

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:  # type: ignore[override]
        for group in self.param_groups:
            first = self._ensure_shared_state(group)
            if first is not None:
                if not self.state[first][TRAIN_MODE]:
                    raise RuntimeError(
                        "Optimizer was not in train mode when step is called. "
                        "Please insert .train() and .eval() calls on the "
                        "optimizer. See documentation for details."
                    )
                break
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        for gi, group in enumerate(self.param_groups):
            if not group[PARAMS]:
                continue
            params: list[torch.Tensor] = []
            grads: list[torch.Tensor] = []
            ms: list[torch.Tensor] = []
            vs: list[torch.Tensor] = []
            zs: list[torch.Tensor] = []
            self._init_group(group, params, grads, ms, vs, zs)

            shared = self.state[group[PARAMS][0]]
            shared[STEP] += 1
            k = shared[STEP].item()
            lr, eps = group[LR], group[EPS]
            beta1, beta2 = group[BETA1], group[BETA2]
            mu_y = group[TRAIN_INTERP_COEFF]
            wd, wd_on_y = group[WEIGHT_DECAY], group[USE_WD_ON_Y]
            bc1, bc2 = 1 - beta1**k, 1 - beta2**k
            lr_max = max(lr, shared[LR_MAX].item())
            shared[LR_MAX].fill_(lr_max)
            assert lr_max > 0, f"lr_max must be positive, got lr_max={lr_max}. Check that lr={lr} is positive."
            c = self.compute_avg_coeff(
                iterate_averaging_type=group[ITERATE_AVERAGING_TYPE],
                eval_interp_coeff=group[EVAL_INTERP_COEFF],
                k=k,
                weight_pow_coeff=group[WEIGHT_POW_COEFF],
                lr_max=lr_max,
                weight_lr_power=group[WEIGHT_LR_POWER],
                weight_sum_ref=shared[WEIGHT_SUM],
            )
            # In Schedule-Free mode ``c`` is a 0-dim tensor (weight / weight_sum), and the reference
            # feeds it to ``lerp_`` and to ``1 - c`` as such: the torch path below does the same, to
            # the bit; only the kernel takes it as a host scalar.
            if self._native_ok(params, zs):
                ext, (table, chunks, n_chunks) = self._table(gi, params, grads, zs, ms, vs)
                ext.gpa_adamw_step(table, n_chunks, chunks, float(lr), beta1, beta2, eps, bc1, bc2, wd, wd_on_y, float(c), mu_y)
                self.native_launches += 1
                continue

            for y, g, m, v, z in zip(params, grads, ms, vs, zs, strict=True):
                m.lerp_(g, 1 - beta1)
                v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
                direction = m.div(bc1).div_(v.div(bc2).sqrt_().add_(eps))
                if wd != 0:
                    (y if wd_on_y else z).mul_(1 - lr * wd)
                y.lerp_(end=z, weight=c)
                y.add_(direction, alpha=lr * (mu_y * (1 - c) - 1))
                z.sub_(direction, alpha=lr)
        return loss
