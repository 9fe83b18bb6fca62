"""Typed configuration objects and state/group key names of the optimizer library.

One module holds the whole configuration surface so that checkpoints (which pickle the config
objects stored in ``param_groups``) depend on a single import path:

* matrix-function configs (root inverse, eigendecomposition, orthogonalisation),
* preconditioner configs (diagonal, Kronecker-factored, sign/spectral descent),
* iterate-averaging configs, weight-decay kinds,
* distributed configs and the small runtime configs,
* the string keys used in ``optimizer.state`` and ``optimizer.param_groups``.

Names, defaults and validation messages follow the reference's
``distributed_shampoo/shampoo_types.py`` and
``distributed_shampoo/preconditioner/matrix_functions_types.py``; ``NativeRuntimeConfig`` is new
and selects the sm_100a kernel back-end.
"""

from __future__ import annotations

import abc
import enum
import inspect
import math
from collections.abc import Callable
from dataclasses import dataclass, field, make_dataclass
from typing import Any

import torch
from torch import Tensor
from torch.distributed.device_mesh import DeviceMesh
from torch.distributed.fsdp import ShardingStrategy
from torch.nn.parameter import Parameter

# --------------------------------------------------------------------------------------------
# Keys.  State keys appear in checkpoints; group keys appear in ``param_groups``.
# --------------------------------------------------------------------------------------------
FILTERED_GRAD = "filtered_grad"
LR_SUM = "lr_sum"
MOMENTUM_BUFFER = "momentum_buffer"
STEP = "step"
TRAIN_MODE = "train_mode"
WEIGHT_BUFFER = "weight_buffer"
SHAMPOO = "shampoo"
ADAGRAD = "adagrad"

BETA3 = "beta3"
BETAS = "betas"
DISTRIBUTED_CONFIG = "distributed_config"
EPSILON = "epsilon"
GRAFTING_CONFIG = "grafting_config"
ITERATE_AVERAGING_CONFIG = "iterate_averaging_config"
LR = "lr"
MAX_PRECONDITIONER_DIM = "max_preconditioner_dim"
PARAMS = "params"
PEAK_LR = "peak_lr"
PRECONDITION_FREQUENCY = "precondition_frequency"
PRECONDITIONER_CONFIG = "preconditioner_config"
START_PRECONDITIONING_STEP = "start_preconditioning_step"
USE_BIAS_CORRECTION = "use_bias_correction"
USE_PIN_MEMORY = "use_pin_memory"
WEIGHT_DECAY = "weight_decay"
WEIGHT_DECAY_TYPE = "weight_decay_type"
OWNER_RANKS = "owner_ranks"

# Keys of the per-group runtime record kept by the optimizer (never checkpointed).
CUDA_STREAM = "cuda_stream"
DISTRIBUTOR = "distributor"
EVAL_INTERP_COEFF = "eval_interp_coeff"
FILTERED_GRAD_LIST = "filtered_grad_list"
GRAFTING_PRECONDITIONER_LIST = "grafting_preconditioner_list"
LR_CPU_PINNED = "lr_cpu_pinned"
LR_TENSOR = "lr_tensor"
MASKED_BLOCKED_GRADS = "masked_blocked_grads"
MASKED_BLOCKED_PARAMS = "masked_blocked_params"
MASKED_FILTERED_GRAD_LIST = "masked_filtered_grad_list"
MASKED_MOMENTUM_BUFFER_LIST = "masked_momentum_buffer_list"
MASKED_WEIGHT_BUFFER_LIST = "masked_weight_buffer_list"
MOMENTUM_BUFFER_LIST = "momentum_buffer_list"
PREVIOUS_GRAD_SELECTOR = "previous_grad_selector"
SHAMPOO_PRECONDITIONER_LIST = "shampoo_preconditioner_list"
TRAIN_INTERP_COEFF = "train_interp_coeff"
WEIGHT_BUFFER_LIST = "weight_buffer_list"


class PreconditionerValueError(ValueError):
    """A factor matrix or a freshly computed preconditioner holds NaN or Inf."""


@dataclass(init=False)
class AbstractDataclass(abc.ABC):
    """Dataclass root whose abstract ``__init__`` keeps the intermediate bases uninstantiable;
    concrete subclasses get their ``__init__`` from ``@dataclass``."""

    @abc.abstractmethod
    def __init__(self, *args: object, **kwargs: object) -> None: ...


# --------------------------------------------------------------------------------------------
# Cost models used by load balancing.
# --------------------------------------------------------------------------------------------
class CostModel(AbstractDataclass):
    @abc.abstractmethod
    def cost(self, tensor: Tensor) -> float:
        """Load contributed by one block."""


@dataclass
class AlignedMemoryCostModel(CostModel):
    """Bytes of the block rounded up to ``alignment_bytes`` (what the block occupies in the
    all-gather buffer)."""

    alignment_bytes: int = 64

    def cost(self, tensor: Tensor) -> float:
        raw = tensor.numel() * tensor.element_size()
        a = self.alignment_bytes
        return -(-raw // a) * a


@dataclass
class PolynomialComputationalCostModel(CostModel):
    """Σ over dims of max(min_cost, poly(dim)), ``coefficients`` in ascending power order; a
    proxy for the O(d³) refresh cost of a block."""

    coefficients: tuple[float, ...]
    min_cost: float = 0

    def cost(self, tensor: Tensor) -> float:
        def poly(x: int) -> float:
            acc = 0.0
            for c in reversed(self.coefficients):
                acc = acc * x + c
            return float(acc)

        return sum(max(self.min_cost, poly(d)) for d in tensor.shape)


DefaultCostModel = AlignedMemoryCostModel()


@dataclass(kw_only=True)
class LoadBalancingConfig:
    @staticmethod
    def _get_default_cost_model() -> CostModel:
        return DefaultCostModel

    cost_model: CostModel = field(default_factory=_get_default_cost_model)


# --------------------------------------------------------------------------------------------
# Matrix-function configs.
# --------------------------------------------------------------------------------------------
@dataclass(init=False)
class RankDeficientStabilityConfig(AbstractDataclass):
    """How a (nearly) singular factor is handled when its inverse root is formed."""


@dataclass(kw_only=True)
class PerturbationConfig(RankDeficientStabilityConfig):
    """Add εI; before the factorisation if ``perturb_before_computation`` else to the eigenvalues."""

    perturb_before_computation: bool = True


DefaultPerturbationConfig = PerturbationConfig()


@dataclass(kw_only=True)
class PseudoInverseConfig(RankDeficientStabilityConfig):
    """Drop eigenvalues ≤ max(rank_atol, rank_rtol·λ_max) (``rank_rtol=None`` → d·eps)."""

    rank_atol: float = 0.0
    rank_rtol: float | None = 0.0


@dataclass(init=False)
class MatrixFunctionConfig(AbstractDataclass):
    """Base of every amortised matrix computation."""


@dataclass(init=False)
class EigendecompositionConfig(MatrixFunctionConfig):
    @staticmethod
    def _get_default_rank_deficient_stability_config() -> RankDeficientStabilityConfig:
        return DefaultPerturbationConfig

    rank_deficient_stability_config: RankDeficientStabilityConfig = field(
        default_factory=_get_default_rank_deficient_stability_config
    )
    tolerance: float = 0.0

    def __post_init__(self) -> None:
        if not (0.0 <= self.tolerance <= 1.0):
            raise ValueError(
                f"Invalid tolerance value: {self.tolerance}. Must be in the interval [0.0, 1.0]."
            )


@dataclass(kw_only=True)
class EighEigendecompositionConfig(EigendecompositionConfig):
    retry_double_precision: bool = True
    eigendecomposition_offload_device: str = ""


DefaultEigendecompositionConfig = EighEigendecompositionConfig()


@dataclass(kw_only=True)
class QREigendecompositionConfig(EigendecompositionConfig):
    max_iterations: int = 1


@dataclass(init=False)
class RootInvConfig(MatrixFunctionConfig):
    """Base of the inverse-root algorithms."""


@dataclass(kw_only=True)
class EigenConfig(RootInvConfig, EighEigendecompositionConfig):
    def __post_init__(self) -> None:
        EighEigendecompositionConfig.__post_init__(self)
        if self.tolerance != 0.0:
            raise ValueError(
                f"Invalid tolerance value: {self.tolerance}. Must be 0.0 for {type(self).__name__}."
            )


DefaultEigenConfig = EigenConfig()


@dataclass(kw_only=True)
class CoupledNewtonConfig(RootInvConfig):
    """Coupled Newton iteration for the inverse root (reference:
    ``preconditioner/matrix_functions_types.py``, ``matrix_functions.py:369-437``).

    ``tolerance`` bounds ``max|M - I|``.  On the native sm_100a path the products run on the tensor
    cores as three tf32 products with an fp32 accumulator that truncates; their rounding floor for
    ``max|M - I|`` lies between 1e-6 and 1e-4, depending on the matrix size.  There the iteration
    also stops for a factor whose error is below 1e-3 and has not improved by 10 % between two
    checks (every fourth iteration): the configured tolerance is then not reached, and not
    reachable, and no warning is logged (the warning of the reference is kept for a factor that
    exhausts ``max_iterations`` above the tolerance).  The torch path honours ``tolerance`` exactly."""

    max_iterations: int = 100
    tolerance: float = 1e-6


@dataclass(kw_only=True)
class CoupledHigherOrderConfig(RootInvConfig):
    rel_epsilon: float
    abs_epsilon: float
    max_iterations: int = 100
    tolerance: float = 1e-8
    order: int = 3
    disable_tf32: bool = True


@dataclass(init=False)
class OrthogonalizationConfig(MatrixFunctionConfig):
    @staticmethod
    def _default_scale_by_dims_fn(d_in: int, d_out: int) -> float:
        return 1.0

    @staticmethod
    def _get_default_scale_by_dims_fn() -> Callable[[int, int], float]:
        return OrthogonalizationConfig._default_scale_by_dims_fn

    scale_by_dims_fn: Callable[[int, int], float] = field(
        default_factory=_get_default_scale_by_dims_fn
    )


@dataclass(kw_only=True)
class SVDOrthogonalizationConfig(OrthogonalizationConfig):
    scale_by_nuclear_norm: bool = False


@dataclass(kw_only=True)
class NewtonSchulzOrthogonalizationConfig(OrthogonalizationConfig):
    num_iterations: int = 5
    coefficients: tuple[float, float, float] = (3.4445, -4.7750, 2.0315)


DefaultNewtonSchulzOrthogonalizationConfig = NewtonSchulzOrthogonalizationConfig()


# --------------------------------------------------------------------------------------------
# Preconditioner configs.
# --------------------------------------------------------------------------------------------
@dataclass(init=False)
class PreconditionerConfig(AbstractDataclass):
    """Base of everything accepted as ``preconditioner_config`` / ``grafting_config``."""


@dataclass
class SGDPreconditionerConfig(PreconditionerConfig):
    """Identity preconditioner."""


@dataclass(kw_only=True)
class AdaGradPreconditionerConfig(PreconditionerConfig):
    epsilon: float = 1e-10

    def __post_init__(self) -> None:
        if not self.epsilon > 0.0:
            raise ValueError(f"Invalid epsilon value: {self.epsilon}. Must be > 0.0.")


@dataclass(kw_only=True)
class RMSpropPreconditionerConfig(AdaGradPreconditionerConfig):
    beta2: float = 0.99
    drop_weighting_factor_on_gsquare: bool = False

    def __post_init__(self) -> None:
        super().__post_init__()
        if not 0.0 < self.beta2 <= 1.0:
            raise ValueError(
                f"Invalid grafting beta2 parameter: {self.beta2}. Must be in (0.0, 1.0]."
            )


@dataclass(kw_only=True)
class AdamPreconditionerConfig(RMSpropPreconditionerConfig):
    beta2: float = 0.999


def _check_orders_nonnegative(name_repr: str, orders: Any) -> None:
    if bad := [o for o in orders if o < 0]:
        raise ValueError(f"Invalid orders in {name_repr}: {bad}. All orders must be >= 0.")


@dataclass(init=False)
class BaseShampooPreconditionerConfig(PreconditionerConfig):
    amortized_computation_config: MatrixFunctionConfig = field(repr=False)
    drop_weighting_factor_on_gsquare: bool = False
    factor_matrix_dtype: torch.dtype = torch.float32
    num_tolerated_failed_amortized_computations: int = 3
    use_symmetric_packing: bool = True
    use_trace_scaling: bool = False
    trace_scaling_exponent: float = 0.5

    def __post_init__(self) -> None:
        if self.num_tolerated_failed_amortized_computations < 0:
            raise ValueError(
                f"Invalid num_tolerated_failed_amortized_computations value: {self.num_tolerated_failed_amortized_computations}. Must be >= 0."
            )
        if self.use_trace_scaling and not 0.0 < self.trace_scaling_exponent <= 1.0:
            raise ValueError(
                f"Invalid trace_scaling_exponent value: {self.trace_scaling_exponent}. Must be in (0.0, 1.0] when use_trace_scaling=True."
            )


@dataclass(init=False)
class ClassicShampooPreconditionerConfig(BaseShampooPreconditionerConfig):
    """``inverse_exponent_override[order]`` is either one exponent for every dim of tensors of
    that order or a ``{dim: exponent}`` map; exponent 0 leaves the dim unpreconditioned."""

    inverse_exponent_override: dict[int, dict[int, float] | float] = field(default_factory=dict)

    def __post_init__(self) -> None:
        super().__post_init__()
        _check_orders_nonnegative(
            f"self.inverse_exponent_override={self.inverse_exponent_override}",
            self.inverse_exponent_override.keys(),
        )
        for order, override in self.inverse_exponent_override.items():
            shown = f"self.inverse_exponent_override[{order}]={override}"
            if isinstance(override, dict):
                top = max(order - 1, 0)
                if bad_dims := [d for d in override if not 0 <= d <= top]:
                    raise ValueError(
                        f"Invalid dimensions in {shown}: {bad_dims}. All dimensions must be within [0, {top}]."
                    )
                if bad_vals := [v for v in override.values() if v < 0]:
                    raise ValueError(
                        f"Invalid override value in {shown}: {bad_vals}. All overrides must be >= 0."
                    )
            else:
                assert isinstance(override, float)
                if override < 0:
                    raise ValueError(
                        f"Invalid override value in {shown}: {override}. All overrides must be >= 0."
                    )


@dataclass(kw_only=True)
class RootInvShampooPreconditionerConfig(ClassicShampooPreconditionerConfig):
    @staticmethod
    def _get_default_amortized_computation_config() -> RootInvConfig:
        return DefaultEigenConfig

    amortized_computation_config: RootInvConfig = field(
        default_factory=_get_default_amortized_computation_config
    )
    inv_factor_matrix_dtype: torch.dtype = torch.float32


DefaultShampooConfig = RootInvShampooPreconditionerConfig()


@dataclass(kw_only=True)
class EigendecomposedShampooPreconditionerConfig(ClassicShampooPreconditionerConfig):
    @staticmethod
    def _get_default_amortized_computation_config() -> EigendecompositionConfig:
        return DefaultEigendecompositionConfig

    amortized_computation_config: EigendecompositionConfig = field(
        default_factory=_get_default_amortized_computation_config
    )
    factor_matrix_eigenvectors_dtype: torch.dtype = torch.float32
    factor_matrix_eigenvalues_dtype: torch.dtype = torch.float32


@dataclass(kw_only=True)
class EigenvalueCorrectedShampooPreconditionerConfig(BaseShampooPreconditionerConfig):
    @staticmethod
    def _get_default_amortized_computation_config() -> EigendecompositionConfig:
        return DefaultEigendecompositionConfig

    amortized_computation_config: EigendecompositionConfig = field(
        default_factory=_get_default_amortized_computation_config
    )
    ignored_basis_change_dims: dict[int, list[int]] = field(default_factory=dict)
    inverse_exponent_override: dict[int, float] = field(default_factory=dict)
    factor_matrix_eigenvectors_dtype: torch.dtype = torch.float32
    corrected_eigenvalues_dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        super().__post_init__()
        stability = self.amortized_computation_config.rank_deficient_stability_config
        if not isinstance(stability, PerturbationConfig):
            raise ValueError(
                f"{type(stability).__name__} is an invalid rank_deficient_stability_config for {type(self).__name__}."
                f" Please use an instance of {PerturbationConfig.__name__} instead."
            )
        _check_orders_nonnegative(
            f"self.ignored_basis_change_dims={self.ignored_basis_change_dims}",
            self.ignored_basis_change_dims.keys(),
        )
        for order, dims in self.ignored_basis_change_dims.items():
            top = max(order - 1, 0)
            if bad := [d for d in dims if not 0 <= d <= top]:
                raise ValueError(
                    f"Invalid dimensions in self.ignored_basis_change_dims[order]={dims}: {bad}. All dimensions must be within [0, {top}]."
                )
            if len(set(dims)) != len(dims):
                raise ValueError(
                    f"Invalid ignored dimensions in self.ignored_basis_change_dims[order]={dims}. Duplicate dimensions found in {dims}. All dimensions must be unique."
                )
        _check_orders_nonnegative(
            f"self.inverse_exponent_override={self.inverse_exponent_override}",
            self.inverse_exponent_override.keys(),
        )
        for order, override in self.inverse_exponent_override.items():
            if override <= 0:
                raise ValueError(
                    f"Invalid override value in self.inverse_exponent_override[order]={override}: {override}. All overrides must be > 0."
                )


DefaultEigenvalueCorrectedShampooConfig = EigenvalueCorrectedShampooPreconditionerConfig()
DefaultSOAPConfig = EigenvalueCorrectedShampooPreconditionerConfig(
    amortized_computation_config=QREigendecompositionConfig(),
)


@dataclass(kw_only=True)
class RootInvKLShampooPreconditionerConfig(RootInvShampooPreconditionerConfig):
    """KL-Shampoo with stored inverse roots: each factor is fed the gradient already
    preconditioned along every other dim."""


@dataclass(kw_only=True)
class EigendecomposedKLShampooPreconditionerConfig(EigendecomposedShampooPreconditionerConfig):
    """KL-Shampoo with stored eigendecompositions."""


@dataclass(kw_only=True)
class SpectralDescentPreconditionerConfig(PreconditionerConfig):
    @staticmethod
    def _default_orthogonalization_config() -> OrthogonalizationConfig:
        return DefaultNewtonSchulzOrthogonalizationConfig

    orthogonalization_config: OrthogonalizationConfig = field(
        default_factory=_default_orthogonalization_config
    )


DefaultSpectralDescentPreconditionerConfig = SpectralDescentPreconditionerConfig()


@dataclass(kw_only=True)
class SignDescentPreconditionerConfig(PreconditionerConfig):
    @staticmethod
    def _default_scale_fn(grad: Tensor) -> float:
        return 1.0

    scale_fn: Callable[[Tensor], float | Tensor] = _default_scale_fn


DefaultSignDescentPreconditionerConfig = SignDescentPreconditionerConfig()


# --------------------------------------------------------------------------------------------
# Iterate averaging, weight decay.
# --------------------------------------------------------------------------------------------
@dataclass(init=False)
class IterateAveragingConfig(AbstractDataclass):
    """Base of momentum / primal-averaging schemes applied after preconditioning."""


@dataclass(kw_only=True)
class ClassicMomentumConfig(IterateAveragingConfig):
    momentum: float = 0.5
    dampening: float = 0.0
    use_nesterov: bool = False

    def __post_init__(self) -> None:
        if not 0.0 < self.momentum < 1.0:
            raise ValueError(f"Invalid self.momentum={self.momentum}. Must be within (0.0, 1.0).")
        if not 0.0 <= self.dampening < 1.0:
            raise ValueError(f"Invalid self.dampening={self.dampening}. Must be within [0.0, 1.0).")


@dataclass(kw_only=True)
class GeneralizedPrimalAveragingConfig(IterateAveragingConfig):
    eval_interp_coeff: float = 0.9
    train_interp_coeff: float = 0.8

    def __post_init__(self) -> None:
        if not 0.0 <= self.eval_interp_coeff < 1.0:
            raise ValueError(
                f"Invalid self.eval_interp_coeff={self.eval_interp_coeff}. Must be within [0.0, 1.0)."
            )
        if not 0.0 < self.train_interp_coeff <= 1.0:
            raise ValueError(
                f"Invalid self.train_interp_coeff={self.train_interp_coeff}. Must be within (0.0, 1.0]."
            )


@dataclass(kw_only=True)
class ScheduleFreeConfig(IterateAveragingConfig):
    train_interp_coeff: float = 0.8
    eval_coeff_lr_power: int = 2

    def __post_init__(self) -> None:
        if not 0.0 < self.train_interp_coeff <= 1.0:
            raise ValueError(
                f"Invalid self.train_interp_coeff={self.train_interp_coeff}. Must be within (0.0, 1.0]."
            )


@enum.unique
class WeightDecayType(enum.Enum):
    """L2: g += wd·w.  DECOUPLED: α = wd.  CORRECTED: α = wd·lr/peak_lr.  INDEPENDENT: α = wd/peak_lr."""

    L2 = "L2"
    DECOUPLED = "DECOUPLED"
    CORRECTED = "CORRECTED"
    INDEPENDENT = "INDEPENDENT"


# --------------------------------------------------------------------------------------------
# Distributed configs.
# --------------------------------------------------------------------------------------------
@dataclass
class FSDPParameterMetadata:
    """Where an original parameter sits inside this rank's FSDP1 flat-parameter shard."""

    fqn: str
    shape: torch.Size
    numel: int
    start_idx: int
    end_idx: int
    sharding_strategy: ShardingStrategy


@enum.unique
class FSDPParamAssignmentStrategy(enum.Enum):
    """DEFAULT: precondition the local shard.  REPLICATE: every rank rebuilds and preconditions
    every full parameter.  ROUND_ROBIN: each full parameter is owned by one rank."""

    DEFAULT = enum.auto()
    REPLICATE = enum.auto()
    ROUND_ROBIN = enum.auto()


@dataclass(init=False)
class DistributedConfig(AbstractDataclass):
    target_parameter_dimensionality: int | float = 1

    def __post_init__(self) -> None:
        t = self.target_parameter_dimensionality
        if isinstance(t, float) and t != math.inf:
            raise ValueError(
                f"Invalid self.target_parameter_dimensionality={t} value. Must be an integer or math.inf."
            )
        if t < 1:
            raise ValueError(f"Invalid self.target_parameter_dimensionality={t} value. Must be >= 1.")


@dataclass(kw_only=True)
class SingleDeviceDistributedConfig(DistributedConfig):
    """No optimizer-side communication."""


DefaultSingleDeviceDistributedConfig = SingleDeviceDistributedConfig()


@dataclass(kw_only=True)
class DDPDistributedConfig(DistributedConfig):
    """Blocks are shared out over groups of ``num_trainers_per_group`` ranks (-1: the local world
    size); search directions travel in ``communication_dtype``."""

    communication_dtype: torch.dtype = torch.float32
    num_trainers_per_group: int = -1
    communicate_params: bool = False

    @staticmethod
    def _get_default_load_balancing_config() -> LoadBalancingConfig:
        return LoadBalancingConfig()

    load_balancing_config: LoadBalancingConfig = field(
        default_factory=_get_default_load_balancing_config
    )


@dataclass(kw_only=True)
class FSDPDistributedConfig(DistributedConfig):
    param_to_metadata: dict[Parameter, FSDPParameterMetadata]


@dataclass(kw_only=True)
class HSDPDistributedConfig(FSDPDistributedConfig, DDPDistributedConfig):
    device_mesh: DeviceMesh


@dataclass(kw_only=True)
class FullyShardDistributedConfig(DistributedConfig):
    param_assignment_strategy: FSDPParamAssignmentStrategy = FSDPParamAssignmentStrategy.DEFAULT
    num_sub_groups: int = 1

    @staticmethod
    def _get_default_load_balancing_config() -> LoadBalancingConfig:
        return LoadBalancingConfig()

    load_balancing_config: LoadBalancingConfig = field(
        default_factory=_get_default_load_balancing_config
    )

    def __post_init__(self) -> None:
        super().__post_init__()
        if self.num_sub_groups < 1:
            raise ValueError(f"Invalid self.num_sub_groups={self.num_sub_groups}. Must be >= 1.")
        if (
            self.num_sub_groups > 1
            and self.param_assignment_strategy == FSDPParamAssignmentStrategy.DEFAULT
        ):
            raise ValueError(
                "num_sub_groups > 1 requires param_assignment_strategy != DEFAULT "
                "(REPLICATE or ROUND_ROBIN); only the lossless FSDP/HSDP "
                "distributors support param-group splitting. Got "
                f"self.num_sub_groups={self.num_sub_groups}, self.param_assignment_strategy={self.param_assignment_strategy!r}."
            )


@dataclass(kw_only=True)
class HybridShardDistributedConfig(FullyShardDistributedConfig, DDPDistributedConfig):
    device_mesh: DeviceMesh


# --------------------------------------------------------------------------------------------
# Runtime configs (constructor-only, never stored in param groups).
# --------------------------------------------------------------------------------------------
_ShampooPT2CompileConfigImpl: type = make_dataclass(
    "_ShampooPT2CompileConfigImpl",
    [
        (name, p.annotation, p.default)
        for name, p in inspect.signature(torch.compile).parameters.items()
        if name != "model"
    ],
    kw_only=True,
)


class ShampooPT2CompileConfig(_ShampooPT2CompileConfigImpl):  # type: ignore[misc, valid-type]
    """Keyword arguments of ``torch.compile`` (minus ``model``), mirrored field by field.

    Accepted for API compatibility.  The CUDA step of this library is a fixed sequence of grouped
    sm_100a launches and is not traced; when this config is given on a device without the native
    back-end, the torch step function is wrapped in ``torch.compile`` with these arguments.
    """

    def __init__(self, **kwargs: object) -> None:
        super().__init__(**kwargs)


@dataclass(kw_only=True)
class ShampooRuntimeConfig:
    eager_nan_check: bool = False


DefaultShampooRuntimeConfig = ShampooRuntimeConfig()


@dataclass(kw_only=True)
class ConcurrencyConfig:
    enable_cuda_stream_for_param_groups: bool = True


DefaultConcurrencyConfig = ConcurrencyConfig()


@dataclass(kw_only=True)
class NativeRuntimeConfig:
    """Selection of the sm_100a execution path (not part of the reference API).

    backend:   ``"auto"`` uses the native kernels for CUDA parameter groups whose configuration
               they cover and the torch path otherwise; ``"torch"`` forces the torch path;
               ``"native"`` raises if a group cannot run natively.
    gemm_mode: ``"tf32x3"`` splits fp32 operands into two tf32 terms and issues three tensor-core
               products (fp32-grade accuracy); ``"tf32"`` issues one (relative error of a product
               about 1e-3) and keeps one operand array instead of a (hi, lo) pair, which halves the
               engine's operand arrays and mirrors (``DistributedShampoo.native_memory_report()``).
    comm_path: ``"nccl"`` uses ``torch.distributed`` collectives; ``"p2p"`` lets the kernels
               load/store peer memory directly over NVLink: the direction epilogue stores each
               block's search direction into every peer's gather buffer (all-gather fused into
               the producing kernel).
    fuse_gradient_reduction: with ``comm_path="p2p"`` and the DDP distributor, gradients are
               accumulated by autograd straight into peer-addressable memory and each block's
               owner sums its peers' gradient blocks inside the prologue kernel (reduce-scatter
               fused into the factor update).  The model must then NOT be wrapped in
               ``DistributedDataParallel`` and ``zero_grad(set_to_none=False)`` must be used.
    fuse_direction_push: with ``comm_path="p2p"`` and root-inverse Shampoo, steps that need no
               owner-side state after the preconditioner (no classic momentum, no primal averaging)
               store the search directions into every peer's gather buffer from the epilogue of
               the last preconditioner GEMM, tile by tile, cast to the communication dtype; every
               rank then finishes ``W <- W - lr (scale P + wd W)`` itself.  Other steps use the
               pointwise epilogue kernel for the stores.  Off by default: on two B200s the 64-byte
               row segments stored from the GEMM epilogue lengthen it more than the separate
               epilogue kernel costs (5.5 ms against 4.9 ms for 32 blocks of 2048 x 2048).
    """

    backend: str = "auto"
    gemm_mode: str = "tf32x3"
    comm_path: str = "nccl"
    fuse_gradient_reduction: bool = False
    fuse_direction_push: bool = False

    def __post_init__(self) -> None:
        if self.backend not in ("auto", "torch", "native"):
            raise ValueError(f"Invalid backend {self.backend!r}. Must be auto, torch or native.")
        if self.gemm_mode not in ("tf32x3", "tf32"):
            raise ValueError(f"Invalid gemm_mode {self.gemm_mode!r}. Must be tf32x3 or tf32.")
        if self.comm_path not in ("nccl", "p2p"):
            raise ValueError(f"Invalid comm_path {self.comm_path!r}. Must be nccl or p2p.")
        if self.fuse_gradient_reduction and self.comm_path != "p2p":
            raise ValueError("fuse_gradient_reduction=True requires comm_path='p2p'.")


DefaultNativeRuntimeConfig = NativeRuntimeConfig()
