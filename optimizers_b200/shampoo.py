"""``DistributedShampoo``: the optimizer runtime.

Per parameter group the constructor builds, in this order: the distributor (blocking and
ownership), empty per-block state dicts, the Shampoo-family preconditioner list, the grafting
list, the step counter, learning-rate tensors, filtered-gradient state, iterate-averaging state,
and finally the execution plan: a native sm_100a engine (grouped launches over a device block
table) when the group is on a B200 and its configuration is covered, else the torch step.

One step of a group, with t the incremented step count:

1. L2 regularisation ``G += wd·W``.
2. Factor / second-moment statistics; at refresh steps the amortised matrix functions.
3. Filtered gradient (EMA with β1, optional separate β3 for the applied estimate, bias corrected).
4. Search direction: grafting only before ``start_preconditioning_step``; afterwards the
   Shampoo direction rescaled per block to the grafting direction's norm.
5. Decoupled-style weight decay, classic momentum, multiplication by ``-lr``, primal averaging.
6. ``distributor.update_params`` (local add, or a collective).

Reference counterpart: ``distributed_shampoo/distributed_shampoo.py`` (constructor :361-561,
state instantiation :564-1012, masking :1014-1079, step pipeline :1082-1722, train/eval
:1729-1797, checkpoint hooks :1803-1996).
"""

from __future__ import annotations

import dataclasses
import logging
import math
from collections.abc import Callable
from contextlib import nullcontext
from types import LambdaType
from typing import Any

import torch
from torch.optim.optimizer import Optimizer, ParamsT, StateDict

from optimizers_b200.config import (
    AdaGradPreconditionerConfig,
    AdamPreconditionerConfig,
    BaseShampooPreconditionerConfig,
    BETA3,
    BETAS,
    ClassicMomentumConfig,
    ConcurrencyConfig,
    CUDA_STREAM,
    DDPDistributedConfig,
    DefaultConcurrencyConfig,
    DefaultNativeRuntimeConfig,
    DefaultShampooConfig,
    DefaultShampooRuntimeConfig,
    DefaultSingleDeviceDistributedConfig,
    DISTRIBUTED_CONFIG,
    DistributedConfig,
    DISTRIBUTOR,
    EigendecomposedKLShampooPreconditionerConfig,
    EigendecomposedShampooPreconditionerConfig,
    EigendecompositionConfig,
    EigenvalueCorrectedShampooPreconditionerConfig,
    EPSILON,
    EVAL_INTERP_COEFF,
    FILTERED_GRAD,
    FILTERED_GRAD_LIST,
    FSDPDistributedConfig,
    FSDPParamAssignmentStrategy,
    FullyShardDistributedConfig,
    GeneralizedPrimalAveragingConfig,
    GRAFTING_CONFIG,
    GRAFTING_PRECONDITIONER_LIST,
    HSDPDistributedConfig,
    HybridShardDistributedConfig,
    ITERATE_AVERAGING_CONFIG,
    IterateAveragingConfig,
    LR,
    LR_CPU_PINNED,
    LR_SUM,
    LR_TENSOR,
    MASKED_BLOCKED_GRADS,
    MASKED_BLOCKED_PARAMS,
    MASKED_FILTERED_GRAD_LIST,
    MASKED_MOMENTUM_BUFFER_LIST,
    MASKED_WEIGHT_BUFFER_LIST,
    MAX_PRECONDITIONER_DIM,
    MOMENTUM_BUFFER,
    MOMENTUM_BUFFER_LIST,
    NativeRuntimeConfig,
    PARAMS,
    PEAK_LR,
    PRECONDITION_FREQUENCY,
    PRECONDITIONER_CONFIG,
    PreconditionerConfig,
    PREVIOUS_GRAD_SELECTOR,
    PseudoInverseConfig,
    RMSpropPreconditionerConfig,
    RootInvKLShampooPreconditionerConfig,
    RootInvShampooPreconditionerConfig,
    ScheduleFreeConfig,
    SGDPreconditionerConfig,
    SHAMPOO_PRECONDITIONER_LIST,
    ShampooPT2CompileConfig,
    ShampooRuntimeConfig,
    SignDescentPreconditionerConfig,
    SingleDeviceDistributedConfig,
    SpectralDescentPreconditionerConfig,
    START_PRECONDITIONING_STEP,
    STEP,
    TRAIN_INTERP_COEFF,
    TRAIN_MODE,
    USE_BIAS_CORRECTION,
    USE_PIN_MEMORY,
    WEIGHT_BUFFER,
    WEIGHT_BUFFER_LIST,
    WEIGHT_DECAY,
    WEIGHT_DECAY_TYPE,
    WeightDecayType,
)
from optimizers_b200.parallel.base import Distributor, DistributorInterface
from optimizers_b200.preconditioner.base import PreconditionerList
from optimizers_b200.preconditioner.kronecker import (
    EigendecomposedKLShampooPreconditionerList,
    EigendecomposedShampooPreconditionerList,
    EigenvalueCorrectedShampooPreconditionerList,
    RootInvKLShampooPreconditionerList,
    RootInvShampooPreconditionerList,
)
from optimizers_b200.preconditioner.simple import (
    AdagradPreconditionerList,
    SGDPreconditionerList,
    SignDescentPreconditionerList,
    SpectralDescentPreconditionerList,
)
from optimizers_b200.utils.blocking import compress_list, split_param_groups
from optimizers_b200.utils.state import extract_state_dict_content, update_param_state_dict_object

logger: logging.Logger = logging.getLogger(__name__)

NATIVE_ENGINE = "native_engine"

_KRONECKER_LISTS: dict[type, type] = {
    RootInvShampooPreconditionerConfig: RootInvShampooPreconditionerList,
    EigendecomposedShampooPreconditionerConfig: EigendecomposedShampooPreconditionerList,
    EigenvalueCorrectedShampooPreconditionerConfig: EigenvalueCorrectedShampooPreconditionerList,
    RootInvKLShampooPreconditionerConfig: RootInvKLShampooPreconditionerList,
    EigendecomposedKLShampooPreconditionerConfig: EigendecomposedKLShampooPreconditionerList,
}


def diagonal_preconditioner_hyperparameters(cfg: AdaGradPreconditionerConfig) -> tuple[float, float, bool]:
    """``(beta2, weighting_factor, use_bias_correction)`` of a diagonal preconditioner config.
    The most derived type decides, except that ``drop_weighting_factor_on_gsquare`` turns any
    RMSprop/Adam config into an unweighted, uncorrected accumulator."""
    if isinstance(cfg, RMSpropPreconditionerConfig):
        if cfg.drop_weighting_factor_on_gsquare:
            return cfg.beta2, 1.0, False
        return cfg.beta2, 1 - cfg.beta2, isinstance(cfg, AdamPreconditionerConfig)
    return 1.0, 1.0, False


def _check_group(group: dict[str, Any]) -> None:
    """Validate (and normalise in place) the hyperparameters of one parameter group."""
    if not group[LR] >= 0.0:
        raise ValueError(f"Invalid param_group[LR]={group[LR]}. Must be >= 0.0.")
    beta1, beta2 = group[BETAS]
    if not 0.0 <= beta1 < 1.0:
        raise ValueError(f"Invalid param_group[BETAS][0]={beta1}. Must be in [0.0, 1.0).")
    if not 0.0 <= beta2 <= 1.0:
        raise ValueError(f"Invalid param_group[BETAS][1]={beta2}. Must be in [0.0, 1.0].")
    if group[BETA3] == -1.0:
        group[BETA3] = beta1
    elif not 0.0 <= group[BETA3] < 1.0:
        raise ValueError(f"Invalid param_group[BETA3]={group[BETA3]}. Must be in [0.0, 1.0).")

    pc = group[PRECONDITIONER_CONFIG]
    uses_pseudo_inverse = (
        isinstance(pc, BaseShampooPreconditionerConfig)
        and isinstance(pc.amortized_computation_config, EigendecompositionConfig)
        and isinstance(pc.amortized_computation_config.rank_deficient_stability_config, PseudoInverseConfig)
    )
    if uses_pseudo_inverse:
        if group[EPSILON] != 0.0:
            raise ValueError(
                f"Invalid param_group[EPSILON]={group[EPSILON]}. Must be == 0.0 when PseudoInverseConfig is used."
            )
    elif not group[EPSILON] > 0.0:
        raise ValueError(f"Invalid param_group[EPSILON]={group[EPSILON]}. Must be > 0.0.")
    if not group[WEIGHT_DECAY] >= 0.0:
        raise ValueError(f"Invalid param_group[WEIGHT_DECAY]={group[WEIGHT_DECAY]}. Must be >= 0.0.")
    if (
        group[WEIGHT_DECAY_TYPE] in (WeightDecayType.CORRECTED, WeightDecayType.INDEPENDENT)
        and not group[PEAK_LR] > 0.0
    ):
        raise ValueError(
            f"Invalid param_group[PEAK_LR]={group[PEAK_LR]}. Must be > 0.0 when using WeightDecayType.CORRECTED or WeightDecayType.INDEPENDENT."
        )
    mpd = group[MAX_PRECONDITIONER_DIM]
    if isinstance(mpd, float) and mpd != math.inf:
        raise ValueError(f"Invalid param_group[MAX_PRECONDITIONER_DIM]={mpd}. Must be an integer or math.inf.")
    if not mpd >= 1:
        raise ValueError(f"Invalid param_group[MAX_PRECONDITIONER_DIM]={mpd}. Must be >= 1.")
    if not group[PRECONDITION_FREQUENCY] >= 1:
        raise ValueError(
            f"Invalid param_group[PRECONDITION_FREQUENCY]={group[PRECONDITION_FREQUENCY]}. Must be >= 1."
        )
    if not group[START_PRECONDITIONING_STEP] >= -1:
        raise ValueError(
            f"Invalid param_group[START_PRECONDITIONING_STEP]={group[START_PRECONDITIONING_STEP]}. Must be >= -1."
        )

    if isinstance(pc, (SignDescentPreconditionerConfig, SpectralDescentPreconditionerConfig)):
        name = type(pc).__name__
        logger.warning(f"param_group[BETAS][1]={beta2} does not have any effect when {name} is used.")
        logger.warning(f"param_group[EPSILON]={group[EPSILON]} does not have any effect when {name} is used.")
        logger.warning(
            f"param_group[PRECONDITION_FREQUENCY]={group[PRECONDITION_FREQUENCY]} does not have any effect when {name} is used. Setting precondition_frequency to 1..."
        )
        group[PRECONDITION_FREQUENCY] = 1
    if (
        isinstance(pc, SpectralDescentPreconditionerConfig)
        and group[DISTRIBUTED_CONFIG].target_parameter_dimensionality != 2
    ):
        logger.warning(
            f"param_group[DISTRIBUTED_CONFIG].target_parameter_dimensionality={group[DISTRIBUTED_CONFIG].target_parameter_dimensionality} is not equal to 2. Setting target_parameter_dimensionality to 2..."
        )
        group[DISTRIBUTED_CONFIG].target_parameter_dimensionality = 2

    if group[START_PRECONDITIONING_STEP] == -1:
        group[START_PRECONDITIONING_STEP] = group[PRECONDITION_FREQUENCY]
        logger.warning(
            f"start_preconditioning_step set to -1. Setting start_preconditioning_step equal to param_group[PRECONDITION_FREQUENCY]={group[PRECONDITION_FREQUENCY]} by default."
        )
    if group[START_PRECONDITIONING_STEP] < group[PRECONDITION_FREQUENCY]:
        raise ValueError(
            f"Invalid param_group[START_PRECONDITIONING_STEP]={group[START_PRECONDITIONING_STEP]}. Must be >= param_group[PRECONDITION_FREQUENCY]={group[PRECONDITION_FREQUENCY]}."
        )


def _is_primal_averaging(cfg: IterateAveragingConfig | None) -> bool:
    return isinstance(cfg, (GeneralizedPrimalAveragingConfig, ScheduleFreeConfig))


class DistributedShampoo(Optimizer):
    """Distributed Shampoo.

    Args mirror the reference constructor; every argument up to ``preconditioner_config`` also
    becomes a key of each ``param_group`` (plus ``peak_lr``), so it can differ between groups.

        params, lr=1e-2, betas=(0.9, 1.0), beta3=-1.0 (use beta1), epsilon=1e-12,
        weight_decay=0.0, weight_decay_type=DECOUPLED, max_preconditioner_dim=1024,
        precondition_frequency=1, start_preconditioning_step=-1 (use precondition_frequency),
        use_bias_correction=True, iterate_averaging_config=None, grafting_config=None,
        use_pin_memory=False, shampoo_pt2_compile_config=None,
        distributed_config=SingleDeviceDistributedConfig(),
        preconditioner_config=RootInvShampooPreconditionerConfig(),
        shampoo_runtime_config, concurrency_config,
        native_runtime_config   (new: sm_100a back-end selection)
    """

    def __init__(
        self,
        params: ParamsT,
        lr: float = 1e-2,
        betas: tuple[float, float] = (0.9, 1.0),
        beta3: float = -1.0,
        epsilon: float = 1e-12,
        weight_decay: float = 0.0,
        weight_decay_type: WeightDecayType = WeightDecayType.DECOUPLED,
        max_preconditioner_dim: int | float = 1024,
        precondition_frequency: int = 1,
        start_preconditioning_step: int = -1,
        use_bias_correction: bool = True,
        iterate_averaging_config: IterateAveragingConfig | None = None,
        grafting_config: PreconditionerConfig | None = None,
        use_pin_memory: bool = False,
        shampoo_pt2_compile_config: ShampooPT2CompileConfig | None = None,
        distributed_config: DistributedConfig = DefaultSingleDeviceDistributedConfig,
        preconditioner_config: PreconditionerConfig = DefaultShampooConfig,
        shampoo_runtime_config: ShampooRuntimeConfig = DefaultShampooRuntimeConfig,
        concurrency_config: ConcurrencyConfig = DefaultConcurrencyConfig,
        native_runtime_config: NativeRuntimeConfig = DefaultNativeRuntimeConfig,
    ) -> None:
        super().__init__(
            params,
            {
                LR: lr,
                BETAS: betas,
                BETA3: beta3,
                EPSILON: epsilon,
                WEIGHT_DECAY: weight_decay,
                PEAK_LR: lr,
                WEIGHT_DECAY_TYPE: weight_decay_type,
                MAX_PRECONDITIONER_DIM: max_preconditioner_dim,
                PRECONDITION_FREQUENCY: precondition_frequency,
                START_PRECONDITIONING_STEP: start_preconditioning_step,
                USE_BIAS_CORRECTION: use_bias_correction,
                ITERATE_AVERAGING_CONFIG: iterate_averaging_config,
                GRAFTING_CONFIG: grafting_config,
                USE_PIN_MEMORY: use_pin_memory,
                DISTRIBUTED_CONFIG: distributed_config,
                PRECONDITIONER_CONFIG: preconditioner_config,
            },
        )
        self.register_state_dict_post_hook(self._post_state_dict_hook)
        self.register_load_state_dict_pre_hook(self._pre_load_state_dict_hook)
        self.register_load_state_dict_post_hook(self._post_load_state_dict_hook)

        self.param_groups[:] = split_param_groups(self.param_groups)
        for i, group in enumerate(self.param_groups):
            logger.info(f"Checking param_group {i} hyperparameters...")
            _check_group(group)

        self._shampoo_pt2_compile_config = shampoo_pt2_compile_config
        self._runtime_config = shampoo_runtime_config
        self._concurrency_config = concurrency_config
        self._native_runtime_config = native_runtime_config
        self._per_group_state_lists: list[dict[str, Any]] = [{} for _ in self.param_groups]

        # Order matters: blocks first, then the empty state slots the other builders fill.
        self._instantiate_distributor()
        self._initialize_blocked_parameters_state()
        self._instantiate_shampoo_preconditioner_list()
        self._instantiate_grafting()
        self._instantiate_steps()
        self._instantiate_lr_tensors()
        self._instantiate_filtered_grads()
        self._instantiate_iterate_averaging()
        self._instantiate_per_group_step(shampoo_pt2_compile_config)

    # ------------------------------------------------------------------------------------------
    # Construction
    # ------------------------------------------------------------------------------------------
    def _groups(self):
        return zip(self._per_group_state_lists, self.param_groups, strict=True)

    def _select_distributor_class(self, distributed_config: DistributedConfig) -> type[DistributorInterface]:
        """Map a group's ``DistributedConfig`` to its distributor class.  Subclasses override this
        to add their own config types and defer to ``super()`` for the rest."""
        from optimizers_b200 import parallel as P  # deferred: the distributors import torch.distributed

        strategy = getattr(distributed_config, "param_assignment_strategy", None)
        lossless = strategy in (FSDPParamAssignmentStrategy.REPLICATE, FSDPParamAssignmentStrategy.ROUND_ROBIN)
        # Most derived config types first: HSDP and HybridShard also are DDP configs.
        match distributed_config:
            case SingleDeviceDistributedConfig():
                return Distributor
            case HSDPDistributedConfig():
                return P.HSDPDistributor
            case HybridShardDistributedConfig():
                return P.HybridShardLosslessDistributor if lossless else P.HybridShardDistributor
            case DDPDistributedConfig():
                return P.DDPDistributor
            case FSDPDistributedConfig():
                return P.FSDPDistributor
            case FullyShardDistributedConfig():
                return P.FullyShardLosslessDistributor if lossless else P.FullyShardDistributor
            case _:
                raise NotImplementedError(f"{distributed_config=} not supported!")

    @torch.no_grad()
    def _instantiate_distributor(self) -> None:
        for rec, group in self._groups():
            if not group[PARAMS]:
                raise ValueError(f"Shampoo got an empty parameter group={group}")
            cls = self._select_distributor_class(group[DISTRIBUTED_CONFIG])
            nrc = self._native_runtime_config
            # The lossless distributors' exchange follows the native comm path (peer-memory pushes
            # instead of all_to_all) unless the torch back-end was asked for.
            from optimizers_b200.parallel import a2a
            from optimizers_b200.parallel.a2a import exchange_comm_path

            on_gpu = group[PARAMS][0].device.type in a2a._PEER_DEVICE_TYPES

            with exchange_comm_path(nrc.comm_path if (nrc.backend != "torch" and on_gpu) else "nccl"):
                rec[DISTRIBUTOR] = cls(group, self._runtime_config)
            if not rec[DISTRIBUTOR].local_blocked_params:
                logger.warning(
                    "There is no params assigned to the current rank. "
                    f"In DDP Shampoo, this may happen when the value of num_trainers_per_group field in group[DISTRIBUTED_CONFIG]={group[DISTRIBUTED_CONFIG]} "
                    "is more than the number of global blocked params so some trainers get assigned no blocked params. "
                    "This will cause idle ranks. Please check the num_trainers_per_group setting and consider reducing it. "
                    "Similarly, in FSDP lossless Shampoo, this can happen under ROUND_ROBIN assignment strategy and "
                    "when the optimizer shard group size is larger than the number of params."
                )
            rec[MASKED_BLOCKED_PARAMS] = rec[DISTRIBUTOR].local_blocked_params
            rec[PREVIOUS_GRAD_SELECTOR] = None

    @torch.no_grad()
    def _initialize_blocked_parameters_state(self) -> None:
        for rec in self._per_group_state_lists:
            for info in rec[DISTRIBUTOR].local_block_info_list:
                slots = self.state[info.param]
                block_id = info.composable_block_ids[1]
                assert block_id not in slots, "Block state must not exist before the distributor is built."
                slots[block_id] = {}

    @torch.no_grad()
    def _preconditioner_config_to_list_cls(
        self, state_lists: dict[str, Any], group: dict[str, Any], preconditioner_config: PreconditionerConfig | None
    ) -> PreconditionerList | None:
        dist = state_lists[DISTRIBUTOR]
        blocks, infos = dist.local_blocked_params, dist.local_block_info_list
        cfg = preconditioner_config
        if cfg is None:
            return None
        if isinstance(cfg, SGDPreconditionerConfig):
            return SGDPreconditionerList(block_list=blocks)
        if isinstance(cfg, AdaGradPreconditionerConfig):
            beta2, weight, bias_correction = diagonal_preconditioner_hyperparameters(cfg)
            return AdagradPreconditionerList(
                block_list=blocks,
                state=self.state,
                block_info_list=infos,
                beta2=beta2,
                weighting_factor=weight,
                epsilon=cfg.epsilon,
                use_bias_correction=bias_correction,
            )
        if type(cfg) in _KRONECKER_LISTS:
            beta2 = group[BETAS][1]
            unweighted = cfg.drop_weighting_factor_on_gsquare or beta2 == 1.0
            return _KRONECKER_LISTS[type(cfg)](
                block_list=blocks,
                preconditioner_config=cfg,
                state=self.state,
                block_info_list=infos,
                beta2=beta2,
                weighting_factor=1.0 if unweighted else 1 - beta2,
                epsilon=group[EPSILON],
                use_bias_correction=group[USE_BIAS_CORRECTION],
            )
        if isinstance(cfg, SignDescentPreconditionerConfig):
            return SignDescentPreconditionerList(block_list=blocks, preconditioner_config=cfg)
        if isinstance(cfg, SpectralDescentPreconditionerConfig):
            assert group[DISTRIBUTED_CONFIG].target_parameter_dimensionality == 2, (
                f"group[DISTRIBUTED_CONFIG].target_parameter_dimensionality={group[DISTRIBUTED_CONFIG].target_parameter_dimensionality} must be 2 when using SpectralDescentPreconditionerConfig."
            )
            nrc = self._native_runtime_config
            return SpectralDescentPreconditionerList(
                block_list=blocks, preconditioner_config=cfg,
                native_gemm_mode=None if nrc.backend == "torch" else nrc.gemm_mode,
            )
        raise NotImplementedError(f"preconditioner_config={cfg!r} not supported!")

    @torch.no_grad()
    def _instantiate_shampoo_preconditioner_list(self) -> None:
        for rec, group in self._groups():
            assert group[PRECONDITIONER_CONFIG] is not None, (
                f"group[PRECONDITIONER_CONFIG]={group[PRECONDITIONER_CONFIG]} is None. Please check the instantiation of DistributedShampoo."
            )
            rec[SHAMPOO_PRECONDITIONER_LIST] = self._preconditioner_config_to_list_cls(
                rec, group, group[PRECONDITIONER_CONFIG]
            )

    @torch.no_grad()
    def _instantiate_grafting(self) -> None:
        for rec, group in self._groups():
            rec[GRAFTING_PRECONDITIONER_LIST] = self._preconditioner_config_to_list_cls(
                rec, group, group[GRAFTING_CONFIG]
            )

    @torch.no_grad()
    def _instantiate_steps(self) -> None:
        # One CPU counter per group (no device sync to read it), aliased under every parameter
        # of the group so that the checkpoint key set does not depend on how parameters are
        # spread over groups, sub-groups or ranks.
        for rec, group in self._groups():
            rec[STEP] = torch.tensor(0, dtype=torch.int64, device="cpu")
            for p in group[PARAMS]:
                self.state[p][STEP] = rec[STEP]

    @torch.no_grad()
    def _instantiate_lr_tensors(self) -> None:
        # Persistent tensors: lr reaches the device by one async copy per step, and the
        # interpolation coefficients stay tensors so that changing values need no host sync.
        for rec, group in self._groups():
            device = group[PARAMS][0].device
            rec[LR_TENSOR] = torch.empty((), dtype=torch.float, device=device)
            rec[LR_CPU_PINNED] = torch.empty((), dtype=torch.float, pin_memory=group[USE_PIN_MEMORY])
            rec[TRAIN_INTERP_COEFF] = torch.zeros((), dtype=torch.float, device=device)
            rec[EVAL_INTERP_COEFF] = torch.zeros((), dtype=torch.float, device=device)

    def _allocate_block_buffer_list(
        self, state_lists: dict[str, Any], buffer_key: str, list_key: str, masked_list_key: str, init_from_param: bool = False
    ) -> None:
        dist = state_lists[DISTRIBUTOR]
        buffers = []
        for block, info in zip(dist.local_blocked_params, dist.local_block_info_list, strict=True):
            block_id = info.composable_block_ids[1]
            assert block_id in self.state[info.param], f"block_index={block_id} has no state slot."
            slot = self.state[info.param][block_id]
            slot[buffer_key] = info.allocate_zeros_tensor(size=block.size(), dtype=block.dtype, device=block.device)
            local = info.get_tensor(slot[buffer_key])
            if init_from_param:
                local.copy_(block)
            buffers.append(local)
        state_lists[list_key] = buffers
        state_lists[masked_list_key] = buffers

    @torch.no_grad()
    def _instantiate_filtered_grads(self) -> None:
        for rec, group in self._groups():
            if group[BETAS][0] != 0.0:
                self._allocate_block_buffer_list(rec, FILTERED_GRAD, FILTERED_GRAD_LIST, MASKED_FILTERED_GRAD_LIST)

    @torch.no_grad()
    def _instantiate_iterate_averaging(self) -> None:
        for rec, group in self._groups():
            cfg = group[ITERATE_AVERAGING_CONFIG]
            if cfg is None:
                continue
            if isinstance(cfg, ClassicMomentumConfig):
                self._allocate_block_buffer_list(
                    rec, MOMENTUM_BUFFER, MOMENTUM_BUFFER_LIST, MASKED_MOMENTUM_BUFFER_LIST
                )
            elif _is_primal_averaging(cfg):
                # z starts at the current parameters (the y sequence the gradients are taken at).
                self._allocate_block_buffer_list(
                    rec, WEIGHT_BUFFER, WEIGHT_BUFFER_LIST, MASKED_WEIGHT_BUFFER_LIST, init_from_param=True
                )
                rec[LR_SUM] = torch.tensor(0.0, dtype=torch.float, device=group[PARAMS][0].device)
                rec[TRAIN_MODE] = torch.tensor(True, dtype=torch.bool, device="cpu")
                for p in group[PARAMS]:
                    self.state[p][TRAIN_MODE] = rec[TRAIN_MODE]
                    self.state[p][LR_SUM] = rec[LR_SUM]
            else:
                raise NotImplementedError(
                    f"group[ITERATE_AVERAGING_CONFIG]={cfg!r} is not supported! "
                    "Supported configs: ClassicMomentumConfig, GeneralizedPrimalAveragingConfig, ScheduleFreeConfig."
                )

    @torch.no_grad()
    def _instantiate_per_group_step(self, shampoo_pt2_compile_config: ShampooPT2CompileConfig | None) -> None:
        self._per_group_step: Callable[..., None] = self._per_group_step_impl
        if shampoo_pt2_compile_config is not None:
            self._per_group_step = torch.compile(
                self._per_group_step_impl, **dataclasses.asdict(shampoo_pt2_compile_config)
            )
            logger.info(f"DistributedShampoo optimizer initialization is using shampoo_pt2_compile_config={shampoo_pt2_compile_config}")

        # Native engines: one per group whose configuration the sm_100a kernels cover.
        from optimizers_b200.native_engine import maybe_build_native_engine

        for rec, group in self._groups():
            rec[NATIVE_ENGINE] = maybe_build_native_engine(self, rec, group, self._native_runtime_config)

        all_cuda = all(g[PARAMS][0].device.type == "cuda" for g in self.param_groups)
        self._use_cuda_streams = self._concurrency_config.enable_cuda_stream_for_param_groups and all_cuda
        if self._use_cuda_streams:
            for i, (rec, group) in enumerate(self._groups()):
                rec[CUDA_STREAM] = torch.cuda.Stream(device=group[PARAMS][0].device)
                logger.info("param_group_%d: stream_id=%s", i, rec[CUDA_STREAM].stream_id)

    def native_coverage(self) -> list[str]:
        """Per parameter group: ``"native"`` when its steps run on the sm_100a engine, else
        ``"torch: <why>"`` (what ``backend="native"`` would have raised)."""
        return [
            "native" if rec.get(NATIVE_ENGINE) is not None
            else f"torch: {rec.get('native_engine_fallback_reason', 'no engine was built')}"
            for rec, _ in self._groups()
        ]

    def native_memory_report(self) -> list[dict[str, int] | None]:
        """Per parameter group: the device bytes its sm_100a engine keeps, by purpose (see
        ``NativeGroupEngine.memory_report``), or None where the group runs the torch step."""
        return [
            rec[NATIVE_ENGINE].memory_report() if rec.get(NATIVE_ENGINE) is not None else None
            for rec, _ in self._groups()
        ]

    # ------------------------------------------------------------------------------------------
    # Masking (blocks without a gradient drop out of every per-block list)
    # ------------------------------------------------------------------------------------------
    @staticmethod
    @torch.no_grad()
    def _mask_state_lists(state_lists: dict[str, Any], group: dict[str, Any], shampoo_pt2_enabled: bool = False) -> None:
        rec = state_lists
        selector = rec[DISTRIBUTOR].local_grad_selector
        previous = rec[PREVIOUS_GRAD_SELECTOR]
        if selector == previous:
            return
        if previous is not None and shampoo_pt2_enabled:
            changed = [i for i, (a, b) in enumerate(zip(selector, previous, strict=True)) if a != b]
            logger.warning(
                "PT2 will recompile because the gradient selection of model parameters have changed from the previous step. "
                "Possible reasons include some gradients are None. If this is not intended, please check the data and/or model.\n"
                f"Details:\n- Current step: {rec[STEP].item()}\n- Changed gradient selector indices: {changed}"
            )
        rec[PREVIOUS_GRAD_SELECTOR] = selector
        rec[MASKED_BLOCKED_PARAMS] = rec[DISTRIBUTOR].local_masked_blocked_params
        rec[SHAMPOO_PRECONDITIONER_LIST].compress_preconditioner_list(local_grad_selector=selector)
        if group[GRAFTING_CONFIG] is not None:
            rec[GRAFTING_PRECONDITIONER_LIST].compress_preconditioner_list(local_grad_selector=selector)
        for full_key, masked_key in (
            (FILTERED_GRAD_LIST, MASKED_FILTERED_GRAD_LIST),
            (WEIGHT_BUFFER_LIST, MASKED_WEIGHT_BUFFER_LIST),
            (MOMENTUM_BUFFER_LIST, MASKED_MOMENTUM_BUFFER_LIST),
        ):
            if full_key in rec:
                rec[masked_key] = compress_list(rec[full_key], selector)
        if rec.get(NATIVE_ENGINE) is not None:
            rec[NATIVE_ENGINE].on_selector_change(selector)

    # ------------------------------------------------------------------------------------------
    # The torch step pipeline
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    @torch.compiler.disable
    def _precondition_and_grafting(
        self, state_lists, masked_filtered_grad_list, use_grafting_method: bool, grafting_config_not_none: bool
    ) -> tuple[torch.Tensor, ...]:
        if use_grafting_method:
            return state_lists[GRAFTING_PRECONDITIONER_LIST].precondition(masked_grad_list=masked_filtered_grad_list)
        directions = state_lists[SHAMPOO_PRECONDITIONER_LIST].precondition(masked_grad_list=masked_filtered_grad_list)
        if grafting_config_not_none:
            graft_norms = torch._foreach_norm(
                state_lists[GRAFTING_PRECONDITIONER_LIST].precondition(masked_grad_list=masked_filtered_grad_list)
            )
            own_norms = torch._foreach_norm(directions)
            torch._foreach_add_(own_norms, 1e-16)
            torch._foreach_div_(graft_norms, own_norms)
            torch._foreach_mul_(directions, graft_norms)
        return directions

    @torch.no_grad()
    def _add_l2_regularization(self, state_lists, weight_decay: float, weight_decay_type: WeightDecayType) -> None:
        if weight_decay != 0.0 and weight_decay_type == WeightDecayType.L2:
            torch._foreach_add_(state_lists[MASKED_BLOCKED_GRADS], state_lists[MASKED_BLOCKED_PARAMS], alpha=weight_decay)

    @torch.no_grad()
    def _update_preconditioners(self, state_lists, step, perform_amortized_computation: bool, grafting_config_not_none: bool) -> None:
        state_lists[SHAMPOO_PRECONDITIONER_LIST].update_preconditioners(
            masked_grad_list=state_lists[MASKED_BLOCKED_GRADS],
            step=step,
            perform_amortized_computation=perform_amortized_computation,
        )
        if grafting_config_not_none:
            state_lists[GRAFTING_PRECONDITIONER_LIST].update_preconditioners(
                masked_grad_list=state_lists[MASKED_BLOCKED_GRADS], step=step
            )

    @torch.no_grad()
    def _compute_filtered_grad_list(self, state_lists, step, beta1: float, beta3: float, use_bias_correction: bool):
        grads = state_lists[MASKED_BLOCKED_GRADS]
        if beta1 == 0.0:
            return grads
        ema = state_lists[MASKED_FILTERED_GRAD_LIST]
        # With a separate β3 the applied estimate mixes the *old* EMA with the new gradient.
        applied = torch._foreach_lerp(ema, grads, weight=1 - beta3) if beta3 != beta1 else ema
        torch._foreach_lerp_(ema, grads, weight=1 - beta1)
        if use_bias_correction:
            applied = torch._foreach_div(applied, 1.0 - beta3 * beta1 ** (step - 1))
        return applied

    @torch.no_grad()
    def _apply_weight_decay(
        self, state_lists, masked_blocked_search_directions, lr, weight_decay: float, peak_lr: float,
        weight_decay_type: WeightDecayType, iterate_averaging_enabled: bool,
    ) -> None:
        """Without primal averaging the decay joins the search direction (``P += α·W``) so that it
        travels through the distributor's collective and reaches every rank's copy; with primal
        averaging ``Z`` is shrunk instead, because ``P`` feeds the averaging update."""
        if weight_decay == 0.0 or weight_decay_type == WeightDecayType.L2:
            return
        match weight_decay_type:
            case WeightDecayType.DECOUPLED:
                alpha = weight_decay
            case WeightDecayType.CORRECTED:
                alpha = weight_decay * state_lists[LR_CPU_PINNED].item() / peak_lr
            case WeightDecayType.INDEPENDENT:
                alpha = weight_decay / peak_lr
            case _:
                raise ValueError(f"Invalid weight decay type: weight_decay_type={weight_decay_type}!")
        if iterate_averaging_enabled:
            torch._foreach_mul_(state_lists[MASKED_WEIGHT_BUFFER_LIST], 1 - lr * alpha)
        else:
            torch._foreach_add_(masked_blocked_search_directions, state_lists[MASKED_BLOCKED_PARAMS], alpha=alpha)

    @torch.no_grad()
    def _apply_classic_momentum(self, state_lists, masked_blocked_search_directions, momentum_param: float, dampening: float, use_nesterov: bool) -> None:
        """M ← μM + (1-damp)P;  P ← (1-damp)P + μM (Nesterov) or P ← M."""
        buf = state_lists[MASKED_MOMENTUM_BUFFER_LIST]
        torch._foreach_mul_(buf, momentum_param)
        torch._foreach_add_(buf, masked_blocked_search_directions, alpha=1 - dampening)
        if use_nesterov:
            torch._foreach_mul_(masked_blocked_search_directions, 1 - dampening)
            torch._foreach_add_(masked_blocked_search_directions, buf, alpha=momentum_param)
        else:
            torch._foreach_copy_(masked_blocked_search_directions, buf)

    @staticmethod
    @torch.no_grad()
    def _get_train_and_eval_interp_coeffs(iterate_averaging_config, lr: torch.Tensor | None, state_lists):
        """Fill and return the persistent (μy, μx) tensors.  Schedule-Free derives μx from the
        running sum of lr^power, entirely on the device."""
        mu_y = state_lists[TRAIN_INTERP_COEFF]
        mu_x = state_lists[EVAL_INTERP_COEFF]
        match iterate_averaging_config:
            case GeneralizedPrimalAveragingConfig():
                mu_y.fill_(iterate_averaging_config.train_interp_coeff)
                mu_x.fill_(iterate_averaging_config.eval_interp_coeff)
            case ScheduleFreeConfig():
                mu_y.fill_(iterate_averaging_config.train_interp_coeff)
                if lr is not None:
                    lr_pow = torch.pow(lr, iterate_averaging_config.eval_coeff_lr_power)
                    state_lists[LR_SUM] += lr_pow
                    mu_x.copy_(1.0 - lr_pow / state_lists[LR_SUM])
                else:
                    logger.warning(
                        "lr or lr_sum not provided to _get_train_and_eval_interp_coeffs; returning eval_interp_coeff = 0.0!"
                    )
                    mu_x.fill_(0.0)
            case _:
                raise ValueError(
                    f"Iterate averaging config iterate_averaging_config={iterate_averaging_config} is not supported "
                    "for retrieving train and eval interpolation coefficients; only "
                    "GeneralizedPrimalAveragingConfig and ScheduleFreeConfig are supported."
                )
        return mu_y, mu_x

    @torch.no_grad()
    def _apply_in_place_primal_averaging(self, state_lists, masked_blocked_search_directions, train_interp_coeff, eval_interp_coeff) -> None:
        """T = Z - W;  Z += D;  D ← (1 - μx μy)·D + (1 - μx)·T."""
        if not state_lists[TRAIN_MODE]:
            raise RuntimeError(
                "Called _apply_in_place_primal_averaging when not in train mode. Call optimizer.train() before calling optimizer.step()!"
            )
        z = state_lists[MASKED_WEIGHT_BUFFER_LIST]
        gap = torch._foreach_sub(z, state_lists[MASKED_BLOCKED_PARAMS])
        torch._foreach_add_(z, masked_blocked_search_directions)
        torch._foreach_mul_(masked_blocked_search_directions, 1 - train_interp_coeff * eval_interp_coeff)
        torch._foreach_add_(masked_blocked_search_directions, gap, alpha=1 - eval_interp_coeff)

    @torch.no_grad()
    def _compute_search_directions(
        self, state_lists, step, lr, beta1, beta3, weight_decay, peak_lr, weight_decay_type,
        grafting_config_not_none, perform_amortized_computation, use_bias_correction, use_grafting_method,
        iterate_averaging_enabled, classic_momentum_enabled, train_interp_coeff, eval_interp_coeff,
        momentum_param, dampening, use_nesterov,
    ) -> tuple[torch.Tensor, ...]:
        self._add_l2_regularization(state_lists, weight_decay, weight_decay_type)
        self._update_preconditioners(state_lists, step, perform_amortized_computation, grafting_config_not_none)
        filtered = self._compute_filtered_grad_list(state_lists, step, beta1, beta3, use_bias_correction)
        directions = self._precondition_and_grafting(state_lists, filtered, use_grafting_method, grafting_config_not_none)
        self._apply_weight_decay(state_lists, directions, lr, weight_decay, peak_lr, weight_decay_type, iterate_averaging_enabled)
        if classic_momentum_enabled:
            self._apply_classic_momentum(state_lists, directions, momentum_param, dampening, use_nesterov)
        torch._foreach_mul_(directions, -lr)
        if iterate_averaging_enabled:
            self._apply_in_place_primal_averaging(state_lists, directions, train_interp_coeff, eval_interp_coeff)
        return directions

    @torch.no_grad()
    def _per_group_step_impl(self, state_lists, *args: Any) -> None:
        # With no gradient anywhere the distributor is still called (with nothing) so that ranks
        # stay in lock-step on its collective.
        directions = self._compute_search_directions(state_lists, *args) if state_lists[MASKED_BLOCKED_GRADS] else ()
        state_lists[DISTRIBUTOR].update_params(blocked_search_directions=directions)

    @torch.no_grad()
    def _group_step_body(self, state_lists: dict[str, Any], group: dict[str, Any], per_group_step: Callable[..., None]) -> None:
        rec = state_lists
        engine = rec.get(NATIVE_ENGINE)
        if engine is None:
            rec[MASKED_BLOCKED_GRADS] = rec[DISTRIBUTOR].merge_and_block_gradients()
        else:
            rec[MASKED_BLOCKED_GRADS] = engine.collect_gradients()
        DistributedShampoo._mask_state_lists(rec, group, self._shampoo_pt2_compile_config is not None)

        step = rec[STEP].add_(1)
        t = step.item()
        rec[LR_CPU_PINNED].fill_(group[LR])
        lr = rec[LR_TENSOR]
        lr.copy_(rec[LR_CPU_PINNED], non_blocking=True)

        start = group[START_PRECONDITIONING_STEP]
        has_grafting = group[GRAFTING_CONFIG] is not None
        refresh = (t % group[PRECONDITION_FREQUENCY] == 0 and t > start) or t == start
        graft_only = t < start and has_grafting
        avg_cfg = group[ITERATE_AVERAGING_CONFIG]
        primal = _is_primal_averaging(avg_cfg)
        classic = isinstance(avg_cfg, ClassicMomentumConfig)
        if primal:
            mu_y, mu_x = self._get_train_and_eval_interp_coeffs(avg_cfg, lr, rec)
        else:
            mu_y, mu_x = rec[TRAIN_INTERP_COEFF], rec[EVAL_INTERP_COEFF]
        momentum, dampening, nesterov = (
            (avg_cfg.momentum, avg_cfg.dampening, avg_cfg.use_nesterov) if classic else (0.0, 0.0, False)
        )
        args = (
            step, lr, group[BETAS][0], group[BETA3], group[WEIGHT_DECAY], group[PEAK_LR], group[WEIGHT_DECAY_TYPE],
            has_grafting, refresh, group[USE_BIAS_CORRECTION], graft_only, primal, classic, mu_y, mu_x,
            momentum, dampening, nesterov,
        )
        if engine is None:
            per_group_step(rec, *args)
        else:
            engine.step(group, *args)
        rec[MASKED_BLOCKED_GRADS] = None

    @torch.no_grad()
    def step(self, closure: Callable[[], float] | None = None) -> float | None:  # type: ignore[override]
        """One optimisation step.  With ``ConcurrencyConfig.enable_cuda_stream_for_param_groups``
        and every group on CUDA, each group runs on its own stream so that the collectives of
        different groups overlap; the default stream waits for all of them at the end."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for rec, group in self._groups():
            if self._use_cuda_streams:
                stream = rec[CUDA_STREAM]
                stream.wait_stream(torch.cuda.current_stream(stream.device))
                ctx: Any = torch.cuda.stream(stream)
            else:
                ctx = nullcontext()
            with ctx:
                self._group_step_body(rec, group, self._per_group_step)
        if self._use_cuda_streams:
            self._sync_streams_to_default()
        return loss

    @torch.no_grad()
    def _sync_streams_to_default(self) -> None:
        for rec, group in self._groups():
            torch.cuda.current_stream(group[PARAMS][0].device).wait_stream(rec[CUDA_STREAM])

    # ------------------------------------------------------------------------------------------
    # train() / eval(): switch the parameters between the y (gradient) and x (averaged) sequences
    # ------------------------------------------------------------------------------------------
    def _switch_mode(self, to_train: bool) -> None:
        for rec, group in self._groups():
            cfg = group[ITERATE_AVERAGING_CONFIG]
            if not _is_primal_averaging(cfg) or bool(rec[TRAIN_MODE]) == to_train:
                continue
            mu_y, _ = self._get_train_and_eval_interp_coeffs(cfg, None, rec)
            engine = rec.get(NATIVE_ENGINE)
            coeff = (1 - cfg.train_interp_coeff) if to_train else (1 - 1 / cfg.train_interp_coeff)
            if engine is not None and engine.mode_switch(coeff):
                rec[TRAIN_MODE].fill_(to_train)
                continue
            delta: list[torch.Tensor] = []
            if rec[WEIGHT_BUFFER_LIST]:  # a rank that owns no block still joins the distributor's collective
                delta = list(torch._foreach_sub(rec[WEIGHT_BUFFER_LIST], rec[DISTRIBUTOR].local_blocked_params))
                torch._foreach_mul_(delta, (1 - mu_y) if to_train else (1 - torch.reciprocal(mu_y)))
            rec[DISTRIBUTOR].update_params(blocked_search_directions=tuple(delta), use_masked_tensors=False)
            rec[TRAIN_MODE].fill_(to_train)

    @torch.no_grad()
    def train(self) -> None:
        """W ← W + (Z - W)(1 - μy): parameters become the y sequence gradients are taken at."""
        logger.info("Enabling train mode in Distributed Shampoo!")
        self._switch_mode(True)

    @torch.no_grad()
    def eval(self) -> None:
        """W ← W + (Z - W)(1 - 1/μy): parameters become the averaged x sequence."""
        logger.info("Enabling eval mode in Distributed Shampoo!")
        self._switch_mode(False)

    # ------------------------------------------------------------------------------------------
    # Checkpointing
    # ------------------------------------------------------------------------------------------
    def __setstate__(self, state: dict[str, Any]) -> None:
        """Called by ``Optimizer.load_state_dict`` with the re-keyed, device-cast state.  Loaded
        values are copied *into* the live tensors and state modules (views held by block tables
        and distributors stay valid); the per-group scalars aliased under several parameters
        must agree in the checkpoint."""
        if "state" not in state:
            super().__setstate__(state)
            return

        seen: dict[int, Any] = {}
        for p, loaded in state["state"].items():
            live = self.state.get(p) if p in self.state else None
            if live is None:
                continue
            for key in (STEP, LR_SUM, TRAIN_MODE):
                if key not in live or key not in loaded:
                    continue
                value = loaded[key].item() if isinstance(loaded[key], torch.Tensor) else loaded[key]
                alias = id(live[key])
                if alias not in seen:
                    seen[alias] = value
                    continue
                first = seen[alias]
                if key == LR_SUM:
                    differ = not ((math.isnan(first) and math.isnan(value)) or math.isclose(first, value, rel_tol=1e-6))
                else:
                    differ = first != value
                if differ:
                    raise ValueError(
                        f"Cannot load optimizer state: the per-group scalar '{key}' is aliased across parameters sharing a group, "
                        f"but the checkpoint stored differing values ({first} != {value}). This happens when parameters are regrouped "
                        "across groups that had different histories (e.g. different learning rates), which distributed_shampoo does not support."
                    )

        for p, loaded in state["state"].items():
            if p in self.state:
                update_param_state_dict_object(self.state[p], loaded, enable_missing_key_check=False)
            else:
                logger.warning(
                    f"Found parameter {p} in state dict to load that doesn't exist in current state. Directly assigning it."
                )
                self.state[p] = loaded
        del state["state"]
        super().__setstate__(state)

    @staticmethod
    def _post_state_dict_hook(optimizer: Optimizer, state_dict: StateDict) -> None:
        """Turn state modules into nested dicts of tensors, give every parameter an entry (ranks
        that own nothing of a parameter still expose its key), and warn about configs holding
        lambdas, which cannot be pickled."""

        def holds_lambda(obj: Any) -> bool:
            if isinstance(obj, LambdaType) and obj.__name__ == "<lambda>":
                return True
            if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
                return any(holds_lambda(getattr(obj, f.name)) for f in dataclasses.fields(obj))
            return False

        state_dict["state"] = {k: extract_state_dict_content(v) for k, v in state_dict["state"].items()}
        for group in state_dict["param_groups"]:
            for v in group.values():
                if holds_lambda(v):
                    logger.warning(
                        f"Found v={v}. Note that lambda function cannot be pickled. "
                        "torch.save() cannot serialize lambda functions, because it relies on Python's pickle module for serialization, and pickle does not support lambda functions."
                    )
            for pid in group["params"]:
                state_dict["state"].setdefault(pid, {})

    @staticmethod
    def _pre_load_state_dict_hook(optimizer: Optimizer, state_dict: StateDict) -> None:
        """Remember each primal-averaging group's mode so it can be restored after the load."""
        optimizer._pre_load_train_modes = [  # type: ignore[attr-defined]
            bool(rec[TRAIN_MODE].item())
            for rec, group in zip(optimizer._per_group_state_lists, optimizer.param_groups, strict=True)  # type: ignore[attr-defined]
            if _is_primal_averaging(group[ITERATE_AVERAGING_CONFIG])
        ]

    @staticmethod
    def _post_load_state_dict_hook(optimizer: Optimizer) -> None:
        """Re-gather cached full parameters of lossless distributors, rebuild derived kernel
        operands, and return to the mode the optimizer was in before the load."""
        for rec in optimizer._per_group_state_lists:  # type: ignore[attr-defined]
            dist = rec[DISTRIBUTOR]
            if hasattr(dist, "refresh_assigned_full_params"):
                dist.refresh_assigned_full_params()
                rec[MASKED_BLOCKED_PARAMS] = dist.local_blocked_params
            if rec.get(NATIVE_ENGINE) is not None:
                rec[NATIVE_ENGINE].on_state_loaded()
        modes = getattr(optimizer, "_pre_load_train_modes", [])
        if modes:
            assert all(m == modes[0] for m in modes), "Mixed train/eval modes across parameter groups is not supported."
            (optimizer.train if modes[0] else optimizer.eval)()  # type: ignore[attr-defined]
            del optimizer._pre_load_train_modes  # type: ignore[attr-defined]
