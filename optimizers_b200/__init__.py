"""optimizers_b200: Distributed Shampoo and GPA-AdamW built for NVIDIA B200 (sm_100a).

The public names match ``facebookresearch/optimizers`` (``distributed_shampoo`` and ``gpa``
packages), so ``from optimizers_b200 import DistributedShampoo, AdamPreconditionerConfig, ...``
replaces ``from distributed_shampoo import ...``.
"""

from optimizers_b200.config import (
    AdaGradPreconditionerConfig,
    AdamPreconditionerConfig,
    AlignedMemoryCostModel,
    BaseShampooPreconditionerConfig,
    ClassicMomentumConfig,
    ClassicShampooPreconditionerConfig,
    ConcurrencyConfig,
    CoupledHigherOrderConfig,
    CoupledNewtonConfig,
    DDPDistributedConfig,
    DefaultEigenConfig,
    DefaultEigendecompositionConfig,
    DefaultEigenvalueCorrectedShampooConfig,
    DefaultNewtonSchulzOrthogonalizationConfig,
    DefaultPerturbationConfig,
    DefaultShampooConfig,
    DefaultSignDescentPreconditionerConfig,
    DefaultSingleDeviceDistributedConfig,
    DefaultSOAPConfig,
    DefaultSpectralDescentPreconditionerConfig,
    DistributedConfig,
    EigenConfig,
    EigendecomposedKLShampooPreconditionerConfig,
    EigendecomposedShampooPreconditionerConfig,
    EigendecompositionConfig,
    EigenvalueCorrectedShampooPreconditionerConfig,
    EighEigendecompositionConfig,
    FSDPDistributedConfig,
    FSDPParamAssignmentStrategy,
    FSDPParameterMetadata,
    FullyShardDistributedConfig,
    GeneralizedPrimalAveragingConfig,
    HSDPDistributedConfig,
    HybridShardDistributedConfig,
    IterateAveragingConfig,
    LoadBalancingConfig,
    MatrixFunctionConfig,
    NativeRuntimeConfig,
    NewtonSchulzOrthogonalizationConfig,
    OrthogonalizationConfig,
    PerturbationConfig,
    PolynomialComputationalCostModel,
    PreconditionerConfig,
    PreconditionerValueError,
    PseudoInverseConfig,
    QREigendecompositionConfig,
    RankDeficientStabilityConfig,
    RMSpropPreconditionerConfig,
    RootInvConfig,
    RootInvKLShampooPreconditionerConfig,
    RootInvShampooPreconditionerConfig,
    ScheduleFreeConfig,
    SGDPreconditionerConfig,
    ShampooPT2CompileConfig,
    ShampooRuntimeConfig,
    SignDescentPreconditionerConfig,
    SingleDeviceDistributedConfig,
    SpectralDescentPreconditionerConfig,
    SVDOrthogonalizationConfig,
    WeightDecayType,
)
from optimizers_b200.shampoo import DistributedShampoo


def __getattr__(name: str):
    # Deferred: these pull in torch.distributed.fsdp internals / the GPA optimizer module.
    if name == "compile_fsdp_parameter_metadata":
        from optimizers_b200.parallel.fsdp_utils import compile_fsdp_parameter_metadata

        return compile_fsdp_parameter_metadata
    if name in ("GPAAdamW", "IterateAveragingType"):
        from optimizers_b200 import gpa_adamw

        return getattr(gpa_adamw, name)
    raise AttributeError(name)


__all__ = [n for n in dir() if not n.startswith("_")] + [
    "compile_fsdp_parameter_metadata",
    "GPAAdamW",
    "IterateAveragingType",
]
