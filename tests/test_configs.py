"""Validation rules of the configuration dataclasses."""

import math
import pickle

import pytest
import torch

import optimizers_b200 as ob
from optimizers_b200 import config as C


def test_abstract_bases_cannot_be_instantiated():
    for cls in (C.PreconditionerConfig, C.MatrixFunctionConfig, C.RootInvConfig, C.EigendecompositionConfig,
                C.OrthogonalizationConfig, C.IterateAveragingConfig, C.DistributedConfig, C.RankDeficientStabilityConfig,
                C.BaseShampooPreconditionerConfig, C.ClassicShampooPreconditionerConfig, C.CostModel):
        with pytest.raises(TypeError):
            cls()


@pytest.mark.parametrize(
    "factory,message",
    [
        (lambda: ob.AdaGradPreconditionerConfig(epsilon=0.0), "Invalid epsilon value: 0.0. Must be > 0.0."),
        (lambda: ob.RMSpropPreconditionerConfig(beta2=0.0), "Invalid grafting beta2 parameter: 0.0. Must be in (0.0, 1.0]."),
        (lambda: ob.AdamPreconditionerConfig(beta2=1.5), "Invalid grafting beta2 parameter"),
        (lambda: ob.RootInvShampooPreconditionerConfig(num_tolerated_failed_amortized_computations=-1), "Must be >= 0."),
        (lambda: ob.RootInvShampooPreconditionerConfig(use_trace_scaling=True, trace_scaling_exponent=0.0), "Must be in (0.0, 1.0] when use_trace_scaling=True."),
        (lambda: ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={-1: 0.5}), "All orders must be >= 0."),
        (lambda: ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: {2: 0.5}}), "All dimensions must be within [0, 1]."),
        (lambda: ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: {0: -0.5}}), "All overrides must be >= 0."),
        (lambda: ob.RootInvShampooPreconditionerConfig(inverse_exponent_override={2: -0.5}), "All overrides must be >= 0."),
        (lambda: ob.EigenvalueCorrectedShampooPreconditionerConfig(
            amortized_computation_config=ob.EighEigendecompositionConfig(rank_deficient_stability_config=ob.PseudoInverseConfig())),
         "PseudoInverseConfig is an invalid rank_deficient_stability_config for EigenvalueCorrectedShampooPreconditionerConfig"),
        (lambda: ob.EigenvalueCorrectedShampooPreconditionerConfig(ignored_basis_change_dims={2: [2]}), "All dimensions must be within [0, 1]."),
        (lambda: ob.EigenvalueCorrectedShampooPreconditionerConfig(ignored_basis_change_dims={2: [0, 0]}), "All dimensions must be unique."),
        (lambda: ob.EigenvalueCorrectedShampooPreconditionerConfig(inverse_exponent_override={2: 0.0}), "All overrides must be > 0."),
        (lambda: ob.EighEigendecompositionConfig(tolerance=1.5), "Must be in the interval [0.0, 1.0]."),
        (lambda: ob.EigenConfig(tolerance=0.1), "Must be 0.0 for EigenConfig."),
        (lambda: ob.ClassicMomentumConfig(momentum=1.0), "Must be within (0.0, 1.0)."),
        (lambda: ob.ClassicMomentumConfig(dampening=1.0), "Must be within [0.0, 1.0)."),
        (lambda: ob.GeneralizedPrimalAveragingConfig(eval_interp_coeff=1.0), "Must be within [0.0, 1.0)."),
        (lambda: ob.GeneralizedPrimalAveragingConfig(train_interp_coeff=0.0), "Must be within (0.0, 1.0]."),
        (lambda: ob.ScheduleFreeConfig(train_interp_coeff=1.5), "Must be within (0.0, 1.0]."),
        (lambda: ob.SingleDeviceDistributedConfig(target_parameter_dimensionality=1.5), "Must be an integer or math.inf."),
        (lambda: ob.SingleDeviceDistributedConfig(target_parameter_dimensionality=0), "Must be >= 1."),
        (lambda: ob.FullyShardDistributedConfig(num_sub_groups=0), "Must be >= 1."),
        (lambda: ob.FullyShardDistributedConfig(num_sub_groups=2), "num_sub_groups > 1 requires param_assignment_strategy != DEFAULT"),
        (lambda: ob.NativeRuntimeConfig(backend="triton"), "Invalid backend"),
        (lambda: ob.NativeRuntimeConfig(fuse_gradient_reduction=True), "requires comm_path='p2p'"),
    ],
)
def test_invalid_configs(factory, message):
    with pytest.raises(ValueError) as err:
        factory()
    assert message in str(err.value)


def test_defaults_and_relations():
    assert isinstance(ob.DefaultShampooConfig.amortized_computation_config, ob.EigenConfig)
    assert isinstance(ob.DefaultSOAPConfig.amortized_computation_config, ob.QREigendecompositionConfig)
    assert isinstance(ob.DefaultEigenvalueCorrectedShampooConfig.amortized_computation_config, ob.EighEigendecompositionConfig)
    assert ob.AdamPreconditionerConfig().beta2 == 0.999 and ob.RMSpropPreconditionerConfig().beta2 == 0.99
    assert issubclass(ob.HSDPDistributedConfig, ob.DDPDistributedConfig) and issubclass(ob.HSDPDistributedConfig, ob.FSDPDistributedConfig)
    assert issubclass(ob.HybridShardDistributedConfig, ob.FullyShardDistributedConfig)
    assert ob.SingleDeviceDistributedConfig(target_parameter_dimensionality=math.inf).target_parameter_dimensionality == math.inf
    assert ob.DDPDistributedConfig().communication_dtype == torch.float32
    assert ob.ShampooPT2CompileConfig(fullgraph=True).fullgraph is True
    assert [e.name for e in ob.FSDPParamAssignmentStrategy] == ["DEFAULT", "REPLICATE", "ROUND_ROBIN"]


def test_configs_are_picklable():
    for cfg in (ob.DefaultShampooConfig, ob.DefaultSOAPConfig, ob.DefaultSpectralDescentPreconditionerConfig,
                ob.DefaultSignDescentPreconditionerConfig, ob.DDPDistributedConfig(), ob.AdamPreconditionerConfig()):
        assert pickle.loads(pickle.dumps(cfg)) == cfg
