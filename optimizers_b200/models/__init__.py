"""Model definitions used by the examples and benchmarks (synthetic-data friendly)."""

from optimizers_b200.models.convnet import ConvNet, MLP
from optimizers_b200.models.gpt2 import GPT2, GPT2Config
from optimizers_b200.models.llama import Llama, LlamaConfig
from optimizers_b200.models.resnet import ResNet18

__all__ = ["ConvNet", "MLP", "GPT2", "GPT2Config", "Llama", "LlamaConfig", "ResNet18"]
