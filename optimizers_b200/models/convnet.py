"""Small models of the examples: the one-convolution ConvNet and a two-layer MLP."""

from __future__ import annotations

import math

import torch
from torch import nn


class ConvNet(nn.Module):
    """3x3 convolution (no bias) -> ReLU -> linear classifier over the flattened feature map."""

    def __init__(self, height: int, width: int, out_channels: int = 64, disable_bias: bool = False, num_classes: int = 10) -> None:
        super().__init__()
        kernel, stride, padding = 3, 1, 1
        self.conv = nn.Conv2d(3, out_channels, kernel_size=kernel, stride=stride, padding=padding, bias=False)
        self.activation = nn.ReLU()
        out_hw = self._infer_conv_output_shape((height, width), kernel, stride, padding)
        self.linear = nn.Linear(math.prod(out_hw) * out_channels, num_classes, bias=not disable_bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(torch.flatten(self.activation(self.conv(x)), start_dim=1))

    @staticmethod
    def _infer_conv_output_shape(input_shape: tuple[int, ...], kernel_size: int, stride: int, padding: int) -> list[int]:
        out = []
        for length in input_shape:
            value = (length - kernel_size + 2 * padding) / stride + 1
            assert value.is_integer(), (
                f"Stride {stride} is not compatible with input shape {input_shape}, kernel size {kernel_size} and padding {padding}!"
            )
            out.append(int(value))
        return out


class MLP(nn.Module):
    """784 -> hidden -> 10 with ReLU (the CPU baseline configuration uses hidden = 512)."""

    def __init__(self, in_features: int = 784, hidden: int = 512, num_classes: int = 10) -> None:
        super().__init__()
        self.net = nn.Sequential(nn.Linear(in_features, hidden), nn.ReLU(), nn.Linear(hidden, num_classes))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.net(torch.flatten(x, start_dim=1))
