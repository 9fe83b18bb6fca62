"""``CombinedLinear``: a linear layer whose weight and bias live in one ``[out, in + 1]``
parameter, so that Shampoo preconditions them jointly (the bias is the last column).

Reference counterpart: ``distributed_shampoo/utils/shampoo_model_utils.py:16-113``.
"""

from __future__ import annotations

import math

import torch
from torch.nn.parameter import Parameter


class CombinedLinear(torch.nn.Module):
    __constants__ = ["in_features", "out_features"]

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.bias = bias
        self.in_features_with_bias = in_features + int(bias)
        self.combined_weight = Parameter(torch.empty((out_features, self.in_features_with_bias), device=device, dtype=dtype))
        self.reset_parameters()

    def _split(self) -> tuple[torch.Tensor, torch.Tensor | None]:
        w = self.combined_weight
        return (w[:, :-1], w[:, -1]) if self.bias else (w, None)

    def reset_parameters(self) -> None:
        """Same initialisation as ``torch.nn.Linear``."""
        weight, bias = self._split()
        torch.nn.init.kaiming_uniform_(weight, a=math.sqrt(5))
        if bias is not None:
            fan_in, _ = torch.nn.init._calculate_fan_in_and_fan_out(weight)
            bound = 1 / math.sqrt(fan_in) if fan_in > 0 else 0
            torch.nn.init.uniform_(bias, -bound, bound)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        weight, bias = self._split()
        return torch.nn.functional.linear(input, weight, bias)

    def extra_repr(self) -> str:
        return f"self.in_features={self.in_features}, self.out_features={self.out_features}, self.in_features_with_bias={self.in_features_with_bias}"
