"""Storage-dtype shell for optimizer state: keep a list of tensors in a (smaller) floating-point
dtype and hand out a computation-dtype copy while it is being worked on.  Only float-to-float
conversion is implemented; integer formats raise ``NotImplementedError``.

Reference counterpart: ``distributed_shampoo/utils/shampoo_quantization.py:35-292``.
"""

from __future__ import annotations

import logging
from collections.abc import Sequence

import torch
from torch import Tensor

from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.utils.blocking import compress_list, ParameterizeEnterExitContext
from optimizers_b200.utils.state import OptimizerModule

logger: logging.Logger = logging.getLogger(__name__)

_FLOAT_DTYPES: tuple[torch.dtype, ...] = (torch.float16, torch.bfloat16, torch.float32, torch.float64)


def _unsupported(dtype: torch.dtype) -> NotImplementedError:
    return NotImplementedError(f"Quantization for {dtype} is not yet supported!")


class QuantizedTensor(OptimizerModule):
    """One stored tensor plus the (min, max) metadata an integer format would need."""

    def __init__(self, quantized_values: Tensor, block_info: BlockInfo, min_value: Tensor | None = None, max_value: Tensor | None = None) -> None:
        self.quantized_values = quantized_values
        self.min_value = min_value
        self.max_value = max_value
        self.block_info = block_info
        if quantized_values.dtype in _FLOAT_DTYPES:
            assert min_value is None and max_value is None
        elif min_value is None and max_value is None:
            assert torch.count_nonzero(quantized_values) == 0
            self.min_value = torch.zeros(1)
            self.max_value = torch.zeros(1)

    @classmethod
    def init_from_dequantized_tensor(cls, dequantized_values: Tensor, quantized_dtype: torch.dtype, block_info: BlockInfo) -> "QuantizedTensor":
        stored = block_info.allocate_zeros_tensor(size=dequantized_values.shape, dtype=quantized_dtype, device=dequantized_values.device)
        lo, hi = cls._quantize_and_return_metadata(block_info.get_tensor(dequantized_values), block_info.get_tensor(stored))
        return cls(stored, block_info, lo, hi)

    def dequantize(self, dequantized_dtype: torch.dtype) -> Tensor:
        if self.quantized_values.dtype == dequantized_dtype:
            return self.quantized_values
        if self.quantized_values.dtype not in _FLOAT_DTYPES:
            raise _unsupported(self.quantized_values.dtype)
        return self.quantized_values.to(dtype=dequantized_dtype)

    def quantize(self, dequantized_tensor: Tensor) -> None:
        self.min_value, self.max_value = self._quantize_and_return_metadata(dequantized_tensor, self.quantized_values)

    @staticmethod
    def _quantize_and_return_metadata(dequantized_values: Tensor, quantized_values: Tensor) -> tuple[Tensor | None, Tensor | None]:
        if quantized_values.dtype not in _FLOAT_DTYPES:
            raise _unsupported(quantized_values.dtype)
        quantized_values.copy_(dequantized_values)
        return None, None


class QuantizedTensorList:
    """A list of stored tensors with an optional cached computation-dtype copy."""

    def __init__(
        self,
        quantized_data: Sequence[tuple[Tensor, Tensor | None, Tensor | None]] | Sequence[QuantizedTensor],
        quantized_dtype: torch.dtype,
        computation_dtype: torch.dtype = torch.float32,
    ) -> None:
        if all(isinstance(x, QuantizedTensor) for x in quantized_data):
            self.quantized_value_list = tuple(x.block_info.get_tensor(x.quantized_values) for x in quantized_data)
            self._min_values = tuple(x.min_value for x in quantized_data)
            self._max_values = tuple(x.max_value for x in quantized_data)
        elif all(isinstance(x, tuple) for x in quantized_data):
            columns = tuple(zip(*quantized_data)) or ((), (), ())
            self.quantized_value_list, self._min_values, self._max_values = (tuple(c) for c in columns)
        else:
            raise TypeError(
                f"quantized_data must be a sequence of (values, min, max) tuples or of QuantizedTensor but get {type(quantized_data)}"
            )
        self.dequantized_value_list: tuple[Tensor, ...] | None = None
        assert all(v.dtype == quantized_dtype for v in self.quantized_value_list)
        assert computation_dtype in _FLOAT_DTYPES, (
            f"computation_dtype={computation_dtype} is not supported! It must be one of {_FLOAT_DTYPES}!"
        )
        self.quantized_dtype = quantized_dtype
        self.computation_dtype = computation_dtype
        pairs = list(zip(self._min_values, self._max_values, strict=True))
        assert all(a is None and b is None for a, b in pairs) or not any(a is None or b is None for a, b in pairs)

    def __len__(self) -> int:
        return len(self.quantized_value_list)

    @staticmethod
    def _convert_float_to_float(src_list, target_dtype: torch.dtype, dest_list=None) -> tuple[Tensor, ...]:
        if dest_list is None:
            dest_list = tuple(torch.zeros_like(t, dtype=target_dtype) for t in src_list)
        if dest_list:
            torch._foreach_copy_(dest_list, src_list)
        return dest_list

    def dequantize(self) -> tuple[Tensor, ...]:
        if self.quantized_dtype == self.computation_dtype:
            return self.quantized_value_list
        if self.quantized_dtype not in _FLOAT_DTYPES:
            raise _unsupported(self.quantized_dtype)
        return self._convert_float_to_float(self.quantized_value_list, self.computation_dtype)

    def dequantize_(self) -> None:
        if self.is_dequantized_stored():
            logger.warning("Dequantized values are already stored; overwriting these values...")
        self.dequantized_value_list = self.dequantize()

    def quantize(self, tensor_list: tuple[Tensor, ...]) -> None:
        if tensor_list is not self.dequantized_value_list and self.is_dequantized_stored():
            logger.warning(
                "Existing stored dequantized values.\nWriting quantized values with input tensor_list without using these stored dequantized values..."
            )
        if self.quantized_dtype not in _FLOAT_DTYPES:
            raise _unsupported(self.quantized_dtype)
        self._convert_float_to_float(tensor_list, self.quantized_dtype, self.quantized_value_list)

    def quantize_(self) -> None:
        if not self.is_dequantized_stored():
            logger.warning(
                f"No stored dequantized values self.dequantized_value_list={self.dequantized_value_list}. Must first call dequantize_()."
            )
            return
        if self.quantized_dtype != self.computation_dtype:
            assert self.dequantized_value_list is not None
            self.quantize(self.dequantized_value_list)
        self.dequantized_value_list = None

    @property
    def dequantized_value(self) -> tuple[Tensor, ...]:
        assert self.dequantized_value_list is not None
        return self.dequantized_value_list

    @property
    def quantized_value(self) -> tuple[Tensor, ...]:
        return self.quantized_value_list

    def is_dequantized_stored(self) -> bool:
        return self.dequantized_value_list is not None

    def compress(self, selector: tuple[bool, ...]) -> "QuantizedTensorList":
        assert not self.is_dequantized_stored()
        kept = zip(
            compress_list(self.quantized_value_list, selector),
            compress_list(self._min_values, selector),
            compress_list(self._max_values, selector),
            strict=True,
        )
        return QuantizedTensorList(tuple(kept), self.quantized_dtype, self.computation_dtype)


class DequantizeQuantizedTensorListContext(ParameterizeEnterExitContext):
    """``with`` block during which the list holds a computation-dtype copy; written back on exit."""

    def __init__(self, quantized_tensor_list: QuantizedTensorList) -> None:
        super().__init__(quantized_tensor_list, QuantizedTensorList.dequantize_, QuantizedTensorList.quantize_)
