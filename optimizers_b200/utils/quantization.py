"""Optimizer state kept in a storage dtype and worked on in a computation dtype.

The public classes mirror ``distributed_shampoo/utils/shampoo_quantization.py:35-292`` of the
reference (``QuantizedTensor``, ``QuantizedTensorList``, ``DequantizeQuantizedTensorListContext``);
the implementation is organised for the GPU:

* a *storage format* object per dtype owns both directions of the conversion for a whole list at
  once, so a list is converted by one multi-tensor launch; the floating-point formats are a
  rounding cast, integer formats are not registered and raise ``NotImplementedError``;
* the computation-dtype copies of a list are views of one flat workspace per device instead of
  one allocation per tensor; the in-place pair ``dequantize_`` / ``quantize_`` (what the ``with``
  context calls every step) keeps that workspace between uses, so a step allocates nothing.
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

_Bounds = tuple[Tensor | None, Tensor | None]


class _CastFormat:
    """Floating-point storage: storing is a rounding cast, loading a widening one, and there is
    no range metadata (both bounds are None)."""

    @staticmethod
    def store(values: Sequence[Tensor], into: Sequence[Tensor]) -> list[_Bounds]:
        if len(into) > 0:
            torch._foreach_copy_(list(into), list(values))
        return [(None, None)] * len(into)

    @staticmethod
    def load(stored: Sequence[Tensor], into: Sequence[Tensor]) -> None:
        if len(into) > 0:
            torch._foreach_copy_(list(into), list(stored))


_FORMATS: dict[torch.dtype, _CastFormat] = {
    dtype: _CastFormat() for dtype in (torch.float16, torch.bfloat16, torch.float32, torch.float64)
}


_FLOAT_DTYPES: tuple[torch.dtype, ...] = tuple(_FORMATS)


def _format_of(dtype: torch.dtype) -> _CastFormat:
    try:
        return _FORMATS[dtype]
    except KeyError:
        raise NotImplementedError(f"Quantization for {dtype} is not yet supported!") from None


def _workspace_like(tensors: Sequence[Tensor], dtype: torch.dtype) -> tuple[Tensor, ...]:
    """Tensors of ``dtype`` shaped like ``tensors``, carved out of one flat allocation per device
    (each view starts on a 16-element boundary, so 16-byte vector accesses stay aligned)."""
    cursor: dict[torch.device, int] = {}
    offsets = []
    for t in tensors:
        start = cursor.get(t.device, 0)
        offsets.append(start)
        cursor[t.device] = start + (t.numel() + 15) // 16 * 16
    flat = {device: torch.empty(size, dtype=dtype, device=device) for device, size in cursor.items()}
    return tuple(
        flat[t.device][start : start + t.numel()].view(t.shape) for t, start in zip(tensors, offsets, strict=True)
    )


class QuantizedTensor(OptimizerModule):
    """One stored tensor with the range metadata (``min_value``, ``max_value``) that an integer
    format would need; for the floating-point formats both stay None."""

    def __init__(
        self, quantized_values: Tensor, block_info: BlockInfo, min_value: Tensor | None = None, max_value: Tensor | None = None
    ) -> None:
        self.quantized_values = quantized_values
        self.block_info = block_info
        if quantized_values.dtype in _FORMATS:
            assert min_value is None and max_value is None
        elif min_value is None and max_value is None:
            # an all-zero integer tensor needs no range: give it the degenerate one
            assert torch.count_nonzero(quantized_values) == 0
            min_value, max_value = torch.zeros(1), torch.zeros(1)
        self.min_value = min_value
        self.max_value = max_value

    @classmethod
    def init_from_dequantized_tensor(
        cls, dequantized_values: Tensor, quantized_dtype: torch.dtype, block_info: BlockInfo
    ) -> "QuantizedTensor":
        storage = block_info.allocate_zeros_tensor(
            size=dequantized_values.shape, dtype=quantized_dtype, device=dequantized_values.device
        )
        fresh = cls(storage, block_info)
        fresh.quantize(block_info.get_tensor(dequantized_values))
        return fresh

    def quantize(self, dequantized_tensor: Tensor) -> None:
        local = self.block_info.get_tensor(self.quantized_values)
        ((self.min_value, self.max_value),) = _format_of(local.dtype).store([dequantized_tensor], [local])

    def dequantize(self, dequantized_dtype: torch.dtype) -> Tensor:
        stored = self.quantized_values
        if stored.dtype == dequantized_dtype:
            return stored
        _format_of(stored.dtype)  # refuses storage dtypes that cannot be read back
        return stored.to(dtype=dequantized_dtype)

    @staticmethod
    def _quantize_and_return_metadata(dequantized_values: Tensor, quantized_values: Tensor) -> _Bounds:
        return _format_of(quantized_values.dtype).store([dequantized_values], [quantized_values])[0]


class QuantizedTensorList:
    """Stored tensors of one storage dtype and, while they are being worked on, their copies in
    the computation dtype.  Built either from ``QuantizedTensor`` objects or from
    ``(values, min, max)`` triples."""

    def __init__(
        self,
        quantized_data: Sequence[tuple[Tensor, Tensor | None, Tensor | None]] | Sequence[QuantizedTensor],
        quantized_dtype: torch.dtype,
        computation_dtype: torch.dtype = torch.float32,
    ) -> None:
        kinds = {type(item) for item in quantized_data}
        if kinds <= {QuantizedTensor}:
            triples = [(q.block_info.get_tensor(q.quantized_values), q.min_value, q.max_value) for q in quantized_data]
        elif kinds <= {tuple}:
            triples = list(quantized_data)
        else:
            raise TypeError(
                f"quantized_data must be a sequence of (values, min, max) tuples or of QuantizedTensor but get {type(quantized_data)}"
            )
        self.quantized_value_list: tuple[Tensor, ...] = tuple(values for values, _, _ in triples)
        self._min_values = tuple(lo for _, lo, _ in triples)
        self._max_values = tuple(hi for _, _, hi in triples)
        self.quantized_dtype = quantized_dtype
        self.computation_dtype = computation_dtype
        self.dequantized_value_list: tuple[Tensor, ...] | None = None
        self._workspace: tuple[Tensor, ...] | None = None  # kept between dequantize_ / quantize_ pairs

        assert all(values.dtype == quantized_dtype for values in self.quantized_value_list)
        assert computation_dtype in _FORMATS, (
            f"computation_dtype={computation_dtype} is not supported! It must be one of {_FLOAT_DTYPES}!"
        )
        with_range = sum(lo is not None and hi is not None for lo, hi in zip(self._min_values, self._max_values))
        without = sum(lo is None and hi is None for lo, hi in zip(self._min_values, self._max_values))
        assert with_range == len(triples) or without == len(triples), "either every entry has a (min, max) range or none has"

    def __len__(self) -> int:
        return len(self.quantized_value_list)

    # -- views ---------------------------------------------------------------------------------
    @property
    def quantized_value(self) -> tuple[Tensor, ...]:
        return self.quantized_value_list

    @property
    def dequantized_value(self) -> tuple[Tensor, ...]:
        assert self.dequantized_value_list is not None
        return self.dequantized_value_list

    def is_dequantized_stored(self) -> bool:
        return self.dequantized_value_list is not None

    # -- conversions that return / take tensors ------------------------------------------------
    def dequantize(self) -> tuple[Tensor, ...]:
        """Fresh computation-dtype copies (the stored tensors themselves when the dtypes agree)."""
        if self.quantized_dtype == self.computation_dtype:
            return self.quantized_value_list
        fmt = _format_of(self.quantized_dtype)
        out = _workspace_like(self.quantized_value_list, self.computation_dtype)
        fmt.load(self.quantized_value_list, out)
        return out

    def quantize(self, tensor_list: tuple[Tensor, ...]) -> None:
        """Store ``tensor_list`` (computation dtype) into the stored tensors."""
        if self.is_dequantized_stored() and tensor_list is not self.dequantized_value_list:
            logger.warning(
                "Existing stored dequantized values.\nWriting quantized values with input tensor_list without using these stored dequantized values..."
            )
        bounds = _format_of(self.quantized_dtype).store(tensor_list, self.quantized_value_list)
        self._min_values = tuple(lo for lo, _ in bounds)
        self._max_values = tuple(hi for _, hi in bounds)

    # -- the in-place pair used around a step ----------------------------------------------------
    def dequantize_(self) -> None:
        if self.is_dequantized_stored():
            logger.warning("Dequantized values are already stored; overwriting these values...")
        if self.quantized_dtype == self.computation_dtype:
            self.dequantized_value_list = self.quantized_value_list
            return
        fmt = _format_of(self.quantized_dtype)
        if self._workspace is None:
            self._workspace = _workspace_like(self.quantized_value_list, self.computation_dtype)
        fmt.load(self.quantized_value_list, self._workspace)
        self.dequantized_value_list = self._workspace

    def quantize_(self) -> None:
        if not self.is_dequantized_stored():
            logger.warning(
                f"No stored dequantized values self.dequantized_value_list={self.dequantized_value_list}. Must first call dequantize_()."
            )
            return
        working, self.dequantized_value_list = self.dequantized_value_list, None
        if self.quantized_dtype != self.computation_dtype:
            self.quantize(working)

    def compress(self, selector: tuple[bool, ...]) -> "QuantizedTensorList":
        """The sub-list of the entries whose selector is True (stored tensors are shared)."""
        assert not self.is_dequantized_stored()
        kept = [
            triple
            for triple in zip(self.quantized_value_list, self._min_values, self._max_values, strict=True)
        ]
        return QuantizedTensorList(compress_list(kept, selector), self.quantized_dtype, self.computation_dtype)


class DequantizeQuantizedTensorListContext(ParameterizeEnterExitContext):
    """``with`` block during which the list holds its computation-dtype copies; they are stored
    back (and dropped) on exit."""

    def __init__(self, quantized_tensor_list: QuantizedTensorList) -> None:
        super().__init__(
            input_with_enter_exit_context=quantized_tensor_list,
            enter_method_caller=QuantizedTensorList.dequantize_,
            exit_method_caller=QuantizedTensorList.quantize_,
        )
