"""Helper idioms, quantization shell, CombinedLinear."""

import pytest
import torch

from optimizers_b200.parallel.block_info import BlockInfo
from optimizers_b200.utils.misc import batched, DictZipIterator, get_all_non_abstract_subclasses
from optimizers_b200.utils.model_utils import CombinedLinear
from optimizers_b200.utils.quantization import DequantizeQuantizedTensorListContext, QuantizedTensor, QuantizedTensorList


def test_dict_zip_iterator_and_batched():
    assert list(DictZipIterator({"a": [1, 2], "b": "xy"})) == [{"a": 1, "b": "x"}, {"a": 2, "b": "y"}]
    with pytest.raises(ValueError, match="different lengths"):
        list(DictZipIterator({"a": [1, 2], "b": [1]}))
    assert list(batched(range(5), 2)) == [(0, 1), (2, 3), (4,)]
    with pytest.raises(ValueError):
        list(batched([1], 0))


def test_non_abstract_subclasses():
    from optimizers_b200 import config as C

    found = set(get_all_non_abstract_subclasses(C.RootInvConfig))
    assert {C.EigenConfig, C.CoupledNewtonConfig, C.CoupledHigherOrderConfig} <= found and C.RootInvConfig not in found


def test_quantized_tensor_list_round_trip():
    info = BlockInfo(param=torch.zeros(1), composable_block_ids=(0, "block_0"))
    values = [torch.randn(3, 3), torch.randn(5)]
    stored = [QuantizedTensor.init_from_dequantized_tensor(v, torch.bfloat16, info) for v in values]
    qlist = QuantizedTensorList(stored, torch.bfloat16, torch.float32)
    assert len(qlist) == 2 and not qlist.is_dequantized_stored()
    with DequantizeQuantizedTensorListContext(qlist):
        assert qlist.dequantized_value[0].dtype == torch.float32
        torch._foreach_mul_(qlist.dequantized_value, 2.0)
    assert not qlist.is_dequantized_stored()
    for q, v in zip(qlist.quantized_value, values):
        torch.testing.assert_close(q.float(), (v.bfloat16().float() * 2).bfloat16().float())
    assert len(qlist.compress((True, False))) == 1
    assert stored[0].dequantize(torch.bfloat16) is stored[0].quantized_values
    with pytest.raises(NotImplementedError):
        QuantizedTensorList([(torch.zeros(2, dtype=torch.int8), torch.zeros(1), torch.zeros(1))], torch.int8).dequantize()


@pytest.mark.parametrize("bias", [True, False])
def test_combined_linear_matches_linear(bias):
    torch.manual_seed(0)
    layer = CombinedLinear(5, 3, bias=bias)
    ref = torch.nn.Linear(5, 3, bias=bias)
    with torch.no_grad():
        if bias:
            ref.weight.copy_(layer.combined_weight[:, :-1])
            ref.bias.copy_(layer.combined_weight[:, -1])
        else:
            ref.weight.copy_(layer.combined_weight)
    x = torch.randn(4, 5)
    torch.testing.assert_close(layer(x), ref(x))
    assert layer.combined_weight.shape == (3, 5 + int(bias))


def test_quantized_tensor_list_workspace_warnings_and_edge_cases(caplog):
    """Behaviours pinned by the reference's ``utils/tests/shampoo_quantization_test.py``, plus the
    properties of this implementation: the in-place pair reuses one flat workspace, the copying
    ``dequantize`` hands out fresh tensors."""
    import logging

    triples = [(torch.full((3, 2), float(i), dtype=torch.float16), None, None) for i in range(5)]
    qlist = QuantizedTensorList(triples, torch.float16, torch.float64)
    assert len(qlist) == 5 and len(qlist.compress((True, False, True, False, False))) == 2

    with caplog.at_level(logging.WARNING):
        qlist.quantize_()  # nothing to store yet
    assert "Must first call dequantize_()" in caplog.text and not qlist.is_dequantized_stored()

    qlist.dequantize_()
    first = qlist.dequantized_value
    assert all(t.dtype == torch.float64 for t in first)
    # one flat allocation: the views follow each other in one storage
    assert len({t.untyped_storage().data_ptr() for t in first}) == 1
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        qlist.dequantize_()
    assert "already stored" in caplog.text
    torch._foreach_add_(qlist.dequantized_value, 0.5)
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        qlist.quantize(tuple(torch.zeros(3, 2, dtype=torch.float64) for _ in range(5)))
    assert "Existing stored dequantized values" in caplog.text
    qlist.quantize_()
    assert not qlist.is_dequantized_stored()
    for i, t in enumerate(qlist.quantized_value):
        assert t.dtype == torch.float16 and torch.equal(t, torch.full((3, 2), i + 0.5, dtype=torch.float16))
    qlist.dequantize_()
    assert qlist.dequantized_value[0].data_ptr() == first[0].data_ptr()  # the workspace is kept
    qlist.quantize_()
    fresh = qlist.dequantize()
    assert fresh[0].data_ptr() != first[0].data_ptr() and torch.equal(fresh[2], torch.full((3, 2), 2.5, dtype=torch.float64))

    same = QuantizedTensorList(triples, torch.float16, torch.float16)
    assert same.dequantize() is same.quantized_value
    with DequantizeQuantizedTensorListContext(same):
        assert same.dequantized_value is same.quantized_value
    assert not same.is_dequantized_stored()

    assert len(QuantizedTensorList([], torch.float16)) == 0
    with pytest.raises(TypeError, match="quantized_data must be"):
        QuantizedTensorList([torch.zeros(2)], torch.float32)
    with pytest.raises(AssertionError, match="is not supported"):
        QuantizedTensorList(triples, torch.float16, torch.int8)
    with pytest.raises(AssertionError):
        QuantizedTensorList([(torch.zeros(2, dtype=torch.int8), torch.zeros(1), None)], torch.int8)
    info = BlockInfo(param=torch.zeros(1), composable_block_ids=(0, "block_0"))
    assert QuantizedTensor(torch.zeros(4, dtype=torch.int8), info).min_value is not None
    with pytest.raises(NotImplementedError, match="Quantization for torch.int8"):
        QuantizedTensor(torch.zeros(4, dtype=torch.int8), info).dequantize(torch.float32)
    with pytest.raises(NotImplementedError):
        QuantizedTensor(torch.zeros(4, dtype=torch.int8), info).quantize(torch.ones(4))
