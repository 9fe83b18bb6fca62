"""Shape merging, blocking, packing and load-balancing primitives."""

import math

import pytest
import torch

from optimizers_b200.config import AlignedMemoryCostModel, LoadBalancingConfig, PolynomialComputationalCostModel
from optimizers_b200.parallel.a2a import _compute_chunk_sizes
from optimizers_b200.parallel.fsdp import recover_rectangles
from optimizers_b200.utils import blocking as B


@pytest.mark.parametrize(
    "threshold,target,expected",
    [
        (10, 1, (32, 3, 64, 64)), (200, 1, (32, 192, 64)), (8192, 1, (96, 4096)), (1_000_000, 1, (96 * 4096,)),
        (10, 2, (32, 3, 64, 64)), (200, 2, (32, 192, 64)), (8192, 2, (96, 4096)), (1_000_000, 2, (32, 3 * 4096)),
        (8192, 3, (32, 3, 4096)), (8192, 4, (32, 3, 64, 64)), (8192, math.inf, (32, 3, 64, 64)),
    ],
)
def test_merge_small_dims_convolution_like(threshold, target, expected):
    assert B.merge_small_dims((32, 3, 64, 64), threshold, target) == expected


def test_merge_small_dims_special_shapes():
    assert B.merge_small_dims((1, 2, 1), 10, 1) == (2,)
    assert B.merge_small_dims((1, 1, 1), 10, 1) == (1,)
    assert B.merge_small_dims((1, 1, 1), 1, 1) == (1,)
    assert B.merge_small_dims((), 10, 1) == (1,)
    assert B.merge_small_dims((0,), 10, 1) == (0,)
    assert B.merge_small_dims((3, 0, 2), 10, 1) == (0,)
    assert B.merge_small_dims((1, 2, 5, 1), 10, math.inf) == (1, 2, 5, 1)


def test_multi_dim_split_and_block_slices_agree():
    t = torch.arange(5 * 7 * 3).reshape(5, 7, 3)
    blocks = B.multi_dim_split(t, 3)
    slices = B.block_slices(tuple(t.shape), 3)
    assert len(blocks) == len(slices) == 2 * 3 * 1
    for blk, sl in zip(blocks, slices):
        ref = t[tuple(slice(a, b) for a, b in sl)]
        assert torch.equal(blk, ref)
    assert B.multi_dim_split(t, math.inf) == (t,)
    assert [tuple(b.shape) for b in B.multi_dim_split(torch.zeros(4, 5), 2)] == [(2, 2), (2, 2), (2, 1)] * 2


def test_small_helpers():
    assert B.compress_list([1, 2, 3], (True, False, True)) == (1, 3)
    with pytest.raises(AssertionError):
        B.compress_list([1, 2], (True,))
    assert B.get_dtype_size(torch.bool) == 1 and B.get_dtype_size(torch.bfloat16) == 2
    assert B.get_dtype_size(torch.int64) == 8 and B.get_dtype_size(torch.float32) == 4
    assert list(B.generate_pairwise_indices([4, 3, 2])) == [(0, 4), (4, 7), (7, 9)]
    log = []
    with B.ParameterizeEnterExitContext(log, lambda l: l.append("in"), lambda l: l.append("out")):
        log.append("body")
    assert log == ["in", "body", "out"]


def _metas(sizes):
    return tuple(torch.empty(s, dtype=torch.int8, device="meta") for s in sizes)


@pytest.mark.parametrize(
    "sizes,groups,cfg,expected",
    [
        ((128, 64, 500, 256), 2, LoadBalancingConfig(), ((128, 1), (64, 1), (512, 0), (256, 1))),
        ((128, 64, 500, 256), 1, LoadBalancingConfig(), ((128, 0), (64, 0), (512, 0), (256, 0))),
        ((128, 64), 4, LoadBalancingConfig(), ((128, 0), (64, 1))),
        ((), 2, LoadBalancingConfig(), ()),
        ((128, 64, 512, 256), 2, LoadBalancingConfig(cost_model=PolynomialComputationalCostModel(coefficients=(0, 2))),
         ((128, 1), (64, 1), (512, 0), (256, 1))),
        ((256, 128, 384, 256), 2, LoadBalancingConfig(cost_model=PolynomialComputationalCostModel(coefficients=(0, 0, 1))),
         ((256, 1), (128, 1), (384, 0), (256, 1))),
    ],
)
def test_distribute_buffer_sizes(sizes, groups, cfg, expected):
    assert B.distribute_buffer_sizes(_metas(sizes), groups, cfg) == expected


def test_cost_models():
    assert AlignedMemoryCostModel().cost(torch.empty(65, dtype=torch.int8)) == 128
    assert AlignedMemoryCostModel(alignment_bytes=16).cost(torch.empty(5, dtype=torch.float32)) == 32
    model = PolynomialComputationalCostModel(coefficients=(1, 0, 2), min_cost=10)
    assert model.cost(torch.empty(2, 3)) == max(10, 1 + 2 * 4) + max(10, 1 + 2 * 9)


def test_lpt_ties_and_bin_pack():
    owners, loads = B.lpt_assign([5, 5, 5, 5], 2)
    assert owners == [0, 1, 0, 1] and loads == [10.0, 10.0]
    bins, costs = B.greedy_bin_pack(["a", "bb", "ccc", "dddd"], 2, cost_fn=len)
    assert sorted(map(sorted, bins)) == [["a", "dddd"], ["bb", "ccc"]] and sorted(costs) == [5, 5]


@pytest.mark.parametrize("d", [1, 2, 3, 5, 8])
def test_pack_unpack_round_trip(d):
    m = torch.randn(d, d)
    sym = m + m.T
    packed = B.pack_upper_triangular(sym)
    assert packed.shape == (d * (d + 1) // 2,) == (B.packed_size(d),)
    assert torch.equal(B.unpack_upper_triangular(packed, d), sym)
    for i in range(d):
        assert packed[B.packed_row_offset(i, d)] == sym[i, i]
    assert torch.equal(
        B.pack_upper_triangular(torch.tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0], [7.0, 8.0, 9.0]])),
        torch.tensor([1.0, 2.0, 3.0, 5.0, 6.0, 9.0]),
    )
    for dtype in (torch.float64, torch.bfloat16):
        assert B.pack_upper_triangular(torch.zeros(3, 3, dtype=dtype)).dtype == dtype


@pytest.mark.parametrize("numel", [0, 1, 3, 7, 8, 9, 16, 17])
@pytest.mark.parametrize("chunks", [1, 2, 4, 8])
def test_chunk_sizes_match_torch_chunk(numel, chunks):
    got = _compute_chunk_sizes(numel, chunks)
    want = [c.shape[0] for c in torch.chunk(torch.zeros(numel), chunks)] if numel else []
    want += [0] * (chunks - len(want))
    assert got == want and sum(got) == numel


@pytest.mark.parametrize("shape", [(4, 6), (2, 3, 4), (7,), (3, 1, 5)])
def test_recover_rectangles_cover_the_range_with_rectangles(shape):
    n = math.prod(shape)
    flat = torch.arange(n)
    full = flat.view(shape)
    for start in range(0, n, 3):
        for end in range(start, n + 1, 4):
            pieces = recover_rectangles(shape, start, end)
            covered = []
            for flat_start, piece_shape in pieces:
                size = math.prod(piece_shape)
                piece = flat[flat_start : flat_start + size].view(piece_shape)
                covered.extend(piece.flatten().tolist())
                # a rectangle: trailing dims are whole trailing dims of the tensor
                assert tuple(piece_shape[1:]) == tuple(shape[len(shape) - len(piece_shape) + 1 :])
            assert covered == list(range(start, end))


def test_split_param_groups_passthrough_for_other_configs():
    from optimizers_b200.config import DefaultSingleDeviceDistributedConfig

    groups = [{"params": [torch.zeros(2)], "distributed_config": DefaultSingleDeviceDistributedConfig}]
    assert B.split_param_groups(groups) == groups


def test_against_reference_utils():
    from ref_oracle import reference, reference_available

    if not reference_available():
        pytest.skip("reference not installed")
    reference()
    from distributed_shampoo.utils import shampoo_utils as R

    for shape in [(3, 4, 5), (64, 3, 3, 3), (1, 7, 1, 9), (2048, 768), (5,), ()]:
        for th in (1, 8, 16, 100, 10_000):
            for target in (1, 2, 3, math.inf):
                assert B.merge_small_dims(shape, th, target) == R.merge_small_dims(shape, th, target)
    g = torch.Generator().manual_seed(0)
    for trial in range(20):
        sizes = torch.randint(1, 5000, (int(torch.randint(1, 30, (1,), generator=g)),), generator=g).tolist()
        blocks = _metas(sizes)
        for groups in (1, 2, 3, 8):
            assert B.distribute_buffer_sizes(blocks, groups, LoadBalancingConfig()) == R.distribute_buffer_sizes(
                blocks, groups, R.LoadBalancingConfig()
            )
        bins_a = B.greedy_bin_pack(sizes, 3, cost_fn=lambda x: x)
        bins_b = R.greedy_bin_pack(sizes, 3, cost_fn=lambda x: x)
        assert bins_a == bins_b


def test_random_shapes_block_like_the_reference():
    """Property test: for random parameter shapes, merge thresholds and block sizes, the merged
    shape, the shapes and contents of the blocks and the split of a list of parameter groups agree
    with the reference's ``utils/shampoo_utils.py``; so does the whole optimizer's block list
    (``distributor/shampoo_distributor.py`` there), compared through the state keys."""
    from hypothesis import given, settings, strategies as st

    from ref_oracle import reference, reference_available

    if not reference_available():
        pytest.skip("reference not installed")
    ref = reference()
    from distributed_shampoo.utils import shampoo_utils as R

    import optimizers_b200 as ob

    shapes = st.lists(st.integers(1, 9), min_size=0, max_size=4).map(tuple)

    @settings(max_examples=150, deadline=None)
    @given(shape=shapes, threshold=st.integers(1, 200), target=st.sampled_from([1, 2, 3, math.inf]),
           block=st.sampled_from([1, 2, 3, 5, 8, math.inf]))
    def check(shape, threshold, target, block):
        merged = B.merge_small_dims(shape, threshold, target)
        assert merged == R.merge_small_dims(shape, threshold, target)
        numel = math.prod(shape)
        t = torch.arange(numel, dtype=torch.float32).reshape(merged)
        mine, theirs = B.multi_dim_split(t, block), R.multi_dim_split(t, block)
        assert len(mine) == len(theirs)
        assert all(torch.equal(a, b) for a, b in zip(mine, theirs))

    check()

    @settings(max_examples=25, deadline=None)
    @given(shape_list=st.lists(st.lists(st.integers(1, 7), min_size=1, max_size=3).map(tuple), min_size=1, max_size=4),
           block=st.sampled_from([2, 3, 4, 8]), target=st.sampled_from([1, 2, math.inf]))
    def check_optimizer(shape_list, block, target):
        keys = []
        for lib in (ref, ob):
            params = [torch.nn.Parameter(torch.zeros(s)) for s in shape_list]
            opt = lib.DistributedShampoo(
                params, max_preconditioner_dim=block, precondition_frequency=1,
                distributed_config=lib.SingleDeviceDistributedConfig(target_parameter_dimensionality=target),
            )
            for p in params:
                p.grad = torch.ones_like(p)
            opt.step()
            state = opt.state_dict()["state"]
            keys.append({
                index: sorted((name, tuple(value["filtered_grad"].shape) if "filtered_grad" in value else ()) for name, value in entry.items() if name.startswith("block_"))
                for index, entry in state.items()
            })
        assert keys[0] == keys[1]

    check_optimizer()
