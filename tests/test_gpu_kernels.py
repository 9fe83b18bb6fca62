"""GPU numerics of the sm_100a kernels against plain PyTorch fp32/fp64 references."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from optimizers_b200.ops import build

    return build.load()


def _pad4(n):
    return (n + 3) // 4 * 4


def _split(ext, x):
    rows, k = x.shape
    hi = torch.zeros(rows, _pad4(k), device=x.device)
    lo = torch.zeros_like(hi)
    ext.tf32_split(x, hi[:, :k], lo[:, :k])
    return hi[:, :k], lo[:, :k]


def _packed(full):
    d = full.shape[0]
    r, c = torch.triu_indices(d, d, device=full.device)
    return full[r, c].contiguous()


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize(
    "M,N,K", [(128, 128, 32), (128, 128, 256), (256, 384, 100), (1, 200, 200), (37, 5, 7), (300, 129, 1000), (513, 64, 36)]
)
def test_grouped_gemm_full(ext, split, M, N, K):
    torch.manual_seed(M * 7 + N * 3 + K)
    dev = torch.device("cuda")
    A = torch.randn(M, K, device=dev)
    B = torch.randn(N, K, device=dev)
    C0 = torch.randn(M, N, device=dev)
    C = C0.clone()
    a_hi, a_lo = _split(ext, A)
    b_hi, b_lo = _split(ext, B)
    if not split:
        # raw operands in padded storage
        a_hi = torch.zeros(M, _pad4(K), device=dev)[:, :K].copy_(A)
        b_hi = torch.zeros(N, _pad4(K), device=dev)[:, :K].copy_(B)
        a_lo = b_lo = None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sumsq = torch.zeros(1, device=dev)
    plan = ext.build_gemm_plan([(a_hi, a_lo, b_hi, b_lo, C, None, None, sumsq, N, 0, ext.FLAG_SUMSQ, False)])
    ext.run_gemm_plan(*plan, 0.5, 2.0, split, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = 2.0 * C0.double() + 0.5 * (A.double() @ B.double().T)
    scale = math.sqrt(K)
    tol = 2e-5 * scale if split else 4e-3 * scale
    assert (C.double() - ref).abs().max().item() < tol
    assert abs(sumsq.item() - (ref**2).sum().item()) <= 1e-2 * (ref**2).sum().item() + 1e-3


@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("d,K", [(128, 64), (200, 300), (384, 32), (5, 3), (129, 1024)])
def test_grouped_syrk_packed_ema(ext, split, d, K):
    torch.manual_seed(d + K)
    dev = torch.device("cuda")
    X = torch.randn(d, K, device=dev)
    F0 = torch.randn(d, d, device=dev)
    F0 = F0 @ F0.T
    Fp = _packed(F0)
    x_hi, x_lo = _split(ext, X)
    if not split:
        x_hi = torch.zeros(d, _pad4(K), device=dev)[:, :K].copy_(X)
        x_lo = None
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    plan = ext.build_gemm_plan([(x_hi, x_lo, x_hi, x_lo, Fp, None, None, None, d, 0, ext.FLAG_PACKED_C, True)])
    ext.run_gemm_plan(*plan, 0.25, 0.9, split, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = _packed((0.9 * F0.double() + 0.25 * (X.double() @ X.double().T)).float())
    # tensor-core fp32 accumulation truncates, so the error grows with the magnitude of the sums
    tol = (2e-5 if split else 4e-3) * math.sqrt(K) + (3e-5 if split else 2e-3) * ref.abs().max().item()
    assert (Fp - ref).abs().max().item() < tol


def test_grouped_gemm_many_problems_and_split_out(ext):
    torch.manual_seed(0)
    dev = torch.device("cuda")
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    specs, checks = [], []
    for i, (M, N, K) in enumerate([(130, 70, 90), (64, 64, 64), (400, 300, 200), (17, 257, 33)] * 3):
        A, B = torch.randn(M, K, device=dev), torch.randn(N, K, device=dev)
        a_hi, a_lo = _split(ext, A)
        b_hi, b_lo = _split(ext, B)
        d_hi = torch.zeros(M, _pad4(N), device=dev)
        d_lo = torch.zeros_like(d_hi)
        specs.append((a_hi, a_lo, b_hi, b_lo, None, d_hi, d_lo, None, 0, _pad4(N), ext.FLAG_NO_C | ext.FLAG_SPLIT_OUT, False))
        checks.append((A, B, d_hi, d_lo, N, K))
    plan = ext.build_gemm_plan(specs)
    ext.run_gemm_plan(*plan, 1.0, 0.0, True, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    for A, B, d_hi, d_lo, N, K in checks:
        ref = A.double() @ B.double().T
        got = d_hi[:, :N].double() + d_lo[:, :N].double()
        assert (got - ref).abs().max().item() < 2e-5 * math.sqrt(K)
        # hi must be representable in tf32: the 13 low mantissa bits are zero
        assert (d_hi.view(torch.int32) & 0x1FFF).abs().max().item() == 0


def _mlp(dev):
    torch.manual_seed(0)
    return torch.nn.Sequential(
        torch.nn.Linear(96, 200), torch.nn.ReLU(), torch.nn.Linear(200, 72), torch.nn.ReLU(), torch.nn.Linear(72, 10)
    ).to(dev)


def _train(backend, steps, **kw):
    from optimizers_b200 import DistributedShampoo, NativeRuntimeConfig

    dev = torch.device("cuda")
    model = _mlp(dev)
    opt = DistributedShampoo(
        model.parameters(), native_runtime_config=NativeRuntimeConfig(backend=backend), **kw
    )
    if hasattr(opt, "train"):
        opt.train()
    g = torch.Generator(device="cuda").manual_seed(1)
    losses = []
    for _ in range(steps):
        x = torch.randn(64, 96, device=dev, generator=g)
        y = torch.randint(0, 10, (64,), device=dev, generator=g)
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return model, opt, losses


def _configs():
    from optimizers_b200 import (
        AdaGradPreconditionerConfig,
        AdamPreconditionerConfig,
        ClassicMomentumConfig,
        EigendecomposedKLShampooPreconditionerConfig,
        EigendecomposedShampooPreconditionerConfig,
        EigenvalueCorrectedShampooPreconditionerConfig,
        GeneralizedPrimalAveragingConfig,
        QREigendecompositionConfig,
        RootInvKLShampooPreconditionerConfig,
        RootInvShampooPreconditionerConfig,
        SGDPreconditionerConfig,
        WeightDecayType,
    )

    base = dict(lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64, precondition_frequency=3, start_preconditioning_step=3)
    return {
        "adam_graft": dict(base, grafting_config=AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8)),
        "adagrad_graft_wd": dict(base, grafting_config=AdaGradPreconditionerConfig(), weight_decay=1e-2),
        "sgd_graft_l2_momentum": dict(
            base, grafting_config=SGDPreconditionerConfig(), weight_decay=1e-3, weight_decay_type=WeightDecayType.L2,
            iterate_averaging_config=ClassicMomentumConfig(momentum=0.5, use_nesterov=True),
        ),
        "no_graft_unpacked_beta3": dict(
            base, beta3=0.8, preconditioner_config=RootInvShampooPreconditionerConfig(use_symmetric_packing=False)
        ),
        "eigendecomposed_adam_graft": dict(
            base, grafting_config=AdamPreconditionerConfig(), weight_decay=1e-2,
            preconditioner_config=EigendecomposedShampooPreconditionerConfig(),
        ),
        "kl_rootinv_adam_graft": dict(
            base, grafting_config=AdamPreconditionerConfig(), preconditioner_config=RootInvKLShampooPreconditionerConfig(),
        ),
        "kl_eigendecomposed_no_graft": dict(base, preconditioner_config=EigendecomposedKLShampooPreconditionerConfig()),
        "soap_adam_graft": dict(
            base, grafting_config=AdamPreconditionerConfig(), weight_decay=1e-2,
            preconditioner_config=EigenvalueCorrectedShampooPreconditionerConfig(),
        ),
        "soap_qr_no_graft": dict(
            base, preconditioner_config=EigenvalueCorrectedShampooPreconditionerConfig(
                amortized_computation_config=QREigendecompositionConfig(), use_symmetric_packing=False),
        ),
        "gpa": dict(
            base, grafting_config=AdamPreconditionerConfig(), weight_decay=1e-2,
            iterate_averaging_config=GeneralizedPrimalAveragingConfig(eval_interp_coeff=0.9, train_interp_coeff=0.7),
        ),
    }


@pytest.mark.parametrize(
    "name",
    ["adam_graft", "adagrad_graft_wd", "sgd_graft_l2_momentum", "no_graft_unpacked_beta3", "gpa", "soap_adam_graft",
     "soap_qr_no_graft", "eigendecomposed_adam_graft", "kl_rootinv_adam_graft", "kl_eigendecomposed_no_graft"],
)
def test_native_engine_matches_torch_step(name):
    kw = _configs()[name]
    m_ref, o_ref, l_ref = _train("torch", 8, **kw)
    m_nat, o_nat, l_nat = _train("native", 8, **kw)
    for rec in o_nat._per_group_state_lists:
        assert rec["native_engine"] is not None
        rec["native_engine"].check_status()
    for a, b in zip(l_ref, l_nat):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (l_ref, l_nat)
    # The eigenbasis of nearly degenerate factors reacts to 1e-5 perturbations of the factors, and
    # the per-coordinate scaling in that basis amplifies it: a wider band for the SOAP variants.
    atol = 4e-3 if name.startswith("soap") else 5e-4
    for p, q in zip(m_ref.parameters(), m_nat.parameters()):
        assert torch.allclose(p, q, rtol=5e-3, atol=atol), (p - q).abs().max()
    if name == "gpa":  # train -> eval -> train through the grouped mode-switch kernel
        for o in (o_ref, o_nat):
            o.eval()
        for p, q in zip(m_ref.parameters(), m_nat.parameters()):
            assert torch.allclose(p, q, rtol=5e-3, atol=5e-4)
        o_nat.train()
        o_ref.train()
    if name.startswith("soap") or "eigendecomposed" in name:
        return  # eigenvectors are only defined up to sign/rotation: compare parameters, not the state tree
    # optimizer state trees agree as well (factor matrices are the sensitive part)
    s_ref, s_nat = o_ref.state_dict()["state"], o_nat.state_dict()["state"]

    def walk(a, b, path=""):
        if isinstance(a, dict):
            assert a.keys() == b.keys(), path
            for k in a:
                walk(a[k], b[k], f"{path}/{k}")
        elif isinstance(a, torch.Tensor) and a.is_floating_point() and a.numel():
            denom = a.abs().max().item() + 1e-12
            assert (a - b).abs().max().item() / denom < 2e-2, path

    walk(s_ref, s_nat)


@pytest.mark.parametrize("eigdec", [False, True])
@pytest.mark.parametrize(
    "override",
    [{2: {0: 0.25, 1: 0.0}}, {2: {0: 0.0, 1: 0.5}}, {2: 0.0}, {1: 0.0, 2: {0: 0.5, 1: 0.0}}, {1: 0.0, 2: 0.0}],
    ids=["rows_only", "columns_only", "no_dim_of_matrices", "vectors_off_rows_only", "nothing"],
)
def test_native_engine_with_unpreconditioned_dims_matches_torch_step(override, eigdec):
    """An exponent of 0 leaves a dim without a Kronecker factor (reference:
    distributed_shampoo/preconditioner/shampoo_preconditioner_list.py:1749-1756): one-sided products,
    and blocks whose direction is the filtered gradient itself."""
    from optimizers_b200 import (
        AdamPreconditionerConfig,
        EigendecomposedShampooPreconditionerConfig,
        RootInvShampooPreconditionerConfig,
    )

    cls = EigendecomposedShampooPreconditionerConfig if eigdec else RootInvShampooPreconditionerConfig
    kw = dict(
        lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64, precondition_frequency=3,
        start_preconditioning_step=3, grafting_config=AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8), weight_decay=1e-2,
        preconditioner_config=cls(inverse_exponent_override=override),
    )
    m_ref, _, l_ref = _train("torch", 8, **kw)
    m_nat, o_nat, l_nat = _train("native", 8, **kw)
    for rec in o_nat._per_group_state_lists:
        assert rec["native_engine"] is not None
        rec["native_engine"].check_status()
    for a, b in zip(l_ref, l_nat):
        assert abs(a - b) < 2e-3 * max(1.0, abs(a)), (l_ref, l_nat)
    for p, q in zip(m_ref.parameters(), m_nat.parameters()):
        assert torch.allclose(p, q, rtol=5e-3, atol=5e-4), (p - q).abs().max()


@pytest.mark.parametrize("name", ["soap_adam_graft", "soap_qr_no_graft"])
def test_native_soap_before_first_refresh_is_exact(name):
    """Before the first refresh the eigenbases are identities, so project / second-moment update /
    scale / unproject must reproduce the torch step to rounding: a tight check of the plumbing
    that the chaotic multi-refresh comparison cannot give."""
    kw = _configs()[name]
    m_ref, _, _ = _train("torch", 2, **kw)
    m_nat, o_nat, _ = _train("native", 2, **kw)
    o_nat._per_group_state_lists[0]["native_engine"].check_status()
    for p, q in zip(m_ref.parameters(), m_nat.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=2e-6), (p - q).abs().max()


def test_gpa_adamw_kernel_matches_torch_loop():
    from optimizers_b200.gpa_adamw import GPAAdamW

    dev = torch.device("cuda")
    results = []
    for native in (False, True):
        torch.manual_seed(0)
        model = _mlp(dev)
        opt = GPAAdamW(model.parameters(), lr=1e-2, weight_decay=1e-2, use_native_kernels=native)
        opt.train()
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(6):
            x = torch.randn(32, 96, device=dev, generator=g)
            y = torch.randint(0, 10, (32,), device=dev, generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        opt.eval()
        results.append([p.detach().clone() for p in model.parameters()])
    for a, b in zip(*results):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("split", [True, False])
def test_native_newton_refresh_matches_eigen_roots(split):
    """Batched coupled-Newton refresh on the grouped GEMM against the fp64 eigendecomposition."""
    from optimizers_b200 import CoupledNewtonConfig, DistributedShampoo, NativeRuntimeConfig, RootInvShampooPreconditionerConfig

    dev = torch.device("cuda")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(150, 200), torch.nn.ReLU(), torch.nn.Linear(200, 40)).to(dev)
    opt = DistributedShampoo(
        model.parameters(), lr=1e-3, epsilon=1e-4, max_preconditioner_dim=128, precondition_frequency=1,
        preconditioner_config=RootInvShampooPreconditionerConfig(amortized_computation_config=CoupledNewtonConfig(tolerance=1e-5)),
        native_runtime_config=NativeRuntimeConfig(backend="native", gemm_mode="tf32x3" if split else "tf32"),
    )
    x = torch.randn(256, 150, device=dev)
    model(x).square().mean().backward()
    opt.step()
    engine = opt._per_group_state_lists[0]["native_engine"]
    engine.check_status()
    checked = 0
    for b in engine._blocks:
        kf = b.factors
        for F, X, root in zip(kf.get_unpacked_factor_matrices(), kf.get_unpacked_inv_factor_matrices(), kf.roots):
            A = F.double() + 1e-4 * torch.eye(F.shape[0], device=dev, dtype=torch.float64)
            lam, Q = torch.linalg.eigh(A)
            want = (Q * lam.pow(-1.0 / root)) @ Q.T
            rel = (X.double() - want).abs().max() / want.abs().max()
            assert rel < 2e-3, (F.shape, root, rel)
            checked += 1
    assert checked >= 6


@pytest.mark.parametrize("order,exponent", [(3, 0.25), (2, 0.25), (4, 0.5), (3, 2.0 / 3.0)])
def test_native_higher_order_refresh_matches_eigen_roots(order, exponent):
    """Batched coupled higher-order iteration on the grouped GEMM (Horner products in I - M, Newton
    first step, verification of A_r X^p and the q-th power of a fractional root p / q) against the
    fp64 eigendecomposition of the same ridged matrix."""
    from fractions import Fraction

    from optimizers_b200 import CoupledHigherOrderConfig, DistributedShampoo, NativeRuntimeConfig, RootInvShampooPreconditionerConfig

    dev = torch.device("cuda")
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(150, 200), torch.nn.ReLU(), torch.nn.Linear(200, 40)).to(dev)
    cfg = CoupledHigherOrderConfig(rel_epsilon=1e-4, abs_epsilon=1e-8, order=order, tolerance=1e-6)
    opt = DistributedShampoo(
        model.parameters(), lr=1e-3, epsilon=1e-4, max_preconditioner_dim=128, precondition_frequency=1,
        preconditioner_config=RootInvShampooPreconditionerConfig(
            amortized_computation_config=cfg, inverse_exponent_override={2: exponent}
        ),
        native_runtime_config=NativeRuntimeConfig(backend="native"),
    )
    x = torch.randn(256, 150, device=dev)
    model(x).square().mean().backward()
    opt.step()
    engine = opt._per_group_state_lists[0]["native_engine"]
    assert engine is not None
    engine.check_status()
    checked = 0
    for b in engine._blocks:
        kf = b.factors
        if len(kf.roots) != 2:
            continue
        for F, X, root in zip(kf.get_unpacked_factor_matrices(), kf.get_unpacked_inv_factor_matrices(), kf.roots):
            assert Fraction(root).limit_denominator(64) == Fraction(1 / exponent).limit_denominator(64)
            F = F.double()
            ridge = max(F.abs().sum(dim=1).max().item() * 1e-4, 1e-8)
            lam, Q = torch.linalg.eigh(F + ridge * torch.eye(F.shape[0], device=dev, dtype=torch.float64))
            want = (Q * lam.pow(-exponent)) @ Q.T
            rel = (X.double() - want).abs().max() / want.abs().max()
            assert rel < 2e-3, (F.shape, root, rel)
            checked += 1
    assert checked >= 4


@pytest.mark.parametrize("split", [True, False])
def test_batched_newton_schulz_matches_torch(split):
    from optimizers_b200.matrix import functions as mf
    from optimizers_b200.matrix.batched import BatchedNewtonSchulz
    from optimizers_b200.ops import build

    torch.manual_seed(0)
    shapes = [(200, 96), (64, 300), (128, 128), (33, 7)]
    mats = [torch.randn(m, n, device="cuda") for m, n in shapes]
    coeffs = (3.4445, -4.7750, 2.0315)
    runner = BatchedNewtonSchulz(build.load(), shapes, torch.device("cuda"), split=split)
    for _ in range(2):  # buffers are reused across calls
        got = runner(mats, 5, coeffs)
    runner.check_status()
    for A, X in zip(mats, got):
        want = mf.newton_schulz(A, 5, coeffs)
        tol = 2e-4 if split else 3e-2
        assert X.shape == want.shape
        assert (X - want).abs().max().item() < tol * max(1.0, want.abs().max().item()), (A.shape, (X - want).abs().max())


def test_spectral_descent_native_matches_torch():
    from optimizers_b200 import (
        DistributedShampoo,
        NativeRuntimeConfig,
        SingleDeviceDistributedConfig,
        SpectralDescentPreconditionerConfig,
    )

    results = []
    for backend in ("torch", "auto"):
        torch.manual_seed(0)
        model = torch.nn.Sequential(torch.nn.Linear(96, 160, bias=False), torch.nn.Tanh(), torch.nn.Linear(160, 24, bias=False)).cuda()
        opt = DistributedShampoo(
            model.parameters(), lr=1e-2, betas=(0.9, 1.0), epsilon=1e-12, max_preconditioner_dim=4096,
            preconditioner_config=SpectralDescentPreconditionerConfig(), grafting_config=None,
            distributed_config=SingleDeviceDistributedConfig(target_parameter_dimensionality=2),
            native_runtime_config=NativeRuntimeConfig(backend=backend),
        )
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(5):
            x = torch.randn(32, 96, device="cuda", generator=g)
            opt.zero_grad()
            model(x).square().mean().backward()
            opt.step()
        results.append([p.detach().clone() for p in model.parameters()])
    for a, b in zip(*results):
        assert torch.allclose(a, b, rtol=1e-3, atol=2e-4), (a - b).abs().max()


@pytest.mark.parametrize("graft", ["adam", "none"])
def test_native_engine_order3_blocks_match_torch_step(graft):
    """Convolution kernels whose dims stay unmerged become order-3 blocks (out, in, kh*kw): three
    Kronecker factors with root 6, preconditioned by three chained GEMMs with rotating layouts."""
    from optimizers_b200 import AdamPreconditionerConfig, DistributedShampoo, NativeRuntimeConfig

    results = []
    for backend in ("torch", "native"):
        torch.manual_seed(0)
        model = torch.nn.Sequential(
            torch.nn.Conv2d(64, 64, 3, padding=1, bias=False), torch.nn.ReLU(), torch.nn.Conv2d(64, 32, 3, padding=1),
            torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(32, 10),
        ).cuda()
        opt = DistributedShampoo(
            model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64,
            precondition_frequency=3, start_preconditioning_step=3, weight_decay=1e-2,
            grafting_config=AdamPreconditionerConfig() if graft == "adam" else None,
            native_runtime_config=NativeRuntimeConfig(backend=backend),
        )
        orders = sorted({b.dim() for b in opt._per_group_state_lists[0]["distributor"].local_blocked_params})
        assert 3 in orders, orders
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(8):
            x = torch.randn(16, 64, 8, 8, device="cuda", generator=g)
            y = torch.randint(0, 10, (16,), device="cuda", generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        if backend == "native":
            eng = opt._per_group_state_lists[0]["native_engine"]
            assert eng is not None
            eng.check_status()
        results.append(([p.detach().clone() for p in model.parameters()], opt.state_dict()["state"]))
    for p, q in zip(results[0][0], results[1][0]):
        assert torch.allclose(p, q, rtol=5e-3, atol=5e-4), (p - q).abs().max()

    def walk(a, b, path=""):
        if isinstance(a, dict):
            assert a.keys() == b.keys(), path
            for k in a:
                walk(a[k], b[k], f"{path}/{k}")
        elif isinstance(a, torch.Tensor) and a.is_floating_point() and a.numel():
            denom = a.abs().max().item() + 1e-12
            assert (a - b).abs().max().item() / denom < 5e-2, path  # 8 steps of a ReLU conv net amplify 1e-5 differences

    walk(results[0][1], results[1][1])


def test_native_engine_order3_blocks_with_eigenvalue_correction_match_torch_step():
    """Order-3 blocks under eigenvalue-corrected Shampoo: raw and filtered gradient projected through
    the three eigenbases side by side (second moment in the eigenbasis from the squared-EMA epilogue),
    the scaled direction taken back through them.  The first refresh waits for twelve steps so that the
    9 x 9 factor of the kernel window has distinct eigenvalues."""
    from optimizers_b200 import (
        AdamPreconditionerConfig,
        DistributedShampoo,
        EigenvalueCorrectedShampooPreconditionerConfig,
        NativeRuntimeConfig,
    )

    results = []
    for backend in ("torch", "native"):
        torch.manual_seed(0)
        model = torch.nn.Sequential(
            torch.nn.Conv2d(64, 64, 3, padding=1, bias=False), torch.nn.ReLU(), torch.nn.Conv2d(64, 32, 3, padding=1),
            torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(32, 10),
        ).cuda()
        opt = DistributedShampoo(
            model.parameters(), lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64,
            precondition_frequency=12, start_preconditioning_step=12, weight_decay=1e-2,
            grafting_config=AdamPreconditionerConfig(), preconditioner_config=EigenvalueCorrectedShampooPreconditionerConfig(),
            native_runtime_config=NativeRuntimeConfig(backend=backend),
        )
        assert 3 in {b.dim() for b in opt._per_group_state_lists[0]["distributor"].local_blocked_params}
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(16):
            x = torch.randn(16, 64, 8, 8, device="cuda", generator=g)
            y = torch.randint(0, 10, (16,), device="cuda", generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        if backend == "native":
            eng = opt._per_group_state_lists[0]["native_engine"]
            assert eng is not None and any(b.dims3 is not None for b in eng._blocks)
            eng.check_status()
        results.append([p.detach().clone() for p in model.parameters()])
    for p, q in zip(*results):
        assert torch.allclose(p, q, rtol=5e-3, atol=4e-3), (p - q).abs().max()


@pytest.mark.parametrize("name", ["adam_graft", "soap_adam_graft", "eigendecomposed_adam_graft", "gpa"])
def test_native_engine_resumes_from_checkpoint(name):
    """Train 5 steps, checkpoint (model + optimizer), train 4 more; a fresh model / optimizer loaded
    from the checkpoint must retrace those 4 steps: the engine's operand mirrors are rebuilt from
    the loaded state (``on_state_loaded``)."""
    import copy

    from optimizers_b200 import DistributedShampoo, NativeRuntimeConfig

    kw = _configs()[name]
    dev = torch.device("cuda")

    def make():
        torch.manual_seed(0)
        model = _mlp(dev)
        opt = DistributedShampoo(model.parameters(), native_runtime_config=NativeRuntimeConfig(backend="native"), **kw)
        opt.train()
        return model, opt

    def run(model, opt, first, count):
        g = torch.Generator(device="cuda").manual_seed(100 + first)
        for _ in range(count):
            x = torch.randn(64, 96, device=dev, generator=g)
            y = torch.randint(0, 10, (64,), device=dev, generator=g)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()

    model, opt = make()
    run(model, opt, 0, 5)
    ckpt = copy.deepcopy({"model": model.state_dict(), "opt": opt.state_dict()})
    run(model, opt, 5, 4)

    model2, opt2 = make()
    model2.load_state_dict(ckpt["model"])
    opt2.load_state_dict(ckpt["opt"])
    run(model2, opt2, 5, 4)
    for rec in opt2._per_group_state_lists:
        rec["native_engine"].check_status()
    for p, q in zip(model.parameters(), model2.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-6), (p - q).abs().max()


def test_jacobi_eigh_settles_on_a_tiny_scaled_matrix(ext):
    """Entries of 1e-13 (a leaf deep in the null cluster of a factor): squared column norms are
    1e-24, their product is below the smallest fp32 number, and a convergence test written with
    sqrt(alpha * beta) never passes."""
    torch.manual_seed(3)
    dev = torch.device("cuda")
    n = 63
    G = torch.randn(n, 2 * n, device=dev, dtype=torch.float64)
    A = ((G @ G.T) / (2 * n) * 2e-13).float()
    lams, qs, sweeps = ext.jacobi_eigh([A], 24, 2e-6)
    torch.cuda.synchronize()
    assert int(sweeps[0]) <= 24
    ref = torch.linalg.eigvalsh(A.double())
    assert (lams[0].double() - ref).abs().max().item() < 1e-4 * ref.abs().max().item()
    Q = qs[0].double()
    assert (Q.T @ Q - torch.eye(n, device=dev, dtype=torch.float64)).abs().max().item() < 1e-5


@pytest.mark.parametrize("n", [1, 2, 7, 64, 100, 128])
def test_jacobi_eigh_matches_lapack(ext, n):
    """Batched shared-memory Jacobi eigensolver against fp64 eigh: eigenvalues, orthogonality and
    the reconstruction; includes a rank-deficient matrix plus a ridge, the shape Shampoo factors
    have early in training."""
    torch.manual_seed(n)
    mats = []
    for rank in (n, max(1, n // 4)):
        B = torch.randn(n, rank, device="cuda", dtype=torch.float64)
        A = (B @ B.T) / rank + 1e-6 * torch.eye(n, device="cuda", dtype=torch.float64)
        mats.append(A.float().contiguous())
    lams, qs, sweeps = ext.jacobi_eigh(mats, 24, 2e-6)
    assert max(sweeps.cpu().tolist()) <= 24
    for A, lam, Q in zip(mats, lams, qs):
        want = torch.linalg.eigvalsh(A.double())
        scale = want.abs().max().item()
        assert torch.all(lam[1:] >= lam[:-1])
        assert (lam.double() - want).abs().max().item() < 1e-4 * scale
        eye = torch.eye(n, device="cuda")
        assert (Q.T @ Q - eye).abs().max().item() < 5e-6
        assert ((Q * lam) @ Q.T - A).abs().max().item() < 1e-4 * scale
