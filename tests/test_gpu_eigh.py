"""GPU numerics of the eigensolver building blocks (symmetric GEMM epilogues, operand views,
Householder panels and the batched QR, per-matrix passes) and of the batched divide-and-conquer
eigensolver itself, against fp64 PyTorch."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from optimizers_b200.ops import build

    return build.load()


def _pad4(n):
    return (n + 3) // 4 * 4


def _padded(x):
    rows, k = x.shape
    out = torch.zeros(rows, _pad4(k), device=x.device)[:, :k]
    out.copy_(x)
    return out


def _split(ext, x):
    rows, k = x.shape
    hi = torch.zeros(rows, _pad4(k), device=x.device)[:, :k]
    lo = torch.zeros(rows, _pad4(k), device=x.device)[:, :k]
    ext.tf32_split(_padded(x), hi, lo)
    return hi, lo


def _status(dev):
    return torch.zeros(1, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("n", [64, 128, 300, 517])
def test_symmetric_gemm_mirror_add_diag_trace(ext, n):
    torch.manual_seed(n)
    dev = torch.device("cuda")
    X = torch.randn(n, n, device=dev)
    X = 0.5 * (X + X.T) / n**0.5
    C0 = torch.randn(n, n, device=dev)
    C0 = 0.5 * (C0 + C0.T)
    x_hi, x_lo = _split(ext, X)
    C = _padded(C0)
    d_hi, d_lo = (torch.full((n, _pad4(n)), float("nan"), device=dev)[:, :n] for _ in range(2))
    stats = torch.zeros(2, device=dev)
    flags = ext.FLAG_MIRROR | ext.FLAG_ADD_DIAG | ext.FLAG_TRACE | ext.FLAG_SUMSQ | ext.FLAG_SPLIT_OUT
    plan = ext.build_gemm_plan([(x_hi, x_lo, x_hi, x_lo, C, d_hi, d_lo, stats, C.stride(0), d_hi.stride(0), flags, True)])
    status = _status(dev)
    ext.run_gemm_plan(*plan, 0.7, -0.3, True, status, 1.25)
    torch.cuda.synchronize()
    assert status.item() == 0
    ref = 0.7 * (X.double() @ X.double()) - 0.3 * C0.double() + 1.25 * torch.eye(n, device=dev, dtype=torch.float64)
    assert torch.allclose(C.double(), ref, rtol=1e-5, atol=1e-5)
    assert torch.equal(C, C.T)  # the lower triangle is the mirrored upper one, bit for bit
    assert torch.allclose((d_hi + d_lo).double(), ref, rtol=1e-5, atol=1e-5)
    assert torch.allclose(stats[0].double(), (ref * ref).sum(), rtol=1e-4)
    assert torch.allclose(stats[1].double(), torch.trace(ref), rtol=1e-4, atol=1e-3)


def test_gemm_operand_views_share_tensor_maps(ext):
    """Problems given as views (origin + extent) of larger arrays, the way the blocked QR
    addresses its panels: several launches from one table."""
    torch.manual_seed(0)
    dev = torch.device("cuda")
    A = torch.randn(200, 160, device=dev)
    B = torch.randn(96, 160, device=dev)
    a_hi, a_lo = _split(ext, A)
    b_hi, b_lo = _split(ext, B)
    outs, launches, refs = [], [], []
    for (ar, ak, br, bk, M, N, K) in [(40, 32, 16, 32, 100, 48, 128), (0, 96, 0, 96, 200, 96, 64), (3, 0, 5, 0, 7, 9, 160)]:
        C = torch.zeros(M, _pad4(N), device=dev)[:, :N]
        outs.append(C)
        launches.append([(a_hi, a_lo, b_hi, b_lo, C, None, None, None, C.stride(0), 0, 0, False, None, (ar, ak, br, bk, M, N, K))])
        refs.append(A[ar : ar + M, ak : ak + K].double() @ B[br : br + N, bk : bk + K].double().T)
    table, tiles, ranges = ext.build_gemm_plans(launches)
    status = _status(dev)
    for first, count in ranges:
        ext.run_gemm_plan_range(table, tiles, first, count, 1.0, 0.0, True, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    for C, ref in zip(outs, refs):
        assert torch.allclose(C.double(), ref, rtol=1e-5, atol=1e-4)


def test_per_matrix_passes(ext):
    torch.manual_seed(1)
    dev = torch.device("cuda")
    mats = [_padded(torch.randn(n, n, device=dev)) for n in (5, 130, 257)]
    mats = [m.copy_(0.5 * (m + m.T)) for m in mats]
    stats = torch.zeros(len(mats), 2, device=dev)
    his = [torch.zeros_like(m) for m in mats]
    los = [torch.zeros_like(m) for m in mats]
    table = ext.build_sym_table([(m, h, l, stats[i], 0.5, -2.0) for i, (m, h, l) in enumerate(zip(mats, his, los))])
    ext.sym_measure(table[0], len(mats))
    ext.shift_scale_split(*table)
    off = torch.zeros(len(mats), 2, device=dev)
    table2 = ext.build_sym_table([(m, None, None, off[i], 0.0, 0.0) for i, m in enumerate(mats)])
    ext.sq_offdiag(table2[0], len(mats))
    torch.cuda.synchronize()
    for i, m in enumerate(mats):
        n = m.shape[0]
        sigma = torch.trace(m.double()) / n
        spread = torch.linalg.norm(m.double() - sigma * torch.eye(n, device=dev, dtype=torch.float64))
        assert torch.allclose(stats[i, 0].double(), sigma, rtol=1e-5, atol=1e-6)
        assert torch.allclose(stats[i, 1].double(), spread, rtol=1e-5)
        ref = 0.5 * m - 2.0 * torch.eye(n, device=dev)
        assert torch.allclose(his[i] + los[i], ref, rtol=1e-6, atol=1e-6)
        assert torch.allclose(off[i, 0].double(), (m.double() ** 2).sum(), rtol=1e-5)
        assert torch.allclose(off[i, 1].double(), (torch.diagonal(m).double() ** 2).sum(), rtol=1e-5)
    src = torch.randn(70, 45, device=dev)
    dst, dst_hi, dst_lo = (torch.zeros(45, 72, device=dev)[:, :70] for _ in range(3))
    tt = ext.build_transpose_table([(src, dst, dst_hi, dst_lo)])
    ext.transpose_split(*tt)
    torch.cuda.synchronize()
    assert torch.equal(dst, src.T) and torch.equal(dst_hi + dst_lo, src.T)


@pytest.mark.parametrize("n,k", [(16, 16), (40, 17), (130, 64), (300, 300), (257, 100), (1024, 500), (3200, 48), (4100, 20)])
def test_householder_qr_matches_lapack(ext, n, k):
    """Q^T from the panel kernel + block-reflector sweeps against torch.linalg.qr in fp64 (same
    Householder sign convention, so the leading k columns agree, not only their span).  n = 3200
    takes the panel path that works in global memory."""
    torch.manual_seed(n + k)
    dev = torch.device("cuda")
    Y = torch.randn(n, k, device=dev, dtype=torch.float64)
    Y[:, k // 2] *= 1e-3  # uneven column scales
    Yt = _padded(Y.T.float().contiguous())
    zt, zt_hi, zt_lo = (torch.full((n, _pad4(n)), float("nan"), device=dev)[:, :n] for _ in range(3))
    ext.householder_qr([(Yt, n, k, zt, zt_hi, zt_lo)])
    torch.cuda.synchronize()
    Q = zt.double().T
    eye = torch.eye(n, device=dev, dtype=torch.float64)
    assert float((Q.T @ Q - eye).abs().max()) < 2e-5
    assert torch.equal(zt_hi + zt_lo, zt)
    Qr, _ = torch.linalg.qr(Y.float().double())
    assert float((Q[:, :k] - Qr).abs().max()) < 5e-4  # ill-scaled column included
    if k < n:
        resid = Q[:, k:].T @ Y.float().double()
        assert float(resid.abs().max()) < 1e-4 * float(Y.abs().max())
    R = torch.triu(Yt.double().T[:k, :k])
    assert float((Q[:, :k] @ R - Y.float().double()).abs().max()) < 2e-5 * float(Y.abs().max()) * n**0.5


@pytest.mark.parametrize("n,k,rows", [(300, 77, 77), (513, 300, 5), (130, 64, 130)])
def test_householder_qr_leading_rows_only(ext, n, k, rows):
    """The optional seventh field asks for the first rows of Q^T only (what a second range pass
    reads): same values as the full accumulation, nothing written behind them."""
    torch.manual_seed(n + k + rows)
    dev = torch.device("cuda")
    Y = torch.randn(n, k, device=dev)
    full = [torch.zeros(n, _pad4(n), device=dev)[:, :n] for _ in range(3)]
    ext.householder_qr([(_padded(Y.T.contiguous()), n, k, *full)])
    sentinel = -3.0e30
    part = [torch.full((rows + 3, _pad4(n)), sentinel, device=dev) for _ in range(3)]
    ext.householder_qr([(_padded(Y.T.contiguous()), n, k, *(p[:rows, :n] for p in part), rows)])
    torch.cuda.synchronize()
    for whole, some in zip(full, part):
        assert torch.equal(some[:rows, :n], whole[:rows])
        assert bool((some[rows:] == sentinel).all())


def test_householder_qr_batch_of_mixed_shapes(ext):
    torch.manual_seed(2)
    dev = torch.device("cuda")
    shapes = [(200, 77), (64, 64), (513, 300), (48, 5)]
    specs, keep = [], []
    for n, k in shapes:
        Y = torch.randn(n, k, device=dev)
        Yt = _padded(Y.T.contiguous())
        z = [torch.zeros(n, _pad4(n), device=dev)[:, :n] for _ in range(3)]
        specs.append((Yt, n, k, *z))
        keep.append((Y, z[0]))
    ext.householder_qr(specs)
    torch.cuda.synchronize()
    for (n, k), (Y, zt) in zip(shapes, keep):
        Q = zt.double().T
        assert float((Q.T @ Q - torch.eye(n, device=dev, dtype=torch.float64)).abs().max()) < 2e-5
        if k < n:
            assert float((Q[:, k:].T @ Y.double()).abs().max()) < 1e-4


def _spectrum(kind, d, dev, gen):
    if kind == "lowrank_ridge":  # rank-deficient Gram matrix plus a ridge, the first refresh of a factor
        G = torch.randn(d, max(d // 3, 1), device=dev, dtype=torch.float64, generator=gen)
        return G @ G.T / d + 1e-6 * torch.eye(d, device=dev, dtype=torch.float64)
    lam = {
        "power": 1.0 / torch.arange(1, d + 1, device=dev, dtype=torch.float64) ** 2,
        "uniform": torch.rand(d, device=dev, dtype=torch.float64, generator=gen),
        "clustered": torch.cat([torch.ones(d // 2, device=dev), torch.full((d - d // 2,), 1e-3, device=dev)]).double()
        + 1e-7 * torch.randn(d, device=dev, dtype=torch.float64, generator=gen),
    }[kind]
    q, _ = torch.linalg.qr(torch.randn(d, d, device=dev, dtype=torch.float64, generator=gen))
    return (q * lam) @ q.T


@pytest.mark.parametrize("d", [129, 256, 768, 1024, 2048])
def test_native_divide_and_conquer_eigh_matches_fp64(ext, d):
    from optimizers_b200.matrix.eigh_dc import NativeBackend, eigh_divide_and_conquer

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(d)
    kinds = ["power", "uniform", "clustered", "lowrank_ridge"]
    mats64 = [_spectrum(k, d, dev, gen) for k in kinds]
    backend = NativeBackend(ext, dev)
    lams, vecs, info = eigh_divide_and_conquer(backend, [m.float() for m in mats64])
    torch.cuda.synchronize()
    assert backend.status.item() == 0
    assert info["failed"] == [] and backend.failed_in_finish == [], info
    eye = torch.eye(d, device=dev, dtype=torch.float64)
    for kind, A, lam, Q in zip(kinds, mats64, lams, vecs):
        lam, Q = lam.double(), Q.double()
        ref, ref_q = torch.linalg.eigh(A)
        scale = float(ref.abs().max())
        assert torch.all(lam[1:] >= lam[:-1]), kind
        # The tensor-core accumulator truncates: a sum of K like-signed terms comes out low by about
        # K * 2e-8 relative, so eigenvalues (two products per level) and vector norms carry a
        # relative error of up to ~1e-4 at d = 2048; orthogonality between different vectors is finer.
        assert float((lam - ref).abs().max()) <= 3e-4 * scale, (kind, float((lam - ref).abs().max()) / scale)
        gram = Q.T @ Q
        assert float((torch.diagonal(gram) - 1).abs().max()) < 5e-4, kind
        assert float((gram - torch.diag(torch.diagonal(gram))).abs().max()) < 1e-4, (kind, float((gram - torch.diag(torch.diagonal(gram))).abs().max()))
        recon = float(torch.linalg.norm((Q * lam) @ Q.T - A)) / float(torch.linalg.norm(A))
        assert recon < 5e-4, (kind, recon)
        # the quantity the optimizer uses: the inverse fourth root with a ridge at 1e-6 of the top eigenvalue
        eps = 1e-6 * scale
        want = (ref_q * (ref.clamp(min=0) + eps).pow(-0.25)) @ ref_q.T
        got = (Q * ((lam - lam.min().clamp(max=0)) + eps).pow(-0.25)) @ Q.T
        err = float(torch.linalg.norm(got - want) / torch.linalg.norm(want))
        # fp32 eigensolvers resolve eigenvalues to ~1e-7 of the largest one; the library's fp32 eigh gives 1e-2 here
        assert err < 5e-2, (kind, err)


@pytest.mark.parametrize("d", [96, 300, 1024])
def test_native_qr_iteration_matches_torch_path(ext, d):
    """Warm-started QR iteration on ill-conditioned factors (condition number 1e8) against the
    torch formulation in fp64: same eigenvalue estimates, an orthonormal basis, and an off-diagonal
    residue that is no worse."""
    from optimizers_b200.matrix import functions as mf
    from optimizers_b200.matrix.batched import native_qr_iteration

    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(d)
    mats, starts = [], []
    for k in range(3):
        q, _ = torch.linalg.qr(torch.randn(d, d, device=dev, dtype=torch.float64, generator=gen))
        lam = torch.logspace(0, -8, d, device=dev, dtype=torch.float64)
        A = (q * lam) @ q.T
        # previous eigenvectors: the true ones rotated a little (a refresh interval later)
        S = 0.05 * torch.randn(d, d, device=dev, dtype=torch.float64, generator=gen)
        rot, _ = torch.linalg.qr(torch.eye(d, device=dev, dtype=torch.float64) + (S - S.T))
        mats.append(A)
        starts.append((q @ rot).contiguous())
    status = _status(dev)
    got = native_qr_iteration(ext, [m.float() for m in mats], [v.float() for v in starts], 2, 1e-6, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    eye = torch.eye(d, device=dev, dtype=torch.float64)
    for A, V0, V in zip(mats, starts, got):
        lam_ref, V_ref = mf._qr_iteration(A, V0, 2, 1e-6)
        V = V.double()
        assert float((V.T @ V - eye).abs().max()) < 1e-4
        B, B_ref = V.T @ A @ V, V_ref.T @ A @ V_ref
        assert torch.allclose(torch.diagonal(B), lam_ref, atol=2e-4 * float(lam_ref.abs().max()), rtol=0)
        off = torch.linalg.norm(B - torch.diag(torch.diagonal(B)))
        off_ref = torch.linalg.norm(B_ref - torch.diag(torch.diagonal(B_ref)))
        assert float(off) <= 1.5 * float(off_ref) + 2e-4 * float(torch.linalg.norm(A))
