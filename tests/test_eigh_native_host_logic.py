"""Host logic of the sm_100a backend of the divide-and-conquer eigensolver, on the CPU.

``NativeBackend`` (optimizers_b200/matrix/eigh_dc.py) only builds launch tables and calls the
extension; with the torch stand-in of ``tests/fake_ext.py`` in place of the extension the whole
driver runs on the CPU: operand views, ping-pong buffers of the sign iteration, rank and
idempotency read-back, both forms of the second range pass, projection and basis tracking, leaves.
"""

import pytest
import torch

from fake_ext import FakeExt
from optimizers_b200.matrix.eigh_dc import NativeBackend, eigh_divide_and_conquer


def _spectrum(kind, n, gen):
    q, _ = torch.linalg.qr(torch.randn(n, n, dtype=torch.float64, generator=gen))
    if kind == "heavy_tail":
        k = int(0.35 * n)
        lam = torch.zeros(n, dtype=torch.float64)
        lam[:k] = 1.0 / torch.arange(1, k + 1, dtype=torch.float64) ** 2.5
        lam[k:] = 1e-13 * torch.rand(n - k, dtype=torch.float64, generator=gen)
    elif kind == "clustered":
        third = n // 3
        lam = torch.cat([
            torch.full((third,), 1.0, dtype=torch.float64),
            0.5 + 1e-5 * torch.rand(third, dtype=torch.float64, generator=gen),
            1e-3 * torch.rand(n - 2 * third, dtype=torch.float64, generator=gen),
        ])
    else:
        lam = torch.rand(n, dtype=torch.float64, generator=gen)
    return ((q * lam) @ q.T).float()


@pytest.mark.parametrize("polish", ["householder", "newton_schulz"])
@pytest.mark.parametrize("kind", ["uniform", "heavy_tail", "clustered"])
def test_native_backend_driver_on_cpu(kind, polish):
    gen = torch.Generator().manual_seed(7)
    mats = [_spectrum(kind, n, gen) for n in (300, 129, 96, 260)]  # 96: a root that is itself a leaf
    ext = FakeExt()
    backend = NativeBackend(ext, torch.device("cpu"), polish=polish)
    lams, vecs, info = eigh_divide_and_conquer(backend, mats)
    assert info["failed"] == [], info["reasons"]
    assert "householder_qr" in ext.calls and ext.gemm_launches > 50
    for A, lam, V in zip(mats, lams, vecs):
        n = A.shape[0]
        ref = torch.linalg.eigvalsh(A.double())
        scale = ref.abs().max().item()
        assert (lam.double() - ref).abs().max().item() < 5e-6 * scale
        Vd = V.double()
        assert (Vd.T @ Vd - torch.eye(n, dtype=torch.float64)).abs().max().item() < 2e-5
        assert ((Vd * lam.double()) @ Vd.T - A.double()).abs().max().item() < 2e-5 * scale


def test_native_backend_single_pass_and_profile_on_cpu():
    gen = torch.Generator().manual_seed(3)
    mats = [_spectrum("uniform", 200, gen)]
    backend = NativeBackend(FakeExt(), torch.device("cpu"), range_passes=1)
    backend.profile = {}
    lams, vecs, info = eigh_divide_and_conquer(backend, mats)
    assert info["failed"] == []
    assert (lams[0].double() - torch.linalg.eigvalsh(mats[0].double())).abs().max().item() < 5e-6
    assert "sign_projector" in backend.profile
