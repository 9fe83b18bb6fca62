"""Out-of-bounds, race and tracing checks of the native kernels on a B200.

The reference has no sanitizer tier (its kernels are ATen's); these tests stand in for one:

* every output of a kernel is a view into a larger allocation filled with a canary pattern, the
  shapes are ragged (1, 3, 5, 17, 65, 127, 129), and the canaries must survive the launch;
* the whole native step is compared with the torch step on layers of those sizes;
* two runs from the same seed must agree bit for bit (a data race between CTAs or launches shows up
  as a difference) wherever no floating-point atomic is involved;
* the NVTX / per-launch timing switch of the bindings reports the kernels that ran.
"""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

_CANARY = -7.25e30
_SIZES = (1, 3, 5, 17, 65, 127, 129)


@pytest.fixture(scope="module")
def ext():
    from optimizers_b200.ops import build

    return build.load()


def _pad4(n):
    return (n + 3) // 4 * 4


class _Guarded:
    """A rows x cols fp32 view (row pitch pad4(cols) + 4) inside a canary-filled allocation with
    ``margin`` canary elements in front and behind and 4 canary columns after every row."""

    def __init__(self, rows, cols, dev, margin=256, fill=0.0):
        self.rows, self.cols = rows, cols
        self.pitch = _pad4(cols) + 4
        self.margin = margin
        self.raw = torch.full((2 * margin + rows * self.pitch,), _CANARY, device=dev)
        self.view = self.raw[margin : margin + rows * self.pitch].view(rows, self.pitch)[:, :cols]
        self.view.fill_(fill)

    def intact(self):
        body = self.raw[self.margin : self.margin + self.rows * self.pitch].view(self.rows, self.pitch)
        # columns between cols and pad4(cols) may legitimately be zero-filled padding of an operand
        return bool(
            (self.raw[: self.margin] == _CANARY).all()
            and (self.raw[self.margin + self.rows * self.pitch :] == _CANARY).all()
            and (body[:, _pad4(self.cols) :] == _CANARY).all()
        )


class _GuardedFlat:
    def __init__(self, n, dev, margin=256):
        self.raw = torch.full((2 * margin + n,), _CANARY, device=dev)
        self.view = self.raw[margin : margin + n]
        self.view.zero_()
        self.margin, self.n = margin, n

    def intact(self):
        return bool((self.raw[: self.margin] == _CANARY).all() and (self.raw[self.margin + self.n :] == _CANARY).all())


def _operand(x):
    out = torch.zeros(x.shape[0], _pad4(x.shape[1]), device=x.device)[:, : x.shape[1]]
    return out.copy_(x)


@pytest.mark.parametrize("split", [True, False])
def test_grouped_gemm_outputs_stay_inside_their_views(ext, split):
    dev = torch.device("cuda")
    torch.manual_seed(0)
    specs, checks = [], []
    for i, m in enumerate(_SIZES):
        n = _SIZES[(i + 3) % len(_SIZES)]
        k = _SIZES[(i + 5) % len(_SIZES)]
        A, B = torch.randn(m, k, device=dev), torch.randn(n, k, device=dev)
        if split:
            a_hi, a_lo, b_hi, b_lo = (_operand(torch.zeros_like(t)) for t in (A, A, B, B))
            ext.tf32_split(A, a_hi, a_lo)
            ext.tf32_split(B, b_hi, b_lo)
        else:
            a_hi, b_hi, a_lo, b_lo = _operand(A), _operand(B), None, None
        C, D_hi, D_lo = _Guarded(m, n, dev), _Guarded(m, n, dev), _Guarded(m, n, dev)
        specs.append((a_hi, a_lo, b_hi, b_lo, C.view, D_hi.view, D_lo.view, None, C.pitch, D_hi.pitch, ext.FLAG_SPLIT_OUT, False))
        checks.append((A, B, C, D_hi, D_lo))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ext.run_gemm_plan(*ext.build_gemm_plan(specs), 1.0, 0.0, split, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    for A, B, C, D_hi, D_lo in checks:
        ref = A.double() @ B.double().T
        tol = (2e-5 if split else 4e-3) * math.sqrt(A.shape[1]) + (1e-6 if split else 2e-3) * ref.abs().max().item() + 1e-6
        assert (C.view.double() - ref).abs().max().item() < tol
        assert (D_hi.view.double() + D_lo.view.double() - ref).abs().max().item() < tol
        assert C.intact() and D_hi.intact() and D_lo.intact(), (A.shape, B.shape)


def test_packed_syrk_stays_inside_its_triangle(ext):
    dev = torch.device("cuda")
    torch.manual_seed(1)
    specs, checks = [], []
    for i, d in enumerate(_SIZES):
        k = _SIZES[(i + 2) % len(_SIZES)]
        G = torch.randn(d, k, device=dev)
        hi, lo = _operand(torch.zeros_like(G)), _operand(torch.zeros_like(G))
        ext.tf32_split(G, hi, lo)
        packed = _GuardedFlat(d * (d + 1) // 2, dev)
        specs.append((hi, lo, hi, lo, packed.view, None, None, None, d, 0, ext.FLAG_PACKED_C, True))
        checks.append((G, packed, d))
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ext.run_gemm_plan(*ext.build_gemm_plan(specs), 1.0, 0.0, True, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    for G, packed, d in checks:
        r, c = torch.triu_indices(d, d, device=dev)
        ref = (G.double() @ G.double().T)[r, c]
        assert (packed.view.double() - ref).abs().max().item() < 2e-5 * math.sqrt(G.shape[1]) + 3e-5 * ref.abs().max().item() + 1e-6
        assert packed.intact(), d


def test_table_kernels_stay_inside_their_views(ext):
    dev = torch.device("cuda")
    torch.manual_seed(2)
    unpack_specs, pack_specs, sym_specs, tr_specs, checks = [], [], [], [], []
    for i, d in enumerate(_SIZES):
        full = torch.randn(d, d, device=dev)
        full = 0.5 * (full + full.T)
        r, c = torch.triu_indices(d, d, device=dev)
        packed = full[r, c].contiguous()
        u_hi, u_lo = _Guarded(d, d, dev), _Guarded(d, d, dev)
        unpack_specs.append((packed, d, u_hi.view, u_lo.view))
        repacked = _GuardedFlat(d * (d + 1) // 2, dev)
        pack_specs.append((_operand(full), repacked.view))
        s_hi, s_lo = _Guarded(d, d, dev), _Guarded(d, d, dev)
        stats = torch.zeros(2, device=dev)
        sym_specs.append((_operand(full), s_hi.view, s_lo.view, stats, 0.5, -2.0))
        rows = _SIZES[(i + 4) % len(_SIZES)]
        src = torch.randn(rows, d, device=dev)
        t_plain, t_hi, t_lo = _Guarded(d, rows, dev), _Guarded(d, rows, dev), _Guarded(d, rows, dev)
        tr_specs.append((src, t_plain.view, t_hi.view, t_lo.view))
        checks.append((full, packed, u_hi, u_lo, repacked, s_hi, s_lo, src, t_plain, t_hi, t_lo))
    ext.unpack_split(*ext.build_unpack_table(unpack_specs))
    ext.pack_upper(*ext.build_pack_table(pack_specs))
    ext.shift_scale_split(*ext.build_sym_table(sym_specs))
    ext.transpose_split(*ext.build_transpose_table(tr_specs))
    torch.cuda.synchronize()
    for full, packed, u_hi, u_lo, repacked, s_hi, s_lo, src, t_plain, t_hi, t_lo in checks:
        d = full.shape[0]
        assert torch.equal(u_hi.view + u_lo.view, full)
        assert torch.equal(repacked.view, packed)
        assert torch.allclose(s_hi.view + s_lo.view, 0.5 * full - 2.0 * torch.eye(d, device=dev), rtol=1e-6, atol=1e-6)
        assert torch.equal(t_plain.view, src.T) and torch.equal(t_hi.view + t_lo.view, src.T)
        for g in (u_hi, u_lo, repacked, s_hi, s_lo, t_plain, t_hi, t_lo):
            assert g.intact(), d


def _layer_run(backend, din, dout, steps=5, seed=0, **kw):
    from optimizers_b200 import AdamPreconditionerConfig, DistributedShampoo, NativeRuntimeConfig

    dev = torch.device("cuda")
    torch.manual_seed(seed)
    model = torch.nn.Sequential(torch.nn.Linear(din, dout), torch.nn.Tanh(), torch.nn.Linear(dout, 3)).to(dev)
    args = dict(
        lr=1e-3, betas=(0.9, 0.999), epsilon=1e-6, max_preconditioner_dim=64, precondition_frequency=2,
        start_preconditioning_step=2, grafting_config=AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8),
        weight_decay=1e-3,
    )
    args.update(kw)
    opt = DistributedShampoo(model.parameters(), native_runtime_config=NativeRuntimeConfig(backend=backend), **args)
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    for _ in range(steps):
        x = torch.randn(32, din, device=dev, generator=g)
        y = torch.randint(0, 3, (32,), device=dev, generator=g)
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(x), y).backward()
        opt.step()
    torch.cuda.synchronize()
    return model, opt


@pytest.mark.parametrize("din,dout", [(1, 3), (3, 1), (5, 17), (17, 5), (65, 127), (129, 65), (127, 129), (1, 129), (64, 128)])
def test_native_step_on_ragged_layers_matches_torch_step(din, dout):
    m_ref, _ = _layer_run("torch", din, dout)
    m_nat, o_nat = _layer_run("native", din, dout)
    for rec in o_nat._per_group_state_lists:
        assert rec["native_engine"] is not None
        rec["native_engine"].check_status()
    for p, q in zip(m_ref.parameters(), m_nat.parameters()):
        assert torch.allclose(p, q, rtol=5e-3, atol=5e-4), (din, dout, (p - q).abs().max().item())


@pytest.mark.parametrize("name", ["adam_graft", "soap_adam_graft", "eigendecomposed_adam_graft"])
def test_two_native_runs_are_bitwise_identical(name):
    """Blocks of at most one tile per kernel: every floating-point sum has a fixed order, so any
    difference between two runs is a race."""
    from optimizers_b200 import (
        AdamPreconditionerConfig,
        EigendecomposedShampooPreconditionerConfig,
        EigenvalueCorrectedShampooPreconditionerConfig,
    )

    kw = {
        "adam_graft": {},
        "soap_adam_graft": dict(preconditioner_config=EigenvalueCorrectedShampooPreconditionerConfig()),
        "eigendecomposed_adam_graft": dict(preconditioner_config=EigendecomposedShampooPreconditionerConfig()),
    }[name]
    kw = dict(kw, grafting_config=AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8))
    m1, o1 = _layer_run("native", 65, 127, steps=7, **kw)
    m2, o2 = _layer_run("native", 65, 127, steps=7, **kw)
    for p, q in zip(m1.parameters(), m2.parameters()):
        assert torch.equal(p, q)

    def walk(a, b, path=""):
        if isinstance(a, dict):
            for k in a:
                walk(a[k], b[k], f"{path}/{k}")
        elif isinstance(a, torch.Tensor):
            assert torch.equal(a, b), path

    walk(o1.state_dict()["state"], o2.state_dict()["state"])


def test_two_runs_with_multi_tile_blocks_agree_to_rounding():
    """Blocks larger than one tile reduce their norms with floating-point atomics whose order is not
    fixed: the runs may differ in the last bits of those sums, not more."""
    m1, _ = _layer_run("native", 300, 260, steps=6, max_preconditioner_dim=512)
    m2, _ = _layer_run("native", 300, 260, steps=6, max_preconditioner_dim=512)
    for p, q in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(p, q, rtol=1e-5, atol=5e-6), (p - q).abs().max().item()


def test_launch_tracing_reports_the_native_kernels():
    from optimizers_b200.utils import tracing

    tracing.enable(nvtx=True, timing=True)
    try:
        tracing.launch_timings(reset=True)
        _layer_run("native", 65, 127, steps=4)
        timings = tracing.launch_timings(reset=True)
    finally:
        tracing.disable()
    for name in ("ob200::grouped_gemm", "ob200::grad_prologue", "ob200::direction_epilogue", "ob200::jacobi_eigh"):
        assert name in timings, sorted(timings)
        calls, ms = timings[name]
        assert calls >= 1 and ms > 0.0, (name, calls, ms)
    _layer_run("native", 5, 17, steps=2)
    assert tracing.launch_timings() == {}
