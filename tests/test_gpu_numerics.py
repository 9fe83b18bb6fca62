"""Numerical behaviour of the tensor-core path over many steps: the factor accumulation against
an fp64 accumulator, and training outcomes of the native step against the seed-to-seed spread of
the torch step."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pad4(n):
    return (n + 3) // 4 * 4


def test_thousand_ema_steps_of_the_packed_syrk_stay_near_an_fp64_accumulator():
    """F <- beta2 F + (1 - beta2) G G^T for 1000 steps, packed triangle, tf32x3 products.  Every
    product is low by up to ~K * 2e-8 relative because the tensor-core accumulator truncates; with
    beta2 = 0.999 the errors of about 1000 steps are averaged, not summed, so the bound is that of
    one product (K = 256: 5e-6) plus fp32 rounding of the running average."""
    from optimizers_b200.ops import build

    ext = build.load()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    d, K, beta2 = 192, 256, 0.999
    r, c = torch.triu_indices(d, d, device=dev)
    packed = torch.zeros(r.numel(), device=dev)
    exact = torch.zeros(d, d, device=dev, dtype=torch.float64)
    hi = torch.zeros(d, _pad4(K), device=dev)[:, :K]
    lo = torch.zeros(d, _pad4(K), device=dev)[:, :K]
    plan = ext.build_gemm_plan([(hi, lo, hi, lo, packed, None, None, None, d, 0, ext.FLAG_PACKED_C, True)])
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    scales = torch.logspace(0, -3, d, device=dev).unsqueeze(1)  # rows of very different magnitude
    # the kernel takes its coefficients as fp32 scalars, like an fp32 tensor operation would
    b32 = float(torch.tensor(beta2, dtype=torch.float32))
    w32 = float(torch.tensor(1 - beta2, dtype=torch.float32))
    for _ in range(1000):
        G = torch.randn(d, K, device=dev) * scales
        ext.tf32_split(G, hi, lo)
        ext.run_gemm_plan(*plan, 1 - beta2, beta2, True, status)
        exact.mul_(b32).add_(G.double() @ G.double().T, alpha=w32)
    torch.cuda.synchronize()
    assert status.item() == 0
    got = torch.zeros(d, d, device=dev, dtype=torch.float64)
    got[r, c] = packed.double()
    want = torch.triu(exact)
    # entry-wise against the scale of the entry's row and column (the Cauchy-Schwarz size of an entry)
    size = torch.sqrt(torch.diagonal(exact)).unsqueeze(1) * torch.sqrt(torch.diagonal(exact)).unsqueeze(0)
    assert float(((got - want).abs() / size).max()) < 2e-5
    rel_diag = ((torch.diagonal(got) - torch.diagonal(exact)) / torch.diagonal(exact))
    assert float(rel_diag.abs().max()) < 2e-5
    assert float(rel_diag.max()) < 2e-6  # truncation only ever lowers a sum of squares


def _final_loss(backend: str, seed: int) -> float:
    import optimizers_b200 as lib
    from optimizers_b200.models import GPT2, GPT2Config

    dev = torch.device("cuda")
    vocab, seq, batch = 128, 32, 16
    g = torch.Generator().manual_seed(7)  # the language is the same for every run; the seed varies the model
    table = torch.randint(0, vocab, (vocab, vocab), generator=g)
    data = []
    for _ in range(8):
        t = torch.empty(batch, seq + 1, dtype=torch.long)
        t[:, :2] = torch.randint(0, vocab, (batch, 2), generator=g)
        for i in range(2, seq + 1):
            nxt = table[t[:, i - 2], t[:, i - 1]]
            noise = torch.randint(0, vocab, (batch,), generator=g)
            t[:, i] = torch.where(torch.rand(batch, generator=g) < 0.1, noise, nxt)
        data.append(t.to(dev))
    torch.manual_seed(seed)
    model = GPT2(GPT2Config(vocab_size=vocab, n_ctx=seq, n_layer=2, n_head=4, d_model=128, d_mlp=512, fused=False)).to(dev)
    opt = lib.DistributedShampoo(
        model.parameters(), lr=3e-3, betas=(0.9, 0.999), epsilon=1e-8, weight_decay=1e-4, max_preconditioner_dim=256,
        precondition_frequency=10, start_preconditioning_step=10,
        grafting_config=lib.AdamPreconditionerConfig(beta2=0.999, epsilon=1e-8),
        native_runtime_config=lib.NativeRuntimeConfig(backend=backend),
    )
    tail = []
    for step in range(150):
        t = data[step % len(data)]
        loss = model(t[:, :-1], t[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        if step >= 140:
            tail.append(float(loss.detach()))
    return sum(tail) / len(tail)


def test_native_training_outcomes_lie_within_the_seed_to_seed_spread_of_the_torch_step():
    """Six seeds per implementation of the same optimizer on a small language-model task.  The
    two implementations differ by rounding (tensor-core products, another eigensolver), which a
    training run amplifies like any perturbation; the claim tested is that this moves the outcome
    no more than changing the seed does."""
    torch.backends.cuda.matmul.allow_tf32 = False
    seeds = range(6)
    torch_losses = [_final_loss("torch", s) for s in seeds]
    native_losses = [_final_loss("native", s) for s in seeds]
    assert all(math.isfinite(x) for x in torch_losses + native_losses)
    mean_t = sum(torch_losses) / len(torch_losses)
    mean_n = sum(native_losses) / len(native_losses)
    spread = max(torch_losses) - min(torch_losses)
    std_t = (sum((x - mean_t) ** 2 for x in torch_losses) / (len(torch_losses) - 1)) ** 0.5
    # both learn the task (ln(128) = 4.85 at the start)
    assert mean_t < 3.5 and mean_n < 3.5, (torch_losses, native_losses)
    # the native mean lies within the torch runs' range widened by two of their standard deviations
    assert min(torch_losses) - 2 * std_t <= mean_n <= max(torch_losses) + 2 * std_t, (torch_losses, native_losses)
    # and the native runs scatter no more than twice as much
    assert max(native_losses) - min(native_losses) <= 2 * spread + 4 * std_t, (torch_losses, native_losses)
