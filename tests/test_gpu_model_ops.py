"""GPU tests of the fused model kernels against plain PyTorch fp32 formulations."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ext():
    from optimizers_b200.ops import build

    return build.load()


@pytest.mark.parametrize("V", [50257, 1000, 64, 7])
def test_xent_kernel_matches_fp32_reference(ext, V):
    torch.manual_seed(0)
    T, ld = 96, (V + 63) // 64 * 64
    logits = torch.zeros(T, ld, device="cuda", dtype=torch.bfloat16)
    logits[:, :V] = (torch.randn(T, V, device="cuda") * 3).to(torch.bfloat16)
    targets = torch.randint(0, V, (T,), device="cuda")
    targets[5] = -100
    ref_in = logits[:, :V].float().requires_grad_()
    ref_rows = F.cross_entropy(ref_in, targets, ignore_index=-100, reduction="none")
    ref_rows.sum().backward()
    work = logits.clone()
    rows = ext.xent_fwd_bwd(work, V, targets, -100)
    assert torch.allclose(rows, ref_rows, rtol=1e-4, atol=1e-4)
    assert torch.allclose(work[:, :V].float(), ref_in.grad, rtol=1e-2, atol=1e-3)  # bf16 storage of the gradient
    assert work[:, V:].abs().max().item() == 0 if ld > V else True
    assert work[5].abs().max().item() == 0


@pytest.mark.parametrize("C", [256, 768, 1024, 2048])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("in_dtype,out_bf16", [(torch.float32, True), (torch.float32, False), (torch.bfloat16, True)])
def test_norm_kernels_match_fp32_reference(ext, C, rms, in_dtype, out_bf16):
    torch.manual_seed(1)
    rows = 333
    x = (torch.randn(rows, C, device="cuda") * 2 + 0.5).to(in_dtype)
    gamma = torch.randn(C, device="cuda")
    beta = torch.randn(C, device="cuda")
    dy = torch.randn(rows, C, device="cuda").to(torch.bfloat16 if out_bf16 else torch.float32)
    xr = x.float().requires_grad_()
    gr, br = gamma.clone().requires_grad_(), beta.clone().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * gr
    else:
        yr = F.layer_norm(xr, (C,), gr, br, 1e-5)
    yr.backward(dy.float())
    y, mean, rstd = ext.norm_fwd(x, gamma, None if rms else beta, 1e-5, rms, out_bf16)
    tol = dict(rtol=2e-2, atol=2e-2) if out_bf16 else dict(rtol=1e-4, atol=1e-4)
    assert torch.allclose(y.float(), yr, **tol)
    dx, partial = ext.norm_bwd(dy, x, gamma, mean, rstd, rms)
    tol_dx = dict(rtol=2e-2, atol=2e-2) if in_dtype == torch.bfloat16 else dict(rtol=1e-3, atol=1e-4)
    assert torch.allclose(dx.float(), xr.grad, **tol_dx)
    sums = partial.sum(0)
    assert torch.allclose(sums[0], gr.grad, rtol=1e-3, atol=1e-2)
    if not rms:
        assert torch.allclose(sums[1], br.grad, rtol=1e-3, atol=1e-2)


def test_fused_gpt2_matches_plain_under_autocast():
    from optimizers_b200.models import GPT2, GPT2Config

    cfgs = dict(n_layer=2, vocab_size=50257, d_model=256, n_head=4, d_mlp=512, n_ctx=64)
    torch.manual_seed(0)
    fused = GPT2(GPT2Config(fused=True, **cfgs)).cuda()
    torch.manual_seed(0)
    plain = GPT2(GPT2Config(fused=False, **cfgs)).cuda()
    idx = torch.randint(0, 50257, (4, 65), device="cuda")
    losses = []
    for m in (fused, plain):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(idx[:, :-1], idx[:, 1:])
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 2e-2, losses
    for (n, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        scale = b.grad.abs().max().item() + 1e-8
        assert (a.grad - b.grad).abs().max().item() <= 0.08 * scale + 1e-5, n


def test_fused_llama_matches_plain_under_autocast():
    from optimizers_b200.models import Llama, LlamaConfig

    cfgs = dict(n_layer=2, vocab_size=32000, d_model=256, n_head=4, d_ffn=512)
    torch.manual_seed(0)
    fused = Llama(LlamaConfig(fused=True, **cfgs)).cuda()
    torch.manual_seed(0)
    plain = Llama(LlamaConfig(fused=False, **cfgs)).cuda()
    idx = torch.randint(0, 32000, (2, 65), device="cuda")
    losses = []
    for m in (fused, plain):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = m(idx[:, :-1], idx[:, 1:])
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) < 2e-2, losses
    for (n, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        scale = b.grad.abs().max().item() + 1e-8
        assert (a.grad - b.grad).abs().max().item() <= 0.08 * scale + 1e-5, n


@pytest.mark.parametrize("shape", [(16384, 768), (1000, 2304), (37, 12), (5, 3072)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_colsum_kernel_matches_torch(ext, shape, dtype):
    torch.manual_seed(0)
    x = torch.randn(*shape, device="cuda").to(dtype)
    got = ext.colsum(x)
    want = x.double().sum(0)
    assert torch.allclose(got.double(), want, rtol=1e-4, atol=1e-3 * shape[0] ** 0.5)


def test_fused_linear_matches_torch_under_autocast():
    from optimizers_b200.models import fused_ops

    torch.manual_seed(0)
    x = torch.randn(8, 64, 256, device="cuda", requires_grad=True)
    lin = torch.nn.Linear(256, 512).cuda()
    x2 = x.detach().clone().requires_grad_()
    lin2 = torch.nn.Linear(256, 512).cuda()
    lin2.load_state_dict(lin.state_dict())
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = fused_ops.linear(x, lin.weight, lin.bias)
        y2 = lin2(x2)
    g = torch.randn_like(y)
    y.backward(g)
    y2.backward(g)
    assert torch.equal(y, y2)
    assert torch.allclose(x.grad, x2.grad, rtol=1e-2, atol=1e-3)
    assert torch.allclose(lin.weight.grad, lin2.weight.grad, rtol=2e-2, atol=2e-2)
    assert torch.allclose(lin.bias.grad, lin2.bias.grad, rtol=2e-2, atol=2e-2)
