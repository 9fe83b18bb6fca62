"""GPT-2 style decoder (pre-LN, learned positions, tied input/output embedding) used by the
examples and the throughput benchmark.  Defaults are the 124M configuration: 12 layers,
d_model 768, 12 heads, MLP 3072, vocabulary 50257, context 1024.

With ``fused=True`` (default) the normalisations and the LM head + cross-entropy go through
``optimizers_b200.models.fused_ops`` (CUDA kernels on a GPU, the same formulas in PyTorch
elsewhere); ``fused=False`` is the stock-module formulation."""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from optimizers_b200.models import fused_ops


@dataclass
class GPT2Config:
    vocab_size: int = 50257
    n_ctx: int = 1024
    n_layer: int = 12
    n_head: int = 12
    d_model: int = 768
    d_mlp: int = 3072
    fused: bool = True


class _Block(nn.Module):
    def __init__(self, cfg: GPT2Config) -> None:
        super().__init__()
        self.n_head = cfg.n_head
        self.fused = cfg.fused
        self.ln_1 = nn.LayerNorm(cfg.d_model)
        self.attn_qkv = nn.Linear(cfg.d_model, 3 * cfg.d_model)
        self.attn_proj = nn.Linear(cfg.d_model, cfg.d_model)
        self.ln_2 = nn.LayerNorm(cfg.d_model)
        self.mlp_fc = nn.Linear(cfg.d_model, cfg.d_mlp)
        self.mlp_proj = nn.Linear(cfg.d_mlp, cfg.d_model)

    def _norm(self, ln: nn.LayerNorm, x: torch.Tensor) -> torch.Tensor:
        return fused_ops.layer_norm(x, ln.weight, ln.bias, ln.eps) if self.fused else ln(x)

    def _lin(self, layer: nn.Linear, x: torch.Tensor) -> torch.Tensor:
        return fused_ops.linear(x, layer.weight, layer.bias) if self.fused else layer(x)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        q, k, v = self._lin(self.attn_qkv, self._norm(self.ln_1, x)).split(C, dim=2)
        shape = (B, T, self.n_head, C // self.n_head)
        q, k, v = (t.view(shape).transpose(1, 2) for t in (q, k, v))
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self._lin(self.attn_proj, a.transpose(1, 2).reshape(B, T, C))
        h = F.gelu(self._lin(self.mlp_fc, self._norm(self.ln_2, x)), approximate="tanh")
        return x + self._lin(self.mlp_proj, h)


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config | None = None) -> None:
        super().__init__()
        self.cfg = cfg = cfg or GPT2Config()
        self.wte = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.wpe = nn.Embedding(cfg.n_ctx, cfg.d_model)
        self.blocks = nn.ModuleList(_Block(cfg) for _ in range(cfg.n_layer))
        self.ln_f = nn.LayerNorm(cfg.d_model)
        for m in self.modules():
            self._init(m)
        for name, p in self.named_parameters():
            if name.endswith("proj.weight"):
                nn.init.normal_(p, mean=0.0, std=0.02 / math.sqrt(2 * cfg.n_layer))

    @staticmethod
    def _init(m: nn.Module) -> None:
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, mean=0.0, std=0.02)
        if isinstance(m, nn.Linear) and m.bias is not None:
            nn.init.zeros_(m.bias)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        B, T = idx.shape
        pos = torch.arange(T, device=idx.device)
        x = self.wte(idx) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        if self.cfg.fused:
            h = fused_ops.layer_norm(x, self.ln_f.weight, self.ln_f.bias, self.ln_f.eps)
            if targets is not None:
                return fused_ops.lm_head_cross_entropy(h, self.wte.weight, targets)
            return F.linear(h, self.wte.weight)
        logits = F.linear(self.ln_f(x), self.wte.weight)
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))
