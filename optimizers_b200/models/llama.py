"""Llama-style decoder: RMSNorm, rotary position embedding, SwiGLU feed-forward, untied output
head.  Defaults are the 1B configuration of the benchmarks: 16 layers, d_model 2048, 32 heads,
FFN 8192, vocabulary 32000.

With ``fused=True`` (default) RMSNorm and the head + cross-entropy go through
``optimizers_b200.models.fused_ops``."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from optimizers_b200.models import fused_ops


@dataclass
class LlamaConfig:
    vocab_size: int = 32000
    n_layer: int = 16
    n_head: int = 32
    d_model: int = 2048
    d_ffn: int = 8192
    max_seq: int = 2048
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    fused: bool = True


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, fused: bool = True) -> None:
        super().__init__()
        self.eps = eps
        self.fused = fused
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return fused_ops.rms_norm(x, self.weight, self.eps)
        scale = torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps)
        return (x.float() * scale).to(x.dtype) * self.weight


def _rope_tables(seq: int, head_dim: int, theta: float, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    angles = torch.outer(torch.arange(seq, device=device).float(), inv)
    return angles.cos(), angles.sin()


def _apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    a, b = x[..., 0::2], x[..., 1::2]
    out = torch.stack((a * cos - b * sin, a * sin + b * cos), dim=-1)
    return out.flatten(-2).to(x.dtype)


class _Layer(nn.Module):
    def __init__(self, cfg: LlamaConfig) -> None:
        super().__init__()
        self.n_head = cfg.n_head
        self.attn_norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.fused)
        self.wq = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wk = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wv = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wo = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.ffn_norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.fused)
        self.w_gate = nn.Linear(cfg.d_model, cfg.d_ffn, bias=False)
        self.w_up = nn.Linear(cfg.d_model, cfg.d_ffn, bias=False)
        self.w_down = nn.Linear(cfg.d_ffn, cfg.d_model, bias=False)

    def forward(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        B, T, C = x.shape
        h = self.attn_norm(x)
        shape = (B, T, self.n_head, C // self.n_head)
        q = _apply_rope(self.wq(h).view(shape).transpose(1, 2), cos, sin)
        k = _apply_rope(self.wk(h).view(shape).transpose(1, 2), cos, sin)
        v = self.wv(h).view(shape).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        x = x + self.wo(a.transpose(1, 2).reshape(B, T, C))
        h = self.ffn_norm(x)
        return x + self.w_down(F.silu(self.w_gate(h)) * self.w_up(h))


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig | None = None) -> None:
        super().__init__()
        self.cfg = cfg = cfg or LlamaConfig()
        self.embed = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList(_Layer(cfg) for _ in range(cfg.n_layer))
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps, cfg.fused)
        self.head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=0.02)

    def forward(self, idx: torch.Tensor, targets: torch.Tensor | None = None):
        T = idx.shape[1]
        cos, sin = _rope_tables(T, self.cfg.d_model // self.cfg.n_head, self.cfg.rope_theta, idx.device)
        x = self.embed(idx)
        for layer in self.layers:
            x = layer(x, cos, sin)
        if self.cfg.fused and targets is not None:
            return fused_ops.lm_head_cross_entropy(self.norm(x), self.head.weight, targets)
        logits = self.head(self.norm(x))
        if targets is None:
            return logits
        return F.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))
