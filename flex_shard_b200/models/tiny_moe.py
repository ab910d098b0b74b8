"""Tiny MoE transformer in plain PyTorch (any device, any dtype).

The CPU/gloo acceptance model: RMSNorm + RoPE attention, MoE FFN with a softmax
top-k router and SwiGLU experts. Role parity: ``examples/tiny_moe_transformer.py`` of
the reference (a toy model for end-to-end sharding checks); this one routes tokens
sparsely instead of evaluating every expert densely.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.moe import route_topk


@dataclass
class TinyMoEConfig:
    vocab_size: int = 1024
    d_model: int = 256
    n_layers: int = 4
    n_heads: int = 4
    n_experts: int = 4
    top_k: int = 2
    expert_hidden: int = 512
    max_seq_len: int = 128
    rope_theta: float = 10000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02


class RMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


def rope_cache(seq_len, head_dim, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq_len, device=device, dtype=torch.float32), inv)
    return torch.polar(torch.ones_like(ang), ang)


def apply_rope(x, freqs):
    # x: [B, S, H, hd]; interleaved pairs rotated in fp32
    xc = torch.view_as_complex(x.float().reshape(*x.shape[:-1], -1, 2))
    out = torch.view_as_real(xc * freqs[None, : x.shape[1], None, :]).flatten(3)
    return out.to(x.dtype)


class Attention(nn.Module):
    def __init__(self, cfg: TinyMoEConfig):
        super().__init__()
        self.n_heads = cfg.n_heads
        self.head_dim = cfg.d_model // cfg.n_heads
        self.wq = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wk = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wv = nn.Linear(cfg.d_model, cfg.d_model, bias=False)
        self.wo = nn.Linear(cfg.d_model, cfg.d_model, bias=False)

    def forward(self, x, freqs):
        B, S, _ = x.shape
        q = self.wq(x).view(B, S, self.n_heads, self.head_dim)
        k = self.wk(x).view(B, S, self.n_heads, self.head_dim)
        v = self.wv(x).view(B, S, self.n_heads, self.head_dim)
        q, k = apply_rope(q, freqs), apply_rope(k, freqs)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        return self.wo(o.transpose(1, 2).reshape(B, S, -1))


class Experts(nn.Module):
    """Stacked SwiGLU experts: w13 [E, 2F, D], w2 [E, D, F]."""

    def __init__(self, cfg: TinyMoEConfig):
        super().__init__()
        E, D, Fh = cfg.n_experts, cfg.d_model, cfg.expert_hidden
        self.w13 = nn.Parameter(torch.empty(E, 2 * Fh, D))
        self.w2 = nn.Parameter(torch.empty(E, D, Fh))

    def forward(self, x, expert_idx, weights):
        # x: [T, D]; expert_idx, weights: [T, k]
        out = torch.zeros_like(x)
        E = self.w13.shape[0]
        for e in range(E):
            tok, slot = torch.where(expert_idx == e)
            if tok.numel() == 0:
                # keep every expert in the graph so all ranks reduce identical buckets
                out = out + 0.0 * (self.w13[e].sum() + self.w2[e].sum())
                continue
            h = x[tok] @ self.w13[e].t()
            g, u = h.chunk(2, dim=-1)
            y = (F.silu(g) * u) @ self.w2[e].t()
            out = out.index_add(0, tok, y * weights[tok, slot, None])
        return out


class MoE(nn.Module):
    def __init__(self, cfg: TinyMoEConfig):
        super().__init__()
        self.top_k = cfg.top_k
        self.router = nn.Linear(cfg.d_model, cfg.n_experts, bias=False)
        self.experts = Experts(cfg)

    def forward(self, x):
        B, S, D = x.shape
        xt = x.reshape(-1, D)
        idx, w = route_topk(self.router(xt).float(), self.top_k, mode="softmax", normalize=True)
        w = w.to(x.dtype)
        return self.experts(xt, idx, w).view(B, S, D)


class Block(nn.Module):
    def __init__(self, cfg: TinyMoEConfig):
        super().__init__()
        self.attention_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.attention = Attention(cfg)
        self.ffn_norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.moe = MoE(cfg)

    def forward(self, x, freqs):
        x = x + self.attention(self.attention_norm(x), freqs)
        return x + self.moe(self.ffn_norm(x))


class TinyMoETransformer(nn.Module):
    def __init__(self, cfg: TinyMoEConfig):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.layers = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layers)])
        self.norm = RMSNorm(cfg.d_model, cfg.norm_eps)
        self.output = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)
        self._freqs = None

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("norm.weight"):
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32) * self.cfg.init_std)

    def forward(self, tokens):
        if self._freqs is None or self._freqs.device != tokens.device:
            self._freqs = rope_cache(self.cfg.max_seq_len, self.cfg.d_model // self.cfg.n_heads,
                                     self.cfg.rope_theta, tokens.device)
        h = self.tok_embeddings(tokens)
        for layer in self.layers:
            h = layer(h, self._freqs)
        return self.output(self.norm(h))


def next_token_loss(logits, tokens):
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1))
