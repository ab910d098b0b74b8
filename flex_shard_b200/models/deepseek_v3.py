"""DeepSeek-V3-style MoE decoder: MLA attention, a dense first block, routed + shared experts.

Hot ops run on this library's kernels: every projection is a tcgen05 GEMM, the routed experts are
grouped tcgen05 GEMMs over an expert-major token layout planned on the device (no host sync),
norms / SwiGLU / cross-entropy are the fused bandwidth kernels. Multi-head latent attention has
192-wide query/key heads and 128-wide value heads; the flash-attention kernel of this library is
specialised for 128/128, so MLA's softmax(QK^T)V itself runs on PyTorch's SDPA here.

Role parity: ``examples/deepseek_v3/model.py`` of the reference (a plain-PyTorch DeepSeek-V3 with
sigmoid top-k routing, an auxiliary-loss-free expert bias and shared experts); parameters are
stored stacked (``w13``: gate and up projections) as the reference's grouped-mm experts are.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import elementwise as ew
from ..ops import moe as moe_ops
from ..ops.gemm import linear


@dataclass
class DeepSeekV3Config:
    vocab_size: int = 102400
    d_model: int = 2048
    n_layers: int = 24
    n_dense_layers: int = 1
    n_heads: int = 16
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_dim: int = 128
    qk_rope_dim: int = 64
    v_dim: int = 128
    dense_hidden: int = 10944
    n_experts: int = 64
    expert_hidden: int = 1408
    top_k: int = 6
    n_shared_experts: int = 1
    route_scale: float = 1.0
    rope_theta: float = 10000.0
    rope_factor: float = 1.0          # > 1: YaRN context stretch (with original_seq_len, beta_fast, beta_slow, mscale)
    original_seq_len: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 0.70
    router_fp32_out_bf16: bool = False   # router logits: bf16 operands -> fp32 output, split-precision backward
    norm_eps: float = 1e-6
    max_seq_len: int = 4096
    init_std: float = 0.02
    activation_checkpointing: bool = False   # recompute every block in backward (non-reentrant checkpoint per block)
    aux_loss_coeff: float = 0.0              # > 0: sequence-wise balance loss on the router scores

    @property
    def qk_dim(self) -> int:
        return self.qk_nope_dim + self.qk_rope_dim


def _rms(x, w, eps):
    return ew.rmsnorm(x, w, eps)


class MLA(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        kw = dict(dtype=dtype, device=device)
        H = cfg.n_heads
        self.wq_a = nn.Parameter(torch.empty(cfg.q_lora_rank, cfg.d_model, **kw))
        self.q_norm = nn.Parameter(torch.empty(cfg.q_lora_rank, **kw))
        self.wq_b = nn.Parameter(torch.empty(H * cfg.qk_dim, cfg.q_lora_rank, **kw))
        self.wkv_a = nn.Parameter(torch.empty(cfg.kv_lora_rank + cfg.qk_rope_dim, cfg.d_model, **kw))
        self.kv_norm = nn.Parameter(torch.empty(cfg.kv_lora_rank, **kw))
        self.wkv_b = nn.Parameter(torch.empty(H * (cfg.qk_nope_dim + cfg.v_dim), cfg.kv_lora_rank, **kw))
        self.wo = nn.Parameter(torch.empty(cfg.d_model, H * cfg.v_dim, **kw))

    def forward(self, x, rope_table, doc_mask=None):
        cfg = self.cfg
        B, S, _ = x.shape
        H = cfg.n_heads
        q = linear(_rms(linear(x, self.wq_a), self.q_norm, cfg.norm_eps), self.wq_b).view(B, S, H, cfg.qk_dim)
        kv = linear(x, self.wkv_a)
        c_kv, k_pe = kv.split([cfg.kv_lora_rank, cfg.qk_rope_dim], dim=-1)
        kvb = linear(_rms(c_kv.contiguous(), self.kv_norm, cfg.norm_eps), self.wkv_b).view(
            B, S, H, cfg.qk_nope_dim + cfg.v_dim)
        k_nope, v = kvb.split([cfg.qk_nope_dim, cfg.v_dim], dim=-1)
        q_nope, q_pe = q.split([cfg.qk_nope_dim, cfg.qk_rope_dim], dim=-1)
        q_pe = ew._rope_ref(q_pe, rope_table, False)
        k_pe = ew._rope_ref(k_pe.reshape(B, S, 1, cfg.qk_rope_dim), rope_table, False)
        qf = torch.cat([q_nope, q_pe], dim=-1)
        kf = torch.cat([k_nope, k_pe.expand(B, S, H, cfg.qk_rope_dim)], dim=-1)
        # doc_mask [B, 1, S, S] (True = attend): causal within documents; without it plain causal attention
        o = F.scaled_dot_product_attention(qf.transpose(1, 2), kf.transpose(1, 2), v.transpose(1, 2),
                                           attn_mask=doc_mask, is_causal=doc_mask is None,
                                           scale=ew.yarn_attention_scale(cfg.qk_dim, cfg.rope_factor, cfg.mscale))
        return linear(o.transpose(1, 2).reshape(B, S, H * cfg.v_dim), self.wo)


class _InjectAuxLoss(torch.autograd.Function):
    """Identity on ``x`` whose backward also back-propagates a gradient of 1 into ``loss``: an auxiliary loss
    joins the backward pass without being added to (or changing the value of) the reported main loss."""

    @staticmethod
    def forward(ctx, x, loss):
        ctx.loss_dtype = loss.dtype
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return g, torch.ones((), dtype=ctx.loss_dtype, device=g.device)


def document_causal_mask(positions: torch.Tensor) -> torch.Tensor:
    """``positions`` [B, S]: position of every token inside its document (a document starts where it is 0).
    Returns a boolean [B, 1, S, S] mask: token q attends token k iff k <= q and both sit in one document."""
    doc = torch.cumsum((positions == 0).int(), dim=1)
    S = positions.shape[1]
    causal = torch.ones(S, S, dtype=torch.bool, device=positions.device).tril()
    return (causal[None] & (doc[:, :, None] == doc[:, None, :]))[:, None]


class DenseFFN(nn.Module):
    def __init__(self, d_model, hidden, dtype, device):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(2 * hidden, d_model, dtype=dtype, device=device))
        self.w2 = nn.Parameter(torch.empty(d_model, hidden, dtype=dtype, device=device))

    def forward(self, x):
        return linear(ew.swiglu(linear(x, self.w13)), self.w2)


class RoutedExperts(nn.Module):
    """Stacked expert weights; under expert parallelism only this rank's experts are kept."""

    def __init__(self, n_experts, d_model, hidden, dtype, device):
        super().__init__()
        self.w13 = nn.Parameter(torch.empty(n_experts, 2 * hidden, d_model, dtype=dtype, device=device))
        self.w2 = nn.Parameter(torch.empty(n_experts, d_model, hidden, dtype=dtype, device=device))

    def forward(self, rows, plan):
        h = ew.swiglu(moe_ops.grouped_linear(rows, self.w13, plan))
        return moe_ops.grouped_linear(h, self.w2, plan)


class MoE(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.gate = nn.Parameter(torch.empty(cfg.n_experts, cfg.d_model, dtype=torch.float32, device=device))
        self.register_buffer("expert_bias", torch.zeros(cfg.n_experts, dtype=torch.float32, device=device))
        self.register_buffer("tokens_per_expert", torch.zeros(cfg.n_experts, dtype=torch.float32, device=device),
                             persistent=False)
        self.routed_experts = RoutedExperts(cfg.n_experts, cfg.d_model, cfg.expert_hidden, dtype, device)
        self.shared = DenseFFN(cfg.d_model, cfg.expert_hidden * cfg.n_shared_experts, dtype, device) \
            if cfg.n_shared_experts else None
        self.dispatcher = None  # set by apply_expert_parallel

    def route(self, xt):
        cfg = self.cfg
        if cfg.router_fp32_out_bf16:
            from ..ops.gemm import fp32_output_linear

            logits = fp32_output_linear(xt, self.gate)
        else:
            logits = F.linear(xt.float(), self.gate.float())
        idx, w = moe_ops.route_topk(logits, cfg.top_k, bias=self.expert_bias, mode="sigmoid",
                                    scale=cfg.route_scale, normalize=True, counts=self.tokens_per_expert)
        if cfg.aux_loss_coeff > 0 and torch.is_grad_enabled():
            w = _InjectAuxLoss.apply(w, self._balance_loss(logits, idx) * cfg.aux_loss_coeff)
        return idx, w

    def _balance_loss(self, logits, idx):
        """Sequence-wise balance loss ``sum_e f_e * p_e``: ``f`` = share of the selections each expert got
        (times the number of experts), ``p`` = the experts' normalised scores summed over tokens; summed over
        this microbatch's tokens and divided by ``aux_loss_denominator`` (the step's token count over all
        ranks, set by the trainer; defaults to this microbatch's). Parity: the router of the reference's
        example (``examples/deepseek_v3/model.py:489-530``)."""
        E = self.cfg.n_experts
        scores = torch.sigmoid(logits.float())
        counts = torch.zeros(E, dtype=scores.dtype, device=scores.device).index_add_(
            0, idx.reshape(-1).long(), torch.ones(idx.numel(), dtype=scores.dtype, device=scores.device))
        f = counts / counts.sum().clamp_min(1) * E
        p = (scores / scores.sum(-1, keepdim=True).clamp_min(1e-20)).sum(0)
        denom = getattr(self, "aux_loss_denominator", None)
        denom = float(logits.shape[0]) if denom is None else denom
        return (f * p).sum() / denom

    def forward(self, x):
        B, S, D = x.shape
        xt = x.reshape(-1, D)
        idx, w = self.route(xt)
        if self.dispatcher is not None:
            y = self.dispatcher(xt, idx, w, self.routed_experts)
        else:
            plan = moe_ops.plan_routes(idx, self.cfg.n_experts)
            rows = moe_ops.moe_dispatch(xt, plan)
            y = moe_ops.moe_combine(self.routed_experts(rows, plan), w, plan)
        if self.shared is not None:
            y = y + self.shared(xt)
        return y.view(B, S, D)

    @torch.no_grad()
    def update_expert_bias(self, rate: float = 1e-3, group=None):
        """Auxiliary-loss-free balancing: nudge the selection bias of under/over-loaded experts."""
        counts = self.tokens_per_expert.clone()
        if group is not None or torch.distributed.is_initialized():
            torch.distributed.all_reduce(counts, group=group)
        self.expert_bias += rate * torch.sign(counts.mean() - counts)
        self.tokens_per_expert.zero_()


class Block(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, layer: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.attention_norm = nn.Parameter(torch.empty(cfg.d_model, dtype=dtype, device=device))
        self.attention = MLA(cfg, dtype, device)
        self.ffn_norm = nn.Parameter(torch.empty(cfg.d_model, dtype=dtype, device=device))
        if layer < cfg.n_dense_layers:
            self.ffn = DenseFFN(cfg.d_model, cfg.dense_hidden, dtype, device)
        else:
            self.moe = MoE(cfg, dtype, device)

    def _forward(self, x, rope_table, doc_mask):
        x = x + self.attention(_rms(x, self.attention_norm, self.cfg.norm_eps), rope_table, doc_mask)
        h = _rms(x, self.ffn_norm, self.cfg.norm_eps)
        return x + (self.ffn(h) if hasattr(self, "ffn") else self.moe(h))

    def forward(self, x, rope_table, doc_mask=None):
        if self.cfg.activation_checkpointing and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            # per-block recompute (parity: ``examples/deepseek_v3/model.py:597-611`` of the reference)
            return checkpoint(self._forward, x, rope_table, doc_mask, use_reentrant=False)
        return self._forward(x, rope_table, doc_mask)


class DeepSeekV3(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device)
        self.layers = nn.ModuleList([Block(cfg, i, dtype, device) for i in range(cfg.n_layers)])
        self.norm = nn.Parameter(torch.empty(cfg.d_model, dtype=dtype, device=device))
        self.output = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device))
        self._rope = None

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        from ..param_init import init_from_full

        dev = self.tok_embeddings.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith("norm"):
                init_from_full(p, lambda t: t.fill_(1.0))
            else:
                init_from_full(p, lambda t: t.normal_(0.0, self.cfg.init_std, generator=g))

    def forward(self, tokens, positions=None):
        """``positions`` [B, S] (optional): token positions inside their documents; attention is then causal
        within documents (the rotary phase keeps following the position in the sequence)."""
        B, S = tokens.shape
        if self._rope is None or self._rope.device != tokens.device:
            c = self.cfg
            yarn = dict(factor=c.rope_factor, original_seq_len=c.original_seq_len, beta_fast=c.beta_fast,
                        beta_slow=c.beta_slow) if c.rope_factor != 1.0 else None
            self._rope = ew.rope_table(c.max_seq_len, c.qk_rope_dim, c.rope_theta, tokens.device, yarn=yarn)
        x = self.tok_embeddings(tokens)
        doc_mask = document_causal_mask(positions) if positions is not None else None
        for layer in self.layers:
            x = layer(x, self._rope[:S], doc_mask)
        return linear(_rms(x, self.norm, self.cfg.norm_eps), self.output).view(B * S, -1)

    def loss(self, tokens, targets, loss_is_root: bool = True, positions=None):
        return ew.cross_entropy(self(tokens, positions), targets.reshape(-1), unit_grad=loss_is_root)

    def moe_layers(self):
        return [b.moe for b in self.layers if hasattr(b, "moe")]


def deepseek_buckets(model: DeepSeekV3, mesh=None, expert_mesh=None, mp_policy=None, dense_dp_size=None):
    """tok_embeddings | per block: non-expert params (+ an expert bucket on ``expert_mesh``) | norm+output.
    Routed-expert weights are ``Shard(1)`` (their dim 0 is the expert axis), everything else
    ``Shard(0)``; router gates stay fp32 (a bucket of their own without a compute dtype). Mirrors the bucket recipe of the reference's example
    (``examples/deepseek_v3/train.py:114-175``)."""
    from ..bucket_storage import BucketSpec, MixedPrecisionPolicy
    from ..placements.shard import Shard

    mp = mp_policy or MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)

    def fn(named, m):
        return {n: Shard(1) if ".routed_experts." in n else Shard(0) for n, _ in named}

    def bucket(patterns, **kw):
        return BucketSpec(patterns, placement_fn=fn, mp_policy=mp, gradient_divide_factor=1.0, **kw)

    specs = [bucket(["tok_embeddings.*"], mesh=mesh)]
    for i, block in enumerate(model.layers):
        names = [f"layers.{i}.{n}" for n, _ in block.named_parameters()]
        experts = [n for n in names if ".routed_experts." in n]
        gates = [n for n in names if n.endswith(".gate")]
        rest = [n for n in names if n not in experts and n not in gates]
        specs.append(bucket(rest, mesh=mesh))
        if gates:
            specs.append(BucketSpec(gates, placement_fn=fn, mesh=mesh, gradient_divide_factor=1.0))
        if experts:
            specs.append(bucket(experts, mesh=expert_mesh if expert_mesh is not None else mesh))
    specs.append(bucket(["norm", "output"], mesh=mesh, reshard_after_forward=False))
    return specs
