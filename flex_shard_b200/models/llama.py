"""Llama-3-shaped dense decoder running on this library's sm_100a kernels.

Per block: RMSNorm -> fused QKV projection (tcgen05 GEMM) -> RoPE + causal GQA
flash attention -> output projection -> fused residual-add + RMSNorm -> fused
gate/up projection -> SwiGLU -> down projection. The query/key/value and gate/up
weights are stored fused (``wqkv``, ``w13``) so each is one GEMM and one shard.
The loss is a fused cross-entropy that leaves dlogits in place of the logits.

The same module runs on CPU tensors through the ops' PyTorch reference paths
(used by the CPU test-suite with tiny shapes).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import elementwise as ew
from ..ops.attention import qkv_attention
from ..ops.gemm import linear


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    ffn_hidden: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    max_seq_len: int = 8192
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    def num_params(self) -> int:
        d, f, v = self.d_model, self.ffn_hidden, self.vocab_size
        qkv = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim * d
        per_layer = qkv + d * d + 2 * f * d + f * d + 2 * d
        return self.n_layers * per_layer + 2 * v * d + d

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (fwd + bwd = 3x fwd), causal attention counted at half."""
        d, f, v = self.d_model, self.ffn_hidden, self.vocab_size
        qkv = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim * d
        dense = self.n_layers * (qkv + d * d + 3 * f * d) + v * d
        attn = self.n_layers * 2 * seq_len * d * 0.5  # QK^T and PV, causal
        return 6.0 * dense + 6.0 * attn


LLAMA3_8B = LlamaConfig()


class LlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        d, f, hd = cfg.d_model, cfg.ffn_hidden, cfg.head_dim
        kw = dict(dtype=dtype, device=device)
        self.attention_norm = nn.Parameter(torch.empty(d, **kw))
        self.wqkv = nn.Parameter(torch.empty((cfg.n_heads + 2 * cfg.n_kv_heads) * hd, d, **kw))
        self.wo = nn.Parameter(torch.empty(d, d, **kw))
        self.ffn_norm = nn.Parameter(torch.empty(d, **kw))
        self.w13 = nn.Parameter(torch.empty(2 * f, d, **kw))
        self.w2 = nn.Parameter(torch.empty(d, f, **kw))

    def forward(self, x, delta, rope_table):
        """``x`` is the residual stream, ``delta`` the previous block's MLP output not yet added
        (``None`` for the first block). Returns the new pair."""
        cfg = self.cfg
        if delta is None:
            a = ew.rmsnorm(x, self.attention_norm, cfg.norm_eps)
        else:
            a, x = ew.add_rmsnorm(delta, x, self.attention_norm, cfg.norm_eps)
        qkv = linear(a, self.wqkv)
        o = qkv_attention(qkv, rope_table, cfg.n_heads, cfg.n_kv_heads)
        attn_out = linear(o, self.wo)
        m, x = ew.add_rmsnorm(attn_out, x, self.ffn_norm, cfg.norm_eps)
        h = ew.swiglu(linear(m, self.w13))
        return x, linear(h, self.w2)


class LlamaHead(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.norm = nn.Parameter(torch.empty(cfg.d_model, dtype=dtype, device=device))
        self.output = nn.Parameter(torch.empty(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device))

    def forward(self, x, delta):
        h, _ = ew.add_rmsnorm(delta, x, self.norm, self.cfg.norm_eps)
        return linear(h, self.output)


class Llama(nn.Module):
    def __init__(self, cfg: LlamaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.tok_embeddings = nn.Embedding(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device)
        self.layers = nn.ModuleList([LlamaBlock(cfg, dtype, device) for _ in range(cfg.n_layers)])
        self.head = LlamaHead(cfg, dtype, device)
        self._rope = None

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        from ..param_init import init_from_full

        dev = self.tok_embeddings.weight.device
        g = torch.Generator(device=dev).manual_seed(seed)
        std = self.cfg.init_std
        for name, p in self.named_parameters():
            if name.endswith("norm"):
                init_from_full(p, lambda t: t.fill_(1.0))
            else:
                init_from_full(p, lambda t: t.normal_(0.0, std, generator=g))

    def rope_table(self, device):
        if self._rope is None or self._rope.device != device:
            self._rope = ew.rope_table(self.cfg.max_seq_len, self.cfg.head_dim, self.cfg.rope_theta, device)
        return self._rope

    def forward(self, tokens):
        """tokens [B, S] -> logits [B*S, V] (bf16)."""
        B, S = tokens.shape
        table = self.rope_table(tokens.device)[:S]
        x = self.tok_embeddings(tokens)
        delta = None
        for layer in self.layers:
            x, delta = layer(x, delta, table)
        logits = self.head(x, delta)
        return logits.view(B * S, -1)

    def loss(self, tokens, targets, loss_is_root: bool = True):
        """Mean next-token cross-entropy over all positions of ``targets`` (ignore_index -100).
        With ``loss_is_root`` the returned loss must be what ``backward()`` is called on (its
        incoming gradient is taken to be 1, which saves a pass over the logits)."""
        logits = self(tokens)  # through __call__, so that root-level bucket hooks run
        return ew.cross_entropy(logits, targets.reshape(-1), unit_grad=loss_is_root)


def llama_quantized_buckets(model: Llama, mesh=None, kind: str = "fp8", mp_policy=None):
    """Buckets for a quantised all-gather: every block's 2-D weights travel as FP8 128x128 blocks
    (``kind="fp8"``) or MXFP8 (``kind="mxfp8"``) and feed the block-scaled GEMMs; norms, embedding and
    head stay ``Shard(0)`` in bf16."""
    from ..bucket_storage import BucketSpec, MixedPrecisionPolicy
    from ..placements import make_fp8_bucketed_block_shard_placement_fn, make_mxfp8_bucketed_block_shard_placement_fn
    from ..placements.shard import shard_placement_fn

    mp = mp_policy or MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    qfn = make_fp8_bucketed_block_shard_placement_fn() if kind == "fp8" else make_mxfp8_bucketed_block_shard_placement_fn()
    plain = dict(mesh=mesh, mp_policy=mp, placement_fn=shard_placement_fn(0))
    specs = [BucketSpec(["tok_embeddings"], **plain)]
    for i in range(len(model.layers)):
        specs.append(BucketSpec([f"layers.{i}.w*"], mesh=mesh, mp_policy=mp, placement_fn=qfn))
        specs.append(BucketSpec([f"layers.{i}.*norm"], **plain))
    specs.append(BucketSpec(["head"], reshard_after_forward=False, **plain))
    return specs


def llama_buckets(model: Llama, mesh=None, mp_policy=None, placement_fn=None, fsdp2_compatible=True):
    """One bucket per block plus embedding and head buckets, FSDP2-style."""
    from ..bucket_storage import BucketSpec, MixedPrecisionPolicy

    from ..placements.shard import shard_placement_fn

    mp = mp_policy or MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    placement_fn = placement_fn or shard_placement_fn(0, grad_bucket=True)
    kw = dict(mesh=mesh, mp_policy=mp, placement_fn=placement_fn, fsdp2_compatible=fsdp2_compatible)
    specs = [BucketSpec(["tok_embeddings"], **kw)]
    for i in range(len(model.layers)):
        specs.append(BucketSpec([f"layers.{i}"], **kw))
    specs.append(BucketSpec(["head"], reshard_after_forward=False, **kw))
    return specs
