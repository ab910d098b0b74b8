"""Muon for the DeepSeek-V3 example: Kimi-K2-style matrix split and a communication-free optimizer.

Attention projections are orthogonalised per head (and per role), routed experts per expert, every
other matrix whole, with the update scale ``0.2 * sqrt(max(rows, cols))``; embeddings, norms, router
gates and the output projection train with AdamW. Role parity: ``examples/deepseek_v3/muon.py:29-104``.
"""
from __future__ import annotations


from flex_shard_b200 import relayout_bucket
from flex_shard_b200.dist_muon import build_local_dist_muon
from flex_shard_b200.optim.adamw import FusedAdamW
from flex_shard_b200.placements import make_bucketed_owned_full_param_placement_fn


def is_muon_param(name: str, p) -> bool:
    shape = getattr(p, "_fsb_global_shape", None) or tuple(p.shape)
    if len(shape) < 2:
        return False
    return not (name.startswith("tok_embeddings") or name == "output" or name.endswith(".gate"))


def kimi_block_rows(cfg, split: str = "head") -> dict:
    """Rows of the orthogonalisation blocks of the attention projections.

    ``"head"``: one matrix per attention head (``wq_b``, ``wkv_b``).  ``"role"``: a head's parts are matrices of
    their own, as in the Kimi-K2 recipe: the no-position and rotary rows of ``wq_b``, the key and value rows of
    ``wkv_b``, and the latent and shared-rotary rows of ``wkv_a`` (parity: ``kimi_matrices`` of the reference's
    ``examples/deepseek_v3/muon.py:29-48``)."""
    if split == "head":
        return {"wq_b": cfg.qk_dim, "wkv_b": cfg.qk_nope_dim + cfg.v_dim}
    if split == "role":
        return {"wq_b": (cfg.qk_nope_dim, cfg.qk_rope_dim), "wkv_b": (cfg.qk_nope_dim, cfg.v_dim),
                "wkv_a": (cfg.kv_lora_rank, cfg.qk_rope_dim)}
    raise ValueError(f"split must be 'head' or 'role', got {split!r}")


def store_on_owners(model) -> None:
    """Move every block's non-expert bucket to whole-parameter owners (LPT with carried loads)."""
    fn = make_bucketed_owned_full_param_placement_fn(carry_loads=True)
    for st in list(model.sharded_bucket_storages):
        if st.name.startswith("layers.") and ".moe" not in st.name:
            relayout_bucket(model, st, fn)


def store_heads_blockwise(model) -> None:
    """The other communication-free layout: per-head matrices (``wq_b``, ``wkv_b``) are stored in whole head
    blocks spread over the ranks (``BlockShard`` by attention head), every other matrix whole on an owner, vectors
    as ``Shard(0)``, all in one mixed bucket per block.  Each rank then orthogonalises its own heads; the Newton-
    Schulz work of the head matrices is spread over all ranks instead of sitting on one owner."""
    from flex_shard_b200.dist_muon.placement import get_dim0_block_partitions
    from flex_shard_b200.parallel.comm import mesh_group
    from flex_shard_b200.placements import BlockShard, MixedBucketPlacement, Shard

    H = model.cfg.n_heads
    owners = make_bucketed_owned_full_param_placement_fn(carry_loads=True)

    def fn(named, mesh):
        _, _, W, _ = mesh_group(mesh)
        whole = [(n, p) for n, p in named if p.dim() >= 2 and not n.endswith(("wq_b", "wkv_b"))]
        owned = owners(whole, mesh)
        out = {}
        for n, p in named:
            if n.endswith(("wq_b", "wkv_b")):
                out[n] = MixedBucketPlacement(BlockShard(get_dim0_block_partitions(H, W), 0))
            elif n in owned:
                out[n] = MixedBucketPlacement(owned[n])
            else:
                out[n] = MixedBucketPlacement(Shard(0))
        return out

    for st in list(model.sharded_bucket_storages):
        if st.name.startswith("layers.") and ".moe" not in st.name and any(len(i.global_shape) >= 2 for i in st.infos):
            relayout_bucket(model, st, fn)


def build_muon(model, lr: float, weight_decay: float, adamw_lr: float | None = None, split: str = "head"):
    """Muon over every matrix (per head, or per head and role, for the attention up-projections, per expert for
    routed experts, whole otherwise) + AdamW for the rest. The split needs the model's config (``model.cfg``)."""
    cfg = getattr(model, "cfg", None)
    heads = kimi_block_rows(cfg, split) if cfg is not None and hasattr(cfg, "qk_nope_dim") else None
    muon = build_local_dist_muon(model, is_muon_param=is_muon_param, block_rows_by_fqn=heads, lr=lr,
                                 weight_decay=weight_decay, adjust_lr_fn="match_rms_adamw")
    rest = [p for n, p in model.named_parameters() if not is_muon_param(n, p)]
    adam = FusedAdamW(rest, lr=adamw_lr or lr, betas=(0.9, 0.95), weight_decay=weight_decay)
    return muon, adam
