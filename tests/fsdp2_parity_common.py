"""Shared pieces of the FSDP2-parity tests: a small decoder, the two ways to shard it, a training
loop that records every all-gather and reduce-scatter input, and the comparison.

The contract under test is the reference's first promise: ``Shard`` buckets marked
``fsdp2_compatible`` issue the same collectives on the same bytes as
``torch.distributed.fsdp.fully_shard`` with the same grouping, so losses, gradients and
parameters are equal bit for bit on any backend
(``src/flex_shard/tests/test_flex_shard_fsdp2_parity.py:45-69,207-238,493-603``).
"""
import contextlib
import itertools
from collections import defaultdict

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

VOCAB, DIM, HIDDEN, BATCH = 13, 11, 8, 5   # DIM odd: every dim-0 shard pads; HIDDEN divides by 2 and 4

DTYPES = [(None, None), (torch.bfloat16, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.bfloat16, None)]
FACTORS = [None, 1.0]
ACCUMULATION = [(1, False), (2, False), (2, True)]   # (microbatches, skip the reduction on all but the last)


def configs():
    return list(itertools.product(DTYPES, FACTORS, ACCUMULATION))


class PairedProjection(nn.Module):
    """Gate and up projections stored as one ``[2, HIDDEN, DIM]`` tensor, sharded on its matrix rows."""

    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(2, HIDDEN, DIM) * 0.3)
        self.bias = nn.Parameter(torch.randn(2, HIDDEN) * 0.1)

    def forward(self, x):
        y = torch.einsum("bd,nfd->nbf", x, self.weight) + self.bias[:, None, :]
        return F.silu(y[0]) * y[1]


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.gain = nn.Parameter(torch.rand(DIM) + 0.5)   # own parameter, registered before the children
        self.pair = PairedProjection()
        self.down = nn.Linear(HIDDEN, DIM)
        self.idle = nn.Linear(DIM, 3)                     # never used: gets no gradient; 3 rows leave rank 3 of 4 empty

    def forward(self, x):
        return x + self.down(self.pair(x * self.gain)) * self.gain   # gain is used twice


class Decoder(nn.Module):
    def __init__(self, n_layers: int = 2):
        super().__init__()
        self.tok_embeddings = nn.Embedding(VOCAB, DIM)
        self.layers = nn.ModuleList(Block() for _ in range(n_layers))
        self.norm = nn.LayerNorm(DIM)
        self.lm_head = nn.Linear(DIM, VOCAB, bias=False)
        self.norm.bias.requires_grad_(False)
        self.return_hidden = False    # chunked loss: the caller applies lm_head itself
        self.head_twice = False       # multi-token-prediction style: the head group runs twice per forward

    def forward(self, tokens):
        h = self.tok_embeddings(tokens)
        for layer in self.layers:
            h = layer(h)
        if self.return_hidden:
            return self.norm(h)
        out = self.lm_head(self.norm(h))
        if self.head_twice:
            out = out + self.lm_head(self.norm(torch.flip(h, dims=(0,))))
        return out


def shard_dim(fqn: str) -> int:
    return 1 if ".pair." in fqn else 0


def apply_fsdp2(model, mesh, param_dtype, reduce_dtype, factor, head_reshard=False):
    from torch.distributed.fsdp import FSDPModule, MixedPrecisionPolicy, fully_shard
    from torch.distributed.tensor import Shard as DShard

    dims = {p: shard_dim(n) for n, p in model.named_parameters()}
    kw = dict(mesh=mesh, mp_policy=MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype,
                                                       cast_forward_inputs=False))
    fully_shard(model.tok_embeddings, reshard_after_forward=True, **kw)
    fully_shard([model.norm, model.lm_head], reshard_after_forward=head_reshard, **kw)
    for layer in model.layers:
        fully_shard(layer, reshard_after_forward=True, shard_placement_fn=lambda p: DShard(dims[p]), **kw)
    fully_shard(model, **kw)
    if factor is not None:
        for m in model.modules():
            if isinstance(m, FSDPModule):
                m.set_gradient_divide_factor(factor)
                if mesh.device_type == "cpu":   # gloo has no pre-multiplied sum: sum, then divide by the factor
                    m.set_force_sum_reduction_for_comms(True)


def apply_flex(model, mesh, param_dtype, reduce_dtype, factor, head_reshard=False, fsdp2_compatible=True):
    from flex_shard_b200 import BucketSpec, MixedPrecisionPolicy, flex_shard
    from flex_shard_b200.placements import Shard

    def placement_fn(named, mesh_):
        return {fqn: Shard(shard_dim(fqn)) for fqn, _ in named}

    def bucket(patterns, reshard):
        return BucketSpec(patterns, placement_fn=placement_fn, mesh=mesh,
                          mp_policy=MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype),
                          gradient_divide_factor=factor, reshard_after_forward=reshard,
                          fsdp2_compatible=fsdp2_compatible)

    flex_shard(model, [bucket(["tok_embeddings"], True),
                       *(bucket([f"layers.{i}"], True) for i in range(len(model.layers))),
                       bucket(["norm", "lm_head"], head_reshard)])


@contextlib.contextmanager
def record_collectives():
    """Record the input of every all-gather / reduce-scatter issued through ``torch.distributed``."""
    seen = defaultdict(list)
    ag, rs = dist.all_gather_into_tensor, dist.reduce_scatter_tensor

    def rec_ag(output_tensor, input_tensor, *a, **k):
        seen["all_gather"].append(input_tensor.detach().clone())
        return ag(output_tensor, input_tensor, *a, **k)

    def rec_rs(output, input, *a, **k):
        seen["reduce_scatter"].append(input.detach().clone())
        return rs(output, input, *a, **k)

    dist.all_gather_into_tensor, dist.reduce_scatter_tensor = rec_ag, rec_rs
    try:
        yield seen
    finally:
        dist.all_gather_into_tensor, dist.reduce_scatter_tensor = ag, rs


def local(t):
    return t.to_local() if hasattr(t, "to_local") else t


def chunked_loss(model, tokens, targets, chunks: int):
    """The loss torchtitan-style trainers use for large vocabularies: the trunk runs once, the head is
    applied per chunk of the batch on detached hidden states, and the trunk's backward runs on the
    accumulated hidden-state gradient."""
    from torch.distributed.fsdp import FSDPModule

    head = model.lm_head
    model.return_hidden = True
    hidden = model(tokens)
    model.return_hidden = False
    leaf = hidden.detach().requires_grad_(True)
    total = None
    pieces = list(zip(leaf.chunk(chunks), targets.chunk(chunks)))
    for i, (h, t) in enumerate(pieces):
        last = i == len(pieces) - 1
        if isinstance(head, FSDPModule):
            head.set_requires_gradient_sync(last, recurse=False)
            head.set_reshard_after_backward(last, recurse=False)
        else:
            st = model.bucket_storage_of(head.weight)
            st.set_requires_gradient_sync(last)
            st.set_reshard_after_backward(last)
        loss = F.cross_entropy(head(h).float(), t, reduction="sum") / tokens.numel()
        loss.backward()
        total = loss.detach() if total is None else total + loss.detach()
    hidden.backward(leaf.grad)
    return total


def train(model, device, rank, steps, microbatches, no_sync, loss_chunks=0):
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2, foreach=True)
    history = []
    for step in range(steps):
        losses = []
        for mb in range(microbatches):
            if no_sync:
                model.set_requires_gradient_sync(mb == microbatches - 1)
            g = torch.Generator().manual_seed(10_000 * step + 100 * mb + rank)
            tokens = torch.randint(VOCAB, (BATCH * (loss_chunks or 1),), generator=g).to(device)
            targets = torch.randint(VOCAB, (BATCH * (loss_chunks or 1),), generator=g).to(device)
            if loss_chunks:
                losses.append(chunked_loss(model, tokens, targets, loss_chunks))
            else:
                loss = F.cross_entropy(model(tokens).float(), targets)
                loss.backward()
                losses.append(loss.detach())
        grads = {n: None if p.grad is None else local(p.grad).detach().clone() for n, p in model.named_parameters()}
        opt.step()
        opt.zero_grad()
        params = {n: local(p).detach().clone() for n, p in model.named_parameters()}
        history.append({"losses": losses, "grads": grads, "params": params})
    return history


def compare(a, b, what=""):
    """Return a list of mismatch descriptions between two training histories (empty: bitwise equal)."""
    bad = []
    for s, (ha, hb) in enumerate(zip(a, b)):
        for i, (la, lb) in enumerate(zip(ha["losses"], hb["losses"])):
            if not torch.equal(la, lb):
                bad.append(f"{what} step {s} loss {i}: {float(la)!r} vs {float(lb)!r}")
        for key in ("grads", "params"):
            for n in ha[key]:
                x, y = ha[key][n], hb[key][n]
                if (x is None) != (y is None):
                    bad.append(f"{what} step {s} {key[:-1]} {n}: one side is None")
                elif x is not None and (x.shape != y.shape or x.dtype != y.dtype or not torch.equal(x, y)):
                    bad.append(f"{what} step {s} {key[:-1]} {n}: shape {tuple(x.shape)}/{tuple(y.shape)} "
                               f"dtype {x.dtype}/{y.dtype} maxdiff "
                               f"{float((x.float() - y.float()).abs().max()) if x.shape == y.shape and x.numel() else 'n/a'}")
    return bad


def compare_collectives(ra, rb, what=""):
    bad = []
    for kind in ("all_gather", "reduce_scatter"):
        xa, xb = ra.get(kind, []), rb.get(kind, [])
        if len(xa) != len(xb):
            bad.append(f"{what} {kind}: {len(xa)} vs {len(xb)} calls")
            continue
        for i, (x, y) in enumerate(zip(xa, xb)):
            # bytes, not dtypes: one side may hand the collective a byte view of the same memory
            xb_, yb_ = x.contiguous().view(-1).view(torch.uint8), y.contiguous().view(-1).view(torch.uint8)
            if xb_.numel() != yb_.numel() or not torch.equal(xb_, yb_):
                bad.append(f"{what} {kind} call {i}: dtype {x.dtype}/{y.dtype} bytes {xb_.numel()}/{yb_.numel()}")
    return bad


def run_pair(device, mesh, rank, cfg, steps=2, variant="plain", record=True):
    """Train the FSDP2 model and the flex_shard model from the same initial weights; returns the
    list of mismatches."""
    import copy

    (param_dtype, reduce_dtype), factor, (microbatches, no_sync) = cfg
    torch.manual_seed(42)
    base = Decoder().to(device)
    base.head_twice = variant == "head_twice"
    chunks = 3 if variant == "chunked" else 0
    a, b = copy.deepcopy(base), copy.deepcopy(base)
    apply_fsdp2(a, mesh, param_dtype, reduce_dtype, factor)
    apply_flex(b, mesh, param_dtype, reduce_dtype, factor)
    with record_collectives() as ra:
        ha = train(a, device, rank, steps, microbatches, no_sync, chunks)
    with record_collectives() as rb:
        hb = train(b, device, rank, steps, microbatches, no_sync, chunks)
    tag = (f"[param={param_dtype} reduce={reduce_dtype} factor={factor} mb={microbatches} no_sync={no_sync} "
           f"{variant}]")
    bad = compare(ha, hb, tag)
    if record:
        bad += compare_collectives(ra, rb, tag)
    return bad
