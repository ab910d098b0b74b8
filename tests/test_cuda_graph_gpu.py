"""Forward + backward with gradient reduction into the fp32 buckets, captured in a CUDA graph,
replays bitwise like the eager step and leaves the runtime idle (parity with the reference's
``tests/test_flex_shard_cuda_graph.py:48-211`` for the single-rank case)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(seed):
    from flex_shard_b200 import flex_shard
    from flex_shard_b200.models.llama import Llama, LlamaConfig, llama_buckets
    from flex_shard_b200.optim.adamw import FusedAdamW

    dev = torch.device("cuda")
    cfg = LlamaConfig(vocab_size=2048, d_model=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_hidden=512, max_seq_len=256)
    torch.manual_seed(seed)
    model = Llama(cfg, dtype=torch.bfloat16, device=dev)
    model.init_weights(seed)
    for p in model.parameters():
        p.grad_dtype = torch.float32
    flex_shard(model, llama_buckets(model, mesh=None))
    opt = FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.1, capturable=True) \
        if "capturable" in FusedAdamW.__init__.__code__.co_varnames else FusedAdamW(model.parameters(), lr=1e-3, weight_decay=0.1)
    return cfg, model, opt


def test_captured_step_replays_like_eager():
    from flex_shard_b200 import ops

    dev = torch.device("cuda")
    cfg, eager, eopt = _build(0)
    _, graphed, gopt = _build(0)
    toks = [torch.randint(0, cfg.vocab_size, (2, 257), generator=torch.Generator().manual_seed(s)).to(dev) for s in range(6)]

    def step(model, opt, tok):
        loss = model.loss(tok[:, :-1], tok[:, 1:])
        loss.backward()
        grads = [p.grad.detach().float().clone() for p in model.parameters() if p.grad is not None]
        opt.zero_grad()
        return loss.detach(), grads

    # warm-up on a side stream (allocations, learned prefetch order, kernel attributes)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(3):
            step(graphed, gopt, toks[i])
    torch.cuda.current_stream().wait_stream(s)
    static_tok = toks[3].clone()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        static_loss, static_grads = step(graphed, gopt, static_tok)
    for i in range(3, 6):
        static_tok.copy_(toks[i])
        g.replay()
        loss_e, grads_e = step(eager, eopt, toks[i])
        assert torch.equal(static_loss, loss_e)
        assert len(static_grads) == len(grads_e) and len(grads_e) > 0
        for a, b in zip(static_grads, grads_e):
            assert torch.equal(a, b)
    torch.cuda.synchronize()
    ops.check_status()
    assert graphed.sharded_bucket_storages[0].runtime.context.idle()
