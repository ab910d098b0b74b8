"""Runs ONE kernel of the library on a small, fixed case: the workload behind each profile summary.

    python -m flex_shard_b200.utils.kernel_cases <case> [--iters N]

Cases: gemm_fwd, gemm_dgrad, gemm_wgrad, attn_fwd, attn_bwd, attn_bwd_ordered, adamw, rmsnorm, rmsnorm_bwd, swiglu, cross_entropy,
newton_schulz, newton_schulz_batched, fp8_quant, fp8_gemm, mxfp8_gemm, allgather_gemm, segment_cast. Each prints one JSON line with the CUDA-event time (median of
``iters`` launches after 3 warm-up launches, L2 flushed between launches by writing a 256 MB buffer)
and the achieved FLOP/s or bytes/s. Inputs are a few hundred MB, larger than the 126 MB L2, so DRAM
counters of a profiler capture of the same command stay meaningful.
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters):
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    from flex_shard_b200 import ops
    from flex_shard_b200.ops import attention as att
    from flex_shard_b200.ops import elementwise as ew

    dev = torch.device("cuda")
    torch.manual_seed(0)
    out = {"case": args.case}
    if args.case.startswith("gemm_"):
        M, N, K = 8192, 14336, 4096
        kind = args.case[5:]
        if kind == "fwd":
            a = torch.randn(M, K, device=dev).bfloat16()
            b = torch.randn(N, K, device=dev).bfloat16()
            d = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: ops.gemm(a, b, out=d)
        elif kind == "dgrad":
            a = torch.randn(M, N, device=dev).bfloat16()   # dy [T, out]
            b = torch.randn(N, K, device=dev).bfloat16()   # W  [out, in]
            d = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
            fn = lambda: ops.gemm(a, b, b_t=True, out=d)
        else:
            a = torch.randn(M, N, device=dev).bfloat16()   # dy [T, out]
            b = torch.randn(M, K, device=dev).bfloat16()   # x  [T, in]
            d = torch.empty(N, K, device=dev, dtype=torch.float32)
            fn = lambda: ops.gemm(a, b, a_t=True, b_t=True, out=d)
        ms = _time(fn, args.iters)
        out.update(M=M, N=N, K=K, ms=ms, tflops=2.0 * M * N * K / ms / 1e9)
    elif args.case in ("attn_fwd", "attn_bwd", "attn_bwd_ordered"):
        att.set_deterministic(args.case == "attn_bwd_ordered")
        B, S, Hq, Hkv = 1, 8192, 16, 4
        qkv = (0.5 * torch.randn(B, S, (Hq + 2 * Hkv) * 128, device=dev)).bfloat16()
        flops_fwd = 4.0 * B * Hq * S * S * 128 * 0.5
        if args.case == "attn_fwd":
            with torch.no_grad():
                fn = lambda: att.qkv_attention(qkv, None, Hq, Hkv)
                ms = _time(fn, args.iters)
            out.update(B=B, S=S, Hq=Hq, Hkv=Hkv, ms=ms, tflops=flops_fwd / ms / 1e9)
        else:
            x = qkv.clone().requires_grad_()
            o = att.qkv_attention(x, None, Hq, Hkv)
            g = torch.randn_like(o)
            fn = lambda: torch.autograd.grad(o, x, g, retain_graph=True)
            ms = _time(fn, args.iters)
            out.update(B=B, S=S, Hq=Hq, Hkv=Hkv, ms=ms, tflops=2.5 * flops_fwd / ms / 1e9,
                       note="time includes the delta, dq-zero and dq-cast helper kernels")
    elif args.case == "adamw":
        n = 128 * 1024 * 1024
        p = torch.randn(n, device=dev).bfloat16()
        g = torch.randn(n, device=dev)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        fn = lambda: ew.adamw_step_(p, g, m, v, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1, step=3)
        ms = _time(fn, args.iters)
        out.update(n=n, ms=ms, gbs=n * 24 / ms / 1e6)
    elif args.case == "segment_cast":
        # a Llama layer bucket's gradient copy-in: seven bf16 weight gradients widened into one fp32 row
        from flex_shard_b200.ops.segments import run_segment_ops

        shapes = [(6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (4096,), (4096,)]
        srcs = [torch.randn(*sh, device=dev).bfloat16() for sh in shapes]
        n = sum(t.numel() for t in srcs)
        row = torch.empty(n, device=dev)
        dsts, o = [], 0
        for t in srcs:
            dsts.append(row[o:o + t.numel()].view(t.shape))
            o += t.numel()
        fn = lambda: run_segment_ops(list(zip(dsts, srcs)))
        ms = _time(fn, args.iters)
        out.update(elements=n, ms=ms, gbs=n * 6 / ms / 1e6)
    elif args.case == "rmsnorm":
        T, D = 32768, 4096
        x = torch.randn(T, D, device=dev).bfloat16()
        w = torch.ones(D, device=dev).bfloat16()
        with torch.no_grad():
            ms = _time(lambda: ew.rmsnorm(x, w), args.iters)
        out.update(T=T, D=D, ms=ms, gbs=T * D * 4 / ms / 1e6)
    elif args.case == "rmsnorm_bwd":
        # the Llama step's shape: one sequence of 8192 tokens, with the residual-stream gradient added in
        T, D = 8192, 4096
        x = torch.randn(T, D, device=dev).bfloat16().requires_grad_()
        res = torch.randn(T, D, device=dev).bfloat16().requires_grad_()
        w = torch.ones(D, device=dev).bfloat16().requires_grad_()
        y, s2 = ew.add_rmsnorm(x, res, w)
        gy, gs = torch.randn_like(y), torch.randn_like(s2)
        fn = lambda: torch.autograd.grad((y, s2), (x, res, w), (gy, gs), retain_graph=True)
        ms = _time(fn, args.iters)
        out.update(T=T, D=D, ms=ms, gbs=T * D * 2 * 4 / ms / 1e6,
                   note="bytes: dy, x, residual gradient in, dx out; time includes the column-sum kernel of dw")
    elif args.case == "swiglu":
        T, F = 16384, 14336
        gu = torch.randn(T, 2 * F, device=dev).bfloat16()
        with torch.no_grad():
            ms = _time(lambda: ew.swiglu(gu), args.iters)
        out.update(T=T, F=F, ms=ms, gbs=T * F * 6 / ms / 1e6)
    elif args.case == "cross_entropy":
        T, V = 4096, 128256
        logits = torch.randn(T, V, device=dev).bfloat16()
        tgt = torch.randint(0, V, (T,), device=dev)
        with torch.no_grad():
            ms = _time(lambda: ew.cross_entropy(logits, tgt), args.iters)
        out.update(T=T, V=V, ms=ms, gbs=T * V * 4 / ms / 1e6)
    elif args.case == "newton_schulz":
        from flex_shard_b200.ops.newton_schulz import newton_schulz

        x = torch.randn(4096, 14336, device=dev).bfloat16()
        ms = _time(lambda: newton_schulz(x, steps=5), args.iters)
        s, l = 4096, 14336
        dense = 5 * (2 * 2 * s * s * l + 2 * s * s * s)            # every product computed in full
        done = 5 * (3 * s * s * l + s * s * s)                     # the two symmetric products computed by halves
        out.update(rows=s, cols=l, ms=ms, tflops=dense / ms / 1e9, tflops_executed=done / ms / 1e9,
                   note="tflops counts the dense algorithm; tflops_executed discounts the mirrored halves "
                        "(diagonal tiles are computed in full, so it is a slight under-count)")
    elif args.case == "newton_schulz_batched":
        # sixteen expert-sized matrices: one grouped launch per product against one matrix at a time
        from flex_shard_b200.ops.newton_schulz import newton_schulz

        E, s, l = 16, 1024, 2048
        x = torch.randn(E, s, l, device=dev).bfloat16()
        ms = _time(lambda: newton_schulz(x, steps=5), args.iters)
        ms_loop = _time(lambda: [newton_schulz(x[i], steps=5) for i in range(E)], args.iters)
        dense = E * 5 * (2 * 2 * s * s * l + 2 * s * s * s)
        out.update(matrices=E, rows=s, cols=l, ms=ms, tflops=dense / ms / 1e9, one_at_a_time_ms=ms_loop)
    elif args.case == "fp8_quant":
        from flex_shard_b200.ops.fp8 import quantize_blockwise

        w = torch.randn(14336, 4096, device=dev).bfloat16()
        ms = _time(lambda: quantize_blockwise(w), args.iters)
        out.update(rows=14336, cols=4096, ms=ms, gbs=14336 * 4096 * 3 / ms / 1e6)
    elif args.case == "fp8_gemm":
        from flex_shard_b200.ops.fp8 import fp8_linear_forward, quantize_blockwise

        M, N, K = 8192, 14336, 4096
        x = torch.randn(M, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        wq, ws = quantize_blockwise(w)
        ms = _time(lambda: fp8_linear_forward(x, wq, ws), args.iters)
        out.update(M=M, N=N, K=K, ms=ms, tflops=2.0 * M * N * K / ms / 1e9,
                   note="includes the 1x128 activation quantisation")
    elif args.case == "mxfp8_gemm":
        from flex_shard_b200.ops import mxfp8 as mx

        M, N, K = 8192, 14336, 4096
        x = torch.randn(M, K, device=dev).bfloat16()
        w = torch.randn(N, K, device=dev).bfloat16()
        wq, e = mx.mx_quantize_weight(w)
        fwd = mx.mx_expand_scales(e, N, K, False)
        xq, sx = mx.mx_quantize_act(x)
        ms = _time(lambda: mx.gemm_mxfp8(xq, sx, wq, fwd), args.iters)
        out.update(M=M, N=N, K=K, ms=ms, tflops=2.0 * M * N * K / ms / 1e9, note="GEMM only (operands pre-quantised)")
        ms_q = _time(lambda: mx.mx_quantize_act(x), args.iters)
        out.update(act_quant_ms=ms_q, act_quant_gbs=M * K * 3 / ms_q / 1e6)
        try:   # the library's block-scaled product on the same operands, when this torch build has it
            sa = sx.view(torch.float8_e8m0fnu)
            sb = fwd.view(torch.float8_e8m0fnu)
            f = lambda: torch._scaled_mm(xq, wq.t(), scale_a=sa, scale_b=sb, out_dtype=torch.bfloat16)
            ref = f()
            ours = mx.gemm_mxfp8(xq, sx, wq, fwd)
            ms_l = _time(f, args.iters)
            out.update(cublaslt_ms=ms_l, cublaslt_tflops=2.0 * M * N * K / ms_l / 1e9,
                       max_abs_diff_vs_cublaslt=float((ref.float() - ours.float()).abs().max()))
        except Exception as ex:  # noqa: BLE001
            out.update(cublaslt="unavailable: " + str(ex).split("\n")[0][:120])
    elif args.case == "allgather_gemm":
        # 8 emulated peers on one GPU (the stager CTAs run the same bulk-copy ring; on a multi-GPU
        # job the sources are NVLink peer addresses instead of local ones)
        from flex_shard_b200.ops.fused import AllGatherLinear

        M, N, K, W = 8192, 14336, 4096, 8
        w = torch.randn(N, K, device=dev).bfloat16()
        c = N // W
        shards = [w[r * c:(r + 1) * c].clone() for r in range(W)]
        lin = AllGatherLinear([t.data_ptr() for t in shards], N, K, c, dev, n_stagers=12)
        x = torch.randn(M, K, device=dev).bfloat16()
        ms = _time(lambda: lin(x), args.iters)
        out.update(M=M, N=N, K=K, world=W, ms=ms, tflops=2.0 * M * N * K / ms / 1e9,
                   gathered_gbs=N * K * 2 / ms / 1e6)
    else:
        raise SystemExit(f"unknown case {args.case}")
    ops.check_status()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
