"""Single-kernel timing through the C ABI, for roofline numbers and profiler captures.

    python -m turbotransformers_b200.microbench linear    --m 18424 --n 2304 --k 768 --epilogue bias [--dtype f16|bf16|i8]
    python -m turbotransformers_b200.microbench attention --lens varlen64 | --batch 32 --seq 512 [--heads 12] [--causal]
    python -m turbotransformers_b200.microbench layernorm --m 18424 --n 768
    python -m turbotransformers_b200.microbench gelu      --m 18424 --n 3072
    python -m turbotransformers_b200.microbench decode    --batch 64 --seq 1024 [--heads 12]   # one-token step over a cache

Each run launches the kernel `--warmup` + `--iters` times on synthetic data, writes a >L2 buffer between timed
launches, times every launch with CUDA events on the launching stream, and prints one JSON line with the
mean duration and the achieved algorithmic FLOP/s or bytes/s.
"""
import argparse
import json

import numpy as np
import torch

from . import _capi, synthetic

DT = {"f16": (torch.float16, _capi.F16), "bf16": (torch.bfloat16, _capi.BF16), "f32": (torch.float32, _capi.F32)}
EPI = {"none": 0, "bias": 1, "bias_gelu": 2, "bias_residual": 3, "bias_tanh": 4}


def timed_burst(fns, warmup, iters):
    """Mean duration of one launch inside a back-to-back run over len(fns) different buffer sets (launch latency is
    hidden as it is inside a model step; the rotating buffers keep the inputs out of L2)."""
    for _ in range(warmup):
        for f in fns:
            f()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for f in fns:
            f()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) / len(fns))
    ts.sort()
    return sum(ts) / len(ts), ts[len(ts) // 2], ts[0]


def timed_graph(ctx, fns, warmup, iters):
    """Mean device time of one launch with the host out of the picture: the launches of `fns` (different buffer sets) are
    recorded once into a CUDA graph and the graph is replayed. What is left is the kernel and the gap to its neighbour,
    as inside a replayed forward pass."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ctx.set_stream(side.cuda_stream)
        for _ in range(max(1, warmup)):
            for f in fns:
                f()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for f in fns:
                f()
    torch.cuda.current_stream().wait_stream(side)
    ctx.set_stream(torch.cuda.current_stream().cuda_stream)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) / len(fns))
    ts.sort()
    return sum(ts) / len(ts), ts[len(ts) // 2], ts[0]


def timed(fn, warmup, iters, flush=True):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for s, e in evs:
        if flush:
            buf.zero_()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    t = sorted(s.elapsed_time(e) for s, e in evs)
    return sum(t) / len(t), t[len(t) // 2], t[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["linear", "matmul", "attention", "layernorm", "gelu", "decode"])
    ap.add_argument("--m", type=int, default=18424)
    ap.add_argument("--n", type=int, default=2304)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16", "f32", "i8"])
    ap.add_argument("--epilogue", default="bias", choices=list(EPI))
    ap.add_argument("--lens", default=None, help="'varlen64' = the benchmark's 64 lengths in [8,512]")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--key-mask", default=None, choices=["padding", "scattered"],
                    help="attention: pass a per-key additive mask [B, max_len]: a padding mask (a suffix of every sequence at -10000) or a quarter of the keys at random")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--burst", type=int, default=0, help="linear/attention: time this many back-to-back launches on rotating buffer sets")
    ap.add_argument("--graph", action="store_true", help="with --burst: replay the launches from a CUDA graph (no host time in the number)")
    ap.add_argument("--b-trans", action="store_true", help="matmul: B is stored [N, K]")
    ap.add_argument("--yardstick", action="store_true", help="matmul: also time torch.matmul (cuBLAS SGEMM, TF32 off) on the same operands")
    ap.add_argument("--fuse-ln", action="store_true", help="linear: ttb_linear_layernorm (bias + residual + LayerNorm); one kernel only with TTB_GEMM_LN=1 or 2 in the environment")
    ap.add_argument("--plain", action="store_true", help="layernorm: the in-place LayerNorm the encoder layers run (no residual / bias add)")
    ap.add_argument("--pad-rows", action="store_true", help="linear: output rows padded to a multiple of 8 elements, padding declared scratch")
    a = ap.parse_args()
    ctx = _capi.Context(0)
    out = {"op": a.op}
    if a.op == "linear":
        M, N, K = a.m, a.n, a.k
        odt, ocode = DT["f16" if a.dtype == "i8" else a.dtype]
        b = torch.randn(N, device="cuda", dtype=odt)
        r = torch.randn(M, N, device="cuda", dtype=odt)
        o = torch.empty(M, N, device="cuda", dtype=odt)
        if a.dtype == "i8":
            x = torch.randint(-127, 128, (M, K), device="cuda", dtype=torch.int8)
            w = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
            xs, ws = torch.rand(M, device="cuda"), torch.rand(1, device="cuda")
            fn = lambda: ctx.call("linear_int8", ocode, x, xs, w, ws, b, r, N, M, N, K, EPI[a.epilogue], o, N)
        else:
            x = torch.randn(M, K, device="cuda", dtype=odt)
            w = torch.randn(N, K, device="cuda", dtype=odt) * 0.03
            ldo, flag = ((N + 7) // 8 * 8, 0x100) if a.pad_rows else (N, 0)
            o = torch.empty(M, ldo, device="cuda", dtype=odt)
            if a.epilogue == "none":
                b = None
            if a.epilogue != "bias_residual":
                r = None
            fn = lambda: ctx.call("linear", ocode, x, K, w, b, r, N if r is not None else 0, M, N, K, EPI[a.epilogue] | flag, o, ldo)
            if a.fuse_ln:
                gam, bet = torch.ones(N, device="cuda", dtype=odt), torch.zeros(N, device="cuda", dtype=odt)
                b, r = torch.randn(N, device="cuda", dtype=odt), torch.randn(M, N, device="cuda", dtype=odt)
                fn = lambda: ctx.call("linear_layernorm", ocode, x, K, w, b, r, N, gam, bet, 1e-12, M, N, K, o, N)
        if a.burst:
            def make():
                xx, oo = torch.randn_like(x) if a.dtype != "i8" else x.clone(), torch.empty_like(o)
                if a.dtype == "i8":
                    return lambda: ctx.call("linear_int8", ocode, xx, xs, w, ws, b, r, N, M, N, K, EPI[a.epilogue], oo, N)
                if a.fuse_ln:
                    return lambda: ctx.call("linear_layernorm", ocode, xx, K, w, b, r, N, gam, bet, 1e-12, M, N, K, oo, N)
                return lambda: ctx.call("linear", ocode, xx, K, w, b, r, N if r is not None else 0, M, N, K, EPI[a.epilogue] | flag, oo, ldo)
            fns = [make() for _ in range(a.burst)]
            mean, med, best = timed_graph(ctx, fns, a.warmup, a.iters) if a.graph else timed_burst(fns, a.warmup, a.iters)
        else:
            mean, med, best = timed(fn, a.warmup, a.iters, not a.no_flush)
        out.update(shape=[M, N, K], dtype=a.dtype, epilogue=a.epilogue, us=round(mean * 1e3, 2), us_median=round(med * 1e3, 2),
                   tflops=round(2.0 * M * N * K / mean / 1e9, 1))
    elif a.op == "matmul":  # the exact fp32 GEMM of the fp32 models: C = A [M,K] x B [K,N] (or B stored [N,K])
        M, N, K = a.m, a.n, a.k
        tdt, code = DT[a.dtype]
        x = torch.randn(M, K, device="cuda", dtype=tdt)
        w = torch.randn((N, K) if a.b_trans else (K, N), device="cuda", dtype=tdt) * 0.03
        o = torch.empty(M, N, device="cuda", dtype=tdt)
        fn = lambda: ctx.call("matmul", code, x, 0, w, int(a.b_trans), M, N, K, 1.0, 0.0, o)
        mean, med, best = timed(fn, a.warmup, a.iters, not a.no_flush)
        out.update(shape=[M, N, K], dtype=a.dtype, b_trans=a.b_trans, us=round(mean * 1e3, 2), us_median=round(med * 1e3, 2),
                   tflops=round(2.0 * M * N * K / mean / 1e9, 1))
        if a.yardstick:
            torch.backends.cuda.matmul.allow_tf32 = False
            wt = w.t() if a.b_trans else w
            ymean, _, _ = timed(lambda: torch.matmul(x, wt, out=o), a.warmup, a.iters, not a.no_flush)
            out.update(yardstick_us=round(ymean * 1e3, 2), yardstick_tflops=round(2.0 * M * N * K / ymean / 1e9, 1))
    elif a.op == "attention":
        lens = synthetic.varlen_lengths(64, 8, 512, 0) if a.lens == "varlen64" else [a.seq] * a.batch
        tdt, code = DT[a.dtype]
        H = a.heads * 64
        T = sum(lens)
        qkv = torch.randn(T, 3 * H, device="cuda", dtype=tdt)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
        o = torch.empty(T, H, device="cuda", dtype=tdt)
        mask, pitch = None, 0
        if a.key_mask:
            pitch = max(lens)
            if a.key_mask == "scattered":
                mask = torch.where(torch.rand(len(lens), pitch, device="cuda") < 0.25, -10000.0, 0.0).float()
                mask[:, 0] = 0
            else:  # padding: each sequence keeps a prefix of between half and all of its keys
                keep = torch.tensor([int(n * (0.5 + 0.5 * ((i * 37) % 100) / 100.0)) for i, n in enumerate(lens)], device="cuda").clamp_min(1)
                mask = torch.where(torch.arange(pitch, device="cuda")[None, :] < keep[:, None], 0.0, -10000.0).float()
        fn = lambda: ctx.call("attention_fwd", code, qkv, T, cu, len(lens), max(lens), a.heads, 64, mask, pitch, 0, int(a.causal), 0.125, o)
        if a.burst:
            def make():
                qq, oo = torch.randn_like(qkv), torch.empty_like(o)
                return lambda: ctx.call("attention_fwd", code, qq, T, cu, len(lens), max(lens), a.heads, 64, mask, pitch, 0, int(a.causal), 0.125, oo)
            fns = [make() for _ in range(a.burst)]
            mean, med, best = timed_graph(ctx, fns, a.warmup, a.iters) if a.graph else timed_burst(fns, a.warmup, a.iters)
        else:
            mean, med, best = timed(fn, a.warmup, a.iters, not a.no_flush)
        fl = sum((2.0 * H * L * (L + 1)) if a.causal else (4.0 * H * L * L) for L in lens)
        out.update(sequences=len(lens), tokens=T, heads=a.heads, dtype=a.dtype, causal=a.causal, us=round(mean * 1e3, 2),
                   us_median=round(med * 1e3, 2), tflops=round(fl / mean / 1e9, 1))
    elif a.op == "decode":
        tdt, code = DT[a.dtype]
        B, T, H = a.batch, a.seq, a.heads * 64
        qkv = torch.randn(B, 3 * H, device="cuda", dtype=tdt)
        pages = (T + 1 + 15) // 16
        kc = torch.randn(pages, B, 16, H, device="cuda", dtype=tdt)
        vc = torch.randn(pages, B, 16, H, device="cuda", dtype=tdt)
        o = torch.empty(B, H, device="cuda", dtype=tdt)
        fn = lambda: ctx.call("attention_decode", code, qkv, B, 1, a.heads, 64, kc, vc, T, 0.125, o)
        mean, med, best = timed(fn, a.warmup, a.iters, not a.no_flush)
        nbytes = 2.0 * (T + 1) * B * H * qkv.element_size()  # K and V read once
        out.update(batch=B, cached=T, heads=a.heads, dtype=a.dtype, us=round(mean * 1e3, 2), us_median=round(med * 1e3, 2),
                   gbs=round(nbytes / mean / 1e6, 1))
    else:
        tdt, code = DT[a.dtype]
        M, N = a.m, a.n
        x = torch.randn(M, N, device="cuda", dtype=tdt)
        r = torch.randn(M, N, device="cuda", dtype=tdt)
        g = torch.ones(N, device="cuda", dtype=tdt)
        z = torch.zeros(N, device="cuda", dtype=tdt)
        if a.op == "layernorm" and a.plain:
            fn = lambda: ctx.call("layernorm", code, x, x, g, z, M, N, 1e-12)
            nbytes = 2.0 * M * N * x.element_size()
        elif a.op == "layernorm":
            fn = lambda: ctx.call("add_bias_layernorm", code, x, r, z, g, z, M, N, 1e-12)
            nbytes = 3.0 * M * N * x.element_size()
        else:
            fn = lambda: ctx.call("add_bias_act", code, x, z, M, N, 0)
            nbytes = 2.0 * M * N * x.element_size()
        mean, med, best = timed(fn, a.warmup, a.iters, not a.no_flush)
        out.update(shape=[M, N], dtype=a.dtype, us=round(mean * 1e3, 2), us_median=round(med * 1e3, 2), gbs=round(nbytes / mean / 1e6, 1))
    assert ctx.device_status() == 0
    print(json.dumps(out))


if __name__ == "__main__":
    main()
