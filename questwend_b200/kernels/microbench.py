"""Times one kernel of the library at a given size with CUDA events.

    python -m questwend_b200.kernels.microbench gemm --m 8 --n 24576 --k 4096 [--impl stream|small|library]
    python -m questwend_b200.kernels.microbench attn_decode --batch 8 --ctx 1152 [--heads 32 --kv-heads 8 --head-dim 128]
    python -m questwend_b200.kernels.microbench attn_prefill --tokens 2048
    python -m questwend_b200.kernels.microbench rmsnorm --m 8 --k 4096
    python -m questwend_b200.kernels.microbench sample --batch 8 --vocab 151936 --temp 0.8 --top-k 40 --top-p 0.95
    python -m questwend_b200.kernels.microbench decode_shapes --m 8        (every product of a Qwen3-8B decode step)

Inputs rotate through enough copies to exceed the 126 MB L2, so every timed launch reads from HBM.
Prints one JSON line per case: microseconds (median of the timed launches), the bytes the kernel has to
move, and GB/s.  Also the program to put under ncu for a capture of one kernel on a small case.
"""
from __future__ import annotations

import argparse
import json
import math
import statistics

import torch

from . import ops

L2_BYTES = 126 * 1024 * 1024


def _time(fn, n_variants: int, iters: int, warmup: int = 3, burst: int = 10) -> float:
    """Median microseconds per launch; each timed region holds `burst` launches back to back, so that
    the host's launch overhead does not hide a kernel of a few microseconds."""
    for i in range(warmup):
        fn(i % n_variants)
    torch.cuda.synchronize()
    burst = max(burst, n_variants)
    graph = torch.cuda.CUDAGraph()          # the burst is replayed from a graph: no host time between launches
    with torch.cuda.graph(graph):
        for k in range(burst):
            fn(k % n_variants)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / burst)
    return statistics.median(times)


def bench_gemm(M: int, N: int, K: int, impl: str, iters: int, dtype=torch.bfloat16, tile_n=None) -> dict:
    elem = 2 if dtype == torch.bfloat16 else 4
    copies = max(2, math.ceil(2 * L2_BYTES / (N * K * elem)))
    ws = [torch.randn(N, K, device="cuda", dtype=torch.float32).mul_(0.02).to(dtype) for _ in range(copies)]
    x = torch.randn(M, K, device="cuda").to(dtype)
    if impl == "stream":
        fn = lambda i: ops.gemm_stream(x, ws[i])
    elif impl == "ring":
        fn = lambda i: ops.gemm_ring(x, ws[i])
    elif impl == "ring_swiglu":
        fn = lambda i: ops.gemm_ring_swiglu(x, ws[i])
    elif impl == "ring_add":                # added onto a 32-bit matrix (the residual stream) in the epilogue
        acc = torch.zeros(M, N, device="cuda")
        fn = lambda i: ops.gemm_ring(x, ws[i], residual=acc)
    elif impl == "ring_split":              # equal shares per block, the pieces left as planes (where whole tiles are as
        plan = ops.ring_split_plan(N, K, x.device)          # good there is no split form: the plain one is timed)
        fn = (lambda i: ops.gemm_ring_split(x, ws[i], plan)) if plan else (lambda i: ops.gemm_ring(x, ws[i]))
    elif impl == "stream_swiglu":
        fn = lambda i: ops.gemm_stream_swiglu(x, ws[i])
    elif impl == "small":
        fn = lambda i: ops.gemm_small(x, ws[i])
    elif impl == "tc":
        fn = lambda i: ops.gemm_tc(x, ws[i], tile_n=tile_n)
    elif impl == "tc_add":
        acc = torch.zeros(M, N, device="cuda")
        fn = lambda i: ops.gemm_tc(x, ws[i], epilogue="add", out=acc, tile_n=tile_n)
    elif impl == "tc_swiglu":
        fn = lambda i: ops.gemm_tc(x, ws[i], epilogue="swiglu", tile_n=tile_n)
    elif impl == "library_add":
        acc = torch.zeros(M, N, device="cuda")
        fn = lambda i: torch.addmm(acc, x, ws[i].t(), out_dtype=torch.float32, out=acc)
    elif impl == "library_swiglu":
        fn = lambda i: ops.silu_mul(torch.mm(x, ws[i].t(), out_dtype=torch.float32), torch.bfloat16, ops.GATE_UP_GROUP)
    else:
        fn = (lambda i: torch.mm(x, ws[i].t(), out_dtype=torch.float32)) if dtype == torch.bfloat16 else \
             (lambda i: torch.mm(x, ws[i].t()))
    us = _time(fn, copies, iters)
    nbytes = N * K * elem + M * K * elem + M * N * 4
    return {"kernel": f"gemm_{impl}", "M": M, "N": N, "K": K, "us": us, "bytes": nbytes,
            "GBps": nbytes / us / 1e3, "TFLOPs": 2.0 * M * N * K / us / 1e6}


def bench_attn_decode(B, ctx, Hq, Hkv, hd, iters, dtype=torch.bfloat16, split=0, runs_target=0, run_pages_max=0, max_len=0,
                      fused=False) -> dict:
    page = ops.PAGE_SIZE
    pages_per = math.ceil(ctx / page)
    per_copy = B * pages_per
    elem = 2 if dtype == torch.bfloat16 else 4
    copy_bytes = 2 * per_copy * Hkv * page * hd * elem
    copies = max(2, math.ceil(2 * L2_BYTES / copy_bytes))
    n_pages = per_copy * copies
    k_pool = torch.randn(n_pages, Hkv, page, hd, device="cuda").to(dtype)
    v_pool = torch.randn(n_pages, Hkv, page, hd, device="cuda").to(dtype)
    tables = [(torch.arange(per_copy, dtype=torch.int32, device="cuda") + c * per_copy).reshape(B, pages_per).contiguous()
              for c in range(copies)]
    q = torch.randn(B, Hq, hd, device="cuda").to(dtype)
    seq_len = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    if split:       # runs of exactly this many keys instead of the kernels' own choice
        how = dict(split_tokens=split, runs_target=1, run_pages_max=max(1, split // page))
    else:
        how = {}
        if runs_target:
            how["runs_target"] = runs_target
        if run_pages_max:
            how["run_pages_max"] = run_pages_max
    max_len = max_len or ctx            # the bound a graph is captured for may be larger than the sequences
    fn = lambda i: ops.attn_decode(q, k_pool, v_pool, tables[i], seq_len, 1 / math.sqrt(hd), max_len, **how)
    if fused:       # the kernel that also norms and rotates q and k and writes the new key and value (what a step of few sequences runs)
        how.pop("split_tokens", None)
        qkv = torch.randn(B, (Hq + 2 * Hkv) * hd, device="cuda")
        w = torch.ones(hd, device="cuda")
        inv = torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
        cos, sin = ops.rope_table(seq_len - 1, inv)
        fn = lambda i: ops.attn_decode_fused(qkv, w, w, cos, sin, 1e-6, k_pool, v_pool, tables[i], seq_len, 1 / math.sqrt(hd), max_len,
                                             Hq, Hkv, hd, **how)
    us = _time(fn, copies, iters)
    nbytes = 2 * B * ctx * Hkv * hd * elem
    return {"kernel": "attn_decode_fused" if fused else "attn_decode", "B": B, "ctx": ctx, "Hq": Hq, "Hkv": Hkv, "hd": hd, "us": us, "bytes": nbytes,
            "GBps": nbytes / us / 1e3}


def bench_attn_prefill(T, Hq, Hkv, hd, iters, dtype=torch.bfloat16) -> dict:
    page = ops.PAGE_SIZE
    n_pages = math.ceil(T / page)
    k_pool = torch.randn(n_pages, Hkv, page, hd, device="cuda").to(dtype)
    v_pool = torch.randn(n_pages, Hkv, page, hd, device="cuda").to(dtype)
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").reshape(1, n_pages)
    q = torch.randn(T, Hq, hd, device="cuda").to(dtype)
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    pos0 = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lambda i: ops.attn_prefill(q, k_pool, v_pool, table, cu, pos0, T, 1 / math.sqrt(hd))
    us = _time(fn, 1, iters)
    flops = 4.0 * Hq * hd * T * (T + 1) / 2
    return {"kernel": "attn_prefill", "T": T, "Hq": Hq, "Hkv": Hkv, "hd": hd, "us": us, "TFLOPs": flops / us / 1e6}


def bench_rmsnorm(M, K, iters) -> dict:
    copies = max(2, math.ceil(2 * L2_BYTES / (M * K * 4)))
    copies = min(copies, 64)
    xs = [torch.randn(M, K, device="cuda") for _ in range(copies)]
    d = torch.randn(M, K, device="cuda")
    w = torch.ones(K, device="cuda")
    fn = lambda i: ops.rmsnorm(xs[i], w, 1e-6, torch.bfloat16, delta=d, write_sum=True)
    us = _time(fn, copies, iters)
    return {"kernel": "rmsnorm", "M": M, "K": K, "us": us}


def bench_rope(T, Hq, Hkv, hd, iters, store_kv=True) -> dict:
    """q/k norm + rotation + cache write of one prompt of T tokens (``rope``)."""
    page = ops.PAGE_SIZE
    n_pages = math.ceil(T / page)
    copies = max(2, min(8, math.ceil(2 * L2_BYTES / (T * (Hq + 2 * Hkv) * hd * 4))))
    qkvs = [torch.randn(T, (Hq + 2 * Hkv) * hd, device="cuda") for _ in range(copies)]
    k_pool = torch.zeros(n_pages * copies, Hkv, page, hd, device="cuda", dtype=torch.bfloat16)
    v_pool = torch.zeros_like(k_pool)
    tables = [(torch.arange(n_pages, dtype=torch.int32, device="cuda") + c * n_pages).reshape(1, n_pages) for c in range(copies)]
    w = torch.ones(hd, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    seq = torch.zeros(T, dtype=torch.int32, device="cuda")
    inv_freq = torch.tensor([1e6 ** (-2.0 * i / hd) for i in range(hd // 2)], dtype=torch.float64, device="cuda")
    cos, sin = ops.rope_table(pos, inv_freq)
    fn = lambda i: ops.qk_norm_rope_store(qkvs[i], w, w, cos, sin, seq, pos, tables[i], k_pool, v_pool, Hq, Hkv, hd, hd, 1e-6,
                                          store_kv=store_kv)
    us = _time(fn, copies, iters)
    nbytes = T * (Hq + 2 * Hkv) * hd * 4 + T * (Hq + 2 * Hkv) * hd * 2
    return {"kernel": "qk_norm_rope_store", "T": T, "Hq": Hq, "Hkv": Hkv, "hd": hd, "us": us, "bytes": nbytes, "GBps": nbytes / us / 1e3}


def bench_sample(B, V, temperature, top_k, top_p, iters, spread=3.0) -> dict:
    copies = max(2, math.ceil(2 * L2_BYTES / (B * V * 4)))
    copies = min(copies, 64)
    rows = [torch.randn(B, V, device="cuda") * spread for _ in range(copies)]
    seq = torch.arange(B, dtype=torch.int32, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    fn = lambda i: ops.sample(rows[i], temperature, top_k=top_k, top_p=top_p, seed=1, sequence_index=seq, step=i, out=out)
    us = _time(fn, copies, iters)
    return {"kernel": "sample", "B": B, "V": V, "temperature": temperature, "top_k": top_k, "top_p": top_p, "us": us,
            "bytes": B * V * 4, "GBps": B * V * 4 / us / 1e3}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attn_decode", "attn_prefill", "rmsnorm", "rope", "decode_shapes", "sample"])
    ap.add_argument("--m", type=int, default=8)
    ap.add_argument("--n", type=int, default=24576)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--impl", default="stream", choices=["stream", "stream_swiglu", "ring", "ring_swiglu", "ring_add", "ring_split", "small", "library", "tc", "tc_add", "tc_swiglu", "library_add", "library_swiglu"])
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1152)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--temp", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tile-n", type=int, default=None)
    ap.add_argument("--max-len", type=int, default=0, help="decode attention: the bound on the lengths (default: the context)")
    ap.add_argument("--split", type=int, default=0, help="keys per run of the decode attention kernel (0: its own choice)")
    ap.add_argument("--runs-target", type=int, default=0, help="tensor-core decode attention: about this many runs a sequence")
    ap.add_argument("--run-pages-max", type=int, default=0, help="tensor-core decode attention: at most this many pages a run")
    ap.add_argument("--fused", action="store_true", help="decode attention with the q/k norm, rotation and cache write inside")
    args = ap.parse_args()
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    if args.what == "gemm":
        print(json.dumps(bench_gemm(args.m, args.n, args.k, args.impl, args.iters, dtype, args.tile_n)))
    elif args.what == "decode_shapes":
        for name, n, k in (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288),
                           ("lm_head", 151936, 4096)):
            r = bench_gemm(args.m, n, k, args.impl, args.iters, dtype, args.tile_n)
            r["name"] = name
            print(json.dumps(r))
    elif args.what == "attn_decode":
        print(json.dumps(bench_attn_decode(args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim, args.iters, dtype, args.split,
                                           args.runs_target, args.run_pages_max, fused=args.fused, max_len=args.max_len)))
    elif args.what == "sample":
        print(json.dumps(bench_sample(args.batch, args.vocab, args.temp, args.top_k, args.top_p, args.iters)))
    elif args.what == "attn_prefill":
        print(json.dumps(bench_attn_prefill(args.tokens, args.heads, args.kv_heads, args.head_dim, args.iters, dtype)))
    elif args.what == "rope":
        print(json.dumps(bench_rope(args.tokens, args.heads, args.kv_heads, args.head_dim, args.iters)))
    else:
        print(json.dumps(bench_rmsnorm(args.m, args.k, args.iters)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
