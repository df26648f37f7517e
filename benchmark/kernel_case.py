"""Single-kernel workloads for timing and profiling.

    python benchmark/kernel_case.py <case> [--tokens 64] [--iters 16] [--layers 8] [--tp 1] [--eager] [--json out.json]

cases: gemm_qkv gemm_o gemm_gate_up gemm_down gemm_lm_head gemm_prefill gemm_qkv_fused gemm_gate_up_fused w4_qkv w4_down attention_decode
       attention_prefill norm rope sample argmax all; moe_fp4_gate_up moe_fp4_down moe_fp4b_gate_up moe_fp4b_down moe_bf16_gate_up moe_bf16_down
       (gpt-oss-20b experts, packed MXFP4 in the fp16 form, in the bf16 form (fp4b) or bf16 weights; not part of `all`)

Each case runs the kernel at the Llama-3.1-8B (or, for w4_*, Phi-3-mini) shapes with `--layers` distinct
weight sets rotated between launches (so weights come from HBM, not L2), captures `--iters` launches
in a CUDA graph and times graph replays with CUDA events.  It prints microseconds per launch and
the achieved fraction of the algorithmic bytes or FLOPs over the measured peaks in
MEASURED_PEAKS.json (when that file is next to the repository root).  With few `--layers` and
`--iters` the same command is the small case used under `ncu`.
"""
import argparse
import json
import math
import os
import sys

import numpy as np
import torch

import os as _os, sys as _sys
_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
from onnxruntime_genai_b200 import ops

H, I, V, HQ, HKV, D = 4096, 14336, 128256, 32, 8, 128


def _bf(*shape, std=0.02):
    return (torch.randn(*shape, device="cuda") * std).to(torch.bfloat16)


def _time_eager(fn, iters):
    """Plain launches (no graph): the form to run under a profiler."""
    fn(0); fn(1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def _time_graph(fn, iters, reps=3):
    fn(0); fn(1)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(iters):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with ops.graph_capture(g):
        for i in range(iters):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); g.replay(); e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters * 1e3)
    return best


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


NO_FUSED = False     # --tp shapes without the fused all-reduce (the GEMM alone)
ATTN_SPLITS = None   # None: the library's choice; (splits, kv_chunk) to force one
KV_BITS = 16         # --kv_bits 8: the attention cases read an int8 cache
GEMM_SPLITS = 0      # --gemm_splits: force the split-K cluster size of the GEMM cases (0: the library's choice)
ATTN_ORDER = False   # --attn_order: longest request first


def build_case(name, T, L, tp=1):
    """Returns (fn(i), algorithmic_bytes, flops).  tp > 1: the per-rank shapes of tensor parallelism; the row-parallel
    projections then run the fused all-reduce against a world of one (protocol cost without a peer)."""
    HQ, HKV = globals()["HQ"] // tp, max(1, globals()["HKV"] // tp)
    if name in ("gemm_qkv_fused", "gemm_gate_up_fused"):
        # the decode-step fusions: RMS norm folded into the projection (+ rotary embedding and KV-cache append for QKV)
        x = _bf(T, H, std=1.0)
        if name == "gemm_gate_up_fused":
            N = 2 * I // tp
            ws = [ops.interleave_gate_up(_bf(N, H)) for _ in range(L)]
            return (lambda i: ops.gate_up_act(x, ws[i % L], interleaved=True, norm_eps=1e-5)), N * H * 2 + T * (H + N // 2) * 2, 2.0 * T * N * H
        N = (HQ + 2 * HKV) * D
        ws = [_bf(N, H) for _ in range(L)]
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        slots = torch.arange(T, dtype=torch.int32, device="cuda")
        cos, sin = torch.randn(4096, D // 2, device="cuda"), torch.randn(4096, D // 2, device="cuda")
        kc, vc = _bf(T + 16, HKV, D), _bf(T + 16, HKV, D)
        return (lambda i: ops.qkv_rope_append(x, ws[i % L], None, pos, slots, cos, sin, kc, vc, HQ, HKV, D, D, norm_eps=1e-5)), \
            N * H * 2 + T * (H + N) * 2, 2.0 * T * N * H
    if name.startswith("gemm_") or name.startswith("w4_"):
        shapes = {"gemm_qkv": ((HQ + 2 * HKV) * D, H), "gemm_o": (H, HQ * D), "gemm_gate_up": (2 * I // tp, H), "gemm_down": (H, I // tp),
                  "gemm_lm_head": (V // tp, H), "gemm_prefill": (2 * I // tp, H), "w4_qkv": (9216 // tp, 3072), "w4_down": (3072, 8192 // tp)}
        N, K = shapes[name]
        fused = tp > 1 and name in ("gemm_o", "gemm_down") and not NO_FUSED
        if name == "gemm_lm_head":
            L = min(L, 2)
        x = _bf(T, K, std=1.0)
        if name.startswith("w4_"):
            from onnxruntime_genai_b200.models.builder import quantize_int4_block32
            from onnxruntime_genai_b200.ops.w4 import W4Weight, unpack_ort_q4
            ws = []
            for _ in range(L):
                qw, s, zp = quantize_int4_block32(torch.randn(N, K, device="cuda") * 0.02)   # quantised and repacked on the device
                q, z = unpack_ort_q4(qw, zp, N, K)
                ws.append(W4Weight.from_quantized(q, s, z, "cuda", keep_host=False))
            nbytes = ws[0].packed.numel()
            return (lambda i: ops.linear(x, ws[i % L])), nbytes + T * (K + N) * 2, 2.0 * T * N * K
        ws = [_bf(N, K) for _ in range(L)]
        if name in ("gemm_gate_up", "gemm_prefill"):
            ws = [ops.interleave_gate_up(w) for w in ws]
            return (lambda i: ops.gate_up_act(x, ws[i % L], interleaved=True, splits=GEMM_SPLITS)), N * K * 2 + T * (K + N // 2) * 2, 2.0 * T * N * K
        fp32 = name == "gemm_lm_head"
        return (lambda i: ops.linear(x, ws[i % L], out_fp32=fp32, all_reduce=fused, splits=GEMM_SPLITS)), N * K * 2 + T * K * 2 + T * N * (4 if fp32 else 2), 2.0 * T * N * K
    if name.startswith("moe_"):
        # gpt-oss-20b experts: 32 experts, 4 per token, hidden 2880, intermediate 2880; tokens routed uniformly at random.
        # moe_fp4_*: MXFP4 experts kept packed (csrc/gemm_fp4.cu); moe_bf16_*: the same shapes with bf16 experts.
        E, k, Hm, Im = 32, 4, 2880, 2880
        gate_up = name.endswith("gate_up")
        N, K = (2 * Im, Hm) if gate_up else (Hm, Im)
        L = min(L, 2 if "bf16" in name else 4)
        logits = torch.randn(T, E, device="cuda")
        plan = ops.moe_route(logits, k, 0, (0, E))
        xs = _bf(T * k, K, std=1.0)
        touched = int(torch.unique(plan.topk_idx).numel())
        if "fp4" in name:
            from onnxruntime_genai_b200.ops.fp4 import Fp4Experts
            half = "fp4b" not in name       # moe_fp4b_*: the bf16 form of the packed experts
            xs = xs.to(torch.float16) if half else xs
            ws = [Fp4Experts.from_codes(torch.randint(0, 16, (E, N, K), device="cuda", dtype=torch.uint8),
                                        torch.randint(119, 123, (E, N, K // 32), device="cuda", dtype=torch.uint8), "cuda", keep_host=False,
                                        half=half)
                  for _ in range(L)]
            wbytes = touched * N * K * 17 // 32
        else:
            ws = [_bf(E, N, K) for _ in range(L)]
            wbytes = touched * N * K * 2
        bias = _bf(E, N, std=0.1)
        if gate_up:
            return (lambda i: ops.moe_gemm(xs, ws[i % L], plan, bias, act_kind=2, alpha=1.702, limit=7.0)), wbytes + T * k * (K + N // 2) * 2, 2.0 * T * k * N * K
        return (lambda i: ops.moe_gemm(xs, ws[i % L], plan, bias)), wbytes + T * k * (K + N) * 2, 2.0 * T * k * N * K
    if name in ("attention_decode", "attention_prefill"):
        bs = 16
        rng = np.random.RandomState(2)
        decode = name == "attention_decode"
        B = T if decode else max(1, T // 1024)
        q_lens = [1] * B if decode else [T // B] * B
        past = (rng.randint(128, 2049, size=B) + 64).tolist() if decode else [0] * B
        cols = max((p + q + bs - 1) // bs for p, q in zip(past, q_lens))
        nblk = sum((p + q + bs - 1) // bs for p, q in zip(past, q_lens)) + 4
        Lk = min(L, 4)
        if KV_BITS == 8:
            def q8():   # int8 rows with an inline fp32 scale (row pitch D + 16 bytes)
                c = torch.randint(-127, 128, (nblk * bs, HKV, D + 16), dtype=torch.int8, device="cuda")
                c[:, :, D:D + 4] = torch.full((nblk * bs, HKV, 1), 1.0 / 64, device="cuda").view(torch.int8).view(nblk * bs, HKV, 4)
                return c
            kc, vc = [q8() for _ in range(Lk)], [q8() for _ in range(Lk)]
        else:
            kc = [_bf(nblk * bs, HKV, D, std=1.0) for _ in range(Lk)]
            vc = [_bf(nblk * bs, HKV, D, std=1.0) for _ in range(Lk)]
        table = torch.zeros(B, cols, dtype=torch.int32)
        used = 0
        for b in range(B):
            n = (past[b] + q_lens[b] + bs - 1) // bs
            table[b, :n] = torch.arange(used, used + n, dtype=torch.int32)
            used += n
        table = table.cuda()
        Tq = sum(q_lens)
        qkv = _bf(Tq, (HQ + 2 * HKV) * D, std=1.0)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32).cuda()
        pl = torch.tensor(past, dtype=torch.int32).cuda()
        kv_tokens = sum(p + q for p, q in zip(past, q_lens))
        nbytes = kv_tokens * HKV * ((D + 16) if KV_BITS == 8 else D * 2) * 2 + Tq * HQ * D * 2 * 2
        flops = sum(4.0 * HQ * D * (q * p + q * (q + 1) / 2) for p, q in zip(past, q_lens))
        order = torch.argsort(-pl.long(), stable=True).to(torch.int32) if ATTN_ORDER else None   # longest request first
        return (lambda i: ops.paged_attention(qkv, kc[i % Lk], vc[i % Lk], cu, pl, table, bs, HQ, HKV, D, 1 / math.sqrt(D),
                                              max_q_len=max(q_lens), max_kv_len=max(p + q for p, q in zip(past, q_lens)),
                                              splits=ATTN_SPLITS, order=order)), nbytes, flops
    if name == "norm":
        x, r, w = _bf(T, H, std=1.0), _bf(T, H, std=1.0), _bf(H, std=1.0)
        return (lambda i: ops.norm(x, w, 1e-5, r)), T * H * 2 * 4, 0.0
    if name == "rope":
        qkv = _bf(T, (HQ + 2 * HKV) * D, std=1.0)
        pos = torch.arange(T, dtype=torch.int32, device="cuda")
        slots = torch.arange(T, dtype=torch.int32, device="cuda")
        cos, sin = torch.randn(4096, D // 2, device="cuda"), torch.randn(4096, D // 2, device="cuda")
        kc, vc = _bf(T + 16, HKV, D), _bf(T + 16, HKV, D)
        return (lambda i: ops.rope_kv_append(qkv, pos, slots, cos, sin, kc, vc, HQ, HKV, D, D)), T * (HQ + 2 * HKV) * D * 2 * 2, 0.0
    if name == "gated_delta":
        # one decode step of a gated-delta-net layer for T requests (Qwen3.5 shapes: 16 key heads, 32 value heads, head sizes 128): every
        # request's fp32 state [32, 128, 128] (2 MiB) is read and written once
        Hk, Hv, dk, dv = 16, 32, 128, 128
        q, k, v = _bf(T, Hk, dk, std=0.1), _bf(T, Hk, dk, std=0.1), _bf(T, Hv, dv, std=1.0)
        g = -torch.rand(T, Hv, device="cuda") * 0.2
        beta = torch.rand(T, Hv, device="cuda")
        pools = [torch.randn(T, Hv, dk, dv, device="cuda") * 0.1 for _ in range(max(2, min(L, 4)))]
        slots = torch.arange(T, dtype=torch.int32, device="cuda")
        cu = torch.arange(T + 1, dtype=torch.int32, device="cuda")
        past = torch.full((T,), 7, dtype=torch.int32, device="cuda")
        return (lambda i: ops.gated_delta(q, k, v, g, beta, pools[i % len(pools)], slots, cu, past)), \
            T * Hv * dk * dv * 4 * 2 + T * (2 * Hk * dk + 2 * Hv * dv) * 2, 6.0 * T * Hv * dk * dv
    if name == "mamba2_scan":
        # one decode step of a Mamba-2 layer for T requests (heads 128, head size 64, state size 128, one B / C group): every request's
        # fp32 state [heads, N, P] is read and written once; L state pools are rotated so that the states come from HBM
        heads, P, N, groups = 128, 64, 128, 1
        x = _bf(T, heads, P, std=1.0)
        dt = torch.rand(T, heads, device="cuda") * 0.5 + 0.01
        neg_a = -(torch.rand(heads, device="cuda") + 0.1)
        Bm, Cm = _bf(T, groups, N, std=0.5), _bf(T, groups, N, std=0.5)
        Dv = torch.randn(heads, device="cuda")
        pools = [torch.randn(T, heads, N, P, device="cuda") * 0.1 for _ in range(max(2, min(L, 4)))]
        slots = torch.arange(T, dtype=torch.int32, device="cuda")
        cu = torch.arange(T + 1, dtype=torch.int32, device="cuda")
        past = torch.full((T,), 7, dtype=torch.int32, device="cuda")
        return (lambda i: ops.mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, pools[i % len(pools)], slots, cu, past)), \
            T * heads * N * P * 4 * 2 + T * heads * P * 2 * 2, 4.0 * T * heads * N * P
    if name in ("sample", "argmax"):
        logits = torch.randn(T, V, device="cuda") * 3
        k = torch.full((T,), 50, dtype=torch.int32, device="cuda")
        p = torch.full((T,), 0.9, device="cuda")
        t = torch.full((T,), 0.7, device="cuda")
        seeds = torch.arange(T, dtype=torch.int64, device="cuda")
        pos = torch.zeros(T, dtype=torch.int32, device="cuda")
        if name == "argmax":
            return (lambda i: ops.argmax(logits)), T * V * 4, 0.0
        return (lambda i: ops.sample(logits, k, p, t, seeds, pos)), T * V * 4, 0.0
    raise SystemExit(f"unknown case {name}")


ALL = ["gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "gemm_lm_head", "w4_qkv", "w4_down", "attention_decode", "norm", "rope",
       "sample", "argmax"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--iters", type=int, default=16)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--json", default="")
    ap.add_argument("--eager", action="store_true", help="plain launches instead of a CUDA graph (for profilers; includes launch gaps)")
    ap.add_argument("--no_fused", action="store_true", help="with --tp: run the row-parallel GEMMs without the fused all-reduce")
    ap.add_argument("--attn_splits", default="", help="force the attention split: 'S' (even division) or 'S,chunk' (fixed key ranges)")
    ap.add_argument("--kv_bits", type=int, default=16, choices=[16, 8], help="attention cases: bf16 or int8 key/value cache")
    ap.add_argument("--gemm_splits", type=int, default=0, help="force the split-K cluster size of the GEMM cases (1, 2, 4, 8)")
    ap.add_argument("--attn_order", action="store_true", help="issue the attention CTAs of the longest requests first")
    ap.add_argument("--tp", type=int, default=1, help="use the per-rank shapes of this tensor-parallel degree")
    a = ap.parse_args()
    torch.manual_seed(0)
    globals()["NO_FUSED"] = a.no_fused
    globals()["ATTN_ORDER"] = a.attn_order
    globals()["GEMM_SPLITS"] = a.gemm_splits
    globals()["KV_BITS"] = a.kv_bits
    if a.attn_splits:
        v = [int(x) for x in a.attn_splits.split(",")]
        globals()["ATTN_SPLITS"] = v[0] if len(v) == 1 else (v[0], v[1])
    comm = None
    if a.tp > 1:
        from onnxruntime_genai_b200.parallel.symm import LocalComm
        comm = LocalComm(torch.device("cuda", 0))
    hbm, tflops, src = _peaks()
    out = {}
    for name in (ALL if a.case == "all" else [a.case]):
        T = a.tokens if name != "gemm_prefill" and name != "attention_prefill" else max(a.tokens, 2048)
        fn, nbytes, flops = build_case(name, T, a.layers, a.tp)
        iters = a.iters if name not in ("gemm_lm_head", "sample", "argmax") else min(a.iters, 4)
        us = _time_eager(fn, iters) if a.eager else _time_graph(fn, iters)
        gbs, tf = nbytes / us / 1e3, flops / us / 1e6
        out[name] = {"tokens": T, "us": round(us, 2), "GBps": round(gbs, 1), "TFLOPs": round(tf, 1),
                     "frac_hbm": round(gbs / hbm, 3), "frac_bf16": round(tf / tflops, 3), "peaks": src}
        print(f"{name:18s} T={T:5d} {us:9.2f} us  {gbs:8.1f} GB/s ({gbs / hbm:5.2f} of {src} HBM)  {tf:8.1f} TFLOP/s ({tf / tflops:5.2f} of {src} bf16)",
              flush=True)
        del fn
        torch.cuda.empty_cache()
    ops.check_kernel_status()
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
