"""Checks and times the tensor-parallel communication kernels on every rank of a torchrun job.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 benchmark/tp_fused_check.py
        [--tokens 64] [--prefill_tokens 2048] [--hidden 4096] [--inner 14336] [--iters 20] [--out file.json] [--check_only]

Correctness (all ranks, against NCCL on the same data): GEMM + all-reduce in one kernel in every available form
(flagged lines one-hop / two-hop, NVLS one-shot / two-shot) at a decode-sized and a prefill-sized token count,
GEMM -> reduce-scatter, all-gather -> GEMM, and the stand-alone all-reduce / all-gather / reduce-scatter kernels.
Timing: every candidate is captured in a CUDA graph of `--iters` launches and replayed (device time without host launch
cost, as in the engine's decode graph), CUDA events, max over ranks; next to `GEMM then ncclAllReduce` (NCCL with NVLS left on).
The roofline of GEMM + all-reduce is the slower of the weight stream at the measured HBM rate and the bytes each rank must
receive over NVLink at the measured 770 GB/s.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=64)
    ap.add_argument("--prefill_tokens", type=int, default=2048)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inner", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--check_only", action="store_true")
    a = ap.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(300, exit=True)   # a stuck rank reports where and ends instead of hanging the job
    from onnxruntime_genai_b200 import ops
    from onnxruntime_genai_b200.ops import _lib
    from onnxruntime_genai_b200.parallel.tp import TensorParallel, leave
    tp = TensorParallel.from_env("fused")
    rank, world, dev = tp.rank, tp.size, tp.device
    res = {"world": world, "backend": tp.backend}
    if tp.comm is None:
        res["error"] = "symmetric memory unavailable"
        if rank == 0:
            print(json.dumps(res))
        leave(1)
    comm = tp.comm
    res["nvls"] = bool(comm.nvls)
    L = _lib.lib()

    def set_form(form):
        """form: p2p1 / p2p2 (flagged lines, one / two hops), nvls1 / nvls2 (multicast, one / two shots)."""
        if form.startswith("nvls"):
            L.ogb_comm_set_options(1, 0 if form == "nvls2" else (1 << 60), -2)
        else:
            L.ogb_comm_set_options(0, -1, 1 if form == "p2p2" else 0)

    forms = (["p2p1"] if world < 4 else ["p2p2", "p2p1"]) + (["nvls1", "nvls2"] if comm.nvls and world > 2 else (["nvls1"] if comm.nvls else []))
    k_local = a.inner // world
    g = torch.Generator(device=dev).manual_seed(1234 + rank)

    def rnd(*shape, std):
        return (torch.randn(*shape, generator=g, device=dev) * std).to(torch.bfloat16)

    errs = {}
    # ---- GEMM + all-reduce (decode and prefill sizes), GEMM -> reduce-scatter
    for label, T in (("decode", a.tokens), ("prefill", a.prefill_tokens)):
        x, w = rnd(T, k_local, std=0.5), rnd(a.hidden, k_local, std=0.02)
        resid = rnd(T, a.hidden, std=0.5)
        want = ops.linear(x, w, out_fp32=True)
        dist.all_reduce(want)
        scale = float(want.abs().mean())
        want_r = want + resid.float()
        per = -(-T // world)
        for form in forms:
            if not form.startswith("nvls") and T > comm.plane_elems // a.hidden:
                continue
            if not form.startswith("nvls") and T > 256:
                continue
            set_form(form)
            for _ in range(3):     # both parities and a reuse
                got = ops.linear(x, w, residual=resid, all_reduce=True)
                errs[f"gemm_allreduce_{label}_{form}"] = float((got.float() - want_r).abs().max()) / scale
            rs = ops.linear(x, w, reduce_scatter=(rank, world))
            errs[f"gemm_reduce_scatter_{label}_{form}"] = (float((rs.float() - want[rank * per:rank * per + rs.shape[0]]).abs().max()) / scale
                                                          if rs.shape[0] else 0.0)
    # ---- stand-alone collectives
    for label, T in (("small", a.tokens), ("large", a.prefill_tokens)):
        y = rnd(T, a.hidden, std=0.5)
        ar_want = y.float()
        dist.all_reduce(ar_want)
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        stacked = torch.stack([y * (r + 1) for r in range(world)]).contiguous()
        rs_want = torch.empty_like(y, dtype=torch.float32)
        dist.reduce_scatter_tensor(rs_want, stacked.float())
        for form in forms:
            set_form(form)
            if not comm.fits(y):
                continue
            scale = float(ar_want.abs().mean())
            errs[f"allreduce_{label}_{form}"] = float((comm.all_reduce(y).float() - ar_want).abs().max()) / scale
            if form.startswith("nvls") and world * y.numel() > comm.nvls_plane_elems:
                continue
            errs[f"allgather_{label}_{form}"] = 0.0 if torch.equal(comm.all_gather(y), torch.stack(parts)) else 1.0
            if form.startswith("nvls") or stacked.numel() // world <= comm.plane_elems:
                errs[f"reducescatter_{label}_{form}"] = float((comm.reduce_scatter(stacked).float() - rs_want).abs().max()) / float(rs_want.abs().mean())
    # ---- all-gather -> GEMM (flagged lines): every rank pushes its token rows, then multiplies all rows
    set_form(forms[0])
    per = -(-a.tokens // world)
    gx = torch.Generator(device=dev).manual_seed(99)
    X = (torch.randn(a.tokens, a.hidden, generator=gx, device=dev) * 0.5).to(torch.bfloat16)
    wg = rnd(1024, a.hidden, std=0.02)
    comm.all_gather_push(X[rank * per:(rank + 1) * per].contiguous())
    yg = ops.linear_gathered(a.tokens, wg)
    errs["all_gather_gemm"] = 0.0 if torch.equal(yg, ops.linear(X, wg)) else 1.0
    comm.all_reduce(X[:8].contiguous())     # a waiting call before any further push
    ops.check_kernel_status()
    worst = torch.tensor([max(errs.values())], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    res["errors_relative_to_mean_abs"] = {k: round(v, 5) for k, v in errs.items()}
    res["worst_error_any_rank"] = float(worst)
    # largest |error| over millions of elements, relative to the MEAN magnitude: a few bf16 roundings of partials and sums
    res["ok"] = bool(float(worst) < 0.08)

    def timed(fn):
        """us per call of `fn`, replayed from a CUDA graph of --iters calls; max over ranks."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with ops.graph_capture(graph, stream=side):
                for _ in range(a.iters):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize(); dist.barrier()
        best = 1e30
        for _ in range(3):
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); graph.replay(); e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / a.iters * 1e3)
        t = torch.tensor([best], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t), 2)

    if not a.check_only:
        times = {}
        for label, T in (("decode", a.tokens), ("prefill", a.prefill_tokens)):
            for shape, (N, K) in (("down", (a.hidden, a.inner // world)), ("o", (a.hidden, a.hidden // world))):
                ws = [rnd(N, K, std=0.02) for _ in range(4)]      # rotate weights: they come from HBM, not L2
                x, resid = rnd(T, K, std=0.5), rnd(T, N, std=0.5)
                it = [0]

                def nxt():
                    it[0] += 1
                    return ws[it[0] % 4]
                key = f"{label}_{shape}"
                times[f"{key}_gemm_only_us"] = timed(lambda: ops.linear(x, nxt(), residual=resid))

                def base():
                    y = ops.linear(x, nxt())
                    dist.all_reduce(y)
                    return y
                times[f"{key}_gemm_then_nccl_us"] = timed(base)
                for form in forms:
                    if not form.startswith("nvls") and T > 256:
                        continue
                    set_form(form)
                    times[f"{key}_fused_{form}_us"] = timed(lambda: ops.linear(x, nxt(), residual=resid, all_reduce=True))
                # roofline: weight stream at the measured HBM rate vs bytes a rank must receive at 770 GB/s (two-shot: 2 * T * N * 2 / world * (world - 1))
                hbm_us = N * K * 2 / 6454e9 * 1e6
                link_us = 2 * T * N * 2 * (world - 1) / world / 770e9 * 1e6
                flop_us = 2.0 * T * N * K / 1417e12 * 1e6
                times[f"{key}_roofline_us"] = round(max(hbm_us, link_us, flop_us), 2)
        for label, T in (("small", a.tokens), ("large", a.prefill_tokens)):
            y = rnd(T, a.hidden, std=0.5)
            times[f"allreduce_{label}_nccl_us"] = timed(lambda: dist.all_reduce(y))
            for form in forms:
                set_form(form)
                if comm.fits(y) and (form.startswith("nvls") or y.numel() <= comm.plane_elems):
                    times[f"allreduce_{label}_{form}_us"] = timed(lambda: comm.all_reduce(y))
        res["times"] = times
        ops.check_kernel_status()
    if rank == 0:
        print(json.dumps(res))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f, indent=1)
    leave(0 if res["ok"] else 1)


if __name__ == "__main__":
    main()
