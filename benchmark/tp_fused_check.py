"""Checks the fused GEMM + all-reduce kernel against GEMM followed by `dist.all_reduce`, and the stand-alone
all-reduce / all-gather / reduce-scatter kernels against their NCCL counterparts, on every rank of a
torchrun job, and times both sides (device events, max over ranks).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 benchmark/tp_fused_check.py [--tokens 64]
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
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--inner", type=int, default=14336)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)   # a stuck rank reports where and ends instead of hanging the job
    from onnxruntime_genai_b200 import ops
    from onnxruntime_genai_b200.parallel.tp import TensorParallel
    tp = TensorParallel.from_env("fused")
    rank, world, dev = tp.rank, tp.size, tp.device
    res = {"world": world, "backend": tp.backend, "two_shot_env": os.environ.get("OGB_AR_TWO_SHOT", "auto")}
    if tp.comm is None:
        res["error"] = "symmetric memory unavailable"
    else:
        k_local = a.inner // world
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        x = (torch.randn(a.tokens, k_local, generator=g, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(a.hidden, k_local, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        resid = torch.zeros(a.tokens, a.hidden, dtype=torch.bfloat16, device=dev)
        want = ops.linear(x, w, out_fp32=True)
        dist.all_reduce(want)
        errs = []
        for _ in range(3):
            got = ops.linear(x, w, residual=resid, all_reduce=True)
            errs.append(float((got.float() - want).abs().max()))
        per = -(-a.tokens // world)
        rs = ops.linear(x, w, reduce_scatter=(rank, world))          # GEMM -> reduce-scatter by token rows, one kernel
        errs_rs = float((rs.float() - want[rank * per:rank * per + rs.shape[0]]).abs().max()) if rs.shape[0] else 0.0
        res["gemm_reduce_scatter_err"] = errs_rs
        # all-gather -> GEMM: every rank pushes its token rows of a common activation matrix, then multiplies all rows
        gx = torch.Generator(device=dev).manual_seed(99)
        X = (torch.randn(a.tokens, a.hidden, generator=gx, device=dev) * 0.5).to(torch.bfloat16)
        wg = (torch.randn(1024, a.hidden, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        comm0 = tp.comm
        comm0.all_gather_push(X[rank * per:(rank + 1) * per].contiguous())
        yg = ops.linear_gathered(a.tokens, wg)
        res["all_gather_gemm_exact"] = bool(torch.equal(yg, ops.linear(X, wg)))
        comm0.all_reduce(X[:8].contiguous())     # a waiting call before any further push
        ops.check_kernel_status()
        res["max_err"] = max(errs)
        res["ref_scale"] = float(want.abs().mean())

        def timed(fn):
            for _ in range(3):
                fn()
            dist.barrier(); torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                fn()
            e1.record(); torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / a.iters * 1e3], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t)

        def baseline():
            y = ops.linear(x, w)
            dist.all_reduce(y)
            return y

        # stand-alone collectives against NCCL
        comm = tp.comm
        y = ops.linear(x, w)
        ar_want = y.float()
        dist.all_reduce(ar_want)
        ar = comm.all_reduce(y)
        res["allreduce_err"] = float((ar.float() - ar_want).abs().max())
        parts = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(parts, y)
        ag = comm.all_gather(y)
        res["allgather_exact"] = bool(torch.equal(ag, torch.stack(parts)))
        stacked = torch.stack([y * (r + 1) for r in range(world)]).contiguous()
        rs_want = torch.empty_like(y, dtype=torch.float32)
        dist.reduce_scatter_tensor(rs_want, stacked.float())
        rs = comm.reduce_scatter(stacked)
        res["reducescatter_err"] = float((rs.float() - rs_want).abs().max())
        ops.check_kernel_status()
        res["allreduce_us"] = timed(lambda: comm.all_reduce(y))
        res["nccl_allreduce_us"] = timed(lambda: dist.all_reduce(y.clone()))
        res["allgather_us"] = timed(lambda: comm.all_gather(y))
        res["nccl_allgather_us"] = timed(lambda: dist.all_gather(parts, y))

        # all-gather -> GEMM (column-parallel projection over gathered token rows) against ncclAllGather + GEMM; every
        # iteration ends with a waiting call (a tiny all-reduce) as the protocol requires between two pushes
        xs_local = X[rank * per:(rank + 1) * per].contiguous()
        tiny = X[:8].contiguous()
        gathered = [torch.empty_like(xs_local) for _ in range(world)]

        def ag_fused():
            comm.all_gather_push(xs_local)
            y_ = ops.linear_gathered(a.tokens, wg)
            comm.all_reduce(tiny)
            return y_

        def ag_nccl():
            dist.all_gather(gathered, xs_local)
            y_ = ops.linear(torch.cat(gathered), wg)
            comm.all_reduce(tiny)
            return y_

        res["all_gather_gemm_fused_us"] = timed(ag_fused)
        res["all_gather_gemm_nccl_us"] = timed(ag_nccl)
        res["fused_us"] = timed(lambda: ops.linear(x, w, residual=resid, all_reduce=True))
        res["fused_reduce_scatter_us"] = timed(lambda: ops.linear(x, w, reduce_scatter=(rank, world)))
        res["gemm_plus_nccl_us"] = timed(baseline)
        res["gemm_only_us"] = timed(lambda: ops.linear(x, w))
        ops.check_kernel_status()
    if rank == 0:
        print(json.dumps(res))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f)
    from onnxruntime_genai_b200.parallel.tp import leave
    leave(0)


if __name__ == "__main__":
    main()
