"""Checks the fused GEMM + all-reduce kernel against GEMM followed by `dist.all_reduce` on every rank
of a torchrun job, and times both (device events, max over ranks).

    torchrun --nproc-per-node N --master-addr 127.0.0.1 -m onnxruntime_genai_b200.parallel.fused_check [--tokens 64]
"""
import argparse
import json
import os

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
    from onnxruntime_genai_b200 import ops
    from onnxruntime_genai_b200.parallel.tp import TensorParallel
    tp = TensorParallel.from_env("fused")
    rank, world, dev = tp.rank, tp.size, tp.device
    res = {"world": world, "backend": tp.backend}
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

        res["fused_us"] = timed(lambda: ops.linear(x, w, residual=resid, all_reduce=True))
        res["gemm_plus_nccl_us"] = timed(baseline)
        res["gemm_only_us"] = timed(lambda: ops.linear(x, w))
        ops.check_kernel_status()
    if rank == 0:
        print(json.dumps(res))
        if a.out:
            with open(a.out, "w") as f:
                json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
