"""The reference's own CUDA kernels against this framework's, on the same GPU.

    python baseline/build_ref_kernels.py          (once, on a machine with the reference tree and nvcc)
    python benchmark/benchmark_tail_kernels.py [--iters 200] [--json out.json]

The reference's runtime cannot be built offline, but its self-contained "tail" kernels can (baseline/build_ref_kernels.py
compiles src/cuda/cuda_topk.cu, beam_search_topk.cu and model_kernels.cu unmodified).  Compared here, at the shapes of the
named workloads, CUDA events around `--iters` back-to-back calls after warm-up (the reference's top-k dispatcher benchmarks
its eight algorithms on the first call of a shape and caches the fastest; that call is part of the warm-up):

  top-k              reference RunTopK (its autotuned pick)            vs  ops.topk (one radix-select kernel)
  sampling           reference RunTopK alone (its sampler runs on top of it: src/cuda/cuda_sampling.cu, not buildable
                     stand-alone - so this is a LOWER bound of the reference's sampling time)   vs  ops.sample (temperature +
                     top-k + top-p + draw in one kernel)
  beam top-k         reference BeamSearchTopK on log-probabilities     vs  ops.beam_candidates (log-softmax + running scores +
                     top 2 * beams + per-batch merge; does MORE work: the reference runs its softmax in a separate kernel)
  grammar mask       reference LaunchAddLogitsMask                     vs  ops.logits_bitmask

Both sides are called through ctypes from this process, so host launch cost is the same; inputs are rotated between calls so
that they come from HBM, not L2.  Results are checked against each other (top-k sets, masked positions).
"""
import argparse
import ctypes
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from onnxruntime_genai_b200 import ops

REF_SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "ref_kernels", "libref_kernels.so")


def load_ref():
    if not os.path.exists(REF_SO):
        return None
    lib = ctypes.CDLL(REF_SO)
    P, I = ctypes.c_void_p, ctypes.c_int
    lib.ref_topk_create.restype = P
    lib.ref_topk_create.argtypes = [I, I, P]
    lib.ref_topk_destroy.argtypes = [P]
    lib.ref_topk_run.restype = I
    lib.ref_topk_run.argtypes = [P, P, I, I, I, P, ctypes.POINTER(P), ctypes.POINTER(P), ctypes.POINTER(I)]
    lib.ref_beam_topk.restype = I
    lib.ref_beam_topk.argtypes = [P, I, I, I, I, P, P, P, P, P]
    lib.ref_add_logits_mask.restype = I
    lib.ref_add_logits_mask.argtypes = [P, I, I, P, P]
    return lib


def timed(fn, iters):
    for i in range(5):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=200)
    ap.add_argument("--json", default="")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    ref = load_ref()
    stream = lambda: torch.cuda.current_stream().cuda_stream
    out = {"reference_kernels": "built from the reference tree, unmodified" if ref else "libref_kernels.so not built (baseline/build_ref_kernels.py)"}
    L = 6      # input sets rotated between calls

    # ---- top-k and sampling
    for name, rows, vocab, k in (("llama_64x128256", 64, 128256, 50), ("gptoss_1x201088", 1, 201088, 50), ("gptoss_32x201088", 32, 201088, 50),
                                 ("phi3_1x32064", 1, 32064, 50)):
        xs = [torch.randn(rows, vocab, device=dev) * 3 for _ in range(L)]
        r = {"rows": rows, "vocab": vocab, "k": k}
        r["ours_topk_us"] = round(timed(lambda i: ops.topk(xs[i % L], k), a.iters), 2)
        kk = torch.full((rows,), k, dtype=torch.int32, device=dev)
        pp = torch.full((rows,), 0.9, device=dev)
        tt = torch.full((rows,), 0.7, device=dev)
        seeds = torch.arange(rows, dtype=torch.int64, device=dev)
        pos = torch.zeros(rows, dtype=torch.int32, device=dev)
        r["ours_sample_us"] = round(timed(lambda i: ops.sample(xs[i % L], kk, pp, tt, seeds, pos), a.iters), 2)
        if ref:
            h = ref.ref_topk_create(rows, vocab, stream())
            sc, ix, st = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_int()

            def run_ref(i):
                rc = ref.ref_topk_run(h, xs[i % L].data_ptr(), vocab, rows, k, stream(), ctypes.byref(sc), ctypes.byref(ix), ctypes.byref(st))
                assert rc == 0, "the reference top-k threw"
            r["reference_topk_us"] = round(timed(run_ref, a.iters), 2)
            # same sets?
            run_ref(0)
            torch.cuda.synchronize()
            stride = st.value
            try:
                from cuda import cudart
                idx_ref = torch.empty(rows * stride, dtype=torch.int32, device=dev)
                cudart.cudaMemcpy(idx_ref.data_ptr(), ix.value, rows * stride * 4, cudart.cudaMemcpyKind.cudaMemcpyDeviceToDevice)
                mine = ops.topk(xs[0], k)[1]
                r["same_topk_sets"] = bool(all(set(idx_ref.view(rows, stride)[b, :k].tolist()) == set(mine[b].tolist()) for b in range(min(rows, 4))))
            except Exception as e:      # the comparison needs cuda-python for a raw device copy
                r["same_topk_sets"] = f"not checked: {e}"
            r["topk_speedup_vs_reference"] = round(r["reference_topk_us"] / r["ours_topk_us"], 2)
            r["sample_vs_reference_topk_alone"] = round(r["reference_topk_us"] / r["ours_sample_us"], 2)
            ref.ref_topk_destroy(h)
        out["topk_" + name] = r
        del xs
        torch.cuda.empty_cache()

    # ---- beam-search top-k (BASELINE config 2: batch 8 x 4 beams, Phi-3 vocabulary)
    batch, beams, vocab = 8, 4, 32064
    k = 2 * beams
    xs = [torch.randn(batch * beams, vocab, device=dev) for _ in range(L)]
    lps = [torch.log_softmax(x, dim=-1) for x in xs]
    scores = torch.zeros(batch * beams, device=dev)
    r = {"batch": batch, "beams": beams, "vocab": vocab}
    r["ours_beam_candidates_us"] = round(timed(lambda i: ops.beam_candidates(xs[i % L], scores, batch, beams), a.iters), 2)
    if ref:
        tmp = torch.zeros(batch * beams * 129 * beams * 2 * 2 + 1024, device=dev)
        ov = torch.empty(batch * k, device=dev)
        ot = torch.empty(batch * k, dtype=torch.int32, device=dev)
        oi = torch.empty(batch * k, dtype=torch.int32, device=dev)

        def run_beam(i):
            rc = ref.ref_beam_topk(lps[i % L].data_ptr(), batch, beams, vocab, k, tmp.data_ptr(), ov.data_ptr(), ot.data_ptr(), oi.data_ptr(), stream())
            assert rc == 0
        r["reference_beam_topk_us"] = round(timed(run_beam, a.iters), 2)
        run_beam(0)
        mine = ops.beam_candidates(xs[0], scores, batch, beams)
        torch.cuda.synchronize()
        r["same_best_token"] = bool((ot.view(batch, k)[:, 0] == mine[1][:, 0]).all())
        r["speedup_vs_reference"] = round(r["reference_beam_topk_us"] / r["ours_beam_candidates_us"], 2)
    out["beam_topk"] = r

    # ---- grammar mask
    rows, vocab = 64, 128256
    words = (vocab - 1) // 32 + 1
    xs = [torch.randn(rows, vocab, device=dev) for _ in range(L)]
    mask = torch.randint(-2 ** 31, 2 ** 31 - 1, (rows, words), dtype=torch.int32, device=dev)
    r = {"rows": rows, "vocab": vocab}
    r["ours_bitmask_us"] = round(timed(lambda i: ops.logits_bitmask(xs[i % L], mask), a.iters), 2)
    if ref:
        r["reference_add_logits_mask_us"] = round(timed(lambda i: ref.ref_add_logits_mask(xs[i % L].data_ptr(), rows, vocab, mask.data_ptr(), stream()), a.iters), 2)
        r["speedup_vs_reference"] = round(r["reference_add_logits_mask_us"] / r["ours_bitmask_us"], 2)
    out["grammar_mask"] = r
    ops.check_kernel_status()
    print(json.dumps(out, indent=1))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(out, f, indent=1)


if __name__ == "__main__":
    main()
