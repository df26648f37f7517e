"""Tensor-parallel self check: runs a prompt through the model on every rank of a torchrun job and
writes rank 0's next-token logits and greedy continuation to a .npz file.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 -m onnxruntime_genai_b200.parallel.tp_check \
        --model <dir> --out logits.npz [--backend nccl|fused] [--cpu]

Comparing that file with a single-process run of the same checkpoint validates the sharding math
(gloo on CPU) or the NCCL / fused NVLink reductions (CUDA).
"""
import argparse
import os

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--backend", default=None)
    ap.add_argument("--tokens", type=int, default=8)
    ap.add_argument("--engine", action="store_true", help="also run the continuous-batching engine (CUDA graphs on GPU)")
    ap.add_argument("--lora", nargs="*", default=[], help="adapter files: the first is active on the generator, the engine's requests "
                                                          "alternate between them and no adapter")
    a = ap.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(240, exit=True)   # a stuck rank reports where and ends instead of hanging the job
    import torch
    import onnxruntime_genai_b200 as og
    from onnxruntime_genai_b200.parallel.tp import TensorParallel
    tp = TensorParallel.from_env(a.backend)
    model = og.Model(a.model, tp=tp)
    rng = np.random.RandomState(5)
    prompt = rng.randint(0, model.arch.vocab_size, size=(2, 21)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=64, batch_size=2)
    g = og.Generator(model, p)
    adapters = None
    if a.lora:
        adapters = og.Adapters(model)
        for i, path in enumerate(a.lora):
            adapters.load(path, f"adapter{i}")
        g.set_active_adapter(adapters, "adapter0")
    g.append_tokens(prompt)
    logits = g.get_logits()[:, 0, :]
    for _ in range(a.tokens):
        g.generate_next_token()
    seqs = np.stack([g.get_sequence(i) for i in range(2)])
    eng_out = np.zeros((0,), dtype=np.int32)
    if a.engine:
        engine = og.Engine(model)
        reqs = []
        for i in range(3):
            gp = og.GeneratorParams(model)
            gp.set_search_options(max_length=40 + i, do_sample=True, top_k=20, temperature=0.8, random_seed=3 + i)
            r = og.Request(gp)
            r.add_tokens(rng.randint(0, model.arch.vocab_size, size=(9 + 5 * i,)).astype(np.int32))
            if adapters is not None and i % (len(a.lora) + 1) < len(a.lora):
                r.set_active_adapter(adapters, f"adapter{i % (len(a.lora) + 1)}")
            engine.add_request(r)
            reqs.append(r)
        outs = {id(r): [] for r in reqs}
        while engine.has_pending_requests():
            r = engine.step()
            if r is None:
                continue
            while r.has_unseen_tokens():
                outs[id(r)].append(r.get_unseen_token())
            if r.is_turn_complete():
                engine.remove_request(r)
        eng_out = np.concatenate([np.asarray(outs[id(r)], dtype=np.int32) for r in reqs])
    if model.device.type == "cuda":
        from onnxruntime_genai_b200 import ops
        ops.check_kernel_status()
    rank = tp.rank if tp is not None else 0
    if rank == 0:
        np.savez(a.out, logits=logits, seqs=seqs, engine=eng_out, backend=str(getattr(tp, "backend", "single")),
                 sp_steps=int(model.decoder.sp_steps))
    if tp is not None:
        from onnxruntime_genai_b200.parallel.tp import leave
        leave(0)


if __name__ == "__main__":
    main()
