"""Engine throughput with and without constrained decoding (counterpart of the reference's
benchmark/python/benchmark_engine_guidance.py): N concurrent requests through `Engine.step()`, once free-running and once with
a JSON-schema grammar on every request; reports tokens/s, per-step latency and the share of the step the grammar masks cost.

    python benchmark/benchmark_engine_guidance.py -i <model_dir> -n 16 -l 128 -g 128
"""
import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SCHEMA = {"type": "object", "properties": {"name": {"type": "string"}, "tags": {"type": "array", "items": {"type": "string"}},
                                           "score": {"type": "number"}}, "required": ["name", "tags", "score"]}


def run(og, model, n, prompt_len, gen_len, guided, sync):
    engine = og.Engine(model)
    rng = np.random.RandomState(0)
    for i in range(n):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=prompt_len + gen_len, do_sample=True, top_k=40, temperature=0.8, random_seed=i + 1)
        if guided:
            p.set_guidance("json_schema", json.dumps(SCHEMA))
        r = og.Request(p)
        r.add_tokens(rng.randint(3, model.arch.vocab_size - 1, size=prompt_len).astype(np.int32))
        engine.add_request(r)
    sync()
    t0 = time.perf_counter()
    tokens, steps0 = 0, engine.step_count
    while engine.has_pending_requests():
        r = engine.step()
        while r is not None and r.has_unseen_tokens():
            r.get_unseen_token()
            tokens += 1
        if r is not None and r.is_turn_complete():
            engine.remove_request(r)
    sync()
    dt = time.perf_counter() - t0
    steps = engine.step_count - steps0
    return {"guided": guided, "tokens": tokens, "seconds": round(dt, 4), "tokens_per_s": round(tokens / dt, 1),
            "ms_per_step": round(dt / max(1, steps) * 1e3, 3), "steps": steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--input_folder", required=True)
    ap.add_argument("-n", "--num_requests", type=int, default=16)
    ap.add_argument("-l", "--prompt_length", type=int, default=128)
    ap.add_argument("-g", "--generation_length", type=int, default=128)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    import torch
    import onnxruntime_genai_b200 as og
    cfg = og.Config(a.input_folder)
    if a.cpu:
        cfg.clear_providers()
    model = og.Model(cfg)
    sync = (lambda: torch.cuda.synchronize()) if model.device_type == "cuda" else (lambda: None)
    run(og, model, min(2, a.num_requests), a.prompt_length, 8, False, sync)     # warm-up
    free = run(og, model, a.num_requests, a.prompt_length, a.generation_length, False, sync)
    guided = run(og, model, a.num_requests, a.prompt_length, a.generation_length, True, sync)
    print(json.dumps({"model": a.input_folder, "requests": a.num_requests, "free": free, "guided": guided,
                      "guidance_ms_per_step": round(guided["ms_per_step"] - free["ms_per_step"], 3)}))


if __name__ == "__main__":
    main()
