"""End-to-end generation benchmark through the public Generator API (counterpart of the reference's
benchmark/python/benchmark_e2e.py): prompt processing latency (time to first token), per-token generation
latency, tokens/s and wall clock for a grid of batch sizes, prompt lengths and generation lengths.

    python benchmark/benchmark_e2e.py -i <model_dir> -b 1 -l 1024 -g 256 -r 5 -w 2
    python benchmark/benchmark_e2e.py --preset phi3-mini --precision int4 -b 1 -l 1024 -g 256       # synthetic weights
    python benchmark/benchmark_e2e.py --preset phi3-mini --precision int4 -b 8 -l 1024 -g 256 --num_beams 4
    python benchmark/benchmark_e2e.py --preset gpt-oss-20b -b 32 -l 1024 -g 256

With --preset the checkpoint is exported with synthetic weights (the ONNX file only describes the tensors; the
loader draws N(0, 0.02) weights on the device, and quantises them there for int4).  Latencies are wall clock
around the API calls with a device synchronisation on both sides; prompts are random token ids.  Prints one
JSON object per configuration.
"""
import argparse
import json
import os
import statistics
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def intlist(s):
    return [int(x) for x in str(s).split(",") if x]


def run_once(og, model, torch, batch, prompt_len, gen_len, opts, rng, sync):
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=prompt_len + gen_len + 1, batch_size=batch, **opts)
    gen = og.Generator(model, params)
    prompt = rng.randint(0, model.arch.vocab_size - 1, size=(batch, prompt_len)).astype("int32")
    sync()
    t0 = time.perf_counter()
    gen.append_tokens(prompt)
    gen.generate_next_token()
    sync()
    t_first = time.perf_counter()
    steps = []
    n = 1
    while n < gen_len and not gen.is_done():
        t = time.perf_counter()
        gen.generate_next_token()
        steps.append(time.perf_counter() - t)
        n += 1
    sync()
    t_end = time.perf_counter()
    return {"ttft_s": t_first - t0, "decode_s": t_end - t_first, "tokens": n, "steps": steps, "wall_s": t_end - t0}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--input_folder", default="", help="model directory (genai_config.json + model.onnx)")
    ap.add_argument("--preset", default="", help="architecture preset to export with synthetic weights instead of -i")
    ap.add_argument("-pr", "--precision", default="bf16", choices=["bf16", "fp16", "fp32", "int4"])
    ap.add_argument("-e", "--execution_provider", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("-b", "--batch_sizes", type=intlist, default=[1])
    ap.add_argument("-l", "--prompt_lengths", type=intlist, default=[16])
    ap.add_argument("-g", "--generation_lengths", type=intlist, default=[256])
    ap.add_argument("-r", "--repetitions", type=int, default=5)
    ap.add_argument("-w", "--warmup", type=int, default=2)
    ap.add_argument("-k", "--top_k", type=int, default=50)
    ap.add_argument("-p", "--top_p", type=float, default=1.0)
    ap.add_argument("-t", "--temperature", type=float, default=1.0)
    ap.add_argument("--do_sample", action="store_true")
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("-o", "--output", default="", help="append the JSON lines to this file as well")
    a = ap.parse_args()
    import numpy as np
    import torch
    import onnxruntime_genai_b200 as og

    model_dir = a.input_folder
    if not model_dir:
        if not a.preset:
            raise SystemExit("give -i <model_dir> or --preset <name>")
        from onnxruntime_genai_b200.models.builder import create_model
        model_dir = os.path.join(tempfile.gettempdir(), f"ogb_e2e_{a.preset}_{a.precision}_{a.execution_provider}_{os.getuid()}")
        if not os.path.exists(os.path.join(model_dir, "genai_config.json")):
            create_model(a.preset, model_dir, a.precision, a.execution_provider, {"synthetic_weights": 1})
    cfg = og.Config(model_dir)
    cfg.overlay(json.dumps({"model": {"eos_token_id": -1}}))   # fixed amount of work: no sampled id ends a sequence
    t0 = time.perf_counter()
    model = og.Model(cfg)
    load_s = time.perf_counter() - t0
    cuda = model.device.type == "cuda"
    sync = (lambda: torch.cuda.synchronize()) if cuda else (lambda: None)
    opts = {"num_beams": a.num_beams} if a.num_beams > 1 else {}
    if a.do_sample:
        opts.update(do_sample=True, top_k=a.top_k, top_p=a.top_p, temperature=a.temperature, random_seed=1)
    rng = np.random.RandomState(0)
    for b in a.batch_sizes:
        for pl in a.prompt_lengths:
            for gl in a.generation_lengths:
                for _ in range(a.warmup):
                    run_once(og, model, torch, b, pl, min(gl, 16), opts, rng, sync)
                runs = [run_once(og, model, torch, b, pl, gl, opts, rng, sync) for _ in range(a.repetitions)]
                steps = sorted(s for r in runs for s in r["steps"])
                dec_tok = sum((r["tokens"] - 1) * b for r in runs)
                dec_s = sum(r["decode_s"] for r in runs)
                out = {"model": a.preset or os.path.basename(os.path.normpath(model_dir)), "precision": a.precision, "batch_size": b,
                       "prompt_length": pl, "generation_length": gl, "num_beams": a.num_beams, "do_sample": bool(a.do_sample),
                       "ttft_ms_p50": round(statistics.median(r["ttft_s"] for r in runs) * 1e3, 3),
                       "prompt_tokens_per_s": round(b * pl / statistics.median(r["ttft_s"] for r in runs), 1),
                       "tpot_ms_p50": round(steps[len(steps) // 2] * 1e3, 4) if steps else None,
                       "tpot_ms_mean": round(dec_s / max(1, sum(r["tokens"] - 1 for r in runs)) * 1e3, 4),
                       "decode_tokens_per_s": round(dec_tok / dec_s, 1) if dec_s > 0 else None,
                       "wall_s_p50": round(statistics.median(r["wall_s"] for r in runs), 4), "model_load_s": round(load_s, 2),
                       "repetitions": a.repetitions, "device": str(model.device)}
                if cuda:
                    from onnxruntime_genai_b200 import ops
                    ops.check_kernel_status()
                    out["peak_device_memory_gb"] = round(torch.cuda.max_memory_allocated() / 2**30, 2)
                line = json.dumps(out)
                print(line, flush=True)
                if a.output:
                    with open(a.output, "a") as f:
                        f.write(line + "\n")


if __name__ == "__main__":
    main()
