"""Headline benchmark: decode tokens/s (+ p50 TTFT / TPOT) of Llama-3.1-8B-shaped serving through
the paged-attention continuous-batching engine, bf16, tensor-parallel over N GPUs of one node.

Workload (BASELINE config 3): 64 concurrent requests, prompt lengths uniform in [128, 2048] of
random token ids (seed 2), 256 output tokens each, sampling with temperature 0.7, top_k 50,
top_p 0.9, KV block size 16; random-init weights N(0, 0.02) generated on the device.

A "step" is one decode step of the whole batch (64 new tokens).  Two measurements:
  * value: device-timed (CUDA events) consecutive decode steps with the inputs advanced on the device (sampled ids fed
    back, KV lengths growing) — the kernels alone, no host work between steps;
  * e2e:   the same steps through the public API (`Engine.step()`), each step packing its inputs
    on the host, copying them from pinned memory to the device and reading the sampled ids back.
Timing rules: >= 3 warm-up steps, barrier + synchronize on both sides, max over ranks, the
working set (16 GB of weights + KV) is far larger than L2 so no flush is needed, SM clocks and
throttle reasons are sampled with nvidia-smi during the timed region.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config llama8b|gptoss20b|llama70b]
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s"
MODEL = "llama-3.1-8b"
N_REQ, PROMPT_LO, PROMPT_HI, NEW_TOKENS, BLOCK = 64, 128, 2048, 256, 16
SAMPLING = dict(do_sample=True, temperature=0.7, top_k=50, top_p=0.9)
# Other named workloads (--config): same engine, same timing rules.
CONFIGS = {
    "llama8b": dict(model="llama-3.1-8b", label="Llama-3.1-8B shape", n_req=64, lo=128, hi=2048, new=256, sampling=SAMPLING,
                    sampling_label="T=0.7 top_k=50 top_p=0.9"),
    "gptoss20b": dict(model="gpt-oss-20b", label="gpt-oss-20B shape (bf16 experts, expert parallel over the ranks)", n_req=32, lo=1024,
                      hi=1024, new=256, sampling={}, sampling_label="greedy"),
    "llama70b": dict(model="llama-3.1-70b", label="Llama-3.1-70B shape", n_req=16, lo=2048, hi=2048, new=512, sampling={},
                     sampling_label="greedy"),
}


def reference_arm(args):
    """The reference needs ONNX Runtime binaries fetched from a package feed at build time
    (cmake/ortlib.cmake) and the `onnx` / `onnxruntime` Python packages, none of which exist offline."""
    why = "reference cannot be installed offline: its build downloads ONNX Runtime binaries (cmake/ortlib.cmake) and needs onnx/onnxruntime"
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import onnxruntime_genai  # noqa: F401
        why = "reference package imported but no ONNX Runtime CUDA provider / ONNX model exporter is available offline"
    except Exception:
        pass
    finally:
        sys.path.pop(0)
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


class ClockSampler:
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.idx), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def ours(args):
    global MODEL, N_REQ, PROMPT_LO, PROMPT_HI, NEW_TOKENS, SAMPLING
    cfg_w = CONFIGS[args.config]
    MODEL, N_REQ, PROMPT_LO, PROMPT_HI, NEW_TOKENS, SAMPLING = cfg_w["model"], cfg_w["n_req"], cfg_w["lo"], cfg_w["hi"], cfg_w["new"], cfg_w["sampling"]
    import numpy as np
    import torch
    import torch.distributed as dist

    import onnxruntime_genai_b200 as og
    from onnxruntime_genai_b200 import ops
    from onnxruntime_genai_b200.models.builder import create_model
    from onnxruntime_genai_b200.ops import _lib
    from onnxruntime_genai_b200.parallel.tp import TensorParallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} processes (WORLD_SIZE={world})")
    torch.cuda.set_device(local)
    if world > 1:
        import faulthandler
        faulthandler.dump_traceback_later(1500, exit=True)   # a stuck rank reports where and ends instead of hanging the job
    tp = TensorParallel.from_env(args.tp_backend or os.environ.get("OGB_TP_BACKEND")) if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- checkpoint (synthetic weights: the ONNX file only describes the tensors) + model + engine
    ckpt = os.path.join(tempfile.gettempdir(), f"ogb_bench_{MODEL}_{args.precision}_{os.getuid()}" + (f"_spec_{args.draft_model}_{args.draft_seed}" if args.spec else ""))
    if rank == 0 and not os.path.exists(os.path.join(ckpt, "genai_config.json")):
        create_model(MODEL, ckpt, args.precision, "cuda", {"synthetic_weights": 1, "paged_attention": 1, "paged_block_size": BLOCK,
                                                  "max_batch_size": N_REQ, "context_length": 4096})
        if args.spec:
            # speculative decoding: a Llama-3.2-1B-shaped draft next to the target (its own ONNX file, `model.draft` in the config)
            tmp = ckpt + "_draft"
            create_model(args.draft_model, tmp, "bf16", "cuda", {"synthetic_weights": 1, "paged_attention": 1, "paged_block_size": BLOCK,
                                                                  "max_batch_size": N_REQ, "context_length": 4096, "filename": "draft.onnx",
                                                                  "seed": args.draft_seed})
            for fn in os.listdir(tmp):
                if fn.startswith("draft.onnx"):
                    os.replace(os.path.join(tmp, fn), os.path.join(ckpt, fn))
            with open(os.path.join(tmp, "genai_config.json")) as f:
                draft_dec = json.load(f)["model"]["decoder"]
            with open(os.path.join(ckpt, "genai_config.json")) as f:
                full = json.load(f)
            full["model"]["draft"] = draft_dec
            full["speculative"] = {"max_draft_tokens": args.draft_tokens}
            with open(os.path.join(ckpt, "genai_config.json"), "w") as f:
                json.dump(full, f, indent=1)
    if rank == 0 and args.json_schema and not os.path.exists(os.path.join(ckpt, "tokenizer.json")):
        # a byte-level BPE tokenizer trained on a few lines (the grammar needs token -> bytes; ids beyond its vocabulary are never allowed)
        from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
        tok = Tokenizer(models.BPE())
        tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
        tok.decoder = decoders.ByteLevel()
        corpus = ['{"name": "Alice", "score": 30, "notes": "The quick brown fox jumps over the lazy dog."}', "hello world, hello tokens, hello grammar 0123456789",
                  "abcdefghijklmnopqrstuvwxyz ABCDEFGHIJKLMNOPQRSTUVWXYZ : , [] {} true false null"] * 8
        tok.train_from_iterator(corpus, trainers.BpeTrainer(vocab_size=2048, special_tokens=["<s>", "</s>"], show_progress=False,
                                                            initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
        tok.save(os.path.join(ckpt, "tokenizer.json"))
    barrier()
    cfg = og.Config(ckpt)
    blocks = N_REQ * ((PROMPT_HI + NEW_TOKENS + BLOCK - 1) // BLOCK + 1)
    # eos_token_id -1 never matches a sampled id: every request produces exactly NEW_TOKENS tokens (fixed workload).
    # (under a grammar the end-of-sequence id must exist for the matcher: id 1 of the synthetic tokenizer, which the never-ending
    # schema below never allows)
    cfg.overlay(json.dumps({"model": {"eos_token_id": 1 if args.json_schema else -1},
                            "engine": {"dynamic_batching": {"block_size": BLOCK, "num_blocks": blocks, "max_batch_size": N_REQ,
                                                             "max_scheduled_tokens": 4096}}}))
    t0 = time.perf_counter()
    model = og.Model(cfg, tp=tp)
    load_s = time.perf_counter() - t0
    engine = og.Engine(model)

    schema = None
    if args.json_schema:
        # Constrained decoding: every request generates under a JSON schema (llguidance computes a token mask per request and
        # step on the host while the forward runs; the mask is applied on the device before sampling).  The schema's last
        # field is a string too long to finish within the run, so that every request decodes all its tokens under the grammar.
        schema = json.dumps({"type": "object", "properties": {"name": {"type": "string", "maxLength": 12}, "score": {"type": "integer"},
                                                               "notes": {"type": "string", "minLength": 8192}},
                             "required": ["name", "score", "notes"], "additionalProperties": False})

    rng = np.random.RandomState(2)
    lens = rng.randint(PROMPT_LO, PROMPT_HI + 1, size=N_REQ)
    reqs = []
    for i, n in enumerate(lens):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=int(n) + NEW_TOKENS + 1, random_seed=2 + i, **SAMPLING)
        if schema:
            p.set_guidance("json_schema", schema)
        r = og.Request(p)
        r.add_tokens(rng.randint(0, model.arch.vocab_size, size=int(n)).astype(np.int32))
        reqs.append(r)

    def drain(r):
        n = 0
        while r is not None and r.has_unseen_tokens():
            r.get_unseen_token()
            n += 1
        return n

    # ---- engine warm-up (a serving process is warm when requests arrive): one full-length prompt through prefill and a
    # few decode steps, then removed - first-use costs (allocator growth, tensor maps, kernel attributes) leave the TTFT phase
    wp = og.GeneratorParams(model)
    wp.set_search_options(max_length=PROMPT_HI + 8, random_seed=1, **SAMPLING)
    wr = og.Request(wp)
    wr.add_tokens(rng.randint(0, model.arch.vocab_size, size=PROMPT_HI).astype(np.int32))
    engine.add_request(wr)
    while engine.has_pending_requests():
        r_ = engine.step()
        drain(r_)
        if r_ is not None and r_.is_turn_complete():
            engine.remove_request(r_)
    torch.cuda.synchronize()

    # ---- prefill (TTFT): admit everything, step until every request has its first token
    barrier()
    t_start = time.perf_counter()
    for r in reqs:
        engine.add_request(r)
    while any(r.t_first is None for r in reqs):
        drain(engine.step())
    torch.cuda.synchronize()
    ttft = sorted((r.t_first - t_start) * 1e3 for r in reqs)
    prefill_s = time.perf_counter() - t_start
    prefill_tok_s = float(lens.sum()) / prefill_s

    def model_steps(k):
        """Runs k decode steps through the public API; returns tokens produced."""
        done = 0
        target = engine.step_count + k
        while engine.step_count < target:
            done += drain(engine.step())
        # drain what the last model step made ready without running the model again
        return done

    W, K = max(3, args.warmup), args.steps
    K = min(K, NEW_TOKENS - 40 - W)  # requests admitted first have decoded ~20-30 tokens by the end of the prefill phase
    # ---- e2e: public API, pinned H2D of the step inputs + D2H of the sampled ids every step
    model_steps(W)
    barrier()
    hs0 = dict(engine.host_stats)
    sampler = ClockSampler(local)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_e0 = time.perf_counter()
    launches0 = _lib.LAUNCH_COUNT
    ev0.record()
    produced = model_steps(K)
    ev1.record()
    e2e_launches = _lib.LAUNCH_COUNT - launches0
    barrier()
    e2e_wall = time.perf_counter() - t_e0
    e2e_ms = ev0.elapsed_time(ev1)
    hs1 = engine.host_stats
    n_l = max(1, hs1["launches"] - hs0["launches"])
    host = {"launch_ms_per_step": round((hs1["launch_s"] - hs0["launch_s"]) / n_l * 1e3, 4),
            "wait_ms_per_step": round((hs1["wait_s"] - hs0["wait_s"]) / n_l * 1e3, 4)}
    step_wall = e2e_wall / K

    spec = getattr(engine, "spec", None)
    if spec is not None:
        # Speculative decoding: a step verifies several proposed tokens per request, there is no fixed decode graph to replay;
        # the device-timed figure is the CUDA-event time of the same engine steps (draft proposals + one packed verify forward).
        clocks = sampler.stop()
        ops.check_kernel_status()

        def mx(x):
            if world == 1:
                return x
            t = torch.tensor([x], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        e2e_ms, e2e_wall = mx(e2e_ms), mx(e2e_wall)
        if rank == 0:
            st = spec.stats
            print(json.dumps({
                "metric": METRIC, "value": round(produced / (e2e_ms / 1e3), 1), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
                "ms_per_step": round(e2e_ms / K, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic (random token ids, random-init N(0,0.02) weights generated on device)",
                "config": {"model": cfg_w["label"] + f" + speculative decoding, draft {args.draft_model}, {args.draft_tokens} draft tokens per step",
                           "global_batch": N_REQ, "seq_len": f"prompts U[{PROMPT_LO},{PROMPT_HI}] + {NEW_TOKENS} new tokens",
                           "parallelism": f"tp{world}", "kv_block_size": BLOCK, "sampling": cfg_w["sampling_label"],
                           "l2": "inputs larger than L2, no flush", "tp_backend": getattr(tp, "backend", None)},
                "e2e": {"value": round(produced / e2e_wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": st_bytes(engine), "d2h_bytes_per_step": 4 * N_REQ * (args.draft_tokens + 1),
                        "ms_per_step": round(e2e_wall / K * 1e3, 4)},
                "speculative": {"acceptance_rate": round(spec.acceptance_rate, 4), "tokens_per_request_step": round(st["committed"] / max(1, st["rounds"]), 3),
                                "rounds": st["rounds"], "note": "random-init target and draft share no distribution: the acceptance rate of random weights is a floor, not a forecast"},
                "gpu_launches": int(e2e_launches), "clocks": clocks, "ttft_ms_p50": round(ttft[len(ttft) // 2], 2),
                "tpot_ms_p50": round(e2e_wall / max(1, produced) * N_REQ * 1e3, 4), "prefill_tokens_per_s": round(prefill_tok_s, 1)}))
        if world > 1:
            torch.cuda.synchronize(); dist.barrier(); sys.stdout.flush(); sys.stderr.flush(); os._exit(0)
        return 0

    # ---- device-only: the kernels of K consecutive decode steps, inputs advanced on the device (the sampled ids become the
    # next input ids, positions / cache slots / KV lengths move on by one: exactly what the engine enqueues ahead of the host),
    # no host work and no copies between steps
    ex = engine.executor
    key = sorted(ex.graphs.keys())[-1] if ex.graphs else None
    st = engine.staging
    B = N_REQ
    if key is None:
        raise SystemExit("decode graph was not captured")
    # the block tables on the device get spare (unowned) blocks behind each request's own, so that W + K more positions have
    # cache slots; nothing runs through the engine after this point
    advance = ex.kv.win is None      # sliding-window ring tables are advanced on the host: those models replay frozen inputs
    table = st.view("block_table").view(st.max_batch, st.table_cols)
    used = torch.unique(table[table >= 0])
    free = torch.ones(engine.options.num_blocks, dtype=torch.bool, device=table.device)
    free[used.long()] = False
    spare = torch.nonzero(free).flatten().to(torch.int32)
    extra = (W + K) // BLOCK + 2
    if advance:
        assert spare.numel() >= B * extra, "not enough spare cache blocks for the device-timed steps"
        first_free = (table[:B] >= 0).sum(dim=1)
        cols = first_free[:, None] + torch.arange(extra, device=table.device)[None, :]
        ok = cols < st.table_cols
        rows_i = torch.arange(B, device=table.device)[:, None].expand_as(cols)
        table[rows_i[ok], cols[ok]] = spare[:B * extra].view(B, extra)[ok]
    graph, logits = ex.graphs[key]
    sample_args = (st.view("top_k", B), st.view("top_p", B, torch.float32), st.view("temperature", B, torch.float32),
                   st.view("seeds", None, torch.int64)[:B], st.view("sample_pos", B))
    toks = ops.sample(logits[:B], *sample_args)

    def device_step(toks):
        if advance:
            ops.decode_advance(toks, st.view("input_ids", B), st.view("positions", B), st.view("past_lens", B), st.view("slot_mapping", B),
                               st.view("sample_pos", B), table[:B], BLOCK)
        graph.replay()
        return ops.sample(logits[:B], *sample_args)

    for _ in range(W):
        toks = device_step(toks)
    barrier()
    d0, d1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    d0.record()
    for _ in range(K):
        toks = device_step(toks)
    d1.record()
    barrier()
    dev_ms = d0.elapsed_time(d1)
    clocks = sampler.stop()
    ops.check_kernel_status()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev_ms, e2e_ms, e2e_wall = max_over_ranks(dev_ms), max_over_ranks(e2e_ms), max_over_ranks(e2e_wall)
    value = B * K / (dev_ms / 1e3)
    e2e_value = B * K / e2e_wall
    launches = getattr(ex, "graph_launches", {}).get(key, 0) + 2      # + decode_advance + sampler
    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": round(dev_ms / K, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (random token ids, random-init N(0,0.02) weights generated on device)",
            "config": {"model": cfg_w["label"].replace("bf16 experts", "packed MXFP4 experts, int4 attention projections") if args.precision == "int4"
                       else cfg_w["label"], "weights": args.precision, "global_batch": B,
                       "seq_len": f"prompts U[{PROMPT_LO},{PROMPT_HI}] + {NEW_TOKENS} new tokens",
                       "parallelism": f"tp{world}", "kv_block_size": BLOCK, "sampling": cfg_w["sampling_label"],
                       "engine": "paged-attention continuous batching; warmed with one 2048-token request before the TTFT phase", "l2": "inputs larger than L2 (weights + KV of tens of GB), no flush",
                       "tp_backend": getattr(tp, "backend", None),
                       "constrained": "every request under a JSON schema (llguidance masks; the e2e figure includes them)" if schema else None,
                       "device_loop": "inputs advanced on the device between steps" if advance else "frozen inputs (sliding-window ring tables advance on the host)"},
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": st.h2d_bytes, "d2h_bytes_per_step": 4 * B,
                    "ms_per_step": round(e2e_wall / K * 1e3, 4), "device_ms_per_step": round(e2e_ms / K, 4),
                    "host_launch_ms_per_step": host["launch_ms_per_step"], "host_wait_ms_per_step": host["wait_ms_per_step"],
                    "steps_enqueued_ahead": int(engine.lookahead_hits)},
            "gpu_launches": int(launches * K),
            "clocks": clocks,
            "ttft_ms_p50": round(ttft[len(ttft) // 2], 2), "tpot_ms_p50": round(step_wall * 1e3, 4),
            "prefill_tokens_per_s": round(prefill_tok_s, 1), "model_load_s": round(load_s, 1),
            "kv_tokens_in_cache": int(lens.sum() + N_REQ * (W + K)),
        }
        print(json.dumps(out))
    if world > 1:
        # Leave without tearing the communicator down: the captured graphs still hold collective kernels, and
        # destroying the process group under them can block.  Everything timed has completed and been reduced.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


def st_bytes(engine):
    return engine.staging.h2d_bytes


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tp_backend", default="", choices=["", "fused", "nccl"],
                    help="tensor-parallel reductions: fused (GEMM + all-reduce in one kernel over peer memory; the default) or nccl "
                         "(GEMM, then ncclAllReduce: the baseline this framework is measured against, NCCL's own NVLS left on)")
    ap.add_argument("--spec", action="store_true", help="speculative decoding inside the engine with a draft model (config llama70b: Llama-3.2-1B shape)")
    ap.add_argument("--draft_model", default="llama-3.2-1b")
    ap.add_argument("--draft_tokens", type=int, default=4)
    ap.add_argument("--draft_seed", type=int, default=1, help="seed of the draft's random weights (0 with --draft_model equal to the target: "
                                                              "identical networks, the acceptance ceiling)")
    ap.add_argument("--json-schema", dest="json_schema", action="store_true", help="every request decodes under a JSON schema (needs tokenizer.json)")
    ap.add_argument("--config", default="llama8b", choices=sorted(CONFIGS), help="workload; the default is the headline configuration")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "int4"],
                    help="weights of the checkpoint: bf16 (headline) or 4-bit (int4 block-32 linears; gpt-oss experts as packed MXFP4, the form "
                         "the reference publishes its gpt-oss numbers for); activations and the KV cache stay bf16")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    return ours(args)


if __name__ == "__main__":
    sys.exit(main())
