"""Builds and runs the native engine benchmark (engine_bench.cpp, C API only) and, with --replicas, starts one engine process
per GPU (data parallelism: independent replicas, each pinned with CUDA_VISIBLE_DEVICES) and adds their throughput up.

    python benchmark/engine/run.py --model DIR --scenario mixed --concurrency 8 --prompt_len 512 --long_prompt_len 32768
    python benchmark/engine/run.py --model DIR --scenario decode_baseline --replicas 8           # one replica per GPU
    python benchmark/engine/run.py --model DIR --all --out results.json                          # every scenario, gates reported

Reference: benchmark/engine/run.py (scenario dispatcher, --cuda_visible_devices), benchmark/engine/docs/benchmark-requirements.md.
"""
import argparse
import json
import os
import platform
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
C_API = os.path.join(ROOT, "onnxruntime_genai_b200", "native", "c_api")
SCENARIOS = ("decode_baseline", "mixed", "cancellation", "continuation")


def build(out_dir: str) -> str:
    sys.path.insert(0, ROOT)
    from onnxruntime_genai_b200.build_native import build_c_api
    build_c_api()
    exe = os.path.join(out_dir, "engine_bench")
    src = os.path.join(HERE, "engine_bench.cpp")
    if not os.path.exists(exe) or os.path.getmtime(exe) < os.path.getmtime(src):
        subprocess.run(["g++", "-O2", "-std=c++17", "-Wall", "-I" + C_API, src, "-o", exe, "-L" + C_API, "-logb200_genai", "-Wl,-rpath," + C_API],
                       check=True)
    return exe


def vocab_size(model_dir: str) -> int:
    with open(os.path.join(model_dir, "genai_config.json")) as f:
        return int(json.load(f)["model"]["vocab_size"])


def run_one(exe, args, scenario, visible=None):
    cmd = [exe, "--model", args.model, "--vocab", str(vocab_size(args.model)), "--scenario", scenario, "--concurrency", str(args.concurrency),
           "--prompt_len", str(args.prompt_len), "--long_prompt_len", str(args.long_prompt_len), "--new_tokens", str(args.new_tokens),
           "--trials", str(args.trials), "--turns", str(args.turns), "--itl_gate_ratio", str(args.itl_gate_ratio),
           "--cancel_gate_ms", str(args.cancel_gate_ms)]
    env = dict(os.environ, OGB_PYTHON=sys.executable)
    if visible is not None:
        env["CUDA_VISIBLE_DEVICES"] = str(visible)
    return subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)


def collect(proc):
    out, err = proc.communicate()
    try:
        res = json.loads(out[out.index("{"):])
    except ValueError:
        res = {"error": (out + err)[-2000:]}
    res["exit_code"] = proc.returncode
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True)
    ap.add_argument("--scenario", default="decode_baseline", choices=SCENARIOS)
    ap.add_argument("--all", action="store_true")
    ap.add_argument("--concurrency", type=int, default=4)
    ap.add_argument("--prompt_len", type=int, default=512)
    ap.add_argument("--long_prompt_len", type=int, default=8192)
    ap.add_argument("--new_tokens", type=int, default=64)
    ap.add_argument("--trials", type=int, default=8)
    ap.add_argument("--turns", type=int, default=3)
    ap.add_argument("--itl_gate_ratio", type=float, default=1.5, help="decode inter-token latency p95 during a prefill / steady baseline")
    ap.add_argument("--cancel_gate_ms", type=float, default=500.0)
    ap.add_argument("--replicas", type=int, default=1, help="independent engine processes, one per GPU")
    ap.add_argument("--cuda_visible_devices", default="", help="comma-separated device ids for the replicas (default 0..replicas-1)")
    ap.add_argument("--build_dir", default=os.path.join(HERE, "build"))
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    os.makedirs(a.build_dir, exist_ok=True)
    exe = build(a.build_dir)
    meta = {"host": platform.node(), "python": sys.version.split()[0], "time": time.strftime("%Y-%m-%dT%H:%M:%S"), "model": a.model}
    try:
        meta["commit"] = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], capture_output=True, text=True).stdout.strip()
        import torch
        meta["torch"] = torch.__version__
        if torch.cuda.is_available():
            meta["gpu"] = torch.cuda.get_device_name(0)
    except Exception:
        pass
    results = {"environment": meta, "runs": []}
    for scenario in (SCENARIOS if a.all else (a.scenario,)):
        if a.replicas > 1:
            ids = [x for x in a.cuda_visible_devices.split(",") if x] or [str(i) for i in range(a.replicas)]
            procs = [run_one(exe, a, scenario, ids[i % len(ids)]) for i in range(a.replicas)]
            reps = [collect(p) for p in procs]
            total = sum(r.get("tokens_per_s", 0.0) for r in reps)
            results["runs"].append({"scenario": scenario, "replicas": reps, "replica_count": a.replicas, "tokens_per_s_total": total,
                                    "gates_passed": all(r.get("gates_passed") for r in reps)})
        else:
            results["runs"].append(collect(run_one(exe, a, scenario)))
    results["gates_passed"] = all(r.get("gates_passed") for r in results["runs"])
    text = json.dumps(results, indent=1)
    print(text)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text)
    sys.exit(0 if results["gates_passed"] else 1)


if __name__ == "__main__":
    main()
