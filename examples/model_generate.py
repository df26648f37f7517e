"""Token-by-token generation (counterpart of the reference's examples/python/model-generate.py).

    python examples/model_generate.py -m <model_dir> -p "Once upon a time" --max_length 128 --do_sample --top_k 50
"""
import argparse
import time

import onnxruntime_genai_b200 as og


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompts", nargs="*", default=["Hello"])
    ap.add_argument("--max_length", type=int, default=128)
    ap.add_argument("--do_sample", action="store_true")
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--top_p", type=float, default=0.0)
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--cpu", action="store_true", help="ignore the configured providers and run the fp32 CPU path")
    a = ap.parse_args()
    cfg = og.Config(a.model)
    if a.cpu:
        cfg.clear_providers()
    model = og.Model(cfg)
    tok = og.Tokenizer(model)
    ids = tok.encode_batch(a.prompts)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=a.max_length, batch_size=len(a.prompts), do_sample=a.do_sample, top_k=a.top_k, top_p=a.top_p,
                              temperature=a.temperature, num_beams=a.num_beams)
    gen = og.Generator(model, params)
    t0 = time.perf_counter()
    gen.append_tokens(ids)
    t1 = time.perf_counter()
    n = 0
    while not gen.is_done():
        gen.generate_next_token()
        n += 1
    t2 = time.perf_counter()
    for i, p in enumerate(a.prompts):
        print(f"--- {p!r}\n{tok.decode(gen.get_sequence(i))}")
    print(f"prompt {ids.size} tokens in {(t1 - t0) * 1e3:.1f} ms; {n} steps, {n * len(a.prompts) / (t2 - t1):.1f} tokens/s")


if __name__ == "__main__":
    main()
