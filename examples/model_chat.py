"""Interactive chat with streaming output and a rolling conversation (counterpart of the reference's
examples/python/model-chat.py): every turn is appended to the same generator, so the KV cache of the earlier turns is reused.

    python examples/model_chat.py -m <model_dir> [--system "You are terse."] [--rewind]
"""
import argparse
import json

import onnxruntime_genai_b200 as og


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("--system", default="You are a helpful assistant.")
    ap.add_argument("--max_length", type=int, default=2048)
    ap.add_argument("--do_sample", action="store_true")
    ap.add_argument("--top_k", type=int, default=50)
    ap.add_argument("--top_p", type=float, default=0.9)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--rewind", action="store_true", help="forget each exchange after it is answered (rewind to the system prompt)")
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    cfg = og.Config(a.model)
    if a.cpu:
        cfg.clear_providers()
    model = og.Model(cfg)
    tok = og.Tokenizer(model)
    stream = tok.create_stream()
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=a.max_length, do_sample=a.do_sample, top_k=a.top_k, top_p=a.top_p, temperature=a.temperature)
    gen = og.Generator(model, params)
    system = tok.apply_chat_template(json.dumps([{"role": "system", "content": a.system}]), add_generation_prompt=False)
    gen.append_tokens(tok.encode(system))
    base = gen.token_count()
    while True:
        try:
            text = input("> ")
        except EOFError:
            break
        if not text.strip():
            continue
        turn = tok.apply_chat_template(json.dumps([{"role": "user", "content": text}]), add_generation_prompt=True)
        gen.append_tokens(tok.encode(turn))
        while not gen.is_done():
            gen.generate_next_token()
            print(stream.decode(int(gen.get_next_tokens()[0])), end="", flush=True)
        print()
        if a.rewind:
            gen.rewind_to(base)


if __name__ == "__main__":
    main()
