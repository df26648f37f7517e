"""Continuous batching with the paged-attention engine (counterpart of the reference's
examples/python/engine/continuous-batching.py): requests are added while others are running and each
streams its tokens as `engine.step()` hands them back."""
import argparse

import onnxruntime_genai_b200 as og


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompts", nargs="*", default=["The capital of France is", "def fibonacci(n):", "Once upon a time"])
    ap.add_argument("--max_new_tokens", type=int, default=64)
    a = ap.parse_args()
    model = og.Model(a.model)
    tok = og.Tokenizer(model)
    engine = og.Engine(model)
    streams, waiting = {}, list(a.prompts)
    step = 0
    while waiting or engine.has_pending_requests():
        if waiting and step % 4 == 0:      # staggered arrival
            text = waiting.pop(0)
            ids = tok.encode(text)
            params = og.GeneratorParams(model)
            params.set_search_options(max_length=len(ids) + a.max_new_tokens, do_sample=True, top_k=40, temperature=0.8)
            req = og.Request(params)
            req.add_tokens(ids)
            req.set_opaque_data(text)
            engine.add_request(req)
            streams[id(req)] = tok.create_stream()
        step += 1
        req = engine.step()
        if req is None:
            continue
        while req.has_unseen_tokens():
            piece = streams[id(req)].decode(req.get_unseen_token())
            print(f"[{req.get_opaque_data()[:16]!r}] {piece}", flush=True)
        if req.is_turn_complete():
            engine.remove_request(req)


if __name__ == "__main__":
    main()
