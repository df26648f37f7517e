"""Speculative decoding: n-gram lookup (no draft model) or a draft model named by `model.draft` in
genai_config.json (see docs of the reference: docs/SpeculativeDecoding.md)."""
import argparse

import onnxruntime_genai_b200 as og


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompt", default="repeat after me: a b c a b c a b c")
    ap.add_argument("--ngram_size", type=int, default=3)
    ap.add_argument("--max_draft_tokens", type=int, default=4)
    a = ap.parse_args()
    model = og.Model(a.model)
    tok = og.Tokenizer(model)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=200)
    params.set_speculative_options(max_draft_tokens=a.max_draft_tokens, ngram_size=0 if model.draft is not None else a.ngram_size,
                                   min_adaptive_k=2, cooldown=True)
    gen = og.Generator(model, params)
    gen.append_tokens(tok.encode(a.prompt))
    while not gen.is_done():
        gen.generate_next_token()
    print(tok.decode(gen.get_sequence(0)))
    print(gen.get_speculative_stats())


if __name__ == "__main__":
    main()
