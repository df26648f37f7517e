"""Constrained decoding with a JSON schema (counterpart of the reference's examples/python/guidance-example.py)."""
import argparse
import json

import onnxruntime_genai_b200 as og

SCHEMA = {"type": "object", "properties": {"city": {"type": "string"}, "population": {"type": "integer"}},
          "required": ["city", "population"], "additionalProperties": False}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompt", default="Describe Paris as JSON: ")
    a = ap.parse_args()
    model = og.Model(a.model)
    tok = og.Tokenizer(model)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=256)
    params.set_guidance("json_schema", json.dumps(SCHEMA))
    gen = og.Generator(model, params)
    ids = tok.encode(a.prompt)
    gen.append_tokens(ids)
    while not gen.is_done():
        gen.generate_next_token()
    print(tok.decode(gen.get_sequence(0)[len(ids):]))


if __name__ == "__main__":
    main()
