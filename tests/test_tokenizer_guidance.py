"""Tokenizer API and constrained decoding (reference: test/python/test_onnxruntime_genai_api.py tokenizer
tests, test/guidance_tests.cpp): a random-weight model constrained by a JSON schema / regex / Lark grammar
must still emit text that the grammar accepts."""
import json
import re

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from helpers import tiny_model_dir


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d, _ = tiny_model_dir(str(tmp_path_factory.mktemp("tok_model")), std=0.3)
    return og.Model(d)


def test_tokenizer_roundtrip_and_batch(model):
    tok = og.Tokenizer(model)
    text = 'hello world {"age": 30}'
    ids = tok.encode(text)
    assert ids.dtype == np.int32 and tok.decode(ids) == text
    batch = tok.encode_batch(["hello", "hello world, hello tokens"])
    assert batch.shape[0] == 2 and batch[0, -1] == tok.pad_token_id
    assert tok.decode_batch(batch)[1] == "hello world, hello tokens"
    assert tok.to_token_id("</s>") == 1 and list(tok.eos_token_ids) == [1]
    with pytest.raises(RuntimeError):
        tok.to_token_id("definitely-not-one-token-xyz")


def test_tokenizer_stream_matches_full_decode(model):
    tok = og.Tokenizer(model)
    text = "The quick brown fox — café ✓ jumps"
    ids = tok.encode(text)
    stream = tok.create_stream()
    pieces = "".join(stream.decode(int(t)) for t in ids)
    assert pieces == tok.decode(ids)


def test_chat_template(model):
    tok = og.Tokenizer(model)
    msgs = json.dumps([{"role": "user", "content": "hi"}])
    assert tok.apply_chat_template(msgs) == "<|user|>hi\n<|assistant|>"
    assert tok.apply_chat_template(msgs, add_generation_prompt=False) == "<|user|>hi\n"
    assert tok.apply_chat_template(msgs, template_str="{{ messages[0]['content'] }}!") == "hi!"


def _generate(model, prompt_ids, guidance, max_new=60, **search):
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(prompt_ids) + max_new, **search)
    if guidance:
        p.set_guidance(*guidance)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray(prompt_ids, dtype=np.int32))
    while not g.is_done():
        g.generate_next_token()
    out = g.get_sequence(0)[len(prompt_ids):].tolist()
    while out and out[-1] in (0, 1):
        out.pop()
    return out


def test_json_schema_guidance(model):
    tok = og.Tokenizer(model)
    schema = json.dumps({"type": "object", "properties": {"name": {"type": "string", "maxLength": 8}, "age": {"type": "integer"}},
                         "required": ["name", "age"], "additionalProperties": False})
    for seed in (1, 2):
        out = _generate(model, tok.encode("profile:"), ("json_schema", schema), max_new=120, do_sample=True, top_k=20,
                        temperature=1.0, random_seed=seed)
        text = tok.decode(out)
        obj = json.loads(text)
        assert set(obj) == {"name", "age"} and isinstance(obj["age"], int) and isinstance(obj["name"], str)


def test_regex_and_lark_guidance(model):
    tok = og.Tokenizer(model)
    out = _generate(model, tok.encode("id:"), ("regex", r"[a-c]{3}-[0-9]{2}"), do_sample=True, top_k=30, random_seed=3)
    assert re.fullmatch(r"[a-c]{3}-[0-9]{2}", tok.decode(out))
    lark = 'start: "yes" | "no" | "maybe"'
    out = _generate(model, tok.encode("answer:"), ("lark_grammar", lark))
    assert tok.decode(out) in ("yes", "no", "maybe")


def test_guidance_in_engine(model):
    tok = og.Tokenizer(model)
    engine = og.Engine(model)
    reqs = []
    for seed, (kind, data) in enumerate([("regex", r"(ab|cd){2}"), ("lark_grammar", 'start: "true" | "false"'), (None, None)]):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=40, do_sample=True, top_k=10, random_seed=seed)
        if kind:
            p.set_guidance(kind, data)
        r = og.Request(p)
        r.add_tokens(tok.encode("x:"))
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
    assert re.fullmatch(r"(ab|cd){2}", tok.decode(outs[id(reqs[0])]))
    assert tok.decode(outs[id(reqs[1])]) in ("true", "false")


def test_guidance_errors(model):
    p = og.GeneratorParams(model)
    with pytest.raises(RuntimeError):
        p.set_guidance("yaml", "x")
    p.set_guidance("json_schema", "{ not json")
    with pytest.raises(Exception):
        og.Generator(model, p)


def test_guidance_inside_speculative_rounds(model):
    """n-gram speculation with a grammar: every verify row is masked with what the grammar allows after the drafts before it
    (a cloned cursor walks the draft), so greedy speculative decoding gives exactly the constrained greedy text, and sampled
    verification still only emits text the grammar accepts (reference: src/speculative_decoding_strategy.cpp:944-1270)."""
    tok = og.Tokenizer(model)
    schema = json.dumps({"type": "object", "properties": {"name": {"type": "string", "maxLength": 8}, "tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 6}},
                         "required": ["name", "tags"], "additionalProperties": False})
    prompt = tok.encode('{"name": "ab", "tags": ["a", "b", "a", "b"]} {"name": "ab", "tags": ["a", "b", "a", "b"]} ')

    def run(spec, **search):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(prompt) + 90, **search)
        p.set_guidance("json_schema", schema)
        if spec:
            p.set_speculative_options(ngram_size=2, max_draft_tokens=4)
        g = og.Generator(model, p)
        g.append_tokens(np.asarray(prompt, dtype=np.int32))
        while not g.is_done():
            g.generate_next_token()
        out = g.get_sequence(0)[len(prompt):].tolist()
        while out and out[-1] in (0, 1):
            out.pop()
        return out, (g.get_speculative_stats() if spec else {})

    plain, _ = run(False, do_sample=False)
    spec, stats = run(True, do_sample=False)
    assert spec == plain
    assert stats["rounds"] > 0 and stats["proposed"] > 0
    json.loads(tok.decode(spec))
    sampled, stats = run(True, do_sample=True, top_k=20, temperature=1.0, random_seed=5)
    obj = json.loads(tok.decode(sampled))
    assert set(obj) == {"name", "tags"} and stats["rounds"] > 0
