"""Speculative decoding (reference tests: test/python/models/test_speculative_decoding.py — a draft equal to
the target must reproduce plain greedy decoding; n_gram_lookup_tests.cpp; speculative_sampling_tests.cpp)."""
import copy
import json
import os

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model, make_genai_config, random_state_dict
from onnxruntime_genai_b200.native_loader import native


def small_arch(layers=2, hidden=64):
    return ArchConfig(model_type="llama", vocab_size=97, hidden_size=hidden, num_layers=layers, num_heads=4, num_kv_heads=2,
                      head_dim=16, intermediate_size=128, context_length=256, bos_token_id=0, eos_token_id=96, pad_token_id=0)


@pytest.fixture(scope="module")
def spec_dir(tmp_path_factory):
    """Target + a draft that is the same network (acceptance must then be 100 % under greedy)."""
    d = str(tmp_path_factory.mktemp("spec"))
    arch = small_arch()
    sd = random_state_dict(arch, seed=3, std=0.3)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd, filename="draft.onnx", write_config=False)
    weak = small_arch(layers=1)
    export_model(weak, d, "fp32", "cpu", state_dict=random_state_dict(weak, seed=9, std=0.3), filename="weak_draft.onnx", write_config=False)
    return d


def with_draft(spec_dir, filename, tmp_path, layers):
    cfg = json.load(open(os.path.join(spec_dir, "genai_config.json")))
    dec = copy.deepcopy(cfg["model"]["decoder"])
    dec["filename"] = filename
    dec["num_hidden_layers"] = layers
    cfg["model"]["draft"] = dec
    out = str(tmp_path)
    for f in os.listdir(spec_dir):
        if f != "genai_config.json":
            os.symlink(os.path.join(spec_dir, f), os.path.join(out, f))
    json.dump(cfg, open(os.path.join(out, "genai_config.json"), "w"))
    return out


def generate(model, prompt, n, **opts):
    p = og.GeneratorParams(model)
    spec = {k: opts.pop(k) for k in list(opts) if k in ("max_draft_tokens", "ngram_size", "ngram_chained_lookup", "min_adaptive_k", "cooldown")}
    p.set_search_options(max_length=len(prompt) + n, **opts)
    if spec:
        p.set_speculative_options(**spec)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray(prompt, dtype=np.int32))
    calls = 0
    while not g.is_done():
        before = g.token_count()
        g.generate_next_token()
        assert g.token_count() == before + 1, "the API yields exactly one token per call"
        calls += 1
    return g.get_sequence(0).tolist(), g


PROMPT = [5, 17, 40, 3, 22, 9, 61, 5, 17, 40, 3]


def test_self_speculation_equals_greedy(spec_dir, tmp_path):
    plain, _ = generate(og.Model(spec_dir), PROMPT, 40)
    model = og.Model(with_draft(spec_dir, "draft.onnx", tmp_path, 2))
    spec, g = generate(model, PROMPT, 40, max_draft_tokens=4)
    assert spec == plain
    st = g.get_speculative_stats()
    assert st["rounds"] > 0 and st["acceptance_rate"] == 1.0 and st["tokens_per_round"] > 4.0


def test_weak_draft_still_equals_greedy(spec_dir, tmp_path):
    plain, _ = generate(og.Model(spec_dir), PROMPT, 30)
    model = og.Model(with_draft(spec_dir, "weak_draft.onnx", tmp_path, 1))
    spec, g = generate(model, PROMPT, 30, max_draft_tokens=3, cooldown=True)
    assert spec == plain
    st = g.get_speculative_stats()
    assert st["proposed"] >= st["accepted"] and st["corrections"] > 0


def test_ngram_speculation_equals_greedy(spec_dir):
    model = og.Model(spec_dir)
    plain, _ = generate(model, PROMPT, 60)
    for chained in (False, True):
        spec, g = generate(model, PROMPT, 60, ngram_size=3, max_draft_tokens=5, ngram_chained_lookup=chained)
        assert spec == plain
        st = g.get_speculative_stats()
        assert st["ngram_hits"] + st["ngram_misses"] > 0


def test_sampled_speculation_runs_and_respects_support(spec_dir, tmp_path):
    model = og.Model(with_draft(spec_dir, "draft.onnx", tmp_path, 2))
    seq, g = generate(model, PROMPT, 30, max_draft_tokens=4, do_sample=True, top_k=5, temperature=0.9, random_seed=11)
    assert len(seq) <= len(PROMPT) + 30 and g.get_speculative_stats()["rounds"] > 0
    seq2, _ = generate(model, PROMPT, 30, max_draft_tokens=4, do_sample=True, top_k=5, temperature=0.9, random_seed=11)
    assert seq == seq2, "same seed, same tokens"


def test_speculative_guards(spec_dir, tmp_path):
    model = og.Model(spec_dir)
    p = og.GeneratorParams(model)
    p.set_search_options(batch_size=2, max_length=30)
    p.set_speculative_options(ngram_size=3)
    with pytest.raises(RuntimeError, match="batch_size 1"):
        og.Generator(model, p)
    with pytest.raises(RuntimeError):
        p.set_speculative_options(max_draft_tokens=17)


# ------------------------------------------------------------------------------------------ host math
def test_ngram_index():
    ix = native.NGramIndex(3)
    ix.append(np.array([1, 2, 3, 4, 1, 2], dtype=np.int32))
    assert ix.propose(3, False) == [3, 4, 1]
    assert ix.propose(8, True)[:4] == [3, 4, 1, 2]
    ix.append(np.array([9, 1, 2], dtype=np.int32))
    assert ix.propose(2, False) == [9, 1], "the latest occurrence wins"
    assert native.NGramIndex(2).propose(3, False) == []
    with pytest.raises(RuntimeError):
        native.NGramIndex(1)


def test_verify_greedy_math():
    logits = np.full((4, 10), -5.0, dtype=np.float32)
    for i, t in enumerate([3, 7, 2, 9]):
        logits[i, t] = 1.0
    assert native.verify_greedy(np.array([3, 7, 2], dtype=np.int32), logits) == (3, [3, 7, 2, 9], True)
    assert native.verify_greedy(np.array([3, 1, 2], dtype=np.int32), logits) == (1, [3, 7], False)


def test_accept_probability_and_statistics():
    assert native.accept_probability(0.2, 0.4) == pytest.approx(0.5)
    assert native.accept_probability(0.5, 0.4) == 1.0
    assert native.accept_probability(0.0, 0.0) == 0.0
    # distribution equivalence: speculative sampling with a mismatched draft reproduces the target distribution
    vocab, n = 6, 4000
    rng = np.random.RandomState(0)
    target = rng.randn(2, vocab).astype(np.float32)
    q = np.exp(rng.randn(vocab)); q /= q.sum()
    p = native.SearchParams(); p.vocab_size, p.max_length, p.random_seed, p.eos_token_ids = vocab, 4, 5, [99]
    s = native.Search(p)
    counts = np.zeros(vocab)
    ids = np.arange(vocab, dtype=np.int32)
    for _ in range(n):
        d = int(np.searchsorted(np.cumsum(q), s.uniform(), side="right").clip(max=vocab - 1))
        acc, commit, _ = native.verify_sampled(np.array([d], dtype=np.int32), [(ids, q.astype(np.float32))], target, 0, 0.0, 1.0, s)
        counts[commit[0]] += 1
    want = np.exp(target[0] - target[0].max()); want /= want.sum()
    assert 0.5 * np.abs(counts / n - want).sum() < 0.04


def test_adaptive_k_and_cooldown():
    a = native.AdaptiveK(4, 2)
    assert a.k == 2 and a.min_k == 2
    for _ in range(12):
        a.record(a.k, a.k, a.k, a.k + 1, True, 1.0)
    assert a.k > 2 and a.increases > 0
    k_hi = a.k
    for _ in range(30):
        a.record(a.k, a.k, 0, 1, True, 1.0)
    assert a.k < k_hi and a.k >= 2
    fixed = native.AdaptiveK(4, 0)
    fixed.record(4, 4, 4, 5, True, 1.0)
    assert fixed.k == 4
    c = native.ZeroAcceptCooldown(True)
    for _ in range(3):
        assert not c.should_skip_round()
        c.record(4, 0)
    assert c.should_skip_round() and not c.should_skip_round() and c.skips == 1
    assert not native.ZeroAcceptCooldown(False).should_skip_round()


# ------------------------------------------------------------------------------------------------ inside the engine
def _paged(spec_dir, tmp_path, extra):
    """The target checkpoint with a paged-engine section and `extra` merged into its genai_config.json."""
    cfg = json.load(open(os.path.join(spec_dir, "genai_config.json")))
    cfg["engine"] = {"dynamic_batching": {"block_size": 4, "num_blocks": 256, "max_batch_size": 8, "max_scheduled_tokens": 64}}
    for k, v in extra.items():
        if k == "draft":
            dec = copy.deepcopy(cfg["model"]["decoder"])
            dec["filename"], dec["num_hidden_layers"] = v
            cfg["model"]["draft"] = dec
        else:
            cfg[k] = v
    out = str(tmp_path)
    os.makedirs(out, exist_ok=True)
    for f in os.listdir(spec_dir):
        if f != "genai_config.json" and not os.path.exists(os.path.join(out, f)):
            os.symlink(os.path.join(spec_dir, f), os.path.join(out, f))
    json.dump(cfg, open(os.path.join(out, "genai_config.json"), "w"))
    return out


def _engine_run(model, prompts, new_tokens, **search):
    engine = og.Engine(model)
    reqs, outs = [], {}
    for i, p in enumerate(prompts):
        gp = og.GeneratorParams(model)
        gp.set_search_options(max_length=len(p) + new_tokens, random_seed=7 + i, **search)
        r = og.Request(gp)
        r.add_tokens(np.asarray(p, dtype=np.int32))
        engine.add_request(r)
        reqs.append(r)
        outs[id(r)] = []
    guard = 0
    while engine.has_pending_requests():
        guard += 1
        assert guard < 4000
        r = engine.step()
        engine.core.check_invariants()
        if r is None:
            continue
        while r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r.is_turn_complete():
            engine.remove_request(r)
    assert engine.core.free_blocks == engine.options.num_blocks, "every block returns to the pool"
    return [outs[id(r)] for r in reqs], engine


ENGINE_PROMPTS = [PROMPT, [9, 61, 5, 17, 40, 3, 22, 9, 61, 5], [33, 33, 33, 33, 33, 33, 33], [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13],
                  [40, 3, 22, 9, 61, 5, 17, 40, 3, 22, 9, 61, 5, 17, 40, 3, 22]]


def test_engine_self_speculation_equals_plain_greedy(spec_dir, tmp_path):
    """A draft equal to the target inside the engine: every request of the batch accepts every proposal, and the token streams
    are those of the plain engine (reference semantics: src/speculative_decoding_strategy.cpp:460-792, batched here)."""
    plain, _ = _engine_run(og.Model(_paged(spec_dir, tmp_path / "plain", {})), ENGINE_PROMPTS, 24)
    model = og.Model(_paged(spec_dir, tmp_path / "self", {"draft": ("draft.onnx", 2), "speculative": {"max_draft_tokens": 4}}))
    spec, engine = _engine_run(model, ENGINE_PROMPTS, 24)
    assert spec == plain
    st = engine.spec.stats
    assert st["rounds"] > 0 and st["accepted"] == st["proposed"], st
    assert engine.step_count < sum(len(o) for o in plain) / 2, "several tokens per request and step"


def test_engine_weak_draft_and_ngram_still_equal_plain_greedy(spec_dir, tmp_path):
    plain, _ = _engine_run(og.Model(_paged(spec_dir, tmp_path / "plain", {})), ENGINE_PROMPTS, 24)
    weak = og.Model(_paged(spec_dir, tmp_path / "weak", {"draft": ("weak_draft.onnx", 1), "speculative": {"max_draft_tokens": 3}}))
    out, engine = _engine_run(weak, ENGINE_PROMPTS, 24)
    assert out == plain and engine.spec.stats["accepted"] < engine.spec.stats["proposed"]
    ngram = og.Model(_paged(spec_dir, tmp_path / "ngram", {"speculative": {"ngram_size": 3, "max_draft_tokens": 4}}))
    out, engine = _engine_run(ngram, ENGINE_PROMPTS, 24)
    assert out == plain and engine.spec is not None and engine.spec.stats["rounds"] > 0


def test_engine_speculation_with_sampling_is_reproducible_and_valid(spec_dir, tmp_path):
    """Sampled requests verify deterministic proposals by rejection sampling (accept d with probability p(d), else draw from p
    without d): same seeds give the same streams, every token lies in the top-k set of its step, lengths are respected."""
    model = og.Model(_paged(spec_dir, tmp_path / "s", {"draft": ("draft.onnx", 2), "speculative": {"max_draft_tokens": 3}}))
    a, _ = _engine_run(model, ENGINE_PROMPTS[:3], 16, do_sample=True, top_k=5, temperature=0.9)
    b, _ = _engine_run(model, ENGINE_PROMPTS[:3], 16, do_sample=True, top_k=5, temperature=0.9)
    assert a == b and all(len(o) == 16 or 96 in o for o in a)


def test_engine_speculation_with_grammar_equals_plain_constrained_decoding(tmp_path):
    """Requests under a JSON schema are given n-gram proposals too: rows after the first are masked from a cloned grammar cursor
    and the grammar advances over the accepted drafts; greedy output equals the engine's plain constrained output."""
    import json
    import onnxruntime_genai_b200 as og
    from helpers import tiny_model_dir
    d, _ = tiny_model_dir(str(tmp_path / "m"), std=0.3)
    schema = json.dumps({"type": "object", "properties": {"tags": {"type": "array", "items": {"enum": ["a", "b"]}, "maxItems": 8}},
                         "required": ["tags"], "additionalProperties": False})

    def run(spec):
        cfg = og.Config(d)
        if spec:
            cfg.overlay(json.dumps({"speculative": {"ngram_size": 2, "max_draft_tokens": 3}}))
        model = og.Model(cfg)
        tok = og.Tokenizer(model)
        eng = og.Engine(model)
        reqs = []
        for text in ('{"tags": ["a", "b", "a", "b", "a"]} {"tags": ["a", "b", "a", "b", "a"]} ', '{"tags": ["b", "b"]} '):
            p = og.GeneratorParams(model)
            ids = tok.encode(text)
            p.set_search_options(max_length=len(ids) + 60, do_sample=False)
            p.set_guidance("json_schema", schema)
            r = og.Request(p)
            r.add_tokens(ids)
            eng.add_request(r)
            reqs.append(r)
        outs = [[] for _ in reqs]
        for _ in range(400):
            if not eng.has_pending_requests():
                break
            eng.step()
            for i, r in enumerate(reqs):
                while r.has_unseen_tokens():
                    outs[i].append(r.get_unseen_token())
        texts = []
        for o in outs:
            while o and o[-1] in (0, 1):
                o.pop()
            texts.append(tok.decode(np.asarray(o, dtype=np.int32)))
        return texts, (eng.spec.stats if eng.spec is not None else None)

    plain, _ = run(False)
    spec, stats = run(True)
    assert spec == plain
    for t in spec:
        assert set(json.loads(t)) == {"tags"}
    assert stats["rounds"] > 0 and stats["proposed"] > 0
