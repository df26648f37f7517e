"""Feature paths end to end on the GPU (bf16 kernels, CUDA graphs, device-side verification and masks): speculative decoding
with a draft model and with n-gram lookup, the MTP head, Multi-LoRA adapters, constrained decoding in the Generator and the
engine.  bf16 results of differently shaped launches may differ in the last bits, so "equals greedy" is checked as: every
emitted token is within a small margin of the best logit of a plain teacher-forced run."""
import copy
import json
import os
import re

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from dense_reference import logits as dense_logits
from helpers import make_tokenizer
from onnxruntime_genai_b200 import ops
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model, random_state_dict

pytestmark = pytest.mark.gpu

ARCH = dict(model_type="llama", vocab_size=1024, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
            intermediate_size=512, context_length=512, bos_token_id=0, eos_token_id=1023, pad_token_id=0)
PROMPT = [5, 17, 40, 3, 22, 9, 61, 5, 17, 40, 3]


def assert_near_greedy(model, prompt, seq, margin=0.15):
    """Teacher-forces `seq` through a plain generator: each generated token must be (nearly) the best one of its step."""
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(seq) + 1)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([prompt], dtype=np.int32))
    for t in seq[len(prompt):]:
        lg = g.get_logits()[0, 0]
        assert lg[t] >= lg.max() - margin * lg.std(), f"token {t} is not a greedy choice (logit {lg[t]:.3f}, best {lg.max():.3f})"
        forced = np.full((1, lg.shape[0]), -1e9, dtype=np.float32)
        forced[0, t] = 0
        g.set_logits(forced)
        g.generate_next_token()


def run(gen):
    while not gen.is_done():
        n = gen.token_count()
        gen.generate_next_token()
        assert gen.token_count() == n + 1
    return gen.get_sequence(0).tolist()


@pytest.fixture(scope="module")
def spec_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("gpu_spec"))
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=3, std=0.08)
    export_model(copy.deepcopy(arch), d, "bf16", "cuda", state_dict=sd)
    export_model(copy.deepcopy(arch), d, "bf16", "cuda", state_dict=sd, filename="draft.onnx", write_config=False)
    cfg = json.load(open(os.path.join(d, "genai_config.json")))
    plain = str(tmp_path_factory.mktemp("gpu_plain"))
    for f in os.listdir(d):
        if f != "genai_config.json":
            os.symlink(os.path.join(d, f), os.path.join(plain, f))
    json.dump(cfg, open(os.path.join(plain, "genai_config.json"), "w"))      # the same weights without the draft section
    dec = copy.deepcopy(cfg["model"]["decoder"])
    dec["filename"] = "draft.onnx"
    cfg["model"]["draft"] = dec
    json.dump(cfg, open(os.path.join(d, "genai_config.json"), "w"))
    return d, plain


def test_draft_model_speculation_on_gpu(spec_dir):
    with_draft, plain = spec_dir
    model = og.Model(with_draft)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(PROMPT) + 40)
    p.set_speculative_options(max_draft_tokens=4)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([PROMPT], dtype=np.int32))
    seq = run(g)
    st = g.get_speculative_stats()
    assert st["rounds"] > 0 and st["acceptance_rate"] > 0.8 and st["tokens_per_round"] > 2.0
    assert_near_greedy(og.Model(plain), PROMPT, seq)
    # sampled verification on the device: same seed, same tokens
    outs = []
    for _ in range(2):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(PROMPT) + 30, do_sample=True, top_k=5, temperature=0.9, random_seed=11)
        p.set_speculative_options(max_draft_tokens=4)
        g = og.Generator(model, p)
        g.append_tokens(np.asarray([PROMPT], dtype=np.int32))
        outs.append(run(g))
    assert outs[0] == outs[1] and len(outs[0]) > len(PROMPT)
    ops.check_kernel_status()


def test_engine_speculation_on_gpu(spec_dir, tmp_path):
    """Speculative decoding inside the continuous-batching engine on the GPU: several requests, a draft equal to the target.
    One packed verify forward per step serves the whole batch; most proposals are accepted (bf16 launches of different shapes
    may flip a near-tie) and every emitted token is a greedy choice of the plain model."""
    with_draft, plain = spec_dir
    cfg = json.load(open(os.path.join(with_draft, "genai_config.json")))
    cfg["engine"] = {"dynamic_batching": {"block_size": 16, "num_blocks": 256, "max_batch_size": 8, "max_scheduled_tokens": 256}}
    cfg["speculative"] = {"max_draft_tokens": 4}
    d = str(tmp_path)
    for f in os.listdir(with_draft):
        if f != "genai_config.json":
            os.symlink(os.path.join(with_draft, f), os.path.join(d, f))
    json.dump(cfg, open(os.path.join(d, "genai_config.json"), "w"))
    model = og.Model(d)
    engine = og.Engine(model)
    assert engine.spec is not None
    prompts = [PROMPT, PROMPT[3:] + [7, 7, 7], [100, 200, 300, 400, 500, 600], list(range(30, 75))]
    reqs, outs = [], {}
    for pr in prompts:
        gp = og.GeneratorParams(model)
        gp.set_search_options(max_length=len(pr) + 24)
        r = og.Request(gp)
        r.add_tokens(np.asarray(pr, dtype=np.int32))
        engine.add_request(r)
        reqs.append(r)
        outs[id(r)] = []
    while engine.has_pending_requests():
        r = engine.step()
        if r is None:
            continue
        while r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r.is_turn_complete():
            engine.remove_request(r)
    ops.check_kernel_status()
    engine.core.check_invariants()
    st = engine.spec.stats
    assert st["rounds"] > 0 and st["accepted"] >= 0.8 * st["proposed"], st
    assert engine.step_count < sum(len(o) for o in outs.values()) / 2, "several tokens per request and step"
    ref_model = og.Model(plain)
    for pr, r in zip(prompts, reqs):
        assert len(outs[id(r)]) == 24 or 1023 in outs[id(r)]
        assert_near_greedy(ref_model, pr, pr + outs[id(r)])


def test_ngram_speculation_on_gpu(spec_dir):
    model = og.Model(spec_dir[1])
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(PROMPT) + 60)
    p.set_speculative_options(ngram_size=3, max_draft_tokens=5)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([PROMPT], dtype=np.int32))
    seq = run(g)
    st = g.get_speculative_stats()
    assert st["ngram_hits"] + st["ngram_misses"] > 0
    assert_near_greedy(model, PROMPT, seq)


def test_mtp_head_on_gpu(tmp_path):
    from onnxruntime_genai_b200.mtp import export_mtp_head
    arch = ArchConfig(**{**ARCH, "model_type": "qwen3", "qk_norm": True})
    main_dir, head_dir = str(tmp_path / "main"), str(tmp_path / "head")
    export_model(copy.deepcopy(arch), main_dir, "bf16", "cuda", state_dict=random_state_dict(arch, seed=4, std=0.08))
    export_mtp_head(copy.deepcopy(arch), head_dir, "bf16", "cuda", seed=7, std=0.08)
    model = og.Model(main_dir)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(PROMPT) + 32)
    p.set_speculative_options(max_draft_tokens=3)
    g = og.MtpGenerator(model, head_dir, p)
    g.append_tokens(np.asarray([PROMPT], dtype=np.int32))
    seq = run(g)
    assert g.get_speculative_stats()["rounds"] > 0
    assert_near_greedy(model, PROMPT, seq)


def test_lora_adapters_on_gpu(tmp_path):
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=5, std=0.05)
    d = str(tmp_path / "m")
    export_model(copy.deepcopy(arch), d, "bf16", "cuda", state_dict=sd)
    model = og.Model(d)
    g_ = torch.Generator().manual_seed(1)
    t, merged = {}, {k: v.clone() for k, v in sd.items()}
    for layer in range(2):
        for proj, (k, n) in {"q_proj": (256, 256), "v_proj": (256, 128), "o_proj": (256, 256), "up_proj": (256, 512), "down_proj": (512, 256)}.items():
            a, b = torch.randn(k, 8, generator=g_) * 0.1, torch.randn(8, n, generator=g_) * 0.1
            mod = "self_attn" if proj in ("q_proj", "v_proj", "o_proj") else "mlp"
            t[f"model.layers.{layer}.{mod}.{proj}.lora_A.weight"] = a.numpy()
            t[f"model.layers.{layer}.{mod}.{proj}.lora_B.weight"] = b.numpy()
            merged[f"model.layers.{layer}.{mod}.{proj}.weight"] = merged[f"model.layers.{layer}.{mod}.{proj}.weight"] + (a @ b).t() * 2.0
    t["lora_alpha"] = np.float32(2.0)
    np.savez(str(tmp_path / "a.npz"), **t)
    adapters = og.Adapters(model)
    adapters.load(str(tmp_path / "a.npz"), "a")
    prompt = np.random.RandomState(0).randint(0, 1023, size=(1, 14)).astype(np.int32)

    def logits(active):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=40)
        g = og.Generator(model, p)
        if active:
            g.set_active_adapter(adapters, active)
        g.append_tokens(prompt)
        g.generate_next_token()           # one decode step with the adapter too
        return g.get_logits().reshape(-1), int(g.get_next_tokens()[0])

    base, _ = logits(None)
    got, tok = logits("a")
    want = dense_logits(arch, merged, prompt[0].tolist() + [tok])[-1].numpy()
    assert np.abs(got - want).max() < 0.08 * want.std() + 0.03
    assert np.abs(got - base).max() > 0.05
    model.decoder.active_adapter = None
    ops.check_kernel_status()


def test_engine_batch_mixes_lora_adapters_on_gpu(tmp_path):
    """Requests with adapter a, with none and with adapter b share engine steps on the GPU (tokens grouped by adapter, two
    grouped low-rank GEMMs + a combine per adapted projection); each gets the tokens a generator with that adapter produces."""
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=5, std=0.05)
    d = str(tmp_path / "m")
    export_model(copy.deepcopy(arch), d, "bf16", "cuda", state_dict=sd, paged=True, block_size=16, num_blocks=128, max_batch_size=8)
    model = og.Model(d)
    adapters = og.Adapters(model)
    for name, seed in (("a", 1), ("b", 2)):
        g_ = torch.Generator().manual_seed(seed)
        t = {}
        for layer in range(2):
            for proj, (k, n) in {"q_proj": (256, 256), "v_proj": (256, 128), "o_proj": (256, 256), "up_proj": (256, 512), "down_proj": (512, 256)}.items():
                t[f"model.layers.{layer}.x.{proj}.lora_A.weight"] = (torch.randn(k, 8 if name == "a" else 4, generator=g_) * 0.15).numpy()
                t[f"model.layers.{layer}.x.{proj}.lora_B.weight"] = (torch.randn(8 if name == "a" else 4, n, generator=g_) * 0.15).numpy()
        np.savez(str(tmp_path / f"{name}.npz"), **t)
        adapters.load(str(tmp_path / f"{name}.npz"), name)
    rs = np.random.RandomState(3)
    prompts = [rs.randint(0, 1023, size=n).astype(np.int32) for n in (17, 30, 9)]
    names = ["a", None, "b"]
    eng = og.Engine(model)
    reqs = []
    for prompt, name in zip(prompts, names):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(prompt) + 6, do_sample=False)
        r = og.Request(p)
        r.add_tokens(prompt)
        if name:
            r.set_active_adapter(adapters, name)
        eng.add_request(r)
        reqs.append(r)
    got = [[] for _ in reqs]
    for _ in range(100):
        if not eng.has_pending_requests():
            break
        eng.step()
        for i, r in enumerate(reqs):
            while r.has_unseen_tokens():
                got[i].append(r.get_unseen_token())
    for r in reqs:
        eng.remove_request(r)
    want = []
    for prompt, name in zip(prompts, names):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(prompt) + 6, do_sample=False)
        g = og.Generator(model, p)
        model.decoder.active_adapter = None
        if name:
            g.set_active_adapter(adapters, name)
        g.append_tokens(prompt.reshape(1, -1))
        while not g.is_done():
            g.generate_next_token()
        want.append(g.get_sequence(0)[len(prompt):].tolist())
    model.decoder.active_adapter = None
    ops.check_kernel_status()
    assert all(len(x) == 6 for x in got)
    assert [x[0] for x in got] == [x[0] for x in want]                 # the first token of every request
    assert sum(a_ == b_ for a_, b_ in zip(got, want)) >= 2, (got, want)   # whole continuations (bf16: a near-tie may flip one)
    assert want[0] != want[1] or want[2] != want[1]


@pytest.fixture(scope="module")
def text_model(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("gpu_text"))
    vocab = make_tokenizer(d)
    arch = ArchConfig(**{**ARCH, "vocab_size": vocab, "eos_token_id": 1, "pad_token_id": 1})
    export_model(arch, d, "bf16", "cuda", seed=0, std=0.1, paged=True, block_size=16, num_blocks=256, max_batch_size=8)
    return og.Model(d)


def test_constrained_decoding_on_gpu(text_model):
    tok = og.Tokenizer(text_model)
    schema = json.dumps({"type": "object", "properties": {"name": {"type": "string", "maxLength": 8}, "age": {"type": "integer"}},
                         "required": ["name", "age"], "additionalProperties": False})
    ids = tok.encode("profile:")
    p = og.GeneratorParams(text_model)
    p.set_search_options(max_length=len(ids) + 120, do_sample=True, top_k=20, temperature=1.0, random_seed=1)
    p.set_guidance("json_schema", schema)
    g = og.Generator(text_model, p)
    g.append_tokens(ids)
    out = run(g)[len(ids):]
    while out and out[-1] in (0, 1):
        out.pop()
    obj = json.loads(tok.decode(out))
    assert set(obj) == {"name", "age"} and isinstance(obj["age"], int)
    # the engine applies grammar masks per request next to unconstrained requests (no look-ahead for those steps)
    engine = og.Engine(text_model)
    reqs = []
    for seed, (kind, data) in enumerate([("regex", r"(ab|cd){2}"), ("lark_grammar", 'start: "true" | "false"'), (None, None)]):
        p = og.GeneratorParams(text_model)
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
        while r is not None and r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r is not None and r.is_turn_complete():
            engine.remove_request(r)
    assert re.fullmatch(r"(ab|cd){2}", tok.decode(outs[id(reqs[0])]))
    assert tok.decode(outs[id(reqs[1])]) in ("true", "false")
    ops.check_kernel_status()
