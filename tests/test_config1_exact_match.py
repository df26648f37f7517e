"""BASELINE config 1: tiny Llama on CPU in fp32, batch 2, 32-token prompts, greedy, 32 new tokens.
The runtime's tokens must equal the independent NumPy oracle's exactly."""
import numpy as np

import onnxruntime_genai_b200 as og
from oracle import NumpyLlama


def test_tiny_llama_greedy_matches_oracle(tiny_llama_dir):
    model = og.Model(tiny_llama_dir)
    assert model.device_type == "cpu" and model.type == "llama"
    prompts = np.random.RandomState(1).randint(0, 32000, size=(2, 32)).astype(np.int32)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=128, batch_size=2, do_sample=False)
    gen = og.Generator(model, params)
    gen.append_tokens(prompts)
    steps = 0
    while not gen.is_done() and steps < 32:
        gen.generate_next_token()
        steps += 1
    oracle = NumpyLlama(tiny_llama_dir)
    for b in range(2):
        want = oracle.greedy(prompts[b].tolist(), 32)
        got = gen.get_sequence(b).tolist()
        assert got == want, f"row {b}: first mismatch at {next(i for i, (x, y) in enumerate(zip(got, want)) if x != y)}"


def test_logits_close_to_oracle(tiny_llama_dir):
    model = og.Model(tiny_llama_dir)
    prompt = np.random.RandomState(3).randint(0, 32000, size=(1, 17)).astype(np.int32)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=64)
    gen = og.Generator(model, params)
    gen.append_tokens(prompt)
    got = gen.get_logits().reshape(-1)
    want = NumpyLlama(tiny_llama_dir).logits(prompt[0].tolist())
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
