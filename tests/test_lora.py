"""Multi-LoRA adapters (reference: test/python/test_onnxruntime_genai_api.py:712-800): loading, activating and
switching adapters must equal running the model with the low-rank update merged into the dense weights."""
import copy

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from dense_reference import logits as dense_logits
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model, random_state_dict

ARCH = dict(model_type="llama", vocab_size=131, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
            intermediate_size=128, context_length=128, bos_token_id=0, eos_token_id=130, pad_token_id=0)


def make_adapter(path, seed, rank=4, scale=2.0):
    g = torch.Generator().manual_seed(seed)
    t, merged = {}, {}
    for layer in range(2):
        for proj, (k, n) in {"q_proj": (64, 64), "v_proj": (64, 32), "o_proj": (64, 64), "up_proj": (64, 128), "down_proj": (128, 64)}.items():
            a = torch.randn(k, rank, generator=g) * 0.3      # [in, r]
            b = torch.randn(rank, n, generator=g) * 0.3      # [r, out]
            mod = "self_attn" if proj in ("q_proj", "v_proj", "o_proj") else "mlp"
            t[f"model.layers.{layer}.{mod}.{proj}.lora_A.weight"] = a.numpy()
            t[f"model.layers.{layer}.{mod}.{proj}.lora_B.weight"] = b.numpy()
            merged[f"model.layers.{layer}.{mod}.{proj}.weight"] = (a @ b).t() * scale   # delta on the [out, in] weight
    t["lora_alpha"] = np.float32(scale)
    np.savez(path, **t)
    return merged


def test_adapters_equal_merged_weights(tmp_path):
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=5, std=0.15)
    d = str(tmp_path / "m")
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    deltas = {name: make_adapter(str(tmp_path / f"{name}.npz"), seed) for name, seed in (("a", 1), ("b", 2))}
    adapters = og.Adapters(model)
    adapters.load(str(tmp_path / "a.npz"), "a")
    adapters.load(str(tmp_path / "b.npz"), "b")
    with pytest.raises(RuntimeError):
        adapters.load(str(tmp_path / "a.npz"), "a")
    prompt = np.random.RandomState(0).randint(0, 130, size=(1, 14)).astype(np.int32)

    def run(active):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=40)
        g = og.Generator(model, p)
        if active:
            g.set_active_adapter(adapters, active)
        g.append_tokens(prompt)
        return g.get_logits().reshape(-1)

    base = run(None)
    np.testing.assert_allclose(base, dense_logits(arch, sd, prompt[0].tolist())[-1].numpy(), rtol=2e-3, atol=2e-4)
    for name in ("a", "b", "a"):
        got = run(name)
        merged = {k: v.clone() for k, v in sd.items()}
        for k, dv in deltas[name].items():
            merged[k] = merged[k] + dv
        want = dense_logits(arch, merged, prompt[0].tolist())[-1].numpy()
        np.testing.assert_allclose(got, want, rtol=3e-3, atol=5e-4)
        assert np.abs(got - base).max() > 1e-2, "the adapter must change the logits"
    with pytest.raises(RuntimeError):
        adapters.unload("a")            # still active
    model.decoder.active_adapter = None
    adapters.unload("a")
    with pytest.raises(RuntimeError):
        adapters.unload("missing")
