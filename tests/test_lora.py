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


def _lora_model(tmp_path, device="cpu", precision="fp32"):
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=5, std=0.15)
    d = str(tmp_path / "m")
    export_model(copy.deepcopy(arch), d, precision, device, state_dict=sd, paged=True, block_size=16, num_blocks=64, max_batch_size=8)
    return og.Model(d)


def test_onnx_adapter_container_round_trip_and_load(tmp_path):
    """The reference's adapter container (.onnx_adapter): written and read back bit for bit, and loaded by Adapters with the
    same effect as the .npz form of the same tensors."""
    from onnxruntime_genai_b200.utils.onnx_adapter import read_adapter, write_adapter
    model = _lora_model(tmp_path)
    make_adapter(str(tmp_path / "a.npz"), 1)
    z = np.load(str(tmp_path / "a.npz"))
    tensors = {k: np.asarray(z[k]) for k in z.files}
    write_adapter(str(tmp_path / "a.onnx_adapter"), tensors, adapter_version=3, model_version=2)
    back, meta = read_adapter(str(tmp_path / "a.onnx_adapter"))
    assert meta == {"format_version": 1, "adapter_version": 3, "model_version": 2}
    assert set(back) == set(tensors) and all(np.array_equal(back[k][0], tensors[k]) for k in tensors)
    adapters = og.Adapters(model)
    adapters.load(str(tmp_path / "a.npz"), "npz")
    adapters.load(str(tmp_path / "a.onnx_adapter"), "fb")
    prompt = np.random.RandomState(0).randint(0, 130, size=(1, 9)).astype(np.int32)
    outs = []
    for name in ("npz", "fb"):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=20)
        g = og.Generator(model, p)
        g.set_active_adapter(adapters, name)
        g.append_tokens(prompt)
        outs.append(g.get_logits().reshape(-1))
    np.testing.assert_array_equal(outs[0], outs[1])
    with pytest.raises(RuntimeError):
        (tmp_path / "bad.onnx_adapter").write_bytes(b"\x01\x02")
        adapters.load(str(tmp_path / "bad.onnx_adapter"), "bad")


def _engine_tokens(model, adapters, prompts, names, max_new=10):
    eng = og.Engine(model)
    reqs = []
    for prompt, name in zip(prompts, names):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(prompt) + max_new, do_sample=False)
        r = og.Request(p)
        r.add_tokens(np.asarray(prompt, dtype=np.int32))
        if name is not None:
            r.set_active_adapter(adapters, name)
        eng.add_request(r)
        reqs.append(r)
    out = [[] for _ in reqs]
    for _ in range(400):
        if not eng.has_pending_requests():
            break
        eng.step()
        for i, r in enumerate(reqs):
            while r.has_unseen_tokens():
                out[i].append(r.get_unseen_token())
    for r in reqs:
        eng.remove_request(r)
    return out


def test_engine_batch_mixes_adapters_per_request(tmp_path):
    """Two adapters and no adapter in ONE engine batch give each request the tokens it gets when it runs alone."""
    model = _lora_model(tmp_path)
    adapters = og.Adapters(model)
    for name, seed in (("a", 1), ("b", 2)):
        make_adapter(str(tmp_path / f"{name}.npz"), seed)
        adapters.load(str(tmp_path / f"{name}.npz"), name)
    rs = np.random.RandomState(3)
    prompts = [rs.randint(0, 130, size=n).tolist() for n in (7, 12, 5, 9)]
    names = ["a", None, "b", "a"]
    together = _engine_tokens(model, adapters, prompts, names)
    alone = [_engine_tokens(model, adapters, [p], [n])[0] for p, n in zip(prompts, names)]
    assert together == alone
    base = [_engine_tokens(model, adapters, [p], [None])[0] for p in prompts]
    assert base[0] != alone[0] and base[2] != alone[2] and base[1] == alone[1]     # the adapters do change the output
