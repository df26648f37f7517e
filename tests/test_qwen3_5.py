"""Qwen3.5 text checkpoints (reference builder: src/python/py/models/builders/qwen.py, Qwen35TextModel): gated-delta-net layers beside
attention layers whose q_proj carries a per-head output gate, zero-centred RMS norms, partial rotary embedding given through
`rope_parameters`.  The oracle is the family's own implementation in `transformers` with a small random configuration; the checkpoint
goes through config.json + safetensors -> create_model like a real one, once under the plain decoder names and once under the
multimodal wrapper's (`text_config`, `model.language_model.` prefix)."""
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.builder import create_model

hf_modeling = pytest.importorskip("transformers.models.qwen3_5.modeling_qwen3_5")
hf_config = pytest.importorskip("transformers.models.qwen3_5.configuration_qwen3_5")

VOCAB = 97


def _hf_model(seed=0):
    torch.manual_seed(seed)
    cfg = hf_config.Qwen3_5TextConfig(
        vocab_size=VOCAB, hidden_size=64, intermediate_size=96, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
        linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_num_key_heads=2, linear_num_value_heads=4,
        max_position_embeddings=128, layer_types=["linear_attention", "full_attention", "linear_attention", "full_attention"],
        bos_token_id=0, eos_token_id=VOCAB - 1, pad_token_id=0, tie_word_embeddings=False)
    m = hf_modeling.Qwen3_5ForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 3 + 0.5))
            elif n.endswith("dt_bias"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith("linear_attn.norm.weight"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif "norm" in n:
                p.copy_(0.1 * torch.randn_like(p))       # zero-centred: the stored weight is the offset from one
            else:
                p.copy_(torch.randn_like(p) * 0.08)
    return cfg, m


def _export(tmp_path, cfg_dict, sd, name):
    from safetensors.torch import save_file
    src = tmp_path / (name + "_hf")
    os.makedirs(src)
    save_file({k: v.detach().contiguous() for k, v in sd.items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps(cfg_dict))
    out = str(tmp_path / name)
    create_model(str(src), out, "fp32", "cpu")
    return out


def _hf_logits(m, ids):
    with torch.no_grad():
        return m(torch.tensor([ids], dtype=torch.long)).logits[0].float()


def _check(model, m, seed):
    ids = np.random.RandomState(seed).randint(1, VOCAB - 1, size=(1, 15)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(5):
        np.testing.assert_allclose(g.get_logits().reshape(-1), _hf_logits(m, seq)[-1].numpy(), rtol=3e-3, atol=3e-4)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break


def test_text_checkpoint_matches_the_family_implementation(tmp_path):
    cfg, m = _hf_model()
    d = cfg.to_dict()
    d["architectures"] = ["Qwen3_5ForCausalLM"]
    out = _export(tmp_path, d, m.state_dict(), "t")
    model = og.Model(out)
    a = model.arch
    assert a.attn_output_gate and a.qk_norm and a.has_linear_layers and a.rotary_dim == 8
    _check(model, m, 0)


def test_decoder_of_the_multimodal_wrapper(tmp_path):
    """`Qwen3_5ForConditionalGeneration` checkpoints: the decoder's settings under `text_config`, its weights under `model.language_model.`;
    the vision tower's tensors are ignored by the text export."""
    cfg, m = _hf_model(seed=1)
    sd = {}
    for k, v in m.state_dict().items():
        sd[("model.language_model." + k[len("model."):]) if k.startswith("model.") else k] = v
    sd["model.visual.patch_embed.proj.weight"] = torch.zeros(4, 3, 2, 2)
    d = {"architectures": ["Qwen3_5ForConditionalGeneration"], "model_type": "qwen3_5", "text_config": cfg.to_dict(),
         "vision_config": {"depth": 1, "hidden_size": 8}, "tie_word_embeddings": False}
    out = _export(tmp_path, d, sd, "w")
    _check(og.Model(out), m, 1)


def test_mtp_head_of_the_checkpoint(tmp_path):
    """`mtp.*` tensors of a Qwen3.5 checkpoint (reference: src/python/py/models/builders/qwen_mtp.py) exported with `mtp_head=1` as a
    head directory for MtpGenerator: zero-centred pre-projection norms are stored with their offset applied, the head's layer is an
    attention layer, and self-speculation with it reproduces plain greedy decoding of the hybrid main model."""
    cfg, m = _hf_model(seed=2)
    sd = dict(m.state_dict())
    g = torch.Generator().manual_seed(5)
    H = cfg.hidden_size
    ref_layer = "model.layers.1."                 # an attention layer of the main stack lends the head its shapes
    for k, v in list(sd.items()):
        if k.startswith(ref_layer):
            sd["mtp.layers.0." + k[len(ref_layer):]] = (0.1 * torch.randn(v.shape, generator=g)) if "norm" in k else 0.08 * torch.randn(v.shape, generator=g)
    sd["mtp.fc.weight"] = 0.08 * torch.randn(H, 2 * H, generator=g)
    sd["mtp.norm.weight"] = 0.1 * torch.randn(H, generator=g)
    sd["mtp.pre_fc_norm_embedding.weight"] = 0.1 * torch.randn(H, generator=g)
    sd["mtp.pre_fc_norm_hidden.weight"] = 0.1 * torch.randn(H, generator=g)
    d = cfg.to_dict()
    d["architectures"] = ["Qwen3_5ForCausalLM"]
    from safetensors.torch import save_file
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file({k: v.detach().contiguous() for k, v in sd.items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu", {"mtp_head": 1})
    head_dir = os.path.join(out, "mtp")
    z = np.load(os.path.join(head_dir, "mtp_extra.npz"))
    np.testing.assert_allclose(z["mtp.enorm.weight"], 1 + sd["mtp.pre_fc_norm_embedding.weight"].numpy(), rtol=1e-6)
    np.testing.assert_allclose(z["mtp.fc.weight"], sd["mtp.fc.weight"].numpy(), rtol=1e-6)
    model = og.Model(out)
    _check(model, m, 3)                           # the main model ignores the extra tensors
    head = og.Model(head_dir)
    assert head.arch.num_layers == 1 and head.arch.attn_output_gate and not head.arch.has_linear_layers
    prompt = np.random.RandomState(5).randint(1, VOCAB - 1, size=(1, 9)).astype(np.int32)

    def run(make):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=30)
        gen = make(p)
        gen.append_tokens(prompt)
        while not gen.is_done():
            gen.generate_next_token()
        return gen.get_sequence(0).tolist()

    def spec(p):
        p.set_speculative_options(max_draft_tokens=3)
        return og.MtpGenerator(model, head_dir, p)

    assert run(spec) == run(lambda p: og.Generator(model, p))
