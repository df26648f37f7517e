"""Every decoder family the exporter names, as a Hugging Face checkpoint (config.json + safetensors) through create_model and
the Generator, against the family's own implementation in `transformers` with a small random configuration (reference:
src/python/py/models/builder.py create_model dispatches on `architectures[0]`; one builder class per family under builders/)."""
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.builder import create_model

transformers = pytest.importorskip("transformers")
VOCAB = 83
COMMON = dict(vocab_size=VOCAB, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, intermediate_size=96,
              max_position_embeddings=128, bos_token_id=0, eos_token_id=VOCAB - 1, pad_token_id=0, tie_word_embeddings=False)

# family -> (config class, model class, extra configuration)
FAMILIES = {
    "llama": ("LlamaConfig", "LlamaForCausalLM", dict(rope_theta=500000.0)),
    "llama_bias": ("LlamaConfig", "LlamaForCausalLM", dict(attention_bias=True, mlp_bias=True, head_dim=32)),
    "mistral": ("MistralConfig", "MistralForCausalLM", dict(sliding_window=6, head_dim=16)),
    "qwen2": ("Qwen2Config", "Qwen2ForCausalLM", dict()),
    "qwen3": ("Qwen3Config", "Qwen3ForCausalLM", dict(head_dim=32)),
    "phi3": ("Phi3Config", "Phi3ForCausalLM", dict(num_key_value_heads=4, pad_token_id=0)),
    "phi": ("PhiConfig", "PhiForCausalLM", dict(num_key_value_heads=4, partial_rotary_factor=0.5)),
    "gemma": ("GemmaConfig", "GemmaForCausalLM", dict(head_dim=16, tie_word_embeddings=True)),
    "gemma2": ("Gemma2Config", "Gemma2ForCausalLM", dict(head_dim=16, sliding_window=6, query_pre_attn_scalar=24, tie_word_embeddings=True)),
    "gemma3_text": ("Gemma3TextConfig", "Gemma3ForCausalLM", dict(head_dim=16, sliding_window=6, query_pre_attn_scalar=24, tie_word_embeddings=True)),
    "granite": ("GraniteConfig", "GraniteForCausalLM", dict(embedding_multiplier=3.0, logits_scaling=2.0, residual_multiplier=0.4, attention_multiplier=0.2)),
    "olmo": ("OlmoConfig", "OlmoForCausalLM", dict(clip_qkv=None)),
    "olmo2": ("Olmo2Config", "Olmo2ForCausalLM", dict()),
    "exaone4": ("Exaone4Config", "Exaone4ForCausalLM", dict(num_hidden_layers=4, sliding_window=6, sliding_window_pattern=2, head_dim=16)),
    "exaone4_global": ("Exaone4Config", "Exaone4ForCausalLM", dict(sliding_window=None, sliding_window_pattern=4, layer_types=["full_attention"] * 3, head_dim=16)),
    "smollm3": ("SmolLM3Config", "SmolLM3ForCausalLM", dict(no_rope_layers=[1, 0, 1], use_sliding_window=False)),
    "nemotron": ("NemotronConfig", "NemotronForCausalLM", dict(partial_rotary_factor=0.5, head_dim=16)),
    "ernie4_5": ("Ernie4_5Config", "Ernie4_5ForCausalLM", dict(head_dim=16, use_bias=False)),
    "hunyuan_v1_dense": ("HunYuanDenseV1Config", "HunYuanDenseV1ForCausalLM", dict(head_dim=16)),
    "gpt2": ("GPT2Config", "GPT2LMHeadModel", dict(n_embd=64, n_head=4, n_layer=3, n_positions=128)),
    "helium": ("HeliumConfig", "HeliumForCausalLM", dict(head_dim=16)),
    "olmoe": ("OlmoeConfig", "OlmoeForCausalLM", dict(num_experts=4, num_experts_per_tok=2, intermediate_size=48, norm_topk_prob=False)),
    "qwen3_moe": ("Qwen3MoeConfig", "Qwen3MoeForCausalLM", dict(num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48, head_dim=32, norm_topk_prob=True,
                                                                decoder_sparse_step=1, mlp_only_layers=[])),
    "granitemoe": ("GraniteMoeConfig", "GraniteMoeForCausalLM", dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=48, embedding_multiplier=2.0,
                                                                     logits_scaling=2.0, residual_multiplier=0.5, attention_multiplier=0.2)),
    "phimoe": ("PhimoeConfig", "PhimoeForCausalLM", dict(num_local_experts=4, num_experts_per_tok=2, intermediate_size=48)),
    "lfm2": ("Lfm2Config", "Lfm2ForCausalLM", dict(layer_types=["conv", "full_attention", "conv"], conv_L_cache=3, block_ff_dim=96, block_auto_adjust_ff_dim=False,
                                                   tie_word_embeddings=True)),
}


def _randomise(m, std=0.08):
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n.lower() or n.endswith((".ln_1.weight", ".ln_2.weight", "ln_f.weight")):
                centre = 1.0 if float(p.detach().float().mean()) > 0.5 else 0.0      # weights stored as the scale, or as its offset from one
                p.copy_(centre + 0.1 * torch.randn_like(p)) if n.endswith("weight") else p.copy_(0.1 * torch.randn_like(p))
            elif n.endswith("mlp.gate.weight") or "router" in n:
                p.copy_(torch.randn_like(p) * 0.5)
            else:
                p.copy_(torch.randn_like(p) * std)
    return m.float().eval()


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_checkpoint_matches_the_family_implementation(family, tmp_path):
    from safetensors.torch import save_file
    cfg_cls, model_cls, extra = FAMILIES[family]
    if not hasattr(transformers, cfg_cls) or not hasattr(transformers, model_cls):
        pytest.skip(f"transformers has no {model_cls}")
    torch.manual_seed(0)
    kw = {**COMMON, **extra}
    cfg = getattr(transformers, cfg_cls)(**kw)
    if hasattr(cfg, "_attn_implementation"):
        cfg._attn_implementation = "eager"
    m = _randomise(getattr(transformers, model_cls)(cfg))
    sd = {}
    for k, v in m.state_dict().items():          # tied tensors are stored once
        if not (getattr(cfg, "tie_word_embeddings", False) and k == "lm_head.weight"):
            sd[k] = v.detach().clone().contiguous()
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file(sd, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = [model_cls]
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    model = og.Model(out)
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 14)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(4):
        with torch.no_grad():
            want = m(torch.tensor([seq])).logits[0, -1].float().numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=3e-4)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break


def _generate_and_compare(tmp_path, cfg_dict, sd, m):
    from safetensors.torch import save_file
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file({k: v.detach().clone().contiguous() for k, v in sd.items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps(cfg_dict))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    model = og.Model(out)
    ids = np.random.RandomState(1).randint(1, VOCAB - 1, size=(1, 11)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=24)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(3):
        with torch.no_grad():
            want = m(torch.tensor([seq])).logits[0, -1].float().numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=3e-4)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break
    return model


def test_internlm2_layout(tmp_path):
    """InternLM2 keeps llama's mathematics under its own names, with q / k / v packed per key-value group in one `wqkv` matrix
    (reference: builders/internlm.py).  The checkpoint here is a llama model re-laid that way."""
    torch.manual_seed(0)
    cfg = transformers.LlamaConfig(**COMMON)
    m = _randomise(transformers.LlamaForCausalLM(cfg))
    D, Hq, Hkv = 16, 4, 2
    r = Hq // Hkv
    sd = {}
    for k, v in m.state_dict().items():
        k2 = (k.replace("model.embed_tokens.", "model.tok_embeddings.").replace(".input_layernorm.", ".attention_norm.").replace(".post_attention_layernorm.", ".ffn_norm.")
              .replace(".mlp.gate_proj.", ".feed_forward.w1.").replace(".mlp.up_proj.", ".feed_forward.w3.").replace(".mlp.down_proj.", ".feed_forward.w2.")
              .replace(".self_attn.o_proj.", ".attention.wo.").replace("lm_head.", "output."))
        if ".self_attn.q_proj." in k:
            base = k[: k.index("self_attn")]
            q = v.view(Hkv, r, D, -1)
            kk = m.state_dict()[base + "self_attn.k_proj.weight"].view(Hkv, 1, D, -1)
            vv = m.state_dict()[base + "self_attn.v_proj.weight"].view(Hkv, 1, D, -1)
            sd[base + "attention.wqkv.weight"] = torch.cat([q, kk, vv], 1).reshape((Hq + 2 * Hkv) * D, -1)
        elif ".self_attn.k_proj." in k or ".self_attn.v_proj." in k:
            continue
        else:
            sd[k2] = v
    d = cfg.to_dict()
    d.update(architectures=["InternLM2ForCausalLM"], model_type="internlm2", bias=False)
    model = _generate_and_compare(tmp_path, d, sd, m)
    assert model.type == "internlm2"


def test_chatglm_layout(tmp_path):
    """ChatGLM: its own configuration keys (`num_layers`, `ffn_hidden_size`, `multi_query_group_num`, `kv_channels`, `padded_vocab_size`,
    `seq_length`, `rope_ratio`), fused `query_key_value` (+ bias) and `dense_h_to_4h` matrices, half of each head rotated in interleaved
    pairs (reference: builders/chatglm.py).  The oracle is transformers' Glm model, which is the same network under llama-style names."""
    if not hasattr(transformers, "GlmForCausalLM"):
        pytest.skip("transformers has no GlmForCausalLM")
    torch.manual_seed(0)
    cfg = transformers.GlmConfig(**{**COMMON, "head_dim": 16}, attention_bias=True, partial_rotary_factor=0.5)
    m = _randomise(transformers.GlmForCausalLM(cfg))
    st = m.state_dict()
    sd = {"transformer.embedding.word_embeddings.weight": st["model.embed_tokens.weight"], "transformer.encoder.final_layernorm.weight": st["model.norm.weight"],
          "transformer.output_layer.weight": st["lm_head.weight"], "transformer.rotary_pos_emb.inv_freq": torch.zeros(4)}
    for i in range(cfg.num_hidden_layers):
        a, b = f"model.layers.{i}.", f"transformer.encoder.layers.{i}."
        sd[b + "input_layernorm.weight"] = st[a + "input_layernorm.weight"]
        sd[b + "post_attention_layernorm.weight"] = st[a + "post_attention_layernorm.weight"]
        sd[b + "self_attention.query_key_value.weight"] = torch.cat([st[a + f"self_attn.{n}_proj.weight"] for n in "qkv"], 0)
        sd[b + "self_attention.query_key_value.bias"] = torch.cat([st[a + f"self_attn.{n}_proj.bias"] for n in "qkv"], 0)
        sd[b + "self_attention.dense.weight"] = st[a + "self_attn.o_proj.weight"]
        sd[b + "mlp.dense_h_to_4h.weight"] = st[a + "mlp.gate_up_proj.weight"]
        sd[b + "mlp.dense_4h_to_h.weight"] = st[a + "mlp.down_proj.weight"]
    d = dict(architectures=["ChatGLMModel"], model_type="chatglm", num_layers=cfg.num_hidden_layers, hidden_size=64, ffn_hidden_size=96, num_attention_heads=4,
             multi_query_attention=True, multi_query_group_num=2, kv_channels=16, padded_vocab_size=VOCAB, seq_length=128, layernorm_epsilon=cfg.rms_norm_eps,
             add_qkv_bias=True, add_bias_linear=False, rope_ratio=1.0, rmsnorm=True, eos_token_id=VOCAB - 1, pad_token_id=0)
    model = _generate_and_compare(tmp_path, d, sd, m)
    assert model.type == "chatglm" and model.arch.rotary_interleaved and model.arch.rotary_dim == 8


@pytest.mark.gpu
@pytest.mark.parametrize("family", ["gemma3_text", "smollm3", "nemotron", "hunyuan_v1_dense", "olmoe", "olmo2", "exaone4", "ernie4_5", "lfm2", "gpt2"])
def test_checkpoint_on_the_gpu(family, tmp_path):
    """The same checkpoints in bf16 on the CUDA path (per-layer rotary caches in the fused decode step, the squared-ReLU kernel, the
    q / k norm variants), against the fp32 logits of the family's implementation."""
    from safetensors.torch import save_file
    cfg_cls, model_cls, extra = FAMILIES[family]
    if not hasattr(transformers, cfg_cls) or not hasattr(transformers, model_cls):
        pytest.skip(f"transformers has no {model_cls}")
    torch.manual_seed(0)
    kw = {**COMMON, **extra, "hidden_size": 256, "intermediate_size": 384}      # 4 heads of 64: the head size the attention kernels take
    for key, val in (("head_dim", 64), ("n_embd", 256), ("block_ff_dim", 384)):
        if key in kw:
            kw[key] = val
    if family == "olmoe":
        kw["intermediate_size"] = 64
    cfg = getattr(transformers, cfg_cls)(**kw)
    if hasattr(cfg, "_attn_implementation"):
        cfg._attn_implementation = "eager"
    m = _randomise(getattr(transformers, model_cls)(cfg), std=0.04)     # four times the width of the CPU cases: keep the attention scores in the same range
    sd = {k: v.detach().clone().contiguous() for k, v in m.state_dict().items()
          if not (getattr(cfg, "tie_word_embeddings", False) and k == "lm_head.weight")}
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file(sd, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = [model_cls]
    (src / "config.json").write_text(json.dumps(d))
    import copy
    m16 = copy.deepcopy(m).to(torch.bfloat16)
    out = str(tmp_path / "out")
    create_model(str(src), out, "bf16", "cuda")
    model = og.Model(out)
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 14)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(4):
        with torch.no_grad():
            want = m(torch.tensor([seq])).logits[0, -1].float().numpy()
        got = np.asarray(g.get_logits(), dtype=np.float32).reshape(-1)
        # the yardstick for bf16 rounding: the family's own implementation run in bf16 against itself in fp32
        with torch.no_grad():
            own = np.abs(m16(torch.tensor([seq])).logits[0, -1].float().numpy() - want).max()
        assert np.abs(got - want).max() < max(0.04 * max(1.0, np.abs(want).max()), 2.5 * own), (family, np.abs(got - want).max(), own)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break


@pytest.mark.parametrize("wrapper", ["gemma3", "mistral3", "llava"])
def test_text_decoder_of_a_multimodal_wrapper(wrapper, tmp_path):
    """`...ForConditionalGeneration` checkpoints: the decoder's settings sit under `text_config`, its weights under `model.language_model.`;
    create_model exports the text decoder (as the reference's builder does for these architectures) and text prompts match the wrapper."""
    text = dict(vocab_size=VOCAB, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, intermediate_size=96,
                max_position_embeddings=128, head_dim=16)
    vision = dict(hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2, image_size=28, patch_size=14)
    if wrapper == "gemma3":
        cfg = transformers.Gemma3Config(text_config=dict(**text, sliding_window=6, query_pre_attn_scalar=24), vision_config=vision, mm_tokens_per_image=1,
                                        image_token_index=VOCAB - 1)
        cls, kind = transformers.Gemma3ForConditionalGeneration, "gemma3_text"
    elif wrapper == "mistral3":
        cfg = transformers.Mistral3Config(text_config=dict(**text, model_type="mistral", sliding_window=None), vision_config=dict(**vision, head_dim=16),
                                          image_token_index=VOCAB - 1)
        cls, kind = transformers.Mistral3ForConditionalGeneration, "mistral"
    else:
        cfg = transformers.LlavaConfig(text_config=dict(**text, model_type="llama"), vision_config=dict(**vision, model_type="clip_vision_model"),
                                       image_token_index=VOCAB - 1)
        cls, kind = transformers.LlavaForConditionalGeneration, "llama"
    torch.manual_seed(0)
    m = _randomise(cls(cfg))
    sd = {k: v for k, v in m.state_dict().items() if not (k == "lm_head.weight" and getattr(cfg.get_text_config(), "tie_word_embeddings", False))}
    d = cfg.to_dict()
    d["architectures"] = [cls.__name__]
    model = _generate_and_compare(tmp_path, d, sd, m)
    assert model.type == kind


def test_qwen3_vl_text_decoder_and_interleaved_positions(tmp_path):
    """Qwen3-VL's decoder: qwen3 with three position components per token whose rotary pairs alternate t h w t h w ... (reference:
    builders/qwen.py Qwen3VLTextModel).  A text prompt, then a prompt with explicit [3, batch, sequence] positions whose components
    differ, against `transformers`."""
    if not hasattr(transformers, "Qwen3VLForConditionalGeneration"):
        pytest.skip("transformers has no Qwen3VLForConditionalGeneration")
    cfg = transformers.Qwen3VLConfig(
        text_config=dict(vocab_size=VOCAB, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=3, intermediate_size=96,
                         max_position_embeddings=128, head_dim=16, bos_token_id=0, eos_token_id=VOCAB - 1, pad_token_id=0,
                         rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "mrope_interleaved": True, "rope_theta": 10000.0}),
        vision_config=dict(depth=1, hidden_size=32, out_hidden_size=64, num_heads=2, intermediate_size=48, patch_size=14, spatial_merge_size=2,
                           temporal_patch_size=2, deepstack_visual_indexes=[0], num_position_embeddings=16),
        image_token_id=80, video_token_id=81, vision_start_token_id=78, vision_end_token_id=79, tie_word_embeddings=False)
    torch.manual_seed(0)
    m = _randomise(transformers.Qwen3VLForConditionalGeneration(cfg))
    d = cfg.to_dict()
    d["architectures"] = ["Qwen3VLForConditionalGeneration"]
    model = _generate_and_compare(tmp_path, d, dict(m.state_dict()), m)
    assert model.type == "qwen3_vl" and model.arch.mrope_interleaved and model.arch.mrope_section == [2, 3, 3] and model.arch.qk_norm
    ids = np.random.RandomState(2).randint(1, 70, size=(1, 10)).astype(np.int32)
    pos = np.stack([np.arange(10), np.array([0, 1, 2, 2, 2, 3, 3, 3, 5, 6]), np.array([0, 1, 2, 3, 4, 2, 3, 4, 5, 6])])[:, None, :].astype(np.int64)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=24)
    g = og.Generator(model, p)
    g.set_inputs({"input_ids": ids, "position_ids": pos})
    with torch.no_grad():
        want = m(input_ids=torch.tensor(ids.astype(np.int64)), position_ids=torch.from_numpy(pos)).logits[0, -1].float().numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=3e-4)


def test_phi4_multimodal_text_decoder(tmp_path):
    """Phi-4-multimodal: create_model exports the text decoder (packed qkv / gate-up projections, three quarters of each head rotated);
    the image and audio towers' tensors in the checkpoint are ignored.  Text prompts match the family's implementation."""
    if not hasattr(transformers, "Phi4MultimodalForCausalLM"):
        pytest.skip("transformers has no Phi4MultimodalForCausalLM")
    cfg = transformers.Phi4MultimodalConfig(vocab_size=VOCAB, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                                            num_key_value_heads=2, max_position_embeddings=128, original_max_position_embeddings=128,
                                            partial_rotary_factor=0.75, pad_token_id=0, bos_token_id=1, eos_token_id=VOCAB - 1,
                                            tie_word_embeddings=False,
                                            vision_config=dict(hidden_size=32, intermediate_size=48, num_hidden_layers=1, num_attention_heads=2,
                                                               image_size=28, patch_size=14, crop_size=28),
                                            audio_config=dict(hidden_size=32, intermediate_size=48, num_blocks=1, num_attention_heads=2, input_size=16,
                                                              nemo_conv_channels=32, depthwise_separable_out_channel=16))
    torch.manual_seed(0)
    m = _randomise(transformers.Phi4MultimodalForCausalLM(cfg))
    d = cfg.to_dict()
    d["architectures"] = ["Phi4MultimodalForCausalLM"]
    model = _generate_and_compare(tmp_path, d, dict(m.state_dict()), m)
    assert model.type == "phi3" and model.arch.rotary_dim == 12
