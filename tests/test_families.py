"""Model families through export -> load -> generate, against the independent dense reference
(tests/dense_reference.py).  Each family is a set of ArchConfig flags: biases, q/k norms, soft-capping,
sliding windows on some layers, attention sinks, LayerNorm + partial rotary, embedding / logit scales,
post-sublayer norms, mixture of experts."""
import copy

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from dense_reference import logits as dense_logits
from onnxruntime_genai_b200.models.arch import ArchConfig, from_hf_config
from onnxruntime_genai_b200.models.builder import export_model, random_state_dict

BASE = dict(vocab_size=211, hidden_size=64, num_layers=3, num_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
            context_length=256, bos_token_id=0, eos_token_id=210, pad_token_id=0)

FAMILIES = {
    "llama": dict(model_type="llama"),
    "llama3_rope": dict(model_type="llama", rope_theta=500000.0,
                        rope_scaling={"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                      "original_max_position_embeddings": 64}),
    "mistral_window": dict(model_type="mistral", sliding_window=8),
    "qwen2": dict(model_type="qwen2", attn_bias=True),
    "qwen3": dict(model_type="qwen3", qk_norm=True, tie_embeddings=True),
    "phi3": dict(model_type="phi3", num_kv_heads=4),
    "phi": dict(model_type="phi", layernorm=True, partial_rotary_factor=0.5, attn_bias=True, o_bias=True, mlp_bias=True,
                lm_head_bias=True, activation="gelu", num_kv_heads=4),
    "phi_parallel": dict(model_type="phi", layernorm=True, partial_rotary_factor=0.5, attn_bias=True, o_bias=True, mlp_bias=True,
                         lm_head_bias=True, activation="gelu", num_kv_heads=4, mlp_gated=False, parallel_block=True),
    "gpt2": dict(model_type="gpt2", layernorm=True, attn_bias=True, o_bias=True, mlp_bias=True, activation="gelu", num_kv_heads=4,
                 mlp_gated=False, learned_positions=True, tie_embeddings=True),
    "lfm2_hybrid": dict(model_type="lfm2", qk_norm=True, tie_embeddings=True, conv_L_cache=3,
                        layer_types=["conv", "full_attention", "conv"]),
    "lfm2_conv_bias": dict(model_type="lfm2", qk_norm=True, conv_L_cache=4, conv_bias=True, num_layers=4,
                           layer_types=["conv", "conv", "full_attention", "conv"]),
    "mixtral": dict(model_type="mixtral", moe_style="standard", num_experts=4, experts_per_token=2, intermediate_size=64),
    "qwen3_moe": dict(model_type="qwen3_moe", moe_style="standard", moe_norm_topk=False, qk_norm=True, num_experts=8, experts_per_token=3,
                      intermediate_size=64),
    "phimoe": dict(model_type="phimoe", moe_style="standard", moe_sparse_mixer=True, moe_jitter_eps=0.05, layernorm=True, attn_bias=True,
                   o_bias=True, lm_head_bias=True, num_experts=4, experts_per_token=2, intermediate_size=64),
    "gemma2": dict(model_type="gemma2", activation="gelu", norm_offset=1.0, embed_scale=8.0, post_sublayer_norms=True, softcap=20.0,
                   final_logit_softcap=15.0, sliding_window=8, sliding_layers=[0, 2], attn_scale=0.2, tie_embeddings=True),
    "gemma3": dict(model_type="gemma3_text", activation="gelu", norm_offset=1.0, embed_scale=8.0, post_sublayer_norms=True, qk_norm=True,
                   sliding_window=8, sliding_layers=[0, 1], tie_embeddings=True),
    "granite": dict(model_type="granite", residual_multiplier=0.5, logits_scale=0.25, embed_scale=3.0, attn_scale=0.3),
    "interleaved_rope": dict(model_type="chatglm", rotary_interleaved=True, partial_rotary_factor=0.5, attn_bias=True),
    "gptoss": dict(model_type="gptoss", attn_bias=True, o_bias=True, mlp_bias=True, attn_sinks=True, sliding_window=8,
                   sliding_layers=[0, 2], num_experts=4, experts_per_token=2, intermediate_size=64),
}


@pytest.mark.parametrize("family", sorted(FAMILIES))
def test_family_logits_and_decode_match_dense_reference(family, tmp_path):
    arch = ArchConfig(**{**BASE, **FAMILIES[family]})
    sd = random_state_dict(arch, seed=11, std=0.15)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    assert model.type == arch.model_type
    a2 = model.arch
    for f in ("norm_eps", "layernorm", "qk_norm", "attn_bias", "o_bias", "mlp_bias", "softcap", "sliding_window", "attn_sinks",
              "activation", "num_experts", "experts_per_token", "post_sublayer_norms", "rotary_interleaved", "lm_head_bias",
              "mlp_gated", "parallel_block", "learned_positions", "conv_L_cache", "conv_bias", "moe_style", "moe_norm_topk", "moe_sparse_mixer", "moe_jitter_eps"):
        assert getattr(a2, f) == pytest.approx(getattr(arch, f)), f
    assert a2.intermediate_size == arch.intermediate_size and a2.rotary_dim == arch.rotary_dim and a2.layer_types == arch.layer_types
    prompt = np.random.RandomState(4).randint(0, arch.vocab_size - 1, size=(1, 23)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=40)
    g = og.Generator(model, p)
    g.append_tokens(prompt)
    want = dense_logits(arch, sd, prompt[0].tolist())[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=2e-4)
    # decode steps (KV cache, windows crossing the cache) against full recompute
    ids = prompt[0].tolist()
    for _ in range(6):
        g.generate_next_token()
        ids.append(int(g.get_next_tokens()[0]))
        if g.is_done():
            break
        want = dense_logits(arch, sd, ids)[-1].numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)


def test_hf_config_mapping():
    a = from_hf_config({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": 64, "num_attention_heads": 4,
                        "num_key_value_heads": 2, "num_hidden_layers": 2, "intermediate_size": 128, "vocab_size": 100,
                        "max_position_embeddings": 512, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "eos_token_id": [5, 6]})
    assert a.model_type == "qwen2" and a.attn_bias and a.head_dim == 16 and a.eos_list() == [5, 6] and a.norm_eps == 1e-6
    g = from_hf_config({"architectures": ["GptOssForCausalLM"], "model_type": "gpt_oss", "hidden_size": 64, "num_attention_heads": 8,
                        "num_key_value_heads": 2, "head_dim": 16, "num_hidden_layers": 4, "intermediate_size": 64, "vocab_size": 100,
                        "num_local_experts": 8, "num_experts_per_tok": 2, "sliding_window": 16,
                        "layer_types": ["sliding_attention", "full_attention"] * 2})
    assert g.model_type == "gptoss" and g.num_experts == 8 and g.attn_sinks and g.sliding_layers == [0, 2]


def test_int4_checkpoint_roundtrip(tmp_path):
    """MatMulNBits int4 block-32 (asymmetric, uint4 zero points) export -> load reproduces the dequantised weights."""
    from onnxruntime_genai_b200.models.builder import dequantize_int4_block32, quantize_int4_block32
    w = torch.randn(48, 96) * 0.1
    for sym in (False, True):
        q, s, zp = quantize_int4_block32(w, symmetric=sym)
        assert q.shape == (48, 3, 16) and q.dtype == torch.uint8 and (zp is None) == sym
        wd = dequantize_int4_block32(q, s, zp, 48, 96)
        assert (wd - w).abs().max() < (s.max() * (0.51 if not sym else 1.01))
    arch = ArchConfig(**{**BASE, "model_type": "phi3", "num_kv_heads": 4})
    sd = random_state_dict(arch, seed=2, std=0.1)
    export_model(copy.deepcopy(arch), str(tmp_path), "int4", "cpu", state_dict=sd)
    model = og.Model(str(tmp_path))
    q, s, zp = quantize_int4_block32(torch.cat([sd[f"model.layers.0.self_attn.{n}_proj.weight"] for n in "qkv"], 0))
    want = dequantize_int4_block32(q, s.to(torch.float16).float(), zp, q.shape[0], 64)
    got_w = model.decoder.layers[0].qkv_w
    got_w = got_w.dequantize() if hasattr(got_w, "dequantize") else got_w.float()   # int4 weights stay packed for the dequant GEMM
    torch.testing.assert_close(got_w, want, rtol=2e-2, atol=1e-3)
    prompt = np.arange(1, 12, dtype=np.int32).reshape(1, -1)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=20)
    g = og.Generator(model, p)
    g.append_tokens(prompt)
    fp = dense_logits(arch, sd, prompt[0].tolist())[-1].numpy()
    got = g.get_logits().reshape(-1)
    assert np.corrcoef(got, fp)[0, 1] > 0.9, "int4 logits must stay close to the fp32 model"


def test_int4_tied_quantized_embedding(tmp_path):
    """int4 + tied embeddings: one int4 tensor is both the LM head (MatMulNBits) and the embedding table
    (GatherBlockQuantized over its rows); no dense embedding is stored."""
    from onnxruntime_genai_b200.models.builder import dequantize_int4_block32, quantize_int4_block32
    from onnxruntime_genai_b200.ops.w4 import QuantizedEmbedding
    from onnxruntime_genai_b200.utils import onnx_proto as op
    arch = ArchConfig(**{**BASE, "model_type": "qwen3", "qk_norm": True, "tie_embeddings": True})
    sd = random_state_dict(arch, seed=9, std=0.1)
    for sym in (False, True):
        d = str(tmp_path / f"sym{int(sym)}")
        export_model(copy.deepcopy(arch), d, "int4", "cpu", state_dict=sd, int4_tied_embeddings=True, int4_symmetric=sym)
        names = op.LoadedModel(d + "/model.onnx").names()
        assert "model.embed_tokens.weight" not in names and "lm_head.MatMul.weight_Q4" in names
        model = og.Model(d)
        q, s, zp = quantize_int4_block32(sd["model.embed_tokens.weight"], symmetric=sym)
        want = dequantize_int4_block32(q, s.to(torch.float16).float(), zp, arch.vocab_size, arch.hidden_size)
        torch.testing.assert_close(model.decoder.embed.float(), want, rtol=2e-2, atol=1e-3)
        # the table object used on a GPU restates the same rows
        qe = QuantizedEmbedding(q.reshape(arch.vocab_size, -1), s.to(torch.float16).view(arch.vocab_size, -1),
                                zp.reshape(arch.vocab_size, -1) if zp is not None else None, arch.vocab_size, arch.hidden_size)
        torch.testing.assert_close(qe.dequantize(), want, rtol=2e-2, atol=1e-3)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=20)
        g = og.Generator(model, p)
        g.append_tokens(np.arange(1, 12, dtype=np.int32).reshape(1, -1))
        fp = dense_logits(arch, sd, list(range(1, 12)))[-1].numpy()
        assert np.corrcoef(g.get_logits().reshape(-1), fp)[0, 1] > 0.9


@pytest.mark.parametrize("family", ["llama", "lfm2_hybrid"])
def test_beam_search_cache_sharing_matches_full_recompute(family, tmp_path):
    """Beam reordering permutes block tables and copies blocks on write; every row's logits must still equal a
    full recompute of that row's token sequence (prompt ending inside a block, rows crossing block boundaries).
    The hybrid family keeps its convolution inputs in the same paged slots, so its state follows the beams too."""
    arch = ArchConfig(**{**BASE, **FAMILIES[family]})
    sd = random_state_dict(arch, seed=21, std=0.3)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    prompt = np.random.RandomState(8).randint(0, arch.vocab_size - 1, size=(2, 13)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=48, batch_size=2, num_beams=3, num_return_sequences=1, early_stopping=False)
    g = og.Generator(model, p)
    g.append_tokens(prompt)
    moved = False
    for step in range(24):
        g.generate_next_token()
        if g.is_done():
            break
        logits = g.get_logits()
        for r in range(6):
            seq = g.get_sequence(r).tolist()
            want = dense_logits(arch, sd, seq)[-1].numpy()
            np.testing.assert_allclose(logits[r, 0], want, rtol=2e-3, atol=3e-4, err_msg=f"step {step} row {r}")
        moved = moved or g.state._tbl is not None
    assert moved, "the beams never diverged: the test did not exercise the shared-block path"
    # the pool never leaks: every block is either referenced or free
    st = g.state
    assert int((st._ref > 0).sum()) + len(st._free) == st.rows * st.blocks_per_row


def test_mxfp4_expert_round_trip_and_model(tmp_path):
    """MXFP4 (FP4 e2m1 + e8m0 block scales) experts: quantiser / dequantiser agree, the QMoE export loads, and its
    logits follow the bf16-free fp32 model built from the dequantised experts."""
    from onnxruntime_genai_b200.models.builder import dequantize_mxfp4, quantize_mxfp4
    w = torch.randn(64, 96, generator=torch.Generator().manual_seed(3)) * 0.3
    packed, codes = quantize_mxfp4(w)
    assert packed.shape == (96, 32) and codes.shape == (64, 3) and packed.dtype == torch.uint8
    back = dequantize_mxfp4(packed, codes, 64, 96)
    # the scale exponent is rounded to nearest, so a block maximum may clip at 6 * scale: error <= (6 * sqrt(2) - 6) * scale;
    # inside the grid the largest half step is 1 * scale
    scale = torch.pow(2.0, codes.float() - 127.0).repeat_interleave(32, dim=1)
    assert bool(((back - w).abs() <= scale * 2.5 + 1e-6).all())
    assert float(((back - w).abs() / scale).mean()) < 0.3
    arch = ArchConfig(**{**BASE, **FAMILIES["gptoss"]})
    sd = random_state_dict(arch, seed=5, std=0.15)
    d = str(tmp_path / "q")
    export_model(copy.deepcopy(arch), d, "int4", "cpu", state_dict=sd)
    model = og.Model(d)
    assert model.arch.num_experts == 4 and model.arch.intermediate_size == arch.intermediate_size
    # reference: the same network with every quantised tensor replaced by its dequantised value
    from onnxruntime_genai_b200.models.builder import dequantize_int4_block32, quantize_int4_block32
    sd_q = dict(sd)
    for k, v in sd.items():
        if k.endswith(("mlp.experts.gate_up_proj", "mlp.experts.down_proj")):
            sd_q[k] = torch.stack([dequantize_mxfp4(*quantize_mxfp4(v[e].float()), v.shape[1], v.shape[2]) for e in range(v.shape[0])])
    lw = model.decoder.layers[0]
    np.testing.assert_allclose(lw.exp_down_w.float().numpy(), sd_q["model.layers.0.mlp.experts.down_proj"].numpy(), rtol=0, atol=1e-6)


def _read_fp4_records(packed: torch.Tensor, N: int, K: int, half: bool) -> torch.Tensor:
    """Restates on the host what csrc/gemm_fp4.cu does with a packed expert: thread = weight row reads 8 words and
    2 multiplier bytes of a 4352-byte record.  bf16 form: pair p of word j is `(word >> 4p)` (low nibbles of the two 16-bit
    halves), words in k order, the e2m1 value * 2^-126 multiplied by the bf16 whose exponent field is the multiplier byte.
    fp16 form: record word 2q + b holds k = 32b + 8q .. + 8, element i < 4 in nibble 2i and element 4 + i in nibble 2i + 1;
    the e2m1 value times 2^(byte - 6 - 127)."""
    KB, tiles = packed.shape[0], packed.shape[1]
    rec = packed.view(KB, tiles, 128 * 34)
    nib = rec[:, :, :128 * 32].reshape(KB, tiles, 128, 8, 4).to(torch.int64)
    words = nib[..., 0] | (nib[..., 1] << 8) | (nib[..., 2] << 16) | (nib[..., 3] << 24)           # [KB, tiles, 128, 8]
    mul = rec[:, :, 128 * 32:].reshape(KB, tiles, 128, 2).to(torch.int64)
    grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float64)
    out = torch.zeros(tiles * 128, KB * 64, dtype=torch.float64)
    for j in range(8):
        if half:
            q, blk = j >> 1, j & 1
            m = mul[..., blk]
            s = torch.pow(2.0, m.double() - 127.0 - 6.0)
            for i in range(8):
                c = (words[..., j] >> (8 * i if i < 4 else 8 * (i - 4) + 4)) & 0xF
                val = grid[c & 7] * torch.where(c >= 8, -1.0, 1.0) * s
                out.view(tiles, 128, KB, 64)[:, :, :, 32 * blk + 8 * q + i] = val.permute(1, 2, 0)
            continue
        m = mul[..., 0 if j < 4 else 1]
        s = torch.where(m > 0, torch.pow(2.0, m.double() - (127.0 + 126.0)), torch.zeros((), dtype=torch.float64))
        for pr in range(4):
            u = words[..., j] >> (4 * pr)
            for second, sh in ((0, 0), (1, 16)):
                c = (u >> sh) & 0xF
                val = grid[c & 7] * torch.where(c >= 8, -1.0, 1.0) * s                               # [KB, tiles, 128]
                k = j * 8 + pr * 2 + second
                out.view(tiles, 128, KB, 64)[:, :, :, k] = val.permute(1, 2, 0)
    return out[:N, :K].float()


def test_fp4_expert_packing_matches_the_qmoe_tensors():
    """The record layout the grouped FP4 GEMM streams, read back the way the kernel reads it, equals the plain
    dequantisation of the QMoE tensors (codes [E, K, N/2], e8m0 scales [E, N, K/32]); N is padded to 128 rows."""
    from onnxruntime_genai_b200.models.builder import dequantize_mxfp4, quantize_mxfp4
    from onnxruntime_genai_b200.ops.fp4 import Fp4Experts, unpack_qmoe_fp4
    E, N, K = 3, 160, 192
    g = torch.Generator().manual_seed(9)
    w = torch.randn(E, N, K, generator=g) * 0.2
    packs = [quantize_mxfp4(w[e]) for e in range(E)]
    q, sc = torch.stack([a for a, _ in packs]), torch.stack([b for _, b in packs])
    # every code at least once, the subnormal 0.5 and both zeros included
    q[0, 0, :8] = torch.tensor([0x10, 0x32, 0x54, 0x76, 0x98, 0xBA, 0xDC, 0xFE], dtype=torch.uint8)
    codes = unpack_qmoe_fp4(q)
    assert Fp4Experts.fits_fp16(codes, sc) and Fp4Experts.from_codes(codes, sc, "cpu").half
    for half in (False, True):
        fe = Fp4Experts.from_codes(codes, sc, "cpu", half=half)
        assert fe.packed.shape == (E, K // 64, 2, 4352) and fe.shape == (E, N, K) and fe.half == half
        for e in range(E):
            want = dequantize_mxfp4(q[e], sc[e], N, K)
            np.testing.assert_array_equal(fe.dequantize(e).numpy(), want.numpy())
            np.testing.assert_array_equal(_read_fp4_records(fe.packed[e], N, K, half).numpy(), want.numpy())
    assert not Fp4Experts.supported(torch.tensor([200], dtype=torch.uint8), K) and not Fp4Experts.supported(sc, 96)
    tiny = sc.clone()
    tiny[0, 0, 0] = 90                                # 2^-37: outside the fp16 form, fine for the bf16 form
    assert not Fp4Experts.fits_fp16(codes, tiny) and not Fp4Experts.from_codes(codes, tiny, "cpu").half
    zeros = codes.clone()
    zeros[0, 0, :32] &= 8                              # a block of signed zeros may carry any scale
    assert Fp4Experts.fits_fp16(zeros, tiny)


def test_longrope_switches_caches_and_rebuilds_the_kv_cache(tmp_path):
    """Phi-3 long-context RoPE: short-factor caches within the original context length, long-factor caches (and a
    rebuilt KV cache) once the sequence grows past it."""
    half = 8
    arch = ArchConfig(**{**BASE, "model_type": "phi3", "num_kv_heads": 4, "context_length": 128,
                         "rope_scaling": {"rope_type": "longrope", "original_max_position_embeddings": 32,
                                          "short_factor": [1.0 + 0.02 * i for i in range(half)],
                                          "long_factor": [1.5 + 0.3 * i for i in range(half)]}})
    sd = random_state_dict(arch, seed=13, std=0.15)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    assert model.decoder.cos_small is not None and model.decoder.rope_original_context == 32
    prompt = np.random.RandomState(6).randint(0, arch.vocab_size - 1, size=(1, 27)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=60)
    g = og.Generator(model, p)
    g.append_tokens(prompt)
    ids = prompt[0].tolist()
    np.testing.assert_allclose(g.get_logits().reshape(-1), dense_logits(arch, sd, ids)[-1].numpy(), rtol=2e-3, atol=3e-4)
    for _ in range(12):          # crosses 32 tokens on the way
        g.generate_next_token()
        ids.append(int(g.get_next_tokens()[0]))
        if g.is_done():
            break
        want = dense_logits(arch, sd, ids)[-1].numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4, err_msg=f"length {len(ids)}")
    assert len(ids) > 33, "the sequence must cross the original context length"


def test_hybrid_model_rewind_and_continue(tmp_path):
    """Rewinding a hybrid model needs no state snapshot: the convolution reads earlier positions from the paged cache."""
    arch = ArchConfig(**{**BASE, **FAMILIES["lfm2_conv_bias"]})
    sd = random_state_dict(arch, seed=12, std=0.15)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=64)
    g = og.Generator(model, p)
    ids = [3, 9, 27, 81, 32, 96, 77, 20, 60]
    g.append_tokens(np.asarray([ids], dtype=np.int32))
    for _ in range(5):
        g.generate_next_token()
    g.rewind_to(6)
    g.append_tokens(np.asarray([[5, 6]], dtype=np.int32))
    want = dense_logits(arch, sd, ids[:6] + [5, 6])[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)


def test_int8_kv_cache_tracks_the_full_precision_cache(tmp_path):
    """kvCacheQuantizationBits=8 (a provider option of the decoder session): keys and values are stored as int8 rows with one
    scale per token and head; logits stay close to the unquantised cache through prefill, decode and a rewind."""
    from helpers import tiny_model_dir
    d, arch = tiny_model_dir(str(tmp_path), std=0.3)
    prompt = np.random.RandomState(3).randint(2, arch.vocab_size, size=(2, 21)).astype(np.int32)

    def run(bits):
        cfg = og.Config(d)
        if bits:
            cfg.append_provider("cpu")
            cfg.set_provider_option("cpu", "kvCacheQuantizationBits", str(bits))
        model = og.Model(cfg)
        assert model.kv_bits == (bits or 16)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=48, batch_size=2)
        g = og.Generator(model, p)
        g.append_tokens(prompt)
        outs = [g.get_logits().copy()]
        for _ in range(4):
            forced = np.full((2, arch.vocab_size), -1e9, dtype=np.float32)
            forced[:, 7] = 0
            g.set_logits(forced)
            g.generate_next_token()
            outs.append(g.get_logits().copy())
        return g, outs

    g8, q = run(8)
    assert g8.state.kv.full.dtype == torch.int8 and g8.state.kv.full.shape[-1] == arch.head_dim + 16
    _, f = run(0)
    for a, b in zip(q, f):
        assert np.abs(a - b).max() < 0.12 * b.std() + 0.02 and np.corrcoef(a.reshape(-1), b.reshape(-1))[0, 1] > 0.999
        assert np.abs(a - b).max() > 0          # the cache really is quantised
    with pytest.raises(RuntimeError, match="not supported"):
        cfg = og.Config(d)
        cfg.append_provider("cpu")
        cfg.set_provider_option("cpu", "kvCacheQuantizationBits", "4")
        og.Model(cfg)


def test_snapshot_state_and_staged_hidden_states(tmp_path):
    from helpers import tiny_model_dir
    d, arch = tiny_model_dir(str(tmp_path))
    model = og.Model(d)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([[2, 3, 4, 5]], dtype=np.int32))
    before = g.get_logits().copy()
    assert g.snapshot_state() == 4
    for _ in range(3):
        g.generate_next_token()
    g.rewind_to(4)
    g.append_tokens(np.asarray([[9]], dtype=np.int32))
    g.rewind_to(3)
    g.append_tokens(np.asarray([[5]], dtype=np.int32))
    np.testing.assert_allclose(g.get_logits(), before, rtol=1e-5, atol=1e-6)
    hs = np.random.RandomState(0).randn(1, 1, arch.hidden_size).astype(np.float32)
    g.set_hidden_states(hs)
    np.testing.assert_array_equal(g.get_input("hidden_states"), hs)


def test_multimodal_rope_positions(tmp_path):
    """Qwen2-VL style decoder: with ordinary positions it equals plain RoPE; with three-component positions for the prompt
    (an image block whose height / width components differ from the temporal one) the logits follow the dense reference, and
    generated tokens continue one past the largest component."""
    arch = ArchConfig(**{**BASE, "model_type": "qwen2_vl", "attn_bias": True, "mrope_section": [2, 3, 3]})
    sd = random_state_dict(arch, seed=13, std=0.15)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd)
    model = og.Model(d)
    assert model.arch.mrope_section == [2, 3, 3]
    ids = np.random.RandomState(2).randint(0, arch.vocab_size - 1, size=(1, 12)).astype(np.int32)

    def gen():
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=32)
        return og.Generator(model, p)
    g = gen()
    g.append_tokens(ids)
    np.testing.assert_allclose(g.get_logits().reshape(-1), dense_logits(arch, sd, ids[0].tolist())[-1].numpy(), rtol=2e-3, atol=3e-4)
    # tokens 3..8 are a 2 x 3 image block: temporal stays at 3, height 3..4, width 3..5; text resumes at max + 1 = 6
    t = [0, 1, 2, 3, 3, 3, 3, 3, 3, 6, 7, 8]
    h = [0, 1, 2, 3, 3, 3, 4, 4, 4, 6, 7, 8]
    w = [0, 1, 2, 3, 4, 5, 3, 4, 5, 6, 7, 8]
    p3 = np.asarray([t, h, w], dtype=np.int32)
    g = gen()
    g.set_model_input("position_ids", p3[:, None, :])
    g.append_tokens(ids)
    want = dense_logits(arch, sd, ids[0].tolist(), positions3=p3)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)
    assert g.state.rope_delta[0] == 9 - 12
    g.generate_next_token()
    seq = ids[0].tolist() + [int(g.get_next_tokens()[0])]
    p3b = np.concatenate([p3, np.full((3, 1), 9, dtype=np.int32)], axis=1)
    want = dense_logits(arch, sd, seq, positions3=p3b)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=4e-4)


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_block_quantised_float_linears_load_expanded(fmt, tmp_path):
    """MatMulBlockQuantizedFp8Weight (e4m3 rows with a scale per output row) and MatMulBlockQuantizedFp4Weight (NVFP4: e2m1
    codes, e4m3 scale per block of 16, one global scale) are read and expanded at load: logits equal the dense model on
    the dequantised weights."""
    from onnxruntime_genai_b200.models.builder import dequantize_nvfp4, quantize_fp8_rows, quantize_nvfp4
    arch = ArchConfig(**BASE)
    sd = random_state_dict(arch, seed=17, std=0.1)
    d = str(tmp_path)
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd, linear_format=fmt)
    model = og.Model(d)
    sd_q = dict(sd)
    for k, v in sd.items():
        if k.endswith("_proj.weight") or k == "lm_head.weight":
            if fmt == "fp8":
                q8, sc = quantize_fp8_rows(v)
                sd_q[k] = q8.view(torch.float8_e4m3fn).float() * sc
                assert float((sd_q[k] - v).abs().max()) < float(v.abs().max()) * 0.07
            else:
                sd_q[k] = dequantize_nvfp4(*quantize_nvfp4(v))
                assert float((sd_q[k] - v).abs().mean()) < float(v.abs().mean()) * 0.15
    if fmt == "nvfp4":
        # packed projections (qkv, gate/up) are quantised as one stacked matrix: one global scale for the stack
        for i in range(arch.num_layers):
            for names in (("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), ("mlp.gate_proj", "mlp.up_proj")):
                keys = [f"model.layers.{i}.{n}.weight" for n in names]
                deq = dequantize_nvfp4(*quantize_nvfp4(torch.cat([sd[k] for k in keys], 0)))
                for k, part in zip(keys, torch.split(deq, [sd[k].shape[0] for k in keys], 0)):
                    sd_q[k] = part
    prompt = np.random.RandomState(4).randint(0, arch.vocab_size - 1, size=(1, 9)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=16)
    g = og.Generator(model, p)
    g.append_tokens(prompt)
    want = dense_logits(arch, sd_q, prompt[0].tolist())[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)
