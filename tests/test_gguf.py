"""GGUF files as a builder source (reference: src/python/py/models/gguf_model.py)."""
import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import create_model, random_state_dict
from onnxruntime_genai_b200.models import gguf_reader as gg
from dense_reference import logits as dense_logits

ARCH = dict(model_type="llama", vocab_size=96, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=256, context_length=64, bos_token_id=1, eos_token_id=2, pad_token_id=0)
NAMES = {"input_layernorm": "attn_norm", "self_attn.q_proj": "attn_q", "self_attn.k_proj": "attn_k", "self_attn.v_proj": "attn_v",
         "self_attn.o_proj": "attn_output", "post_attention_layernorm": "ffn_norm", "mlp.gate_proj": "ffn_gate", "mlp.up_proj": "ffn_up",
         "mlp.down_proj": "ffn_down"}


def test_block_formats_dequantise_to_their_definitions():
    rng = np.random.RandomState(0)
    w = (rng.randn(4, 64) * 0.3).astype(np.float32)
    q8 = gg.dequantize(np.frombuffer(gg.quantize_q8_0(w), dtype=np.uint8), gg.Q8_0, w.size).reshape(w.shape)
    assert np.abs(q8 - w).max() <= np.abs(w).max() / 127 * 0.51 + 1e-3
    q4 = gg.dequantize(np.frombuffer(gg.quantize_q4_0(w), dtype=np.uint8), gg.Q4_0, w.size).reshape(w.shape)
    assert np.abs(q4 - w).max() <= np.abs(w).max() / 8 * 1.01 + 1e-3     # the range is -8..7 steps: the far end clips by one step
    # one hand-made Q4_0 block: d = 0.5, nibbles 0..15 in the low halves (weights 0..15), 15..0 in the high halves (16..31)
    blk = np.zeros(18, dtype=np.uint8)
    blk[0:2] = np.frombuffer(np.float16(0.5).tobytes(), dtype=np.uint8)
    blk[2:] = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    want = np.concatenate([np.arange(16) - 8, 7 - np.arange(16)]).astype(np.float32) * 0.5
    np.testing.assert_array_equal(gg.dequantize(blk, gg.Q4_0, 32), want)
    # Q4_1: w = q d + m
    blk1 = np.zeros(20, dtype=np.uint8)
    blk1[0:2] = np.frombuffer(np.float16(0.25).tobytes(), dtype=np.uint8)
    blk1[2:4] = np.frombuffer(np.float16(-1.0).tobytes(), dtype=np.uint8)
    blk1[4:] = 0x21
    np.testing.assert_array_equal(gg.dequantize(blk1, gg.Q4_1, 32), np.concatenate([np.full(16, -0.75), np.full(16, -0.5)]).astype(np.float32))
    bf = torch.tensor([1.5, -2.0, 0.0078125]).to(torch.bfloat16)
    np.testing.assert_array_equal(gg.dequantize(bf.view(torch.int16).numpy().view(np.uint8), gg.BF16, 3), bf.float().numpy())
    x = torch.randn(8, 6)
    assert torch.equal(gg.undo_permute(gg.permute(x, 2), 2), x) and not torch.equal(gg.permute(x, 2), x)


def test_gguf_file_exports_and_matches_the_dense_model(tmp_path):
    """A llama GGUF (rows of q / k permuted the way llama.cpp's converter does, fp32 and fp16 tensors) -> fp32 export ->
    logits of the dense model on the original weights."""
    arch = ArchConfig(**ARCH)
    sd = {k: v.to(torch.float16).float() for k, v in random_state_dict(arch, seed=21, std=0.1).items()}
    tensors = {"token_embd.weight": (sd["model.embed_tokens.weight"].numpy(), gg.F16), "output_norm.weight": (sd["model.norm.weight"].numpy(), gg.F32),
               "output.weight": (sd["lm_head.weight"].numpy(), gg.F16)}
    for i in range(arch.num_layers):
        for hf, g in NAMES.items():
            w = sd[f"model.layers.{i}.{hf}.weight"]
            if g == "attn_q":
                w = gg.permute(w, arch.num_heads)
            elif g == "attn_k":
                w = gg.permute(w, arch.num_kv_heads)
            tensors[f"blk.{i}.{g}.weight"] = (w.numpy(), gg.F32 if w.dim() == 1 else gg.F16)
    meta = {"general.architecture": "llama", "llama.block_count": 2, "llama.embedding_length": 128, "llama.feed_forward_length": 256,
            "llama.attention.head_count": 4, "llama.attention.head_count_kv": 2, "llama.context_length": 64,
            "llama.attention.layer_norm_rms_epsilon": 1e-5, "llama.rope.freq_base": 10000.0, "tokenizer.ggml.bos_token_id": 1,
            "tokenizer.ggml.eos_token_id": 2, "tokenizer.ggml.padding_token_id": 0}
    path = str(tmp_path / "tiny.gguf")
    gg.write_gguf(path, meta, tensors)
    m, t = gg.read_gguf(path)
    assert m["llama.block_count"] == 2 and t["blk.1.ffn_down.weight"].shape == (128, 256)
    out = str(tmp_path / "out")
    create_model(path, out, "fp32", "cpu")
    model = og.Model(out)
    assert model.arch.num_kv_heads == 2 and model.arch.intermediate_size == 256
    ids = np.random.RandomState(5).randint(3, 96, size=(1, 11)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=16)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    want = dense_logits(model.arch, sd, ids[0].tolist())[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)
