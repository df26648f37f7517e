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


# ---------------------------------------------------------------------------------------------- k-quants
def _scalar_k(block: bytes, ttype: int):
    """One super-block decoded element by element, as a plain transcription of the k-quant definitions (the vectorised reader is
    checked against this on random bytes)."""
    import struct
    from onnxruntime_genai_b200.models import gguf_reader as G
    b = list(block)
    f16 = lambda lo: struct.unpack("<e", bytes(b[lo:lo + 2]))[0]

    def scale_min(j, sc):
        if j < 4:
            return sc[j] & 63, sc[j + 4] & 63
        return (sc[j + 4] & 0xF) | ((sc[j - 4] >> 6) << 4), (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4)

    y = []
    if ttype == G.Q4_K:
        d, dmin, sc, q = f16(0), f16(2), b[4:16], b[16:144]
        for j in range(4):
            s1, m1 = scale_min(2 * j, sc)
            s2, m2 = scale_min(2 * j + 1, sc)
            y += [d * s1 * (q[32 * j + l] & 0xF) - dmin * m1 for l in range(32)]
            y += [d * s2 * (q[32 * j + l] >> 4) - dmin * m2 for l in range(32)]
    elif ttype == G.Q5_K:
        d, dmin, sc, qh, q = f16(0), f16(2), b[4:16], b[16:48], b[48:176]
        for j in range(4):
            s1, m1 = scale_min(2 * j, sc)
            s2, m2 = scale_min(2 * j + 1, sc)
            y += [d * s1 * ((q[32 * j + l] & 0xF) + (16 if qh[l] & (1 << (2 * j)) else 0)) - dmin * m1 for l in range(32)]
            y += [d * s2 * ((q[32 * j + l] >> 4) + (16 if qh[l] & (2 << (2 * j)) else 0)) - dmin * m2 for l in range(32)]
    elif ttype == G.Q6_K:
        ql, qh, d = b[0:128], b[128:192], f16(208)
        sc = [v - 256 if v > 127 else v for v in b[192:208]]
        for n in range(2):
            out = [0.0] * 128
            for l in range(32):
                i = l // 16
                q1 = ((ql[64 * n + l] & 0xF) | (((qh[32 * n + l] >> 0) & 3) << 4)) - 32
                q2 = ((ql[64 * n + l + 32] & 0xF) | (((qh[32 * n + l] >> 2) & 3) << 4)) - 32
                q3 = ((ql[64 * n + l] >> 4) | (((qh[32 * n + l] >> 4) & 3) << 4)) - 32
                q4 = ((ql[64 * n + l + 32] >> 4) | (((qh[32 * n + l] >> 6) & 3) << 4)) - 32
                out[l], out[l + 32] = d * sc[8 * n + i] * q1, d * sc[8 * n + i + 2] * q2
                out[l + 64], out[l + 96] = d * sc[8 * n + i + 4] * q3, d * sc[8 * n + i + 6] * q4
            y += out
    elif ttype == G.Q2_K:
        scales, q, d, dmin = b[0:16], b[16:80], f16(80), f16(82)
        i = 0
        for n in range(2):
            for j in range(4):
                for part in range(2):
                    s = scales[i]; i += 1
                    y += [d * (s & 0xF) * ((q[32 * n + 16 * part + l] >> (2 * j)) & 3) - dmin * (s >> 4) for l in range(16)]
    elif ttype == G.Q3_K:
        hm, q, sb, d = b[0:32], b[32:96], b[96:108], f16(108)
        sc = [0] * 16
        for k in range(4):
            sc[k] = (sb[k] & 0xF) | (((sb[8 + k] >> 0) & 3) << 4)
            sc[4 + k] = (sb[4 + k] & 0xF) | (((sb[8 + k] >> 2) & 3) << 4)
            sc[8 + k] = (sb[k] >> 4) | (((sb[8 + k] >> 4) & 3) << 4)
            sc[12 + k] = (sb[4 + k] >> 4) | (((sb[8 + k] >> 6) & 3) << 4)
        i, m = 0, 1
        for n in range(2):
            for j in range(4):
                for part in range(2):
                    dl = d * (sc[i] - 32); i += 1
                    y += [dl * (((q[32 * n + 16 * part + l] >> (2 * j)) & 3) - (0 if hm[16 * part + l] & m else 4)) for l in range(16)]
                m <<= 1
    return np.asarray(y, dtype=np.float32)


@pytest.mark.parametrize("name", ["Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K"])
def test_k_quant_blocks_decode_like_their_definition(name):
    from onnxruntime_genai_b200.models import gguf_reader as G
    ttype = getattr(G, name)
    per, nbytes = G._BLOCK[ttype]
    rng = np.random.RandomState(ttype)
    raw = rng.randint(0, 256, size=(5, nbytes)).astype(np.uint8)
    # the fp16 fields must be finite: overwrite them with small numbers
    for off in {G.Q4_K: (0, 2), G.Q5_K: (0, 2), G.Q6_K: (208,), G.Q2_K: (80, 82), G.Q3_K: (108,)}[ttype]:
        raw[:, off:off + 2] = np.asarray(rng.uniform(0.001, 0.02, size=5), dtype=np.float16).view(np.uint8).reshape(5, 2)
    got = G.dequantize(raw.reshape(-1), ttype, 5 * per).reshape(5, per)
    for i in range(5):
        np.testing.assert_allclose(got[i], _scalar_k(raw[i].tobytes(), ttype), rtol=1e-6, atol=1e-6)


def test_k_quant_file_loads(tmp_path):
    """A GGUF file whose projections are Q4_K and whose output matrix is Q6_K (the usual Q4_K_M mix) exports and runs close to
    the float weights it was written from."""
    from onnxruntime_genai_b200.models import gguf_reader as G
    w = (np.random.RandomState(2).randn(8, 512) * 0.05).astype(np.float32)
    for ttype, fn, tol in ((G.Q4_K, G.quantize_q4_k, 0.02), (G.Q6_K, G.quantize_q6_k, 0.005)):
        back = G.dequantize(np.frombuffer(fn(w), dtype=np.uint8), ttype, w.size).reshape(w.shape)
        assert np.abs(back - w).max() < tol
    path = str(tmp_path / "k.gguf")
    G.write_gguf(path, {"general.architecture": "llama"}, {"a": (w, G.Q4_K), "b": (w[:2], G.Q6_K), "c": (w[:1, :32], G.F32)})
    meta, tensors = G.read_gguf(path)
    assert meta["general.architecture"] == "llama" and tuple(tensors["a"].shape) == (8, 512)
    assert float((tensors["a"] - torch.from_numpy(w)).abs().max()) < 0.02 and float((tensors["b"] - torch.from_numpy(w[:2])).abs().max()) < 0.005
    assert torch.equal(tensors["c"], torch.from_numpy(w[:1, :32]))
