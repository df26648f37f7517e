"""GGUF checkpoints as a source for the model builder: the file is parsed here (no external package), its tensors are
dequantised to fp32 and renamed to the Hugging Face names the exporter consumes.

Reference: src/python/py/models/gguf_model.py (tensor-name map :74-214, `undo_permute` :236-256).  Container layout
(GGUF version 2 / 3, little endian): magic "GGUF", version u32, tensor count u64, metadata count u64, metadata
key / value pairs, tensor infos (name, n_dims, dims with the fastest dimension first, type, offset), padding to
`general.alignment` (32), tensor data.  Tensor types read: F32, F16, BF16, Q8_0 (32 int8 + fp16 scale), Q4_0
(32 nibbles + fp16 scale, w = (q - 8) d), Q4_1 (w = q d + m) and the k-quants Q2_K .. Q6_K (super-blocks of 256 weights with
6-bit or 8-bit sub-block scales; layouts in the comments of `_dequant_k`).

llama.cpp's converter permutes the rows of q_proj / k_proj of the llama family (interleaved -> half-split rotary
layout); `undo_permute` restores the Hugging Face order.
"""
from __future__ import annotations

import struct
from typing import Dict, Tuple

import numpy as np
import torch

MAGIC = b"GGUF"
F32, F16, Q4_0, Q4_1, Q8_0, BF16 = 0, 1, 2, 3, 8, 30
Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 10, 11, 12, 13, 14
_BLOCK = {Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34),         # type -> (weights per block, bytes per block)
          Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144), Q5_K: (256, 176), Q6_K: (256, 210)}
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
PERMUTED_ARCHS = ("llama", "mistral", "granite", "olmo")


class _Cursor:
    def __init__(self, data: memoryview):
        self.d, self.o = data, 0

    def take(self, fmt: str):
        v = struct.unpack_from(fmt, self.d, self.o)[0]
        self.o += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.take("<Q")
        s = bytes(self.d[self.o:self.o + n]).decode("utf-8", errors="replace")
        self.o += n
        return s

    def value(self, t: int):
        if t in _SCALAR:
            return self.take(_SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"GGUF metadata value type {t} is not known")


def dequantize(raw: np.ndarray, ttype: int, n: int) -> np.ndarray:
    """raw bytes of one tensor -> fp32 [n]."""
    if ttype == F32:
        return raw.view("<f4")[:n].astype(np.float32)
    if ttype == F16:
        return raw.view("<f2")[:n].astype(np.float32)
    if ttype == BF16:
        return (raw.view("<u2")[:n].astype(np.uint32) << 16).view(np.float32)
    if ttype not in _BLOCK:
        raise NotImplementedError(f"GGUF tensor type {ttype} is not supported (F32, F16, BF16, Q8_0, Q4_0, Q4_1, Q2_K .. Q6_K)")
    per, nbytes = _BLOCK[ttype]
    blocks = raw[: n // per * nbytes].reshape(n // per, nbytes)
    if per == 256:
        return _dequant_k(blocks, ttype).reshape(-1)
    d = blocks[:, 0:2].copy().view("<f2").astype(np.float32)                       # [blocks, 1]
    if ttype == Q8_0:
        return (blocks[:, 2:].copy().view(np.int8).astype(np.float32) * d).reshape(-1)
    if ttype == Q4_0:
        q = blocks[:, 2:]
        vals = np.concatenate([q & 0xF, q >> 4], axis=1).astype(np.float32) - 8.0  # low nibbles = weights 0..15, high = 16..31
        return (vals * d).reshape(-1)
    m = blocks[:, 2:4].copy().view("<f2").astype(np.float32)
    q = blocks[:, 4:]
    vals = np.concatenate([q & 0xF, q >> 4], axis=1).astype(np.float32)
    return (vals * d + m).reshape(-1)


def _f16(b: np.ndarray) -> np.ndarray:
    return b.copy().view("<f2").astype(np.float32)


def _scale_min_k4(sc: np.ndarray):
    """The eight 6-bit (scale, minimum) pairs packed in the 12 `scales` bytes of a Q4_K / Q5_K super-block: pairs 0-3 are the
    low six bits of bytes 0-3 / 4-7, pairs 4-7 take four bits from bytes 8-11 and their top two bits from bytes 0-7."""
    sc = sc.astype(np.uint8)
    d = np.empty(sc.shape[:-1] + (8,), dtype=np.float32)
    m = np.empty_like(d)
    d[..., :4] = sc[..., 0:4] & 63
    m[..., :4] = sc[..., 4:8] & 63
    d[..., 4:] = (sc[..., 8:12] & 0xF) | ((sc[..., 0:4] >> 6) << 4)
    m[..., 4:] = (sc[..., 8:12] >> 4) | ((sc[..., 4:8] >> 6) << 4)
    return d, m


def _dequant_k(b: np.ndarray, ttype: int) -> np.ndarray:
    """Super-blocks [blocks, bytes] -> fp32 [blocks, 256] (llama.cpp's k-quant layouts)."""
    nb = b.shape[0]
    if ttype == Q4_K:
        # d f16, dmin f16, scales[12], qs[128]: four groups of 64 weights; a group's 32 bytes hold sub-block 2j in the low
        # nibbles and sub-block 2j + 1 in the high nibbles; w = d * sc * q - dmin * m
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _scale_min_k4(b[:, 4:16])
        qs = b[:, 16:144].reshape(nb, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        return (q * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(nb, 256)
    if ttype == Q5_K:
        # d, dmin, scales[12], qh[32], qs[128]: as Q4_K with a fifth bit per weight: bit (2j) / (2j + 1) of qh[l]
        d, dmin = _f16(b[:, 0:2]), _f16(b[:, 2:4])
        sc, mn = _scale_min_k4(b[:, 4:16])
        qh = b[:, 16:48]
        qs = b[:, 48:176].reshape(nb, 4, 32)
        q = np.stack([qs & 0xF, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
        hi = np.stack([(qh >> k) & 1 for k in range(8)], axis=1).astype(np.float32)      # [blocks, 8 sub-blocks, 32]
        return ((q + 16.0 * hi) * (d * sc)[:, :, None] - (dmin * mn)[:, :, None]).reshape(nb, 256)
    if ttype == Q6_K:
        # ql[128], qh[64], scales int8[16], d f16: two halves of 128 weights; within a half weight l, l + 32, l + 64, l + 96
        # take their low four bits from ql[l] / ql[l + 32] (low, high nibble) and two bits from qh[l]; 16 weights share a scale
        ql = b[:, 0:128].reshape(nb, 2, 64)
        qh = b[:, 128:192].reshape(nb, 2, 32)
        scales = b[:, 192:208].copy().view(np.int8).astype(np.float32).reshape(nb, 2, 8)
        d = _f16(b[:, 208:210])
        l0, l1 = ql[:, :, :32], ql[:, :, 32:]
        q = np.stack([(l0 & 0xF) | (((qh >> 0) & 3) << 4), (l1 & 0xF) | (((qh >> 2) & 3) << 4),
                      (l0 >> 4) | (((qh >> 4) & 3) << 4), (l1 >> 4) | (((qh >> 6) & 3) << 4)], axis=2).astype(np.float32) - 32.0   # [nb, 2, 4, 32]
        # scale index of weight (quarter k, position l) within a half: l // 16 + 2 k
        idx = (np.arange(32) // 16)[None, :] + 2 * np.arange(4)[:, None]                                                        # [4, 32]
        sc = scales[:, :, idx]                                                                                                  # [nb, 2, 4, 32]
        return (q * sc * d[:, :, None, None]).reshape(nb, 256)
    if ttype == Q2_K:
        # scales[16] (low nibble scale, high nibble minimum), qs[64], d f16, dmin f16: two halves of 128; within a half the
        # four 2-bit fields of byte l give weights l, l + 32, l + 64, l + 96; 16 weights share a (scale, minimum)
        scales = b[:, 0:16]
        qs = b[:, 16:80].reshape(nb, 2, 32)
        d, dmin = _f16(b[:, 80:82]), _f16(b[:, 82:84])
        q = np.stack([(qs >> s) & 3 for s in (0, 2, 4, 6)], axis=2).astype(np.float32)                                          # [nb, 2, 4, 32]
        idx = (np.arange(32) // 16)[None, :] + 2 * np.arange(4)[:, None]
        scl = (scales & 0xF).astype(np.float32).reshape(nb, 2, 8)[:, :, idx]
        mnl = (scales >> 4).astype(np.float32).reshape(nb, 2, 8)[:, :, idx]
        return (d[:, :, None, None] * scl * q - dmin[:, :, None, None] * mnl).reshape(nb, 256)
    if ttype == Q3_K:
        # hmask[32], qs[64], scales[12] (sixteen 6-bit scales, offset 32), d f16: 2-bit fields as in Q2_K plus a high bit from
        # hmask (bit k of hmask[l] for field k of half 0, bit 4 + k for half 1); a clear high bit subtracts 4
        hm = b[:, 0:32]
        qs = b[:, 32:96].reshape(nb, 2, 32)
        sb = b[:, 96:108].astype(np.uint32)
        d = _f16(b[:, 108:110])
        low = np.concatenate([sb[:, 0:8] & 0xF, sb[:, 0:8] >> 4], axis=1)                 # scales 0..15: low four bits
        high = np.concatenate([(sb[:, 8:12] >> s) & 3 for s in (0, 2, 4, 6)], axis=1)     # their top two bits
        sc = ((low | (high << 4)).astype(np.float32) - 32.0).reshape(nb, 2, 8)
        q = np.stack([(qs >> s) & 3 for s in (0, 2, 4, 6)], axis=2).astype(np.float32)    # [nb, 2, 4, 32]
        bit = np.stack([np.stack([(hm >> (4 * h + k)) & 1 for k in range(4)], axis=1) for h in range(2)], axis=1).astype(np.float32)
        idx = (np.arange(32) // 16)[None, :] + 2 * np.arange(4)[:, None]
        return (d[:, :, None, None] * sc[:, :, idx] * (q - 4.0 * (1.0 - bit))).reshape(nb, 256)
    raise NotImplementedError(f"k-quant type {ttype}")


def read_gguf(path: str) -> Tuple[Dict[str, object], Dict[str, torch.Tensor]]:
    """(metadata, tensors): tensors are fp32 with the usual [rows, cols] shape (GGUF lists the fastest dimension first)."""
    data = np.memmap(path, dtype=np.uint8, mode="r")
    cur = _Cursor(memoryview(data))
    if bytes(data[:4]) != MAGIC:
        raise ValueError(f"{path} is not a GGUF file")
    cur.o = 4
    version = cur.take("<I")
    if version not in (2, 3):
        raise NotImplementedError(f"GGUF version {version} is not supported (2, 3)")
    n_tensors, n_kv = cur.take("<Q"), cur.take("<Q")
    meta: Dict[str, object] = {}
    for _ in range(n_kv):
        key = cur.string()
        meta[key] = cur.value(cur.take("<I"))
    infos = []
    for _ in range(n_tensors):
        name = cur.string()
        nd = cur.take("<I")
        dims = [cur.take("<Q") for _ in range(nd)]
        infos.append((name, dims, cur.take("<I"), cur.take("<Q")))
    align = int(meta.get("general.alignment", 32))
    base = (cur.o + align - 1) // align * align
    tensors: Dict[str, torch.Tensor] = {}
    for name, dims, ttype, off in infos:
        n = int(np.prod(dims)) if dims else 1
        per, nbytes = _BLOCK.get(ttype, (1, {F32: 4, F16: 2, BF16: 2}.get(ttype, 0)))
        if nbytes == 0:
            raise NotImplementedError(f"GGUF tensor {name}: type {ttype} is not supported")
        raw = np.asarray(data[base + off: base + off + n // per * nbytes])
        tensors[name] = torch.from_numpy(dequantize(raw, ttype, n).reshape(list(reversed(dims))).copy())
    return meta, tensors


def undo_permute(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """Inverse of llama.cpp's permute of q / k projection rows: per head [2, D/2] (half-split) <- [D/2, 2] (interleaved)."""
    rows = w.shape[0]
    d = rows // n_heads
    return w.reshape(n_heads, d // 2, 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


def permute(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """What llama.cpp's converter does to q / k rows (used to write test files)."""
    rows = w.shape[0]
    d = rows // n_heads
    return w.reshape(n_heads, 2, d // 2, *w.shape[1:]).transpose(1, 2).reshape(w.shape)


_LAYER_NAMES = {"attn_norm": "input_layernorm", "attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj",
                "attn_output": "self_attn.o_proj", "ffn_norm": "post_attention_layernorm", "ffn_gate": "mlp.gate_proj",
                "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj", "attn_qkv": "self_attn.qkv_proj",
                "attn_q_norm": "self_attn.q_norm", "attn_k_norm": "self_attn.k_norm",
                "post_attention_norm": "post_attention_layernorm", "post_ffw_norm": "post_feedforward_layernorm"}


def hf_config_and_state_dict(path: str):
    """(Hugging Face style config dict, state dict) of a GGUF decoder."""
    meta, tensors = read_gguf(path)
    arch = str(meta.get("general.architecture", "llama"))
    g = lambda k, default=None: meta.get(f"{arch}.{k}", default)
    heads = int(g("attention.head_count"))
    kv_heads = int(g("attention.head_count_kv", heads))
    hidden = int(g("embedding_length"))
    vocab = tensors["token_embd.weight"].shape[0]
    cfg = {"architectures": [arch.capitalize() + "ForCausalLM"], "model_type": arch, "vocab_size": int(vocab), "hidden_size": hidden,
           "num_hidden_layers": int(g("block_count")), "num_attention_heads": heads, "num_key_value_heads": kv_heads,
           "head_dim": int(g("attention.key_length", hidden // heads)), "intermediate_size": int(g("feed_forward_length")),
           "max_position_embeddings": int(g("context_length", 2048)), "rms_norm_eps": float(g("attention.layer_norm_rms_epsilon", 1e-5)),
           "rope_theta": float(g("rope.freq_base", 10000.0)), "bos_token_id": int(meta.get("tokenizer.ggml.bos_token_id", 1)),
           "eos_token_id": int(meta.get("tokenizer.ggml.eos_token_id", 2)), "pad_token_id": int(meta.get("tokenizer.ggml.padding_token_id", 0)),
           "tie_word_embeddings": "output.weight" not in tensors}
    sd: Dict[str, torch.Tensor] = {}
    for name, t in tensors.items():
        if name == "token_embd.weight":
            sd["model.embed_tokens.weight"] = t
        elif name in ("output_norm.weight", "output_norm.bias"):
            sd["model.norm." + name.split(".")[1]] = t
        elif name in ("output.weight", "output.bias"):
            sd["lm_head." + name.split(".")[1]] = t
        elif name.startswith("blk."):
            _, idx, part, kind = name.split(".", 3)
            if part not in _LAYER_NAMES:
                continue
            if arch in PERMUTED_ARCHS and part in ("attn_q", "attn_k"):
                t = undo_permute(t, heads if part == "attn_q" else kv_heads)
            sd[f"model.layers.{idx}.{_LAYER_NAMES[part]}.{kind}"] = t
    return cfg, sd


# ---------------------------------------------------------------------------------------------- writer (tests, tooling)
def quantize_q4_0(w: np.ndarray) -> bytes:
    b = w.reshape(-1, 32).astype(np.float32)
    idx = np.abs(b).argmax(1)
    mx = b[np.arange(len(b)), idx]
    d = (mx / -8.0).astype(np.float16)
    inv = np.where(d.astype(np.float32) != 0, 1.0 / np.where(d == 0, 1, d).astype(np.float32), 0.0)
    q = np.clip(np.floor(b * inv[:, None] + 8.5), 0, 15).astype(np.uint8)
    out = np.zeros((len(b), 18), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.tobytes()


def quantize_q8_0(w: np.ndarray) -> bytes:
    b = w.reshape(-1, 32).astype(np.float32)
    d = (np.abs(b).max(1) / 127.0).astype(np.float16)
    inv = np.where(d.astype(np.float32) != 0, 1.0 / np.where(d == 0, 1, d).astype(np.float32), 0.0)
    q = np.clip(np.round(b * inv[:, None]), -127, 127).astype(np.int8)
    out = np.zeros((len(b), 34), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q.view(np.uint8)
    return out.tobytes()


def quantize_q4_k(w: np.ndarray) -> bytes:
    """A plain (min / max per sub-block, no search) Q4_K encoder: enough to write test and tooling files."""
    b = w.reshape(-1, 8, 32).astype(np.float32)
    mn = np.minimum(b.min(-1), 0.0)
    sub_scale = (b.max(-1) - mn) / 15.0                                   # per sub-block
    d = (sub_scale.max(-1) / 63.0).astype(np.float16)
    dmin = ((-mn).max(-1) / 63.0).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    sc = np.clip(np.round(np.divide(sub_scale, df[:, None], out=np.zeros_like(sub_scale), where=df[:, None] != 0)), 0, 63).astype(np.uint8)
    m = np.clip(np.round(np.divide(-mn, dmf[:, None], out=np.zeros_like(mn), where=dmf[:, None] != 0)), 0, 63).astype(np.uint8)
    eff = df[:, None] * sc
    q = np.clip(np.round(np.divide(b + (dmf[:, None] * m)[..., None], eff[..., None], out=np.zeros_like(b), where=eff[..., None] != 0)), 0, 15).astype(np.uint8)
    out = np.zeros((len(b), 144), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(-1, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(-1, 2)
    out[:, 4:8] = (sc[:, :4] & 63) | ((sc[:, 4:] >> 4) << 6)
    out[:, 8:12] = (m[:, :4] & 63) | ((m[:, 4:] >> 4) << 6)
    out[:, 12:16] = (sc[:, 4:] & 0xF) | ((m[:, 4:] & 0xF) << 4)
    qq = q.reshape(-1, 4, 2, 32)
    out[:, 16:144] = (qq[:, :, 0] | (qq[:, :, 1] << 4)).reshape(-1, 128)
    return out.tobytes()


def quantize_q6_k(w: np.ndarray) -> bytes:
    """A plain Q6_K encoder (absolute maximum per 16 weights)."""
    b = w.reshape(-1, 16, 16).astype(np.float32)
    amax = np.abs(b).max(-1)
    d = (amax.max(-1) / (127.0 * 31.0)).astype(np.float16)
    df = d.astype(np.float32)
    sc = np.clip(np.round(np.divide(amax / 31.0, df[:, None], out=np.zeros_like(amax), where=df[:, None] != 0)), -128, 127).astype(np.int8)
    eff = df[:, None] * sc.astype(np.float32)
    q = (np.clip(np.round(np.divide(b, eff[..., None], out=np.zeros_like(b), where=eff[..., None] != 0)), -32, 31) + 32).astype(np.uint8)
    q = q.reshape(-1, 2, 4, 32)                                           # [blocks, half, quarter, l]
    out = np.zeros((len(b), 210), dtype=np.uint8)
    ql = np.concatenate([(q[:, :, 0] & 0xF) | ((q[:, :, 2] & 0xF) << 4), (q[:, :, 1] & 0xF) | ((q[:, :, 3] & 0xF) << 4)], axis=2)   # [blocks, 2, 64]
    qh = (q[:, :, 0] >> 4) | ((q[:, :, 1] >> 4) << 2) | ((q[:, :, 2] >> 4) << 4) | ((q[:, :, 3] >> 4) << 6)
    out[:, 0:128] = ql.reshape(-1, 128)
    out[:, 128:192] = qh.reshape(-1, 64)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(-1, 2)
    return out.tobytes()


def write_gguf(path: str, meta: Dict[str, object], tensors: Dict[str, Tuple[np.ndarray, int]]) -> None:
    """tensors: name -> (fp32 array, GGUF type among F32, F16, Q8_0, Q4_0, Q4_K, Q6_K)."""
    def s(x: str) -> bytes:
        b = x.encode()
        return struct.pack("<Q", len(b)) + b

    head = MAGIC + struct.pack("<IQQ", 3, len(tensors), len(meta))
    for k, v in meta.items():
        head += s(k)
        if isinstance(v, str):
            head += struct.pack("<I", 8) + s(v)
        elif isinstance(v, float):
            head += struct.pack("<If", 6, v)
        else:
            head += struct.pack("<II", 4, int(v))
    blobs, off = [], 0
    for name, (arr, ttype) in tensors.items():
        a = np.ascontiguousarray(arr, dtype=np.float32)
        blob = {F32: lambda: a.tobytes(), F16: lambda: a.astype(np.float16).tobytes(), Q8_0: lambda: quantize_q8_0(a),
                Q4_0: lambda: quantize_q4_0(a), Q4_K: lambda: quantize_q4_k(a), Q6_K: lambda: quantize_q6_k(a)}[ttype]()
        head += s(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(a.shape)) + struct.pack("<IQ", ttype, off)
        blobs.append(blob)
        off += (len(blob) + 31) // 32 * 32
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((len(head) + 31) // 32 * 32 - len(head)))
        for blob in blobs:
            f.write(blob)
            f.write(b"\0" * ((len(blob) + 31) // 32 * 32 - len(blob)))
