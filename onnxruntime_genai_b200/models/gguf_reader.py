"""GGUF checkpoints as a source for the model builder: the file is parsed here (no external package), its tensors are
dequantised to fp32 and renamed to the Hugging Face names the exporter consumes.

Reference: src/python/py/models/gguf_model.py (tensor-name map :74-214, `undo_permute` :236-256).  Container layout
(GGUF version 2 / 3, little endian): magic "GGUF", version u32, tensor count u64, metadata count u64, metadata
key / value pairs, tensor infos (name, n_dims, dims with the fastest dimension first, type, offset), padding to
`general.alignment` (32), tensor data.  Tensor types read: F32, F16, BF16, Q8_0 (32 int8 + fp16 scale), Q4_0
(32 nibbles + fp16 scale, w = (q - 8) d) and Q4_1 (w = q d + m); the k-quants are not.

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
_BLOCK = {Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34)}         # type -> (weights per block, bytes per block)
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
        raise NotImplementedError(f"GGUF tensor type {ttype} is not supported (F32, F16, BF16, Q8_0, Q4_0, Q4_1)")
    per, nbytes = _BLOCK[ttype]
    blocks = raw[: n // per * nbytes].reshape(n // per, nbytes)
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


def write_gguf(path: str, meta: Dict[str, object], tensors: Dict[str, Tuple[np.ndarray, int]]) -> None:
    """tensors: name -> (fp32 array, GGUF type among F32, F16, Q8_0, Q4_0)."""
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
                Q4_0: lambda: quantize_q4_0(a)}[ttype]()
        head += s(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(a.shape)) + struct.pack("<IQ", ttype, off)
        blobs.append(blob)
        off += (len(blob) + 31) // 32 * 32
    with open(path, "wb") as f:
        f.write(head)
        f.write(b"\0" * ((len(head) + 31) // 32 * 32 - len(head)))
        for blob in blobs:
            f.write(blob)
            f.write(b"\0" * ((len(blob) + 31) // 32 * 32 - len(blob)))
