"""Bidirectional transformer encoders for the multimodal models: the Whisper audio encoder (two 1-D convolutions over
the log-mel frames, fixed position table, pre-LayerNorm blocks, final LayerNorm) and a ViT-style image encoder (patch
projection, learned position table, pre-LayerNorm blocks, final LayerNorm, two-layer projector into the language
model's width).

Both run on the same kernels as the decoder: the convolutions and the patch projection are unfold + GEMM
(`ops.linear`, tcgen05), the blocks are LayerNorm -> fused qkv GEMM -> key/value append -> `ops.paged_attention` in its
bidirectional mode (local_window_size < 0: every query sees all cached keys of its sequence) -> output GEMM with the
residual added in the epilogue -> fc1 -> GELU -> fc2 (+residual).  Sequences are packed: one launch per op covers
every image or audio clip of the batch.

The reference runs these encoders as opaque ONNX sessions (src/models/whisper.cpp:19-120, src/models/multi_modal.cpp:
104-260); here the `.onnx` file is a weight container whose single `Encoder` node carries the shape attributes.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..utils import onnx_proto as op

_BS = 16   # key/value block of the encoder's scratch cache


@dataclass
class EncoderConfig:
    kind: str = "audio"            # audio (Whisper) | vision (ViT + projector)
    hidden_size: int = 384
    num_layers: int = 4
    num_heads: int = 6
    intermediate_size: int = 1536
    norm_eps: float = 1e-5
    activation: str = "gelu_erf"
    # audio front end
    num_mel_bins: int = 80
    max_source_positions: int = 1500   # frames after the stride-2 convolution
    # vision front end
    image_size: int = 224
    patch_size: int = 14
    num_channels: int = 3
    projection_size: int = 0           # width of the language model the projector maps to (0 = no projector)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2


def encoder_weight_shapes(c: EncoderConfig) -> Dict[str, tuple]:
    H, I = c.hidden_size, c.intermediate_size
    s: Dict[str, tuple] = {}
    if c.kind == "audio":
        s["encoder.conv1.weight"] = (H, c.num_mel_bins, 3)
        s["encoder.conv1.bias"] = (H,)
        s["encoder.conv2.weight"] = (H, H, 3)
        s["encoder.conv2.bias"] = (H,)
        s["encoder.embed_positions.weight"] = (c.max_source_positions, H)
    else:
        s["encoder.patch_embedding.weight"] = (H, c.num_channels, c.patch_size, c.patch_size)
        s["encoder.patch_embedding.bias"] = (H,)
        s["encoder.embed_positions.weight"] = (c.num_patches, H)
        if c.projection_size:
            s["projector.fc1.weight"] = (c.projection_size, H)
            s["projector.fc1.bias"] = (c.projection_size,)
            s["projector.fc2.weight"] = (c.projection_size, c.projection_size)
            s["projector.fc2.bias"] = (c.projection_size,)
    for i in range(c.num_layers):
        p = f"encoder.layers.{i}."
        for nm in ("self_attn_layer_norm", "final_layer_norm"):
            s[p + nm + ".weight"] = (H,)
            s[p + nm + ".bias"] = (H,)
        for nm in ("q_proj", "k_proj", "v_proj", "out_proj"):
            s[p + f"self_attn.{nm}.weight"] = (H, H)
            s[p + f"self_attn.{nm}.bias"] = (H,)
        s[p + "fc1.weight"], s[p + "fc1.bias"] = (I, H), (I,)
        s[p + "fc2.weight"], s[p + "fc2.bias"] = (H, I), (H,)
    s["encoder.layer_norm.weight"] = (H,)
    s["encoder.layer_norm.bias"] = (H,)
    return s


def sinusoid_positions(length: int, channels: int) -> torch.Tensor:
    """Whisper's fixed encoder position table."""
    inc = math.log(10000.0) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)


def random_encoder_state_dict(c: EncoderConfig, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    from .builder import random_tensor
    sd = {n: random_tensor(n, shp, seed, std) for n, shp in encoder_weight_shapes(c).items()}
    if c.kind == "audio":
        sd["encoder.embed_positions.weight"] = sinusoid_positions(c.max_source_positions, c.hidden_size)
    return sd


# ------------------------------------------------------------------------------------------------ export / load
_DT = {"fp32": (torch.float32, op.FLOAT), "bf16": (torch.bfloat16, op.BFLOAT16), "fp16": (torch.float16, op.FLOAT16)}


def export_encoder(c: EncoderConfig, out_dir: str, filename: str, state_dict: Dict[str, torch.Tensor], precision: str = "bf16") -> str:
    """Writes the encoder's weights as initializers under their canonical names plus one `Encoder` node with the
    configuration as attributes."""
    os.makedirs(out_dir, exist_ok=True)
    prec = "bf16" if precision == "int4" else precision
    tdt, odt = _DT[prec]
    m = op.Model()
    for name in encoder_weight_shapes(c):
        t = state_dict[name].detach().to(tdt).contiguous()
        arr = t.view(torch.int16).numpy() if prec == "bf16" else t.numpy()
        m.initializers[name] = op.Tensor(name=name, dtype=odt, dims=tuple(t.shape), raw=np.ascontiguousarray(arr).tobytes())
    attrs = {k: v for k, v in asdict(c).items()}
    inp = "audio_features" if c.kind == "audio" else "pixel_values"
    out = "encoder_hidden_states" if c.kind == "audio" else "image_features"
    m.nodes.append(op.Node(op_type="Encoder", name="/encoder/Encoder", inputs=[inp] + list(m.initializers), outputs=[out],
                           domain="ogb200", attrs=attrs))
    m.inputs = [op.ValueInfo(inp, odt, ("batch_size", c.num_mel_bins, "num_frames") if c.kind == "audio"
                             else ("num_images", c.num_channels, c.image_size, c.image_size))]
    m.outputs = [op.ValueInfo(out, odt, ("batch_size", "sequence_length", c.projection_size or c.hidden_size))]
    path = os.path.join(out_dir, filename)
    op.save_model(m, path)
    return path


@dataclass
class _Layer:
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    qkv_w: torch.Tensor
    qkv_b: torch.Tensor
    o_w: torch.Tensor
    o_b: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor
    fc1_w: torch.Tensor
    fc1_b: torch.Tensor
    fc2_w: torch.Tensor
    fc2_b: torch.Tensor


def _pad_k(w: torch.Tensor) -> torch.Tensor:
    """GEMM operands need a 16-byte row pitch: pads the inner dimension to a multiple of 8 elements."""
    k = w.shape[1]
    return w if k % 8 == 0 else torch.nn.functional.pad(w, (0, 8 - k % 8))


class TransformerEncoder:
    def __init__(self, cfg: EncoderConfig, sd: Dict[str, torch.Tensor], device, dtype, pad_heads: bool = False):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        t = lambda n: sd[n].to(device=device, dtype=dtype).contiguous()
        self.layers: List[_Layer] = []
        # The attention kernel has head sizes 64, 96 and 128: other sizes (SigLIP's 72, small test models) run zero-padded to
        # the next one - padded q/k dimensions add nothing to the scores, padded v dimensions meet zero columns of out_proj.
        D = cfg.head_dim
        self.head_pad = D
        if (self.device.type == "cuda" or pad_heads) and D not in (64, 96, 128):
            self.head_pad = next((x for x in (64, 96, 128) if x >= D), None)
            if self.head_pad is None:
                raise RuntimeError(f"encoder head size {D} is not supported")
        Dp, nh, Hd = self.head_pad, cfg.num_heads, cfg.hidden_size

        def pad_rows(w):     # [n * nh * D, ...] -> [n * nh * Dp, ...]
            if Dp == D:
                return w
            v = w.view(-1, nh, D, *w.shape[1:])
            out = v.new_zeros(v.shape[0], nh, Dp, *w.shape[1:])
            out[:, :, :D] = v
            return out.reshape(-1, *w.shape[1:]).contiguous()

        def pad_cols(w):     # [H, nh * D] -> [H, nh * Dp]
            if Dp == D:
                return w
            out = w.new_zeros(w.shape[0], nh, Dp)
            out[:, :, :D] = w.view(w.shape[0], nh, D)
            return out.reshape(w.shape[0], nh * Dp).contiguous()

        for i in range(cfg.num_layers):
            p = f"encoder.layers.{i}."
            self.layers.append(_Layer(
                t(p + "self_attn_layer_norm.weight"), t(p + "self_attn_layer_norm.bias"),
                pad_rows(torch.cat([t(p + f"self_attn.{n}.weight") for n in ("q_proj", "k_proj", "v_proj")], 0).contiguous()),
                pad_rows(torch.cat([t(p + f"self_attn.{n}.bias") for n in ("q_proj", "k_proj", "v_proj")], 0).contiguous()),
                pad_cols(t(p + "self_attn.out_proj.weight")), t(p + "self_attn.out_proj.bias"),
                t(p + "final_layer_norm.weight"), t(p + "final_layer_norm.bias"),
                t(p + "fc1.weight"), t(p + "fc1.bias"), t(p + "fc2.weight"), t(p + "fc2.bias")))
        self.ln_w, self.ln_b = t("encoder.layer_norm.weight"), t("encoder.layer_norm.bias")
        self.pos = t("encoder.embed_positions.weight")
        H = cfg.hidden_size
        if cfg.kind == "audio":
            # Conv1d(k=3) as a GEMM over unfolded frames: weight [H, C, 3] -> [H, 3 * C] with the tap index outermost
            self.conv1_w = _pad_k(sd["encoder.conv1.weight"].permute(0, 2, 1).reshape(H, -1)).to(device=device, dtype=dtype).contiguous()
            self.conv1_b = t("encoder.conv1.bias")
            self.conv2_w = _pad_k(sd["encoder.conv2.weight"].permute(0, 2, 1).reshape(H, -1)).to(device=device, dtype=dtype).contiguous()
            self.conv2_b = t("encoder.conv2.bias")
        else:
            self.patch_w = _pad_k(sd["encoder.patch_embedding.weight"].reshape(H, -1)).to(device=device, dtype=dtype).contiguous()
            self.patch_b = t("encoder.patch_embedding.bias")
            self.proj = None
            if cfg.projection_size:
                self.proj = (t("projector.fc1.weight"), t("projector.fc1.bias"), t("projector.fc2.weight"), t("projector.fc2.bias"))

    @staticmethod
    def load(path: str, device, dtype) -> "TransformerEncoder":
        from .loader import _np_to_torch
        lm = op.LoadedModel(path)
        node = next(n for n in lm.model.nodes if n.op_type == "Encoder")
        defaults = EncoderConfig()
        kw = {}
        for k, v in node.attrs.items():
            if hasattr(defaults, k):
                v = v.decode() if isinstance(v, bytes) else v
                kw[k] = type(getattr(defaults, k))(v)
        cfg = EncoderConfig(**kw)
        sd = {name: _np_to_torch(lm.array(name), lm.info(name).dtype).clone() for name in lm.names()}
        lm.close()
        return TransformerEncoder(cfg, sd, device, dtype)

    # ------------------------------------------------------------------------------------ front ends
    def _conv3(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, stride: int) -> torch.Tensor:
        """x [B, S, C] -> gelu(conv1d(k=3, padding=1, stride)) as [B, S / stride, H] through one GEMM."""
        B, S, C = x.shape
        xp = torch.nn.functional.pad(x, (0, 0, 1, 1))
        cols = torch.cat([xp[:, k:k + S:stride] for k in range(3)], dim=-1)          # [B, S/stride, 3C], tap-major
        cols = cols.reshape(-1, 3 * C)
        if cols.shape[1] != w.shape[1]:
            cols = torch.nn.functional.pad(cols, (0, w.shape[1] - cols.shape[1]))
        y = ops.activation(ops.linear(cols.contiguous(), w, b), "gelu_erf")
        return y.view(B, -1, w.shape[0])

    def embed_audio(self, features: torch.Tensor) -> (torch.Tensor, List[int]):
        """features [B, n_mels, frames] -> packed [B * frames / 2, H] with positions added."""
        x = features.to(device=self.device, dtype=self.dtype).transpose(1, 2).contiguous()
        x = self._conv3(x, self.conv1_w, self.conv1_b, 1)
        x = self._conv3(x, self.conv2_w, self.conv2_b, 2)
        B, S, H = x.shape
        if S > self.pos.shape[0]:
            raise RuntimeError(f"audio has {S} encoder frames, the model supports {self.pos.shape[0]}")
        x = x + self.pos[:S][None]
        return x.reshape(B * S, H).contiguous(), [S] * B

    def embed_images(self, pixels: torch.Tensor) -> (torch.Tensor, List[int]):
        """pixels [N, C, size, size] -> packed [N * patches, H]."""
        c = self.cfg
        P = c.patch_size
        x = pixels.to(device=self.device, dtype=self.dtype)
        N, C, Hh, Ww = x.shape
        gh, gw = Hh // P, Ww // P
        cols = x.view(N, C, gh, P, gw, P).permute(0, 2, 4, 1, 3, 5).reshape(N * gh * gw, C * P * P)
        if cols.shape[1] != self.patch_w.shape[1]:
            cols = torch.nn.functional.pad(cols, (0, self.patch_w.shape[1] - cols.shape[1]))
        y = ops.linear(cols.contiguous(), self.patch_w, self.patch_b).view(N, gh * gw, c.hidden_size)
        if gh * gw != self.pos.shape[0]:
            raise RuntimeError(f"image gives {gh * gw} patches, the model's position table has {self.pos.shape[0]}")
        y = y + self.pos[None]
        return y.reshape(N * gh * gw, c.hidden_size).contiguous(), [gh * gw] * N

    # ------------------------------------------------------------------------------------ blocks
    def blocks(self, h: torch.Tensor, seq_lens: List[int]) -> torch.Tensor:
        """Packed rows [sum(seq_lens), H] through the pre-LayerNorm blocks and the final LayerNorm."""
        c, dev = self.cfg, self.device
        Hh, D = c.num_heads, self.head_pad
        nblk = [(n + _BS - 1) // _BS for n in seq_lens]
        table = torch.full((len(seq_lens), max(nblk)), -1, dtype=torch.int32)
        slots, pos, cu, b0 = [], [], [0], 0
        for i, n in enumerate(seq_lens):
            table[i, :nblk[i]] = torch.arange(b0, b0 + nblk[i], dtype=torch.int32)
            slots.append(torch.arange(n, dtype=torch.int32) + b0 * _BS)
            pos.append(torch.arange(n, dtype=torch.int32))
            cu.append(cu[-1] + n)
            b0 += nblk[i]
        table = table.to(dev)
        slots, pos = torch.cat(slots).to(dev), torch.cat(pos).to(dev)
        cu = torch.tensor(cu, dtype=torch.int32, device=dev)
        lens = torch.tensor(seq_lens, dtype=torch.int32, device=dev)
        kc = torch.zeros(b0 * _BS, Hh, D, dtype=self.dtype, device=dev)
        vc = torch.zeros_like(kc)
        scale = 1.0 / math.sqrt(c.head_dim)
        mx = max(seq_lens)
        for lw in self.layers:
            x, _ = ops.norm(h, lw.ln1_w, c.norm_eps, None, lw.ln1_b, True)
            qkv = ops.linear(x, lw.qkv_w, lw.qkv_b)
            ops.rope_kv_append(qkv, pos, slots, None, None, kc, vc, Hh, Hh, D, 0)
            att = ops.paged_attention(qkv, kc, vc, cu, lens, table, _BS, Hh, Hh, D, scale, -1, None, 0.0, max_q_len=mx, max_kv_len=mx)
            h = ops.linear(att, lw.o_w, lw.o_b, residual=h)
            x, _ = ops.norm(h, lw.ln2_w, c.norm_eps, None, lw.ln2_b, True)
            y = ops.activation(ops.linear(x, lw.fc1_w, lw.fc1_b), c.activation)
            h = ops.linear(y, lw.fc2_w, lw.fc2_b, residual=h)
        h, _ = ops.norm(h, self.ln_w, c.norm_eps, None, self.ln_b, True)
        return h

    def encode_audio(self, features: torch.Tensor) -> (torch.Tensor, List[int]):
        with torch.no_grad():
            h, lens = self.embed_audio(features)
            return self.blocks(h, lens), lens

    def encode_images(self, pixels: torch.Tensor) -> (torch.Tensor, List[int]):
        """Returns image features [N * patches, projection_size or H] and the patch count per image."""
        with torch.no_grad():
            h, lens = self.embed_images(pixels)
            h = self.blocks(h, lens)
            if self.proj is not None:
                w1, b1, w2, b2 = self.proj
                h = ops.linear(ops.activation(ops.linear(h, w1, b1), "gelu_erf"), w2, b2)
            return h, lens
