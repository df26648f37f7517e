"""Checkpoint exporter: architecture + weights -> `genai_config.json` + `model.onnx` + `model.onnx.data`.

The output directory follows the reference builder's contract (src/python/py/models/builder.py:289-589,
builders/base.py): transposed `[in, out]` MatMul initializers named
`model.layers.{i}.attn.qkv_proj.MatMul.weight` etc., `SimplifiedLayerNormalization` /
`SkipSimplifiedLayerNormalization` nodes carrying `epsilon`, a `GroupQueryAttention` (or `PagedAttention`)
node per layer carrying `num_heads / kv_num_heads / scale / local_window_size / softcap / do_rotary /
rotary_interleaved`, `cos_cache` / `sin_cache` initializers of shape `[ctx, rot/2]`, MatMulNBits
int4 block-32 weights as `qweight [N, K/32, 16]` + `scales` + packed uint4 `zero_points`
(base.py:1963-2022, quantized_model.py:1060-1107), and the `genai_config.json` layout of
base.py:1033-1128.

CLI:  python -m onnxruntime_genai_b200.models.builder -m <hf_dir | preset> -o <out_dir> -p bf16|fp16|fp32|int4
          -e cuda|cpu [--extra_options k=v ...]

Extension (not in the reference): `--extra_options synthetic_weights=1` writes initializers whose
external-data entry carries `synthetic = normal:<std>:<seed>` instead of bytes on disk, so that a
70B-shaped random-init checkpoint for benchmarking is a few kilobytes; the loader generates those
tensors on the device.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import sys
import zlib
from typing import Dict, Optional

import numpy as np
import torch

from ..utils import onnx_proto as op
from .arch import PRESETS, ArchConfig, from_hf_config, longrope_caches, rope_caches

_ONNX_DT = {"fp32": op.FLOAT, "fp16": op.FLOAT16, "bf16": op.BFLOAT16}
_TORCH_DT = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}


# ---------------------------------------------------------------------------------------------- weights
def weight_shapes(arch: ArchConfig) -> Dict[str, tuple]:
    """Canonical (Hugging Face style, [out, in]) parameter names and shapes."""
    H, I, V = arch.hidden_size, arch.intermediate_size, arch.vocab_size
    s: Dict[str, tuple] = {"model.embed_tokens.weight": (V, H)}
    if arch.learned_positions:
        s["model.position_embeddings.weight"] = (arch.context_length, H)
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        s[p + "input_layernorm.weight"] = (H,)
        if arch.layernorm:
            s[p + "input_layernorm.bias"] = (H,)
        if not arch.parallel_block:
            s[p + "post_attention_layernorm.weight"] = (H,)
            if arch.layernorm:
                s[p + "post_attention_layernorm.bias"] = (H,)
        if arch.post_sublayer_norms:
            s[p + "pre_feedforward_layernorm.weight"] = (H,)
            s[p + "post_feedforward_layernorm.weight"] = (H,)
        if arch.is_conv_layer(i):
            s[p + "conv.in_proj.weight"] = (3 * H, H)
            s[p + "conv.conv.weight"] = (H, arch.conv_L_cache)
            if arch.conv_bias:
                s[p + "conv.conv.bias"] = (H,)
            s[p + "conv.out_proj.weight"] = (H, H)
        elif arch.is_mamba_layer(i):
            I, cd, nh = arch.mamba_intermediate, arch.mamba_conv_dim, arch.mamba_num_heads
            s[p + "mamba.in_proj.weight"] = (I + cd + nh, H)
            s[p + "mamba.conv1d.weight"] = (cd, 1, arch.mamba_conv_kernel)
            s[p + "mamba.conv1d.bias"] = (cd,)
            s[p + "mamba.dt_bias"] = (nh,)
            s[p + "mamba.A_log"] = (nh,)
            s[p + "mamba.D"] = (nh,)
            s[p + "mamba.norm.weight"] = (I,)
            s[p + "mamba.out_proj.weight"] = (H, I)
        elif arch.is_linear_layer(i):
            nv, hv = arch.linear_num_value_heads, arch.linear_value_head_dim
            s[p + "linear_attn.in_proj_qkv.weight"] = (arch.linear_conv_dim, H)
            s[p + "linear_attn.in_proj_z.weight"] = (arch.linear_value_dim, H)
            s[p + "linear_attn.in_proj_b.weight"] = (nv, H)
            s[p + "linear_attn.in_proj_a.weight"] = (nv, H)
            s[p + "linear_attn.conv1d.weight"] = (arch.linear_conv_dim, arch.linear_conv_kernel_dim)
            s[p + "linear_attn.dt_bias"] = (nv,)
            s[p + "linear_attn.A_log"] = (nv,)
            s[p + "linear_attn.norm.weight"] = (hv,)
            s[p + "linear_attn.out_proj.weight"] = (H, arch.linear_value_dim)
        else:
            s[p + "self_attn.q_proj.weight"] = (arch.q_size, H)
            if arch.attn_output_gate:
                s[p + "self_attn.gate_proj.weight"] = (arch.q_size, H)
            s[p + "self_attn.k_proj.weight"] = (arch.kv_size, H)
            s[p + "self_attn.v_proj.weight"] = (arch.kv_size, H)
            s[p + "self_attn.o_proj.weight"] = (H, arch.q_size)
            if arch.attn_bias:
                s[p + "self_attn.q_proj.bias"] = (arch.q_size,)
                s[p + "self_attn.k_proj.bias"] = (arch.kv_size,)
                s[p + "self_attn.v_proj.bias"] = (arch.kv_size,)
            if arch.o_bias:
                s[p + "self_attn.o_proj.bias"] = (H,)
        if arch.cross_attention:
            s[p + "cross_attn_layernorm.weight"] = (H,)
            if arch.layernorm:
                s[p + "cross_attn_layernorm.bias"] = (H,)
            for nm, shp in (("q", (arch.q_size, H)), ("k", (arch.q_size, arch.encoder_hidden_size or H)),
                            ("v", (arch.q_size, arch.encoder_hidden_size or H)), ("o", (H, arch.q_size))):
                s[p + f"cross_attn.{nm}_proj.weight"] = shp
                s[p + f"cross_attn.{nm}_proj.bias"] = (shp[0],)
        if arch.qk_norm and not arch.is_conv_layer(i) and not arch.is_recurrent_layer(i):
            s[p + "self_attn.q_norm.weight"] = (arch.q_size if arch.qk_norm_full_width else arch.head_dim,)
            s[p + "self_attn.k_norm.weight"] = (arch.kv_size if arch.qk_norm_full_width else arch.head_dim,)
        if arch.attn_sinks:
            s[p + "self_attn.sinks"] = (arch.num_heads,)
        if arch.num_experts > 0 and arch.moe_style == "standard":
            E = arch.num_experts
            s[p + "mlp.router.weight"] = (E, H)
            s[p + "mlp.experts.gate_proj"] = (E, I, H)
            s[p + "mlp.experts.up_proj"] = (E, I, H)
            s[p + "mlp.experts.down_proj"] = (E, H, I)
            if arch.shared_expert_intermediate:
                Is = arch.shared_expert_intermediate
                s[p + "mlp.shared_expert.gate_proj.weight"] = (Is, H)
                s[p + "mlp.shared_expert.up_proj.weight"] = (Is, H)
                s[p + "mlp.shared_expert.down_proj.weight"] = (H, Is)
                if arch.shared_expert_gated:
                    s[p + "mlp.shared_expert_gate.weight"] = (1, H)
        elif arch.num_experts > 0:
            E = arch.num_experts
            s[p + "mlp.router.weight"] = (E, H)
            s[p + "mlp.router.bias"] = (E,)
            s[p + "mlp.experts.gate_up_proj"] = (E, 2 * I, H)   # rows interleaved gate0, up0, gate1, up1 ...
            s[p + "mlp.experts.gate_up_proj_bias"] = (E, 2 * I)
            s[p + "mlp.experts.down_proj"] = (E, H, I)
            s[p + "mlp.experts.down_proj_bias"] = (E, H)
        elif not arch.mlp_gated:
            s[p + "mlp.fc1.weight"] = (I, H)
            s[p + "mlp.fc2.weight"] = (H, I)
            if arch.mlp_bias:
                s[p + "mlp.fc1.bias"] = (I,)
                s[p + "mlp.fc2.bias"] = (H,)
        else:
            s[p + "mlp.gate_proj.weight"] = (I, H)
            s[p + "mlp.up_proj.weight"] = (I, H)
            s[p + "mlp.down_proj.weight"] = (H, I)
            if arch.mlp_bias:
                s[p + "mlp.gate_proj.bias"] = (I,)
                s[p + "mlp.up_proj.bias"] = (I,)
                s[p + "mlp.down_proj.bias"] = (H,)
    s["model.norm.weight"] = (H,)
    if arch.layernorm:
        s["model.norm.bias"] = (H,)
    if not arch.tie_embeddings:
        s["lm_head.weight"] = (V, H)
        if arch.lm_head_bias:
            s["lm_head.bias"] = (V,)
    return s


def _is_norm_weight(name: str) -> bool:
    return name.endswith("norm.weight") or name.endswith("layernorm.weight")


def tensor_seed(name: str, seed: int) -> int:
    return (zlib.crc32(name.encode()) ^ (seed * 0x9E3779B1)) & 0x7FFFFFFF


def random_tensor(name: str, shape, seed: int, std: float, device="cpu", dtype=torch.float32) -> torch.Tensor:
    """Deterministic N(0, std) tensor for a parameter name (norm weights are ones, sinks N(0, 1))."""
    if _is_norm_weight(name):
        return torch.ones(shape, dtype=dtype, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(tensor_seed(name, seed))
    s = 1.0 if name.endswith(".sinks") or "router" in name else std
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * s).to(dtype)


def random_state_dict(arch: ArchConfig, seed: int = 0, std: float = 0.02) -> Dict[str, torch.Tensor]:
    return {n: random_tensor(n, shp, seed, std) for n, shp in weight_shapes(arch).items()}


# ---------------------------------------------------------------------------------------------- int4
def quantize_int4_block32(w: torch.Tensor, symmetric: bool = False, block: int = 32):
    """RTN block quantisation in the MatMulNBits layout.  w: [N, K] float.
    Returns qweight uint8 [N, K/block, block/2] (low nibble = even k), scales fp32 [N, K/block],
    zero_points uint8 [N, ceil(K/block/2)] packed two per byte (low nibble first) or None."""
    N, K = w.shape
    assert K % block == 0
    wb = w.float().view(N, K // block, block)
    if symmetric:
        amax_idx = wb.abs().argmax(-1, keepdim=True)
        amax = torch.gather(wb, -1, amax_idx)
        scale = (amax / -8.0).squeeze(-1)
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
        q = torch.clamp(torch.round(wb / scale[..., None]) + 8, 0, 15)
        zp = None
    else:
        mn = wb.amin(-1).clamp(max=0.0)
        mx = wb.amax(-1).clamp(min=0.0)
        scale = (mx - mn) / 15.0
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
        zpf = torch.clamp(torch.round(-mn / scale), 0, 15)
        q = torch.clamp(torch.round(wb / scale[..., None]) + zpf[..., None], 0, 15)
        zp = zpf.to(torch.uint8)
    q = q.to(torch.uint8)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous()
    zp_packed = None
    if zp is not None:
        nb = K // block
        if nb % 2:
            zp = torch.cat([zp, torch.full((N, 1), 8, dtype=torch.uint8, device=zp.device)], dim=1)
        zp_packed = (zp[:, 0::2] | (zp[:, 1::2] << 4)).contiguous()
    return packed, scale, zp_packed


QUANT_METHODS = ("default", "rtn", "k_quant")
# legacy compound names -> (base method, mixed-precision placement) (reference: builders/quant_config.py:285-290)
ALGO_ALIASES = {
    "default": ("default", {}), "rtn": ("rtn", {}), "k_quant": ("k_quant", {}),
    "rtn_last": ("rtn", {"last_matmul": "int8"}), "k_quant_last": ("k_quant", {"last_matmul": "int8"}),
    "k_quant_mixed": ("k_quant", {"last_matmul": "int8", "mixed_layers": "int8"}),
    "k_quant_linear": ("k_quant", {"last_matmul": "int8", "linear_attn": "int8"}),
}


def mixed_precision_layers(num_layers: int):
    """Layers whose qkv / v and down projections are promoted by `mixed_layers` (the selection llama.cpp uses for its mixed
    k-quants; reference: builders/base.py:1224-1239)."""
    return [i for i in range(num_layers) if i < num_layers / 8 or i >= 7 * num_layers / 8 or (i - round(num_layers / 8)) % 3 == 2]


def _k_quant_params(wb: torch.Tensor, nmax: int, symmetric: bool):
    """Scale (and minimum) of every block by a weighted least-squares search over candidate grids, the idea of llama.cpp's
    k-quants that the reference reaches through onnxruntime's `k_quant` algorithm: for a set of candidate scales the values are
    rounded to the grid, the (scale, minimum) that best reproduces the block under the weights |x| + rms(x) is solved in closed
    form, and the candidate with the smallest weighted error wins.  wb: [N, blocks, block] fp32."""
    if symmetric:
        half = (nmax + 1) // 2                                   # 8 for 4 bits, 128 for 8 bits
        amax_idx = wb.abs().argmax(-1, keepdim=True)
        amax = torch.gather(wb, -1, amax_idx).squeeze(-1)
        w2 = wb * wb
        best_err = torch.full_like(amax, float("inf"))
        best_scale = torch.ones_like(amax)
        for step in range(-9, 10):
            iscale = -(half + 0.1 * step) / torch.where(amax == 0, torch.ones_like(amax), amax)
            L = torch.clamp(torch.round(wb * iscale[..., None]), -half, half - 1)
            sumlx, suml2 = (w2 * wb * L).sum(-1), (w2 * L * L).sum(-1)
            sc = torch.where(suml2 > 0, sumlx / suml2.clamp(min=1e-30), torch.zeros_like(suml2))
            err = (w2 * (wb - sc[..., None] * L) ** 2).sum(-1)
            take = err < best_err
            best_err = torch.where(take, err, best_err)
            best_scale = torch.where(take, sc, best_scale)
        best_scale = torch.where(best_scale == 0, torch.ones_like(best_scale), best_scale)
        return best_scale, None
    mn = wb.amin(-1).clamp(max=0.0)
    mx = wb.amax(-1).clamp(min=0.0)
    span = (mx - mn)
    flat = span == 0
    span = torch.where(flat, torch.ones_like(span), span)
    weights = wb.abs() + wb.pow(2).mean(-1, keepdim=True).sqrt()
    sum_w, sum_x = weights.sum(-1), (weights * wb).sum(-1)
    best_scale, best_min = span / nmax, mn.clone()
    L = torch.clamp(torch.round((wb - mn[..., None]) / best_scale[..., None]), 0, nmax)
    best_err = (weights * (best_scale[..., None] * L + mn[..., None] - wb) ** 2).sum(-1)
    for step in range(21):
        iscale = (-1.0 + 0.1 * step + nmax) / span
        L = torch.clamp(torch.round(iscale[..., None] * (wb - mn[..., None])), 0, nmax)
        sum_l, sum_l2, sum_xl = (weights * L).sum(-1), (weights * L * L).sum(-1), (weights * L * wb).sum(-1)
        D = sum_w * sum_l2 - sum_l * sum_l
        ok = D > 0
        Ds = torch.where(ok, D, torch.ones_like(D))
        sc = (sum_w * sum_xl - sum_x * sum_l) / Ds
        m = (sum_l2 * sum_x - sum_l * sum_xl) / Ds
        pos = m > 0                                          # the minimum may not be positive: zero is always representable
        sc = torch.where(pos, sum_xl / sum_l2.clamp(min=1e-30), sc)
        m = torch.where(pos, torch.zeros_like(m), m)
        err = (weights * (sc[..., None] * L + m[..., None] - wb) ** 2).sum(-1)
        take = ok & (err < best_err) & (sc > 0)
        best_err = torch.where(take, err, best_err)
        best_scale = torch.where(take, sc, best_scale)
        best_min = torch.where(take, m, best_min)
    best_scale = torch.where(flat | (best_scale <= 0), torch.ones_like(best_scale), best_scale)
    return best_scale, best_min


def quantize_block(w: torch.Tensor, bits: int = 4, symmetric: bool = False, method: str = "default", block: int = 32):
    """Block quantisation in the MatMulNBits layout with the reference's three methods (builders/quant_config.py:168-173):
    `default` and `rtn` round to the grid spanned by each block's minimum and maximum (absolute maximum when symmetric),
    `k_quant` searches the grid (see _k_quant_params).  bits 4: qweight uint8 [N, K/block, block/2] (low nibble = even k), zero
    points packed two per byte; bits 8: qweight uint8 [N, K/block, block], one zero point per byte.  Scales fp32 [N, K/block];
    zero points are None when symmetric (the op's default, 8 or 128, applies)."""
    if method not in QUANT_METHODS:
        raise ValueError(f"quantisation method must be one of {list(QUANT_METHODS)}, got '{method}'")
    if bits not in (4, 8):
        raise ValueError("bits must be 4 or 8")
    if bits == 4 and method != "k_quant":
        return quantize_int4_block32(w, symmetric, block)
    N, K = w.shape
    assert K % block == 0
    nmax = (1 << bits) - 1
    half = (nmax + 1) // 2
    wb = w.float().view(N, K // block, block)
    if method == "k_quant" and not symmetric:
        # the searched (scale, minimum), then the integer zero point the op needs and one more closed-form fit of the scale for
        # the codes that zero point gives; blocks that the plain min / max grid reproduces better (under the same weights) keep it
        scale, mn = _k_quant_params(wb, nmax, False)
        weights = wb.abs() + wb.pow(2).mean(-1, keepdim=True).sqrt()

        def fit(sc, lo):
            zpf = torch.clamp(torch.round(-lo / sc), 0, nmax)
            c = torch.clamp(torch.round(wb / sc[..., None]) + zpf[..., None], 0, nmax) - zpf[..., None]
            den = (weights * c * c).sum(-1)
            sc2 = torch.where(den > 0, (weights * c * wb).sum(-1) / den.clamp(min=1e-30), sc)
            sc2 = torch.where(sc2 > 0, sc2, sc)
            c2 = torch.clamp(torch.round(wb / sc2[..., None]) + zpf[..., None], 0, nmax) - zpf[..., None]
            return sc2, zpf, (weights * (sc2[..., None] * c2 - wb) ** 2).sum(-1)

        lo0, hi0 = wb.amin(-1).clamp(max=0.0), wb.amax(-1).clamp(min=0.0)
        s0 = (hi0 - lo0) / nmax
        s0 = torch.where(s0 == 0, torch.ones_like(s0), s0)
        zp0 = torch.clamp(torch.round(-lo0 / s0), 0, nmax)
        c0 = torch.clamp(torch.round(wb / s0[..., None]) + zp0[..., None], 0, nmax) - zp0[..., None]
        e0 = (weights * (s0[..., None] * c0 - wb) ** 2).sum(-1)
        s1, zp1, e1 = fit(scale, mn)
        better = e1 < e0
        scale = torch.where(better, s1, s0)
        zpf = torch.where(better, zp1, zp0)
        mn = -zpf * scale
    elif method == "k_quant":
        scale, mn = _k_quant_params(wb, nmax, True)
    elif symmetric:
        amax_idx = wb.abs().argmax(-1, keepdim=True)
        scale = (torch.gather(wb, -1, amax_idx) / -float(half)).squeeze(-1)
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
        mn = None
    else:
        lo, hi = wb.amin(-1).clamp(max=0.0), wb.amax(-1).clamp(min=0.0)
        scale = (hi - lo) / nmax
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
        mn = lo
    if symmetric:
        q = torch.clamp(torch.round(wb / scale[..., None]) + half, 0, nmax)
        zp = None
    else:
        zpf = torch.clamp(torch.round(-mn / scale), 0, nmax)
        q = torch.clamp(torch.round(wb / scale[..., None]) + zpf[..., None], 0, nmax)
        zp = zpf.to(torch.uint8)
    q = q.to(torch.uint8)
    if bits == 8:
        return q.contiguous(), scale, zp
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).contiguous()
    zp_packed = None
    if zp is not None:
        if (K // block) % 2:
            zp = torch.cat([zp, torch.full((N, 1), 8, dtype=torch.uint8, device=zp.device)], dim=1)
        zp_packed = (zp[:, 0::2] | (zp[:, 1::2] << 4)).contiguous()
    return packed, scale, zp_packed


def dequantize_block(qweight, scales, zero_points, N: int, K: int, block: int = 32, bits: int = 4) -> torch.Tensor:
    """fp32 [N, K] from MatMulNBits tensors of 4 or 8 bits: w = (q - zp) * scale."""
    if bits == 4:
        return dequantize_int4_block32(qweight, scales, zero_points, N, K, block)
    nb = K // block
    q = torch.as_tensor(qweight).view(N, nb, block).float()
    zz = torch.as_tensor(zero_points).view(N, -1)[:, :nb].float() if zero_points is not None else torch.full((N, nb), 128.0, device=q.device)
    return ((q - zz[..., None]) * torch.as_tensor(scales).float().view(N, nb)[..., None]).view(N, K)


def dequantize_int4_block32(qweight, scales, zero_points, N: int, K: int, block: int = 32) -> torch.Tensor:
    """Inverse of quantize_int4_block32: returns fp32 [N, K] with w = (q - zp) * scale."""
    q = torch.as_tensor(qweight).view(N, K // block, block // 2)
    lo, hi = (q & 0xF).float(), (q >> 4).float()
    w = torch.stack([lo, hi], dim=-1).view(N, K // block, block)
    nb = K // block
    if zero_points is not None:
        z = torch.as_tensor(zero_points).view(N, -1)
        zz = torch.stack([(z & 0xF), (z >> 4)], dim=-1).view(N, -1)[:, :nb].float()
    else:
        zz = torch.full((N, nb), 8.0, device=q.device)
    s = torch.as_tensor(scales).float().view(N, nb)
    return ((w - zz[..., None]) * s[..., None]).view(N, K)


_FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)   # e2m1 magnitudes; bit 3 of a code is the sign


def quantize_mxfp4(w: torch.Tensor, block: int = 32):
    """MXFP4 (OCP microscaling): FP4 e2m1 codes with one power-of-two (e8m0) scale per block of 32 along K.
    w: [N, K] float.  Returns packed uint8 [K, N/2] in the QMoE layout (a byte holds two adjacent output features of
    the same k: even n in the low nibble) and the scale codes uint8 [N, K/block] (value 2^(code - 127))."""
    N, K = w.shape
    assert K % block == 0 and N % 2 == 0
    wb = w.float().view(N, K // block, block)
    amax = wb.abs().amax(-1)
    code = torch.full_like(amax, 127.0)
    nz = amax > 0
    code[nz] = torch.clamp(torch.round(torch.log2(amax[nz] / 6.0)) + 127.0, 1, 254)
    scale = torch.pow(2.0, code - 127.0)
    v = (wb / scale[..., None]).clamp(-6.0, 6.0)
    grid = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=w.device)
    idx = (v.abs()[..., None] - grid).abs().argmin(-1)        # nearest magnitude
    codes = (idx + 8 * ((v < 0) & (idx > 0)).long()).to(torch.uint8).view(N, K)
    kn = codes.t().contiguous()
    packed = (kn[:, 0::2] | (kn[:, 1::2] << 4)).contiguous()
    return packed, code.to(torch.uint8)


def dequantize_mxfp4(packed: torch.Tensor, scale_codes: torch.Tensor, N: int, K: int, block: int = 32) -> torch.Tensor:
    """Inverse of quantize_mxfp4: fp32 [N, K]."""
    pk = torch.as_tensor(packed).view(K, N // 2)
    kn = torch.stack([pk & 0xF, pk >> 4], dim=-1).view(K, N)
    codes = kn.t().long()
    grid = torch.tensor(_FP4_VALUES, dtype=torch.float32, device=pk.device)
    mag = grid[codes & 7]
    val = torch.where(codes >= 8, -mag, mag)
    scale = torch.pow(2.0, torch.as_tensor(scale_codes).view(N, K // block).float() - 127.0)
    return (val.view(N, K // block, block) * scale[..., None]).view(N, K)


def quantize_fp8_rows(w: torch.Tensor):
    """FP8 e4m3 weights with one scale per output row: (uint8 view of float8_e4m3fn [N, K], fp32 scale [N, 1])."""
    scale = (w.float().abs().amax(1, keepdim=True) / 448.0).clamp(min=1e-12)
    return (w.float() / scale).to(torch.float8_e4m3fn).view(torch.uint8), scale


def quantize_nvfp4(w: torch.Tensor):
    """NVFP4: e2m1 codes with an e4m3 scale per block of 16 along K and one fp32 global scale.
    Returns (codes uint8 [N, K/2], low nibble = even k; uint8 view of the e4m3 scales [N, K/16]; global scale fp32 [1])."""
    N, K = w.shape
    assert K % 16 == 0
    wf = w.float()
    glob = (wf.abs().amax() / (6.0 * 448.0)).clamp(min=1e-12)
    wb = wf.view(N, K // 16, 16)
    sc = (wb.abs().amax(-1) / 6.0 / glob).to(torch.float8_e4m3fn)
    eff = (sc.float() * glob).clamp(min=1e-20)
    v = (wb / eff[..., None]).clamp(-6.0, 6.0)
    grid = torch.tensor(_FP4_VALUES, dtype=torch.float32)
    idx = (v.abs()[..., None] - grid).abs().argmin(-1)
    codes = (idx + 8 * ((v < 0) & (idx > 0)).long()).to(torch.uint8).view(N, K)
    return (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous(), sc.view(torch.uint8), glob.reshape(1)


def dequantize_nvfp4(packed: torch.Tensor, scales_e4m3: torch.Tensor, global_scale: torch.Tensor) -> torch.Tensor:
    """Inverse of quantize_nvfp4: fp32 [N, K]."""
    pk = torch.as_tensor(packed)
    N, K = pk.shape[0], pk.shape[1] * 2
    codes = torch.stack([pk & 0xF, pk >> 4], dim=-1).view(N, K).long()
    grid = torch.tensor(_FP4_VALUES, dtype=torch.float32)
    val = torch.where(codes >= 8, -grid[codes & 7], grid[codes & 7])
    sc = torch.as_tensor(scales_e4m3).view(torch.float8_e4m3fn).float().view(N, K // 16) * torch.as_tensor(global_scale).float().reshape(())
    return (val.view(N, K // 16, 16) * sc[..., None]).view(N, K)


# ---------------------------------------------------------------------------------------------- export
class _Writer:
    def __init__(self, out_dir: str, precision: str, synthetic: bool, seed: int, std: float, filename: str = "model.onnx"):
        self.model = op.Model()
        self.precision = precision
        self.io = "fp32" if precision == "fp32" else ("bf16" if precision in ("bf16", "int4") else "fp16")
        self.ext = None if synthetic else op.ExternalDataWriter(os.path.join(out_dir, filename + ".data"))
        self.synthetic = synthetic
        self.seed, self.std = seed, std

    def add_array(self, name: str, arr: np.ndarray, onnx_dtype: int, dims=None):
        if self.ext is None:
            t = op.Tensor(name=name, dtype=onnx_dtype, dims=tuple(dims if dims is not None else arr.shape),
                          raw=np.ascontiguousarray(arr).tobytes())
        else:
            t = self.ext.add(name, onnx_dtype, arr, dims)
        self.model.initializers[name] = t

    def add_float(self, name: str, t: torch.Tensor, force_fp32: bool = False):
        prec = "fp32" if force_fp32 else self.io
        tt = t.detach().to(_TORCH_DT[prec]).contiguous()
        arr = tt.view(torch.int16).numpy() if prec == "bf16" else tt.numpy()
        self.add_array(name, arr, _ONNX_DT[prec], dims=tuple(tt.shape))

    def add_synthetic(self, name: str, shape, kind: str, onnx_dtype: Optional[int] = None):
        t = op.Tensor(name=name, dtype=_ONNX_DT[self.io] if onnx_dtype is None else onnx_dtype, dims=tuple(shape))
        t.ext_location = "synthetic"
        t.ext_offset = 0
        t.ext_length = 0
        t.raw = None
        self.model.initializers[name] = t

    def node(self, op_type, name, inputs, outputs, domain="", **attrs):
        self.model.nodes.append(op.Node(op_type=op_type, name=name, inputs=list(inputs), outputs=list(outputs), domain=domain, attrs=attrs))


def export_model(arch: ArchConfig, out_dir: str, precision: str = "bf16", execution_provider: str = "cuda",
                 state_dict: Optional[Dict[str, torch.Tensor]] = None, seed: int = 0, std: float = 0.02,
                 paged: bool = False, block_size: int = 16, max_batch_size: int = 64, int4_symmetric: bool = False,
                 synthetic_weights: bool = False, search: Optional[dict] = None, engine: Optional[dict] = None,
                 filename: str = "model.onnx", write_config: bool = True, speculative: Optional[dict] = None,
                 draft_dir_entry: Optional[dict] = None, num_blocks: Optional[int] = None,
                 max_scheduled_tokens: Optional[int] = None, context_length: Optional[int] = None,
                 int4_tied_embeddings: bool = False, linear_format: str = "", int4_algo_config: str = "default",
                 mixed_precision: Optional[dict] = None) -> str:
    """Writes a checkpoint directory.  With state_dict=None the weights are random N(0, std) from `seed`.
    int4_algo_config: quantisation method `default` | `rtn` | `k_quant`, or one of the reference's compound names (`rtn_last`,
    `k_quant_last`, `k_quant_mixed`, `k_quant_linear`); mixed_precision: selector -> type, e.g. {"last_matmul": "int8",
    "mixed_layers": "int8"} (the LM head; the qkv and down projections of the layers llama.cpp's mixed k-quants promote)."""
    os.makedirs(out_dir, exist_ok=True)
    if int4_algo_config not in ALGO_ALIASES:
        raise ValueError(f"int4_algo_config must be one of {sorted(ALGO_ALIASES)}, got '{int4_algo_config}'")
    quant_method, placement = ALGO_ALIASES[int4_algo_config]
    placement = {**placement, **(mixed_precision or {})}
    for sel, typ in placement.items():
        if sel not in ("last_matmul", "mixed_layers", "linear_attn") or typ not in ("int4", "int8"):
            raise ValueError(f"mixed_precision: unknown selector or type {sel}={typ}")
    promoted = set(mixed_precision_layers(arch.num_layers)) if placement.get("mixed_layers") == "int8" else set()

    def bits_of(node_name: str) -> int:
        if node_name == "/lm_head/MatMul":
            return 8 if placement.get("last_matmul") == "int8" else 4
        m = re.match(r"/model/layers\.(\d+)/(attn/qkv_proj|mlp/down_proj)/MatMul$", node_name)
        return 8 if (m and int(m.group(1)) in promoted) else 4
    if precision not in ("fp32", "fp16", "bf16", "int4"):
        raise ValueError(f"unsupported precision {precision}")
    if context_length:
        arch.context_length = context_length
    W = _Writer(out_dir, precision, synthetic_weights, seed, std, filename)
    shapes = weight_shapes(arch)

    def get(name: str) -> torch.Tensor:
        if state_dict is not None:
            if name == "lm_head.weight" and name not in state_dict:
                return state_dict["model.embed_tokens.weight"]
            return state_dict[name]
        return random_tensor(name, shapes[name], seed, std)

    synth_meta: Dict[str, dict] = {}

    def put_plain(onnx_name: str, src_names, transform=None, force_fp32=False):
        """Adds an initializer built from canonical tensors (or a synthetic descriptor)."""
        if synthetic_weights:
            W.add_synthetic(onnx_name, transform["shape"], "")
            synth_meta[onnx_name] = {"sources": src_names, "op": transform["op"], "seed": seed, "std": std}
            return
        ts = [get(n) for n in src_names]
        W.add_float(onnx_name, transform["fn"](ts), force_fp32)

    def put_linear(base: str, node_name: str, src_names, inp: str, out: str, N: int, K: int):
        """A linear layer y = x @ W^T from one or more stacked [n_i, K] canonical weights."""
        pre = [get(n) for n in src_names] if (state_dict is not None and not synthetic_weights) else []
        pre_kind = getattr(pre[0], "kind", "") if pre and all(getattr(t, "kind", "") == getattr(pre[0], "kind", "") for t in pre) else ""
        carried = type(pre[0]).cat(pre) if pre_kind in ("fp8", "nvfp4") else None
        if carried is not None or (linear_format in ("fp8", "nvfp4") and not synthetic_weights):
            # block-quantised float formats: FP8 e4m3 rows or NVFP4 blocks of 16, quantised here (linear_format option) or
            # carried over from a ModelOpt checkpoint
            fmt = pre_kind if carried is not None else linear_format
            w = None if carried is not None else torch.cat([get(n).float() for n in src_names], dim=0)
            if fmt == "fp8":
                q8, sc = (carried.q8, carried.scale) if carried is not None else quantize_fp8_rows(w)
                W.add_array(base + ".fp8_weight", q8.numpy(), op.FLOAT8E4M3FN)
                W.add_array(base + ".fp8_weight_scale", sc.numpy(), op.FLOAT)
                W.node("MatMulBlockQuantizedFp8Weight", node_name, [inp, base + ".fp8_weight", base + ".fp8_weight_scale"], [out],
                       domain="com.microsoft", block_size=K)
            else:
                codes, sc, glob = (carried.codes, carried.scales, carried.global_scale) if carried is not None else quantize_nvfp4(w)
                W.add_array(base + ".nvfp4_weight", codes.numpy(), op.UINT8)
                W.add_array(base + ".nvfp4_weight_scale", sc.numpy(), op.FLOAT8E4M3FN)
                W.add_array(base + ".nvfp4_weight_scale_2", glob.numpy(), op.FLOAT)
                W.node("MatMulBlockQuantizedFp4Weight", node_name, [inp, base + ".nvfp4_weight", base + ".nvfp4_weight_scale",
                                                                    base + ".nvfp4_weight_scale_2"], [out], domain="com.microsoft", block_size=16)
        elif precision == "int4" and synthetic_weights:
            # descriptors only: the loader draws the float weight on the device and quantises it there (RTN block-32)
            nb = K // 32
            for suffix, shp, dt, kind in (("weight_Q4", (N, nb, 16), op.UINT8, "q4_weight"), ("weight_scales", (N * nb,), op.FLOAT16, "q4_scales"),
                                          ("weight_zp", (N * ((nb + 1) // 2),), op.UINT8, "q4_zp")):
                if kind == "q4_zp" and int4_symmetric:
                    continue
                W.add_synthetic(f"{base}.MatMul.{suffix}", shp, "", dt)
                synth_meta[f"{base}.MatMul.{suffix}"] = {"sources": src_names, "op": kind, "seed": seed, "std": std, "symmetric": int(int4_symmetric)}
            ins = [inp, base + ".MatMul.weight_Q4", base + ".MatMul.weight_scales"] + ([] if int4_symmetric else [base + ".MatMul.weight_zp"])
            W.node("MatMulNBits", node_name + "_Q4", ins, [out], domain="com.microsoft", K=K, N=N, bits=4, block_size=32, accuracy_level=4)
        elif precision == "int4":
            srcs = [get(n) for n in src_names]
            if all(hasattr(t, "matmulnbits") for t in srcs):
                # AWQ / GPTQ checkpoint: the quantised tensors are carried over, not quantised a second time
                from .quantized_checkpoint import QuantizedLinear
                q, s, zp = QuantizedLinear.cat(srcs).matmulnbits()
            else:
                nbits = bits_of(node_name)
                q, s, zp = quantize_block(torch.cat([t.float() for t in srcs], dim=0), nbits, int4_symmetric, quant_method)
                if nbits == 8:
                    # promoted node (mixed precision): 8-bit MatMulNBits, one byte per weight, zero points unpacked
                    W.add_array(base + ".MatMul.weight_Q8", q.numpy(), op.UINT8)
                    W.add_array(base + ".MatMul.weight_scales", s.reshape(-1).to(torch.float16).numpy(), op.FLOAT16)
                    ins = [inp, base + ".MatMul.weight_Q8", base + ".MatMul.weight_scales"]
                    if zp is not None:
                        W.add_array(base + ".MatMul.weight_zp", zp.reshape(-1).numpy(), op.UINT8)
                        ins.append(base + ".MatMul.weight_zp")
                    W.node("MatMulNBits", node_name + "_Q8", ins, [out], domain="com.microsoft", K=K, N=N, bits=8, block_size=32, accuracy_level=4)
                    return
            W.add_array(base + ".MatMul.weight_Q4", q.numpy(), op.UINT8)
            W.add_array(base + ".MatMul.weight_scales", s.reshape(-1).to(torch.float16).numpy(), op.FLOAT16)
            ins = [inp, base + ".MatMul.weight_Q4", base + ".MatMul.weight_scales"]
            if zp is not None:
                W.add_array(base + ".MatMul.weight_zp", zp.reshape(-1).numpy(), op.UINT8)
                ins.append(base + ".MatMul.weight_zp")
            W.node("MatMulNBits", node_name + "_Q4", ins, [out], domain="com.microsoft", K=K, N=N, bits=4, block_size=32,
                   accuracy_level=4)
        else:
            put_plain(base + ".MatMul.weight", src_names,
                      {"shape": (K, N), "op": "cat_t", "fn": lambda ts: torch.cat([t.float() for t in ts], 0).t().contiguous()})
            W.node("MatMul", node_name, [inp, base + ".MatMul.weight"], [out])

    def put_vec(onnx_name: str, src_names, offset: float = 0.0):
        if synthetic_weights:
            shp = (sum(shapes[n][0] for n in src_names),)
            W.add_synthetic(onnx_name, shp, "")
            synth_meta[onnx_name] = {"sources": src_names, "op": "cat", "seed": seed, "std": std, "offset": offset}
            return
        W.add_float(onnx_name, torch.cat([get(n).float() for n in src_names], 0) + offset)

    H, I, V, L = arch.hidden_size, arch.intermediate_size, arch.vocab_size, arch.num_layers
    io_dt = _ONNX_DT[W.io]

    # ---- embedding
    tied_q4 = int4_tied_embeddings and precision == "int4" and arch.tie_embeddings
    if tied_q4:
        # one int4 tensor serves the LM head (MatMulNBits) and the embedding (rows gathered and dequantised by block)
        W.model.initializers["/model/constants/INT64/embed_shape"] = op.Tensor("/model/constants/INT64/embed_shape", op.INT64, (2,),
                                                                               raw=np.asarray([V, H // 2], dtype=np.int64).tobytes())
        W.node("Reshape", "/model/embed_tokens/Reshape", ["lm_head.MatMul.weight_Q4", "/model/constants/INT64/embed_shape"],
               ["/model/embed_tokens/Reshape/output_0"])
        gins = ["/model/embed_tokens/Reshape/output_0", "input_ids", "lm_head.MatMul.weight_scales"] + ([] if int4_symmetric else ["lm_head.MatMul.weight_zp"])
        W.node("GatherBlockQuantized", "/model/embed_tokens/GatherBlockQuantized", gins, ["/model/embed_tokens/GatherBlockQuantized/output_0"],
               domain="com.microsoft", bits=4, block_size=32, gather_axis=0, quantize_axis=1)
        hidden = "/model/embed_tokens/GatherBlockQuantized/output_0"
    else:
        put_plain("model.embed_tokens.weight", ["model.embed_tokens.weight"],
                  {"shape": (V, H), "op": "id", "fn": lambda ts: ts[0].float()})
        W.node("Gather", "/model/embed_tokens/Gather", ["model.embed_tokens.weight", "input_ids"], ["/model/embed_tokens/Gather/output_0"])
        hidden = "/model/embed_tokens/Gather/output_0"
    if arch.embed_scale != 1.0:
        W.model.initializers["/model/constants/embed_scale"] = op.Tensor("/model/constants/embed_scale", op.FLOAT, (),
                                                                         raw=np.float32(arch.embed_scale).tobytes())
        W.node("Mul", "/model/embed_tokens/Mul", [hidden, "/model/constants/embed_scale"], ["/model/embed_tokens/Mul/output_0"])
        hidden = "/model/embed_tokens/Mul/output_0"

    if arch.learned_positions:
        # gpt2: a learned table indexed by position joins the token embedding; attention then runs without rotary embedding
        put_plain("model.position_embeddings.weight", ["model.position_embeddings.weight"],
                  {"shape": (arch.context_length, H), "op": "id", "fn": lambda ts: ts[0].float()})
        W.node("Gather", "/model/pos_embed/Gather", ["model.position_embeddings.weight", "position_ids"], ["/model/pos_embed/Gather/output_0"])
        W.node("Add", "/model/pos_embed/Add", [hidden, "/model/pos_embed/Gather/output_0"], ["/model/pos_embed/Add/output_0"])
        hidden = "/model/pos_embed/Add/output_0"

    # ---- rotary caches
    multi = longrope_caches(arch)
    if multi is not None:
        # two cache pairs and the length at which the model switches from the short to the long one
        for nm, arr in zip(("cos_cache_small", "sin_cache_small", "cos_cache_large", "sin_cache_large"), multi[:4]):
            W.add_float(nm, torch.from_numpy(arr), force_fp32=(precision == "fp32"))
        W.model.initializers["/model/rope_caches_subgraph/original_context_length"] = op.Tensor(
            "/model/rope_caches_subgraph/original_context_length", op.INT64, (), raw=np.int64(multi[4]).tobytes())
    cos, sin = rope_caches(arch)
    W.add_float("cos_cache", torch.from_numpy(cos), force_fp32=(precision == "fp32"))
    W.add_float("sin_cache", torch.from_numpy(sin), force_fp32=(precision == "fp32"))
    if arch.rope_local_theta:
        # sliding-window layers rotate with their own base (reference: builders/gemma.py:144-158, cos_cache_local / sin_cache_local)
        cos, sin = rope_caches(arch, local=True)
        W.add_float("cos_cache_local", torch.from_numpy(cos), force_fp32=(precision == "fp32"))
        W.add_float("sin_cache_local", torch.from_numpy(sin), force_fp32=(precision == "fp32"))

    if arch.residual_multiplier != 1.0:
        W.model.initializers["/model/constants/residual_multiplier"] = op.Tensor(
            "/model/constants/residual_multiplier", op.FLOAT, (), raw=np.float32(arch.residual_multiplier).tobytes())

    def residual_scale(name: str, value: str) -> str:
        """Granite-style residual multiplier: the sub-layer output is scaled before it joins the residual stream."""
        if arch.residual_multiplier == 1.0:
            return value
        W.node("Mul", name, [value, "/model/constants/residual_multiplier"], [name + "/output_0"])
        return name + "/output_0"

    norm_op = "LayerNormalization" if arch.layernorm else "SimplifiedLayerNormalization"
    skip_op = "SkipLayerNormalization" if arch.layernorm else "SkipSimplifiedLayerNormalization"
    attn_op = "PagedAttention" if paged else "GroupQueryAttention"
    residual = None
    for i in range(L):
        p, n = f"model.layers.{i}.", f"/model/layers.{i}"
        # input norm
        put_vec(p + "input_layernorm.weight", [p + "input_layernorm.weight"], arch.norm_offset)
        ins = [hidden, p + "input_layernorm.weight"] if residual is None else [hidden, residual, p + "input_layernorm.weight"]
        if arch.layernorm:
            put_vec(p + "input_layernorm.bias", [p + "input_layernorm.bias"])
            ins.append(p + "input_layernorm.bias")
        outs = [f"{n}/input_layernorm/output_0"] + ([] if residual is None else ["", "", f"{n}/input_layernorm/output_3"])
        W.node(norm_op if residual is None else skip_op, f"{n}/input_layernorm/{'LayerNorm' if residual is None else 'SkipLayerNorm'}",
               ins, outs, domain="" if residual is None else "com.microsoft", epsilon=float(arch.norm_eps),
               **({"axis": -1, "stash_type": 1} if residual is None else {}),
               **({} if arch.pre_norm else {"bypass": 1}))     # bypass: the node only adds (its unit weights are placeholders)
        residual = hidden if residual is None else f"{n}/input_layernorm/output_3"
        x = f"{n}/input_layernorm/output_0"
        if arch.is_conv_layer(i):
            # hybrid (LFM2) layer: in_proj -> (b, c, x); depthwise convolution of b * x over the last conv_L_cache positions
            # (state input past_conv.N / output present_conv.N); c * conv -> out_proj
            Lc = arch.conv_L_cache
            put_linear(p + "conv.in_proj", f"{n}/conv/in_proj/MatMul", [p + "conv.in_proj.weight"], x, f"{n}/conv/in_proj/MatMul/output_0", 3 * H, H)
            W.node("Split", f"{n}/conv/Split", [f"{n}/conv/in_proj/MatMul/output_0"], [f"{n}/conv/b", f"{n}/conv/c", f"{n}/conv/x"], axis=-1, num_outputs=3)
            W.node("Mul", f"{n}/conv/Mul_1", [f"{n}/conv/b", f"{n}/conv/x"], [f"{n}/conv/Mul_1/output_0"])
            W.node("Concat", f"{n}/conv/Conv_1", [f"past_conv.{i}", f"{n}/conv/Mul_1/output_0"], [f"{n}/conv/Conv_1/output_0"], axis=1)
            put_plain(p + "conv.conv.weight", [p + "conv.conv.weight"], {"shape": (H, 1, Lc), "op": "id", "fn": lambda ts: ts[0].float().reshape(H, 1, Lc)})
            cins = [f"{n}/conv/Conv_1/output_0", p + "conv.conv.weight"]
            if arch.conv_bias:
                put_vec(p + "conv.conv.bias", [p + "conv.conv.bias"])
                cins.append(p + "conv.conv.bias")
            W.node("Conv", f"{n}/conv/Conv_2", cins, [f"{n}/conv/Conv_2/output_0"], kernel_shape=[Lc], group=H, pads=[0, 0])
            W.node("Mul", f"{n}/conv/Mul_2", [f"{n}/conv/c", f"{n}/conv/Conv_2/output_0"], [f"{n}/conv/Mul_2/output_0"])
            W.node("Identity", f"{n}/conv/present", [f"{n}/conv/Conv_1/output_0"], [f"present_conv.{i}"])
            o_out = f"{n}/conv/out_proj/MatMul/output_0"
            put_linear(p + "conv.out_proj", f"{n}/conv/out_proj/MatMul", [p + "conv.out_proj.weight"], f"{n}/conv/Mul_2/output_0", o_out, H, H)
        elif arch.is_mamba_layer(i):
            # Mamba-2 layer: in_proj -> [gate | x, B, C | dt], causal depthwise convolution + SiLU with a carried window, the selective
            # scan with a carried state, gated RMS norm, out_proj
            mb = f"{n}/mamba"
            mp = p + "mamba."
            Im, cd, nh = arch.mamba_intermediate, arch.mamba_conv_dim, arch.mamba_num_heads
            Kc = arch.mamba_conv_kernel
            put_linear(mp + "in_proj", f"{mb}/in_proj/MatMul", [mp + "in_proj.weight"], x, f"{mb}/in_proj/MatMul/output_0", Im + cd + nh, H)
            put_plain(mp + "conv1d.weight", [mp + "conv1d.weight"], {"shape": (cd, 1, Kc), "op": "id", "fn": lambda ts: ts[0].float().reshape(cd, 1, Kc)})
            put_vec(mp + "conv1d.bias", [mp + "conv1d.bias"])
            put_plain(mp + "dt_bias", [mp + "dt_bias"], {"shape": (nh,), "op": "id", "fn": lambda ts: ts[0].float()}, force_fp32=True)
            put_plain(mp + "neg_exp_A", [mp + "A_log"], {"shape": (nh,), "op": "neg_exp", "fn": lambda ts: -torch.exp(ts[0].float())}, force_fp32=True)
            put_plain(mp + "D", [mp + "D"], {"shape": (nh,), "op": "id", "fn": lambda ts: ts[0].float()}, force_fp32=True)
            put_plain(mp + "norm.weight", [mp + "norm.weight"], {"shape": (Im,), "op": "id", "fn": lambda ts: ts[0].float()})
            W.node("Split", f"{mb}/Split", [f"{mb}/in_proj/MatMul/output_0"], [f"{mb}/Split/output_{j}" for j in range(3)], axis=-1, split=[Im, cd, nh])
            W.node("Transpose", f"{mb}/xbc/Transpose", [f"{mb}/Split/output_1"], [f"{mb}/xbc/Transpose/output_0"], perm=[0, 2, 1])
            W.node("CausalConvWithState", f"{mb}/CausalConvWithState", [f"{mb}/xbc/Transpose/output_0", mp + "conv1d.weight", mp + "conv1d.bias", f"past_key_values.{i}.conv_state"],
                   [f"{mb}/CausalConvWithState/output_0", f"present.{i}.conv_state"], domain="com.microsoft", ndim=1, activation="silu")
            W.node("Transpose", f"{mb}/conv_out/Transpose", [f"{mb}/CausalConvWithState/output_0"], [f"{mb}/conv_out/Transpose/output_0"], perm=[0, 2, 1])
            W.node("Mamba2", f"{mb}/Mamba2", [f"{mb}/conv_out/Transpose/output_0", f"{mb}/Split/output_2", mp + "dt_bias", mp + "neg_exp_A", mp + "D",
                                              f"past_key_values.{i}.recurrent_state"],
                   [f"{mb}/Mamba2/output_0", f"present.{i}.recurrent_state"], domain="com.microsoft", num_heads=nh, head_dim=arch.mamba_head_dim,
                   state_size=arch.mamba_state_size, n_groups=arch.mamba_n_groups)
            W.node("Sigmoid", f"{mb}/gated_norm/Sigmoid", [f"{mb}/Split/output_0"], [f"{mb}/gated_norm/Sigmoid/output_0"])
            W.node("Mul", f"{mb}/gated_norm/Mul_1", [f"{mb}/Split/output_0", f"{mb}/gated_norm/Sigmoid/output_0"], [f"{mb}/gated_norm/Mul_1/output_0"])
            W.node("Mul", f"{mb}/gated_norm/Mul_2", [f"{mb}/Mamba2/output_0", f"{mb}/gated_norm/Mul_1/output_0"], [f"{mb}/gated_norm/Mul_2/output_0"])
            W.node("SimplifiedLayerNormalization", f"{mb}/gated_norm/LayerNorm", [f"{mb}/gated_norm/Mul_2/output_0", mp + "norm.weight"],
                   [f"{mb}/gated_norm/LayerNorm/output_0"], epsilon=float(arch.norm_eps), axis=-1, stash_type=1)
            o_out = f"{mb}/out_proj/MatMul/output_0"
            put_linear(mp + "out_proj", f"{mb}/out_proj/MatMul", [mp + "out_proj.weight"], f"{mb}/gated_norm/LayerNorm/output_0", o_out, H, Im)
        elif arch.is_linear_layer(i):
            # gated-delta-net layer (reference graph: builders/qwen.py:1776-1867): projections, causal depthwise convolution + SiLU
            # with a carried state, per-head L2 norm of q / k, decay / beta gates, LinearAttention (gated delta rule) with a
            # recurrent state, gated RMS norm, output projection
            la = f"{n}/linear_attn"
            lp = p + "linear_attn."
            nk, nv, hk, hv, Kc = arch.linear_num_key_heads, arch.linear_num_value_heads, arch.linear_key_head_dim, arch.linear_value_head_dim, arch.linear_conv_kernel_dim
            cd, vd = arch.linear_conv_dim, arch.linear_value_dim
            put_linear(lp + "in_proj_qkv", f"{la}/in_proj_qkv/MatMul", [lp + "in_proj_qkv.weight"], x, f"{la}/in_proj_qkv/MatMul/output_0", cd, H)
            put_linear(lp + "in_proj_z", f"{la}/in_proj_z/MatMul", [lp + "in_proj_z.weight"], x, f"{la}/in_proj_z/MatMul/output_0", vd, H)
            put_linear(lp + "in_proj_b", f"{la}/in_proj_b/MatMul", [lp + "in_proj_b.weight"], x, f"{la}/in_proj_b/MatMul/output_0", nv, H)
            put_linear(lp + "in_proj_a", f"{la}/in_proj_a/MatMul", [lp + "in_proj_a.weight"], x, f"{la}/in_proj_a/MatMul/output_0", nv, H)
            put_plain(lp + "conv1d.weight", [lp + "conv1d.weight"], {"shape": (cd, 1, Kc), "op": "id", "fn": lambda ts: ts[0].float().reshape(cd, 1, Kc)})
            W.node("Transpose", f"{la}/qkv/Transpose", [f"{la}/in_proj_qkv/MatMul/output_0"], [f"{la}/qkv/Transpose/output_0"], perm=[0, 2, 1])
            W.node("CausalConvWithState", f"{la}/CausalConvWithState", [f"{la}/qkv/Transpose/output_0", lp + "conv1d.weight", "", f"past_key_values.{i}.conv_state"],
                   [f"{la}/CausalConvWithState/output_0", f"present.{i}.conv_state"], domain="com.microsoft", ndim=1, activation="silu")
            W.node("Transpose", f"{la}/conv_out/Transpose", [f"{la}/CausalConvWithState/output_0"], [f"{la}/conv_out/Transpose/output_0"], perm=[0, 2, 1])
            put_plain(lp + "dt_bias", [lp + "dt_bias"], {"shape": (nv,), "op": "id", "fn": lambda ts: ts[0].float()}, force_fp32=True)
            put_plain(lp + "neg_exp_A", [lp + "A_log"], {"shape": (nv,), "op": "neg_exp", "fn": lambda ts: -torch.exp(ts[0].float())}, force_fp32=True)
            W.node("LinearAttentionGate", f"{la}/gate/LinearAttentionGate", [f"{la}/in_proj_a/MatMul/output_0", lp + "dt_bias", lp + "neg_exp_A", f"{la}/in_proj_b/MatMul/output_0"],
                   [f"{la}/gate/LinearAttentionGate/output_0", f"{la}/gate/LinearAttentionGate/output_1"], domain="com.microsoft")
            W.node("LinearAttention", f"{la}/LinearAttention",
                   [f"{la}/conv_out/Transpose/output_0", "", "", f"past_key_values.{i}.recurrent_state", f"{la}/gate/LinearAttentionGate/output_0",
                    f"{la}/gate/LinearAttentionGate/output_1"],
                   [f"{la}/LinearAttention/output_0", f"present.{i}.recurrent_state"], domain="com.microsoft", q_num_heads=nk, kv_num_heads=nv,
                   update_rule="gated_delta", scale=float(1.0 / (hk ** 0.5)), key_head_dim=hk, value_head_dim=hv, packed_qkv=1, l2_normalize_qk=1)
            put_plain(lp + "norm.weight", [lp + "norm.weight"], {"shape": (hv,), "op": "id", "fn": lambda ts: ts[0].float()})
            W.node("SimplifiedLayerNormalization", f"{la}/gated_norm/LayerNorm", [f"{la}/LinearAttention/output_0", lp + "norm.weight"],
                   [f"{la}/gated_norm/LayerNorm/output_0"], epsilon=float(arch.norm_eps), axis=-1, stash_type=1, per_head=hv)
            W.node("Sigmoid", f"{la}/gated_norm/Sigmoid", [f"{la}/in_proj_z/MatMul/output_0"], [f"{la}/gated_norm/Sigmoid/output_0"])
            W.node("Mul", f"{la}/gated_norm/Mul_1", [f"{la}/in_proj_z/MatMul/output_0", f"{la}/gated_norm/Sigmoid/output_0"], [f"{la}/gated_norm/Mul_1/output_0"])
            W.node("Mul", f"{la}/gated_norm/Mul_2", [f"{la}/gated_norm/LayerNorm/output_0", f"{la}/gated_norm/Mul_1/output_0"], [f"{la}/gated_norm/Mul_2/output_0"])
            o_out = f"{la}/out_proj/MatMul/output_0"
            put_linear(lp + "out_proj", f"{la}/out_proj/MatMul", [lp + "out_proj.weight"], f"{la}/gated_norm/Mul_2/output_0", o_out, H, vd)
        else:
            # attention
            qkv_out = f"{n}/attn/qkv_proj/MatMul/output_0"
            put_linear(p + "attn.qkv_proj", f"{n}/attn/qkv_proj/MatMul",
                       [p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"], x, qkv_out,
                       arch.q_size + 2 * arch.kv_size, H)
            if arch.attn_bias:
                put_vec(p + "attn.qkv_proj.Add.bias", [p + "self_attn.q_proj.bias", p + "self_attn.k_proj.bias", p + "self_attn.v_proj.bias"])
                W.node("Add", f"{n}/attn/qkv_proj/Add", [qkv_out, p + "attn.qkv_proj.Add.bias"], [f"{n}/attn/qkv_proj/Add/output_0"])
                qkv_out = f"{n}/attn/qkv_proj/Add/output_0"
            attn_inputs = [qkv_out, "", ""]
            rope_mode = arch.layer_rope_mode(i)
            cos_name, sin_name = ("cos_cache_local", "sin_cache_local") if rope_mode == 1 else ("cos_cache", "sin_cache")
            if paged:
                attn_inputs += [f"past_key_values.{i}.key", f"past_key_values.{i}.value", "cumulative_sequence_lengths",
                                "past_sequence_lengths", "block_table_windowed" if arch.layer_window(i) else "block_table",
                                cos_name, sin_name, ""]
            else:
                attn_inputs += [f"past_key_values.{i}.key", f"past_key_values.{i}.value", "/model/attn_mask_reformat/seqlens_k",
                                "/model/attn_mask_reformat/total_seq_len", cos_name, sin_name, "", ""]
            if arch.attn_sinks:
                put_plain(p + "attn.sinks", [p + "self_attn.sinks"], {"shape": (arch.num_heads,), "op": "id", "fn": lambda ts: ts[0].float()})
                attn_inputs.append(p + "attn.sinks")
            else:
                attn_inputs.append("")
            if arch.qk_norm:
                put_vec(p + "attn.q_norm.layernorm.weight", [p + "self_attn.q_norm.weight"], arch.norm_offset)
                put_vec(p + "attn.k_norm.layernorm.weight", [p + "self_attn.k_norm.weight"], arch.norm_offset)
                attn_inputs += ["", ""] if not paged else []
                attn_inputs += [p + "attn.q_norm.layernorm.weight", p + "attn.k_norm.layernorm.weight"]
            attrs = dict(num_heads=arch.num_heads, kv_num_heads=arch.num_kv_heads, scale=float(arch.scale),
                         local_window_size=int(arch.layer_window(i)) if arch.layer_window(i) else -1, softcap=float(arch.softcap),
                         do_rotary=0 if rope_mode == 2 else 1, rotary_interleaved=int(arch.rotary_interleaved))
            if arch.qk_norm:
                attrs["qk_norm_epsilon"] = float(arch.norm_eps)
                if arch.qk_norm_after_rope:
                    attrs["qk_norm_after_rotary"] = 1
                if arch.qk_norm_full_width:
                    attrs["qk_norm_full_width"] = 1
            if arch.mrope_section:
                attrs["mrope_section"] = [int(v) for v in arch.mrope_section]   # position_ids then carry three components per token
                if arch.mrope_interleaved:
                    attrs["mrope_interleaved"] = 1
            if arch.rotary_dim != arch.head_dim:
                attrs["rotary_embedding_dim"] = int(arch.rotary_dim)
            W.node(attn_op, f"{n}/attn/{attn_op}", attn_inputs, [f"{n}/attn/{attn_op}/output_0", f"present.{i}.key", f"present.{i}.value"],
                   domain="com.microsoft", **attrs)
            o_in = f"{n}/attn/{attn_op}/output_0"
            if arch.attn_output_gate:
                # the attention output is scaled by sigmoid of a second projection of the layer input (stored as the odd head-halves of q_proj)
                put_linear(p + "attn.gate_proj", f"{n}/attn/gate_proj/MatMul", [p + "self_attn.gate_proj.weight"], x, f"{n}/attn/gate_proj/MatMul/output_0",
                           arch.q_size, H)
                W.node("Sigmoid", f"{n}/attn/gate/Sigmoid", [f"{n}/attn/gate_proj/MatMul/output_0"], [f"{n}/attn/gate/Sigmoid/output_0"])
                W.node("Mul", f"{n}/attn/gate/Mul", [o_in, f"{n}/attn/gate/Sigmoid/output_0"], [f"{n}/attn/gate/Mul/output_0"])
                o_in = f"{n}/attn/gate/Mul/output_0"
            o_out = f"{n}/attn/o_proj/MatMul/output_0"
            put_linear(p + "attn.o_proj", f"{n}/attn/o_proj/MatMul", [p + "self_attn.o_proj.weight"], o_in, o_out,
                       H, arch.q_size)
            if arch.o_bias:
                put_vec(p + "attn.o_proj.Add.bias", [p + "self_attn.o_proj.bias"])
                W.node("Add", f"{n}/attn/o_proj/Add", [o_out, p + "attn.o_proj.Add.bias"], [f"{n}/attn/o_proj/Add/output_0"])
                o_out = f"{n}/attn/o_proj/Add/output_0"
        if arch.cross_attention:
            # encoder-decoder: queries from the decoder stream, keys / values projected once from the encoder output
            put_vec(p + "cross_attn_layernorm.weight", [p + "cross_attn_layernorm.weight"], arch.norm_offset)
            ins = [o_out, residual, p + "cross_attn_layernorm.weight"]
            if arch.layernorm:
                put_vec(p + "cross_attn_layernorm.bias", [p + "cross_attn_layernorm.bias"])
                ins.append(p + "cross_attn_layernorm.bias")
            W.node(skip_op, f"{n}/cross_attn_layernorm/SkipLayerNorm", ins,
                   [f"{n}/cross_attn_layernorm/output_0", "", "", f"{n}/cross_attn_layernorm/output_3"], domain="com.microsoft",
                   epsilon=float(arch.norm_eps))
            residual = f"{n}/cross_attn_layernorm/output_3"
            He = arch.encoder_hidden_size or H
            cq, ckv = f"{n}/cross_attn/q_proj/Add/output_0", f"{n}/cross_attn/kv_proj/Add/output_0"
            put_linear(p + "cross_attn.q_proj", f"{n}/cross_attn/q_proj/MatMul", [p + "cross_attn.q_proj.weight"],
                       f"{n}/cross_attn_layernorm/output_0", f"{n}/cross_attn/q_proj/MatMul/output_0", arch.q_size, H)
            put_vec(p + "cross_attn.q_proj.Add.bias", [p + "cross_attn.q_proj.bias"])
            W.node("Add", f"{n}/cross_attn/q_proj/Add", [f"{n}/cross_attn/q_proj/MatMul/output_0", p + "cross_attn.q_proj.Add.bias"], [cq])
            put_linear(p + "cross_attn.kv_proj", f"{n}/cross_attn/kv_proj/MatMul", [p + "cross_attn.k_proj.weight", p + "cross_attn.v_proj.weight"],
                       "encoder_hidden_states", f"{n}/cross_attn/kv_proj/MatMul/output_0", 2 * arch.q_size, He)
            put_vec(p + "cross_attn.kv_proj.Add.bias", [p + "cross_attn.k_proj.bias", p + "cross_attn.v_proj.bias"])
            W.node("Add", f"{n}/cross_attn/kv_proj/Add", [f"{n}/cross_attn/kv_proj/MatMul/output_0", p + "cross_attn.kv_proj.Add.bias"], [ckv])
            W.node("Split", f"{n}/cross_attn/kv_proj/Split", [ckv], [f"{n}/cross_attn/k", f"{n}/cross_attn/v"], axis=-1, num_outputs=2)
            W.node("MultiHeadAttention", f"{n}/cross_attn/MultiHeadAttention", [cq, f"{n}/cross_attn/k", f"{n}/cross_attn/v"],
                   [f"{n}/cross_attn/MultiHeadAttention/output_0"], domain="com.microsoft", num_heads=arch.num_heads, scale=float(arch.scale))
            put_linear(p + "cross_attn.o_proj", f"{n}/cross_attn/o_proj/MatMul", [p + "cross_attn.o_proj.weight"],
                       f"{n}/cross_attn/MultiHeadAttention/output_0", f"{n}/cross_attn/o_proj/MatMul/output_0", H, arch.q_size)
            put_vec(p + "cross_attn.o_proj.Add.bias", [p + "cross_attn.o_proj.bias"])
            o_out = f"{n}/cross_attn/o_proj/Add/output_0"
            W.node("Add", f"{n}/cross_attn/o_proj/Add", [f"{n}/cross_attn/o_proj/MatMul/output_0", p + "cross_attn.o_proj.Add.bias"], [o_out])
        if arch.post_sublayer_norms:
            put_vec(p + "post_attention_layernorm.weight", [p + "post_attention_layernorm.weight"], arch.norm_offset)
            W.node(norm_op, f"{n}/post_attention_layernorm/LayerNorm", [o_out, p + "post_attention_layernorm.weight"],
                   [f"{n}/post_attention_layernorm/output_0"], epsilon=float(arch.norm_eps), axis=-1, stash_type=1)
            o_out = f"{n}/post_attention_layernorm/output_0"
            mid_name = "pre_feedforward_layernorm"
        else:
            mid_name = "post_attention_layernorm"
        o_out = residual_scale(f"{n}/attn/residual_mul/Mul", o_out)
        if not arch.parallel_block:
            # norm before the MLP (adds the attention output to the residual stream)
            put_vec(p + mid_name + ".weight", [p + mid_name + ".weight"], arch.norm_offset)
            ins = [o_out, residual, p + mid_name + ".weight"]
            if arch.layernorm:
                put_vec(p + mid_name + ".bias", [p + mid_name + ".bias"])
                ins.append(p + mid_name + ".bias")
            W.node(skip_op, f"{n}/{mid_name}/SkipLayerNorm", ins, [f"{n}/{mid_name}/output_0", "", "", f"{n}/{mid_name}/output_3"],
                   domain="com.microsoft", epsilon=float(arch.norm_eps))
            residual = f"{n}/{mid_name}/output_3"
            x = f"{n}/{mid_name}/output_0"
        # (parallel block: the MLP reads the same normalised input as the attention)
        # MLP / MoE
        if arch.num_experts > 0 and arch.moe_style == "standard":
            # MoE contrib op with three expert matrices: fc1 = gate [E, I, H], fc2 = down [E, H, I], fc3 = up [E, I, H];
            # silu(fc1 x) * fc3 x, routing weights = softmax over all experts (renormalised over the selected if asked)
            E = arch.num_experts
            put_linear(p + "moe.router", f"{n}/moe/router/MatMul", [p + "mlp.router.weight"], x, f"{n}/moe/router/MatMul/output_0", E, H)
            for nm in ("gate_proj", "down_proj", "up_proj"):
                put_plain(p + f"moe.experts.{nm}.weight", [p + f"mlp.experts.{nm}"], {"shape": shapes[p + f"mlp.experts.{nm}"], "op": "id", "fn": lambda ts: ts[0].float()})
            W.node("MoE", f"{n}/moe/MoE", [x, f"{n}/moe/router/MatMul/output_0", p + "moe.experts.gate_proj.weight", "",
                                          p + "moe.experts.down_proj.weight", "", p + "moe.experts.up_proj.weight", ""],
                   [f"{n}/moe/MoE/output_0"], domain="com.microsoft", k=arch.experts_per_token, activation_type="silu", activation_alpha=1.0,
                   activation_beta=0.0, swiglu_fusion=0, normalize_routing_weights=int(arch.moe_norm_topk),
                   use_sparse_mixer=int(arch.moe_sparse_mixer), **({"sparse_mixer_jitter_eps": float(arch.moe_jitter_eps)} if arch.moe_sparse_mixer else {}))
            mlp_out = f"{n}/moe/MoE/output_0"
            if arch.shared_expert_intermediate:
                # the always-on dense gated MLP beside the routed experts (reference graph: builders/qwen.py make_shared_expert); its output is
                # scaled by sigmoid of a one-row projection where the family has that gate, then added to the routed output
                Is, sh = arch.shared_expert_intermediate, f"{n}/moe/shared_expert"
                put_linear(p + "moe.shared_expert.gate_up_proj", f"{sh}/gate_up_proj/MatMul",
                           [p + "mlp.shared_expert.gate_proj.weight", p + "mlp.shared_expert.up_proj.weight"], x, f"{sh}/gate_up_proj/MatMul/output_0", 2 * Is, H)
                W.node("Split", f"{sh}/gate_up_proj/Split", [f"{sh}/gate_up_proj/MatMul/output_0"], [f"{sh}/gate", f"{sh}/up"], axis=-1, num_outputs=2)
                W.node("Sigmoid", f"{sh}/act_fn/Sigmoid", [f"{sh}/gate"], [f"{sh}/act_fn/Sigmoid/output_0"])
                W.node("Mul", f"{sh}/act_fn/Mul", [f"{sh}/gate", f"{sh}/act_fn/Sigmoid/output_0"], [f"{sh}/act_fn/output_0"])
                W.node("Mul", f"{sh}/Mul", [f"{sh}/act_fn/output_0", f"{sh}/up"], [f"{sh}/Mul/output_0"])
                put_linear(p + "moe.shared_expert.down_proj", f"{sh}/down_proj/MatMul", [p + "mlp.shared_expert.down_proj.weight"], f"{sh}/Mul/output_0",
                           f"{sh}/down_proj/MatMul/output_0", H, Is)
                sh_out = f"{sh}/down_proj/MatMul/output_0"
                if arch.shared_expert_gated:
                    put_linear(p + "moe.shared_expert_gate", f"{n}/moe/shared_expert_gate/MatMul", [p + "mlp.shared_expert_gate.weight"], x,
                               f"{n}/moe/shared_expert_gate/MatMul/output_0", 1, H)
                    W.node("Sigmoid", f"{n}/moe/shared_expert_gate/Sigmoid", [f"{n}/moe/shared_expert_gate/MatMul/output_0"], [f"{n}/moe/shared_expert_gate/Sigmoid/output_0"])
                    W.node("Mul", f"{n}/moe/shared_expert_gate/Mul", [sh_out, f"{n}/moe/shared_expert_gate/Sigmoid/output_0"], [f"{n}/moe/shared_expert_gate/Mul/output_0"])
                    sh_out = f"{n}/moe/shared_expert_gate/Mul/output_0"
                W.node("Add", f"{n}/moe/shared_expert/Add", [mlp_out, sh_out], [f"{n}/moe/shared_expert/Add/output_0"])
                mlp_out = f"{n}/moe/shared_expert/Add/output_0"
        elif arch.num_experts > 0:
            E = arch.num_experts
            put_linear(p + "moe.router", f"{n}/moe/router/MatMul", [p + "mlp.router.weight"], x, f"{n}/moe/router/MatMul/output_0", E, H)
            put_vec(p + "moe.router.Add.bias", [p + "mlp.router.bias"])
            W.node("Add", f"{n}/moe/router/Add", [f"{n}/moe/router/MatMul/output_0", p + "moe.router.Add.bias"], [f"{n}/moe/router/Add/output_0"])
            if precision == "int4" and synthetic_weights:
                # descriptors only: the loader draws random e2m1 codes and scale codes on the device (no float weight is made)
                ins = [x, f"{n}/moe/router/Add/output_0"]
                for nm, (Nn, Kk) in (("gate_up_proj", (2 * I, H)), ("down_proj", (H, I))):
                    for suffix, shp, kind in (("weight_fp4", (E, Kk, Nn // 2), "fp4_codes"), ("scales_e8m0", (E, Nn, Kk // 32), "fp4_scales")):
                        W.add_synthetic(p + f"moe.experts.{nm}.{suffix}", shp, "", op.UINT8)
                        synth_meta[p + f"moe.experts.{nm}.{suffix}"] = {"sources": [p + f"mlp.experts.{nm}"], "op": kind, "seed": seed, "std": std,
                                                                        "shape": list(shp)}
                    put_plain(p + f"moe.experts.{nm}.bias", [p + f"mlp.experts.{nm}_bias"],
                              {"shape": (E, Nn), "op": "id", "fn": lambda ts: ts[0].float()})
                    ins += [p + f"moe.experts.{nm}.weight_fp4", p + f"moe.experts.{nm}.scales_e8m0", p + f"moe.experts.{nm}.bias"]
                W.node("QMoE", f"{n}/moe/QMoE", ins, [f"{n}/moe/MoE/output_0"], domain="com.microsoft", k=arch.experts_per_token,
                       activation_type="swiglu", activation_alpha=float(arch.moe_swiglu_alpha), activation_beta=1.0, swiglu_fusion=1,
                       swiglu_limit=float(arch.moe_swiglu_limit), normalize_routing_weights=1, expert_weight_bits=4, block_size=32,
                       quant_type="fp4", use_sparse_mixer=0)
            elif precision == "int4":
                # quantised experts: QMoE with MXFP4 weights (FP4 e2m1 codes [E, K, N/2], e8m0 scales [E, N, K/32], unit global scales)
                ins = [x, f"{n}/moe/router/Add/output_0"]
                for nm in ("gate_up_proj", "down_proj"):
                    wt = get(p + f"mlp.experts.{nm}").float()
                    packs = [quantize_mxfp4(wt[e]) for e in range(E)]
                    W.add_array(p + f"moe.experts.{nm}.weight_fp4", torch.stack([q for q, _ in packs]).numpy(), op.UINT8)
                    W.add_array(p + f"moe.experts.{nm}.scales_e8m0", torch.stack([c for _, c in packs]).numpy(), op.UINT8)
                    W.add_float(p + f"moe.experts.{nm}.bias", get(p + f"mlp.experts.{nm}_bias").float())
                    ins += [p + f"moe.experts.{nm}.weight_fp4", p + f"moe.experts.{nm}.scales_e8m0", p + f"moe.experts.{nm}.bias"]
                ins += [""] * (15 - len(ins))      # fc3, zero points, router weights: unused
                for nm in ("gate_up_proj", "down_proj"):
                    W.add_array(p + f"moe.experts.{nm}.global_scale", np.ones((E,), dtype=np.float32), op.FLOAT)
                    ins.append(p + f"moe.experts.{nm}.global_scale")
                W.node("QMoE", f"{n}/moe/QMoE", ins, [f"{n}/moe/MoE/output_0"], domain="com.microsoft", k=arch.experts_per_token,
                       activation_type="swiglu", activation_alpha=float(arch.moe_swiglu_alpha), activation_beta=1.0, swiglu_fusion=1,
                       swiglu_limit=float(arch.moe_swiglu_limit), normalize_routing_weights=1, expert_weight_bits=4, block_size=32,
                       quant_type="fp4", use_sparse_mixer=0)
            else:
                for nm, shape in (("gate_up_proj", (E, 2 * I, H)), ("down_proj", (E, H, I))):
                    put_plain(p + f"moe.experts.{nm}.weight", [p + f"mlp.experts.{nm}"], {"shape": shape, "op": "id", "fn": lambda ts: ts[0].float()})
                    put_plain(p + f"moe.experts.{nm}.bias", [p + f"mlp.experts.{nm}_bias"],
                              {"shape": shape[:2], "op": "id", "fn": lambda ts: ts[0].float()})
                W.node("MoE", f"{n}/moe/MoE", [x, f"{n}/moe/router/Add/output_0", p + "moe.experts.gate_up_proj.weight",
                                               p + "moe.experts.gate_up_proj.bias", p + "moe.experts.down_proj.weight",
                                               p + "moe.experts.down_proj.bias"], [f"{n}/moe/MoE/output_0"], domain="com.microsoft",
                       k=arch.experts_per_token, activation_type="swiglu", activation_alpha=float(arch.moe_swiglu_alpha),
                       activation_beta=1.0, swiglu_fusion=1, swiglu_limit=float(arch.moe_swiglu_limit), normalize_routing_weights=1)
            mlp_out = f"{n}/moe/MoE/output_0"
        elif not arch.mlp_gated:
            f1 = f"{n}/mlp/fc1/MatMul/output_0"
            put_linear(p + "mlp.fc1", f"{n}/mlp/fc1/MatMul", [p + "mlp.fc1.weight"], x, f1, I, H)
            if arch.mlp_bias:
                put_vec(p + "mlp.fc1.Add.bias", [p + "mlp.fc1.bias"])
                W.node("Add", f"{n}/mlp/fc1/Add", [f1, p + "mlp.fc1.Add.bias"], [f"{n}/mlp/fc1/Add/output_0"])
                f1 = f"{n}/mlp/fc1/Add/output_0"
            if arch.activation == "silu":
                W.node("Sigmoid", f"{n}/mlp/act_fn/Sigmoid", [f1], [f"{n}/mlp/act_fn/Sigmoid/output_0"])
                W.node("Mul", f"{n}/mlp/act_fn/Mul", [f1, f"{n}/mlp/act_fn/Sigmoid/output_0"], [f"{n}/mlp/act_fn/output_0"])
            elif arch.activation == "gelu_erf":
                W.node("Gelu", f"{n}/mlp/act_fn/Gelu", [f1], [f"{n}/mlp/act_fn/output_0"], domain="com.microsoft")
            elif arch.activation == "relu":
                W.node("Relu", f"{n}/mlp/act_fn/Relu", [f1], [f"{n}/mlp/act_fn/output_0"])
            elif arch.activation == "relu2":
                W.node("Relu", f"{n}/mlp/act_fn/Relu", [f1], [f"{n}/mlp/act_fn/Relu/output_0"])
                W.node("Mul", f"{n}/mlp/act_fn/Square", [f"{n}/mlp/act_fn/Relu/output_0", f"{n}/mlp/act_fn/Relu/output_0"], [f"{n}/mlp/act_fn/output_0"])
            else:
                W.node("FastGelu", f"{n}/mlp/act_fn/FastGelu", [f1], [f"{n}/mlp/act_fn/output_0"], domain="com.microsoft")
            mlp_out = f"{n}/mlp/fc2/MatMul/output_0"
            put_linear(p + "mlp.fc2", f"{n}/mlp/fc2/MatMul", [p + "mlp.fc2.weight"], f"{n}/mlp/act_fn/output_0", mlp_out, H, I)
            if arch.mlp_bias:
                put_vec(p + "mlp.fc2.Add.bias", [p + "mlp.fc2.bias"])
                W.node("Add", f"{n}/mlp/fc2/Add", [mlp_out, p + "mlp.fc2.Add.bias"], [f"{n}/mlp/fc2/Add/output_0"])
                mlp_out = f"{n}/mlp/fc2/Add/output_0"
        else:
            gu = f"{n}/mlp/gate_up_proj/MatMul/output_0"
            put_linear(p + "mlp.gate_up_proj", f"{n}/mlp/gate_up_proj/MatMul", [p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"], x, gu, 2 * I, H)
            if arch.mlp_bias:
                put_vec(p + "mlp.gate_up_proj.Add.bias", [p + "mlp.gate_proj.bias", p + "mlp.up_proj.bias"])
                W.node("Add", f"{n}/mlp/gate_up_proj/Add", [gu, p + "mlp.gate_up_proj.Add.bias"], [f"{n}/mlp/gate_up_proj/Add/output_0"])
                gu = f"{n}/mlp/gate_up_proj/Add/output_0"
            W.node("Split", f"{n}/mlp/gate_up_proj/Split", [gu], [f"{n}/mlp/gate", f"{n}/mlp/up"], axis=-1, num_outputs=2)
            if arch.activation == "silu":
                W.node("Sigmoid", f"{n}/mlp/act_fn/Sigmoid", [f"{n}/mlp/gate"], [f"{n}/mlp/act_fn/Sigmoid/output_0"])
                W.node("Mul", f"{n}/mlp/act_fn/Mul", [f"{n}/mlp/gate", f"{n}/mlp/act_fn/Sigmoid/output_0"], [f"{n}/mlp/act_fn/Mul/output_0"])
            else:
                W.node("FastGelu", f"{n}/mlp/act_fn/FastGelu", [f"{n}/mlp/gate"], [f"{n}/mlp/act_fn/Mul/output_0"], domain="com.microsoft")
            W.node("Mul", f"{n}/mlp/Mul", [f"{n}/mlp/act_fn/Mul/output_0", f"{n}/mlp/up"], [f"{n}/mlp/Mul/output_0"])
            mlp_out = f"{n}/mlp/down_proj/MatMul/output_0"
            put_linear(p + "mlp.down_proj", f"{n}/mlp/down_proj/MatMul", [p + "mlp.down_proj.weight"], f"{n}/mlp/Mul/output_0", mlp_out, H, I)
            if arch.mlp_bias:
                put_vec(p + "mlp.down_proj.Add.bias", [p + "mlp.down_proj.bias"])
                W.node("Add", f"{n}/mlp/down_proj/Add", [mlp_out, p + "mlp.down_proj.Add.bias"], [f"{n}/mlp/down_proj/Add/output_0"])
                mlp_out = f"{n}/mlp/down_proj/Add/output_0"
        if arch.post_sublayer_norms:
            put_vec(p + "post_feedforward_layernorm.weight", [p + "post_feedforward_layernorm.weight"], arch.norm_offset)
            W.node(norm_op, f"{n}/post_feedforward_layernorm/LayerNorm", [mlp_out, p + "post_feedforward_layernorm.weight"],
                   [f"{n}/post_feedforward_layernorm/output_0"], epsilon=float(arch.norm_eps), axis=-1, stash_type=1)
            mlp_out = f"{n}/post_feedforward_layernorm/output_0"
        hidden = residual_scale(f"{n}/mlp/residual_mul/Mul", mlp_out)
        if arch.parallel_block:
            W.node("Add", f"{n}/parallel_block/Add", [o_out, hidden], [f"{n}/parallel_block/Add/output_0"])
            hidden = f"{n}/parallel_block/Add/output_0"

    # ---- final norm + head
    fname = f"model.layers.{L}.final_norm_layernorm.weight"
    put_vec(fname, ["model.norm.weight"], arch.norm_offset)
    ins = [hidden, residual, fname]
    if arch.layernorm:
        put_vec(f"model.layers.{L}.final_norm_layernorm.bias", ["model.norm.bias"])
        ins.append(f"model.layers.{L}.final_norm_layernorm.bias")
    W.node(skip_op, f"/model/layers.{L}/final_norm_layernorm/SkipLayerNorm", ins,
           [f"/model/layers.{L}/final_norm_layernorm/output_0", "", "", ""], domain="com.microsoft", epsilon=float(arch.norm_eps))
    head_src = ["model.embed_tokens.weight"] if arch.tie_embeddings else ["lm_head.weight"]
    put_linear("lm_head", "/lm_head/MatMul", head_src, f"/model/layers.{L}/final_norm_layernorm/output_0", "/lm_head/MatMul/output_0", V, H)
    logits_name = "/lm_head/MatMul/output_0"
    if arch.lm_head_bias:
        put_vec("lm_head.Add.bias", ["lm_head.bias"])
        W.node("Add", "/lm_head/Add", [logits_name, "lm_head.Add.bias"], ["/lm_head/Add/output_0"])
        logits_name = "/lm_head/Add/output_0"
    if arch.logits_scale != 1.0:
        W.model.initializers["/model/constants/logits_scale"] = op.Tensor("/model/constants/logits_scale", op.FLOAT, (),
                                                                          raw=np.float32(arch.logits_scale).tobytes())
        W.node("Mul", "/lm_head/Mul", [logits_name, "/model/constants/logits_scale"], ["/lm_head/Mul/output_0"])
        logits_name = "/lm_head/Mul/output_0"
    if arch.final_logit_softcap > 0:
        W.node("Softcap", "/lm_head/softcap", [logits_name], ["/lm_head/softcap/output_0"], domain="com.microsoft",
               softcap=float(arch.final_logit_softcap))
        logits_name = "/lm_head/softcap/output_0"
    W.node("Cast" if W.io != "fp32" else "Identity", "/lm_head/Cast", [logits_name], ["logits"], **({"to": op.FLOAT} if W.io != "fp32" else {}))

    # ---- graph inputs / outputs
    m = W.model
    if paged:
        m.inputs = [op.ValueInfo("input_ids", op.INT64, ("num_tokens",)),
                    op.ValueInfo("block_table", op.INT32, ("batch_size", "max_num_blocks")),
                    op.ValueInfo("cumulative_sequence_lengths", op.INT32, ("batch_size_plus_1",)),
                    op.ValueInfo("past_sequence_lengths", op.INT32, ("batch_size",)),
                    op.ValueInfo("attention_metadata", op.INT32, (3,))]
        if arch.sliding_window > 0 and arch.sliding_layers is not None:
            m.inputs.insert(2, op.ValueInfo("block_table_windowed", op.INT32, ("batch_size", "max_num_blocks")))
        kv_shape = ("num_blocks", block_size, arch.num_kv_heads, arch.head_dim)
        m.outputs = [op.ValueInfo("logits", op.FLOAT, ("batch_size", V))]
    else:
        m.inputs = [op.ValueInfo("input_ids", op.INT64, ("batch_size", "sequence_length")),
                    op.ValueInfo("attention_mask", op.INT64, ("batch_size", "total_sequence_length"))]
        kv_shape = ("batch_size", arch.num_kv_heads, "past_sequence_length", arch.head_dim)
        m.outputs = [op.ValueInfo("logits", op.FLOAT, ("batch_size", "sequence_length", V))]
    if arch.cross_attention:
        m.inputs.append(op.ValueInfo("encoder_hidden_states", io_dt, ("batch_size", "encoder_sequence_length", arch.encoder_hidden_size or H)))
    if arch.learned_positions:
        m.inputs.append(op.ValueInfo("position_ids", op.INT64, ("num_tokens",) if paged else ("batch_size", "sequence_length")))
    for i in range(L):
        if arch.is_conv_layer(i):
            m.inputs.append(op.ValueInfo(f"past_conv.{i}", io_dt, ("batch_size", H, arch.conv_L_cache)))
            m.outputs.append(op.ValueInfo(f"present_conv.{i}", io_dt, ("batch_size", H, arch.conv_L_cache)))
            continue
        if arch.is_recurrent_layer(i):
            if arch.is_mamba_layer(i):
                cs = ("batch_size", arch.mamba_conv_dim, arch.mamba_conv_kernel - 1)
                rs = ("batch_size", arch.mamba_num_heads, arch.mamba_head_dim, arch.mamba_state_size)
            else:
                cs = ("batch_size", arch.linear_conv_dim, arch.linear_conv_kernel_dim - 1)
                rs = ("batch_size", arch.linear_num_value_heads, arch.linear_key_head_dim, arch.linear_value_head_dim)
            m.inputs += [op.ValueInfo(f"past_key_values.{i}.conv_state", io_dt, cs), op.ValueInfo(f"past_key_values.{i}.recurrent_state", io_dt, rs)]
            m.outputs += [op.ValueInfo(f"present.{i}.conv_state", io_dt, cs), op.ValueInfo(f"present.{i}.recurrent_state", io_dt, rs)]
            continue
        m.inputs += [op.ValueInfo(f"past_key_values.{i}.key", io_dt, kv_shape), op.ValueInfo(f"past_key_values.{i}.value", io_dt, kv_shape)]
        m.outputs += [op.ValueInfo(f"present.{i}.key", io_dt, kv_shape), op.ValueInfo(f"present.{i}.value", io_dt, kv_shape)]

    if W.ext is not None:
        W.ext.close()
    _save_with_synthetic(m, os.path.join(out_dir, filename), synth_meta)

    if write_config:
        cfg = make_genai_config(arch, precision, execution_provider, paged, block_size, max_batch_size, filename, search, engine,
                                num_blocks=num_blocks, max_scheduled_tokens=max_scheduled_tokens)
        if speculative:
            cfg["speculative"] = speculative
        if draft_dir_entry:
            cfg["model"]["draft"] = draft_dir_entry
        with open(os.path.join(out_dir, "genai_config.json"), "w") as f:
            json.dump(cfg, f, indent=4)
    return out_dir


def _save_with_synthetic(model: op.Model, path: str, synth_meta: Dict[str, dict]) -> None:
    """Synthetic initializers are stored as external-data entries {location: 'synthetic', spec: <json>}."""
    if not synth_meta:
        op.save_model(model, path)
        return
    # Encode the synthetic spec in the `location` string so that the stock wire format is kept.
    for name, meta in synth_meta.items():
        t = model.initializers[name]
        t.ext_location = "synthetic:" + json.dumps(meta, separators=(",", ":"))
        t.ext_offset = 0
        t.ext_length = 0
    op.save_model(model, path)


def make_genai_config(arch: ArchConfig, precision: str, ep: str, paged: bool, block_size: int, max_batch_size: int,
                      filename: str = "model.onnx", search: Optional[dict] = None, engine: Optional[dict] = None,
                      num_blocks: Optional[int] = None, max_scheduled_tokens: Optional[int] = None) -> dict:
    inputs = {"input_ids": "input_ids", "past_key_names": "past_key_values.%d.key", "past_value_names": "past_key_values.%d.value"}
    if paged:
        inputs.update({"block_table": "block_table", "cumulative_sequence_lengths": "cumulative_sequence_lengths",
                       "past_sequence_lengths": "past_sequence_lengths", "attention_metadata": "attention_metadata"})
        if arch.sliding_window > 0 and arch.sliding_layers is not None:
            inputs["block_table_windowed"] = "block_table_windowed"
    else:
        inputs["attention_mask"] = "attention_mask"
    if arch.learned_positions:
        inputs["position_ids"] = "position_ids"
    provider_options = [] if ep == "cpu" else [{ep: {"enable_cuda_graph": "0"} if ep == "cuda" else {}}]
    decoder = {
        "session_options": {"log_id": "onnxruntime-genai", "provider_options": provider_options},
        "filename": filename, "head_size": arch.head_dim, "hidden_size": arch.hidden_size, "inputs": inputs,
        "outputs": {"logits": "logits", "present_key_names": "present.%d.key", "present_value_names": "present.%d.value"},
        "num_attention_heads": arch.num_heads, "num_hidden_layers": arch.num_layers, "num_key_value_heads": arch.num_kv_heads,
    }
    if arch.sliding_window > 0:
        sw = {"window_size": arch.sliding_window, "slide_key_value_cache": False, "slide_inputs": False}
        if arch.sliding_layers is not None:
            sw["layers"] = list(arch.sliding_layers)
        decoder["sliding_window"] = sw
    if arch.has_linear_layers:
        decoder["layer_types"] = list(arch.layer_types)
    if arch.layer_types is not None and "conv" in arch.layer_types:
        decoder["layer_types"] = list(arch.layer_types)
        decoder["conv_cache_size"] = int(arch.conv_L_cache)
        inputs["past_conv_names"] = "past_conv.%d"
        decoder["outputs"]["present_conv_names"] = "present_conv.%d"
    cfg = {
        "model": {"bos_token_id": arch.bos_token_id, "context_length": arch.context_length, "decoder": decoder,
                  "eos_token_id": arch.eos_token_id, "pad_token_id": arch.pad_token_id, "type": arch.model_type,
                  "vocab_size": arch.vocab_size},
        "search": {"diversity_penalty": 0.0, "do_sample": False, "early_stopping": True, "length_penalty": 1.0,
                   "max_length": arch.context_length, "min_length": 0, "no_repeat_ngram_size": 0, "num_beams": 1,
                   "num_return_sequences": 1, "past_present_share_buffer": ep == "cuda", "repetition_penalty": 1.0,
                   "temperature": 1.0, "top_k": 50, "top_p": 1.0},
    }
    if search:
        cfg["search"].update(search)
    if paged or engine:
        dyn = {"block_size": block_size, "gpu_utilization_factor": 0.6, "max_batch_size": max_batch_size}
        if num_blocks:
            dyn["num_blocks"] = num_blocks
        if max_scheduled_tokens:
            dyn["max_scheduled_tokens"] = max_scheduled_tokens
        cfg["engine"] = engine or {"dynamic_batching": dyn}
    return cfg


# ---------------------------------------------------------------------------------------------- HF loading
# ------------------------------------------------------------------------------------------------ multimodal checkpoints
def _patch_config(out_dir: str, edit) -> None:
    path = os.path.join(out_dir, "genai_config.json")
    with open(path) as f:
        cfg = json.load(f)
    edit(cfg)
    with open(path, "w") as f:
        json.dump(cfg, f, indent=4)


def whisper_decoder_arch(vocab_size: int, hidden_size: int, num_layers: int, num_heads: int, intermediate_size: int,
                         encoder_hidden_size: int = 0, context_length: int = 448, **kw) -> ArchConfig:
    """The decoder half of a Whisper model as family flags: LayerNorm, learned positions, biased projections, fc1 -> GELU(erf)
    -> fc2, cross-attention to the encoder output in every layer, tied output embedding."""
    return ArchConfig(model_type="whisper", vocab_size=vocab_size, hidden_size=hidden_size, num_layers=num_layers, num_heads=num_heads,
                      num_kv_heads=num_heads, head_dim=hidden_size // num_heads, intermediate_size=intermediate_size,
                      context_length=context_length, layernorm=True, norm_eps=1e-5, learned_positions=True, cross_attention=True,
                      encoder_hidden_size=encoder_hidden_size, attn_bias=True, o_bias=True, mlp_bias=True, mlp_gated=False,
                      activation="gelu_erf", tie_embeddings=True, **kw)


def export_whisper(arch: ArchConfig, enc, out_dir: str, precision: str = "bf16", execution_provider: str = "cuda",
                   decoder_state_dict=None, encoder_state_dict=None, seed: int = 0, std: float = 0.02, num_frames: int = 3000,
                   search: Optional[dict] = None) -> str:
    """Encoder-decoder speech checkpoint: decoder.onnx (cross-attention decoder), encoder.onnx, genai_config.json with
    model.type "whisper" and an `encoder` section, audio_processor_config.json for the log-mel front end."""
    from .encoder import export_encoder, random_encoder_state_dict
    export_model(arch, out_dir, precision, execution_provider, state_dict=decoder_state_dict, seed=seed, std=std, filename="decoder.onnx",
                 search=search)
    export_encoder(enc, out_dir, "encoder.onnx", encoder_state_dict or random_encoder_state_dict(enc, seed, std), precision)

    def edit(cfg):
        cfg["model"]["type"] = "whisper"
        cfg["model"]["encoder"] = {"filename": "encoder.onnx", "hidden_size": enc.hidden_size, "num_attention_heads": enc.num_heads,
                                   "num_hidden_layers": enc.num_layers, "head_size": enc.head_dim,
                                   "inputs": {"audio_features": "audio_features"}, "outputs": {"encoder_hidden_states": "encoder_hidden_states"}}
        cfg["model"]["decoder"]["inputs"]["encoder_hidden_states"] = "encoder_hidden_states"
    _patch_config(out_dir, edit)
    with open(os.path.join(out_dir, "audio_processor_config.json"), "w") as f:
        json.dump({"processor": {"name": "whisper_log_mel", "num_mel_bins": enc.num_mel_bins, "n_fft": 400, "hop_length": 160,
                                 "sample_rate": 16000, "num_frames": num_frames}}, f, indent=2)
    return out_dir


def whisper_from_hf(cfg: dict, sd: Dict[str, torch.Tensor]):
    """A Hugging Face Whisper checkpoint (`WhisperForConditionalGeneration`) as this exporter's inputs: the decoder's family flags
    and the encoder's configuration, and both state dictionaries under the names `export_whisper` reads (reference:
    src/python/py/models/builders/whisper.py).  The key projections of Whisper carry no bias: zero biases are written."""
    from .encoder import EncoderConfig
    D = int(cfg["d_model"])
    arch = whisper_decoder_arch(int(cfg["vocab_size"]), D, int(cfg["decoder_layers"]), int(cfg["decoder_attention_heads"]), int(cfg["decoder_ffn_dim"]),
                                encoder_hidden_size=D, context_length=int(cfg.get("max_target_positions", 448)),
                                bos_token_id=int(cfg.get("decoder_start_token_id") or cfg.get("bos_token_id") or 0),
                                eos_token_id=cfg.get("eos_token_id") if cfg.get("eos_token_id") is not None else 0,
                                pad_token_id=int(cfg.get("pad_token_id") if cfg.get("pad_token_id") is not None else 0))
    act = {"gelu": "gelu_erf", "gelu_new": "gelu", "relu": "relu"}.get(cfg.get("activation_function", "gelu"), "gelu_erf")
    arch.activation = act
    enc = EncoderConfig(kind="audio", hidden_size=D, num_layers=int(cfg["encoder_layers"]), num_heads=int(cfg["encoder_attention_heads"]),
                        intermediate_size=int(cfg["encoder_ffn_dim"]), num_mel_bins=int(cfg.get("num_mel_bins", 80)),
                        max_source_positions=int(cfg.get("max_source_positions", 1500)), activation=act)
    dec_sd, enc_sd = {}, {}
    renames = ((".self_attn_layer_norm.", ".input_layernorm."), (".encoder_attn_layer_norm.", ".cross_attn_layernorm."),
               (".final_layer_norm.", ".post_attention_layernorm."), (".self_attn.out_proj.", ".self_attn.o_proj."),
               (".encoder_attn.out_proj.", ".cross_attn.o_proj."), (".encoder_attn.", ".cross_attn."), (".fc1.", ".mlp.fc1."), (".fc2.", ".mlp.fc2."))
    for k, v in sd.items():
        if k.startswith("model.encoder."):
            enc_sd[k[len("model."):]] = v
        elif k.startswith("model.decoder."):
            k2 = "model." + k[len("model.decoder."):]
            k2 = k2.replace("model.embed_positions.", "model.position_embeddings.").replace("model.layer_norm.", "model.norm.")
            for old, new in renames:
                if old in k2:
                    k2 = k2.replace(old, new)
                    break
            dec_sd[k2] = v
    for i in range(enc.num_layers):
        enc_sd.setdefault(f"encoder.layers.{i}.self_attn.k_proj.bias", torch.zeros(D))
    for i in range(arch.num_layers):
        dec_sd.setdefault(f"model.layers.{i}.self_attn.k_proj.bias", torch.zeros(D))
        dec_sd.setdefault(f"model.layers.{i}.cross_attn.k_proj.bias", torch.zeros(D))
    dec_sd["model.position_embeddings.weight"] = dec_sd["model.position_embeddings.weight"][: arch.context_length]
    return arch, enc, dec_sd, enc_sd


def export_vision_language(arch: ArchConfig, vis, out_dir: str, image_token_id: int, precision: str = "bf16",
                           execution_provider: str = "cuda", decoder_state_dict=None, vision_state_dict=None, seed: int = 0,
                           std: float = 0.02, model_type: str = "phi3v", image_token: str = "<|image|>", **export_kw) -> str:
    """Vision-language checkpoint: model.onnx (the text decoder), vision.onnx (ViT + projector into the decoder's width),
    genai_config.json with a `vision` section and `image_token_id`, processor_config.json for the image front end."""
    from .encoder import export_encoder, random_encoder_state_dict
    if vis.projection_size != arch.hidden_size:
        raise ValueError("the projector must map to the decoder's hidden size")
    export_model(arch, out_dir, precision, execution_provider, state_dict=decoder_state_dict, seed=seed, std=std, **export_kw)
    export_encoder(vis, out_dir, "vision.onnx", vision_state_dict or random_encoder_state_dict(vis, seed, std), precision)

    def edit(cfg):
        cfg["model"]["type"] = model_type
        cfg["model"]["image_token_id"] = int(image_token_id)
        cfg["model"]["vision"] = {"filename": "vision.onnx", "config_filename": "processor_config.json", "patch_size": vis.patch_size,
                                  "num_visual_tokens": vis.num_patches,
                                  "inputs": {"pixel_values": "pixel_values", "image_sizes": "image_sizes"},
                                  "outputs": {"image_features": "image_features"}}
        cfg["model"]["embedding"] = {"filename": cfg["model"]["decoder"]["filename"],
                                     "inputs": {"input_ids": "input_ids", "image_features": "image_features"},
                                     "outputs": {"inputs_embeds": "inputs_embeds"}}
    _patch_config(out_dir, edit)
    with open(os.path.join(out_dir, "processor_config.json"), "w") as f:
        json.dump({"processor": {"name": "image_processing", "image_size": vis.image_size, "patch_size": vis.patch_size,
                                 "image_mean": [0.48145466, 0.4578275, 0.40821073], "image_std": [0.26862954, 0.26130258, 0.27577711],
                                 "image_token": image_token, "image_token_id": int(image_token_id), "num_image_tokens": vis.num_patches}}, f, indent=2)
    return out_dir


def export_qwen_vl(arch: ArchConfig, vis, out_dir: str, image_token_id: int, precision: str = "bf16", execution_provider: str = "cuda",
                   decoder_state_dict=None, vision_state_dict=None, seed: int = 0, std: float = 0.02, image_token: str = "<|image_pad|>",
                   **export_kw) -> str:
    """Qwen2-VL checkpoint: model.onnx (the text decoder with multimodal RoPE), vision.onnx (`models/qwen_vl.py`: patch embedding,
    2-D rotary attention blocks, patch merger), genai_config.json with the `vision` section, processor_config.json with the
    pixel budget of the image front end."""
    from . import qwen_vl
    if arch.mrope_section is None:
        raise ValueError("a Qwen2-VL decoder needs mrope_section")
    if vis.hidden_size != arch.hidden_size:
        raise ValueError("the patch merger must map to the decoder's hidden size")
    export_model(arch, out_dir, precision, execution_provider, state_dict=decoder_state_dict, seed=seed, std=std, **export_kw)
    qwen_vl.export_qwen_vision(vis, out_dir, vision_state_dict or qwen_vl.random_state_dict(vis, seed, std), "vision.onnx", precision)

    def edit(cfg):
        cfg["model"]["image_token_id"] = int(image_token_id)
        cfg["model"]["vision"] = {"filename": "vision.onnx", "config_filename": "processor_config.json", "patch_size": vis.patch_size,
                                  "spatial_merge_size": vis.spatial_merge_size,
                                  "inputs": {"pixel_values": "pixel_values", "image_grid_thw": "image_grid_thw"},
                                  "outputs": {"image_features": "image_features"}}
    _patch_config(out_dir, edit)
    with open(os.path.join(out_dir, "processor_config.json"), "w") as f:
        json.dump({"processor": {"name": "qwen2_vl_image_processing", "patch_size": vis.patch_size, "merge_size": vis.spatial_merge_size,
                                 "temporal_patch_size": vis.temporal_patch_size, "min_pixels": vis.min_pixels, "max_pixels": vis.max_pixels,
                                 "image_mean": list(qwen_vl.IMAGE_MEAN), "image_std": list(qwen_vl.IMAGE_STD), "image_token": image_token,
                                 "image_token_id": int(image_token_id)}}, f, indent=2)
    return out_dir


def load_hf_state_dict(model_dir: str) -> Dict[str, torch.Tensor]:
    """Reads *.safetensors (preferred) or pytorch_model*.bin from a Hugging Face model directory."""
    sd: Dict[str, torch.Tensor] = {}
    files = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
    if files:
        from safetensors.torch import load_file
        for f in files:
            sd.update(load_file(os.path.join(model_dir, f)))
    else:
        for f in sorted(f for f in os.listdir(model_dir) if f.startswith("pytorch_model") and f.endswith(".bin")):
            sd.update(torch.load(os.path.join(model_dir, f), map_location="cpu", weights_only=True))
    if not sd:
        raise FileNotFoundError(f"no weights found in {model_dir}")
    cfg_path = os.path.join(model_dir, "config.json")
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            qc = json.load(f).get("quantization_config")
        if qc and (any(k.endswith(".qweight") for k in sd) or str(qc.get("quant_method", "")).lower() == "modelopt"):
            # AWQ / GPTQ linears become QuantizedLinear entries: an int4 export writes them as they are
            from .quantized_checkpoint import convert_state_dict
            sd = convert_state_dict(sd, qc)
    out = {}
    if any(k.startswith("model.language_model.") for k in sd):
        # the decoder of a multimodal checkpoint: its weights under the plain decoder names (the towers keep theirs)
        sd = {("model." + k[len("model.language_model."):] if k.startswith("model.language_model.") else k): v for k, v in sd.items()}
    for k, v in sd.items():
        if k.endswith("qkv_proj.weight"):  # phi3 packs q, k, v
            base = k[: -len("qkv_proj.weight")]
            out[base + "q_proj.weight"], out[base + "k_proj.weight"], out[base + "v_proj.weight"] = v, None, None
            out[base + "__packed_qkv__"] = v
        elif k.endswith("gate_up_proj.weight"):
            base = k[: -len("gate_up_proj.weight")]
            half = v.shape[0] // 2
            out[base + "gate_proj.weight"], out[base + "up_proj.weight"] = (v.rows(0, half), v.rows(half, 2 * half)) if hasattr(v, "rows") else (v[:half], v[half:])
        elif k.endswith("shared_mlp.input_linear.weight"):   # granitemoehybrid: the dense feed-forward, gate rows then up rows
            base = k[: -len("shared_mlp.input_linear.weight")] + "mlp."
            half = v.shape[0] // 2
            out[base + "gate_proj.weight"], out[base + "up_proj.weight"] = (v.rows(0, half), v.rows(half, 2 * half)) if hasattr(v, "rows") else (v[:half], v[half:])
        elif k.endswith("shared_mlp.output_linear.weight"):
            out[k[: -len("shared_mlp.output_linear.weight")] + "mlp.down_proj.weight"] = v
        else:
            out[k] = v
    return out


def _canonical_moe_names(sd: Dict[str, torch.Tensor], arch: ArchConfig) -> None:
    """Routed experts of a Hugging Face checkpoint under this exporter's names: `mlp.router.weight` [E, H] and
    `mlp.experts.{gate,up,down}_proj` stacked over the experts.  Sources: one module per expert (`block_sparse_moe.experts.N.w1/w3/w2`,
    `mlp.experts.N.gate_proj/up_proj/down_proj`), stacked and fused tensors (`mlp.experts.gate_up_proj` [E, 2I, H] gate rows first,
    `block_sparse_moe.input_linear / output_linear`); a dense MLP stored beside them becomes the shared expert."""
    if arch.num_experts == 0 or arch.moe_style != "standard":
        return
    E = arch.num_experts
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        for src in ("block_sparse_moe.gate.weight", "block_sparse_moe.router.layer.weight", "mlp.gate.weight"):
            if p + src in sd:
                sd[p + "mlp.router.weight"] = sd.pop(p + src)
        for base, names in (("block_sparse_moe.experts.", ("w1", "w3", "w2")), ("mlp.experts.", ("gate_proj", "up_proj", "down_proj"))):
            if f"{p}{base}0.{names[0]}.weight" in sd:
                for nm, dst in zip(names, ("gate_proj", "up_proj", "down_proj")):
                    sd[p + "mlp.experts." + dst] = torch.stack([sd.pop(f"{p}{base}{e}.{nm}.weight").float() for e in range(E)])
        for fused, down in (("mlp.experts.gate_up_proj", None), ("block_sparse_moe.input_linear.weight", "block_sparse_moe.output_linear.weight")):
            if p + fused in sd and sd[p + fused].dim() == 3:
                gu = sd.pop(p + fused)
                half = gu.shape[1] // 2
                sd[p + "mlp.experts.gate_proj"], sd[p + "mlp.experts.up_proj"] = gu[:, :half].contiguous(), gu[:, half:].contiguous()
                if down is not None:
                    sd[p + "mlp.experts.down_proj"] = sd.pop(p + down)
        if arch.shared_expert_intermediate and p + "mlp.gate_proj.weight" in sd:      # from `shared_mlp.input_linear / output_linear`
            for nm in ("gate_proj", "up_proj", "down_proj"):
                sd[p + f"mlp.shared_expert.{nm}.weight"] = sd.pop(p + f"mlp.{nm}.weight")


def _canonical_family_names(sd: Dict[str, torch.Tensor], arch: ArchConfig) -> None:
    """Families whose checkpoints name (or lay out) their tensors differently from the llama convention this exporter reads."""
    mt = arch.model_type
    def rename(pairs):
        for k in list(sd):
            for old, new in pairs:
                if old in k:
                    sd[k.replace(old, new)] = sd.pop(k)
                    break
    if mt == "gpt2":
        # Conv1D modules keep [in, out] matrices; q, k, v share one of them
        H = arch.hidden_size
        for k in list(sd):
            v = sd[k]
            if k.endswith((".attn.bias", ".attn.masked_bias")):
                sd.pop(k)
                continue
            nk = k.replace("transformer.h.", "model.layers.").replace("transformer.wte.", "model.embed_tokens.").replace(
                "transformer.wpe.", "model.position_embeddings.").replace("transformer.ln_f.", "model.norm.").replace(
                ".ln_1.", ".input_layernorm.").replace(".ln_2.", ".post_attention_layernorm.")
            sd.pop(k)
            if ".attn.c_attn." in nk:
                parts = (v.t() if v.dim() == 2 else v).split(H, dim=0)
                for nm, part in zip(("q_proj", "k_proj", "v_proj"), parts):
                    sd[nk.replace(".attn.c_attn.", f".self_attn.{nm}.")] = part.contiguous()
            elif ".attn.c_proj." in nk:
                sd[nk.replace(".attn.c_proj.", ".self_attn.o_proj.")] = v.t().contiguous() if v.dim() == 2 else v
            elif ".mlp.c_fc." in nk:
                sd[nk.replace(".mlp.c_fc.", ".mlp.fc1.")] = v.t().contiguous() if v.dim() == 2 else v
            elif ".mlp.c_proj." in nk:
                sd[nk.replace(".mlp.c_proj.", ".mlp.fc2.")] = v.t().contiguous() if v.dim() == 2 else v
            else:
                sd[nk] = v
        sd["model.position_embeddings.weight"] = sd["model.position_embeddings.weight"][: arch.context_length]
    elif mt == "phi":
        rename([(".self_attn.dense.", ".self_attn.o_proj."), ("model.final_layernorm.", "model.norm.")])
    elif mt == "lfm2":
        rename([(".operator_norm.", ".input_layernorm."), (".ffn_norm.", ".post_attention_layernorm."), (".feed_forward.w1.", ".mlp.gate_proj."),
                (".feed_forward.w3.", ".mlp.up_proj."), (".feed_forward.w2.", ".mlp.down_proj."), (".self_attn.out_proj.", ".self_attn.o_proj."),
                (".self_attn.q_layernorm.", ".self_attn.q_norm."), (".self_attn.k_layernorm.", ".self_attn.k_norm."),
                ("model.embedding_norm.", "model.norm.")])
        for k in [k for k in sd if k.endswith("conv.conv.weight") and sd[k].dim() == 3]:
            sd[k] = sd[k].squeeze(1)
    elif mt == "nemotron":
        rename([(".mlp.up_proj.", ".mlp.fc1."), (".mlp.down_proj.", ".mlp.fc2.")])
    elif mt == "hunyuandensev1":
        rename([(".self_attn.query_layernorm.", ".self_attn.q_norm."), (".self_attn.key_layernorm.", ".self_attn.k_norm.")])
    elif mt == "chatglm":
        # transformer.encoder.layers.N.{self_attention.query_key_value, self_attention.dense, mlp.dense_h_to_4h [gate; up], mlp.dense_4h_to_h}
        rename([("transformer.embedding.word_embeddings.", "model.embed_tokens."), ("transformer.encoder.final_layernorm.", "model.norm."),
                ("transformer.output_layer.", "lm_head."), ("transformer.encoder.layers.", "model.layers.")])
        rename([(".self_attention.dense.", ".self_attn.o_proj."), (".mlp.dense_4h_to_h.", ".mlp.down_proj.")])
        for k in [k for k in sd if ".self_attention.query_key_value." in k]:
            v = sd.pop(k)
            for nm, part in zip(("q_proj", "k_proj", "v_proj"), torch.split(v, [arch.q_size, arch.kv_size, arch.kv_size], dim=0)):
                sd[k.replace(".self_attention.query_key_value.", f".self_attn.{nm}.")] = part.contiguous()
        for k in [k for k in sd if ".mlp.dense_h_to_4h." in k]:
            v = sd.pop(k)
            half = v.shape[0] // 2
            sd[k.replace(".mlp.dense_h_to_4h.", ".mlp.gate_proj.")], sd[k.replace(".mlp.dense_h_to_4h.", ".mlp.up_proj.")] = v[:half].contiguous(), v[half:].contiguous()
        for k in [k for k in sd if "rotary_pos_emb" in k]:
            sd.pop(k)
    elif mt == "internlm2":
        # wqkv rows are grouped by key/value head: the group's query heads, then its key head, then its value head
        # (reference: builders/internlm.py load_weights)
        rename([("model.tok_embeddings.", "model.embed_tokens."), (".attention_norm.", ".input_layernorm."), (".ffn_norm.", ".post_attention_layernorm."),
                (".feed_forward.w1.", ".mlp.gate_proj."), (".feed_forward.w3.", ".mlp.up_proj."), (".feed_forward.w2.", ".mlp.down_proj."),
                (".attention.wo.", ".self_attn.o_proj.")])
        if "output.weight" in sd:
            sd["lm_head.weight"] = sd.pop("output.weight")
        D, r = arch.head_dim, arch.num_heads // arch.num_kv_heads
        for k in [k for k in sd if ".attention.wqkv." in k]:
            v = sd.pop(k)
            g = v.reshape(arch.num_kv_heads, r + 2, D, *v.shape[1:])
            parts = (g[:, :r].reshape(arch.q_size, *v.shape[1:]), g[:, r].reshape(arch.kv_size, *v.shape[1:]), g[:, r + 1].reshape(arch.kv_size, *v.shape[1:]))
            for nm, part in zip(("q_proj", "k_proj", "v_proj"), parts):
                sd[k.replace(".attention.wqkv.", f".self_attn.{nm}.")] = part.contiguous()
    elif mt in ("olmo2", "exaone4"):
        # no norms before the sub-layers: placeholders for the exporter's node chain (the runtime adds without normalising)
        for i in range(arch.num_layers):
            sd.setdefault(f"model.layers.{i}.input_layernorm.weight", torch.ones(arch.hidden_size))
            sd.setdefault(f"model.layers.{i}.pre_feedforward_layernorm.weight", torch.ones(arch.hidden_size))
    elif mt == "olmo":
        H = arch.hidden_size
        for nm in [f"model.layers.{i}.{w}" for i in range(arch.num_layers) for w in ("input_layernorm", "post_attention_layernorm")] + ["model.norm"]:
            sd.setdefault(nm + ".weight", torch.ones(H))
            sd.setdefault(nm + ".bias", torch.zeros(H))


def _split_gated_q(sd: Dict[str, torch.Tensor], arch: ArchConfig) -> None:
    """q_proj of a gated-attention checkpoint holds [query | gate] per head: the gate halves become a projection of their own."""
    if not arch.attn_output_gate:
        return
    D = arch.head_dim
    for k in [k for k in sd if k.endswith("self_attn.q_proj.weight")]:
        v = sd[k]
        if v.shape[0] != 2 * arch.q_size:
            continue
        w = v.reshape(arch.num_heads, 2, D, v.shape[1])
        sd[k] = w[:, 0].reshape(arch.q_size, v.shape[1]).contiguous()
        sd[k[: -len("q_proj.weight")] + "gate_proj.weight"] = w[:, 1].reshape(arch.q_size, v.shape[1]).contiguous()


def _split_packed_qkv(sd: Dict[str, torch.Tensor], arch: ArchConfig) -> None:
    for k in [k for k in sd if k.endswith("__packed_qkv__")]:
        base = k[: -len("__packed_qkv__")]
        v = sd.pop(k)
        if hasattr(v, "rows"):   # a pre-quantised (AWQ / GPTQ) packed projection
            a, b = arch.q_size, arch.q_size + arch.kv_size
            q, kk, vv = v.rows(0, a), v.rows(a, b), v.rows(b, b + arch.kv_size)
        else:
            q, kk, vv = torch.split(v, [arch.q_size, arch.kv_size, arch.kv_size], dim=0)
        sd[base + "q_proj.weight"], sd[base + "k_proj.weight"], sd[base + "v_proj.weight"] = q, kk, vv


def create_model(model_name_or_dir: str, output_dir: str, precision: str, execution_provider: str, extra_options: Optional[dict] = None):
    extra = dict(extra_options or {})
    state_dict = None
    if model_name_or_dir in PRESETS:
        import copy
        arch = copy.deepcopy(PRESETS[model_name_or_dir])
    elif model_name_or_dir.endswith(".gguf") and os.path.isfile(model_name_or_dir):
        # a GGUF file: metadata -> architecture, tensors dequantised to fp32 under their Hugging Face names
        from .gguf_reader import hf_config_and_state_dict
        cfg, state_dict = hf_config_and_state_dict(model_name_or_dir)
        arch = from_hf_config(cfg)
    else:
        with open(os.path.join(model_name_or_dir, "config.json")) as f:
            raw_cfg = json.load(f)
        if (raw_cfg.get("architectures") or [""])[0] == "WhisperForConditionalGeneration" or raw_cfg.get("model_type") == "whisper":
            # encoder-decoder speech checkpoint: decoder.onnx + encoder.onnx + the log-mel front end's configuration
            arch, enc, dsd, esd = whisper_from_hf(raw_cfg, load_hf_state_dict(model_name_or_dir))
            for fn in ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "generation_config.json", "preprocessor_config.json",
                       "vocab.json", "merges.txt", "added_tokens.json", "normalizer.json"):
                if os.path.exists(os.path.join(model_name_or_dir, fn)):
                    os.makedirs(output_dir, exist_ok=True)
                    shutil.copy(os.path.join(model_name_or_dir, fn), os.path.join(output_dir, fn))
            return export_whisper(arch, enc, output_dir, precision, execution_provider, decoder_state_dict=dsd, encoder_state_dict=esd,
                                  num_frames=2 * enc.max_source_positions)
        arch = from_hf_config(raw_cfg)
        if not int(extra.get("random_weights", 0)) and not int(extra.get("synthetic_weights", 0)):
            state_dict = load_hf_state_dict(model_name_or_dir)
            _canonical_family_names(state_dict, arch)
            _split_packed_qkv(state_dict, arch)
            _split_gated_q(state_dict, arch)
            _canonical_moe_names(state_dict, arch)
            if precision != "int4":   # an int4 checkpoint exported at a float precision: dequantise
                state_dict = {k: (v.float() if hasattr(v, "matmulnbits") else v) for k, v in state_dict.items()}
        for fn in ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "tokenizer.model", "chat_template.jinja",
                   "generation_config.json"):
            src = os.path.join(model_name_or_dir, fn)
            if os.path.exists(src):
                os.makedirs(output_dir, exist_ok=True)
                shutil.copy(src, os.path.join(output_dir, fn))
    if state_dict is not None and int(extra.get("mtp_head", 0)):
        # the checkpoint's multi-token-prediction head as a model directory of its own under <output>/mtp (for MtpGenerator)
        from ..mtp import export_mtp_head, mtp_state_dict_from_hf
        head_sd = mtp_state_dict_from_hf(arch, state_dict)
        if head_sd is None:
            raise ValueError("mtp_head=1: the checkpoint has no mtp.* tensors")
        _split_gated_q(head_sd, arch)
        _canonical_moe_names(head_sd, arch)
        export_mtp_head(arch, os.path.join(output_dir, "mtp"), precision, execution_provider, state_dict=head_sd)
    if state_dict is not None:
        state_dict = {k: v for k, v in state_dict.items() if not k.startswith("mtp.")}
    qwen_vision = None
    if state_dict is not None and os.path.isdir(model_name_or_dir):
        with open(os.path.join(model_name_or_dir, "config.json")) as f:
            raw = json.load(f)
        if isinstance(raw.get("vision_config"), dict) and arch.model_type in ("qwen2_vl", "qwen2_5_vl") and not int(extra.get("text_only", 0)):
            # a Qwen2-VL / Qwen2.5-VL checkpoint: the vision tower is exported beside the decoder
            from . import qwen_vl
            vc = raw["vision_config"]
            v25 = arch.model_type == "qwen2_5_vl"
            vis = qwen_vl.QwenVisionConfig(
                depth=int(vc["depth"]), embed_dim=int(vc["hidden_size"] if v25 else vc["embed_dim"]), hidden_size=arch.hidden_size,
                num_heads=int(vc["num_heads"]), mlp_ratio=float(vc.get("mlp_ratio", 4.0)), in_channels=int(vc.get("in_channels", vc.get("in_chans", 3))),
                patch_size=int(vc.get("patch_size", 14)), spatial_merge_size=int(vc.get("spatial_merge_size", 2)),
                temporal_patch_size=int(vc.get("temporal_patch_size", 2)), variant="qwen2_5_vl" if v25 else "qwen2_vl",
                intermediate_size=int(vc.get("intermediate_size", 0)) if v25 else 0, window_size=int(vc.get("window_size", 112)),
                fullatt_blocks=",".join(str(int(b)) for b in vc.get("fullatt_block_indexes", [])) if v25 else "")
            qwen_vision = (vis, qwen_vl.strip_prefix(state_dict), int(raw.get("image_token_id", 151655)))
            state_dict = {k: v for k, v in state_dict.items() if not k.startswith(("model.visual.", "visual."))}
    if qwen_vision is not None:
        vis, vsd, image_token_id = qwen_vision
        return export_qwen_vl(
            arch, vis, output_dir, image_token_id, precision, execution_provider, decoder_state_dict=state_dict, vision_state_dict=vsd,
            seed=int(extra.get("seed", 0)), paged=bool(int(extra.get("paged_attention", extra.get("use_paged_attention", 0)))),
            block_size=int(extra.get("paged_block_size", 16)), max_batch_size=int(extra.get("max_batch_size", 64)),
            int4_symmetric=bool(int(extra.get("int4_is_symmetric", 0))), filename=extra.get("filename", "model.onnx"),
            context_length=int(extra["context_length"]) if "context_length" in extra else None, linear_format=str(extra.get("linear_format", "")),
            int4_algo_config=str(extra.get("int4_algo_config", "default")))
    return export_model(
        arch, output_dir, precision, execution_provider, state_dict=state_dict, seed=int(extra.get("seed", 0)),
        paged=bool(int(extra.get("paged_attention", extra.get("use_paged_attention", 0)))),
        block_size=int(extra.get("paged_block_size", 16)), max_batch_size=int(extra.get("max_batch_size", 64)),
        int4_symmetric=bool(int(extra.get("int4_is_symmetric", 0))), synthetic_weights=bool(int(extra.get("synthetic_weights", 0))),
        filename=extra.get("filename", "model.onnx"), context_length=int(extra["context_length"]) if "context_length" in extra else None,
        int4_tied_embeddings=bool(int(extra.get("int4_tied_embeddings", 0))), linear_format=str(extra.get("linear_format", "")),
        int4_algo_config=str(extra.get("int4_algo_config", "default")),
        mixed_precision={k: str(extra[k]) for k in ("last_matmul", "mixed_layers", "linear_attn") if k in extra} or None)


def main(argv=None):
    ap = argparse.ArgumentParser(description="Export a model directory (genai_config.json + ONNX + external data)")
    ap.add_argument("-m", "--model_name", required=True, help="Hugging Face model directory or a preset: " + ", ".join(PRESETS))
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("-p", "--precision", required=True, choices=["int4", "bf16", "fp16", "fp32"])
    ap.add_argument("-e", "--execution_provider", default="cuda", choices=["cpu", "cuda"])
    ap.add_argument("--extra_options", nargs="*", default=[], help="key=value pairs")
    a = ap.parse_args(argv)
    extra = dict(kv.split("=", 1) for kv in a.extra_options)
    out = create_model(a.model_name, a.output, a.precision, a.execution_provider, extra)
    print("saved", out)


if __name__ == "__main__":
    main()
