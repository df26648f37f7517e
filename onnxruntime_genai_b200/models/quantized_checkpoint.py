"""Readers for pre-quantised Hugging Face checkpoints: AWQ and GPTQ int4 tensors are carried over into the MatMulNBits
layout, ModelOpt FP8 / NVFP4 tensors into MatMulBlockQuantizedFp8Weight / MatMulBlockQuantizedFp4Weight, without a
second quantisation.

Reference: src/python/py/models/quantized_model.py (`AWQModel`, `GPTQModel`, unpack / repack at :1017-1107).  Those
checkpoints group the scales over 128 (or 64, 32) input features; the kernels here use blocks of 32, and a group of
g = 32 * r features is the same quantisation as r blocks of 32 sharing one scale and zero point, so the conversion
repeats each scale / zero point r times and loses nothing.

    AWQ  (quant_method "awq"):  qweight int32 [K, N/8], qzeros int32 [K/g, N/8], scales fp16 [K/g, N];
                                the eight nibbles of a word hold output features in the order 0 2 4 6 1 3 5 7
    Quark (quant_method "quark"): dense layers packed like AWQ.
    Olive (quant_method "olive"): qweight uint8 [N, K/2], scales [N, K/g], qzeros uint8 [N, K/g/2], unsigned, per-layer overrides.
    GPTQ (quant_method "gptq"): qweight int32 [K/8, N] (eight consecutive input features per word),
                                qzeros int32 [K/g, N/8] (sequential nibbles; stored minus one by the v1 format),
                                scales fp16 [K/g, N], g_idx int32 [K] (group of each input feature)

`QuantizedLinear` is what the exporter receives in the state dict in place of a float weight.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

AWQ_ORDER = (0, 2, 4, 6, 1, 3, 5, 7)   # nibble i of a word holds column 8 * word + AWQ_ORDER... inverse below


@dataclass
class QuantizedLinear:
    """w[n, k] = (q[n, k] - zp[n, k // 32]) * scales[n, k // 32]"""
    q: torch.Tensor        # uint8 [N, K], values 0..15
    scales: torch.Tensor   # fp32 [N, K/32]
    zp: torch.Tensor       # uint8 [N, K/32]

    @property
    def shape(self):
        return tuple(self.q.shape)

    def float(self) -> torch.Tensor:
        N, K = self.q.shape
        return ((self.q.float().view(N, K // 32, 32) - self.zp.float()[..., None]) * self.scales[..., None]).view(N, K)

    def rows(self, lo: int, hi: int) -> "QuantizedLinear":
        return QuantizedLinear(self.q[lo:hi], self.scales[lo:hi], self.zp[lo:hi])

    @staticmethod
    def cat(parts) -> "QuantizedLinear":
        return QuantizedLinear(torch.cat([p.q for p in parts], 0), torch.cat([p.scales for p in parts], 0), torch.cat([p.zp for p in parts], 0))

    def matmulnbits(self):
        """(qweight uint8 [N, K/32, 16], scales fp32 [N, K/32], zero points packed two per byte [N, ceil(K/64)])."""
        N, K = self.q.shape
        qb = self.q.view(N, K // 32, 32)
        packed = (qb[..., 0::2] | (qb[..., 1::2] << 4)).contiguous()
        zp = self.zp
        if zp.shape[1] % 2:
            zp = torch.cat([zp, torch.full((N, 1), 8, dtype=torch.uint8)], dim=1)
        return packed, self.scales, (zp[:, 0::2] | (zp[:, 1::2] << 4)).contiguous()


@dataclass
class Fp8Linear:
    """ModelOpt FP8 linear: w[n, k] = e4m3(q8[n, k]) * scale[n]  (a scalar scale of the checkpoint is repeated per row)."""
    q8: torch.Tensor       # uint8 view of float8_e4m3fn [N, K]
    scale: torch.Tensor    # fp32 [N, 1]
    kind = "fp8"

    @property
    def shape(self):
        return tuple(self.q8.shape)

    def float(self) -> torch.Tensor:
        return self.q8.view(torch.float8_e4m3fn).float() * self.scale

    def rows(self, lo: int, hi: int) -> "Fp8Linear":
        return Fp8Linear(self.q8[lo:hi], self.scale[lo:hi])

    @staticmethod
    def cat(parts) -> "Fp8Linear":
        return Fp8Linear(torch.cat([p.q8 for p in parts], 0), torch.cat([p.scale for p in parts], 0))


@dataclass
class Nvfp4Linear:
    """ModelOpt NVFP4 linear: e2m1 codes [N, K/2] (low nibble = even k), e4m3 scales per block of 16 [N, K/16] (uint8 view), one
    fp32 global scale."""
    codes: torch.Tensor
    scales: torch.Tensor
    global_scale: torch.Tensor
    kind = "nvfp4"

    @property
    def shape(self):
        return (self.codes.shape[0], self.codes.shape[1] * 2)

    def float(self) -> torch.Tensor:
        from .builder import dequantize_nvfp4
        return dequantize_nvfp4(self.codes, self.scales, self.global_scale)

    def rows(self, lo: int, hi: int) -> "Nvfp4Linear":
        return Nvfp4Linear(self.codes[lo:hi], self.scales[lo:hi], self.global_scale)

    @staticmethod
    def cat(parts):
        """Stacked projections share one global scale only if the checkpoint gave them the same one; otherwise None (the
        caller falls back to the dequantised weights)."""
        g0 = float(parts[0].global_scale.reshape(-1)[0])
        if any(float(p.global_scale.reshape(-1)[0]) != g0 for p in parts):
            return None
        return Nvfp4Linear(torch.cat([p.codes for p in parts], 0), torch.cat([p.scales for p in parts], 0), parts[0].global_scale)


def convert_modelopt(sd: Dict[str, torch.Tensor]) -> Dict[str, object]:
    """ModelOpt checkpoints: `<name>.weight` in float8_e4m3fn with `<name>.weight_scale` (FP8), or packed uint8 codes with
    `<name>.weight_scale` (e4m3 per block of 16) and `<name>.weight_scale_2` (NVFP4).  Activation scales (`input_scale`) and
    KV scales are dropped: activations stay 16-bit here."""
    out: Dict[str, object] = {}
    for k, v in sd.items():
        if k.endswith((".input_scale", ".k_scale", ".v_scale")):
            continue
        if k.endswith((".weight_scale", ".weight_scale_2")) and k.rsplit(".", 1)[0] + ".weight" in sd:
            continue
        if k.endswith(".weight") and k[:-len(".weight")] + ".weight_scale" in sd:
            base = k[:-len(".weight")]
            if base + ".weight_scale_2" in sd:
                sc = sd[base + ".weight_scale"]
                out[k] = Nvfp4Linear(v.view(torch.uint8), sc.view(torch.uint8) if sc.dtype != torch.uint8 else sc,
                                     sd[base + ".weight_scale_2"].float().reshape(1))
            else:
                q8 = v.view(torch.uint8) if v.dtype != torch.uint8 else v
                scale = sd[base + ".weight_scale"].float().reshape(-1, 1)
                out[k] = Fp8Linear(q8, scale.expand(q8.shape[0], 1).contiguous() if scale.numel() == 1 else scale)
        else:
            out[k] = v
    return out


def _nibbles(words: torch.Tensor) -> torch.Tensor:
    """int32 [...] -> uint8 [..., 8]: nibble i = bits 4i .. 4i+3."""
    w = words.to(torch.int64) & 0xFFFFFFFF
    return torch.stack([(w >> (4 * i)) & 0xF for i in range(8)], dim=-1).to(torch.uint8)


def _to_block32(q_kn: torch.Tensor, scales_gn: torch.Tensor, zeros_gn: torch.Tensor, group: int) -> QuantizedLinear:
    """q [K, N], scales / zeros [K/group, N] -> block-32 form with [N, ...] tensors."""
    K, N = q_kn.shape
    if group % 32 or K % group:
        raise NotImplementedError(f"group size {group} is not a multiple of 32 dividing K = {K}")
    r = group // 32
    return QuantizedLinear(q_kn.t().contiguous(), scales_gn.float().t().repeat_interleave(r, dim=1).contiguous(),
                           zeros_gn.to(torch.uint8).t().repeat_interleave(r, dim=1).contiguous())


def unpack_awq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group: int) -> QuantizedLinear:
    K = qweight.shape[0]
    inv = torch.tensor([AWQ_ORDER.index(i) for i in range(8)])          # column j of a word sits in nibble inv[j]
    q = _nibbles(qweight)[..., inv].reshape(K, -1)                      # [K, N]
    z = _nibbles(qzeros)[..., inv].reshape(qzeros.shape[0], -1)         # [K/g, N]
    return _to_block32(q, scales, z, group)


def unpack_gptq(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group: int, g_idx: Optional[torch.Tensor] = None,
                zero_offset: int = 1) -> QuantizedLinear:
    N = qweight.shape[1]
    q = _nibbles(qweight).permute(0, 2, 1).reshape(-1, N)               # [K, N]: word w, nibble i -> input feature 8w + i
    K = q.shape[0]
    if group <= 0:
        group = K
    z = (_nibbles(qzeros).reshape(qzeros.shape[0], -1).to(torch.int16) + zero_offset) & 0xF    # v1 stores zero - 1
    if g_idx is not None and not torch.equal(g_idx.to(torch.int64), torch.arange(K) // group):
        # act-order (desc_act): input feature k belongs to group g_idx[k], groups are no longer runs of consecutive features, so
        # the codes cannot be carried into block-32 tensors.  The weight is reconstructed exactly as the checkpoint defines it
        # and handed on as a float tensor (an int4 export quantises it again with the exporter's own method).
        g = g_idx.to(torch.int64)
        w_kn = (q.float() - z[:, :N].float()[g]) * scales.float()[g]
        return w_kn.t().contiguous()
    return _to_block32(q, scales, z[:, :N], group)


def unpack_olive(qweight: torch.Tensor, qzeros: Optional[torch.Tensor], scales: torch.Tensor, group: int) -> QuantizedLinear:
    """Olive's layout is the MatMulNBits one before blocking: qweight uint8 [N, K/2] (low nibble = even input feature), scales
    [N, K/group], qzeros uint8 [N, K/group/2] packed the same way, unsigned codes (reference: quantized_model.py:1598-1648)."""
    N = qweight.shape[0]
    qb = qweight.to(torch.uint8)
    q = torch.stack([qb & 0xF, qb >> 4], dim=-1).reshape(N, -1)                    # [N, K]
    K = q.shape[1]
    if group <= 0:
        group = K
    if group % 32 or K % group:
        raise NotImplementedError(f"group size {group} is not a multiple of 32 dividing K = {K}")
    G = K // group
    if qzeros is not None and qzeros.numel():
        zb = qzeros.to(torch.uint8).reshape(N, -1)
        z = torch.stack([zb & 0xF, zb >> 4], dim=-1).reshape(N, -1)[:, :G]
    else:
        z = torch.full((N, G), 8, dtype=torch.uint8)
    r = group // 32
    return QuantizedLinear(q.contiguous(), scales.float().reshape(N, G).repeat_interleave(r, dim=1).contiguous(),
                           z.repeat_interleave(r, dim=1).contiguous())


def convert_state_dict(sd: Dict[str, torch.Tensor], quant_config: dict) -> Dict[str, object]:
    """Replaces every `<name>.qweight / .qzeros / .scales (/ .g_idx)` group by `<name>.weight = QuantizedLinear`."""
    method = str(quant_config.get("quant_method", "")).lower()
    if method == "modelopt":
        return convert_modelopt(sd)
    bits = int(quant_config.get("bits", quant_config.get("w_bit", 4)))
    group = int(quant_config.get("group_size", quant_config.get("q_group_size", 128)))
    if method not in ("awq", "gptq", "quark", "olive") or bits != 4:
        raise NotImplementedError(f"quantised checkpoint of method {method!r} with {bits} bits is not supported (awq / gptq / quark / olive, 4 bits)")
    overrides = (quant_config.get("overrides") or {}) if method == "olive" else {}
    # GPTQ v1 stores zero points minus one; the v2 format (checkpoint_format "gptq_v2") stores them as they are
    zero_offset = 0 if str(quant_config.get("checkpoint_format", "gptq")).lower() == "gptq_v2" else 1
    out: Dict[str, object] = {}
    for k, v in sd.items():
        if k.endswith(".qweight"):
            base = k[: -len(".qweight")]
            if method in ("awq", "quark"):       # Quark's dense layers use AWQ's packing (reference: quantized_model.py:802-868)
                out[base + ".weight"] = unpack_awq(v, sd[base + ".qzeros"], sd[base + ".scales"], group)
            elif method == "olive":
                ov = overrides.get(base, {})
                if int(ov.get("bits", 4)) != 4:
                    raise NotImplementedError(f"{base}: Olive override to {ov['bits']} bits is not supported")
                out[base + ".weight"] = unpack_olive(v, sd.get(base + ".qzeros"), sd[base + ".scales"], int(ov.get("group_size", group)))
            else:
                out[base + ".weight"] = unpack_gptq(v, sd[base + ".qzeros"], sd[base + ".scales"], group, sd.get(base + ".g_idx"), zero_offset)
        elif k.endswith((".qzeros", ".scales", ".g_idx")) and k.rsplit(".", 1)[0] + ".qweight" in sd:
            continue
        else:
            out[k] = v
    return out


# ---------------------------------------------------------------------------------------------- writers (tests, tooling)
def pack_awq(ql: QuantizedLinear, group: int):
    """Inverse of unpack_awq for a block-32 tensor whose scales repeat over `group` (used to make test checkpoints)."""
    N, K = ql.q.shape
    r = group // 32
    order = torch.tensor(AWQ_ORDER)
    shifts = (4 * torch.arange(8)).to(torch.int64)

    def words(x_kn):   # [R, N] -> int32 [R, N/8]
        v = x_kn.to(torch.int64).view(x_kn.shape[0], N // 8, 8)[..., order]
        w = (v << shifts).sum(-1)
        return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)

    return words(ql.q.t()), words(ql.zp[:, ::r].t()), ql.scales[:, ::r].t().contiguous().to(torch.float16)


def pack_gptq(ql: QuantizedLinear, group: int, zero_offset: int = 1):
    N, K = ql.q.shape
    r = group // 32
    shifts = (4 * torch.arange(8)).to(torch.int64)

    def signed(w):
        return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)

    qw = signed((ql.q.t().to(torch.int64).view(K // 8, 8, N).permute(0, 2, 1) << shifts).sum(-1))          # [K/8, N]
    z = ((ql.zp[:, ::r].t().to(torch.int64) - zero_offset) & 0xF).view(-1, N // 8, 8)
    return qw, signed((z << shifts).sum(-1)), ql.scales[:, ::r].t().contiguous().to(torch.float16), (torch.arange(K) // group).to(torch.int32)
