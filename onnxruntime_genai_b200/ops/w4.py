"""int4 block-32 weights (MatMulNBits) in the tile-contiguous layout of csrc/gemm_w4.cu.

`W4Weight.from_quantized(q, scales, zero_points)` repacks once at load time; `ops.linear` and
`ops.gate_up_act` accept a W4Weight wherever they accept a dense bf16 weight.  `dequantize()` restates
exactly what the kernel computes ((q - zp) times the checkpoint's scale, rounded to bf16 once) for the CPU
path and for the tests.  The scale travels as two bf16 numbers hi + lo (lo = scale - hi needs three mantissa bits for an fp16
scale, so the pair is exact; the zero point rides in lo's four spare mantissa bits).
"""
from __future__ import annotations

from typing import Optional

import torch

RECORD = 128 * 32 + 128 * 8


class W4Weight:
    def __init__(self, packed: torch.Tensor, N: int, K: int, q, scales, zp, interleaved: bool = False):
        self.packed, self.N, self.K = packed, N, K
        self._q, self._s, self._zp = q, scales, zp   # kept on the host for dequantize() (tests / CPU path)
        self.interleaved = interleaved
        self.shape = (N, K)

    @property
    def device(self):
        return self.packed.device

    @staticmethod
    def from_quantized(q: torch.Tensor, scales: torch.Tensor, zp: Optional[torch.Tensor], device, keep_host: bool = True,
                       interleaved: bool = False) -> "W4Weight":
        """q: uint8 [N, K] in 0..15; scales [N, K/32]; zp uint8 [N, K/32] (None = 8)."""
        N, K = q.shape
        assert K % 64 == 0, "K must be a multiple of 64"
        nb = K // 32
        dev = q.device   # the repack runs where the quantised tensors live (host for checkpoints, device for synthetic weights)
        if zp is None:
            zp = torch.full((N, nb), 8, dtype=torch.uint8, device=dev)
        Np = (N + 127) // 128 * 128
        qp = torch.zeros(Np, K, dtype=torch.int64, device=dev)
        qp[:N] = q.to(torch.int64)
        sp = torch.zeros(Np, nb, dtype=torch.float32, device=dev)
        sp[:N] = scales.float()
        zpp = torch.zeros(Np, nb, dtype=torch.float32, device=dev)
        zpp[:N] = zp.float()
        # nibble m of a word: pair p = m // 2 at bit 4p, second element of the pair 16 bits higher
        shifts = torch.tensor([0, 16, 4, 20, 8, 24, 12, 28], dtype=torch.int64, device=dev)
        words = (qp.view(Np, K // 8, 8) << shifts).sum(-1)                       # [Np, K/8] values < 2^32
        b = torch.stack([(words >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)  # little endian bytes
        nib = b.view(Np // 128, 128, K // 64, 32).permute(2, 0, 1, 3)             # [K/64, tiles, 128, 32]
        hi, lo_bits = split_scale(sp)
        second = (lo_bits | zpp.to(torch.int32)).to(torch.int16)                   # lo with the zero point in its low mantissa bits
        sz = torch.stack([hi.view(torch.int16), second], dim=-1)                   # [Np, nb, 2]
        szb = sz.view(Np, K // 64, 4).contiguous().view(torch.uint8).view(Np, K // 64, 8)
        szt = szb.view(Np // 128, 128, K // 64, 8).permute(2, 0, 1, 3)
        packed = torch.cat([nib.reshape(K // 64, Np // 128, 128 * 32), szt.reshape(K // 64, Np // 128, 128 * 8)], dim=-1).contiguous()
        return W4Weight(packed.to(device), N, K, q if keep_host else None, scales.float() if keep_host else None,
                        zp if keep_host else None, interleaved)

    def dequantize(self) -> torch.Tensor:
        """fp32 [N, K] weights exactly as the kernel reconstructs them."""
        if self._q is None:
            raise RuntimeError("host copy of the quantised weight was dropped")
        nb = self.K // 32
        d = self._q.float().view(self.N, nb, 32) - self._zp.float().view(self.N, nb, 1)
        hi, lo_bits = split_scale(self._s.view(self.N, nb).float())
        s = hi.float() + (lo_bits.to(torch.int32) << 16).view(torch.float32)
        return (d * s.view(self.N, nb, 1)).to(torch.bfloat16).float().view(self.N, self.K)


def split_scale(s: torch.Tensor):
    """fp32 scales -> (hi bf16, bits of lo as int32 in 0..0xFFF0): hi = bf16(s), lo = bf16(s - hi) with the low four mantissa
    bits cleared.  hi + lo == s for every fp16 value (11 significant bits = 8 + 3)."""
    hi = s.to(torch.bfloat16)
    lo = (s - hi.float()).to(torch.bfloat16)
    lo_bits = lo.view(torch.int16).to(torch.int32) & 0xFFF0
    return hi, lo_bits


def unpack_ort_q4(qweight: torch.Tensor, zero_points: Optional[torch.Tensor], N: int, K: int):
    """MatMulNBits tensors ([N, K/32, 16] bytes, low nibble = even k; zero points packed two per byte) ->
    q uint8 [N, K], zp uint8 [N, K/32] or None."""
    qb = torch.as_tensor(qweight).view(N, K // 32, 16)
    q = torch.stack([qb & 0xF, qb >> 4], dim=-1).view(N, K)
    zp = None
    if zero_points is not None:
        z = torch.as_tensor(zero_points).view(N, -1)
        zp = torch.stack([z & 0xF, z >> 4], dim=-1).view(N, -1)[:, :K // 32].contiguous()
    return q.contiguous(), zp


class QuantizedEmbedding:
    """An embedding table kept as the int4 block-32 tensors of a tied LM head (GatherBlockQuantized): q uint8 [V, K/2]
    (low nibble = even k), scales fp16 [V, K/32], zero points uint8 packed two per byte [V, ceil(K/64)] or None (8).
    `ops.embedding` gathers and dequantises rows on the fly; 5 bits per weight of HBM instead of 16."""
    dtype = torch.bfloat16

    def __init__(self, q: torch.Tensor, scales: torch.Tensor, zp: Optional[torch.Tensor], V: int, K: int):
        self.q, self.scales, self.zp, self.V, self.K = q.contiguous(), scales.contiguous(), zp.contiguous() if zp is not None else None, V, K
        self.shape = (V, K)

    @property
    def device(self):
        return self.q.device

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        """[V, K] exactly as the gather kernel reconstructs the rows (bf16 roundings included)."""
        V, K = self.V, self.K
        nb = K // 32
        qb = self.q.view(V, K // 2)
        qv = torch.stack([qb & 0xF, qb >> 4], dim=-1).view(V, nb, 32).float()
        if self.zp is not None:
            z = self.zp.view(V, -1)
            zp = torch.stack([z & 0xF, z >> 4], dim=-1).view(V, -1)[:, :nb].float()
        else:
            zp = torch.full((V, nb), 8.0, device=self.q.device)
        sc = self.scales.view(V, nb).float()
        return ((qv - zp[:, :, None]) * sc[:, :, None]).to(torch.bfloat16).to(dtype).view(V, K)
