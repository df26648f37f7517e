"""MXFP4 expert weights (QMoE: FP4 e2m1 codes + one e8m0 power-of-two scale per block of 32 along K) kept packed
on the device in the tile-contiguous layout of csrc/gemm_fp4.cu: 4.25 bits per weight of HBM instead of 16.

`Fp4Experts.from_codes(codes, scale_codes)` repacks once at load time; `ops.moe_gemm` accepts an Fp4Experts
wherever it accepts the dense bf16 [E, N, K] tensor.  `dequantize()` restates what the kernel computes (the e2m1
value times 2^(scale - 127), exact in bf16) for the CPU path and the tests.

Reference semantics: QMoE with quant_type fp4 as emitted by src/python/py/models/builders/base.py:4276-4408
(weights [E, K, N/2] with two output features per byte, scales [E, N, K/32]).
"""
from __future__ import annotations

from typing import Optional

import torch

RECORD = 128 * 32 + 128 * 2
F16_SCALE_CODES = (113, 140)   # fp16 form: 2^(code - 127) must be a normal fp16 and 6 * scale finite
E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
MAX_SCALE_CODE = 128   # 2^(code - 1) must be a finite bf16: the kernel multiplies by 2^126 * 2^(code - 127)


def unpack_qmoe_fp4(packed: torch.Tensor) -> torch.Tensor:
    """QMoE weight bytes [E, K, N/2] (even n in the low nibble) -> e2m1 codes uint8 [E, N, K]."""
    E, K, half = packed.shape
    kn = torch.stack([packed & 0xF, packed >> 4], dim=-1).view(E, K, half * 2)
    return kn.transpose(1, 2).contiguous()


class Fp4Experts:
    """E matrices of [N, K] MXFP4 weights.  `packed` is the device tensor the grouped GEMM streams; `codes` /
    `scale_codes` stay on the host when `keep_host` (tests, CPU restatement)."""

    def __init__(self, packed: torch.Tensor, E: int, N: int, K: int, codes, scale_codes, half: bool = False):
        self.packed, self.E, self.N, self.K = packed, E, N, K
        self.half = half       # fp16 form: fp16 multipliers, fp16 activations
        self._codes, self._scales = codes, scale_codes
        self.shape = (E, N, K)
        self.dtype = torch.bfloat16

    @property
    def device(self):
        return self.packed.device

    @property
    def is_cuda(self):
        return self.packed.is_cuda

    @staticmethod
    def supported(scale_codes: torch.Tensor, K: int) -> bool:
        return K % 64 == 0 and int(scale_codes.max()) <= MAX_SCALE_CODE

    @staticmethod
    def fits_fp16(codes: torch.Tensor, scale_codes: torch.Tensor) -> bool:
        """True when every block that holds a non-zero weight has its scale inside the fp16 form's range."""
        E, N, K = codes.shape
        nz = ((codes & 7) != 0).view(E, N, K // 32, 32).any(-1)
        s = scale_codes.to(torch.int16)
        return bool(((s >= F16_SCALE_CODES[0]) & (s <= F16_SCALE_CODES[1]) | ~nz).all())

    @staticmethod
    def from_codes(codes: torch.Tensor, scale_codes: torch.Tensor, device, keep_host: bool = True, half=None) -> "Fp4Experts":
        """codes uint8 [E, N, K] in 0..15 (bit 3 = sign); scale_codes uint8 [E, N, K/32].  half: the fp16 form
        (None = whenever the block scales allow it)."""
        E, N, K = codes.shape
        assert K % 64 == 0, "K must be a multiple of 64"
        if half is None:
            half = Fp4Experts.fits_fp16(codes, scale_codes)
        if half:
            assert Fp4Experts.fits_fp16(codes, scale_codes), "block scale outside 2^-14 .. 2^13"
        else:
            assert int(scale_codes.max()) <= MAX_SCALE_CODE, "block scale above 2^1 cannot be folded into a bf16 multiplier"
        dev = codes.device
        nb = K // 32
        Np = (N + 127) // 128 * 128
        parts = []
        # bf16 form: element m of a word at pair p = m // 2, bit 4p, second element of the pair 16 bits higher.
        # fp16 form: element i < 4 at nibble 2i, element 4 + i at nibble 2i + 1 (the even nibbles of a word are four
        # consecutive k values, the odd nibbles the next four), and the eight words of a row's 64 k values are stored in
        # the order (q, b) -> word 2q + b holds k = 32b + 8q .. + 8: the 16 codes that one lane of the streaming kernel
        # needs (8 of each block of 32) are 8 contiguous bytes.
        order = [0, 8, 16, 24, 4, 12, 20, 28] if half else [0, 16, 4, 20, 8, 24, 12, 28]
        shifts = torch.tensor(order, dtype=torch.int64, device=dev)
        word_src = torch.tensor([4 * (w & 1) + (w >> 1) for w in range(8)], dtype=torch.int64, device=dev)   # record word -> k chunk
        for e in range(E):   # one expert at a time bounds the int64 temporaries
            qp = torch.zeros(Np, K, dtype=torch.int64, device=dev)
            qp[:N] = codes[e].to(torch.int64)
            words = (qp.view(Np, K // 8, 8) << shifts).sum(-1)
            if half:
                words = words.view(Np, K // 64, 8)[:, :, word_src].reshape(Np, K // 8)
            b = torch.stack([(words >> (8 * i)) & 0xFF for i in range(4)], dim=-1).to(torch.uint8)
            nib = b.view(Np // 128, 128, K // 64, 32).permute(2, 0, 1, 3)                 # [K/64, tiles, 128, 32]
            mul = torch.zeros(Np, nb, dtype=torch.uint8, device=dev)
            if half:    # code + 6 (the kernels subtract to the fp16 exponent field they need); blocks of zeros may carry any scale
                mul[:N] = (scale_codes[e].to(torch.int16).clamp(*F16_SCALE_CODES) + 6).to(torch.uint8)
            else:       # bf16 exponent field of 2^(code - 1)
                mul[:N] = (scale_codes[e].to(torch.int16) + 126).to(torch.uint8)
            mt = mul.view(Np // 128, 128, K // 64, 2).permute(2, 0, 1, 3)
            parts.append(torch.cat([nib.reshape(K // 64, Np // 128, 128 * 32), mt.reshape(K // 64, Np // 128, 128 * 2)], dim=-1))
        packed = torch.stack(parts).contiguous().to(device)
        return Fp4Experts(packed, E, N, K, codes.cpu() if keep_host else None, scale_codes.cpu() if keep_host else None, half)

    def dequantize(self, e: Optional[int] = None) -> torch.Tensor:
        """fp32 [E, N, K] (or [N, K] of one expert) exactly as the kernel reconstructs the weights."""
        if self._codes is None:
            raise RuntimeError("host copy of the quantised experts was dropped")
        c = self._codes if e is None else self._codes[e:e + 1]
        s = self._scales if e is None else self._scales[e:e + 1]
        grid = torch.tensor(E2M1, dtype=torch.float32)
        mag = grid[(c & 7).long()]
        val = torch.where(c >= 8, -mag, mag)
        scale = torch.pow(2.0, s.float() - 127.0)
        w = (val.view(c.shape[0], self.N, self.K // 32, 32) * scale[..., None]).view(c.shape[0], self.N, self.K)
        return w if e is None else w[0]
