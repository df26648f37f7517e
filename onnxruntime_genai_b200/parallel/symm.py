"""Symmetric peer memory for the fused GEMM + all-reduce kernel (csrc/gemm_tcgen05.cu).

Every rank owns one receive buffer `[2 parities][world sources][plane_elems / 4 lines]` of 16-byte lines
(8 payload bytes + the call's flag twice), mapped into every peer (NVLink peer access through
`torch.distributed._symmetric_memory`, which exchanges the memory handles over the process group).
The pointers are registered once with the kernel library (`ogb_comm_register`); after that the GEMM
launcher only needs a flag to run the fused path, so the call captures into CUDA graphs unchanged.

`LocalComm` registers a world of one on a single GPU: the kernel then pushes to and waits on its
own buffers, which exercises the whole protocol (parity, flagged lines, call counter) without peers.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from ..ops import _lib

DEFAULT_PLANE_ELEMS = int(__import__("os").environ.get("OGB_COMM_PLANE_ELEMS", 2048 * 4096))  # bf16 elements per source plane of the receive buffer
NVLS_PLANE_ELEMS = int(__import__("os").environ.get("OGB_NVLS_PLANE_ELEMS", 4096 * 8192))       # bf16 elements per NVLS plane (64 MiB)
NV_MAX_CTAS = 4096     # csrc/gemm_common.cuh


def _register(device_index: int, world: int, rank: int, buf_ptrs: List[int], epoch: torch.Tensor, plane_elems: int) -> None:
    arr_t = ctypes.c_void_p * world
    rc = _lib.lib().ogb_comm_register(device_index, world, rank, arr_t(*buf_ptrs), epoch.data_ptr(), plane_elems)
    if rc != 0:
        raise RuntimeError(f"ogb_comm_register failed with {rc}")


class _Collectives:
    """Stand-alone collectives over the registered buffers (csrc/collectives.cu).  Tensors are taken as raw 16-byte
    vectors for the gather; reductions are bf16.  `fits` tells whether a tensor can go through the kernels; callers
    fall back to NCCL otherwise."""

    nvls = False          # NVSwitch multicast buffers registered (SymmetricComm on a world with multicast support)
    nvls_plane_elems = 0

    @property
    def nvls_active(self) -> bool:
        """The reductions go through the multicast buffers (registered and switched on: OGB_TP_NVLS=1 or ogb_comm_set_options)."""
        return self.nvls and _lib.lib().ogb_comm_has_nvls(self.device.index) == 2

    def fits(self, x: torch.Tensor, planes: int = 1) -> bool:
        """planes: leading slices of a reduce-scatter input (each is one plane of the flagged-line buffers)."""
        nbytes = x.numel() * x.element_size()
        if not (x.is_cuda and x.is_contiguous() and (nbytes // planes) % 16 == 0 and x.data_ptr() % 16 == 0):
            return False
        return nbytes // planes // 2 <= self.plane_elems or (self.nvls_active and nbytes // 2 <= self.nvls_plane_elems)

    def fits_gather(self, x: torch.Tensor) -> bool:
        return self.fits(x) and (x.numel() * x.element_size() // 2 <= self.plane_elems or
                                 (self.nvls_active and self.size * x.numel() * x.element_size() // 2 <= self.nvls_plane_elems))

    def _run(self, mode: int, x: torch.Tensor, out: torch.Tensor, residual, n_units: int):
        from .. import ops
        ws = ops.workspace(x.device)
        rc = _lib.lib().ogb_collective(mode, x.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None,
                                       n_units, x.device.index, ws.status, ws.sm_count, torch.cuda.current_stream(x.device).cuda_stream)
        _lib.check(rc, "collective")
        return out

    def all_reduce(self, x: torch.Tensor, residual=None, out=None) -> torch.Tensor:
        """Sum over ranks (+ residual) of a bf16 tensor; every rank gets bit-identical results."""
        assert x.dtype == torch.bfloat16 and self.fits(x)
        return self._run(0, x, torch.empty_like(x) if out is None else out, residual, x.numel())

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[world, *x.shape]: every rank's tensor, any dtype."""
        assert self.fits_gather(x)
        out = torch.empty((self.size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        return self._run(1, x, out, None, x.numel() * x.element_size() // 2)

    def all_gather_push(self, x: torch.Tensor) -> None:
        """First half of all-gather -> GEMM: pushes this rank's token rows [rows, K] (bf16) into every rank's receive
        buffer and returns; the GEMM launched next (`ops.linear_gathered`) assembles its activation tiles from the lines
        as they arrive.  The call after that GEMM must be one that waits on every peer (any fused reduction)."""
        assert x.dtype == torch.bfloat16 and self.fits(x)
        self._run(3, x, x, None, x.numel())

    def reduce_scatter(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        """x [world, ...] bf16 partials -> sum over ranks of slice [rank] (+ residual)."""
        assert x.dtype == torch.bfloat16 and x.shape[0] == self.size and self.fits(x, self.size)
        out = torch.empty(x.shape[1:], dtype=x.dtype, device=x.device)
        return self._run(2, x, out, residual, out.numel())


class LocalComm(_Collectives):
    """World of one: the fused path talking to itself (single-GPU tests of the protocol)."""

    def __init__(self, device: torch.device, plane_elems: int = DEFAULT_PLANE_ELEMS):
        self.device = device
        self.plane_elems = plane_elems
        self.rank, self.size = 0, 1
        self.max_tokens = 256
        self.buf = torch.zeros(2 * plane_elems * 2, dtype=torch.bfloat16, device=device)   # lines carry 8 of their 16 bytes as payload
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        _lib.init_device(device.index)
        _register(device.index, 1, 0, [self.buf.data_ptr()], self.epoch, plane_elems)

    def close(self):
        _lib.lib().ogb_comm_register(self.device.index, 0, 0, None, None, 0)


class SymmetricComm(_Collectives):
    def __init__(self, rank: int, size: int, device: torch.device, group=None, plane_elems: int = DEFAULT_PLANE_ELEMS):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.rank, self.size, self.device, self.plane_elems = rank, size, device, plane_elems
        self.max_tokens = 256
        group = group or dist.group.WORLD
        self.buf = symm_mem.empty(2 * size * plane_elems * 2, dtype=torch.bfloat16, device=device)
        self.buf_h = symm_mem.rendezvous(self.buf, group)
        self.buf.zero_()     # a flag of zero never matches a call
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        _lib.init_device(device.index)
        _register(device.index, size, rank, [int(p) for p in self.buf_h.buffer_ptrs], self.epoch, plane_elems)
        dist.barrier(group=group)
        if __import__("os").environ.get("OGB_TP_NVLS", "") != "0":      # "0": do not even map the multicast buffers
            self._register_nvls(symm_mem, group, NVLS_PLANE_ELEMS)

    def _register_nvls(self, symm_mem, group, elems: int) -> None:
        """Second symmetric allocation for the multicast (NVLS) kernels: [data: 2 planes][out: 2 planes][counters], reached both
        through this rank's address and through the allocation's multicast address.  Skipped (the flagged-line kernels keep
        serving) when the allocation has no multicast mapping: no NVSwitch, or multicast objects cannot be shared here."""
        import torch.distributed as dist
        dev = self.device
        ctr_bytes = 2 * NV_MAX_CTAS * 4
        total = 2 * (2 * elems * 2) + ctr_bytes
        self.nv_buf = symm_mem.empty(total, dtype=torch.uint8, device=dev)
        self.nv_h = symm_mem.rendezvous(self.nv_buf, group)
        mc = int(getattr(self.nv_h, "multicast_ptr", 0) or 0)
        ok = torch.tensor([1 if mc else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if not int(ok.item()):
            self.nv_buf = self.nv_h = None
            return
        self.nv_buf.zero_()
        self.nv_expected = torch.zeros(2 * NV_MAX_CTAS, dtype=torch.int32, device=dev)
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)
        base = self.nv_buf.data_ptr()
        o_out, o_ctr = 2 * elems * 2, 2 * (2 * elems * 2)
        P = ctypes.c_void_p
        rc = _lib.lib().ogb_comm_register_nvls(dev.index, P(base), P(mc), P(base + o_out), P(mc + o_out), P(base + o_ctr), P(mc + o_ctr),
                                               P(self.nv_expected.data_ptr()), elems)
        if rc != 0:
            raise RuntimeError(f"ogb_comm_register_nvls failed with {rc}")
        self.nvls, self.nvls_plane_elems = True, elems
        dist.barrier(group=group)
