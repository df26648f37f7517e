"""Tensor parallelism over one node: one process per GPU, `torch.distributed` (NCCL) for rendezvous.

The reference has no distributed layer at all (no NCCL / MPI anywhere in its tree), so everything
here is new: attention heads and MLP columns are sharded at load time (models/loader.py), the
row-parallel projections (o_proj, down_proj) produce partial sums that must be added over ranks,
and the vocabulary-parallel LM head is gathered.

Two reduction back ends:
  * "nccl": `dist.all_reduce` — the baseline;
  * "fused": the one-shot all-reduce over NVLink peer memory, inside the GEMM epilogue for the row-parallel
    projections (csrc/gemm_common.cuh) and stand-alone for everything else (csrc/collectives.cu): every rank
    writes its partial tile into every rank's symmetric buffer, stamps an arrival flag, then sums all ranks'
    tiles from its own buffer in a fixed rank order, so every rank produces bit-identical results; see
    parallel/symm.py.
On CPU (gloo) the same class runs the multi-rank tests of the sharding math.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist


class TensorParallel:
    def __init__(self, rank: int, size: int, device: torch.device, group=None, backend: str = "nccl"):
        self.rank, self.size, self.device, self.group = rank, size, device, group
        self.backend = backend
        self.comm = None
        # steps with at least this many tokens (and a multiple of the world size) take the sequence-parallel form;
        # 0 (the default) keeps every step in the all-reduce form
        self.sp_min_tokens = int(os.environ.get("OGB_TP_SP_MIN_TOKENS", "0"))
        # mixture-of-experts layers: "replicated" (every rank routes all tokens, runs its experts, the all-reduce combines) or
        # "all_to_all" (tokens sharded, dispatch / combine exchange: parallel/ep.py)
        self.ep_mode = os.environ.get("OGB_EP_MODE", "replicated")
        if self.ep_mode not in ("replicated", "all_to_all"):
            raise RuntimeError("OGB_EP_MODE must be replicated or all_to_all")
        if backend == "fused":
            try:
                from .symm import SymmetricComm
                self.comm = SymmetricComm(rank, size, device, group)
            except Exception as e:  # symmetric memory unavailable: keep running on the NCCL baseline, loudly
                import warnings
                warnings.warn(f"fused tensor-parallel kernels disabled, falling back to NCCL: {e}")
                self.backend = "nccl"
            if self.comm is not None and os.environ.get("OGB_TP_SELF_TEST", "1") != "0" and not self._self_test():
                import warnings
                warnings.warn("fused tensor-parallel kernels failed their start-up check against NCCL; using the NCCL back end")
                self.comm = None
                self.backend = "nccl"

    def _self_test(self) -> bool:
        """One decode-sized GEMM + all-reduce in a single kernel and one stand-alone all-reduce, both against NCCL on the same
        data; every rank takes the same decision (the flags are min-reduced).  Bounded waits that run out surface as a kernel
        status, which is cleared here - a world whose peer protocol does not work runs on NCCL instead of failing later."""
        from .. import ops
        from ..ops import _lib
        dev = self.device
        ok = True
        try:
            g = torch.Generator(device="cpu").manual_seed(1234 + self.rank)
            x = (torch.randn(64, 512, generator=g) * 0.5).to(dev, torch.bfloat16)
            w = (torch.randn(1024, 512, generator=torch.Generator().manual_seed(99)) * 0.05).to(dev, torch.bfloat16)
            for _ in range(3):      # both buffer parities and a reuse
                want = ops.linear(x, w).float()
                dist.all_reduce(want, group=self.group)
                got = ops.linear(x, w, all_reduce=True).float()
                ok = ok and bool(torch.allclose(got, want, rtol=3e-2, atol=3e-2))
                y = x.clone()
                want2 = x.float().clone()
                dist.all_reduce(want2, group=self.group)
                got2 = self.comm.all_reduce(y).float()
                ok = ok and bool(torch.allclose(got2, want2, rtol=3e-2, atol=3e-2))
            torch.cuda.synchronize(dev)
            ok = ok and _lib.lib().ogb_status_read_and_clear(dev.index if dev.index is not None else torch.cuda.current_device()) == 0
        except Exception:
            ok = False
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        return bool(flag.item())

    @classmethod
    def from_env(cls, backend: Optional[str] = None) -> Optional["TensorParallel"]:
        """Builds the TP context from torchrun's environment; returns None for a single process."""
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world <= 1:
            return None
        rank = int(os.environ["RANK"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
            device = torch.device("cuda", local)
            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=device)
            be = backend or os.environ.get("OGB_TP_BACKEND", "fused")
        else:
            device = torch.device("cpu")
            if not dist.is_initialized():
                dist.init_process_group("gloo")
            be = "nccl"
        return cls(rank, world, device, None, be)

    def fused_ok(self, x: torch.Tensor, n_out: Optional[int] = None) -> bool:
        """True when the GEMM + all-reduce kernel can take this activation: decode-sized token counts with the flagged-line
        protocol; with NVLS switched on and OGB_TP_FUSED_PREFILL=1 also any step whose [tokens, n_out] output fits the
        multicast plane (measured slower than the persistent GEMM followed by a stand-alone all-reduce at two ranks)."""
        if self.comm is None or not x.is_cuda:
            return False
        if x.shape[0] <= self.comm.max_tokens:
            return True
        if self.comm.nvls_active and os.environ.get("OGB_TP_FUSED_PREFILL", "0") == "1":
            return n_out is None or x.shape[0] * n_out <= self.comm.nvls_plane_elems
        return False

    # row-parallel output: sum of partials over ranks (in place)
    def reduce(self, x: torch.Tensor, residual=None) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.comm is not None and x.dtype == torch.bfloat16 and (self.comm.nvls_active or x.numel() <= (1 << 20)) and self.comm.fits(x):
            # NVLS: the switch adds the ranks' planes (one-shot for small tensors, owner-reduces-and-multicasts for large ones).
            # Without multicast: one-shot pushes over peer memory, which win while the tensor is small (latency bound); larger
            # ones go to NCCL's bandwidth-optimal algorithms
            return self.comm.all_reduce(x.contiguous(), residual)
        if x.dtype == torch.bfloat16 and not x.is_cuda:
            y = x.float()
            dist.all_reduce(y, group=self.group)
            return (y if residual is None else y + residual.float()).to(x.dtype)
        dist.all_reduce(x, group=self.group)
        return x if residual is None else x + residual

    # vocabulary-parallel logits [B, V/size] -> [B, V]
    def gather_logits(self, x: torch.Tensor) -> torch.Tensor:
        if self.size == 1:
            return x
        if self.comm is not None and self.comm.fits_gather(x.contiguous()):
            g = self.comm.all_gather(x.contiguous())
            return g.permute(1, 0, 2).reshape(x.shape[0], -1)
        parts = [torch.empty_like(x) for _ in range(self.size)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def barrier(self):
        if self.size > 1:
            dist.barrier(group=self.group)


def leave(code: int = 0) -> None:
    """Ends a multi-rank process once its work is done: synchronise, meet the other ranks, flush, and exit
    without tearing the communicator down (captured graphs may still hold collective kernels, and destroying
    the process group under them can block)."""
    import sys
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(code)
