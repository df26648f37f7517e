"""Device ops.  CUDA tensors run the hand-written sm_100a kernels (ctypes into
libogb200_kernels.so); CPU tensors run the fp32 PyTorch restatements in `reference.py`.

There is deliberately no third path: a CUDA tensor never falls back to PyTorch math, and a missing
kernel library on a GPU machine is an error.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import numpy as np
import torch

from . import reference as ref
from . import _lib
from .fp4 import Fp4Experts
from .w4 import QuantizedEmbedding, W4Weight, unpack_ort_q4

_ACT = {"silu": 0, "gelu": 1, "gelu_tanh": 1, "relu": 2, "gelu_erf": 3, "relu2": 4}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


class _Workspace:
    """Per-device state shared by the kernels: the status word and the split-KV scratch of attention
    (the GEMM's split-K reduces on chip and needs none).  Allocated once (outside graph capture)."""

    def __init__(self, device: torch.device):
        self.device = device
        idx = device.index if device.index is not None else torch.cuda.current_device()
        self.index = idx
        _lib.init_device(idx)
        self.status = _lib.lib().ogb_status_device_ptr(idx)
        self.sm_count = _lib.lib().ogb_sm_count(idx)
        self.attn_ws = torch.empty(64 << 20, dtype=torch.uint8, device=device)
        self._retired = []

    def attn_scratch(self, nbytes: int) -> torch.Tensor:
        if nbytes > self.attn_ws.numel():
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("attention scratch too small during CUDA graph capture; warm up eagerly first")
            # captured graphs hold the raw address of the buffer they were recorded with: a replaced buffer is kept alive
            # for the life of the process instead of going back to the allocator, where a replay would write into it
            self._retired.append(self.attn_ws)
            self.attn_ws = torch.empty(int(nbytes * 1.25), dtype=torch.uint8, device=self.device)
        return self.attn_ws


_workspaces = {}


def workspace(device: torch.device) -> _Workspace:
    key = device.index if device.index is not None else torch.cuda.current_device()
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = _Workspace(torch.device("cuda", key))
    return ws


def check_kernel_status(device=None) -> None:
    """Synchronises and raises if any kernel reported that a bounded wait ran out."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index
    _lib.init_device(idx)
    _lib.check_status(idx)


# ------------------------------------------------------------------------------------------ graph capture
import contextlib
import gc


@contextlib.contextmanager
def graph_capture(graph, **kw):
    """torch.cuda.graph with the cyclic garbage collector off for the duration of the capture: a collected object that owns CUDA
    resources (an older graph, a pinned buffer) frees them from inside the capture and invalidates it
    ("operation failed due to a previous error during capture" at the next launch)."""
    was_on = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph, **kw):
            yield
    finally:
        if was_on:
            gc.enable()


# ------------------------------------------------------------------------------------------ debug bounds checks
# OGB_DEBUG_BOUNDS=1: every index tensor an op is about to hand to a kernel (token ids, cache slots, block-table entries,
# gathered rows, rotary positions) is range-checked first and a bad one raises IndexError naming the op, instead of the kernel
# reading or writing out of bounds.  The checks synchronise the stream, so this is a debugging mode (and CUDA graphs that
# were captured with it on replay without checks).
DEBUG_BOUNDS = os.environ.get("OGB_DEBUG_BOUNDS", "0") == "1"


def _check_index(op: str, name: str, t, hi: int, lo: int = 0) -> None:
    if not DEBUG_BOUNDS or t is None or t.numel() == 0 or (t.is_cuda and torch.cuda.is_current_stream_capturing()):
        return
    bad = (t < lo) | (t >= hi)
    if bool(bad.any()):
        v = t[bad].flatten()[0].item()
        raise IndexError(f"{op}: {name} holds {v}, outside [{lo}, {hi})")


# ------------------------------------------------------------------------------------------ embedding
def embedding(ids: torch.Tensor, table, scale: float = 1.0) -> torch.Tensor:
    _check_index("embedding", "ids", ids, table.V if isinstance(table, QuantizedEmbedding) else table.shape[0])
    if isinstance(table, QuantizedEmbedding):
        if table.device.type != "cuda":
            return ref.embedding(ids, table.dequantize(), scale)
        T = ids.numel()
        out = torch.empty(T, table.K, dtype=torch.bfloat16, device=table.device)
        _lib.check(_lib.lib().ogb_embedding_q4(_ptr(ids), _ptr(table.q), _ptr(table.scales), _ptr(table.zp), _ptr(out), T, table.K,
                                              table.V, float(scale), _stream()), "embedding_q4")
        return out
    if not table.is_cuda:
        return ref.embedding(ids, table, scale)
    assert table.dtype == torch.bfloat16 and ids.dtype == torch.int32
    T, H = ids.numel(), table.shape[1]
    out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _lib.check(_lib.lib().ogb_embedding(_ptr(ids), _ptr(table), _ptr(out), T, H, table.shape[0], float(scale), _stream()), "embedding")
    return out


# ------------------------------------------------------------------------------------------ norm
def norm(x, weight, eps, residual=None, bias=None, layernorm=False, out=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Returns (normalised, new_residual).  With `residual`, normalises x + residual and returns the
    sum as new_residual (written in place into `residual`)."""
    if not x.is_cuda:
        y, r = ref.norm(x, weight, eps, residual, bias, layernorm)
        if residual is not None:
            residual.copy_(r)
            r = residual
        return y, r
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    rows, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    _lib.check(_lib.lib().ogb_norm(_ptr(x), _ptr(residual), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out), rows, H,
                                   float(eps), int(layernorm), _stream()), "norm")
    return out, residual


class PendingCombine:
    """The output of a mixture-of-experts layer before its combine step: the experts' rows `y` and the routing plan.
    `norm_moe_combine` folds the weighted sum into the residual add + norm that consumes it."""
    __slots__ = ("y", "plan")

    def __init__(self, y, plan):
        self.y, self.plan = y, plan


def norm_moe_combine(pending: PendingCombine, weight, eps, residual, bias=None, layernorm=False):
    """norm(moe_combine(pending.y, pending.plan), weight, eps, residual, ...) in one launch; same results bit for bit."""
    y, plan = pending.y, pending.plan
    assert y.is_cuda and y.dtype == torch.bfloat16 and y.stride(-1) == 1 and residual is not None
    H = y.shape[1]
    out = torch.empty(plan.T, H, dtype=torch.bfloat16, device=y.device)
    _lib.check(_lib.lib().ogb_norm_moe_combine(_ptr(y), y.stride(0), _ptr(plan.inv_pos), _ptr(plan.topk_w), plan.k, _ptr(residual),
                                               _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out), plan.T, H, float(eps), int(layernorm),
                                               _stream()), "norm_moe_combine")
    return out, residual


# ------------------------------------------------------------------------------------------ GEMM
GEMM_FP32_OUT, GEMM_ACT_PAIR, GEMM_ALLREDUCE, GEMM_REDUCE_SCATTER, GEMM_GATHERED_A = 1, 2, 4, 8, 16


FUSED_MAX_TOKENS = 128     # the decode-step fusions (folded norm, rotary + cache append) run in the decode-sized GEMM kernel


def _gemm(x, w, out, bias, residual, flags, splits, fused=None):
    ws = workspace(x.device)
    T, K = x.shape
    if fused is None:
        rc = _lib.lib().ogb_gemm_bf16(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), T, w.shape[0], K, _ptr(bias),
                                      _ptr(residual), residual.stride(0) if residual is not None else 0, int(flags), int(splits),
                                      ws.index, ws.status, ws.sm_count, _stream())
    else:
        import ctypes
        rc = _lib.lib().ogb_gemm_bf16_fused(_ptr(x), x.stride(0), _ptr(w), w.stride(0), _ptr(out), out.stride(0), T, w.shape[0], K,
                                            _ptr(bias), _ptr(residual), residual.stride(0) if residual is not None else 0, int(flags),
                                            int(splits), ws.index, ws.status, ws.sm_count, _stream(), ctypes.byref(fused))
    _lib.check(rc, "gemm_bf16")
    return out


_ones = {}


def _unit_weight(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    t = _ones.get(key)
    if t is None:
        t = _ones[key] = torch.ones(n, dtype=torch.bfloat16, device=device)
    return t


def rms_scale(x, eps: float):
    """x / rms(x) (no weight): the rows a GEMM with a folded norm would see, for the paths that cannot fold."""
    if not x.is_cuda:
        return ref.rms_scale(x, eps)
    return norm(x, _unit_weight(x.shape[1], x.device), eps)[0]


def _gemm_w4(x, w, out, bias, residual, flags, splits):
    ws = workspace(x.device)
    rc = _lib.lib().ogb_gemm_w4(_ptr(x), x.stride(0), _ptr(w.packed), _ptr(out), out.stride(0), x.shape[0], w.N, w.K, _ptr(bias),
                                _ptr(residual), residual.stride(0) if residual is not None else 0, int(flags), int(splits),
                                ws.status, ws.sm_count, _stream())
    _lib.check(rc, "gemm_w4")
    return out


def linear(x, w, bias=None, residual=None, out_fp32=False, out=None, splits=0, all_reduce=False, reduce_scatter=None, norm_eps=0.0):
    """y = x @ w.T (+bias) (+residual).  x [T, K] bf16, w [N, K] bf16 (K contiguous).  With all_reduce the
    partial products of the tensor-parallel ranks are summed inside the kernel over NVLink peer memory.
    reduce_scatter=(rank, world): the sum is scattered by token rows instead (sequence-parallel form): the result has
    this rank's rows [rank * ceil(T / world), ...) only, and `residual` is that slice.
    norm_eps > 0: an RMS norm folded into the GEMM - x holds the un-normalised rows, w already carries the norm's weight
    (w * norm_weight along K), and row m of the product is scaled by rsqrt(mean(x[m]^2) + norm_eps)."""
    if isinstance(w, W4Weight):
        if norm_eps > 0:
            x = rms_scale(x, norm_eps)
        if not x.is_cuda:
            return ref.linear(x, w.dequantize(), bias, residual, out_fp32)
        if all_reduce:
            raise RuntimeError("the fused all-reduce is not available for int4 weights")
        if out is None:
            out = torch.empty(x.shape[0], w.N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
        return _gemm_w4(x, w, out, bias, residual, GEMM_FP32_OUT if out_fp32 else 0, splits)
    if not x.is_cuda:
        return ref.linear(x, w, bias, residual, out_fp32, norm_eps)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert x.stride(-1) == 1 and w.stride(-1) == 1
    fused = None
    if norm_eps > 0:
        if x.shape[0] > FUSED_MAX_TOKENS:
            x = rms_scale(x, norm_eps)     # prefill-sized steps run the persistent kernel: normalise first
        else:
            fused = _lib.GemmFused(norm_eps=float(norm_eps))
    rows_out = x.shape[0]
    if reduce_scatter is not None:
        rank, world = reduce_scatter
        per = -(-x.shape[0] // world)
        rows_out = max(0, min(per, x.shape[0] - rank * per))
    if out is None:
        out = torch.empty(rows_out, w.shape[0], dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    flags = (GEMM_FP32_OUT if out_fp32 else 0) | (GEMM_ALLREDUCE if all_reduce else 0) | (GEMM_REDUCE_SCATTER if reduce_scatter else 0)
    return _gemm(x, w, out, bias, residual, flags, splits, fused)


def qkv_rope_append(x, w, bias, positions, slots, cos_cache, sin_cache, k_cache, v_cache, Hq, Hkv, D, rot, norm_eps=0.0):
    """QKV projection + rotary embedding + KV-cache append (+ folded RMS norm) as one kernel for decode-sized steps.
    Returns a tensor whose first Hq * D columns are the rotated queries (what paged_attention reads); rotated keys and the
    values of token m are written to row slots[m] of the caches.  Non-interleaved rotation only; head_dim must divide 128,
    the rotary dimension must be a multiple of 16 and the caches bf16 - `qkv_fusable` tells; other cases (and prefill-sized
    steps) take the separate kernels."""
    T = x.shape[0]
    _check_index("qkv_rope_append", "slots", slots[:T], k_cache.shape[0], -1)
    if cos_cache is not None:
        _check_index("qkv_rope_append", "positions", positions[:T], cos_cache.shape[0])
    if x.is_cuda and T <= FUSED_MAX_TOKENS and not isinstance(w, W4Weight) and qkv_fusable(D, rot, k_cache):
        assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] == (Hq + 2 * Hkv) * D
        q = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=x.device)
        f = _lib.GemmFused(norm_eps=float(norm_eps), positions=_ptr(positions), slots=_ptr(slots), cos=_ptr(cos_cache), sin=_ptr(sin_cache),
                           k_cache=_ptr(k_cache), v_cache=_ptr(v_cache), Hq=Hq, Hkv=Hkv, D=D, rot=int(rot if cos_cache is not None else 0),
                           max_pos=cos_cache.shape[0] if cos_cache is not None else 1)
        return _gemm(x, w, q, bias, None, 0, 0, f)
    qkv = linear(x, w, bias, norm_eps=norm_eps)
    rope_kv_append(qkv, positions, slots, cos_cache, sin_cache, k_cache, v_cache, Hq, Hkv, D, rot)
    return qkv


def qkv_fusable(D: int, rot: int, k_cache) -> bool:
    return 128 % D == 0 and rot % 16 == 0 and k_cache.dtype == torch.bfloat16


def linear_gathered(M: int, w, bias=None, out_fp32=False, act_pair=False, splits=0):
    """all-gather -> GEMM in one kernel: y[M, N] = X @ w.T where X's token rows were pushed by the ranks with
    `comm.all_gather_push` (rank r: rows [r * ceil(M / world), ...)) just before; the kernel builds its activation
    tiles from the flagged lines in the local receive buffer as they arrive.  act_pair: silu(gate) * up epilogue for
    weights in the 64-row gate/up block layout."""
    N, K = w.shape
    dev = w.device
    out = torch.empty(M, N // 2 if act_pair else N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=dev)
    ws = workspace(dev)
    flags = (GEMM_FP32_OUT if out_fp32 else 0) | (GEMM_ACT_PAIR if act_pair else 0) | GEMM_GATHERED_A
    rc = _lib.lib().ogb_gemm_bf16(_ptr(w), K, _ptr(w), w.stride(0), _ptr(out), out.stride(0), M, N, K, _ptr(bias), None, 0, int(flags),
                                  int(splits), ws.index, ws.status, ws.sm_count, _stream())
    _lib.check(rc, "gemm_bf16 (gathered activations)")
    return out


def interleave_gate_up(w: torch.Tensor, block: int = 64) -> torch.Tensor:
    """[gate; up] stacked rows ([2I, ...]) -> blocks of 64 gate rows followed by the 64 up rows of the same
    features, the row order the paired-activation GEMM epilogue expects.  Works for weights and biases."""
    inter = w.shape[0] // 2
    assert inter % block == 0
    g, u = w[:inter].reshape(inter // block, 1, block, *w.shape[1:]), w[inter:].reshape(inter // block, 1, block, *w.shape[1:])
    return torch.cat([g, u], dim=1).reshape(w.shape).contiguous()


def gate_up_act(x, w, bias=None, act="silu", out=None, splits=0, interleaved=False, norm_eps=0.0):
    """act(x @ Wg.T) * (x @ Wu.T).  w is [2I, K]: stacked [Wg; Wu], or (interleaved=True) blocks of 64 gate
    rows + 64 up rows as produced by interleave_gate_up (the layout the fused kernel needs).  norm_eps: as in `linear`."""
    fused = None
    if norm_eps > 0:
        if not x.is_cuda:
            return ref.gate_up_act(x, w.dequantize() if isinstance(w, W4Weight) else w, bias, act,
                                   w.interleaved if isinstance(w, W4Weight) else interleaved, norm_eps)
        if isinstance(w, W4Weight) or x.shape[0] > FUSED_MAX_TOKENS or act != "silu" or not interleaved or (w.shape[0] // 2) % 64:
            x = rms_scale(x, norm_eps)
        else:
            fused = _lib.GemmFused(norm_eps=float(norm_eps))
    if isinstance(w, W4Weight):
        if not x.is_cuda:
            return ref.gate_up_act(x, w.dequantize(), bias, act, w.interleaved)
        inter = w.N // 2
        if act == "silu" and w.interleaved:
            if out is None:
                out = torch.empty(x.shape[0], inter, dtype=torch.bfloat16, device=x.device)
            return _gemm_w4(x, w, out, bias, None, GEMM_ACT_PAIR, splits)
        y = linear(x, w, bias)
        if w.interleaved:
            y = y.view(-1, inter // 64, 2, 64).transpose(1, 2).reshape(-1, 2 * inter)
        return act_mul(y.contiguous(), act)
    if not x.is_cuda:
        return ref.gate_up_act(x, w, bias, act, interleaved)
    inter = w.shape[0] // 2
    if act != "silu" or not interleaved or inter % 64:
        y = linear(x, w, bias)
        if interleaved:
            y = y.view(-1, inter // 64, 2, 64).transpose(1, 2).reshape(-1, 2 * inter)
        return act_mul(y.contiguous(), act)
    if out is None:
        out = torch.empty(x.shape[0], inter, dtype=torch.bfloat16, device=x.device)
    return _gemm(x, w, out, bias, None, GEMM_ACT_PAIR, splits, fused)


def act_mul(x, act="silu"):
    if not x.is_cuda:
        return ref.act_mul(x, act)
    T, two_i = x.shape
    out = torch.empty(T, two_i // 2, dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().ogb_act_mul(_ptr(x), _ptr(out), T, two_i // 2, _ACT[act], _stream()), "act_mul")
    return out


def short_conv(bcx, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, block_size: int):
    """Gated short depthwise convolution of a hybrid (LFM2) layer over packed sequences; appends b * x of this step's tokens
    to the paged `cache` [slots, C] (see ops/reference.py::short_conv for the definition).  Returns [T, C]."""
    if not bcx.is_cuda:
        return ref.short_conv(bcx, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, block_size)
    T, C = bcx.shape[0], weight.shape[0]
    assert bcx.dtype == torch.bfloat16 and bcx.stride(1) == 1 and weight.is_contiguous() and cache.is_contiguous()
    assert block_table.stride(1) == 1
    out = torch.empty(T, C, dtype=bcx.dtype, device=bcx.device)
    _lib.check(_lib.lib().ogb_short_conv(_ptr(bcx), bcx.stride(0), _ptr(weight), _ptr(bias), _ptr(cache), _ptr(slots), _ptr(positions),
                                        _ptr(cu_seqlens), _ptr(past_lens), _ptr(block_table), block_table.stride(0), int(block_size),
                                        _ptr(out), T, past_lens.shape[0], C, weight.shape[1], _stream()), "short_conv")
    return out


def causal_conv(x, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, block_size: int, silu: bool = True):
    """Causal depthwise convolution (no gates) of the recurrent layer kinds over packed sequences, with the window of earlier
    positions read from the paged `cache` [slots, C] that this step's rows are appended to; optional SiLU.  x [T, C] may be a
    column slice of a wider tensor.  Returns [T, C] in x's dtype."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.stride(1) != 1 or (x.stride(0) % 8) or (x.data_ptr() % 16):
        ones = torch.ones_like(x)
        y = short_conv(torch.cat([ones, ones, x], dim=1).contiguous(), weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, block_size)
        return torch.nn.functional.silu(y.float()).to(x.dtype) if silu else y
    T, C = x.shape[0], weight.shape[0]
    assert weight.is_contiguous() and cache.is_contiguous() and block_table.stride(1) == 1
    out = torch.empty(T, C, dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().ogb_causal_conv(_ptr(x), x.stride(0), _ptr(weight), _ptr(bias), _ptr(cache), _ptr(slots), _ptr(positions),
                                         _ptr(cu_seqlens), _ptr(past_lens), _ptr(block_table), block_table.stride(0), int(block_size),
                                         _ptr(out), T, past_lens.shape[0], C, weight.shape[1], int(silu), _stream()), "causal_conv")
    return out


def gated_delta(q, k, v, g, beta, state, slots, cu_seqlens, past_lens):
    """Gated-delta-rule recurrence of a linear-attention layer over packed sequences (see ops/reference.py::gated_delta).
    state [slots, Hv, dk, dv] fp32 is updated in place."""
    if not q.is_cuda:
        return ref.gated_delta(q, k, v, g, beta, state, slots, cu_seqlens, past_lens)
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and state.dtype == torch.float32
    assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous() and state.is_contiguous()
    gf, bf = g.float().contiguous(), beta.float().contiguous()
    out = torch.empty(T, Hv, dv, dtype=torch.bfloat16, device=q.device)
    B = past_lens.shape[0]
    _lib.check(_lib.lib().ogb_gated_delta(_ptr(q), _ptr(k), _ptr(v), _ptr(gf), _ptr(bf), _ptr(state), _ptr(slots), _ptr(cu_seqlens), _ptr(past_lens),
                                          _ptr(out), B, Hk, Hv, dk, dv, _stream()), "gated_delta")
    return out


def gated_delta_layer(conv, proj, cd, vd, Hk, Hv, dk, dv, neg_exp_a, dt_bias, norm_w, norm_eps, state, slots, cu_seqlens, past_lens):
    """The part of a gated-delta-net layer between its convolution and its output projection, as two kernels on bf16 CUDA tensors:
    conv [T, cd] = silu(conv1d([q | k | v])), proj [T, cd + vd + 2 Hv] = the input projection [qkv | z | b | a].  q and k are
    L2-normalised per head (q also scaled by dk^-0.5), beta = sigmoid(b), log-decay = neg_exp_a * softplus(a + dt_bias), the
    recurrence updates `state` in place, and the result is RMS-normalised per value head, weighted and gated by silu(z).
    Returns [T, Hv * dv]."""
    T = conv.shape[0]
    assert conv.is_cuda and conv.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16 and conv.stride(1) == 1 and proj.stride(1) == 1
    kd = Hk * dk
    o = torch.empty(T, Hv, dv, dtype=torch.bfloat16, device=conv.device)
    B = past_lens.shape[0]
    _lib.check(_lib.lib().ogb_gated_delta_fused(_ptr(conv), conv.stride(0), 0, kd, 2 * kd, _ptr(proj), proj.stride(0), cd + vd, cd + vd + Hv,
                                                _ptr(neg_exp_a), _ptr(dt_bias), float(dk) ** -0.5, _ptr(state), _ptr(slots), _ptr(cu_seqlens),
                                                _ptr(past_lens), _ptr(o), B, Hk, Hv, dk, dv, _stream()), "gated_delta_fused")
    out = torch.empty(T, Hv * dv, dtype=torch.bfloat16, device=conv.device)
    z = proj[:, cd:cd + vd]
    _lib.check(_lib.lib().ogb_gdn_gate_norm(_ptr(o), _ptr(z), proj.stride(0), _ptr(norm_w), float(norm_eps), _ptr(out), T, Hv, dv, _stream()),
               "gdn_gate_norm")
    return out


def mamba2_layer(conv, proj, heads, groups, P, N, dt_bias, neg_a, Dv, norm_w, norm_eps, state, slots, cu_seqlens, past_lens):
    """The part of a Mamba-2 layer between its convolution and its output projection, as two kernels on bf16 CUDA tensors:
    conv [T, I + 2 G N] = silu(conv1d([x | B | C])), proj [T, I + conv width + heads] = the input projection [z | xBC | dt].
    step = softplus(dt + dt_bias), the scan updates `state` in place, y * silu(z) is RMS-normalised over the whole width I = heads * P
    and weighted.  Returns [T, I]."""
    T = conv.shape[0]
    I = heads * P
    assert conv.is_cuda and conv.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16 and conv.stride(1) == 1 and proj.stride(1) == 1
    y = torch.empty(T, I, dtype=torch.bfloat16, device=conv.device)
    dt_raw = proj[:, I + conv.shape[1]:]
    _lib.check(_lib.lib().ogb_mamba2_scan_fused(_ptr(conv), conv.stride(0), _ptr(dt_raw), proj.stride(0), _ptr(dt_bias), _ptr(neg_a), _ptr(Dv),
                                                _ptr(state), _ptr(slots), _ptr(cu_seqlens), _ptr(past_lens), _ptr(y), past_lens.shape[0], heads,
                                                groups, P, N, _stream()), "mamba2_scan_fused")
    out = torch.empty(T, I, dtype=torch.bfloat16, device=conv.device)
    _lib.check(_lib.lib().ogb_mamba_gate_norm(_ptr(y), _ptr(proj), proj.stride(0), _ptr(norm_w), float(norm_eps), _ptr(out), T, I, _stream()),
               "mamba_gate_norm")
    return out


def mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu_seqlens, past_lens):
    """Mamba-2 selective scan of a state-space layer over packed sequences (see ops/reference.py::mamba2_scan).
    state [slots, heads, N, P] fp32 is updated in place."""
    if not x.is_cuda:
        return ref.mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu_seqlens, past_lens)
    T, heads, P = x.shape
    groups, N = Bm.shape[1], Bm.shape[2]
    assert x.dtype == torch.bfloat16 and Bm.dtype == torch.bfloat16 and Cm.dtype == torch.bfloat16 and state.dtype == torch.float32
    assert x.is_contiguous() and Bm.is_contiguous() and Cm.is_contiguous() and state.is_contiguous()
    dtf, af, df = dt.float().contiguous(), neg_a.float().contiguous(), Dv.float().contiguous()
    out = torch.empty(T, heads, P, dtype=torch.bfloat16, device=x.device)
    _lib.check(_lib.lib().ogb_mamba2_scan(_ptr(x), _ptr(dtf), _ptr(af), _ptr(Bm), _ptr(Cm), _ptr(df), _ptr(state), _ptr(slots), _ptr(cu_seqlens),
                                          _ptr(past_lens), _ptr(out), past_lens.shape[0], heads, groups, P, N, _stream()), "mamba2_scan")
    return out


def copy_state_slots(src: torch.Tensor, dst: torch.Tensor, src_slots, dst_slots) -> None:
    """dst[:, dst_slots[i]] = src[:, src_slots[i]] for recurrent-state pools [layers, slots, ...] fp32 of the same shape (snapshots
    of linear-attention states around a speculative round)."""
    assert src.shape == dst.shape and src.dtype == dst.dtype == torch.float32 and src.is_contiguous() and dst.is_contiguous()
    ss = torch.as_tensor(src_slots, dtype=torch.int32, device=src.device).reshape(-1)
    ds = torch.as_tensor(dst_slots, dtype=torch.int32, device=src.device).reshape(-1)
    assert ss.numel() == ds.numel()
    if ss.numel() == 0:
        return
    if not src.is_cuda:
        dst[:, ds.long()] = src[:, ss.long()]
        return
    L, S = src.shape[0], src.shape[1]
    elems = src[0, 0].numel()
    _lib.check(_lib.lib().ogb_copy_state_slots(_ptr(src), _ptr(dst), L, S, elems, _ptr(ss), _ptr(ds), ss.numel(), _stream()), "copy_state_slots")


def decode_advance(sampled, input_ids, positions, past_lens, slot_mapping, sample_pos, block_table, block_size: int):
    """In place: the packed inputs of a one-token-per-request step become those of the next step (see
    csrc/elementwise.cu::decode_advance_kernel).  block_table [B, cols] int32, everything else [B] int32."""
    B = sampled.shape[0]
    if DEBUG_BOUNDS:
        _check_index("decode_advance", "positions + 1 (block-table column)", positions[:B] + 1, block_table.shape[1] * block_size)
    if not sampled.is_cuda:
        pos = positions[:B] + 1
        input_ids[:B] = sampled
        positions[:B] = pos
        past_lens[:B] += 1
        sample_pos[:B] += 1
        col = (pos // block_size).long()
        blk = torch.where(col < block_table.shape[1], block_table[torch.arange(B), col.clamp(max=block_table.shape[1] - 1)], torch.full_like(pos, -1))
        slot_mapping[:B] = torch.where(blk < 0, torch.full_like(pos, -1), blk * block_size + pos % block_size)
        return
    assert block_table.stride(1) == 1
    _lib.check(_lib.lib().ogb_decode_advance(_ptr(sampled), _ptr(input_ids), _ptr(positions), _ptr(past_lens), _ptr(slot_mapping),
                                            _ptr(sample_pos), _ptr(block_table), block_table.stride(0), int(block_size), B, _stream()),
               "decode_advance")


def activation(x, act="gelu"):
    """Elementwise activation of a bf16 tensor (the fc1 -> act -> fc2 MLPs of phi and gpt2)."""
    if not x.is_cuda:
        return ref.activation(x, act)
    x = x.contiguous()
    out = torch.empty_like(x)
    _lib.check(_lib.lib().ogb_act(_ptr(x), _ptr(out), x.numel(), _ACT[act], _stream()), "activation")
    return out


# ------------------------------------------------------------------------------------------ mixture of experts
def interleave_experts_gate_up(w: torch.Tensor, fused_interleaved: bool = True, block: int = 64) -> torch.Tensor:
    """Per-expert gate/up rows ([E, 2I, ...]; fused_interleaved: even rows = gate, odd rows = up, else [gate; up])
    -> per expert blocks of 64 gate rows followed by the 64 up rows of the same features."""
    E, two_i = w.shape[0], w.shape[1]
    inter = two_i // 2
    assert inter % block == 0
    if fused_interleaved:
        g, u = w[:, 0::2], w[:, 1::2]
    else:
        g, u = w[:, :inter], w[:, inter:]
    g = g.reshape(E, inter // block, 1, block, *w.shape[2:])
    u = u.reshape(E, inter // block, 1, block, *w.shape[2:])
    return torch.cat([g, u], dim=2).reshape(w.shape).contiguous()


class MoePlan:
    """Device-side routing of one MoE layer call (no host readback): which expert serves which sorted row."""
    __slots__ = ("T", "k", "E", "bt", "max_tiles", "topk_idx", "topk_w", "expert_offsets", "sorted_token", "inv_pos", "tile_expert",
                 "tile_row0", "tile_rows", "num_tiles")


def moe_route(router_logits: torch.Tensor, k: int, mode: int = 0, expert_range=None, token_tile: int = 0, topk=None) -> MoePlan:
    """router_logits [T, E] fp32 -> MoePlan (top-k, routing weights, rows grouped by expert, GEMM tile list).
    mode 0: softmax over the selected logits; 1: softmax over all experts; 2: the latter renormalised.
    expert_range (lo, hi): only these experts are local (expert parallelism).  topk = (idx int32 [T, k], weights fp32 [T, k]):
    a selection made elsewhere (PhiMoE's sparse mixer); only the grouping by expert is computed."""
    assert router_logits.is_cuda and router_logits.dtype == torch.float32 and router_logits.stride(-1) == 1
    T, E = router_logits.shape
    L = _lib.lib()
    dev = router_logits.device
    lo, hi = expert_range if expert_range is not None else (0, E)
    pl = MoePlan()
    n = T * k
    bt = token_tile or L.ogb_gemm_token_tile(max(1, min(T, -(-2 * n // max(1, hi - lo)))), 0)
    pl.T, pl.k, pl.E, pl.bt = T, k, E, bt
    pl.max_tiles = L.ogb_moe_max_tiles(n, hi - lo, bt)
    i32 = dict(dtype=torch.int32, device=dev)
    if topk is not None:
        pl.topk_idx, pl.topk_w = topk
        assert pl.topk_idx.dtype == torch.int32 and pl.topk_w.dtype == torch.float32 and pl.topk_idx.shape == (T, k)
    else:
        pl.topk_idx = torch.empty(T, k, **i32)
        pl.topk_w = torch.empty(T, k, dtype=torch.float32, device=dev)
    pl.expert_offsets = torch.empty(E + 1, **i32)
    pl.sorted_token = torch.empty(n, **i32)
    pl.inv_pos = torch.empty(T, k, **i32)
    tiles = torch.empty(3 * pl.max_tiles + 1, **i32)
    pl.tile_expert, pl.tile_row0, pl.tile_rows = tiles[:pl.max_tiles], tiles[pl.max_tiles:2 * pl.max_tiles], tiles[2 * pl.max_tiles:3 * pl.max_tiles]
    pl.num_tiles = tiles[3 * pl.max_tiles:]
    if topk is None:
        _lib.check(L.ogb_moe_topk(_ptr(router_logits), router_logits.stride(0), T, E, k, mode, _ptr(pl.topk_idx), _ptr(pl.topk_w), _stream()),
                   "moe_topk")
    _lib.check(L.ogb_moe_sort(_ptr(pl.topk_idx), T, k, E, lo, hi, bt, _ptr(pl.expert_offsets), _ptr(pl.sorted_token), _ptr(pl.inv_pos),
                              _ptr(pl.tile_expert), _ptr(pl.tile_row0), _ptr(pl.tile_rows), _ptr(pl.num_tiles), pl.max_tiles, _stream()),
               "moe_sort")
    return pl


def moe_fp4_reads_rows(w, plan: MoePlan) -> bool:
    """True when moe_gemm over these packed experts takes the un-gathered bf16 rows plus the plan's row map (row_map=True)."""
    return isinstance(w, Fp4Experts) and w.half and bool(_lib.lib().ogb_moe_fp4_reads_row_map(plan.bt, w.K, 1))


def moe_gemm(xs: torch.Tensor, w: torch.Tensor, plan: MoePlan, bias=None, act_kind: int = 0, alpha: float = 1.0, limit: float = 0.0,
             out_dtype=torch.bfloat16, row_map: bool = False):
    """Grouped expert GEMM over rows sorted by expert.  xs [T*k, K] bf16; w [E, N, K] bf16; bias [E, N].
    act_kind 0: plain; 1: silu(gate)*up; 2: clamped SwiGLU(alpha, limit) — both need the 64-row gate/up blocks
    of interleave_experts_gate_up and return N/2 columns."""
    E, N, K = w.shape
    assert xs.is_cuda and xs.stride(-1) == 1
    ws = workspace(xs.device)
    if isinstance(w, Fp4Experts):
        # MXFP4 experts stay packed in HBM; the kernel expands each tile in shared memory (csrc/gemm_fp4.cu).  The fp16 form
        # takes fp16 rows (ops.gather_rows(..., f16=True) or the previous grouped GEMM with out_dtype=torch.float16).
        # row_map: xs holds the bf16 token rows [T, K] as they are; the kernel reads sorted row r from xs[plan.sorted_token[r]]
        assert out_dtype in (torch.bfloat16, torch.float16)
        assert xs.dtype == (torch.bfloat16 if row_map else (torch.float16 if w.half else torch.bfloat16))
        rows = plan.T * plan.k if row_map else xs.shape[0]
        out = torch.empty(rows, N // 2 if act_kind else N, dtype=out_dtype, device=xs.device)
        flags = (GEMM_ACT_PAIR if act_kind else 0) | (16 if w.half else 0) | (32 if out_dtype == torch.float16 else 0)
        rc = _lib.lib().ogb_moe_gemm_fp4(_ptr(xs), xs.stride(0), _ptr(w.packed), _ptr(out), out.stride(0), rows, N, K, E, _ptr(bias),
                                         flags, int(act_kind), float(alpha), float(limit),
                                         _ptr(plan.tile_expert), _ptr(plan.tile_row0), _ptr(plan.tile_rows), _ptr(plan.num_tiles),
                                         plan.max_tiles, plan.bt, plan.T, _ptr(plan.sorted_token) if row_map else None, ws.status,
                                         _stream())   # plan.T: an expert sees a token at most once
        _lib.check(rc, "moe_gemm_fp4")
        return out
    assert xs.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous()
    out = torch.empty(xs.shape[0], N // 2 if act_kind else N, dtype=torch.bfloat16, device=xs.device)
    rc = _lib.lib().ogb_moe_gemm(_ptr(xs), xs.stride(0), _ptr(w), K, _ptr(out), out.stride(0), xs.shape[0], N, K, E, _ptr(bias),
                                 GEMM_ACT_PAIR if act_kind else 0, int(act_kind), float(alpha), float(limit), _ptr(plan.tile_expert),
                                 _ptr(plan.tile_row0), _ptr(plan.tile_rows), _ptr(plan.num_tiles), plan.max_tiles, plan.bt, ws.status,
                                 _stream())
    _lib.check(rc, "moe_gemm")
    return out


def moe_combine(y: torch.Tensor, plan: MoePlan, residual=None) -> torch.Tensor:
    """out[t] = (residual[t]) + sum_j w[t, j] * y[row(t, j)]; rows of experts that are not local are skipped."""
    out = torch.empty(plan.T, y.shape[1], dtype=torch.bfloat16, device=y.device)
    rc = _lib.lib().ogb_moe_combine(_ptr(y), y.stride(0), _ptr(plan.inv_pos), _ptr(plan.topk_w), plan.T, plan.k, y.shape[1], _ptr(residual),
                                    residual.stride(0) if residual is not None else 0, _ptr(out), out.stride(0), _stream())
    _lib.check(rc, "moe_combine")
    return out


# ------------------------------------------------------------------------------------------ RoPE + KV append
def rope_kv_append(qkv, positions, slots, cos_cache, sin_cache, k_cache, v_cache, Hq, Hkv, D, rot, interleaved=False,
                   q_norm_w=None, k_norm_w=None, norm_eps=1e-6, positions3=None, mrope_section=None, mrope_interleaved=False):
    """positions3 [3, T] int32 + mrope_section (rotary pairs per component: temporal, height, width): multimodal RoPE, the
    pairs of each section rotate by their own position component.  mrope_interleaved: the components alternate pair by pair
    (t h w t h w ... while a component has pairs left) instead of occupying three contiguous ranges."""
    _check_index("rope_kv_append", "slots", None if slots is None else slots[:qkv.shape[0]], k_cache.shape[0] if k_cache is not None else 0, -1)
    if cos_cache is not None:
        _check_index("rope_kv_append", "positions", positions[:qkv.shape[0]] if positions3 is None else positions3, cos_cache.shape[0])
    if not qkv.is_cuda:
        return ref.rope_kv_append(qkv, positions, slots, cos_cache, sin_cache, k_cache, v_cache, Hq, Hkv, D, rot, interleaved,
                                  q_norm_w, k_norm_w, norm_eps, positions3, mrope_section, mrope_interleaved)
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1
    assert cos_cache is None or cos_cache.dtype == torch.float32
    T = qkv.shape[0]
    max_pos = cos_cache.shape[0] if cos_cache is not None else 1
    kv_bits = 8 if k_cache.dtype == torch.int8 else 16      # an int8 cache has rows of D values + inline scale (D + 16 bytes)
    rc = _lib.lib().ogb_rope_kv_append_bits(_ptr(qkv), qkv.stride(0), _ptr(positions), _ptr(slots), _ptr(cos_cache), _ptr(sin_cache),
                                            _ptr(k_cache), _ptr(v_cache), _ptr(q_norm_w), _ptr(k_norm_w), float(norm_eps), T, Hq, Hkv,
                                            D, int(rot if cos_cache is not None else 0), int(interleaved), max_pos, kv_bits,
                                            _ptr(positions3.contiguous()) if positions3 is not None else None,
                                            (0 if positions3 is None else -3 * int(mrope_section[1]) if mrope_interleaved else int(mrope_section[0])),
                                            (0 if positions3 is None else 3 * int(mrope_section[2]) if mrope_interleaved
                                             else int(mrope_section[0] + mrope_section[1])), _stream())
    _lib.check(rc, "rope_kv_append")
    return qkv


# ------------------------------------------------------------------------------------------ attention
def choose_kv_splits(batch: int, Hkv: int, max_q_len: int, max_kv_len: int, sm_count: int = 148, group: int = 1, ordered: bool = False):
    """(splits, kv_chunk) of a paged-attention launch.  A launch whose (request, kv head) grid already fills the GPU
    twice over is not split (measured on B200: at 64 requests x 8 heads any split costs more in partial traffic and
    the merge than it gains in balance).  Smaller decode-sized launches split every request's keys into fixed chunks
    of 64..512 keys sized for about four CTAs per SM; other launches: (1, 0).

    ordered: the caller issues the requests longest first.  Then every request is divided evenly into as many parts as
    bring the launch to about 1.75 waves of CTAs - measured on B200 with 64 requests of 192..2112 keys and 4 / 2 / 1 kv
    heads per GPU (the tensor-parallel shapes): 2 parts 35.3 us against 43.1 us for fixed chunks, 4 parts 25.1 against
    29.4, 4 parts 18.7 against 22.0."""
    ctas = max(1, batch * Hkv)
    if ordered and ctas >= 32 and max_q_len * group <= 16 and max_kv_len > 128:
        s = int(round(1.75 * 2 * sm_count / ctas))
        s = max(1, min(4, s, max_kv_len // 256))     # more than 4 parts: the pieces get too short (1 kv head: 8 parts 20.5 us, 16 parts 27.7)
        return s, 0
    if max_q_len * group > 16 or max_kv_len <= 128 or ctas >= 2 * sm_count:
        return 1, 0
    chunks_wanted = max(1, (4 * sm_count + ctas - 1) // ctas)
    chunk = (max_kv_len + chunks_wanted - 1) // chunks_wanted
    chunk = min(512, max(64, (chunk + 63) // 64 * 64))
    splits = min(64, (max_kv_len + chunk - 1) // chunk)
    if splits <= 1:
        return 1, 0
    chunk = ((max_kv_len + splits - 1) // splits + 63) // 64 * 64   # the splits must cover the bound
    return int(splits), int(chunk)


TC_ATTENTION_MIN_ROWS = 128      # query rows (tokens x heads of a GQA group) from which a request takes the tcgen05 prefill kernel
_TC_ATTENTION = os.environ.get("OGB_ATTN_TC", "1") != "0"


def paged_attention(q, k_cache, v_cache, cu_seqlens, past_lens, block_table, block_size, Hq, Hkv, D, scale, window=0,
                    sinks=None, softcap=0.0, max_q_len=None, max_kv_len=None, splits=None, out=None, total_tokens=None, order=None,
                    min_q_len=None):
    """q: [T, stride] with the Hq*D query columns first.  Returns [T, Hq*D].  total_tokens: the requests of this call only cover
    the first `total_tokens` rows of q (sizes the split-KV scratch).  min_q_len: shortest request of the call when the caller
    knows it (a call whose every request is long runs on the tensor-core prefill kernel alone)."""
    _check_index("paged_attention", "block_table", block_table, k_cache.shape[0] // block_size, -1)
    _check_index("paged_attention", "cu_seqlens", cu_seqlens[:past_lens.shape[0] + 1], q.shape[0] + 1)
    if not q.is_cuda:
        return ref.paged_attention(q, k_cache, v_cache, cu_seqlens, past_lens, block_table, block_size, Hq, Hkv, D, scale,
                                   window, sinks, softcap)
    T = q.shape[0] if total_tokens is None else total_tokens
    B = past_lens.shape[0]
    if out is None:
        out = torch.empty(q.shape[0], Hq * D, dtype=q.dtype, device=q.device)
    if max_q_len is None:
        max_q_len = T
    G = Hq // Hkv
    ws = workspace(q.device)
    use_tc = (_TC_ATTENTION and max_q_len * G >= TC_ATTENTION_MIN_ROWS and k_cache.dtype == torch.bfloat16 and q.dtype == torch.bfloat16
              and out.stride(0) % 8 == 0 and _lib.lib().ogb_attention_tc_supported(D, block_size, 16, int(k_cache.shape[0])))
    if use_tc:
        all_long = min_q_len is not None and min_q_len * G >= TC_ATTENTION_MIN_ROWS
        if not all_long:
            # the short requests first (its split-KV combine pass may scribble on the rows of the long ones)
            paged_attention_small = _lib.lib().ogb_paged_attention_skip
            sp, ch = splits if isinstance(splits, tuple) else ((splits, 0) if splits else choose_kv_splits(
                B, Hkv, max_q_len, max_kv_len or 1024, group=G, ordered=order is not None))
            need = _lib.lib().ogb_attention_scratch_bytes(T, Hq, D, sp)
            scratch = ws.attn_scratch(need) if sp > 1 else None
            _lib.check(paged_attention_small(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(cu_seqlens), _ptr(past_lens),
                                             _ptr(block_table), block_table.stride(0), block_size, _ptr(out), out.stride(0), _ptr(sinks),
                                             float(scale), float(softcap), int(window), B, T, int(max_q_len), Hq, Hkv, D, int(sp), int(ch),
                                             _ptr(scratch), scratch.numel() if scratch is not None else 0, int(k_cache.shape[0]),
                                             _ptr(order), ws.status, _stream(), TC_ATTENTION_MIN_ROWS), "paged_attention")
            if sp > 1:
                _lib.LAUNCH_COUNT += 1
        _lib.check(_lib.lib().ogb_attention_tc(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(cu_seqlens), _ptr(past_lens),
                                               _ptr(block_table), block_table.stride(0), block_size, _ptr(out), out.stride(0), _ptr(sinks),
                                               float(scale), float(softcap), int(window), B, int(max_q_len), Hq, Hkv, D,
                                               TC_ATTENTION_MIN_ROWS, int(k_cache.shape[0]), ws.status, _stream()), "attention_tc")
        return out
    kv_chunk = 0
    if splits is None:
        splits, kv_chunk = choose_kv_splits(B, Hkv, max_q_len, max_kv_len or 1024, group=Hq // Hkv, ordered=order is not None)
    elif isinstance(splits, tuple):
        splits, kv_chunk = splits
    need = _lib.lib().ogb_attention_scratch_bytes(T, Hq, D, splits)
    scratch = ws.attn_scratch(need) if splits > 1 else None
    fn = _lib.lib().ogb_paged_attention_kv8 if k_cache.dtype == torch.int8 else _lib.lib().ogb_paged_attention
    rc = fn(_ptr(q), q.stride(0), _ptr(k_cache), _ptr(v_cache), _ptr(cu_seqlens), _ptr(past_lens),
                                        _ptr(block_table), block_table.stride(0), block_size, _ptr(out), out.stride(0),
                                        _ptr(sinks), float(scale), float(softcap), int(window), B, T, int(max_q_len),
                                        Hq, Hkv, D, int(splits), int(kv_chunk), _ptr(scratch),
                                        scratch.numel() if scratch is not None else 0, int(k_cache.shape[0]), _ptr(order), ws.status, _stream())
    _lib.check(rc, "paged_attention")
    if splits > 1:
        _lib.LAUNCH_COUNT += 1  # the combine kernel
    return out


# ------------------------------------------------------------------------------------------ logits processing
def logits_bitmask(logits, mask_words, mask_rows=None):
    if not logits.is_cuda:
        return ref.logits_bitmask(logits, mask_words, mask_rows)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and mask_words.dtype == torch.int32
    _lib.check(_lib.lib().ogb_logits_bitmask(_ptr(logits), rows, V, _ptr(mask_words), _ptr(mask_rows), _stream()), "logits_bitmask")
    return logits


def logits_edit(logits, rows, tokens, ops, values):
    _check_index("logits_edit", "rows", rows, logits.shape[0])
    _check_index("logits_edit", "tokens", tokens, logits.shape[1])
    if not logits.is_cuda:
        return ref.logits_edit(logits, rows, tokens, ops, values)
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    _lib.check(_lib.lib().ogb_logits_edit(_ptr(logits), logits.shape[1], _ptr(rows), _ptr(tokens), _ptr(ops), _ptr(values),
                                          rows.numel(), _stream()), "logits_edit")
    return logits


def to_float32(x):
    if x.dtype == torch.float32:
        return x
    if not x.is_cuda:
        return x.float()
    out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().ogb_bf16_to_f32(_ptr(x.contiguous()), _ptr(out), x.numel(), _stream()), "bf16_to_f32")
    return out


def gather_rows(x, rows, f16: bool = False):
    """out[i] = x[rows[i]]; f16: bf16 rows come out as fp16 (input of the fp16 form of the packed FP4 expert GEMM)."""
    _check_index("gather_rows", "rows", rows, x.shape[0])
    if not x.is_cuda:
        return x[rows.long()].to(torch.float16) if f16 else x[rows.long()]
    out = torch.empty(rows.numel(), x.shape[1], dtype=torch.float16 if f16 else x.dtype, device=x.device)
    if f16:
        assert x.dtype == torch.bfloat16
        _lib.check(_lib.lib().ogb_gather_rows_f16(_ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1] * 2, _stream()), "gather_rows_f16")
        return out
    _lib.check(_lib.lib().ogb_gather_rows(_ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[1] * x.element_size(), _stream()),
               "gather_rows")
    return out


# ------------------------------------------------------------------------------------------ sampling
def _cpu_sample_row(row, k, p, t, seed, pos):
    if k == 1 or t <= 0:
        return int(torch.argmax(row))
    ids, probs = ref.sampled_distribution(row, k if k > 1 else None, p if 0 < p < 1 else None, t)
    rng = np.random.Generator(np.random.Philox(key=int(seed) & ((1 << 64) - 1), counter=[int(pos), 0x5A17, 0, 0]))
    u = rng.random()
    cum = torch.cumsum(probs, 0)
    j = int(torch.searchsorted(cum, torch.tensor(u, dtype=cum.dtype)).clamp(max=len(ids) - 1))
    return int(ids[j])


def sample(logits, top_k, top_p, temperature, seeds, positions, out=None):
    """Per-row sampling.  logits [B, V] fp32; top_k int32 [B] (1 = greedy, <= 0 = no top-k);
    top_p / temperature fp32 [B]; seeds int64 [B]; positions int32 [B] (RNG counter)."""
    B, V = logits.shape
    if not logits.is_cuda:
        res = [_cpu_sample_row(logits[i].float(), int(top_k[i]), float(top_p[i]), float(temperature[i]), int(seeds[i]),
                               int(positions[i])) for i in range(B)]
        return torch.tensor(res, dtype=torch.int32)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().ogb_sample(_ptr(logits), logits.stride(0), B, V, _ptr(top_k), _ptr(top_p), _ptr(temperature),
                                     _ptr(seeds), _ptr(positions), _ptr(out), _stream()), "sample")
    return out


def argmax(logits, out=None):
    if not logits.is_cuda:
        return torch.argmax(logits.float(), dim=-1).to(torch.int32)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().ogb_argmax(_ptr(logits), logits.stride(0), B, V, _ptr(out), _stream()), "argmax")
    return out


def topk(x, k, log_softmax=False, add=None):
    """Sorted top-k per row (k <= 128).  With log_softmax the values are log-probabilities (+ add[row])."""
    if not x.is_cuda:
        return ref.topk(x, k, log_softmax, add)
    assert x.dtype == torch.float32 and x.stride(1) == 1 and k <= 128
    R, n = x.shape
    vals = torch.empty(R, k, dtype=torch.float32, device=x.device)
    idx = torch.empty(R, k, dtype=torch.int32, device=x.device)
    _lib.check(_lib.lib().ogb_topk(_ptr(x), x.stride(0), R, n, k, int(log_softmax), _ptr(add), _ptr(vals), _ptr(idx), _stream()), "topk")
    return vals, idx


def beam_candidates(logits, beam_scores, batch, beams):
    """Beam-search scoring: log-softmax + running beam score, top 2*beams per beam, merged to the best
    2*beams per batch entry.  Returns (scores, tokens, source_beams), each [batch, 2*beams]."""
    cand = 2 * beams
    vals, idx = topk(logits, cand, log_softmax=True, add=beam_scores)
    if not logits.is_cuda:
        v = vals.view(batch, beams * cand)
        order = torch.sort(v, dim=-1, descending=True, stable=True).indices[:, :cand]
        scores = torch.gather(v, 1, order)
        tokens = torch.gather(idx.view(batch, beams * cand), 1, order)
        return scores, tokens.to(torch.int32), (order // cand).to(torch.int32)
    scores = torch.empty(batch, cand, dtype=torch.float32, device=logits.device)
    tokens = torch.empty(batch, cand, dtype=torch.int32, device=logits.device)
    src = torch.empty(batch, cand, dtype=torch.int32, device=logits.device)
    _lib.check(_lib.lib().ogb_beam_merge(_ptr(vals), _ptr(idx), batch, beams, cand, _ptr(scores), _ptr(tokens), _ptr(src), _stream()),
               "beam_merge")
    return scores, tokens, src


_verify_scratch = {}


def verify_sampled(logits, draft, q_dists, top_k: int, top_p: float, temperature: float, seed: int, first_position: int):
    """Sampled speculative verification on the device.  logits [K+1, V] fp32 (target rows for the K draft
    positions and the bonus position); draft: K token ids; q_dists: per draft position None (deterministic
    proposal) or (ids, probs) of the draft model's sampled distribution.  Row i draws with the random stream of
    (seed, first_position + i).  Returns (accepted, commit list, accept probabilities [K])."""
    K = len(draft)
    dev = logits.device
    assert logits.is_cuda and logits.dtype == torch.float32 and logits.shape[0] == K + 1 and 1 < top_k <= 1024
    R = K + 1
    ki = torch.full((R,), int(top_k), dtype=torch.int32, device=dev)
    pp = torch.full((R,), float(top_p), dtype=torch.float32, device=dev)
    tt = torch.full((R,), float(temperature), dtype=torch.float32, device=dev)
    seeds = torch.full((R,), int(seed) & ((1 << 63) - 1), dtype=torch.int64, device=dev)
    pos = torch.arange(first_position, first_position + R, dtype=torch.int32, device=dev)
    d = torch.tensor(list(draft) or [0], dtype=torch.int32, device=dev)
    qs = max([len(q[0]) for q in q_dists if q is not None] + [1])
    qi = np.zeros((max(K, 1), qs), dtype=np.int32)
    qp = np.zeros((max(K, 1), qs), dtype=np.float32)
    qn = np.zeros((max(K, 1),), dtype=np.int32)
    for i, q in enumerate(q_dists):
        if q is not None:
            m = len(q[0])
            qi[i, :m], qp[i, :m], qn[i] = q[0], q[1], m
    qi_d, qp_d, qn_d = torch.from_numpy(qi).to(dev), torch.from_numpy(qp).to(dev), torch.from_numpy(qn).to(dev)
    key = (dev.index, K)
    if key not in _verify_scratch:
        _verify_scratch[key] = torch.zeros(2 * R + 1, dtype=torch.int32, device=dev)
    scratch = _verify_scratch[key]
    out = torch.zeros(R + 2, dtype=torch.int32, device=dev)     # [accepted, status, commit...]
    aprob = torch.zeros(max(K, 1), dtype=torch.float32, device=dev)
    rc = _lib.lib().ogb_verify_sampled(_ptr(logits), logits.stride(0), logits.shape[1], K, _ptr(ki), _ptr(pp), _ptr(tt), _ptr(seeds), _ptr(pos),
                                       _ptr(d), _ptr(qi_d), _ptr(qp_d), _ptr(qn_d), qs, _ptr(scratch), _ptr(aprob), _ptr(out[0:1]),
                                       _ptr(out[2:]), _ptr(out[1:2]), _stream())
    _lib.check(rc, "verify_sampled")
    res = out.tolist()
    if res[1] != 0:
        raise RuntimeError("verify_sampled: sampling parameters outside the device path (needs 1 < top_k <= 1024, temperature > 0)")
    accepted = res[0]
    return accepted, res[2:2 + accepted + 1], aprob[:K].tolist()
