"""Mixture-of-experts MLP: router -> top-k -> routing weights -> per-expert gated MLP -> weighted sum.
Two styles: gpt-oss (biases, softmax over the selected logits, clamped SwiGLU(alpha, limit)) and standard (Mixtral, Qwen-MoE,
PhiMoE, GraniteMoE: no biases, silu(gate) * up, softmax over all experts with or without renormalisation).

Semantics follow the MoE / QMoE contrib op the reference's builder emits
(src/python/py/models/builders/base.py:4176-4408, builders/gptoss.py:653-847): `k` experts per token,
`normalize_routing_weights` (softmax over the k selected router logits), `swiglu_fusion = 1`
(gate and up interleaved along the output dimension: even = gate, odd = up), activation
gate * sigmoid(alpha * gate) * (up + 1) with gate clamped to <= limit and up to [-limit, limit].

CUDA path (everything on the device, no counts read back, so it replays inside a CUDA graph):
router GEMM (fp32 out) -> `moe_topk` -> `moe_sort` (rows grouped by expert + tile list) -> row gather ->
grouped tcgen05 GEMM gate/up with the clamped SwiGLU in its epilogue -> grouped GEMM down -> `moe_combine`.

Expert parallelism: attention is tensor parallel, so after its all-reduce every rank already holds every
token; a rank therefore needs no dispatch — it routes all tokens, runs only the experts it owns
(`lw.exp_lo .. lw.exp_hi`), and the partial outputs are summed by the same all-reduce a dense row-parallel
MLP uses.  The combine of the all-to-all formulation is that all-reduce.
"""
from __future__ import annotations

import os

import torch

from .. import ops


# OGB_MOE_ROW_MAP=0: the token rows of packed experts are gathered into a copy instead of being read through the row map
_ROW_MAP = os.environ.get("OGB_MOE_ROW_MAP", "1") != "0"


def swiglu_interleaved(gu: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    g, u = gu[..., 0::2].float(), gu[..., 1::2].float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


def route(model, lw, x):
    """Routing weights and expert ids [T, k].  Softmax over the selected logits equals softmax over all experts renormalised
    over the selected; the standard style without renormalisation keeps the probabilities of the full softmax."""
    a = model.arch
    logits = ops.linear(x, lw.router_w, lw.router_b).float()
    if a.moe_sparse_mixer:
        return sparse_mixer(logits, a.moe_jitter_eps)
    top_v, top_i = torch.topk(logits, a.experts_per_token, dim=-1)
    if a.moe_style == "standard" and not a.moe_norm_topk:
        return torch.softmax(logits, dim=-1).gather(-1, top_i), top_i
    return torch.softmax(top_v, dim=-1), top_i


def sparse_mixer(logits: torch.Tensor, eps: float):
    """PhiMoE's inference-time routing (reference: the MoE contrib op's use_sparse_mixer attribute,
    src/python/py/models/builders/phi.py:542-547): the best expert, then the best of the rest; each weight is that
    expert's probability in a softmax over the logits that lie within a relative margin of 2 * eps below the current
    maximum.  Pure tensor ops (no host synchronisation), so the step still captures into a CUDA graph."""
    s = logits.float()
    neg = torch.finfo(torch.float32).min

    def pick(scores):
        top, idx = scores.max(dim=-1, keepdim=True)
        factor = s.abs().clamp(min=top)
        keep = ((top - s) / factor) <= 2.0 * eps
        gates = torch.softmax(torch.where(keep, scores, torch.full_like(scores, neg)), dim=-1)
        return gates.gather(-1, idx), idx

    w1, i1 = pick(s)
    w2, i2 = pick(s.scatter(-1, i1, neg))
    return torch.cat([w1, w2], dim=-1), torch.cat([i1, i2], dim=-1)


def silu_mul_interleaved(gu: torch.Tensor) -> torch.Tensor:
    g, u = gu[..., 0::2].float(), gu[..., 1::2].float()
    return (torch.nn.functional.silu(g) * u).to(gu.dtype)


def _unblock(t: torch.Tensor) -> torch.Tensor:
    """[.., 2I, ..] in blocks of 64 gate + 64 up rows -> even/odd interleaved rows."""
    two_i = t.shape[0]
    v = t.reshape(two_i // 128, 2, 64, *t.shape[1:])
    return torch.stack([v[:, 0], v[:, 1]], dim=2).reshape(t.shape)


def expert_mlp(model, lw, e: int, xs: torch.Tensor) -> torch.Tensor:
    """One expert (index into this rank's slice) over its rows: the unfused path (CPU, odd shapes)."""
    a = model.arch
    packed = isinstance(lw.exp_gate_up_w, ops.Fp4Experts)   # MXFP4 experts: expand this one expert
    w = lw.exp_gate_up_w.dequantize(e).to(xs) if packed else lw.exp_gate_up_w[e]
    b = lw.exp_gate_up_b[e] if lw.exp_gate_up_b is not None else None
    if lw.exp_blocked:
        w, b = _unblock(w).contiguous(), _unblock(b).contiguous() if b is not None else None
    gu = ops.linear(xs, w, b)
    act = silu_mul_interleaved(gu) if a.moe_style == "standard" else swiglu_interleaved(gu, a.moe_swiglu_alpha, a.moe_swiglu_limit)
    wd = lw.exp_down_w.dequantize(e).to(xs) if packed else lw.exp_down_w[e]
    return ops.linear(act.contiguous(), wd, lw.exp_down_b[e] if lw.exp_down_b is not None else None)


def _forward_loop(model, lw, x):
    a = model.arch
    lo, hi = lw.exp_lo, lw.exp_hi or a.num_experts
    weights, experts = route(model, lw, x)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    counts = torch.bincount(flat_e, minlength=a.num_experts).tolist()
    tok = order // a.experts_per_token
    w_sorted = weights.reshape(-1)[order]
    start = 0
    for e, n in enumerate(counts):
        if n and lo <= e < hi:
            idx = tok[start:start + n]
            y = expert_mlp(model, lw, e - lo, x[idx].contiguous()).float()
            out.index_add_(0, idx, y * w_sorted[start:start + n, None])
        start += n
    return out.to(x.dtype)


def _forward_device(model, lw, x, defer=False):
    a = model.arch
    lo, hi = lw.exp_lo, lw.exp_hi or a.num_experts
    standard = a.moe_style == "standard"
    mode = 1 if standard and not a.moe_norm_topk else 0
    logits = ops.linear(x, lw.router_w, lw.router_b, out_fp32=True)
    if a.moe_sparse_mixer:
        tw, ti = sparse_mixer(logits, a.moe_jitter_eps)
        plan = ops.moe_route(logits, 2, 0, (lo, hi), topk=(ti.to(torch.int32).contiguous(), tw.contiguous()))
    else:
        plan = ops.moe_route(logits, a.experts_per_token, mode, (lo, hi))
    half = isinstance(lw.exp_gate_up_w, ops.Fp4Experts) and lw.exp_gate_up_w.half and lw.exp_down_w.half
    if half:
        # packed MXFP4 experts in their fp16 form: fp16 rows in, fp16 between the two grouped GEMMs, bf16 out; the streaming
        # kernel of decode-sized steps reads the token rows through the plan's row map instead of a gathered copy
        mapped = _ROW_MAP and ops.moe_fp4_reads_rows(lw.exp_gate_up_w, plan) and x.dtype == torch.bfloat16 and x.stride(0) % 8 == 0
        xs = x if mapped else ops.gather_rows(x, plan.sorted_token, f16=True)
        h = ops.moe_gemm(xs, lw.exp_gate_up_w, plan, lw.exp_gate_up_b, act_kind=2, alpha=a.moe_swiglu_alpha, limit=a.moe_swiglu_limit,
                         out_dtype=torch.float16, row_map=mapped)
        y = ops.moe_gemm(h, lw.exp_down_w, plan, lw.exp_down_b)
        return ops.PendingCombine(y, plan) if defer else ops.moe_combine(y, plan)
    xs = ops.gather_rows(x, plan.sorted_token)
    if standard:
        h = ops.moe_gemm(xs, lw.exp_gate_up_w, plan, None, act_kind=1)
    else:
        h = ops.moe_gemm(xs, lw.exp_gate_up_w, plan, lw.exp_gate_up_b, act_kind=2, alpha=a.moe_swiglu_alpha, limit=a.moe_swiglu_limit)
    y = ops.moe_gemm(h, lw.exp_down_w, plan, lw.exp_down_b)
    return ops.PendingCombine(y, plan) if defer else ops.moe_combine(y, plan)


def moe_forward(model, lw, x: torch.Tensor, defer: bool = False):
    """defer: the caller folds the combine step into the residual add + norm that follows (`ops.norm_moe_combine`); the
    result is then an `ops.PendingCombine` when the layer ran on the device path of a single rank."""
    a = model.arch
    fast = x.is_cuda and lw.exp_blocked and a.hidden_size % 8 == 0 and a.num_experts <= 1024 and a.experts_per_token <= 32
    if model.tp.size > 1 and getattr(model.tp, "ep_mode", "replicated") == "all_to_all":
        # token-sharded expert parallelism: dispatch / combine all-to-all, the output is complete on every rank
        from ..parallel.ep import moe_all_to_all
        return moe_all_to_all(model, lw, x)
    if fast:
        return _forward_device(model, lw, x, defer and model.tp.size == 1) if model.tp.size == 1 else model.tp.reduce(_forward_device(model, lw, x))
    out = _forward_loop(model, lw, x)
    return model.tp.reduce(out) if model.tp.size > 1 else out
