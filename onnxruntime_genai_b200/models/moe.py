"""Mixture-of-experts MLP (gpt-oss style): router -> top-k -> softmax over the selected logits ->
per-expert SwiGLU(alpha, limit) MLP -> weighted sum.

Semantics follow the MoE / QMoE contrib op the reference's builder emits
(src/python/py/models/builders/base.py:4176-4408, builders/gptoss.py:653-847): `k` experts per token,
`normalize_routing_weights` (softmax over the k selected router logits), `swiglu_fusion = 1`
(gate and up interleaved along the output dimension: even = gate, odd = up), activation
gate * sigmoid(alpha * gate) * (up + 1) with gate clamped to <= limit and up to [-limit, limit].

Expert matmuls run on the tcgen05 GEMM, one launch per (active expert, projection) over the tokens
routed to that expert; routing and the activation are elementwise glue.  With expert parallelism
(parallel/ep.py) each rank owns a contiguous slice of the experts and the token exchange is an
all-to-all.
"""
from __future__ import annotations

import torch

from .. import ops


def swiglu_interleaved(gu: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    g, u = gu[..., 0::2].float(), gu[..., 1::2].float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


def route(model, lw, x):
    a = model.arch
    logits = ops.linear(x, lw.router_w, lw.router_b).float()
    top_v, top_i = torch.topk(logits, a.experts_per_token, dim=-1)
    return torch.softmax(top_v, dim=-1), top_i


def expert_mlp(model, lw, e: int, xs: torch.Tensor) -> torch.Tensor:
    a = model.arch
    gu = ops.linear(xs, lw.exp_gate_up_w[e], lw.exp_gate_up_b[e] if lw.exp_gate_up_b is not None else None)
    act = swiglu_interleaved(gu, a.moe_swiglu_alpha, a.moe_swiglu_limit)
    return ops.linear(act.contiguous(), lw.exp_down_w[e], lw.exp_down_b[e] if lw.exp_down_b is not None else None)


def moe_forward(model, lw, x: torch.Tensor) -> torch.Tensor:
    ep = getattr(model, "ep", None)
    if ep is not None and ep.size > 1:
        return ep.moe_forward(model, lw, x)
    weights, experts = route(model, lw, x)
    out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
    flat_e = experts.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    counts = torch.bincount(flat_e, minlength=model.arch.num_experts).tolist()
    tok = (order // model.arch.experts_per_token)
    w_sorted = weights.reshape(-1)[order]
    start = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        idx = tok[start:start + n]
        y = expert_mlp(model, lw, e, x[idx].contiguous()).float()
        out.index_add_(0, idx, y * w_sorted[start:start + n, None])
        start += n
    return out.to(x.dtype)
