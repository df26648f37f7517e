"""Expert parallelism in its all-to-all form: tokens are sharded over the ranks, every rank routes its own tokens, sends each
(token, expert) row to the rank that owns the expert, runs its experts over what it received, and sends the results back.

    rank r:  x_r [T_r, H] -> router -> top-k experts and weights per token
             dispatch:  rows sorted by owner rank; `all_to_all_single` of the row counts, of the rows and of their expert ids
             compute:   the received rows grouped by local expert -> gate/up GEMM + activation -> down GEMM (the grouped
                        expert GEMMs on the GPU, one expert at a time on the CPU)
             combine:   `all_to_all_single` back with the splits reversed; out_r[t] = sum_j w[t, j] * y[row(t, j)]

This is the collective-library form of the exchange (NCCL on GPUs, gloo on the CPU): the routing / ownership arithmetic, the
row order both ways and the equivalence with the replicated form are what it pins down.  The default layout of this
framework does not need it - attention is tensor parallel, so every rank already holds every token after the attention
all-reduce, runs its experts over the replicated tokens and the partial outputs are summed by the all-reduce that a dense
row-parallel MLP uses too (`models/moe.py`).  `OGB_EP_MODE=all_to_all` (or `TensorParallel.ep_mode`) switches a MoE layer to
this form: the replicated tokens are split by rows, exchanged, and the per-rank outputs are all-gathered; the all-reduce of
the layer is skipped.  No reference counterpart: the reference runs MoE as one fused operator on one GPU
(src/python/py/models/builders/base.py:4176-4217).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from .. import ops


def owner_of(expert: torch.Tensor, experts_per_rank: int) -> torch.Tensor:
    return torch.div(expert, experts_per_rank, rounding_mode="floor")


def token_slice(T: int, rank: int, world: int) -> Tuple[int, int]:
    """Rows [lo, hi) of the replicated token matrix that `rank` routes (the first T % world ranks take one row more)."""
    base, extra = divmod(T, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _route(model, lw, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(expert ids [T, k] int64, weights [T, k] fp32) of this rank's tokens: the selection rule of `models/moe.py::route`."""
    from ..models.moe import route
    w, idx = route(model, lw, x)
    return idx.long(), w.float()


def _local_experts(model, lw, rows: torch.Tensor, local_expert: torch.Tensor) -> torch.Tensor:
    """rows [n, H] with the local expert index of every row -> expert outputs [n, H] in the same row order."""
    from ..models.moe import expert_mlp
    a = model.arch
    n_local = (lw.exp_hi or a.num_experts) - lw.exp_lo
    out = torch.empty(rows.shape[0], a.hidden_size, dtype=rows.dtype, device=rows.device)
    if rows.shape[0] == 0:
        return out
    if rows.is_cuda and lw.exp_blocked and not isinstance(lw.exp_gate_up_w, ops.Fp4Experts):
        # every received row is a "token" with one expert: the device-side grouping and the grouped GEMMs do the rest
        idx = local_expert.to(torch.int32).reshape(-1, 1).contiguous()
        ones = torch.ones(rows.shape[0], 1, dtype=torch.float32, device=rows.device)
        dummy = torch.zeros(rows.shape[0], n_local, dtype=torch.float32, device=rows.device)
        plan = ops.moe_route(dummy, 1, 0, (0, n_local), topk=(idx, ones))
        xs = ops.gather_rows(rows.contiguous(), plan.sorted_token)
        if a.moe_style == "standard":
            h = ops.moe_gemm(xs, lw.exp_gate_up_w, plan, None, act_kind=1)
        else:
            h = ops.moe_gemm(xs, lw.exp_gate_up_w, plan, lw.exp_gate_up_b, act_kind=2, alpha=a.moe_swiglu_alpha, limit=a.moe_swiglu_limit)
        y = ops.moe_gemm(h, lw.exp_down_w, plan, lw.exp_down_b)
        return ops.moe_combine(y, plan)
    for e in range(n_local):
        sel = (local_expert == e).nonzero().flatten()
        if sel.numel():
            out[sel] = expert_mlp(model, lw, e, rows[sel].contiguous()).to(out.dtype)
    return out


def moe_all_to_all(model, lw, x: torch.Tensor) -> torch.Tensor:
    """x [T, H]: the replicated tokens of the step.  Returns the layer's full output [T, H] on every rank (already complete:
    no all-reduce follows)."""
    tp = model.tp
    world, rank, group = tp.size, tp.rank, tp.group
    a = model.arch
    per_rank = a.num_experts // world
    T = x.shape[0]
    lo, hi = token_slice(T, rank, world)
    mine = x[lo:hi].contiguous()
    k = a.experts_per_token if not a.moe_sparse_mixer else 2
    if mine.shape[0]:
        idx, w = _route(model, lw, mine)
    else:
        idx = torch.zeros(0, k, dtype=torch.int64, device=x.device)
        w = torch.zeros(0, k, dtype=torch.float32, device=x.device)
    # ---- dispatch: assignments in (owner rank, token, j) order
    flat_e = idx.reshape(-1)
    dest = owner_of(flat_e, per_rank)
    order = torch.argsort(dest, stable=True)
    send_rows = mine[torch.div(order, idx.shape[1], rounding_mode="floor")].contiguous() if order.numel() else mine[:0]
    send_exp = (flat_e[order] - dest[order] * per_rank).to(torch.int32).contiguous()
    send_counts = torch.bincount(dest, minlength=world).to(torch.int64)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    s_list, r_list = send_counts.tolist(), recv_counts.tolist()
    n_recv = int(sum(r_list))
    recv_rows = torch.empty(n_recv, x.shape[1], dtype=x.dtype, device=x.device)
    recv_exp = torch.empty(n_recv, dtype=torch.int32, device=x.device)
    dist.all_to_all_single(recv_rows, send_rows, r_list, s_list, group=group)
    dist.all_to_all_single(recv_exp, send_exp, r_list, s_list, group=group)
    # ---- this rank's experts over the rows it received
    y = _local_experts(model, lw, recv_rows, recv_exp.long()).contiguous()
    # ---- combine: the results travel back along the same splits, then the weighted sum per token in j order
    back = torch.empty(send_rows.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
    dist.all_to_all_single(back, y, s_list, r_list, group=group)
    out_mine = torch.zeros(mine.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    if order.numel():
        unsorted = torch.empty_like(back)
        unsorted[order] = back                                    # row (t, j) at position t * k + j
        out_mine = (unsorted.float().view(mine.shape[0], idx.shape[1], -1) * w[..., None]).sum(1)
    # ---- every rank needs every token again for the next (tensor-parallel) layer
    sizes = [token_slice(T, r, world) for r in range(world)]
    widest = max(h - l for l, h in sizes)
    padded = torch.zeros(widest, x.shape[1], dtype=x.dtype, device=x.device)
    padded[:out_mine.shape[0]] = out_mine.to(x.dtype)
    parts: List[torch.Tensor] = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:h - l] for p, (l, h) in zip(parts, sizes)], dim=0)
