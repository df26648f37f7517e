"""Plain PyTorch fp32 restatements of every device op.

They serve two purposes: (1) the CPU execution path (tiny models, CI without a GPU) and (2) the
numerical oracle that the GPU tests compare each sm_100a kernel against.  All math is done in fp32
regardless of the storage dtype; results are cast back to the input dtype.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def embedding(ids, table, scale=1.0):
    out = table[ids.long().clamp(0, table.shape[0] - 1)]
    if scale != 1.0:
        out = (out.float() * scale).to(table.dtype)
    return out


def norm(x, weight, eps, residual=None, bias=None, layernorm=False):
    h = x.float()
    new_res = None
    if residual is not None:
        new_res = (h + residual.float()).to(x.dtype)
        h = new_res.float()
    if layernorm:
        mean = h.mean(-1, keepdim=True)
        var = ((h - mean) ** 2).mean(-1, keepdim=True)
        y = (h - mean) * torch.rsqrt(var + eps)
    else:
        y = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps)
    y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype), new_res


def rms_scale(x, eps):
    """x / rms(x) without a weight, in x's dtype: what a norm folded into the next GEMM applies to the rows."""
    h = x.float()
    return (h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps)).to(x.dtype)


def linear(x, w, bias=None, residual=None, out_fp32=False, norm_eps=0.0):
    if norm_eps > 0:
        x = rms_scale(x, norm_eps)
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    if residual is not None:
        y = y + residual.float()
    return y if out_fp32 else y.to(x.dtype)


def gate_up_act(x, w, bias=None, act="silu", interleaved=False, norm_eps=0.0):
    """w is the stacked [gate; up] weight of shape [2I, K] (or 64-row interleaved blocks)."""
    if norm_eps > 0:
        x = rms_scale(x, norm_eps)
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    inter = y.shape[-1] // 2
    if interleaved:
        y = y.view(-1, inter // 64, 2, 64).transpose(1, 2).reshape(-1, 2 * inter)
    g, u = y[..., :inter], y[..., inter:]
    a = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    return (a * u).to(x.dtype)


def act_mul(x, act="silu"):
    inter = x.shape[-1] // 2
    g, u = x[..., :inter].float(), x[..., inter:].float()
    a = torch.nn.functional.silu(g) if act == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
    return (a * u).to(x.dtype)


def activation(x, act="gelu"):
    f = x.float()
    if act == "silu":
        y = torch.nn.functional.silu(f)
    elif act == "relu":
        y = torch.relu(f)
    elif act == "relu2":
        y = torch.relu(f) ** 2
    elif act == "gelu_erf":
        y = torch.nn.functional.gelu(f)
    else:
        y = torch.nn.functional.gelu(f, approximate="tanh")
    return y.to(x.dtype)


def full_width_qk_norm(qkv, q_size, kv_size, q_norm_w, k_norm_w, norm_eps):
    """Families that normalise q and k over all their heads at once (olmoe): returns qkv with those two parts normalised."""
    x = qkv.float().clone()
    for a, b, w in ((0, q_size, q_norm_w), (q_size, q_size + kv_size, k_norm_w)):
        t = x[:, a:b]
        x[:, a:b] = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()
    return x.to(qkv.dtype)


def rope_then_head_norm(qkv, positions, cos_cache, sin_cache, Hq, Hkv, D, rot, interleaved, q_norm_w, k_norm_w, norm_eps):
    """Families whose per-head q / k norms follow the rotary embedding (hunyuan): returns qkv with q and k rotated, then normalised; plain
    tensor operations on the tensor's own device."""
    T = qkv.shape[0]
    x = qkv.float().view(T, Hq + 2 * Hkv, D).clone()
    qk = x[:, :Hq + Hkv]
    if rot > 0:
        pos = positions.long().clamp(0, cos_cache.shape[0] - 1)
        qk = _rotate(qk, cos_cache[pos].float(), sin_cache[pos].float(), rot, interleaved)
    w = torch.cat([q_norm_w.float().expand(Hq, D), k_norm_w.float().expand(Hkv, D)], 0)
    x[:, :Hq + Hkv] = qk * torch.rsqrt((qk * qk).mean(-1, keepdim=True) + norm_eps) * w
    return x.view(T, -1).to(qkv.dtype)


def _rotate(v, cos, sin, rot, interleaved):
    # v: [T, H, D] fp32, cos/sin: [T, rot/2]
    out = v.clone()
    c, s = cos[:, None, :], sin[:, None, :]
    if interleaved:
        x1, x2 = v[..., 0:rot:2], v[..., 1:rot:2]
        out[..., 0:rot:2] = x1 * c - x2 * s
        out[..., 1:rot:2] = x2 * c + x1 * s
    else:
        half = rot // 2
        x1, x2 = v[..., :half], v[..., half:rot]
        out[..., :half] = x1 * c - x2 * s
        out[..., half:rot] = x2 * c + x1 * s
    return out


def rope_kv_append(qkv, positions, slots, cos_cache, sin_cache, k_cache, v_cache, Hq, Hkv, D, rot, interleaved=False,
                   q_norm_w=None, k_norm_w=None, norm_eps=1e-6, positions3=None, mrope_section=None, mrope_interleaved=False):
    """In place: rotates q inside `qkv`, writes rotated k and v into the caches at `slots`."""
    T = qkv.shape[0]
    dt = qkv.dtype
    x = qkv.float().view(T, Hq + 2 * Hkv, D)
    q, k, v = x[:, :Hq], x[:, Hq:Hq + Hkv], x[:, Hq + Hkv:]

    def head_norm(t, w):
        y = t * torch.rsqrt((t * t).mean(-1, keepdim=True) + norm_eps) * w.float()
        return y.to(dt).float()

    if q_norm_w is not None:
        q = head_norm(q, q_norm_w)
    if k_norm_w is not None:
        k = head_norm(k, k_norm_w)
    if rot > 0:
        pos = positions.long().clamp(0, cos_cache.shape[0] - 1)
        cos, sin = cos_cache[pos].float(), sin_cache[pos].float()
        if positions3 is not None:
            # multimodal RoPE: rotary pair i takes the angle of its section's position component
            p3 = positions3.long().clamp(0, cos_cache.shape[0] - 1)
            comp = torch.repeat_interleave(torch.arange(3), torch.tensor([mrope_section[0], mrope_section[1], rot // 2 - mrope_section[0] - mrope_section[1]]))
            if mrope_interleaved:
                pair = torch.arange(rot // 2)
                comp = torch.where((pair % 3 == 1) & (pair < 3 * mrope_section[1]), 1, torch.where((pair % 3 == 2) & (pair < 3 * mrope_section[2]), 2, 0))
            idx = torch.arange(rot // 2)
            cos = cos_cache[p3[comp], idx[:, None]].t().float()      # [T, rot/2]
            sin = sin_cache[p3[comp], idx[:, None]].t().float()
        q = _rotate(q, cos, sin, rot, interleaved)
        k = _rotate(k, cos, sin, rot, interleaved)
    qkv.view(T, Hq + 2 * Hkv, D)[:, :Hq] = q.to(dt)
    if slots is not None:
        ok = slots >= 0
        idx = slots[ok].long()
        if k_cache.dtype == torch.int8:
            kv8_store(k_cache, idx, k[ok], Hkv, D)
            kv8_store(v_cache, idx, v[ok], Hkv, D)
        else:
            k_cache.view(-1, Hkv, D)[idx] = k[ok].to(k_cache.dtype)
            v_cache.view(-1, Hkv, D)[idx] = v[ok].to(v_cache.dtype)
    return qkv


def kv8_store(cache, idx, rows, Hkv, D):
    """8-bit cache rows: D int8 values, the row's fp32 scale (absmax / 127), 12 bytes of padding."""
    c = cache.view(-1, Hkv, D + 16)
    amax = rows.abs().amax(-1, keepdim=True)
    scale = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax)).float()
    q = torch.round(rows.float() * (1.0 / scale)).clamp(-127, 127).to(torch.int8)
    c[idx, :, :D] = q
    c[idx, :, D:D + 4] = scale.contiguous().view(torch.int8).view(-1, Hkv, 4)


def kv8_load(cache, Hkv, D):
    """fp32 [slots, Hkv, D] values of an 8-bit cache, as the attention kernel expands them (value * scale rounded to bf16)."""
    c = cache.view(-1, Hkv, D + 16)
    scale = c[:, :, D:D + 4].contiguous().view(torch.float32)
    return (c[:, :, :D].float() * scale).to(torch.bfloat16).float()


def paged_attention(q, k_cache, v_cache, cu_seqlens, past_lens, block_table, block_size, Hq, Hkv, D, scale,
                    window=0, sinks=None, softcap=0.0):
    """q: [T, >=Hq*D] (only the first Hq*D columns are read).  Returns [T, Hq*D]."""
    T = q.shape[0]
    out = torch.zeros(T, Hq * D, dtype=q.dtype, device=q.device)
    if k_cache.dtype == torch.int8:
        kc, vc = kv8_load(k_cache, Hkv, D), kv8_load(v_cache, Hkv, D)
    else:
        kc = k_cache.view(-1, Hkv, D)
        vc = v_cache.view(-1, Hkv, D)
    G = Hq // Hkv
    B = past_lens.shape[0]
    cu = cu_seqlens.tolist()
    for b in range(B):
        t0, t1 = cu[b], cu[b + 1]
        n = t1 - t0
        if n == 0:
            continue
        past = int(past_lens[b])
        full = window is not None and window < 0     # bidirectional over the `past` cached keys (encoders, cross-attention)
        total = past if full else past + n
        pos = torch.arange(total, device=q.device)
        slots = block_table[b, (pos // block_size).long()].long() * block_size + pos % block_size
        k = kc[slots].float()  # [total, Hkv, D]
        v = vc[slots].float()
        qq = q[t0:t1, :Hq * D].float().view(n, Hq, D)
        k = k.repeat_interleave(G, dim=1)
        v = v.repeat_interleave(G, dim=1)
        s = torch.einsum("qhd,khd->hqk", qq, k) * scale
        if softcap and softcap > 0:
            s = softcap * torch.tanh(s / softcap)
        qpos = past + torch.arange(n, device=q.device)
        mask = (pos[None, :] <= qpos[:, None]) | full
        if window and window > 0:
            mask = mask & (pos[None, :] > qpos[:, None] - window)
        s = s.masked_fill(~mask[None], float("-inf"))
        if sinks is not None:
            sk = sinks.float().view(Hq, 1, 1).expand(Hq, n, 1)
            p = torch.softmax(torch.cat([s, sk], dim=-1), dim=-1)[..., :-1]
        else:
            p = torch.softmax(s, dim=-1)
        o = torch.einsum("hqk,khd->qhd", p, v)
        out[t0:t1] = o.reshape(n, Hq * D).to(q.dtype)
    return out


def sampled_distribution(logits_row, top_k, top_p, temperature):
    """Kept token ids and renormalised probabilities for one row (fp64 math, sorted descending)."""
    x = logits_row.double() / max(temperature, 1e-30)
    order = torch.sort(x, descending=True, stable=True).indices
    if top_k is not None and 1 < top_k < x.numel():
        order = order[:top_k]
    p = torch.softmax(x[order], dim=-1)
    if top_p is not None and 0.0 < top_p < 1.0:
        cum = torch.cumsum(p, 0)
        keep = int(torch.searchsorted(cum, torch.tensor(top_p, dtype=cum.dtype)).item()) + 1
        keep = min(keep, p.numel())
        order, p = order[:keep], p[:keep]
        p = p / p.sum()
    return order, p


def logits_bitmask(logits, mask_words, mask_rows=None):
    V = logits.shape[-1]
    v = torch.arange(V, device=logits.device)
    lowest = torch.finfo(torch.float32).min
    for r in range(logits.shape[0]):
        mr = r if mask_rows is None else int(mask_rows[r])
        if mr < 0:
            continue
        words = mask_words[mr].to(torch.int64) & 0xFFFFFFFF
        bits = (words[(v // 32).long()] >> (v % 32)) & 1
        logits[r][bits == 0] = lowest
    return logits


def logits_edit(logits, rows, tokens, ops, values):
    lowest = torch.finfo(torch.float32).min
    for r, t, o, val in zip(rows.tolist(), tokens.tolist(), ops.tolist(), values.tolist()):
        if t < 0 or t >= logits.shape[-1]:
            continue
        if o == 0:
            logits[r, t] = lowest
        else:
            x = logits[r, t]
            logits[r, t] = torch.where(x < 0, x * val, x / val)  # fp32 arithmetic (may saturate to -inf like the kernel)
    return logits


def topk(x, k, log_softmax=False, add=None):
    y = x.float()
    if log_softmax:
        y = torch.log_softmax(y, dim=-1)
        if add is not None:
            y = y + add.float()[:, None]
    # ties resolved towards the lower index
    vals, idx = torch.sort(y, dim=-1, descending=True, stable=True)
    return vals[:, :k].contiguous(), idx[:, :k].to(torch.int32).contiguous()


def short_conv(bcx, weight, bias, cache, slots, positions, cu_seqlens, past_lens, block_table, block_size):
    """Gated short depthwise convolution of a hybrid (LFM2) layer over packed sequences.
    bcx [T, 3C]: per token the gates b, c and the value x; weight [C, L]; cache [slots, C] holds b * x of every cached
    position (this step's are written at `slots`).  y[t] = c[t] * sum_k weight[:, L-1-k] * (b*x)[position(t) - k] (+ bias),
    positions before the start of the sequence contribute nothing."""
    T, C3 = bcx.shape
    C, L = weight.shape
    f = bcx.float()
    b, c, x = f[:, :C], f[:, C:2 * C], f[:, 2 * C:]
    bx = (b * x).to(bcx.dtype)
    ok = slots >= 0
    cache[slots[ok].long()] = bx[ok].to(cache.dtype)
    out = torch.zeros(T, C, dtype=torch.float32, device=bcx.device)
    cu = cu_seqlens.tolist()
    w = weight.float()
    for r in range(len(cu) - 1):
        for t in range(cu[r], cu[r + 1]):
            p = int(positions[t])
            acc = torch.zeros(C, dtype=torch.float32, device=bcx.device)
            for k in range(L):
                q = p - k
                if q < 0:
                    break
                slot = int(block_table[r, q // block_size]) * block_size + q % block_size
                acc += w[:, L - 1 - k] * cache[slot].float()
            if bias is not None:
                acc = acc + bias.float()
            out[t] = c[t] * acc
    return out.to(bcx.dtype)


def gated_delta(q, k, v, g, beta, state, slots, cu_seqlens, past_lens):
    """Gated delta rule over packed sequences (the LinearAttention op with update_rule "gated_delta", reference:
    src/python/py/models/builders/base.py:3419-3452, qwen.py:1842-1860).  q, k [T, Hk, dk] (already L2-normalised, q scaled),
    v [T, Hv, dv], g [T, Hv] log decay (<= 0), beta [T, Hv]; state [slots, Hv, dk, dv] fp32, updated in place for the request
    slots named by `slots` [B] (a request whose past length is 0 starts from a zero state).  Value head h reads key head
    h // (Hv / Hk).  Per token:  S *= exp(g);  delta = (v - S^T k) * beta;  S += k (x) delta;  out = S^T q."""
    T, Hk, dk = q.shape
    Hv, dv = v.shape[1], v.shape[2]
    rep = Hv // Hk
    out = torch.zeros(T, Hv, dv, dtype=torch.float32, device=q.device)
    cu = cu_seqlens.tolist()
    qf, kf = q.float().repeat_interleave(rep, dim=1), k.float().repeat_interleave(rep, dim=1)      # [T, Hv, dk]
    vf, gf, bf = v.float(), g.float(), beta.float()
    for r in range(len(cu) - 1):
        slot = int(slots[r])
        S = state[slot].float()
        if int(past_lens[r]) == 0:
            S = torch.zeros_like(S)
        for t in range(cu[r], cu[r + 1]):
            S = S * torch.exp(gf[t])[:, None, None]
            mem = torch.einsum("hkv,hk->hv", S, kf[t])
            delta = (vf[t] - mem) * bf[t][:, None]
            S = S + kf[t][:, :, None] * delta[:, None, :]
            out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
        state[slot] = S.to(state.dtype)
    return out.to(v.dtype)


def mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu_seqlens, past_lens):
    """Mamba-2 selective scan over packed sequences.  x [T, heads, P], dt [T, heads] (after softplus), neg_a [heads] (= -exp(A_log)),
    Bm / Cm [T, groups, N], Dv [heads]; state [slots, heads, N, P] fp32, updated in place for the request slots (a request whose
    past length is 0 starts from a zero state).  Head h reads group h // (heads / groups).  Per token:
    S *= exp(dt * A);  S[n][p] += dt * x[p] * B[n];  y[p] = sum_n S[n][p] * C[n] + D * x[p]."""
    T, heads, P = x.shape
    groups = Bm.shape[1]
    rep = heads // groups
    out = torch.zeros(T, heads, P, dtype=torch.float32, device=x.device)
    cu = cu_seqlens.tolist()
    xf, dtf = x.float(), dt.float()
    Bf, Cf = Bm.float().repeat_interleave(rep, dim=1), Cm.float().repeat_interleave(rep, dim=1)      # [T, heads, N]
    for r in range(len(cu) - 1):
        slot = int(slots[r])
        S = state[slot].float()
        if int(past_lens[r]) == 0:
            S = torch.zeros_like(S)
        for t in range(cu[r], cu[r + 1]):
            S = S * torch.exp(dtf[t] * neg_a.float())[:, None, None]
            S = S + Bf[t][:, :, None] * (dtf[t][:, None] * xf[t])[:, None, :]
            out[t] = torch.einsum("hnp,hn->hp", S, Cf[t]) + Dv.float()[:, None] * xf[t]
        state[slot] = S.to(state.dtype)
    return out.to(x.dtype)

