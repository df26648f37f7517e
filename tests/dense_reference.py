"""Independent dense fp32 reference of the decoder families (full recompute, no cache, no paging, no ops
from the package): canonical Hugging Face style state dict + ArchConfig -> next-token logits."""
import math

import torch

from onnxruntime_genai_b200.models.arch import longrope_caches, rope_caches


def _norm(x, w, b, arch):
    if arch.layernorm:
        y = torch.nn.functional.layer_norm(x, (x.shape[-1],), None, None, arch.norm_eps)
    else:
        y = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + arch.norm_eps)
    y = y * (w.float() + arch.norm_offset)
    return y + b.float() if b is not None else y


def _rope(x, cos, sin, rot, interleaved):
    out = x.clone()
    c, s = cos[:, None, :], sin[:, None, :]
    if interleaved:
        a, b = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2], out[..., 1:rot:2] = a * c - b * s, b * c + a * s
    else:
        h = rot // 2
        a, b = x[..., :h], x[..., h:rot]
        out[..., :h], out[..., h:rot] = a * c - b * s, b * c + a * s
    return out


def logits(arch, sd, ids, encoder_hidden=None, inputs_embeds=None, positions3=None):
    """ids: list of token ids; returns logits [len(ids), vocab] (fp32).  encoder_hidden [S_enc, H_enc]: output of the
    encoder for cross-attention decoders; inputs_embeds [len(ids), H] overrides the token embeddings."""
    sd = {k: v.float() for k, v in sd.items()}
    S = len(ids)
    pos = torch.arange(S)
    cos, sin = rope_caches(arch, max(S, 8))
    multi = longrope_caches(arch)
    if multi is not None and S <= multi[4]:
        cos, sin = multi[0], multi[1]      # sequences within the original context use the short-factor caches
    cos_t, sin_t = torch.from_numpy(cos), torch.from_numpy(sin)
    cos, sin = cos_t[pos], sin_t[pos]
    if positions3 is not None:
        # multimodal RoPE: rotary pair i turns by the angle of its section's position component ([3, S] positions)
        half = arch.rotary_dim // 2
        sec = list(arch.mrope_section)
        comp = [0] * sec[0] + [1] * sec[1] + [2] * (half - sec[0] - sec[1])
        p3 = torch.as_tensor(positions3).long()
        cos = torch.stack([cos_t[p3[comp[i]], i] for i in range(half)], dim=1)
        sin = torch.stack([sin_t[p3[comp[i]], i] for i in range(half)], dim=1)
    h = sd["model.embed_tokens.weight"][torch.tensor(ids)] * arch.embed_scale
    if inputs_embeds is not None:
        h = inputs_embeds.float()
    if arch.learned_positions:
        h = h + sd["model.position_embeddings.weight"][pos]
    G = arch.num_heads // arch.num_kv_heads
    D = arch.head_dim
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        g = lambda n: sd.get(p + n)
        x = _norm(h, g("input_layernorm.weight"), g("input_layernorm.bias"), arch)
        lin = lambda t, n: t @ g(n + ".weight").t() + (g(n + ".bias") if g(n + ".bias") is not None else 0)
        if arch.is_conv_layer(i):
            # gated short convolution: causal depthwise conv1d of b * x, gated by c
            H, Lc = arch.hidden_size, arch.conv_L_cache
            b_, c_, x_ = lin(x, "conv.in_proj").split(H, dim=-1)
            bx = (b_ * x_).t()[None]                                              # [1, H, S]
            conv = torch.nn.functional.conv1d(torch.nn.functional.pad(bx, (Lc - 1, 0)), g("conv.conv.weight").view(H, 1, Lc),
                                              g("conv.conv.bias"), groups=H)[0].t()
            h = h + lin(c_ * conv, "conv.out_proj")
            x = _norm(h, g("post_attention_layernorm.weight"), g("post_attention_layernorm.bias"), arch)
            h = h + lin(torch.nn.functional.silu(lin(x, "mlp.gate_proj")) * lin(x, "mlp.up_proj"), "mlp.down_proj")
            continue
        q = lin(x, "self_attn.q_proj").view(S, arch.num_heads, D)
        k = lin(x, "self_attn.k_proj").view(S, arch.num_kv_heads, D)
        v = lin(x, "self_attn.v_proj").view(S, arch.num_kv_heads, D)
        if arch.qk_norm:
            hn = lambda t, w: t * torch.rsqrt((t * t).mean(-1, keepdim=True) + arch.norm_eps) * (w + arch.norm_offset)
            q, k = hn(q, g("self_attn.q_norm.weight")), hn(k, g("self_attn.k_norm.weight"))
        if not arch.learned_positions:
            q, k = _rope(q, cos, sin, arch.rotary_dim, arch.rotary_interleaved), _rope(k, cos, sin, arch.rotary_dim, arch.rotary_interleaved)
        k, v = k.repeat_interleave(G, 1), v.repeat_interleave(G, 1)
        s = torch.einsum("qhd,khd->hqk", q, k) * arch.scale
        if arch.softcap > 0:
            s = arch.softcap * torch.tanh(s / arch.softcap)
        mask = pos[None, :] <= pos[:, None]
        w = arch.layer_window(i)
        if w > 0:
            mask &= pos[None, :] > pos[:, None] - w
        s = s.masked_fill(~mask[None], float("-inf"))
        if arch.attn_sinks:
            sk = g("self_attn.sinks").view(-1, 1, 1).expand(-1, S, 1)
            pr = torch.softmax(torch.cat([s, sk], -1), -1)[..., :-1]
        else:
            pr = torch.softmax(s, -1)
        att = torch.einsum("hqk,khd->qhd", pr, v).reshape(S, arch.num_heads * D)
        o = lin(att, "self_attn.o_proj")
        if arch.cross_attention:
            h = h + o
            xc = _norm(h, g("cross_attn_layernorm.weight"), g("cross_attn_layernorm.bias"), arch)
            e = encoder_hidden.float()
            cq = lin(xc, "cross_attn.q_proj").view(S, arch.num_heads, D)
            ckk = lin(e, "cross_attn.k_proj").view(-1, arch.num_heads, D)
            cvv = lin(e, "cross_attn.v_proj").view(-1, arch.num_heads, D)
            cp = torch.softmax(torch.einsum("qhd,khd->hqk", cq, ckk) * arch.scale, -1)
            o = lin(torch.einsum("hqk,khd->qhd", cp, cvv).reshape(S, -1), "cross_attn.o_proj")
        if arch.parallel_block:      # attention and MLP both read the one normalised input
            h = h + o + lin(torch.nn.functional.gelu(lin(x, "mlp.fc1"), approximate="tanh"), "mlp.fc2")
            continue
        if arch.post_sublayer_norms:
            o = _norm(o, g("post_attention_layernorm.weight"), None, arch)
            mid = "pre_feedforward_layernorm"
        else:
            mid = "post_attention_layernorm"
        h = h + o * arch.residual_multiplier
        x = _norm(h, g(mid + ".weight"), g(mid + ".bias"), arch)
        if arch.num_experts > 0 and arch.moe_style == "standard":
            rl = x @ g("mlp.router.weight").t()
            probs = torch.softmax(rl, -1)
            tw, ti = torch.topk(probs, arch.experts_per_token, -1)
            if arch.moe_norm_topk:
                tw = tw / tw.sum(-1, keepdim=True)
            if arch.moe_sparse_mixer:
                tw, ti = _sparse_mixer_loop(rl, arch.moe_jitter_eps)
            y = torch.zeros_like(x)
            for t in range(S):
                for j in range(arch.experts_per_token):
                    e = int(ti[t, j])
                    a_ = torch.nn.functional.silu(x[t] @ g("mlp.experts.gate_proj")[e].t()) * (x[t] @ g("mlp.experts.up_proj")[e].t())
                    y[t] += tw[t, j] * (a_ @ g("mlp.experts.down_proj")[e].t())
        elif arch.num_experts > 0:
            router = x @ g("mlp.router.weight").t() + g("mlp.router.bias")
            tv, ti = torch.topk(router, arch.experts_per_token, -1)
            tw = torch.softmax(tv, -1)
            y = torch.zeros_like(x)
            for t in range(S):
                for j in range(arch.experts_per_token):
                    e = int(ti[t, j])
                    gu = x[t] @ g("mlp.experts.gate_up_proj")[e].t() + g("mlp.experts.gate_up_proj_bias")[e]
                    gt, up = gu[0::2].clamp(max=arch.moe_swiglu_limit), gu[1::2].clamp(-arch.moe_swiglu_limit, arch.moe_swiglu_limit)
                    a = gt * torch.sigmoid(arch.moe_swiglu_alpha * gt) * (up + 1)
                    y[t] += tw[t, j] * (a @ g("mlp.experts.down_proj")[e].t() + g("mlp.experts.down_proj_bias")[e])
        elif not arch.mlp_gated:
            approx = "none" if arch.activation == "gelu_erf" else "tanh"
            y = lin(torch.nn.functional.gelu(lin(x, "mlp.fc1"), approximate=approx), "mlp.fc2")
        else:
            gt, up = lin(x, "mlp.gate_proj"), lin(x, "mlp.up_proj")
            a = torch.nn.functional.silu(gt) if arch.activation == "silu" else torch.nn.functional.gelu(gt, approximate="tanh")
            y = lin(a * up, "mlp.down_proj")
        if arch.post_sublayer_norms:
            y = _norm(y, g("post_feedforward_layernorm.weight"), None, arch)
        h = h + y * arch.residual_multiplier
    x = _norm(h, sd["model.norm.weight"], sd.get("model.norm.bias"), arch)
    head = sd["model.embed_tokens.weight"] if arch.tie_embeddings else sd["lm_head.weight"]
    out = x @ head.t()
    if sd.get("lm_head.bias") is not None and not arch.tie_embeddings:
        out = out + sd["lm_head.bias"]
    out = out * arch.logits_scale
    if arch.final_logit_softcap > 0:
        out = torch.tanh(out / arch.final_logit_softcap) * arch.final_logit_softcap
    return out


def encoder(cfg, sd, x):
    """The audio / vision encoder on one sequence of embedded frames or patches x [S, H] (positions already added):
    pre-LayerNorm blocks with bidirectional attention, final LayerNorm."""
    F = torch.nn.functional
    sd = {k: v.float() for k, v in sd.items()}
    H, nh = cfg.hidden_size, cfg.num_heads
    D = H // nh
    ln = lambda t, n: F.layer_norm(t, (H,), sd[n + ".weight"], sd[n + ".bias"], cfg.norm_eps)
    h = x.float()
    S = h.shape[0]
    for i in range(cfg.num_layers):
        p = f"encoder.layers.{i}."
        lin = lambda t, n: t @ sd[p + n + ".weight"].t() + sd[p + n + ".bias"]
        y = ln(h, p + "self_attn_layer_norm")
        q, k, v = (lin(y, "self_attn." + n).view(S, nh, D) for n in ("q_proj", "k_proj", "v_proj"))
        pr = torch.softmax(torch.einsum("qhd,khd->hqk", q, k) / D ** 0.5, -1)
        h = h + lin(torch.einsum("hqk,khd->qhd", pr, v).reshape(S, H), "self_attn.out_proj")
        y = ln(h, p + "final_layer_norm")
        h = h + lin(F.gelu(lin(y, "fc1")), "fc2")
    return ln(h, "encoder.layer_norm")


def whisper_encoder(cfg, sd, features):
    """features [n_mels, frames] -> encoder output [frames / 2, H]."""
    F = torch.nn.functional
    f = features.float()[None]
    x = F.gelu(F.conv1d(f, sd["encoder.conv1.weight"].float(), sd["encoder.conv1.bias"].float(), padding=1))
    x = F.gelu(F.conv1d(x, sd["encoder.conv2.weight"].float(), sd["encoder.conv2.bias"].float(), padding=1, stride=2))[0].t()
    return encoder(cfg, sd, x + sd["encoder.embed_positions.weight"].float()[:x.shape[0]])


def vision_encoder(cfg, sd, pixels):
    """pixels [C, size, size] -> projected image features [patches, projection_size]."""
    F = torch.nn.functional
    x = F.conv2d(pixels.float()[None], sd["encoder.patch_embedding.weight"].float(), sd["encoder.patch_embedding.bias"].float(),
                 stride=cfg.patch_size)[0].flatten(1).t()
    h = encoder(cfg, sd, x + sd["encoder.embed_positions.weight"].float())
    if cfg.projection_size:
        h = F.gelu(h @ sd["projector.fc1.weight"].float().t() + sd["projector.fc1.bias"].float())
        h = h @ sd["projector.fc2.weight"].float().t() + sd["projector.fc2.bias"].float()
    return h


def _sparse_mixer_loop(logits, eps):
    """PhiMoE routing, token by token in plain Python: pick the best expert, weight it by a softmax over the logits within
    the relative margin of the maximum; remove it and repeat once."""
    T, E = logits.shape
    w, idx = torch.zeros(T, 2), torch.zeros(T, 2, dtype=torch.long)
    for t in range(T):
        s = logits[t].tolist()
        cur = list(s)
        for j in range(2):
            top = max(cur)
            i = cur.index(top)
            kept = [cur[e] for e in range(E) if cur[e] != float("-inf") and (top - s[e]) / max(abs(s[e]), top) <= 2 * eps]
            m = max(kept)
            z = sum(math.exp(v - m) for v in kept)
            w[t, j], idx[t, j] = math.exp(top - m) / z, i
            cur[i] = float("-inf")
    return w, idx
