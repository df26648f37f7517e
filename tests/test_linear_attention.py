"""Gated-delta-net (linear attention) layers: a hybrid stack of recurrent layers and full-attention layers against a plain
per-token restatement of the layer (reference graph: src/python/py/models/builders/qwen.py:1776-1867; ops CausalConvWithState and
LinearAttention with update_rule "gated_delta"; state handling src/models/recurrent_state.h)."""
import copy
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model, random_state_dict

ARCH = dict(model_type="qwen3_next", vocab_size=120, hidden_size=64, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=16,
            intermediate_size=96, context_length=128, bos_token_id=0, eos_token_id=119, pad_token_id=0,
            layer_types=["linear_attention", "linear_attention", "full_attention", "linear_attention"],
            linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=16, linear_value_head_dim=16, linear_conv_kernel_dim=4)


def _rms(x, w, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w


def _rope(x, pos, theta):
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2).float() / d))
    ang = pos[:, None].float() * inv[None]
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def oracle_logits(arch: ArchConfig, sd, tokens):
    """The whole model token by token in fp32, every formula written out (no shared code with the runtime)."""
    T = len(tokens)
    h = sd["model.embed_tokens.weight"].float()[torch.tensor(tokens)]
    pos = torch.arange(T)
    nk, nv, hk, hv, K = arch.linear_num_key_heads, arch.linear_num_value_heads, arch.linear_key_head_dim, arch.linear_value_head_dim, arch.linear_conv_kernel_dim
    kd, vd = nk * hk, nv * hv
    for i in range(arch.num_layers):
        p = f"model.layers.{i}."
        x = _rms(h, sd[p + "input_layernorm.weight"].float(), arch.norm_eps)
        if arch.is_linear_layer(i):
            lp = p + "linear_attn."
            qkv = x @ sd[lp + "in_proj_qkv.weight"].float().t()
            z = x @ sd[lp + "in_proj_z.weight"].float().t()
            b = x @ sd[lp + "in_proj_b.weight"].float().t()
            a = x @ sd[lp + "in_proj_a.weight"].float().t()
            w = sd[lp + "conv1d.weight"].float()                      # [C, K]: tap K-1 multiplies the current position
            conv = torch.zeros_like(qkv)
            for t in range(T):
                for j in range(K):
                    if t - j >= 0:
                        conv[t] += w[:, K - 1 - j] * qkv[t - j]
            conv = F.silu(conv)
            q = F.normalize(conv[:, :kd].view(T, nk, hk), dim=-1, eps=1e-6) / math.sqrt(hk)
            k = F.normalize(conv[:, kd:2 * kd].view(T, nk, hk), dim=-1, eps=1e-6)
            v = conv[:, 2 * kd:].view(T, nv, hv)
            beta = torch.sigmoid(b)
            g = -torch.exp(sd[lp + "A_log"].float()) * F.softplus(a + sd[lp + "dt_bias"].float())
            S = torch.zeros(nv, hk, hv)
            out = torch.zeros(T, nv, hv)
            for t in range(T):
                for hh in range(nv):
                    kk, qq = k[t, hh // (nv // nk)], q[t, hh // (nv // nk)]
                    S[hh] = S[hh] * torch.exp(g[t, hh])
                    delta = (v[t, hh] - S[hh].t() @ kk) * beta[t, hh]
                    S[hh] = S[hh] + torch.outer(kk, delta)
                    out[t, hh] = S[hh].t() @ qq
            out = _rms(out, sd[lp + "norm.weight"].float(), arch.norm_eps).reshape(T, vd) * F.silu(z)
            att = out @ sd[lp + "out_proj.weight"].float().t()
        else:
            sp = p + "self_attn."
            D, Hq, Hkv = arch.head_dim, arch.num_heads, arch.num_kv_heads
            q = (x @ sd[sp + "q_proj.weight"].float().t()).view(T, Hq, D)
            k = (x @ sd[sp + "k_proj.weight"].float().t()).view(T, Hkv, D)
            v = (x @ sd[sp + "v_proj.weight"].float().t()).view(T, Hkv, D)
            q, k = _rope(q, pos, arch.rope_theta), _rope(k, pos, arch.rope_theta)
            k, v = k.repeat_interleave(Hq // Hkv, dim=1), v.repeat_interleave(Hq // Hkv, dim=1)
            sc = torch.einsum("thd,shd->hts", q, k) / math.sqrt(D)
            sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1)[None], float("-inf"))
            att = torch.einsum("hts,shd->thd", torch.softmax(sc, -1), v).reshape(T, Hq * D) @ sd[sp + "o_proj.weight"].float().t()
        h = h + att
        x = _rms(h, sd[p + "post_attention_layernorm.weight"].float(), arch.norm_eps)
        mlp = (F.silu(x @ sd[p + "mlp.gate_proj.weight"].float().t()) * (x @ sd[p + "mlp.up_proj.weight"].float().t())) @ sd[p + "mlp.down_proj.weight"].float().t()
        h = h + mlp
    h = _rms(h, sd["model.norm.weight"].float(), arch.norm_eps)
    head = sd.get("lm_head.weight", sd["model.embed_tokens.weight"]).float()
    return h @ head.t()


@pytest.fixture(scope="module")
def built(tmp_path_factory):
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=11, std=0.2)
    d = str(tmp_path_factory.mktemp("gdn"))
    export_model(copy.deepcopy(arch), d, "fp32", "cpu", state_dict=sd, paged=True, block_size=16, num_blocks=64, max_batch_size=4)
    return arch, sd, d


def test_hybrid_stack_matches_the_per_token_restatement(built):
    arch, sd, d = built
    model = og.Model(d)
    assert model.arch.layer_types == ARCH["layer_types"] and model.arch.linear_num_value_heads == 4
    prompt = np.random.RandomState(1).randint(1, 118, size=13).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=24, do_sample=False)
    g = og.Generator(model, p)
    g.append_tokens(prompt.reshape(1, -1))
    want = oracle_logits(arch, sd, prompt.tolist())
    np.testing.assert_allclose(g.get_logits().reshape(-1), want[-1].numpy(), rtol=2e-3, atol=2e-4)
    # decode steps carry the convolution window (from the paged cache) and the recurrent state (from the request's slot)
    toks = prompt.tolist()
    for _ in range(6):
        g.generate_next_token()
        toks.append(int(g.get_next_tokens()[0]))
        assert toks[-1] == int(oracle_logits(arch, sd, toks[:-1])[-1].argmax())
    # a recurrent state cannot be cropped: rewinding to an earlier length restarts from the empty state and feeds the kept tokens
    g.rewind_to(15)
    assert g.token_count() == 15
    np.testing.assert_allclose(g.get_logits().reshape(-1), oracle_logits(arch, sd, toks[:15])[-1].numpy(), rtol=2e-3, atol=2e-4)
    g.generate_next_token()
    assert int(g.get_next_tokens()[0]) == toks[15]
    g.rewind_to(0)
    g.append_tokens(prompt.reshape(1, -1))
    np.testing.assert_allclose(g.get_logits().reshape(-1), want[-1].numpy(), rtol=2e-3, atol=2e-4)


def test_speculative_decoding_over_recurrent_states(built):
    """N-gram speculation on the hybrid model: the verification pass feeds the drafts into the recurrent states; when drafts are
    rejected the saved states come back and the kept tokens are fed again, so the output equals plain greedy decoding."""
    arch, sd, d = built
    model = og.Model(d)
    prompt = np.asarray([[7, 8, 9, 10, 7, 8, 9, 10, 7, 8, 9, 11, 7, 8]], dtype=np.int32)

    def run(spec):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=44, do_sample=False)
        if spec:
            p.set_speculative_options(ngram_size=2, max_draft_tokens=4)
        g = og.Generator(model, p)
        g.append_tokens(prompt)
        while not g.is_done():
            g.generate_next_token()
        return g.get_sequence(0).tolist(), (g.get_speculative_stats() if spec else None)

    plain, _ = run(False)
    spec, st = run(True)
    assert spec == plain
    assert st["rounds"] > 0 and st["proposed"] > st["accepted"]          # some drafts were rejected: the restore path ran


def test_engine_batches_recurrent_requests(built):
    """Requests of a recurrent model share engine steps (chunked prompts, joining and leaving) and each keeps its own state slot."""
    arch, sd, d = built
    model = og.Model(d)
    rs = np.random.RandomState(5)
    prompts = [rs.randint(1, 118, size=n).astype(np.int32) for n in (9, 21, 5)]

    def run(which):
        eng = og.Engine(model)
        reqs = []
        for i in which:
            p = og.GeneratorParams(model)
            p.set_search_options(max_length=len(prompts[i]) + 8, do_sample=False)
            r = og.Request(p)
            r.add_tokens(prompts[i])
            eng.add_request(r)
            reqs.append(r)
        outs = [[] for _ in reqs]
        for _ in range(200):
            if not eng.has_pending_requests():
                break
            eng.step()
            for j, r in enumerate(reqs):
                while r.has_unseen_tokens():
                    outs[j].append(r.get_unseen_token())
        for r in reqs:
            eng.remove_request(r)
        return outs

    together = run([0, 1, 2])
    for i in range(3):
        want, toks = [], prompts[i].tolist()
        for _ in range(8):
            toks.append(int(oracle_logits(arch, sd, toks)[-1].argmax()))
            want.append(toks[-1])
        assert together[i] == want
    assert run([1])[0] == together[1]
