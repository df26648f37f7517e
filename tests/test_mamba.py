"""Mamba-2 layers in a hybrid stack (granitemoehybrid, dense members: Mamba-2 and attention layers around a gated MLP, no position
encoding).  The oracle is the checkpoint family's own implementation in `transformers` (its pure-torch path), built with a small random
configuration; the checkpoint travels through the same export a real one would (config.json + safetensors -> create_model)."""
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200 import ops
from onnxruntime_genai_b200.models.builder import create_model
from onnxruntime_genai_b200.ops import reference as ref

hf_modeling = pytest.importorskip("transformers.models.granitemoehybrid.modeling_granitemoehybrid")
hf_config = pytest.importorskip("transformers.models.granitemoehybrid.configuration_granitemoehybrid")

VOCAB = 97


def _hf_model(seed=0, layer_types=("mamba", "attention", "mamba", "mamba"), rope=False, hidden=64):
    torch.manual_seed(seed)
    cfg = hf_config.GraniteMoeHybridConfig(
        vocab_size=VOCAB, hidden_size=hidden, intermediate_size=96, num_hidden_layers=len(layer_types), num_attention_heads=4, num_key_value_heads=2,
        max_position_embeddings=128, rms_norm_eps=1e-5, tie_word_embeddings=False, num_local_experts=0, num_experts_per_tok=0,
        shared_intermediate_size=96, layer_types=list(layer_types), mamba_n_heads=8, mamba_d_head=hidden // 4, mamba_d_state=16, mamba_n_groups=2,
        mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=8, mamba_conv_bias=True, mamba_proj_bias=False,
        embedding_multiplier=1.5, logits_scaling=2.0, residual_multiplier=0.7, attention_multiplier=0.2,
        position_embedding_type="rope" if rope else None, bos_token_id=0, eos_token_id=VOCAB - 1, pad_token_id=0)
    m = hf_modeling.GraniteMoeHybridForCausalLM(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 3 + 0.5))
            elif n.endswith("dt_bias"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith(".D"):
                p.copy_(torch.randn_like(p))
            elif "norm" in n:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.copy_(torch.randn_like(p) * 0.08)
    return cfg, m


def _export(tmp_path, cfg, m, name="g", precision="fp32", provider="cpu"):
    from safetensors.torch import save_file
    src = tmp_path / (name + "_hf")
    os.makedirs(src)
    save_file({k: v.detach().contiguous() for k, v in m.state_dict().items()}, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps(cfg.to_dict()))
    out = str(tmp_path / name)
    create_model(str(src), out, precision, provider)
    return out


@pytest.fixture(scope="module")
def exported(tmp_path_factory):
    cfg, m = _hf_model()
    return cfg, m, _export(tmp_path_factory.mktemp("mamba"), cfg, m)


def _hf_logits(m, ids):
    with torch.no_grad():
        return m(torch.tensor([ids], dtype=torch.long)).logits[0].float()


def test_scan_reference_matches_per_token_recurrence():
    """ops.mamba2_scan (the plain restatement on CPU): h_t = exp(dt*A) h_{t-1} + dt * B_t x_t^T ; y_t = C_t . h_t + D x_t, ragged batches
    with carried state."""
    torch.manual_seed(1)
    heads, groups, P, N = 4, 2, 8, 16
    lens, past = [5, 1, 3], [0, 4, 2]
    T = sum(lens)
    x = torch.randn(T, heads, P)
    dt = torch.rand(T, heads) + 0.05
    neg_a = -(torch.rand(heads) + 0.2)
    Bm, Cm = torch.randn(T, groups, N), torch.randn(T, groups, N)
    Dv = torch.randn(heads)
    state = torch.randn(4, heads, N, P)
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    cu = torch.tensor([0, 5, 6, 9], dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    st0 = state.clone()
    got = ops.mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu, pl)
    want = torch.zeros(T, heads, P)
    t0 = 0
    for r, L in enumerate(lens):
        S = st0[slots[r]].clone() if past[r] > 0 else torch.zeros(heads, N, P)
        for t in range(t0, t0 + L):
            for h in range(heads):
                g = h // (heads // groups)
                S[h] = torch.exp(dt[t, h] * neg_a[h]) * S[h] + dt[t, h] * Bm[t, g][:, None] * x[t, h][None, :]
                want[t, h] = Cm[t, g] @ S[h] + Dv[h] * x[t, h]
        torch.testing.assert_close(state[slots[r]], S, rtol=1e-5, atol=1e-5)
        t0 += L
    torch.testing.assert_close(got, want, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(state[1], st0[1])          # a slot no request names is left alone


def test_prefill_logits_match_the_family_implementation(exported):
    cfg, m, out = exported
    model = og.Model(out)
    assert model.arch.layer_types == ["mamba", "full_attention", "mamba", "mamba"] and model.arch.no_rope
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 19)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=40)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    want = _hf_logits(m, ids[0].tolist())[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=2e-4)


def test_token_by_token_decode_matches_one_prefill(exported):
    """The carried convolution window and scan state: greedy continuation, each step against the family's full-sequence logits."""
    cfg, m, out = exported
    model = og.Model(out)
    ids = np.random.RandomState(1).randint(1, VOCAB - 1, size=(2, 7)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=20, batch_size=2)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seqs = [ids[0].tolist(), ids[1].tolist()]
    for _ in range(8):
        lg = g.get_logits()
        for b in range(2):
            want = _hf_logits(m, seqs[b])[-1].numpy()
            np.testing.assert_allclose(lg[b].reshape(-1), want, rtol=3e-3, atol=3e-4)
        g.generate_next_token()
        nt = g.get_next_tokens()
        for b in range(2):
            seqs[b].append(int(nt[b]))
        if g.is_done():
            break


def test_rotary_member_and_rewind(tmp_path):
    """A member with rotary attention layers; rewinding recomputes the recurrent state of the kept prefix."""
    cfg, m = _hf_model(seed=3, layer_types=("attention", "mamba"), rope=True)
    out = _export(tmp_path, cfg, m, "r")
    model = og.Model(out)
    assert not model.arch.no_rope
    ids = np.random.RandomState(2).randint(1, VOCAB - 1, size=(1, 12)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    np.testing.assert_allclose(g.get_logits().reshape(-1), _hf_logits(m, ids[0].tolist())[-1].numpy(), rtol=2e-3, atol=2e-4)
    for _ in range(4):
        g.generate_next_token()
    g.rewind_to(9)
    g.append_tokens(np.array([[5, 6]], dtype=np.int32))
    want = _hf_logits(m, ids[0, :9].tolist() + [5, 6])[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=2e-4)


def test_engine_serves_a_mamba_hybrid(exported):
    """Continuous batching over recurrent slots: two requests of different lengths, greedy, against single-request generation."""
    cfg, m, out = exported
    model = og.Model(out)
    prompts = [[3, 9, 27, 81, 50], [7, 14, 21, 28, 35, 42, 49, 56, 63]]
    want = []
    for pr in prompts:
        seq = list(pr)
        for _ in range(6):
            seq.append(int(_hf_logits(m, seq)[-1].argmax()))
        want.append(seq[len(pr):])
    eng = og.Engine(model)
    reqs = []
    for pr in prompts:
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=len(pr) + 6)
        r = og.Request(p)
        r.add_tokens(np.array(pr, dtype=np.int32))
        eng.add_request(r)
        reqs.append(r)
    got = [[] for _ in prompts]
    while eng.has_pending_requests():
        eng.step()
        for i, r in enumerate(reqs):
            while r.has_unseen_tokens():
                got[i].append(int(r.get_unseen_token()))
    assert got == want


def test_int4_export_of_the_hybrid(exported, tmp_path):
    """The int4 exporter quantises every projection of the hybrid (Mamba in / out projections, attention, MLP): the checkpoint loads
    and follows the fp32 export (a tiny random model: 4-bit rounding is coarse, so the check is the correlation of the logits)."""
    cfg, m, out32 = exported
    out4 = _export(tmp_path, cfg, m, "q4", "int4", "cpu")
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 12)).astype(np.int32)
    logits = []
    for d in (out32, out4):
        model = og.Model(d)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=32)
        g = og.Generator(model, p)
        g.append_tokens(ids)
        logits.append(g.get_logits().reshape(-1).astype(np.float64))
    assert np.isfinite(logits[1]).all()
    assert np.corrcoef(logits[0], logits[1])[0, 1] > 0.8


@pytest.mark.gpu
@pytest.mark.parametrize("heads,groups,P,N", [(8, 2, 16, 16), (24, 1, 64, 128), (4, 4, 64, 256)])
def test_scan_kernel_matches_reference(heads, groups, P, N):
    torch.manual_seed(heads)
    dev = "cuda"
    lens, past = [37, 1, 1, 130], [0, 9, 3, 64]
    T = sum(lens)
    x = torch.randn(T, heads, P, device=dev, dtype=torch.bfloat16)
    dt = (torch.rand(T, heads, device=dev) * 0.5 + 0.01)
    neg_a = -(torch.rand(heads, device=dev) * 2 + 0.1)
    Bm = torch.randn(T, groups, N, device=dev, dtype=torch.bfloat16) * 0.5
    Cm = torch.randn(T, groups, N, device=dev, dtype=torch.bfloat16) * 0.5
    Dv = torch.randn(heads, device=dev)
    state = torch.randn(6, heads, N, P, device=dev)
    slots = torch.tensor([4, 1, 5, 0], dtype=torch.int32, device=dev)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=dev)
    pl = torch.tensor(past, dtype=torch.int32, device=dev)
    st_ref = state.clone().cpu()
    want = ref.mamba2_scan(x.float().cpu(), dt.cpu(), neg_a.cpu(), Bm.float().cpu(), Cm.float().cpu(), Dv.cpu(), st_ref, slots.cpu(), cu.cpu(), pl.cpu())
    got = ops.mamba2_scan(x, dt, neg_a, Bm, Cm, Dv, state, slots, cu, pl)
    torch.testing.assert_close(got.float().cpu(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(state.cpu(), st_ref, rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_gpu_generation_matches_the_family_implementation(tmp_path):
    cfg, m = _hf_model(seed=5, hidden=256)
    out = _export(tmp_path, cfg, m, "gpu", "bf16", "cuda")
    model = og.Model(out)
    assert model.device_type == "cuda"
    ids = np.random.RandomState(4).randint(1, VOCAB - 1, size=(1, 23)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=48)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(6):
        want = _hf_logits(m, seq)[-1].numpy()
        got = np.asarray(g.get_logits(), dtype=np.float32).reshape(-1)
        assert np.abs(got - want).max() < 0.04 * max(1.0, np.abs(want).max())
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break


@pytest.mark.gpu
def test_gpu_engine_graph_steps_equal_eager_steps(tmp_path):
    """Three requests of a Mamba-2 hybrid through the engine in bf16: decode steps replayed from CUDA graphs (state slots in the staging
    buffer, states put back after the capture warm-up) give the tokens of the same run without graphs."""
    cfg, m = _hf_model(seed=6, hidden=256)
    out = _export(tmp_path, cfg, m, "eng", "bf16", "cuda")
    model = og.Model(out)
    prompts = [list(range(3, 3 + n)) for n in (21, 5, 12)]
    runs = []
    for graphs in (True, False):
        eng = og.Engine(model)
        eng.executor.use_graphs = graphs
        reqs = []
        for pr in prompts:
            p = og.GeneratorParams(model)
            p.set_search_options(max_length=len(pr) + 8, min_length=len(pr) + 8)
            r = og.Request(p)
            r.add_tokens(np.array(pr, dtype=np.int32))
            eng.add_request(r)
            reqs.append(r)
        got = [[] for _ in prompts]
        while eng.has_pending_requests():
            eng.step()
            for i, r in enumerate(reqs):
                while r.has_unseen_tokens():
                    got[i].append(int(r.get_unseen_token()))
        assert all(len(g_) == 8 for g_ in got)
        if graphs:
            assert eng.executor.graphs
        runs.append(got)
    assert runs[0] == runs[1]
