"""Mixture-of-experts checkpoints in their Hugging Face layouts through config.json + safetensors -> create_model -> Generator,
against the families' own implementations in `transformers` (small random configurations): stacked fused expert tensors
(`mlp.experts.gate_up_proj`), one module per expert (`block_sparse_moe.experts.N.w1/w3/w2`), shared experts with and without
their sigmoid gate (reference graph: src/python/py/models/builders/qwen.py make_shared_expert), and the hybrids whose other
layers are gated-delta-net or Mamba-2 layers."""
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.builder import create_model

transformers = pytest.importorskip("transformers")
VOCAB = 89
WIDTH = {"hidden": 64}


def _common():
    return dict(COMMON, hidden_size=WIDTH["hidden"])


COMMON = dict(vocab_size=VOCAB, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
              bos_token_id=0, eos_token_id=VOCAB - 1, pad_token_id=0, tie_word_embeddings=False)


def _randomise(m, zero_centred=False):
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("A_log"):
                p.copy_(torch.log(torch.rand_like(p) * 3 + 0.5))
            elif n.endswith("dt_bias"):
                p.copy_(torch.randn_like(p) * 0.5)
            elif n.endswith(".D"):
                p.copy_(torch.randn_like(p))
            elif "norm" in n:
                off = 0.0 if (zero_centred and not n.endswith("linear_attn.norm.weight")) else 1.0
                p.copy_(off + 0.1 * torch.randn_like(p))
            elif n.endswith("mlp.gate.weight") or "router" in n:
                p.copy_(torch.randn_like(p) * 0.5)
            else:
                p.copy_(torch.randn_like(p) * 0.08)
    return m.float().eval()


def _mixtral():
    cfg = transformers.MixtralConfig(**_common(), intermediate_size=48, num_hidden_layers=2, num_local_experts=4, num_experts_per_tok=2, head_dim=WIDTH["hidden"] // 4)
    return cfg, _randomise(transformers.MixtralForCausalLM(cfg)), {}


def _mixtral_per_expert():
    """The older layout of the same family: one module per expert."""
    cfg, m, _ = _mixtral()
    def relayout(sd):
        out = {}
        for k, v in sd.items():
            if k.endswith("mlp.experts.gate_up_proj"):
                base = k[: -len("mlp.experts.gate_up_proj")] + "block_sparse_moe.experts."
                half = v.shape[1] // 2
                for e in range(v.shape[0]):
                    out[f"{base}{e}.w1.weight"], out[f"{base}{e}.w3.weight"] = v[e, :half].clone(), v[e, half:].clone()
            elif k.endswith("mlp.experts.down_proj"):
                base = k[: -len("mlp.experts.down_proj")] + "block_sparse_moe.experts."
                for e in range(v.shape[0]):
                    out[f"{base}{e}.w2.weight"] = v[e].clone()
            elif k.endswith("mlp.gate.weight"):
                out[k[: -len("mlp.gate.weight")] + "block_sparse_moe.gate.weight"] = v
            else:
                out[k] = v
        return out
    return cfg, m, {"relayout": relayout}


def _qwen2_moe():
    cfg = transformers.Qwen2MoeConfig(**_common(), intermediate_size=48, moe_intermediate_size=32, shared_expert_intermediate_size=40, num_hidden_layers=2,
                                      num_experts=4, num_experts_per_tok=2, norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
    return cfg, _randomise(transformers.Qwen2MoeForCausalLM(cfg)), {}


def _qwen3_5_moe():
    c = pytest.importorskip("transformers.models.qwen3_5_moe.configuration_qwen3_5_moe")
    mm = pytest.importorskip("transformers.models.qwen3_5_moe.modeling_qwen3_5_moe")
    cfg = c.Qwen3_5MoeTextConfig(**_common(), num_hidden_layers=3, head_dim=WIDTH["hidden"] // 2, linear_conv_kernel_dim=4, linear_key_head_dim=WIDTH["hidden"] // 4, linear_value_head_dim=WIDTH["hidden"] // 4,
                                 linear_num_key_heads=2, linear_num_value_heads=4, layer_types=["linear_attention", "full_attention", "linear_attention"],
                                 moe_intermediate_size=32, shared_expert_intermediate_size=48, num_experts=8, num_experts_per_tok=2)
    return cfg, _randomise(mm.Qwen3_5MoeForCausalLM(cfg), zero_centred=True), {}


def _granite_hybrid_moe():
    cfg = transformers.GraniteMoeHybridConfig(**_common(), intermediate_size=32, shared_intermediate_size=40, num_hidden_layers=3, num_local_experts=4,
                                              num_experts_per_tok=2, layer_types=["mamba", "attention", "mamba"], mamba_n_heads=8, mamba_d_head=WIDTH["hidden"] // 4,
                                              mamba_d_state=16, mamba_n_groups=1, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=8,
                                              embedding_multiplier=2.0, logits_scaling=3.0, residual_multiplier=0.5, attention_multiplier=0.25,
                                              position_embedding_type=None)
    return cfg, _randomise(transformers.GraniteMoeHybridForCausalLM(cfg)), {}


def _granite_moe_shared():
    if not hasattr(transformers, "GraniteMoeSharedForCausalLM"):
        pytest.skip("transformers has no GraniteMoeSharedForCausalLM")
    cfg = transformers.GraniteMoeSharedConfig(**_common(), intermediate_size=32, shared_intermediate_size=40, num_hidden_layers=2, num_local_experts=4,
                                              num_experts_per_tok=2, embedding_multiplier=2.0, logits_scaling=3.0, residual_multiplier=0.5,
                                              attention_multiplier=0.25)
    return cfg, _randomise(transformers.GraniteMoeSharedForCausalLM(cfg)), {}


@pytest.mark.parametrize("family", [_mixtral, _mixtral_per_expert, _qwen2_moe, _qwen3_5_moe, _granite_hybrid_moe, _granite_moe_shared],
                         ids=lambda f: f.__name__.strip("_"))
def test_moe_checkpoint_matches_the_family_implementation(family, tmp_path):
    from safetensors.torch import save_file
    torch.manual_seed(0)
    cfg, m, opt = family()
    sd = {k: v.detach().contiguous() for k, v in m.state_dict().items()}
    if "relayout" in opt:
        sd = opt["relayout"](sd)
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file(sd, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = [type(m).__name__]
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    model = og.Model(out)
    assert model.arch.num_experts == (cfg.num_local_experts if hasattr(cfg, "num_local_experts") else cfg.num_experts)
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 13)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(4):
        with torch.no_grad():
            want = m(torch.tensor([seq])).logits[0, -1].float().numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=3e-4)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():      # the end-of-sequence token: no further logits
            break


@pytest.mark.gpu
@pytest.mark.parametrize("family", [_mixtral, _qwen2_moe, _qwen3_5_moe, _granite_hybrid_moe], ids=lambda f: f.__name__.strip("_"))
def test_moe_checkpoint_on_the_gpu(family, tmp_path):
    """The same checkpoints four times as wide (heads of 64 and more) in bf16 on the CUDA path - grouped expert GEMMs, shared experts,
    recurrent layers - against the fp32 logits of the family's implementation, with the family's own bf16 error as the yardstick."""
    import copy
    from safetensors.torch import save_file
    WIDTH["hidden"] = 256
    try:
        torch.manual_seed(0)
        cfg, m, opt = family()
    finally:
        WIDTH["hidden"] = 64
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" not in n and not n.endswith(("A_log", "dt_bias", ".D")) and not (n.endswith("mlp.gate.weight") or "router" in n):
                p.mul_(0.5)                 # four times the width: keep the activations in the same range
    import importlib
    for mod in m.modules():                 # the oracle runs on CPU tensors: its pure-torch paths, not the Triton kernels a GPU box offers
        if hasattr(mod, "chunk_gated_delta_rule"):
            hf = importlib.import_module(type(mod).__module__)
            mod.chunk_gated_delta_rule, mod.recurrent_gated_delta_rule = hf.torch_chunk_gated_delta_rule, hf.torch_recurrent_gated_delta_rule
            mod.causal_conv1d_fn, mod.causal_conv1d_update = None, hf.torch_causal_conv1d_update
            if hasattr(hf, "Qwen3_5MoeRMSNormGated") and not isinstance(mod.norm, hf.Qwen3_5MoeRMSNormGated):
                w = mod.norm.weight.detach().float().cpu()
                mod.norm = hf.Qwen3_5MoeRMSNormGated(w.shape[0], eps=mod.layer_norm_epsilon)
                mod.norm.weight = torch.nn.Parameter(w)
    m = m.cpu().float().eval()
    m16 = copy.deepcopy(m).to(torch.bfloat16)
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file({k: v.detach().contiguous() for k, v in m.state_dict().items()}, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = [type(m).__name__]
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "bf16", "cuda")
    model = og.Model(out)
    ids = np.random.RandomState(0).randint(1, VOCAB - 1, size=(1, 13)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=32)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    seq = ids[0].tolist()
    for _ in range(4):
        with torch.no_grad():
            want = m(torch.tensor([seq])).logits[0, -1].float().numpy()
            own = np.abs(m16(torch.tensor([seq])).logits[0, -1].float().numpy() - want).max()
        got = np.asarray(g.get_logits(), dtype=np.float32).reshape(-1)
        assert np.abs(got - want).max() < max(0.05 * max(1.0, np.abs(want).max()), 3.0 * own), (np.abs(got - want).max(), own)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():
            break
