"""AWQ / GPTQ checkpoints are carried into the MatMulNBits layout without a second quantisation
(reference: src/python/py/models/quantized_model.py:1017-1107)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import create_model, random_state_dict
from onnxruntime_genai_b200.models.quantized_checkpoint import (QuantizedLinear, convert_state_dict, pack_awq, pack_gptq, unpack_awq,
                                                                unpack_gptq)
from dense_reference import logits as dense_logits

ARCH = dict(model_type="llama", vocab_size=96, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=256, context_length=64, bos_token_id=1, eos_token_id=2, pad_token_id=0)


def _random_ql(N, K, group, seed):
    g = torch.Generator().manual_seed(seed)
    r = group // 32
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    s = (torch.rand(N, K // group, generator=g) * 0.02 + 0.002).to(torch.float16).float().repeat_interleave(r, dim=1)
    z = torch.randint(0, 16, (N, K // group), generator=g, dtype=torch.uint8).repeat_interleave(r, dim=1)
    return QuantizedLinear(q, s, z)


@pytest.mark.parametrize("group", [32, 64, 128])
def test_awq_and_gptq_words_round_trip(group):
    ql = _random_ql(48, 256, group, 1)
    a = unpack_awq(*pack_awq(ql, group), group)
    assert torch.equal(a.q, ql.q) and torch.equal(a.zp, ql.zp) and torch.equal(a.scales, ql.scales)
    for off in (0, 1):
        qw, qz, sc, g_idx = pack_gptq(ql, group, off)
        b = unpack_gptq(qw, qz, sc, group, g_idx, off)
        assert torch.equal(b.q, ql.q) and torch.equal(b.zp, ql.zp) and torch.equal(b.scales, ql.scales)
    # the AWQ nibble order: nibble 1 of a word holds column 2
    one = QuantizedLinear(torch.zeros(8, 32, dtype=torch.uint8), torch.ones(8, 1), torch.zeros(8, 1, dtype=torch.uint8))
    one.q[2, 0] = 5
    assert int(pack_awq(one, 32)[0][0, 0]) == 5 << 4
    assert isinstance(unpack_gptq(qw, qz, sc, group, torch.flip(g_idx, [0]), 1), torch.Tensor)    # act-order: a float weight
    with pytest.raises(NotImplementedError):
        convert_state_dict({}, {"quant_method": "awq", "bits": 8})


@pytest.mark.parametrize("method", ["awq", "gptq"])
def test_quantised_hf_checkpoint_exports_without_requantisation(method, tmp_path):
    """A Hugging Face directory with AWQ / GPTQ linears (group 64) -> int4 export -> the loaded model computes with exactly
    the checkpoint's quantised weights: logits equal the dense fp32 model built from the dequantised tensors."""
    from safetensors.torch import save_file
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=11, std=0.1)
    group = 64
    hf, dense, qls = {}, {}, {}
    for i, (k, v) in enumerate(sd.items()):
        if k.endswith("_proj.weight"):
            ql = _random_ql(v.shape[0], v.shape[1], group, 100 + i)
            base = k[: -len(".weight")]
            if method == "awq":
                hf[base + ".qweight"], hf[base + ".qzeros"], hf[base + ".scales"] = pack_awq(ql, group)
            else:
                hf[base + ".qweight"], hf[base + ".qzeros"], hf[base + ".scales"], hf[base + ".g_idx"] = pack_gptq(ql, group)
            dense[k] = ql.float()
            qls[k] = ql
        elif k == "lm_head.weight":
            # not quantised in the checkpoint: the int4 export quantises it (round to nearest, block 32, fp16 scales)
            from onnxruntime_genai_b200.models.builder import dequantize_int4_block32, quantize_int4_block32
            q, sc, zp = quantize_int4_block32(v.float())
            hf[k] = v
            dense[k] = dequantize_int4_block32(q, sc.to(torch.float16).float(), zp, v.shape[0], v.shape[1])
        else:
            hf[k] = v
            dense[k] = v
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file({k: v.contiguous() for k, v in hf.items()}, str(src / "model.safetensors"))
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=96, hidden_size=128, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, max_position_embeddings=64,
               rms_norm_eps=1e-5, rope_theta=10000.0, bos_token_id=1, eos_token_id=2, pad_token_id=0, tie_word_embeddings=False,
               quantization_config={"quant_method": method, "bits": 4, "group_size": group})
    (src / "config.json").write_text(json.dumps(cfg))
    out = str(tmp_path / "out")
    create_model(str(src), out, "int4", "cpu")
    model = og.Model(out)
    # the quantised tensors arrive unchanged: codes, scales and zero points of the packed q / k / v projection and of o
    lw = model.decoder.layers[0]
    pre = "model.layers.0.self_attn."
    for got, names in ((lw.qkv_w, ("q_proj", "k_proj", "v_proj")), (lw.o_w, ("o_proj",))):
        want_q = torch.cat([qls[pre + n + ".weight"].q for n in names], 0)
        want_s = torch.cat([qls[pre + n + ".weight"].scales for n in names], 0)
        want_z = torch.cat([qls[pre + n + ".weight"].zp for n in names], 0)
        assert torch.equal(got._q.cpu().to(torch.uint8), want_q) and torch.equal(got._zp.cpu().to(torch.uint8), want_z)
        np.testing.assert_allclose(got._s.cpu().float().numpy(), want_s.numpy(), rtol=0, atol=0)
    ids = np.random.RandomState(3).randint(3, 96, size=(1, 9)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=16)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    want = dense_logits(model.arch, dense, ids[0].tolist())[-1].numpy()
    # the int4 path rounds the dequantised weights and the activations to bf16: logits agree to that precision
    got = g.get_logits().reshape(-1)
    assert np.abs(got - want).max() < 0.05 * want.std() + 0.02


@pytest.mark.parametrize("fmt", ["fp8", "nvfp4"])
def test_modelopt_checkpoint_is_carried_into_the_block_quantised_ops(fmt, tmp_path):
    """A ModelOpt-style Hugging Face directory (FP8: e4m3 `weight` + `weight_scale`; NVFP4: packed `weight`, e4m3 `weight_scale`
    per block of 16, `weight_scale_2`) exports to MatMulBlockQuantizedFp8Weight / Fp4Weight nodes holding the checkpoint's
    own codes; logits equal the dense model on the dequantised weights."""
    from safetensors.torch import save_file
    from onnxruntime_genai_b200.models.builder import dequantize_nvfp4, quantize_fp8_rows, quantize_nvfp4
    from onnxruntime_genai_b200.utils import onnx_proto as op
    arch = ArchConfig(**ARCH)
    sd = random_state_dict(arch, seed=31, std=0.1)
    hf, dense = {}, {}
    for k, v in sd.items():
        if k.endswith("_proj.weight"):
            base = k[: -len(".weight")]
            if fmt == "fp8":
                q8, sc = quantize_fp8_rows(v)
                hf[k], hf[base + ".weight_scale"] = q8.view(torch.float8_e4m3fn), sc.reshape(-1)
                hf[base + ".input_scale"] = torch.tensor(1.0)
                dense[k] = q8.view(torch.float8_e4m3fn).float() * sc
            else:
                # one global scale for every projection (stacked q / k / v must share it to be carried over)
                wf = v.float()
                glob = torch.tensor(0.1 * 4 / (6.0 * 448.0))
                sc8 = (wf.view(v.shape[0], -1, 16).abs().amax(-1) / 6.0 / glob).to(torch.float8_e4m3fn)
                codes, _, _ = quantize_nvfp4(v)          # reference packing helper, re-done below with the shared global
                eff = (sc8.float() * glob).clamp(min=1e-20)
                grid = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
                vv = (wf.view(v.shape[0], -1, 16) / eff[..., None]).clamp(-6, 6)
                idx = (vv.abs()[..., None] - grid).abs().argmin(-1)
                c = (idx + 8 * ((vv < 0) & (idx > 0)).long()).to(torch.uint8).view(v.shape)
                packed = (c[:, 0::2] | (c[:, 1::2] << 4)).contiguous()
                hf[k], hf[base + ".weight_scale"], hf[base + ".weight_scale_2"] = packed, sc8, glob.reshape(())
                dense[k] = dequantize_nvfp4(packed, sc8.view(torch.uint8), glob.reshape(1))
        else:
            hf[k] = v
            dense[k] = v
    src = tmp_path / "hf"
    os.makedirs(src)
    save_file({k: v.contiguous() for k, v in hf.items()}, str(src / "model.safetensors"))
    cfg = dict(architectures=["LlamaForCausalLM"], model_type="llama", vocab_size=96, hidden_size=128, num_hidden_layers=2,
               num_attention_heads=4, num_key_value_heads=2, head_dim=32, intermediate_size=256, max_position_embeddings=64,
               rms_norm_eps=1e-5, rope_theta=10000.0, bos_token_id=1, eos_token_id=2, pad_token_id=0, tie_word_embeddings=False,
               quantization_config={"quant_method": "modelopt", "quant_algo": fmt.upper()})
    (src / "config.json").write_text(json.dumps(cfg))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    ops_seen = {n.op_type for n in op.LoadedModel(os.path.join(out, "model.onnx")).model.nodes}
    assert ("MatMulBlockQuantizedFp8Weight" if fmt == "fp8" else "MatMulBlockQuantizedFp4Weight") in ops_seen
    model = og.Model(out)
    ids = np.random.RandomState(3).randint(3, 96, size=(1, 9)).astype(np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=16)
    g = og.Generator(model, p)
    g.append_tokens(ids)
    want = dense_logits(model.arch, dense, ids[0].tolist())[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)


def test_int4_methods_and_mixed_precision_placement(tmp_path):
    """`default` / `rtn` / `k_quant` and the int8 placements of the reference's builder (builders/quant_config.py:168-173,
    285-290; builders/base.py:1211-1254): k_quant lowers the weighted block error, `k_quant_mixed` writes 8-bit MatMulNBits
    nodes for the LM head and the promoted layers' qkv / down projections, and the promoted export tracks the float model
    more closely than the plain int4 one."""
    import copy
    import numpy as np
    import onnxruntime_genai_b200 as og
    from dense_reference import logits as dense_logits
    from onnxruntime_genai_b200.models.arch import ArchConfig
    from onnxruntime_genai_b200.models.builder import (dequantize_block, export_model, mixed_precision_layers, quantize_block,
                                                      random_state_dict)
    from onnxruntime_genai_b200.utils.onnx_proto import decode_model

    torch.manual_seed(0)
    w = torch.randn(96, 256) * 0.05
    w[:, ::29] *= 5
    wt = (w.view(96, 8, 32).abs() + w.view(96, 8, 32).pow(2).mean(-1, keepdim=True).sqrt()).view(96, 256)
    for bits in (4, 8):
        err = {}
        for method in ("default", "rtn", "k_quant"):
            q, s, zp = quantize_block(w, bits, False, method)
            assert q.shape == (96, 8, 16 if bits == 4 else 32)
            err[method] = float((wt * (dequantize_block(q, s, zp, 96, 256, 32, bits) - w) ** 2).sum())
        assert err["rtn"] == err["default"] and err["k_quant"] < err["default"]
    with pytest.raises(ValueError):
        quantize_block(w, 4, False, "gptq")
    assert mixed_precision_layers(8) == [0, 3, 6, 7] and mixed_precision_layers(32)[:5] == [0, 1, 2, 3, 6]

    arch = ArchConfig(model_type="llama", vocab_size=160, hidden_size=64, num_layers=8, num_heads=4, num_kv_heads=2, head_dim=16,
                      intermediate_size=128, context_length=64, bos_token_id=0, eos_token_id=1, pad_token_id=1)
    sd = random_state_dict(arch, seed=3, std=0.08)
    prompt = np.random.RandomState(1).randint(2, 160, size=12).tolist()
    want = dense_logits(arch, sd, prompt)[-1].numpy()
    errs = {}
    for algo in ("default", "k_quant_mixed"):
        d = str(tmp_path / algo)
        export_model(copy.deepcopy(arch), d, "int4", "cpu", state_dict=sd, int4_algo_config=algo)
        nodes = {n.name: n for n in decode_model(open(os.path.join(d, "model.onnx"), "rb").read()).nodes if n.op_type == "MatMulNBits"}
        eight = sorted(name for name, n in nodes.items() if int(n.attrs["bits"]) == 8)
        if algo == "default":
            assert not eight
        else:
            assert "/lm_head/MatMul_Q8" in eight
            assert {f"/model/layers.{i}/attn/qkv_proj/MatMul_Q8" for i in (0, 3, 6, 7)} <= set(eight)
            assert {f"/model/layers.{i}/mlp/down_proj/MatMul_Q8" for i in (0, 3, 6, 7)} <= set(eight)
            assert "/model/layers.1/attn/qkv_proj/MatMul_Q8" not in eight and "/model/layers.0/mlp/gate_up_proj/MatMul_Q8" not in eight
        model = og.Model(d)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=32)
        g = og.Generator(model, p)
        g.append_tokens(np.asarray([prompt], dtype=np.int32))
        errs[algo] = float(np.abs(g.get_logits().reshape(-1) - want).mean())
    assert errs["k_quant_mixed"] < errs["default"]
    with pytest.raises(ValueError):
        export_model(copy.deepcopy(arch), str(tmp_path / "bad"), "int4", "cpu", state_dict=sd, int4_algo_config="awq_last")


def test_gptq_act_order_quark_and_olive_layouts():
    """GPTQ with a permuted g_idx (desc_act) is reconstructed exactly as a float weight; a Quark checkpoint's dense layers read
    like AWQ; Olive's [N, K/2] bytes carry over unchanged (reference: quantized_model.py GPTQModel / QuarkModel / OliveModel)."""
    from onnxruntime_genai_b200.models.quantized_checkpoint import unpack_olive
    g = torch.Generator().manual_seed(4)
    K, N, group = 128, 16, 32
    q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
    scales = torch.rand(N, K // 32, generator=g) * 0.02 + 0.001
    zp = torch.randint(0, 16, (N, K // 32), generator=g, dtype=torch.uint8)
    ql = QuantizedLinear(q, scales, zp)
    # ---- GPTQ act-order: the same tensors, but feature k is stored at position perm[k] with its group recorded in g_idx
    qweight, qzeros, sc, _ = pack_gptq(ql, group)
    perm = torch.randperm(K, generator=g)
    g_idx = (perm // group).to(torch.int32)                       # position p holds feature perm[p], whose group is perm[p] // group
    q_perm = q[:, perm]                                           # columns reordered the way an act-order file stores them
    qw_perm = pack_gptq(QuantizedLinear(q_perm.contiguous(), scales, zp), group)[0]
    sd = {"l.qweight": qw_perm, "l.qzeros": qzeros, "l.scales": sc, "l.g_idx": g_idx, "other": torch.ones(2)}
    out = convert_state_dict(sd, {"quant_method": "gptq", "bits": 4, "group_size": group, "desc_act": True})
    w = out["l.weight"]
    assert isinstance(w, torch.Tensor) and tuple(w.shape) == (N, K)
    torch.testing.assert_close(w, ql.float()[:, perm], rtol=1e-3, atol=1e-5)       # exact up to the fp16 scales of the file
    # ---- Quark: AWQ packing under another method name
    aw, az, asc = pack_awq(ql, group)
    got = convert_state_dict({"l.qweight": aw, "l.qzeros": az, "l.scales": asc}, {"quant_method": "quark", "bits": 4, "group_size": group})["l.weight"]
    assert torch.equal(got.q, q) and torch.equal(got.zp, zp)
    # ---- Olive: [N, K/2] bytes, low nibble first, zero points packed likewise, a per-layer group size override
    ob = (q[:, 0::2] | (q[:, 1::2] << 4)).contiguous()
    oz = (zp[:, 0::2] | (zp[:, 1::2] << 4)).contiguous()
    ol = unpack_olive(ob, oz, scales, 32)
    assert torch.equal(ol.q, q) and torch.equal(ol.zp, zp) and torch.equal(ol.scales, scales)
    got = convert_state_dict({"m.qweight": ob, "m.qzeros": oz, "m.scales": scales},
                             {"quant_method": "olive", "bits": 4, "group_size": 128, "overrides": {"m": {"group_size": 32}}})["m.weight"]
    torch.testing.assert_close(got.float(), ql.float())
    with pytest.raises(NotImplementedError):
        convert_state_dict({"m.qweight": ob, "m.scales": scales}, {"quant_method": "olive", "bits": 4, "group_size": 32, "overrides": {"m": {"bits": 8}}})
