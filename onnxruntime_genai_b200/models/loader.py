"""Checkpoint loader: `genai_config.json` + ONNX graph + external data -> DecoderModel.

The ONNX file is read as a weight container plus architecture descriptor.  Structure is recovered
from node names / op types / attributes (the naming contract of the reference builder, see
builder.py in this package), weights from the initializers that those nodes name as inputs, so a
checkpoint with separate q/k/v projections, packed qkv, float MatMul or MatMulNBits int4 weights
loads through the same code.  MatMul initializers are stored `[in, out]` and are transposed to the
K-major `[out, in]` layout that the tcgen05 GEMM consumes; tensor-parallel ranks keep only their
shard (attention heads / MLP columns / vocabulary rows).
"""
from __future__ import annotations

import json
import math
import os
import re
from typing import Dict, List, Optional

import numpy as np
import torch

from ..utils import onnx_proto as op
from .arch import ArchConfig
from .builder import dequantize_block, dequantize_int4_block32, dequantize_mxfp4, quantize_int4_block32, random_tensor, tensor_seed, weight_shapes
from .decoder import DecoderModel, LayerWeights


def _np_to_torch(arr: np.ndarray, onnx_dtype: int) -> torch.Tensor:
    if onnx_dtype == op.BFLOAT16:
        return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)
    return torch.from_numpy(np.array(arr, copy=True))


class GraphView:
    """Name-indexed access to nodes and initializers of a loaded ONNX model."""

    def __init__(self, path: str, seed_device="cpu"):
        self.lm = op.LoadedModel(path)
        self.nodes = self.lm.model.nodes
        self.by_name = {n.name: n for n in self.nodes}
        self.device = seed_device

    def find(self, prefix: str, contains: str = "", ops: Optional[List[str]] = None):
        for n in self.nodes:
            if n.name.startswith(prefix) and contains in n.name and (ops is None or n.op_type in ops):
                return n
        return None

    def find_all(self, prefix: str, ops: Optional[List[str]] = None):
        return [n for n in self.nodes if n.name.startswith(prefix) and (ops is None or n.op_type in ops)]

    def has_init(self, name: str) -> bool:
        return bool(name) and self.lm.has(name)

    def tensor(self, name: str, device="cpu") -> torch.Tensor:
        t = self.lm.info(name)
        if t.ext_location and t.ext_location.startswith("synthetic:"):
            return self._synthetic(t, json.loads(t.ext_location[len("synthetic:"):]), device)
        return _np_to_torch(self.lm.array(name), t.dtype)

    def _synthetic(self, t: op.Tensor, meta: dict, device) -> torch.Tensor:
        if meta["op"] in ("fp4_codes", "fp4_scales"):
            # MXFP4 experts: uniform random e2m1 codes; block scales 2^-8 .. 2^-5 (weights of the usual magnitude)
            gen = torch.Generator(device=device)
            gen.manual_seed(tensor_seed(meta["sources"][0] + "." + meta["op"], meta["seed"]))
            lo, hi = (0, 256) if meta["op"] == "fp4_codes" else (119, 123)
            return torch.randint(lo, hi, tuple(meta["shape"]), generator=gen, device=device, dtype=torch.uint8)
        parts = []
        shapes = self._shapes
        for src in meta["sources"]:
            parts.append(random_tensor(src, shapes[src], meta["seed"], meta["std"], device=device))
        x = parts[0] if len(parts) == 1 else torch.cat(parts, 0)
        if meta["op"].startswith("q4_"):
            # the three tensors of one MatMulNBits node come from one quantisation of the same float weight
            key = tuple(meta["sources"])
            cache = getattr(self, "_q4_cache", None)
            if cache is None or cache[0] != key:
                q, sc, zp = quantize_int4_block32(x.float(), symmetric=bool(meta.get("symmetric", 0)))
                cache = self._q4_cache = (key, {"q4_weight": q, "q4_scales": sc.reshape(-1).to(torch.float16), "q4_zp": zp})
            return cache[1][meta["op"]]
        if meta["op"] == "cat_t":
            x = x.t()
        if meta.get("offset"):
            x = x + meta["offset"]
        return x

    def set_arch_shapes(self, arch: ArchConfig):
        self._shapes = weight_shapes(arch)


def _attr(node, name, default=None):
    return node.attrs.get(name, default) if node is not None else default


def arch_from_checkpoint(cfg, g: GraphView, decoder: Optional[dict] = None) -> ArchConfig:
    """Rebuilds the architecture description from genai_config.json and the graph."""
    d = decoder or cfg.decoder
    L = d["num_hidden_layers"]
    a = ArchConfig(model_type=cfg.model_type, vocab_size=cfg.vocab_size, hidden_size=d["hidden_size"], num_layers=L,
                   num_heads=d["num_attention_heads"], num_kv_heads=d["num_key_value_heads"] or d["num_attention_heads"],
                   head_dim=d["head_size"], context_length=cfg.context_length, bos_token_id=cfg.bos_token_id,
                   eos_token_id=list(cfg.eos_token_ids), pad_token_id=cfg.pad_token_id)
    first_norm = g.find("/model/layers.0/input_layernorm/")
    if first_norm is not None:
        a.norm_eps = float(_attr(first_norm, "epsilon", 1e-5))
        a.layernorm = "Simplified" not in first_norm.op_type
        a.pre_norm = not bool(int(_attr(first_norm, "bypass", 0) or 0))
    # the first layer that attends (hybrid models may start with convolution layers)
    fa = next((i for i in range(L) if g.find(f"/model/layers.{i}/attn/", ops=["GroupQueryAttention", "PagedAttention"]) is not None), 0)
    fa = f"/model/layers.{fa}"
    attn = g.find(f"{fa}/attn/", ops=["GroupQueryAttention", "PagedAttention", "MultiHeadAttention"])
    if attn is not None:
        a.attn_scale = float(_attr(attn, "scale", 0.0)) or None
        a.softcap = float(_attr(attn, "softcap", 0.0) or 0.0)
        a.rotary_interleaved = bool(_attr(attn, "rotary_interleaved", 0))
        rd = _attr(attn, "rotary_embedding_dim", 0)
        if rd:
            a.partial_rotary_factor = rd / a.head_dim
        a.qk_norm = "qk_norm_epsilon" in attn.attrs
        a.qk_norm_after_rope = bool(int(_attr(attn, "qk_norm_after_rotary", 0) or 0))
        a.qk_norm_full_width = bool(int(_attr(attn, "qk_norm_full_width", 0) or 0))
        ms = _attr(attn, "mrope_section")
        a.mrope_section = [int(v) for v in ms] if ms else None
        a.mrope_interleaved = bool(int(_attr(attn, "mrope_interleaved", 0) or 0))
        a.attn_sinks = any(".sinks" in i for i in attn.inputs)
    windows, unrotated = [], []
    for i in range(L):
        n = g.find(f"/model/layers.{i}/attn/", ops=["GroupQueryAttention", "PagedAttention"])
        w = int(_attr(n, "local_window_size", -1) or -1)
        windows.append(w if w > 0 else 0)
        if n is not None and int(_attr(n, "do_rotary", 1)) == 0:
            unrotated.append(i)
    attending = [i for i in range(L) if g.find(f"/model/layers.{i}/attn/", ops=["GroupQueryAttention", "PagedAttention"]) is not None]
    if unrotated and len(unrotated) < len(attending):
        a.no_rope_layers = unrotated
    if g.has_init("cos_cache_local"):
        a.rope_local_theta = 1.0       # the local caches are read from the model; only the switch matters here
    if any(windows):
        a.sliding_window = max(windows)
        a.sliding_layers = None if all(windows) else [i for i, w in enumerate(windows) if w > 0]
    a.attn_bias = g.find(f"{fa}/attn/", "_proj/Add") is not None and \
        any(n.name.endswith(("qkv_proj/Add", "q_proj/Add")) for n in g.find_all(f"{fa}/attn/"))
    a.o_bias = g.by_name.get(f"{fa}/attn/o_proj/Add") is not None
    a.post_sublayer_norms = g.find("/model/layers.0/post_feedforward_layernorm/") is not None
    types = ["conv" if g.find(f"/model/layers.{i}/conv/in_proj/", ops=LINEAR_OPS) is not None else
             ("linear_attention" if g.by_name.get(f"/model/layers.{i}/linear_attn/LinearAttention") is not None else
              ("mamba" if g.by_name.get(f"/model/layers.{i}/mamba/Mamba2") is not None else "full_attention"))
             for i in range(a.num_layers)]
    if "mamba" in types:
        a.layer_types = types
        mb = g.by_name[f"/model/layers.{types.index('mamba')}/mamba/Mamba2"]
        a.mamba_num_heads, a.mamba_head_dim = int(mb.attrs["num_heads"]), int(mb.attrs["head_dim"])
        a.mamba_state_size, a.mamba_n_groups = int(mb.attrs["state_size"]), int(mb.attrs["n_groups"])
        a.mamba_conv_kernel = int(g.lm.info(f"model.layers.{types.index('mamba')}.mamba.conv1d.weight").dims[-1])
    if "linear_attention" in types:
        a.layer_types = types
        la = g.by_name[f"/model/layers.{types.index('linear_attention')}/linear_attn/LinearAttention"]
        a.linear_num_key_heads, a.linear_num_value_heads = int(la.attrs["q_num_heads"]), int(la.attrs["kv_num_heads"])
        a.linear_key_head_dim, a.linear_value_head_dim = int(la.attrs["key_head_dim"]), int(la.attrs["value_head_dim"])
        a.linear_conv_kernel_dim = int(g.lm.info(f"model.layers.{types.index('linear_attention')}.linear_attn.conv1d.weight").dims[-1])
    if "conv" in types:
        a.layer_types = types
        first = types.index("conv")
        taps = g.lm.info(f"model.layers.{first}.conv.conv.weight").dims
        a.conv_L_cache = int(taps[-1])
        a.conv_bias = g.has_init(f"model.layers.{first}.conv.conv.bias")
    a.cross_attention = g.find("/model/layers.0/cross_attn/") is not None
    if a.cross_attention:
        a.encoder_hidden_size = _linear_shape(g, g.find("/model/layers.0/cross_attn/kv_proj/", ops=LINEAR_OPS))[1]
    a.parallel_block = g.find("/model/layers.0/parallel_block/") is not None
    a.learned_positions = g.by_name.get("/model/pos_embed/Gather") is not None
    a.no_rope = (not a.learned_positions and attn is not None and attn.op_type in ("GroupQueryAttention", "PagedAttention")
                 and int(_attr(attn, "do_rotary", 1)) == 0 and a.no_rope_layers is None)
    fc1 = g.find("/model/layers.0/mlp/fc1/", ops=LINEAR_OPS)
    if fc1 is not None:
        a.mlp_gated = False
        a.intermediate_size = _linear_shape(g, fc1)[0]
        a.mlp_bias = g.by_name.get("/model/layers.0/mlp/fc1/Add") is not None
    moe = g.find("/model/layers.0/moe/", ops=["MoE", "QMoE"])
    if moe is not None:
        a.experts_per_token = int(_attr(moe, "k", 1))
        a.moe_swiglu_alpha = float(_attr(moe, "activation_alpha", 1.702))
        a.moe_swiglu_limit = float(_attr(moe, "swiglu_limit", 7.0))
        wname = moe.inputs[2]
        shp = g.lm.info(wname).dims
        a.num_experts = shp[0]
        if moe.op_type == "MoE" and int(_attr(moe, "swiglu_fusion", 0)) == 0 and len(moe.inputs) > 6 and moe.inputs[6]:
            # three expert matrices (gate, down, up), silu(gate) * up, no biases
            a.moe_style = "standard"
            a.moe_norm_topk = bool(int(_attr(moe, "normalize_routing_weights", 0)))
            a.moe_sparse_mixer = bool(int(_attr(moe, "use_sparse_mixer", 0)))
            a.moe_jitter_eps = float(_attr(moe, "sparse_mixer_jitter_eps", 0.01))
            a.intermediate_size = shp[1]
            a.mlp_bias = False
        else:
            # MoE weight [E, 2I, H]; QMoE MXFP4 codes [E, H, (2I)/2]
            a.intermediate_size = shp[2] if moe.op_type == "QMoE" else shp[1] // 2
            a.mlp_bias = True
    else:
        gu = g.find("/model/layers.0/mlp/gate_up_proj/", ops=LINEAR_OPS)
        if gu is not None:
            a.intermediate_size = _linear_shape(g, gu)[0] // 2
        else:
            gp = g.find("/model/layers.0/mlp/gate_proj/", ops=LINEAR_OPS)
            if gp is not None:
                a.intermediate_size = _linear_shape(g, gp)[0]
        if fc1 is None:
            a.mlp_bias = g.find("/model/layers.0/mlp/down_proj/Add") is not None
        act = g.find("/model/layers.0/mlp/act_fn/", ops=["FastGelu", "Gelu", "BiasGelu", "Relu"])
        a.activation = "silu" if act is None else {"Gelu": "gelu_erf", "Relu": "relu"}.get(act.op_type, "gelu") if fc1 is not None else "gelu"
        if a.activation == "relu" and g.by_name.get("/model/layers.0/mlp/act_fn/Square") is not None:
            a.activation = "relu2"
    if g.by_name.get("/model/embed_tokens/Mul") is not None:
        a.embed_scale = float(g.tensor("/model/constants/embed_scale").float().item())
    if g.has_init("/model/constants/residual_multiplier"):
        a.residual_multiplier = float(g.tensor("/model/constants/residual_multiplier").float().item())
    if g.by_name.get("/lm_head/Mul") is not None:
        a.logits_scale = float(g.tensor("/model/constants/logits_scale").float().item())
    sc = g.by_name.get("/lm_head/softcap")
    if sc is not None:
        a.final_logit_softcap = float(_attr(sc, "softcap", 0.0))
    a.lm_head_bias = g.by_name.get("/lm_head/Add") is not None
    return a


LINEAR_OPS = ["MatMul", "MatMulNBits", "MatMulBlockQuantizedFp8Weight", "MatMulBlockQuantizedFp4Weight"]


def _linear_shape(g: GraphView, node):
    """(N, K) of a linear node."""
    if node.op_type == "MatMulNBits":
        return int(node.attrs["N"]), int(node.attrs["K"])
    if node.op_type == "MatMulBlockQuantizedFp8Weight":
        n, k = g.lm.info(node.inputs[1]).dims
        return n, k
    if node.op_type == "MatMulBlockQuantizedFp4Weight":
        n, k2 = g.lm.info(node.inputs[1]).dims
        return n, 2 * k2
    k, n = g.lm.info(node.inputs[1]).dims
    return n, k


def _linear_weight(g: GraphView, node, dtype, device, rows: Optional[slice] = None, cols: Optional[slice] = None) -> torch.Tensor:
    """Weight of a linear node as [N, K] (optionally a row/column shard), on `device`."""
    if node.op_type == "MatMulNBits":
        N, K = int(node.attrs["N"]), int(node.attrs["K"])
        bs = int(node.attrs.get("block_size", 32))
        bits = int(node.attrs.get("bits", 4))
        if bits not in (4, 8):
            raise NotImplementedError("MatMulNBits: only 4- and 8-bit weights are supported")
        loc = g.lm.info(node.inputs[1]).ext_location or ""
        src_dev = device if loc.startswith("synthetic:") else "cpu"
        q = g.tensor(node.inputs[1], device=src_dev)
        s = g.tensor(node.inputs[2], device=src_dev)
        zp = g.tensor(node.inputs[3], device=src_dev) if len(node.inputs) > 3 and node.inputs[3] else None
        # 8-bit nodes (the promoted ones of a mixed-precision export) are expanded to the compute type at load
        w = dequantize_int4_block32(q, s, zp, N, K, bs) if bits == 4 else dequantize_block(q, s, zp, N, K, bs, 8)
    elif node.op_type == "MatMulBlockQuantizedFp8Weight":
        # FP8 e4m3 weight [N, K] with one fp32 scale per output row (or one for the matrix), expanded at load: the GEMMs run
        # in bf16 on the dequantised weight; the optional activation scale (input 3) is not used
        # (reference: src/python/py/models/builders/base.py:1878-1917)
        w8 = g.tensor(node.inputs[1]).view(torch.float8_e4m3fn).float()
        w = w8 * g.tensor(node.inputs[2]).float().reshape(-1, 1)
    elif node.op_type == "MatMulBlockQuantizedFp4Weight":
        # NVFP4: e2m1 codes [N, K/2] (low nibble = even k), e4m3 scale per block of 16 [N, K/16], one fp32 global scale
        # (reference: src/python/py/models/builders/base.py:1919-1949); expanded at load
        from .builder import dequantize_nvfp4
        w = dequantize_nvfp4(g.tensor(node.inputs[1]), g.tensor(node.inputs[2]), g.tensor(node.inputs[3]))
    else:
        w = g.tensor(node.inputs[1], device=device if g.lm.info(node.inputs[1]).ext_location and
                     g.lm.info(node.inputs[1]).ext_location.startswith("synthetic:") else "cpu").t()
    if rows is not None:
        w = w[rows]
    if cols is not None:
        w = w[:, cols]
    return w.to(device=device, dtype=dtype).contiguous()


def _is_q4(nodes) -> bool:
    return all(n is not None and n.op_type == "MatMulNBits" and int(n.attrs.get("bits", 4)) == 4 and
               int(n.attrs.get("block_size", 32)) == 32 and int(n.attrs["K"]) % 64 == 0 for n in nodes)


def _q4_weight(g: GraphView, nodes, device, interleave: bool = False):
    """One W4Weight from one or more MatMulNBits nodes stacked along N (kept in int4 for the dequant GEMM)."""
    from ..ops.w4 import W4Weight, unpack_ort_q4
    qs, ss, zs = [], [], []
    synthetic = False
    for n in nodes:
        N, K = int(n.attrs["N"]), int(n.attrs["K"])
        loc = g.lm.info(n.inputs[1]).ext_location or ""
        synthetic = synthetic or loc.startswith("synthetic:")
        src_dev = device if loc.startswith("synthetic:") else "cpu"     # synthetic weights are drawn and quantised on the device
        has_zp = len(n.inputs) > 3 and n.inputs[3]
        q, zp = unpack_ort_q4(g.tensor(n.inputs[1], device=src_dev), g.tensor(n.inputs[3], device=src_dev) if has_zp else None, N, K)
        qs.append(q)
        ss.append(g.tensor(n.inputs[2], device=src_dev).float().view(N, K // 32))
        zs.append(zp if zp is not None else torch.full((N, K // 32), 8, dtype=torch.uint8, device=q.device))
    q, s, z = torch.cat(qs, 0), torch.cat(ss, 0), torch.cat(zs, 0)
    if interleave:
        from ..ops import interleave_gate_up
        q, s, z = interleave_gate_up(q), interleave_gate_up(s), interleave_gate_up(z)
    if synthetic and torch.device(device).type == "cuda":   # no second copy of a weight that was generated on the device
        return W4Weight.from_quantized(q, s, z, device, keep_host=False, interleaved=interleave)
    return W4Weight.from_quantized(q, s, z, device, interleaved=interleave)


def _vec(g: GraphView, name: str, dtype, device, sl: Optional[slice] = None) -> Optional[torch.Tensor]:
    if not g.has_init(name):
        return None
    t = g.tensor(name)
    if sl is not None:
        t = t[sl]
    return t.to(device=device, dtype=dtype).contiguous()


def load_decoder(model_dir: str, cfg, device, dtype, tp=None, decoder: Optional[dict] = None) -> DecoderModel:
    d = decoder or cfg.decoder
    g = GraphView(os.path.join(model_dir, d["filename"]))
    arch = arch_from_checkpoint(cfg, g, d)
    g.set_arch_shapes(arch)
    model = DecoderModel(arch, device, dtype, tp)
    tpn, tpr = model.tp.size, model.tp.rank
    # int4 MatMulNBits weights stay int4 (dequant GEMM) on a single GPU; tensor-parallel shards are dequantised to bf16
    keep_q4 = tpn == 1 and os.environ.get("OGB_DEQUANT_INT4_AT_LOAD", "0") != "1"
    if arch.num_heads % tpn or (arch.num_kv_heads % tpn and tpn % arch.num_kv_heads):
        raise ValueError(f"tensor parallel degree {tpn} does not divide the attention heads")
    if arch.num_kv_heads < tpn:
        raise NotImplementedError("tensor parallel degree larger than the number of KV heads")
    Hq, Hkv, D, I = arch.num_heads, arch.num_kv_heads, arch.head_dim, arch.intermediate_size
    hq_l, hkv_l, i_l = Hq // tpn, Hkv // tpn, I // tpn
    q_rows = slice(tpr * hq_l * D, (tpr + 1) * hq_l * D)
    k_rows = slice(Hq * D + tpr * hkv_l * D, Hq * D + (tpr + 1) * hkv_l * D)
    v_rows = slice(Hq * D + Hkv * D + tpr * hkv_l * D, Hq * D + Hkv * D + (tpr + 1) * hkv_l * D)

    def linear_node(prefix: str, *names):
        for nm in names:
            n = g.find(prefix + nm + "/", ops=LINEAR_OPS)
            if n is not None:
                return n
        return None

    def shard_rows(w: torch.Tensor, slices) -> torch.Tensor:
        return torch.cat([w[s] for s in slices], 0).contiguous() if tpn > 1 else w

    gq = g.by_name.get("/model/embed_tokens/GatherBlockQuantized")
    if gq is not None:
        # Tied quantised embedding: the rows of the int4 LM-head weight (through a Reshape to [vocab, hidden / 2] bytes).  On a
        # CUDA device the table stays int4 and rows are dequantised as they are gathered; elsewhere it is expanded once.
        from ..ops.w4 import QuantizedEmbedding
        rs = g.by_name[gq.inputs[0].rsplit("/", 1)[0]] if gq.inputs[0].endswith("/output_0") else None
        wname = rs.inputs[0] if rs is not None else gq.inputs[0]
        V, Kh = arch.vocab_size, arch.hidden_size
        has_zp = len(gq.inputs) > 3 and gq.inputs[3]
        qe = QuantizedEmbedding(g.tensor(wname, device=device).reshape(V, Kh // 2).to(device), g.tensor(gq.inputs[2], device=device).to(device).view(V, -1),
                                g.tensor(gq.inputs[3], device=device).to(device).view(V, -1) if has_zp else None, V, Kh)
        model.embed = qe if torch.device(device).type == "cuda" else qe.dequantize(dtype).contiguous()
    else:
        emb = g.tensor("model.embed_tokens.weight", device=device)
        model.embed = emb.to(device=device, dtype=dtype).contiguous()
    cos, sin = g.tensor("cos_cache").float(), g.tensor("sin_cache").float()
    model.cos, model.sin = cos.to(device).contiguous(), sin.to(device).contiguous()
    if g.has_init("cos_cache_local"):
        model.cos_local = g.tensor("cos_cache_local").float().to(device).contiguous()
        model.sin_local = g.tensor("sin_cache_local").float().to(device).contiguous()
    if arch.learned_positions:
        model.pos_embed = g.tensor("model.position_embeddings.weight", device=device).to(device=device, dtype=dtype).contiguous()
    if g.has_init("cos_cache_small") and g.has_init("cos_cache_large"):
        # long-context RoPE: short-factor caches up to the original context length, long-factor caches beyond
        model.rope_original_context = int(g.tensor("/model/rope_caches_subgraph/original_context_length").item())
        model.cos_small = g.tensor("cos_cache_small").float().to(device).contiguous()
        model.sin_small = g.tensor("sin_cache_small").float().to(device).contiguous()
        model.cos, model.sin = g.tensor("cos_cache_large").float().to(device).contiguous(), g.tensor("sin_cache_large").float().to(device).contiguous()

    for i in range(arch.num_layers):
        p, n = f"model.layers.{i}.", f"/model/layers.{i}"
        ln1 = g.find(f"{n}/input_layernorm/")
        mid = "pre_feedforward_layernorm" if arch.post_sublayer_norms else "post_attention_layernorm"
        ln2 = g.find(f"{n}/{mid}/")
        w_idx1 = 1 if ln1.op_type in ("SimplifiedLayerNormalization", "LayerNormalization") else 2
        lw = LayerWeights(
            ln1_w=_vec(g, ln1.inputs[w_idx1], dtype, device),
            ln1_b=_vec(g, ln1.inputs[w_idx1 + 1], dtype, device) if arch.layernorm and len(ln1.inputs) > w_idx1 + 1 else None,
            ln2_w=_vec(g, ln2.inputs[2], dtype, device) if ln2 is not None else None,      # parallel blocks have one norm
            ln2_b=_vec(g, ln2.inputs[3], dtype, device) if ln2 is not None and arch.layernorm and len(ln2.inputs) > 3 else None,
            qkv_w=None, o_w=None, window=arch.layer_window(i))
        conv_in = linear_node(f"{n}/conv/", "in_proj")
        if conv_in is not None:
            # hybrid (LFM2) convolution layer: channels are independent, so tensor parallelism splits them - in_proj rows of
            # this rank's channels of b, c and x, the matching taps, out_proj columns
            C = arch.hidden_size
            c_l = C // tpn
            ch = slice(tpr * c_l, (tpr + 1) * c_l)
            if tpn > 1:
                lw.conv_in_w = torch.cat([_linear_weight(g, conv_in, dtype, device, rows=slice(j * C + ch.start, j * C + ch.stop))
                                          for j in range(3)], 0).contiguous()
            else:
                lw.conv_in_w = _linear_weight(g, conv_in, dtype, device)
            taps = g.tensor(f"model.layers.{i}.conv.conv.weight").reshape(C, -1)
            lw.conv_w = (taps[ch] if tpn > 1 else taps).to(device=device, dtype=dtype).contiguous()
            if g.has_init(f"model.layers.{i}.conv.conv.bias"):
                lw.conv_b = _vec(g, f"model.layers.{i}.conv.conv.bias", dtype, device, ch if tpn > 1 else None)
            lw.conv_out_w = _linear_weight(g, linear_node(f"{n}/conv/", "out_proj"), dtype, device, cols=ch if tpn > 1 else None)
        elif arch.is_mamba_layer(i):
            if tpn > 1:
                raise NotImplementedError("Mamba layers are not sharded: run these models on one GPU")
            mb = f"{n}/mamba/"
            lw.mamba_in_w = _linear_weight(g, linear_node(mb, "in_proj"), dtype, device)
            lw.mamba_conv_w = g.tensor(f"model.layers.{i}.mamba.conv1d.weight").reshape(arch.mamba_conv_dim, -1).to(device=device, dtype=dtype).contiguous()
            lw.mamba_conv_b = _vec(g, f"model.layers.{i}.mamba.conv1d.bias", dtype, device)
            lw.mamba_dt_bias = g.tensor(f"model.layers.{i}.mamba.dt_bias").float().to(device)
            lw.mamba_neg_a = g.tensor(f"model.layers.{i}.mamba.neg_exp_A").float().to(device)
            lw.mamba_d = g.tensor(f"model.layers.{i}.mamba.D").float().to(device)
            lw.mamba_norm_w = g.tensor(f"model.layers.{i}.mamba.norm.weight").float().to(device)
            lw.mamba_out_w = _linear_weight(g, linear_node(mb, "out_proj"), dtype, device)
        elif arch.is_linear_layer(i):
            # gated-delta-net layer: four input projections stacked into one GEMM [qkv | z | b | a], the depthwise taps, the gate
            # constants, the per-head norm weight, the output projection
            if tpn > 1:
                raise NotImplementedError("linear-attention (gated delta net) layers are not sharded: run these models on one GPU")
            la = f"{n}/linear_attn/"
            lw.lin_in_w = torch.cat([_linear_weight(g, linear_node(la, nm), dtype, device) for nm in ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a")], 0).contiguous()
            lw.lin_conv_w = g.tensor(f"model.layers.{i}.linear_attn.conv1d.weight").reshape(arch.linear_conv_dim, -1).to(device=device, dtype=dtype).contiguous()
            lw.lin_dt_bias = g.tensor(f"model.layers.{i}.linear_attn.dt_bias").float().to(device)
            lw.lin_neg_exp_a = g.tensor(f"model.layers.{i}.linear_attn.neg_exp_A").float().to(device)
            lw.lin_norm_w = g.tensor(f"model.layers.{i}.linear_attn.norm.weight").float().to(device)
            lw.lin_out_w = _linear_weight(g, linear_node(la, "out_proj"), dtype, device)
        else:
            # attention projections: packed or separate
            qkv = linear_node(f"{n}/attn/", "qkv_proj")
            if qkv is not None:
                if keep_q4 and _is_q4([qkv]):
                    lw.qkv_w = _q4_weight(g, [qkv], device)
                else:
                    w = _linear_weight(g, qkv, dtype, device)
                    lw.qkv_w = shard_rows(w, [q_rows, k_rows, v_rows])
                badd = g.by_name.get(f"{n}/attn/qkv_proj/Add")
                if badd is not None:
                    b = g.tensor(badd.inputs[1])
                    lw.qkv_b = shard_rows(b, [q_rows, k_rows, v_rows]).to(device=device, dtype=dtype)
            else:
                ws, bs = [], []
                for nm, rows in (("q_proj", slice(tpr * hq_l * D, (tpr + 1) * hq_l * D)),
                                 ("k_proj", slice(tpr * hkv_l * D, (tpr + 1) * hkv_l * D)),
                                 ("v_proj", slice(tpr * hkv_l * D, (tpr + 1) * hkv_l * D))):
                    node = linear_node(f"{n}/attn/", nm)
                    ws.append(_linear_weight(g, node, dtype, device, rows=rows if tpn > 1 else None))
                    badd = g.by_name.get(f"{n}/attn/{nm}/Add")
                    if badd is not None:
                        b = g.tensor(badd.inputs[1])
                        bs.append((b[rows] if tpn > 1 else b).to(device=device, dtype=dtype))
                lw.qkv_w = torch.cat(ws, 0).contiguous()
                lw.qkv_b = torch.cat(bs, 0).contiguous() if bs else None
            o = linear_node(f"{n}/attn/", "o_proj")
            if keep_q4 and _is_q4([o]):
                lw.o_w = _q4_weight(g, [o], device)
            else:
                lw.o_w = _linear_weight(g, o, dtype, device, cols=slice(tpr * hq_l * D, (tpr + 1) * hq_l * D) if tpn > 1 else None)
            gate = g.find(f"{n}/attn/gate_proj/", ops=LINEAR_OPS)
            if gate is not None:
                if tpn > 1:
                    raise NotImplementedError("gated attention output is not sharded: run these models on one GPU")
                lw.attn_gate_w = _linear_weight(g, gate, dtype, device)
                arch.attn_output_gate = True
            oadd = g.by_name.get(f"{n}/attn/o_proj/Add")
            if oadd is not None:
                lw.o_b = _vec(g, oadd.inputs[1], dtype, device)
            if arch.cross_attention:
                cn = g.by_name[f"{n}/cross_attn_layernorm/SkipLayerNorm"]
                lw.cross_ln_w = _vec(g, cn.inputs[2], dtype, device)
                lw.cross_ln_b = _vec(g, cn.inputs[3], dtype, device) if arch.layernorm and len(cn.inputs) > 3 else None
                hd = slice(tpr * hq_l * D, (tpr + 1) * hq_l * D)
                Hq = arch.num_heads * D
                kv_rows = [hd, slice(Hq + hd.start, Hq + hd.stop)]
                lw.cross_q_w = _linear_weight(g, linear_node(f"{n}/cross_attn/", "q_proj"), dtype, device, rows=hd if tpn > 1 else None)
                lw.cross_q_b = _vec(g, g.by_name[f"{n}/cross_attn/q_proj/Add"].inputs[1], dtype, device, hd if tpn > 1 else None)
                kvn = linear_node(f"{n}/cross_attn/", "kv_proj")
                kvb = g.tensor(g.by_name[f"{n}/cross_attn/kv_proj/Add"].inputs[1])
                if tpn > 1:
                    lw.cross_kv_w = torch.cat([_linear_weight(g, kvn, dtype, device, rows=r) for r in kv_rows], 0).contiguous()
                    lw.cross_kv_b = shard_rows(kvb, kv_rows).to(device=device, dtype=dtype)
                else:
                    lw.cross_kv_w = _linear_weight(g, kvn, dtype, device)
                    lw.cross_kv_b = kvb.to(device=device, dtype=dtype).contiguous()
                lw.cross_o_w = _linear_weight(g, linear_node(f"{n}/cross_attn/", "o_proj"), dtype, device, cols=hd if tpn > 1 else None)
                lw.cross_o_b = _vec(g, g.by_name[f"{n}/cross_attn/o_proj/Add"].inputs[1], dtype, device)
            attn = g.find(f"{n}/attn/", ops=["GroupQueryAttention", "PagedAttention"])
            for inp in attn.inputs:
                if inp.endswith(".sinks"):
                    s = g.tensor(inp).float()
                    lw.sinks = (s[tpr * hq_l:(tpr + 1) * hq_l] if tpn > 1 else s).to(device).contiguous()
                elif "q_norm" in inp:
                    if arch.qk_norm_full_width and tpn > 1:
                        raise NotImplementedError("q / k norms over all heads are not sharded: run these models on one GPU")
                    lw.q_norm_w = _vec(g, inp, dtype, device)
                elif "k_norm" in inp:
                    lw.k_norm_w = _vec(g, inp, dtype, device)
        if arch.post_sublayer_norms:
            pa = g.find(f"{n}/post_attention_layernorm/")
            pf = g.find(f"{n}/post_feedforward_layernorm/")
            lw.post_attn_norm_w = _vec(g, pa.inputs[1], dtype, device)
            lw.post_ffn_norm_w = _vec(g, pf.inputs[1], dtype, device)
        # MLP / MoE
        moe = g.find(f"{n}/moe/", ops=["MoE", "QMoE"])
        if moe is not None:
            # Experts are not sharded along their matrices: with tensor parallelism every rank loads all experts' routing
            # tables but computes only its own slice of the experts (expert parallelism over replicated tokens, models/moe.py).
            r = linear_node(f"{n}/moe/", "router")
            lw.router_w = _linear_weight(g, r, dtype, device)
            radd = g.by_name.get(f"{n}/moe/router/Add")
            lw.router_b = _vec(g, radd.inputs[1], dtype, device) if radd is not None else None
            E = arch.num_experts
            if E % tpn:
                raise ValueError(f"expert parallel degree {tpn} does not divide the {E} experts")
            lw.exp_lo, lw.exp_hi = tpr * (E // tpn), (tpr + 1) * (E // tpn)

            def experts(name):
                if not name:
                    return None
                t = g.tensor(name, device=device)
                return t[lw.exp_lo:lw.exp_hi].to(device=device, dtype=dtype).contiguous()

            def experts_fp4(wname, sname, gname):
                """MXFP4 experts ([E, K, N/2] codes, [E, N, K/32] e8m0 scales, per-expert global scale) expanded to `dtype`."""
                q, sc = g.tensor(wname)[lw.exp_lo:lw.exp_hi].to(device), g.tensor(sname)[lw.exp_lo:lw.exp_hi].to(device)
                gs = g.tensor(gname)[lw.exp_lo:lw.exp_hi].float().to(device) if gname else None
                Kk, Nn = q.shape[1], q.shape[2] * 2
                out = torch.empty(q.shape[0], Nn, Kk, dtype=dtype, device=device)
                for e in range(q.shape[0]):
                    w = dequantize_mxfp4(q[e], sc[e], Nn, Kk)
                    out[e] = (w * gs[e] if gs is not None else w).to(dtype)
                return out

            def experts_fp4_packed(wname, sname, gname, gate_up):
                """MXFP4 experts kept packed for the grouped FP4 GEMM (ops/fp4.py), or None when this checkpoint or device
                needs the expanded form: CPU, OGB_FP4_EXPERTS=0, non-unit global scales, K not a multiple of 64, block
                scales above 2^1, or gate/up widths the 64-row blocking cannot cover."""
                from ..ops.fp4 import Fp4Experts, unpack_qmoe_fp4
                if torch.device(device).type != "cuda" or os.environ.get("OGB_FP4_EXPERTS", "1") == "0":
                    return None
                if gname and not bool((g.tensor(gname).float() == 1.0).all()):
                    return None
                sc = g.tensor(sname, device=device)[lw.exp_lo:lw.exp_hi]
                q = g.tensor(wname, device=device)[lw.exp_lo:lw.exp_hi]
                Kk, Nn = q.shape[1], q.shape[2] * 2
                if not Fp4Experts.supported(sc, Kk) or (gate_up and (Nn // 2) % 64):
                    return None
                codes, sc = unpack_qmoe_fp4(q.to(device)), sc.to(device)
                if gate_up:
                    from ..ops import interleave_experts_gate_up
                    codes, sc = interleave_experts_gate_up(codes), interleave_experts_gate_up(sc)
                return codes, sc

            packed_experts = False
            if moe.op_type == "QMoE":
                if str(_attr(moe, "quant_type", "")) not in ("fp4", "mxfp4") or int(_attr(moe, "expert_weight_bits", 4)) != 4:
                    raise NotImplementedError("QMoE: only MXFP4 (quant_type fp4, block 32) experts are supported")
                ins = list(moe.inputs) + [""] * 17
                gu_p = experts_fp4_packed(ins[2], ins[3], ins[15], True)
                dn_p = experts_fp4_packed(ins[5], ins[6], ins[16], False) if gu_p is not None else None
                if gu_p is not None and dn_p is not None:
                    from ..ops.fp4 import Fp4Experts
                    # the fp16 form (two codes per conversion instruction) needs both matrices' block scales in its range
                    half = Fp4Experts.fits_fp16(*gu_p) and Fp4Experts.fits_fp16(*dn_p) and os.environ.get("OGB_FP4_FORM", "") != "bf16"
                    gu_p, dn_p = (Fp4Experts.from_codes(c, sc, device, keep_host=c.numel() <= (1 << 24), half=half) for c, sc in (gu_p, dn_p))
                    packed_experts = True
                    lw.exp_gate_up_w, lw.exp_gate_up_b = gu_p, experts(ins[4])
                    lw.exp_down_w, lw.exp_down_b = dn_p, experts(ins[7])
                    if lw.exp_gate_up_b is not None:
                        from ..ops import interleave_experts_gate_up
                        lw.exp_gate_up_b = interleave_experts_gate_up(lw.exp_gate_up_b)
                    lw.exp_blocked = True
                else:
                    lw.exp_gate_up_w, lw.exp_gate_up_b = experts_fp4(ins[2], ins[3], ins[15]), experts(ins[4])
                    lw.exp_down_w, lw.exp_down_b = experts_fp4(ins[5], ins[6], ins[16]), experts(ins[7])
            elif arch.moe_style == "standard":
                # gate [E, I, H] and up [E, I, H] become one matrix with even rows = gate, odd rows = up (the fused layout)
                gate, up = experts(moe.inputs[2]), experts(moe.inputs[6])
                lw.exp_gate_up_w = torch.stack([gate, up], dim=2).reshape(gate.shape[0], 2 * gate.shape[1], gate.shape[2]).contiguous()
                lw.exp_down_w = experts(moe.inputs[4])
                del gate, up
            else:
                lw.exp_gate_up_w, lw.exp_gate_up_b = experts(moe.inputs[2]), experts(moe.inputs[3])
                lw.exp_down_w, lw.exp_down_b = experts(moe.inputs[4]), experts(moe.inputs[5])
            sh = linear_node(f"{n}/moe/shared_expert/", "gate_up_proj")
            if sh is not None:
                # the always-on dense MLP beside the routed experts: [gate rows | up rows], not sharded
                if tpn > 1:
                    raise NotImplementedError("shared experts are not sharded: run these models on one GPU")
                lw.gate_up_w = _linear_weight(g, sh, dtype, device)
                lw.gate_up_interleaved = False
                lw.down_w = _linear_weight(g, linear_node(f"{n}/moe/shared_expert/", "down_proj"), dtype, device)
                sg = linear_node(f"{n}/moe/", "shared_expert_gate")
                lw.shared_gate_w = _linear_weight(g, sg, dtype, device) if sg is not None else None
                arch.shared_expert_intermediate = lw.down_w.shape[1]
                arch.shared_expert_gated = sg is not None
            if not packed_experts:
                lw.exp_blocked = False
            if not packed_experts and torch.device(device).type == "cuda" and (lw.exp_gate_up_w.shape[1] // 2) % 64 == 0:
                # grouped GEMM layout: per expert, blocks of 64 gate rows + the 64 up rows of the same features
                from ..ops import interleave_experts_gate_up
                lw.exp_gate_up_w = interleave_experts_gate_up(lw.exp_gate_up_w)
                if lw.exp_gate_up_b is not None:
                    lw.exp_gate_up_b = interleave_experts_gate_up(lw.exp_gate_up_b)
                lw.exp_blocked = True
        elif not arch.mlp_gated:
            i_rows = slice(tpr * i_l, (tpr + 1) * i_l)
            lw.fc1_w = _linear_weight(g, linear_node(f"{n}/mlp/", "fc1"), dtype, device, rows=i_rows if tpn > 1 else None)
            lw.fc2_w = _linear_weight(g, linear_node(f"{n}/mlp/", "fc2"), dtype, device, cols=i_rows if tpn > 1 else None)
            b1, b2 = g.by_name.get(f"{n}/mlp/fc1/Add"), g.by_name.get(f"{n}/mlp/fc2/Add")
            if b1 is not None:
                lw.fc1_b = _vec(g, b1.inputs[1], dtype, device, i_rows if tpn > 1 else None)
            if b2 is not None:
                lw.fc2_b = _vec(g, b2.inputs[1], dtype, device)
        else:
            gu = linear_node(f"{n}/mlp/", "gate_up_proj")
            g_rows, u_rows = slice(tpr * i_l, (tpr + 1) * i_l), slice(I + tpr * i_l, I + (tpr + 1) * i_l)
            if gu is not None and keep_q4 and _is_q4([gu]):
                il = arch.activation == "silu" and I % 64 == 0
                lw.gate_up_w = _q4_weight(g, [gu], device, interleave=il)
                lw.gate_up_interleaved = il
                badd = g.by_name.get(f"{n}/mlp/gate_up_proj/Add")
                if badd is not None:
                    b = g.tensor(badd.inputs[1])
                    from ..ops import interleave_gate_up as _il
                    lw.gate_up_b = (_il(b) if il else b).to(device=device, dtype=dtype)
            elif gu is not None:
                w = _linear_weight(g, gu, dtype, device)
                lw.gate_up_w = shard_rows(w, [g_rows, u_rows])
                badd = g.by_name.get(f"{n}/mlp/gate_up_proj/Add")
                if badd is not None:
                    lw.gate_up_b = shard_rows(g.tensor(badd.inputs[1]), [g_rows, u_rows]).to(device=device, dtype=dtype)
            else:
                gw = _linear_weight(g, linear_node(f"{n}/mlp/", "gate_proj"), dtype, device, rows=g_rows if tpn > 1 else None)
                uw = _linear_weight(g, linear_node(f"{n}/mlp/", "up_proj"), dtype, device, rows=g_rows if tpn > 1 else None)
                lw.gate_up_w = torch.cat([gw, uw], 0).contiguous()
            if (isinstance(lw.gate_up_w, torch.Tensor) and torch.device(device).type == "cuda" and arch.activation == "silu"
                    and (lw.gate_up_w.shape[0] // 2) % 64 == 0):
                from ..ops import interleave_gate_up
                lw.gate_up_w = interleave_gate_up(lw.gate_up_w)
                if lw.gate_up_b is not None:
                    lw.gate_up_b = interleave_gate_up(lw.gate_up_b)
                lw.gate_up_interleaved = True
            dn = linear_node(f"{n}/mlp/", "down_proj")
            if keep_q4 and _is_q4([dn]):
                lw.down_w = _q4_weight(g, [dn], device)
            else:
                lw.down_w = _linear_weight(g, dn, dtype, device, cols=g_rows if tpn > 1 else None)
            dadd = g.by_name.get(f"{n}/mlp/down_proj/Add")
            if dadd is not None:
                lw.down_b = _vec(g, dadd.inputs[1], dtype, device)
        model.layers.append(lw)

    fin = g.find(f"/model/layers.{arch.num_layers}/final_norm_layernorm/")
    model.final_norm_w = _vec(g, fin.inputs[2 if len(fin.inputs) >= 3 else 1], dtype, device)
    if arch.layernorm and len(fin.inputs) > 3:
        model.final_norm_b = _vec(g, fin.inputs[3], dtype, device)
    head = g.find("/lm_head/", ops=LINEAR_OPS)
    V = arch.vocab_size
    if tpn > 1:
        per = (V + tpn - 1) // tpn
        rows = slice(tpr * per, min(V, (tpr + 1) * per))
        model.vocab_shard = (rows.start, rows.stop, per)
    else:
        rows = None
    if keep_q4 and _is_q4([head]):
        model.lm_head_w = _q4_weight(g, [head], device)
    else:
        model.lm_head_w = _linear_weight(g, head, dtype, device, rows=rows)
    hadd = g.by_name.get("/lm_head/Add")
    if hadd is not None:
        model.lm_head_b = _vec(g, hadd.inputs[1], dtype, device, rows)
    g.lm.close()
    model.fold_norms()      # bf16 CUDA models: the input norms' weights move into the QKV and gate/up projections
    return model
