"""Architecture description of a decoder-only transformer.

One dataclass covers the model families the reference's registry lists as LLM types
(src/models/model_type.h:20): llama, mistral, qwen2, qwen3, phi3, phi, gemma/gemma2/gemma3, granite,
olmo, smollm3, internlm2, ernie4_5, nemotron, chatglm, gptoss (mixture of experts) ...  A family
is a set of flag values, not a class.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional

import numpy as np

LLM_TYPES = [
    "chatglm", "decoder", "ernie4_5", "gemma", "gemma2", "gemma3_text", "gptoss", "gpt_oss", "granite", "hunyuan", "hunyuandensev1", "hunyuan_v1_dense",
    "internlm2", "llama", "mistral", "nemotron", "olmo", "olmo2", "exaone4", "phi", "phi3", "phimoe", "qwen2", "qwen3",
    "smollm3", "lfm2", "gpt2", "helium", "mixtral", "qwen2_moe", "qwen3_moe", "granitemoe", "olmoe", "qwen2_vl", "qwen2_5_vl", "qwen3_vl",
    "qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text", "granitemoehybrid", "granitemoeshared",      # hybrids of gated-delta-net (linear attention) and full-attention layers
]


# Vision-language types share one pipeline: ViT-style encoder + projector, image features spliced into the prompt's embeddings
# at the image-token positions (reference: src/models/model_type.h:20-26 lists the VLM / ALM families).
VLM_TYPES = ["phi3v", "gemma3", "mistral3", "llava", "fara"]
ALM_TYPES = ["whisper"]


@dataclass
class ArchConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    intermediate_size: int = 11008
    context_length: int = 4096
    # normalisation
    norm_eps: float = 1e-5
    layernorm: bool = False          # LayerNorm (mean/var, bias) instead of RMSNorm
    norm_offset: float = 0.0         # gemma stores weight - 1; the exporter bakes the offset in
    post_sublayer_norms: bool = False  # gemma2/3: extra norms after attention and MLP outputs
    qk_norm: bool = False            # qwen3 / gemma3: per-head RMSNorm on q and k before RoPE
    # rotary embedding
    rope_theta: float = 10000.0
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    rotary_interleaved: bool = False
    # attention
    attn_bias: bool = False          # bias on q/k/v projections
    o_bias: bool = False
    attn_scale: Optional[float] = None  # default 1/sqrt(head_dim)
    softcap: float = 0.0
    sliding_window: int = 0
    sliding_layers: Optional[List[int]] = None  # None + sliding_window > 0 = every layer
    attn_sinks: bool = False
    # MLP
    mlp_bias: bool = False
    activation: str = "silu"         # silu | gelu
    # Hybrid models (LFM2): layers of type "conv" replace attention by a gated short depthwise convolution over the last
    # conv_L_cache positions; "full_attention" layers are ordinary attention layers.  None: every layer attends.
    layer_types: Optional[List[str]] = None
    conv_L_cache: int = 3
    conv_bias: bool = False
    # Layers of type "linear_attention" are gated-delta-net layers (Qwen3-Next / Qwen3.5 style): a causal depthwise convolution
    # + SiLU over the packed q / k / v channels, then a recurrent state S [value heads, key dim, value dim] per request updated
    # by the gated delta rule (reference ops: CausalConvWithState, LinearAttention with update_rule "gated_delta").
    linear_num_key_heads: int = 0
    linear_num_value_heads: int = 0
    linear_key_head_dim: int = 0
    linear_value_head_dim: int = 0
    linear_conv_kernel_dim: int = 4
    # Layers of type "mamba" are Mamba-2 state-space layers (GraniteMoeHybrid): in_proj -> [gate | x, B, C | dt], a causal
    # depthwise convolution + SiLU over (x, B, C), the selective scan with one state [state_size, head_dim] per head, a gated
    # RMS norm, out_proj.  The model's other layers are attention layers.
    mamba_num_heads: int = 0
    mamba_head_dim: int = 0
    mamba_state_size: int = 0
    mamba_n_groups: int = 1
    mamba_conv_kernel: int = 4
    # Multimodal RoPE (Qwen2-VL): rotary pairs per position component (temporal, height, width); None: ordinary RoPE
    mrope_section: Optional[List[int]] = None
    mrope_interleaved: bool = False  # qwen3_vl: the three position components alternate over the rotary pairs
    cross_attention: bool = False    # encoder-decoder (whisper): every layer also attends to the encoder's output
    encoder_hidden_size: int = 0     # width of the encoder output the cross-attention keys / values are projected from (0 = hidden_size)
    mlp_gated: bool = True           # False: fc1 -> activation -> fc2 (phi, gpt2) instead of act(gate) * up -> down
    parallel_block: bool = False     # phi: attention and MLP both read the input norm; their outputs are summed
    shared_expert_intermediate: int = 0   # MoE layers with an always-on dense gated MLP beside the routed experts (0 = none)
    shared_expert_gated: bool = False     # its output is scaled by sigmoid(x . w) of a one-row projection
    pre_norm: bool = True            # False (olmo2): the sub-layers read the residual stream itself, their norms follow them (post_sublayer_norms)
    qk_norm_full_width: bool = False # olmoe: q and k are normalised over all their heads at once (weights [q_size] / [kv_size]), before the rotary embedding
    qk_norm_after_rope: bool = False # hunyuan: the per-head q / k norms follow the rotary embedding
    attn_output_gate: bool = False   # q_proj carries a second half per head: sigmoid of it gates the attention output before o_proj
    rope_local_theta: float = 0.0    # gemma3: sliding-window layers rotate with this base and no rescaling (a second cache pair)
    no_rope_layers: Optional[List[int]] = None   # layers whose attention applies no rotary embedding (smollm3)
    no_rope: bool = False            # attention without any position encoding (hybrids whose recurrent layers carry the order)
    learned_positions: bool = False  # gpt2: a learned position table added to the token embedding, no rotary embedding
    # mixture of experts (gpt-oss style)
    num_experts: int = 0
    experts_per_token: int = 0
    moe_swiglu_alpha: float = 1.702
    moe_swiglu_limit: float = 7.0
    # "gptoss": router with bias, fused gate/up with biases, clamped SwiGLU(alpha, limit).  "standard" (Mixtral, Qwen-MoE,
    # PhiMoE, GraniteMoE): bias-free router and experts, separate gate / up matrices, silu(gate) * up, softmax over all
    # experts with the selected weights renormalised (moe_norm_topk) or left as they are.
    moe_style: str = "gptoss"
    moe_norm_topk: bool = True
    moe_sparse_mixer: bool = False   # PhiMoE: two experts picked one after the other, each weighted by a softmax over the logits
    moe_jitter_eps: float = 0.01     # within a relative margin 2 * eps of the current maximum
    # embedding / head
    embed_scale: float = 1.0
    tie_embeddings: bool = False
    lm_head_bias: bool = False
    final_logit_softcap: float = 0.0
    # multipliers (granite)
    residual_multiplier: float = 1.0
    logits_scale: float = 1.0
    # token ids
    bos_token_id: int = 1
    eos_token_id: Any = 2
    pad_token_id: int = 0

    @property
    def rotary_dim(self) -> int:
        r = int(self.head_dim * self.partial_rotary_factor)
        return r - (r % 2)

    def layer_rope_mode(self, layer: int) -> int:
        """0: the model's rotary caches, 1: the local caches (`rope_local_theta`), 2: no rotary embedding."""
        if self.learned_positions or self.no_rope or (self.no_rope_layers is not None and layer in self.no_rope_layers):
            return 2
        return 1 if (self.rope_local_theta and self.layer_window(layer)) else 0

    @property
    def applied_rotary_dim(self) -> int:
        """Rotary width the attention kernels apply: none under a learned position table or without position encoding."""
        return 0 if (self.learned_positions or self.no_rope) else self.rotary_dim

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim

    @property
    def scale(self) -> float:
        return self.attn_scale if self.attn_scale is not None else 1.0 / math.sqrt(self.head_dim)

    def is_conv_layer(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "conv"

    def is_linear_layer(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "linear_attention"

    def is_mamba_layer(self, layer: int) -> bool:
        return self.layer_types is not None and self.layer_types[layer] == "mamba"

    def is_recurrent_layer(self, layer: int) -> bool:
        return self.is_linear_layer(layer) or self.is_mamba_layer(layer)

    @property
    def has_linear_layers(self) -> bool:
        """True for models with layers that carry a recurrent state per request (gated-delta-net or Mamba-2 layers)."""
        return self.layer_types is not None and ("linear_attention" in self.layer_types or "mamba" in self.layer_types)

    @property
    def has_mamba_layers(self) -> bool:
        return self.layer_types is not None and "mamba" in self.layer_types

    @property
    def mamba_intermediate(self) -> int:
        return self.mamba_num_heads * self.mamba_head_dim

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_intermediate + 2 * self.mamba_n_groups * self.mamba_state_size

    @property
    def recurrent_state_shape(self):
        """Per request and layer: gated delta net [value heads, key dim, value dim]; Mamba-2 [heads, state size, head dim]."""
        if self.has_mamba_layers:
            return (self.mamba_num_heads, self.mamba_state_size, self.mamba_head_dim)
        return (self.linear_num_value_heads, self.linear_key_head_dim, self.linear_value_head_dim)

    @property
    def recurrent_conv_dim(self) -> int:
        return self.mamba_conv_dim if self.has_mamba_layers else self.linear_conv_dim

    @property
    def linear_key_dim(self) -> int:
        return self.linear_num_key_heads * self.linear_key_head_dim

    @property
    def linear_value_dim(self) -> int:
        return self.linear_num_value_heads * self.linear_value_head_dim

    @property
    def linear_conv_dim(self) -> int:
        return 2 * self.linear_key_dim + self.linear_value_dim

    def conv_state_channels(self, layer: int) -> int:
        """Channels of the paged convolution-input cache of a layer (0: the layer keeps none)."""
        if self.is_conv_layer(layer):
            return self.hidden_size
        if self.is_linear_layer(layer):
            return self.linear_conv_dim
        if self.is_mamba_layer(layer):
            return self.mamba_conv_dim
        return 0

    def layer_window(self, layer: int) -> int:
        if self.sliding_window <= 0:
            return 0
        if self.sliding_layers is None:
            return self.sliding_window
        return self.sliding_window if layer in self.sliding_layers else 0

    def eos_list(self) -> List[int]:
        return list(self.eos_token_id) if isinstance(self.eos_token_id, (list, tuple)) else [int(self.eos_token_id)]

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


def from_hf_config(cfg: Dict[str, Any]) -> ArchConfig:
    """Maps a Hugging Face `config.json` dictionary to an ArchConfig."""
    if isinstance(cfg.get("text_config"), dict) and "hidden_size" not in cfg:
        # a multimodal checkpoint's configuration: the decoder is described by its text part
        tmt = cfg["text_config"].get("model_type", cfg.get("model_type"))
        if tmt in ("qwen2_vl_text", "qwen2_5_vl_text"):
            tmt = tmt[: -len("_text")]
        cfg = {**{k: v for k, v in cfg.items() if k not in ("text_config", "vision_config", "audio_config")}, **cfg["text_config"],
               "architectures": cfg.get("architectures"), "model_type": tmt}
    if isinstance(cfg.get("rope_parameters"), dict):
        # newer configurations keep the rotary settings in one dictionary
        rp = cfg["rope_parameters"]
        cfg = dict(cfg)
        if isinstance(rp.get("full_attention"), dict):
            # one dictionary per layer kind: the sliding-window layers' base becomes the local base
            if isinstance(rp.get("sliding_attention"), dict) and rp["sliding_attention"].get("rope_theta"):
                cfg.setdefault("rope_local_base_freq", rp["sliding_attention"]["rope_theta"])
            rp = rp["full_attention"]
        cfg.setdefault("rope_theta", rp.get("rope_theta", 10000.0))
        cfg.setdefault("partial_rotary_factor", rp.get("partial_rotary_factor", 1.0))
        if (rp.get("rope_type", "default") not in ("default", None) or rp.get("mrope_section")) and not cfg.get("rope_scaling"):
            cfg["rope_scaling"] = {k: v for k, v in rp.items() if k not in ("rope_theta", "partial_rotary_factor")}
    if "ffn_hidden_size" in cfg and "multi_query_group_num" in cfg:
        # ChatGLM's own key names (reference reads the same fallbacks: builders/base.py:80-121)
        cfg = dict(cfg)
        cfg.setdefault("vocab_size", cfg.get("padded_vocab_size"))
        cfg.setdefault("num_hidden_layers", cfg.get("num_layers"))
        cfg.setdefault("intermediate_size", cfg["ffn_hidden_size"])
        cfg.setdefault("num_key_value_heads", cfg["multi_query_group_num"] if cfg.get("multi_query_attention", True) else cfg.get("num_attention_heads"))
        cfg.setdefault("head_dim", cfg.get("kv_channels"))
        cfg.setdefault("max_position_embeddings", cfg.get("seq_length", 8192))
        cfg.setdefault("rms_norm_eps", cfg.get("layernorm_epsilon", 1e-5))
        cfg.setdefault("rope_theta", 10000.0 * float(cfg.get("rope_ratio", 1.0)))
        cfg.setdefault("attention_bias", bool(cfg.get("add_qkv_bias", False)))
        cfg["model_type"] = "chatglm"
    archs = cfg.get("architectures") or [cfg.get("model_type", "llama")]
    name = archs[0]
    mtype = name.split("For")[0].lower() if "For" in name else cfg.get("model_type", name).lower()
    hs = cfg.get("hidden_size", cfg.get("n_embd"))
    nh = cfg.get("num_attention_heads", cfg.get("n_head"))
    a = ArchConfig(
        model_type=mtype,
        vocab_size=cfg["vocab_size"],
        hidden_size=hs,
        num_layers=cfg.get("num_hidden_layers", cfg.get("n_layer")),
        num_heads=nh,
        num_kv_heads=cfg.get("num_key_value_heads", nh),
        head_dim=cfg.get("head_dim") or hs // nh,
        intermediate_size=cfg.get("intermediate_size", 4 * hs),
        context_length=cfg.get("max_position_embeddings", 4096),
        norm_eps=cfg.get("rms_norm_eps", cfg.get("layer_norm_eps", cfg.get("layer_norm_epsilon", 1e-5))),
        rope_theta=cfg.get("rope_theta", 10000.0),
        rope_scaling=({**cfg["rope_scaling"], "original_max_position_embeddings": cfg["original_max_position_embeddings"]}
                      if cfg.get("rope_scaling") and "original_max_position_embeddings" in cfg and
                      "original_max_position_embeddings" not in cfg["rope_scaling"] else cfg.get("rope_scaling")),
        partial_rotary_factor=cfg.get("partial_rotary_factor", 1.0),
        attn_bias=bool(cfg.get("attention_bias", False)),
        mlp_bias=bool(cfg.get("mlp_bias", False)),
        tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
        bos_token_id=cfg.get("bos_token_id") or 0,
        eos_token_id=cfg.get("eos_token_id") if cfg.get("eos_token_id") is not None else 0,
        pad_token_id=cfg.get("pad_token_id") if cfg.get("pad_token_id") is not None else 0,
    )
    mt = cfg.get("model_type", mtype)
    act = cfg.get("hidden_activation") or cfg.get("hidden_act")
    if act:
        a.activation = {"silu": "silu", "swish": "silu", "gelu": "gelu_erf", "gelu_new": "gelu", "gelu_fast": "gelu", "gelu_pytorch_tanh": "gelu",
                        "relu": "relu", "relu2": "relu2"}.get(act, a.activation)
    if a.model_type not in LLM_TYPES and mt in LLM_TYPES:
        a.model_type = mt      # class names that do not spell the family the way its configuration does (Qwen2Moe..., GraniteMoeHybrid...)
    if mt == "gpt2":
        a.hidden_size = cfg.get("n_embd", a.hidden_size)
        a.num_heads = a.num_kv_heads = cfg.get("n_head", a.num_heads)
        a.num_layers = cfg.get("n_layer", a.num_layers)
        a.head_dim = a.hidden_size // a.num_heads
        a.intermediate_size = cfg.get("n_inner") or 4 * a.hidden_size
        a.context_length = cfg.get("n_positions", a.context_length)
    if cfg.get("attention_bias") and mt not in ("qwen2", "qwen2_moe"):
        a.o_bias = True               # the families that read this switch put the bias on all four projections
    if mt == "smollm3" and cfg.get("no_rope_layers"):
        a.no_rope_layers = [i for i, keep in enumerate(cfg["no_rope_layers"]) if not keep]      # the list marks the layers that DO rotate
    if mt in ("ernie4_5", "helium"):
        a.rotary_interleaved = True   # pairs (x[2i], x[2i+1]) rotate together
        if mt == "ernie4_5":
            a.attn_bias = a.o_bias = a.mlp_bias = bool(cfg.get("use_bias", False))
    if mt in ("hunyuan_v1_dense", "hunyuandensev1", "hunyuan"):
        a.model_type = "hunyuandensev1"
        a.qk_norm = bool(cfg.get("use_qk_norm", True))
        a.qk_norm_after_rope = a.qk_norm
    if mt == "nemotron":
        # layer norms whose stored weight is the offset from one, a two-matrix MLP with squared ReLU
        a.layernorm = True
        a.norm_offset = 1.0
        a.norm_eps = cfg.get("norm_eps", a.norm_eps)
        a.mlp_gated = False
        a.activation = {"relu2": "relu2", "relu": "relu", "gelu": "gelu_erf", "gelu_new": "gelu", "gelu_pytorch_tanh": "gelu"}.get(cfg.get("hidden_act", "relu2"), "relu2")
    if mt == "olmo":
        a.layernorm = True            # layer norm without parameters: exported with unit weights and zero biases
        a.norm_eps = 1e-5
    if mt == "chatglm":
        a.model_type = "chatglm"
        a.partial_rotary_factor = 0.5         # half of every head rotates, in interleaved pairs (reference: builders/chatglm.py:12-17)
        a.rotary_interleaved = True
        a.o_bias = a.mlp_bias = bool(cfg.get("add_bias_linear", False))
        a.tie_embeddings = False
    if mt == "internlm2":
        a.attn_bias = a.o_bias = bool(cfg.get("bias", False))
    if mt == "qwen2":
        a.attn_bias = True
    if mt == "qwen2_moe":
        a.attn_bias = bool(cfg.get("qkv_bias", True))
    if mt in ("phi3small", "phi3_small") or name.startswith("Phi3Small"):
        raise NotImplementedError("phi3small (block-sparse attention, gegelu) is not supported")
    if mt in ("phi4_multimodal", "phi4mm"):
        a.model_type = "phi3"         # the text decoder of Phi-4-multimodal is a phi3 decoder with a partial rotary embedding
    if mt == "exaone4":
        # norms after the sub-layers, per-head q / k norms; with a sliding window the layers alternate and the global ones do not rotate
        a.pre_norm = False
        a.post_sublayer_norms = True
        a.qk_norm = True
        if cfg.get("sliding_window"):
            lt = cfg.get("layer_types") or []
            a.sliding_window = int(cfg["sliding_window"])
            a.sliding_layers = [i for i, t in enumerate(lt) if t == "sliding_attention"]
            a.no_rope_layers = [i for i, t in enumerate(lt) if t != "sliding_attention"]
    if mt == "olmo2":
        a.pre_norm = False
        a.post_sublayer_norms = True
        a.qk_norm = a.qk_norm_full_width = True
    if mt == "exaone":
        raise NotImplementedError("exaone (its own tensor names, not mapped here) is not supported")
    if mt in ("qwen3", "gemma3_text"):
        a.qk_norm = True
    if mt == "olmoe":
        a.qk_norm = a.qk_norm_full_width = True
    if mt in ("mistral", "qwen2", "phi3") and cfg.get("sliding_window") and cfg.get("use_sliding_window", mt != "qwen2"):
        a.sliding_window = int(cfg["sliding_window"])
    if mt.startswith("gemma"):
        a.embed_scale = math.sqrt(hs)
        a.activation = "gelu"
        a.norm_offset = 1.0
        a.tie_embeddings = True
        if mt in ("gemma2", "gemma3_text"):
            a.post_sublayer_norms = True
            a.softcap = cfg.get("attn_logit_softcapping") or 0.0
            a.final_logit_softcap = cfg.get("final_logit_softcapping") or 0.0
            if cfg.get("query_pre_attn_scalar"):
                a.attn_scale = 1.0 / math.sqrt(cfg["query_pre_attn_scalar"])
            sw = cfg.get("sliding_window") or 0
            if sw:
                a.sliding_window = sw
                pattern = cfg.get("sliding_window_pattern", cfg.get("_sliding_window_pattern", 2 if mt == "gemma2" else 6))
                lt = cfg.get("layer_types")
                a.sliding_layers = ([i for i, t in enumerate(lt) if t == "sliding_attention"] if lt
                                    else [i for i in range(a.num_layers) if (i + 1) % pattern != 0])
            if mt == "gemma3_text":
                a.rope_local_theta = float(cfg.get("rope_local_base_freq") or 10000.0)
    if mt in ("gpt_oss", "gptoss"):
        a.model_type = "gptoss"
        a.num_experts = cfg.get("num_local_experts", 32)
        a.experts_per_token = cfg.get("num_experts_per_tok", cfg.get("experts_per_token", 4))
        a.attn_sinks = True
        a.attn_bias = a.o_bias = a.mlp_bias = True
        a.sliding_window = cfg.get("sliding_window", 128)
        lt = cfg.get("layer_types")
        a.sliding_layers = ([i for i, t in enumerate(lt) if t == "sliding_attention"] if lt
                            else [i for i in range(a.num_layers) if i % 2 == 0])
        a.moe_swiglu_limit = cfg.get("swiglu_limit", 7.0)
    if (mt in ("mixtral", "phimoe", "qwen2_moe", "qwen3_moe", "granitemoe", "olmoe", "qwen3_5_moe", "qwen3_5_moe_text", "granitemoeshared") or
            (mt == "granitemoehybrid" and int(cfg.get("num_local_experts") or 0) > 0)):
        a.moe_style = "standard"
        a.num_experts = cfg.get("num_local_experts", cfg.get("num_experts", 8))
        a.experts_per_token = cfg.get("num_experts_per_tok", 2)
        a.moe_norm_topk = bool(cfg.get("norm_topk_prob", True))
        a.intermediate_size = cfg.get("moe_intermediate_size", a.intermediate_size)
        if mt == "qwen3_moe":
            a.qk_norm = True
        if mt in ("qwen2_moe", "qwen3_5_moe", "qwen3_5_moe_text"):
            a.shared_expert_intermediate = int(cfg.get("shared_expert_intermediate_size") or 0)
            a.shared_expert_gated = a.shared_expert_intermediate > 0
        if mt in ("granitemoeshared", "granitemoehybrid"):
            a.shared_expert_intermediate = int(cfg.get("shared_intermediate_size") or 0)
            a.intermediate_size = int(cfg.get("intermediate_size", a.intermediate_size))
        if mt in ("granitemoe", "granitemoeshared", "granitemoehybrid"):
            a.moe_norm_topk = True        # softmax over the selected experts' logits: the softmax over all, renormalised over the selected
        if mt == "phimoe":
            a.moe_sparse_mixer = True
            a.moe_jitter_eps = float(cfg.get("router_jitter_noise", 0.01))
            a.layernorm = True
            a.attn_bias = a.o_bias = bool(cfg.get("attention_bias", True))
            a.lm_head_bias = bool(cfg.get("lm_head_bias", True))
    if mt == "granitemoehybrid":
        # hybrid of Mamba-2 and attention layers; the feed-forward of the dense members is the "shared" gated MLP
        a.layer_types = ["full_attention" if t == "attention" else t for t in (cfg.get("layer_types") or ["mamba"] * a.num_layers)]
        a.mamba_num_heads = int(cfg.get("mamba_n_heads", 128))
        dh = cfg.get("mamba_d_head", 64)
        a.mamba_head_dim = (int(cfg.get("mamba_expand", 2)) * a.hidden_size // a.mamba_num_heads) if dh in (None, 0, "auto") else int(dh)
        a.mamba_state_size = int(cfg.get("mamba_d_state", 256))
        a.mamba_n_groups = int(cfg.get("mamba_n_groups", 1))
        a.mamba_conv_kernel = int(cfg.get("mamba_d_conv", 4))
        if a.num_experts == 0:
            a.intermediate_size = int(cfg.get("shared_intermediate_size", a.intermediate_size))
        a.no_rope = cfg.get("position_embedding_type") != "rope"
    if mt in ("granite", "granitemoe", "granitemoeshared", "granitemoehybrid"):
        a.residual_multiplier = cfg.get("residual_multiplier", 1.0)
        a.logits_scale = 1.0 / cfg.get("logits_scaling", 1.0)
        a.embed_scale = cfg.get("embedding_multiplier", 1.0)
        a.attn_scale = cfg.get("attention_multiplier")
    if mt == "phi":
        a.layernorm = True
        a.activation = "gelu"
        a.attn_bias = a.o_bias = a.mlp_bias = a.lm_head_bias = True
        a.mlp_gated = False
        a.parallel_block = True
    if mt in ("qwen2_vl", "qwen2_5_vl") or (cfg.get("rope_scaling") or {}).get("mrope_section"):
        a.mrope_section = list((cfg.get("rope_scaling") or {}).get("mrope_section") or [16, 24, 24])
        a.mrope_interleaved = bool((cfg.get("rope_scaling") or {}).get("mrope_interleaved", False))
        a.rope_scaling = None
        a.attn_bias = mt not in ("qwen3_vl", "qwen3_vl_text")
    if mt in ("qwen3_vl", "qwen3_vl_text"):
        # the text decoder of Qwen3-VL: qwen3 with three-component rotary positions in the interleaved layout
        a.model_type = "qwen3_vl"
        a.qk_norm = True
    if mt in ("qwen3_next", "qwen3_5", "qwen3_5_text", "qwen3_5_moe", "qwen3_5_moe_text"):
        # zero-centred RMS norms (weights stored as offsets from one), per-head q / k norms, attention output gated by the second half of q_proj
        a.qk_norm = True
        a.norm_offset = 1.0
        a.attn_output_gate = True
        a.mrope_section = None          # text positions: the three rotary components coincide
    if cfg.get("linear_num_value_heads"):
        # hybrid gated-delta-net stacks: every `full_attention_interval`-th layer attends, the others are linear-attention layers
        a.linear_num_key_heads = int(cfg.get("linear_num_key_heads", 0))
        a.linear_num_value_heads = int(cfg["linear_num_value_heads"])
        a.linear_key_head_dim = int(cfg.get("linear_key_head_dim", 128))
        a.linear_value_head_dim = int(cfg.get("linear_value_head_dim", 128))
        a.linear_conv_kernel_dim = int(cfg.get("linear_conv_kernel_dim", 4))
        iv = int(cfg.get("full_attention_interval", 4))
        a.layer_types = list(cfg.get("layer_types") or ["full_attention" if (i + 1) % iv == 0 else "linear_attention" for i in range(a.num_layers)])
    if mt == "lfm2":
        a.layer_types = list(cfg.get("layer_types") or ["full_attention"] * a.num_layers)
        a.conv_L_cache = int(cfg.get("conv_L_cache", 3))
        a.conv_bias = bool(cfg.get("conv_bias", False))
        a.qk_norm = True
        a.norm_eps = cfg.get("norm_eps", a.norm_eps)
        a.intermediate_size = cfg.get("block_ff_dim", a.intermediate_size) if not cfg.get("intermediate_size") else a.intermediate_size
        a.tie_embeddings = bool(cfg.get("tie_embedding", cfg.get("tie_word_embeddings", True)))
    if mt == "gpt2":
        a.layernorm = True
        a.activation = "gelu"
        a.attn_bias = a.o_bias = a.mlp_bias = True
        a.mlp_gated = False
        a.learned_positions = True
        a.tie_embeddings = bool(cfg.get("tie_word_embeddings", True))
        a.norm_eps = cfg.get("layer_norm_epsilon", 1e-5)
        a.activation = {"gelu_new": "gelu", "gelu": "gelu_erf", "relu": "relu"}.get(cfg.get("activation_function", "gelu_new"), "gelu")
    if mt == "phi":
        a.activation = {"gelu_new": "gelu", "gelu": "gelu_erf", "relu": "relu"}.get(cfg.get("hidden_act", "gelu_new"), "gelu")
    return a


# --------------------------------------------------------------------------------------------- RoPE caches
def rope_caches(arch: ArchConfig, max_positions: Optional[int] = None, local: bool = False):
    """cos/sin caches of shape [positions, rotary_dim/2] (fp32), with the frequency rescaling the
    reference's exporter applies (default, linear, llama3, yarn; src/python/py/models/builders/
    base.py:2478-2617, builders/llama.py:15-31)."""
    n = max_positions or arch.context_length
    rot = arch.rotary_dim
    theta = arch.rope_local_theta if local else arch.rope_theta
    inv_freq = 1.0 / (theta ** (np.arange(0, rot, 2, dtype=np.float64) / rot))
    attn_factor = 1.0
    sc = {} if local else (arch.rope_scaling or {})
    kind = sc.get("rope_type", sc.get("type", "default"))
    if kind in ("longrope", "su"):
        multi = longrope_caches(arch)
        return multi[2][:n], multi[3][:n]
    if kind == "linear":
        inv_freq = inv_freq / float(sc["factor"])
    elif kind == "llama3":
        factor = float(sc["factor"])
        low, high = float(sc.get("low_freq_factor", 1.0)), float(sc.get("high_freq_factor", 4.0))
        old = float(sc.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv_freq
        smooth = (old / wavelen - low) / (high - low)
        scaled = np.where(wavelen > old / low, inv_freq / factor, inv_freq)
        mid = (wavelen <= old / low) & (wavelen >= old / high)
        inv_freq = np.where(mid, (1 - smooth) * inv_freq / factor + smooth * inv_freq, scaled)
    elif kind == "yarn":
        factor = float(sc["factor"])
        old = float(sc.get("original_max_position_embeddings", arch.context_length / factor))
        beta_fast, beta_slow = float(sc.get("beta_fast", 32)), float(sc.get("beta_slow", 1))

        def corr(num_rot):
            return (rot * math.log(old / (num_rot * 2 * math.pi))) / (2 * math.log(arch.rope_theta))

        lo, hi = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), rot // 2 - 1)
        ramp = np.clip((np.arange(rot // 2, dtype=np.float64) - lo) / max(hi - lo, 1e-3), 0, 1)
        mask = 1.0 - ramp
        inv_freq = inv_freq / factor * (1 - mask) + inv_freq * mask
        attn_factor = float(sc.get("attention_factor") or (0.1 * math.log(factor) + 1.0))
    t = np.arange(n, dtype=np.float64)
    freqs = np.outer(t, inv_freq)
    return (np.cos(freqs) * attn_factor).astype(np.float32), (np.sin(freqs) * attn_factor).astype(np.float32)


def longrope_caches(arch: ArchConfig):
    """Phi-3 long-context RoPE ("longrope" / "su", src/python/py/models/builders/phi.py:75-95, base.py:2637-2660): two
    cache pairs — per-frequency `short_factor` for sequences up to the original context length, `long_factor` beyond —
    both scaled by sqrt(1 + ln(context / original) / ln(original)) unless the config gives short_mscale / long_mscale.
    Returns None for other scaling types, else (cos_small, sin_small, cos_large, sin_large, original_context)."""
    sc = arch.rope_scaling or {}
    kind = sc.get("rope_type", sc.get("type", "default"))
    if kind not in ("longrope", "su"):
        return None
    rot = arch.rotary_dim
    orig = int(sc.get("original_max_position_embeddings", arch.context_length))
    ratio = arch.context_length / orig
    default_m = 1.0 if ratio <= 1.0 else math.sqrt(1.0 + math.log(ratio) / math.log(orig))
    base = arch.rope_theta ** (np.arange(0, rot, 2, dtype=np.float64) / rot)

    def cache(factors, n, mscale):
        inv_freq = 1.0 / (np.asarray(factors, dtype=np.float64) * base)
        freqs = np.outer(np.arange(n, dtype=np.float64), inv_freq)
        return (np.cos(freqs) * mscale).astype(np.float32), (np.sin(freqs) * mscale).astype(np.float32)

    sm = float(sc.get("short_mscale") or 0) or default_m
    lm = float(sc.get("long_mscale") or 0) or default_m
    cs, ss = cache(sc["short_factor"], orig, sm)
    cl, sl = cache(sc["long_factor"], arch.context_length, lm)
    return cs, ss, cl, sl, orig


# --------------------------------------------------------------------------------------------- presets
PRESETS: Dict[str, ArchConfig] = {
    # BASELINE config 1: tiny Llama-style decoder.
    "tiny-llama": ArchConfig(model_type="llama", vocab_size=32000, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                             head_dim=64, intermediate_size=512, context_length=2048, norm_eps=1e-5, rope_theta=10000.0,
                             bos_token_id=1, eos_token_id=2, pad_token_id=0),
    "phi3-mini": ArchConfig(model_type="phi3", vocab_size=32064, hidden_size=3072, num_layers=32, num_heads=32, num_kv_heads=32,
                            head_dim=96, intermediate_size=8192, context_length=4096, norm_eps=1e-5, rope_theta=10000.0,
                            bos_token_id=1, eos_token_id=32000, pad_token_id=32000),
    "llama-3.1-8b": ArchConfig(model_type="llama", vocab_size=128256, hidden_size=4096, num_layers=32, num_heads=32,
                               num_kv_heads=8, head_dim=128, intermediate_size=14336, context_length=8192, norm_eps=1e-5,
                               rope_theta=500000.0, bos_token_id=128000, eos_token_id=[128001, 128008, 128009],
                               pad_token_id=128001),
    "llama-3.2-1b": ArchConfig(model_type="llama", vocab_size=128256, hidden_size=2048, num_layers=16, num_heads=32,
                               num_kv_heads=8, head_dim=64, intermediate_size=8192, context_length=8192, norm_eps=1e-5,
                               rope_theta=500000.0, bos_token_id=128000, eos_token_id=[128001, 128008, 128009],
                               pad_token_id=128001, tie_embeddings=True),
    "llama-3.1-70b": ArchConfig(model_type="llama", vocab_size=128256, hidden_size=8192, num_layers=80, num_heads=64,
                                num_kv_heads=8, head_dim=128, intermediate_size=28672, context_length=8192, norm_eps=1e-5,
                                rope_theta=500000.0, bos_token_id=128000, eos_token_id=[128001, 128008, 128009],
                                pad_token_id=128001),
    "gpt-oss-20b": ArchConfig(model_type="gptoss", vocab_size=201088, hidden_size=2880, num_layers=24, num_heads=64,
                              num_kv_heads=8, head_dim=64, intermediate_size=2880, context_length=8192, norm_eps=1e-5,
                              rope_theta=150000.0, attn_bias=True, o_bias=True, mlp_bias=True, attn_sinks=True,
                              sliding_window=128, sliding_layers=[i for i in range(24) if i % 2 == 0], num_experts=32,
                              experts_per_token=4, bos_token_id=199998, eos_token_id=[200002, 199999], pad_token_id=199999),
}
