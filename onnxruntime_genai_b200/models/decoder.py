"""Decoder-only transformer runtime over packed variable-length steps and a paged KV cache.

The same forward serves prefill chunks, decode steps and speculative verification: a step is a flat
list of tokens from several requests (`cu_seqlens`), each request has `past_lens[b]` tokens already
in the cache, new K/V rows are appended at `slot_mapping`, and attention reads the cache through
`block_table` (the I/O contract of the reference's paged decoder graph,
src/python/py/models/builders/base.py:484-542 and src/engine/decoders/varlen_decoder_io.h:14-76).

Every op goes through `onnxruntime_genai_b200.ops`: sm_100a kernels on CUDA tensors, fp32 PyTorch
restatements on CPU tensors.  Tensor parallelism shards attention heads and MLP columns; the
row-parallel projections hand their partial sums to `self.tp.reduce` (NCCL baseline or the fused
NVLink kernels in `parallel/`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .. import ops
from ..native_loader import native
from .arch import ArchConfig


@dataclass
class StepInputs:
    input_ids: torch.Tensor        # [T] int32
    positions: torch.Tensor        # [T] int32
    slot_mapping: torch.Tensor     # [T] int32
    cu_seqlens: torch.Tensor       # [B+1] int32
    past_lens: torch.Tensor        # [B] int32
    block_table: torch.Tensor      # [B, cols] int32
    logits_rows: Optional[torch.Tensor] = None  # [R] int32 rows of the packed output that need logits
    slot_mapping_w: Optional[torch.Tensor] = None
    block_table_w: Optional[torch.Tensor] = None
    max_q_len: int = 1
    max_kv_len: int = 1
    min_q_len: int = 0                            # shortest request of the step when the caller knows it (0: unknown)
    inputs_embeds: Optional[torch.Tensor] = None  # overrides the embedding lookup (multimodal / MTP)
    num_decode: int = 0                           # leading requests of the batch that feed exactly one token (mixed steps)
    positions3: Optional[torch.Tensor] = None     # [3, T] int32 position components of multimodal RoPE (None: `positions`)
    attn_order: Optional[torch.Tensor] = None     # [B] int32 permutation of the requests, longest first (attention CTA issue order)
    cross: Optional["CrossKVCache"] = None        # encoder keys / values of an encoder-decoder model
    cross_table: Optional[torch.Tensor] = None    # [B, cols] blocks of each request's encoder keys in `cross`
    cross_lens: Optional[torch.Tensor] = None     # [B] encoder positions per request
    max_cross_len: int = 0
    cross_qk_heads: Optional[list] = None         # [(layer, head)]: alignment heads whose cross-attention scores are wanted
    cross_qk_out: Optional[list] = None           # filled by forward: one [tokens, max_cross_len] fp32 tensor per listed head
    return_hidden: bool = False
    lora_ids: Optional[torch.Tensor] = None      # [T] int32: index of each token's adapter in `lora_names` (len(lora_names) = none)
    lora_names: Optional[tuple] = None           # adapters present in this step (a batch may mix several and none)
    state_slots: Optional[torch.Tensor] = None   # [B] int32 slot of each request in the recurrent-state pool (linear-attention layers)


class PagedKVCache:
    """Per-layer key/value pools of shape [num_blocks * block_size, kv_heads, head_dim].  Layers with a
    sliding window may use a second, smaller pool addressed through ring block tables."""

    def __init__(self, arch: ArchConfig, num_blocks: int, block_size: int, device, dtype, kv_heads: Optional[int] = None,
                 num_window_blocks: int = 0, conv_channels: Optional[int] = None, kv_bits: int = 16):
        self.block_size = block_size
        self.arch, self.device = arch, torch.device(device)
        # kv_bits 8: keys and values are stored as int8 rows with an inline fp32 scale (head_dim + 16 bytes per row and head)
        if kv_bits not in (16, 8):
            raise RuntimeError(f"KV cache quantization: {kv_bits}-bit caches are not supported (8 or none)")
        if kv_bits == 8 and arch.head_dim % 16:
            raise RuntimeError("KV cache quantization requires head_size to be a multiple of 16")
        self.kv_bits = kv_bits
        self.num_blocks = num_blocks
        self.num_window_blocks = num_window_blocks
        hk = kv_heads if kv_heads is not None else arch.num_kv_heads
        conv = [arch.conv_state_channels(i) > 0 for i in range(arch.num_layers)]
        self.windowed = [num_window_blocks > 0 and arch.layer_window(i) > 0 and not conv[i] for i in range(arch.num_layers)]
        n_full = sum(1 for w, c in zip(self.windowed, conv) if not w and not c)
        n_win = sum(1 for w in self.windowed if w)
        # Hybrid models: the gated input (b * x) of every position of every convolution layer, in the same paged slots as
        # the keys and values - rewinding, beam reordering and block sharing need nothing layer-specific.
        self.conv_index = {i: j for j, i in enumerate(i for i, c in enumerate(conv) if c)}
        cc = conv_channels if conv_channels is not None else arch.hidden_size
        if arch.has_linear_layers:
            cc = arch.recurrent_conv_dim
        self.conv = (torch.zeros(len(self.conv_index), num_blocks * block_size, cc, dtype=dtype, device=device)
                     if self.conv_index else None)
        # Recurrent states of linear-attention layers: [layer, request slot, value heads, key dim, value dim] fp32.  Slots are
        # handed out by the owner of the cache (a generator's rows; the engine's requests) and travel in StepInputs.state_slots.
        self.lin_index = {i: j for j, i in enumerate(i for i in range(arch.num_layers) if arch.is_recurrent_layer(i))}
        self.state = None
        self.state_slots = 0
        row, kdt = (arch.head_dim + 16, torch.int8) if kv_bits == 8 else (arch.head_dim, dtype)
        self.full = torch.zeros(max(n_full, 1), 2, num_blocks * block_size, hk, row, dtype=kdt, device=device)
        self.win = (torch.zeros(n_win, 2, num_window_blocks * block_size, hk, row, dtype=kdt, device=device)
                    if n_win else None)
        self._index = []
        fi = wi = 0
        for w, c in zip(self.windowed, conv):
            if c:
                self._index.append((False, -1))
            elif w:
                self._index.append((True, wi)); wi += 1
            else:
                self._index.append((False, fi)); fi += 1

    def layer(self, i: int):
        win, j = self._index[i]
        pool = self.win if win else self.full
        return pool[j, 0], pool[j, 1], win

    def conv_layer(self, i: int) -> torch.Tensor:
        return self.conv[self.conv_index[i]]

    def ensure_state_slots(self, n: int) -> None:
        """At least n request slots in the recurrent-state pool (grown by copying; states of live slots are kept)."""
        if not self.lin_index or n <= self.state_slots:
            return
        a = self.arch
        new = torch.zeros(len(self.lin_index), n, *a.recurrent_state_shape, dtype=torch.float32, device=self.device)
        if self.state is not None:
            new[:, :self.state_slots] = self.state
        self.state, self.state_slots = new, n

    def state_layer(self, i: int) -> torch.Tensor:
        return self.state[self.lin_index[i]]

    @staticmethod
    def bytes_per_block(arch: ArchConfig, block_size: int, dtype, kv_heads: Optional[int] = None, conv_channels: Optional[int] = None,
                        kv_bits: int = 16) -> int:
        hk = kv_heads if kv_heads is not None else arch.num_kv_heads
        n_conv = sum(1 for i in range(arch.num_layers) if arch.conv_state_channels(i) > 0)
        cc = arch.recurrent_conv_dim if arch.has_linear_layers else (conv_channels if conv_channels is not None else arch.hidden_size)
        es = torch.empty((), dtype=dtype).element_size()
        kv_row = arch.head_dim + 16 if kv_bits == 8 else arch.head_dim * es
        return ((arch.num_layers - n_conv) * 2 * hk * kv_row + n_conv * cc * es) * block_size


class CrossKVCache:
    """Keys and values of an encoder's output, projected once per request and per decoder layer: pools of shape
    [layers, 2, num_blocks * block_size, heads, head_dim] addressed through block tables like the self-attention cache, so
    beams of one request (and requests sharing an input) point at the same blocks."""

    def __init__(self, arch: ArchConfig, num_blocks: int, block_size: int, device, dtype, heads: int):
        self.block_size, self.num_blocks = block_size, num_blocks
        self.pool = torch.zeros(arch.num_layers, 2, num_blocks * block_size, heads, arch.head_dim, dtype=dtype, device=device)

    def layer(self, i: int):
        return self.pool[i, 0], self.pool[i, 1]


class NoTP:
    rank, size = 0, 1

    def reduce(self, x, residual=None):
        return x

    def gather_logits(self, x):
        return x

    def fused_ok(self, x, n_out=None):
        return False

    def barrier(self):
        pass


@dataclass
class LayerWeights:
    ln1_w: torch.Tensor
    qkv_w: torch.Tensor
    o_w: torch.Tensor
    ln2_w: torch.Tensor
    ln1_b: Optional[torch.Tensor] = None
    ln2_b: Optional[torch.Tensor] = None
    qkv_b: Optional[torch.Tensor] = None
    o_b: Optional[torch.Tensor] = None
    shared_gate_w: Optional[torch.Tensor] = None # MoE layers with a shared expert (held in gate_up_w / down_w): its output * sigmoid(x @ shared_gate_w^T)
    attn_gate_w: Optional[torch.Tensor] = None   # gated attention output: att * sigmoid(x @ attn_gate_w^T) before o_proj
    q_norm_w: Optional[torch.Tensor] = None
    k_norm_w: Optional[torch.Tensor] = None
    sinks: Optional[torch.Tensor] = None
    post_attn_norm_w: Optional[torch.Tensor] = None
    post_ffn_norm_w: Optional[torch.Tensor] = None
    gate_up_w: Optional[torch.Tensor] = None
    gate_up_b: Optional[torch.Tensor] = None
    down_w: Optional[torch.Tensor] = None
    down_b: Optional[torch.Tensor] = None
    conv_in_w: Optional[torch.Tensor] = None   # hybrid (LFM2) convolution layer: in_proj [3C, H] (b, c, x), depthwise taps [C, L], out_proj
    conv_w: Optional[torch.Tensor] = None
    conv_b: Optional[torch.Tensor] = None
    conv_out_w: Optional[torch.Tensor] = None
    lin_in_w: Optional[torch.Tensor] = None    # gated-delta-net layer: stacked [qkv | z | b | a] input projection
    lin_conv_w: Optional[torch.Tensor] = None  # depthwise taps [conv_dim, K]
    mamba_in_w: Optional[torch.Tensor] = None  # Mamba-2 layer: input projection [gate | x, B, C | dt]
    mamba_conv_w: Optional[torch.Tensor] = None
    mamba_conv_b: Optional[torch.Tensor] = None
    mamba_dt_bias: Optional[torch.Tensor] = None
    mamba_neg_a: Optional[torch.Tensor] = None
    mamba_d: Optional[torch.Tensor] = None
    mamba_norm_w: Optional[torch.Tensor] = None
    mamba_out_w: Optional[torch.Tensor] = None
    lin_dt_bias: Optional[torch.Tensor] = None
    lin_neg_exp_a: Optional[torch.Tensor] = None
    lin_norm_w: Optional[torch.Tensor] = None
    lin_out_w: Optional[torch.Tensor] = None
    cross_ln_w: Optional[torch.Tensor] = None  # encoder-decoder cross-attention (whisper)
    cross_ln_b: Optional[torch.Tensor] = None
    cross_q_w: Optional[torch.Tensor] = None
    cross_q_b: Optional[torch.Tensor] = None
    cross_kv_w: Optional[torch.Tensor] = None  # stacked [k; v] projection of the encoder output
    cross_kv_b: Optional[torch.Tensor] = None
    cross_o_w: Optional[torch.Tensor] = None
    cross_o_b: Optional[torch.Tensor] = None
    fc1_w: Optional[torch.Tensor] = None       # non-gated MLP (phi, gpt2): fc1 -> activation -> fc2
    fc1_b: Optional[torch.Tensor] = None
    fc2_w: Optional[torch.Tensor] = None
    fc2_b: Optional[torch.Tensor] = None
    router_w: Optional[torch.Tensor] = None
    router_b: Optional[torch.Tensor] = None
    exp_gate_up_w: Optional[torch.Tensor] = None  # [E, 2I, H] rows interleaved (gate, up)
    exp_gate_up_b: Optional[torch.Tensor] = None
    exp_down_w: Optional[torch.Tensor] = None     # [E, H, I]
    exp_down_b: Optional[torch.Tensor] = None
    exp_lo: int = 0          # experts [exp_lo, exp_hi) live on this rank (expert parallelism)
    exp_hi: int = 0
    exp_blocked: bool = False  # gate/up rows in blocks of 64 gate + 64 up (grouped-GEMM layout) instead of even/odd
    lora: Dict[str, dict] = field(default_factory=dict)
    fold_ln1: Optional[torch.Tensor] = None    # norm weights that were multiplied into qkv_w / gate_up_w (see DecoderModel.fold_norms)
    fold_ln2: Optional[torch.Tensor] = None
    window: int = 0
    gate_up_interleaved: bool = False  # gate/up rows stored in blocks of 64 (layout of the fused SiLU*mul GEMM)


class DecoderModel:
    def __init__(self, arch: ArchConfig, device, dtype, tp=None):
        self.arch = arch
        self.device = torch.device(device)
        self.dtype = dtype
        self.tp = tp or NoTP()
        self.layers: List[LayerWeights] = []
        self.embed: Optional[torch.Tensor] = None
        self.final_norm_w: Optional[torch.Tensor] = None
        self.final_norm_b: Optional[torch.Tensor] = None
        self.lm_head_w: Optional[torch.Tensor] = None
        self.lm_head_b: Optional[torch.Tensor] = None
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None
        # long-context RoPE (Phi-3 longrope): `cos` / `sin` are the long-factor caches; these serve steps whose KV bound
        # stays within the original context length
        self._rope_modes: Optional[List[int]] = None     # per layer: 0 the model's rotary caches, 1 the local pair, 2 none
        self.cos_local: Optional[torch.Tensor] = None    # sliding-window layers with a rotary base of their own (gemma3)
        self.sin_local: Optional[torch.Tensor] = None
        self.cos_small: Optional[torch.Tensor] = None
        self.sin_small: Optional[torch.Tensor] = None
        self.rope_original_context = 0
        self.pos_embed: Optional[torch.Tensor] = None   # learned position table (gpt2)
        self.heads_local = arch.num_heads // self.tp.size
        self.kv_heads_local = max(1, arch.num_kv_heads // self.tp.size)
        self.conv_channels_local = arch.hidden_size // self.tp.size      # channels of a hybrid model's convolution layers
        self.inter_local = arch.intermediate_size // self.tp.size
        self.active_adapter = None  # name -> used by the LoRA hooks
        self._lora_batch = None     # per-token adapters of the step in flight (models/lora.py::LoraBatch)
        self._dumping = False
        self.norms_folded = False
        self.fuse_steps = True      # decode-sized steps of a folded model take the five-kernel layer (tests compare both forms)

    # ------------------------------------------------------------------------------------ helpers
    def _linear(self, x, w, b=None, residual=None, lora=None, out_fp32=False):
        y = ops.linear(x, w, b, residual, out_fp32=out_fp32)
        if lora is not None:
            from .lora import apply_lora
            y = apply_lora(y, x, lora)
        return y

    @staticmethod
    def _plain(h):
        """A layer output as a tensor (blocks without norms before their sub-layers never defer a mixture-of-experts combine)."""
        if isinstance(h, ops.PendingCombine):
            raise RuntimeError("a deferred mixture-of-experts combine needs the residual add + norm that folds it")
        return h

    def _add_norm(self, h, w, b, residual):
        """(norm(h + residual), h + residual); `h` may be the pending output of a mixture-of-experts layer."""
        a = self.arch
        if isinstance(h, ops.PendingCombine):
            return ops.norm_moe_combine(h, w, a.norm_eps, residual, b, a.layernorm)
        return ops.norm(h, w, a.norm_eps, residual, b, a.layernorm)

    def _layer_rope(self, li: int, cos, sin, rot: int):
        """The rotary caches and width of one layer: the model's, the local pair of sliding-window layers, or none."""
        modes = self._rope_modes
        if modes is None or len(modes) != len(self.layers):
            modes = self._rope_modes = [self.arch.layer_rope_mode(i) for i in range(len(self.layers))]
        mode = modes[li]
        if mode == 2:
            return cos, sin, 0
        if mode == 1 and self.cos_local is not None:
            return self.cos_local, self.sin_local, rot
        return cos, sin, rot

    def _mlp(self, lw: LayerWeights, x, defer: bool = False):
        a = self.arch
        if a.num_experts > 0:
            from .moe import moe_forward
            if lw.gate_up_w is None:
                return moe_forward(self, lw, x, defer)
            # routed experts + the always-on shared expert
            y = moe_forward(self, lw, x, False)
            act = ops.gate_up_act(x, lw.gate_up_w, lw.gate_up_b, a.activation, interleaved=lw.gate_up_interleaved)
            sh = self._linear(act, lw.down_w, lw.down_b)
            if lw.shared_gate_w is not None:
                sh = (sh.float() * torch.sigmoid(x.float() @ lw.shared_gate_w.float().t())).to(sh.dtype)
            return y + sh
        if not a.mlp_gated:
            y = ops.activation(self._linear(x, lw.fc1_w, lw.fc1_b, lora=self._lora(lw, "fc1")), a.activation)
            return self._row_parallel(y, lw.fc2_w, lw.fc2_b, self._lora(lw, "fc2"))
        lora = self._lora(lw, "gate_up_proj")
        if lora is None:
            act = ops.gate_up_act(x, lw.gate_up_w, lw.gate_up_b, a.activation, interleaved=lw.gate_up_interleaved)
        else:
            y = ops.linear(x, lw.gate_up_w, lw.gate_up_b)
            if lw.gate_up_interleaved:
                inter = y.shape[1] // 2
                y = y.view(-1, inter // 64, 2, 64).transpose(1, 2).reshape(-1, 2 * inter).contiguous()
            from .lora import apply_lora
            act = ops.act_mul(apply_lora(y, x, lora), a.activation)
        return self._row_parallel(act, lw.down_w, lw.down_b, self._lora(lw, "down_proj"))

    def _row_parallel(self, x, w, b, lora):
        """Row-parallel projection: partial products summed over the tensor-parallel ranks."""
        bias = b if self.tp.rank == 0 else None
        if self.tp.size > 1 and lora is None and isinstance(w, torch.Tensor) and self.tp.fused_ok(x, w.shape[0]):
            return ops.linear(x, w, bias, all_reduce=True)   # GEMM + all-reduce in one kernel over NVLink
        return self.tp.reduce(self._linear(x, w, bias, lora=lora))

    def _attention(self, s: StepInputs, qkv, kc, vc, table, block_size: int, lw: LayerWeights):
        """Paged attention of one layer.  A mixed step (single-token requests first, then prompt chunks) runs as two launches:
        the single-token requests on the decode tiles (16 rows, the four warps share every K/V tile), the chunks on the
        64-row tiles - in one launch every single-token request would occupy a 64-row tile that one warp walks alone."""
        a = self.arch
        args = (block_size, self.heads_local, self.kv_heads_local, a.head_dim, a.scale, lw.window, lw.sinks, a.softcap)
        nd, B = s.num_decode, s.past_lens.shape[0]
        if not (qkv.is_cuda and 0 < nd < B and s.max_q_len > 1):
            return ops.paged_attention(qkv, kc, vc, s.cu_seqlens, s.past_lens, table, *args, max_q_len=s.max_q_len,
                                       max_kv_len=s.max_kv_len, order=s.attn_order, min_q_len=s.min_q_len or None)
        out = torch.empty(qkv.shape[0], self.heads_local * a.head_dim, dtype=qkv.dtype, device=qkv.device)
        ops.paged_attention(qkv, kc, vc, s.cu_seqlens[:nd + 1], s.past_lens[:nd], table[:nd], *args, max_q_len=1,
                            max_kv_len=s.max_kv_len, out=out, total_tokens=nd)
        ops.paged_attention(qkv, kc, vc, s.cu_seqlens[nd:], s.past_lens[nd:], table[nd:], *args, max_q_len=s.max_q_len,
                            max_kv_len=s.max_kv_len, out=out)
        return out

    def _linear_attention(self, s: StepInputs, kv: PagedKVCache, li: int, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        """A gated-delta-net layer (reference graph: builders/qwen.py:1776-1867).  The causal convolution reads the projected
        q / k / v rows of the last K - 1 positions from the paged cache (the short-convolution kernel of the hybrid models with
        unit gates), so rewinding and block copies need no convolution state; the recurrent state lives in the request's slot."""
        a = self.arch
        if s.state_slots is None:
            raise RuntimeError("this model has linear-attention layers: the caller must provide StepInputs.state_slots")
        T = x.shape[0]
        cd, vd, nk, nv, hk, hv = a.linear_conv_dim, a.linear_value_dim, a.linear_num_key_heads, a.linear_num_value_heads, a.linear_key_head_dim, a.linear_value_head_dim
        proj = self._linear(x, lw.lin_in_w)
        qkv, z, b_, a_ = proj[:, :cd], proj[:, cd:cd + vd], proj[:, cd + vd:cd + vd + nv], proj[:, cd + vd + nv:]
        conv = ops.causal_conv(qkv, lw.lin_conv_w, None, kv.conv_layer(li), s.slot_mapping, s.positions, s.cu_seqlens, s.past_lens,
                               s.block_table, kv.block_size, silu=True)
        if (conv.is_cuda and conv.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16 and hv <= 128 and hk in (16, 32, 64, 128, 256) and
                lw.lin_norm_w.dtype == torch.float32):
            # normalisation, gates, recurrence and the gated output norm in two kernels
            o = ops.gated_delta_layer(conv, proj, cd, vd, nk, nv, hk, hv, lw.lin_neg_exp_a, lw.lin_dt_bias, lw.lin_norm_w, a.norm_eps,
                                      kv.state_layer(li), s.state_slots, s.cu_seqlens, s.past_lens)
            return self._row_parallel(o, lw.lin_out_w, None, None)
        conv = conv.float()
        kd = nk * hk
        q = torch.nn.functional.normalize(conv[:, :kd].view(T, nk, hk), dim=-1, eps=1e-6) * (hk ** -0.5)
        k = torch.nn.functional.normalize(conv[:, kd:2 * kd].view(T, nk, hk), dim=-1, eps=1e-6)
        v = conv[:, 2 * kd:].view(T, nv, hv)
        beta = torch.sigmoid(b_.float())
        g = lw.lin_neg_exp_a * torch.nn.functional.softplus(a_.float() + lw.lin_dt_bias)
        o = ops.gated_delta(q.to(x.dtype).contiguous(), k.to(x.dtype).contiguous(), v.to(x.dtype).contiguous(), g, beta, kv.state_layer(li),
                            s.state_slots, s.cu_seqlens, s.past_lens).float()
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + a.norm_eps) * lw.lin_norm_w          # RMS norm per value head
        o = (o.view(T, vd) * torch.nn.functional.silu(z.float())).to(x.dtype)
        return self._row_parallel(o, lw.lin_out_w, None, None)

    def _mamba(self, s: StepInputs, kv: PagedKVCache, li: int, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
        """A Mamba-2 layer (GraniteMoeHybrid).  Like the gated-delta-net layers, the causal convolution reads the projected
        (x, B, C) rows of the last K - 1 positions from the paged cache and the state of the scan lives in the request's slot."""
        a = self.arch
        if s.state_slots is None:
            raise RuntimeError("this model has Mamba layers: the caller must provide StepInputs.state_slots")
        T = x.shape[0]
        I, cd, nh, P, N, G = a.mamba_intermediate, a.mamba_conv_dim, a.mamba_num_heads, a.mamba_head_dim, a.mamba_state_size, a.mamba_n_groups
        proj = self._linear(x, lw.mamba_in_w)
        z, xbc, dt = proj[:, :I], proj[:, I:I + cd], proj[:, I + cd:]
        conv = ops.causal_conv(xbc, lw.mamba_conv_w, lw.mamba_conv_b, kv.conv_layer(li), s.slot_mapping, s.positions, s.cu_seqlens, s.past_lens,
                               s.block_table, kv.block_size, silu=True)
        if (conv.is_cuda and conv.dtype == torch.bfloat16 and proj.dtype == torch.bfloat16 and P <= 128 and N in (16, 32, 64, 128, 256) and
                I <= 4096 and lw.mamba_norm_w.dtype == torch.float32):
            # step sizes, scan and the gated output norm in two kernels
            y = ops.mamba2_layer(conv, proj, nh, G, P, N, lw.mamba_dt_bias, lw.mamba_neg_a, lw.mamba_d, lw.mamba_norm_w, a.norm_eps,
                                 kv.state_layer(li), s.state_slots, s.cu_seqlens, s.past_lens)
            return self._row_parallel(y, lw.mamba_out_w, None, None)
        xs = conv[:, :I].reshape(T, nh, P).contiguous()
        Bm = conv[:, I:I + G * N].reshape(T, G, N).contiguous()
        Cm = conv[:, I + G * N:].reshape(T, G, N).contiguous()
        step = torch.nn.functional.softplus(dt.float() + lw.mamba_dt_bias)
        y = ops.mamba2_scan(xs, step, lw.mamba_neg_a, Bm, Cm, lw.mamba_d, kv.state_layer(li), s.state_slots, s.cu_seqlens, s.past_lens).float()
        y = y.view(T, I) * torch.nn.functional.silu(z.float())                                    # gate, then RMS norm over the whole width
        y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + a.norm_eps) * lw.mamba_norm_w).to(x.dtype)
        return self._row_parallel(y, lw.mamba_out_w, None, None)

    def _lora(self, lw: LayerWeights, proj: str):
        if self._lora_batch is not None:
            from .lora import grouped_lora
            return grouped_lora(lw, proj, self._lora_batch)
        if self.active_adapter is None:
            return None
        return lw.lora.get(self.active_adapter, {}).get(proj)

    # ------------------------------------------------------------------------------------ decode-step fusions
    def fold_norms(self) -> bool:
        """Multiplies the RMS-norm weights of the attention and MLP inputs into the QKV and gate/up projection weights
        (W[n, k] * g[k]) and replaces the norm weights by ones.  Every forward path stays valid (a norm with unit weight
        followed by the folded projection is the same function), and decode-sized steps can then skip the norm kernels:
        the projection GEMM takes the un-normalised residual stream, sums the squares of each row as the tiles pass through
        shared memory and applies rsqrt(mean + eps) in its epilogue (`ops.linear(..., norm_eps=)`).  Semantics: the
        SkipSimplifiedLayerNormalization -> MatMul pairs of the reference graph
        (src/python/py/models/builders/base.py:2342-2403, 2149-2222).  bf16 CUDA models with plain (unquantised) gated
        MLPs only; returns whether the model was folded."""
        import os
        a = self.arch
        if self.norms_folded:
            return True
        if (self.device.type != "cuda" or self.dtype != torch.bfloat16 or a.layernorm or a.parallel_block or a.num_experts > 0 or not a.pre_norm or
                not a.mlp_gated or os.environ.get("OGB_FOLD_NORMS", "1") == "0"):
            return False
        for lw in self.layers:
            if not (isinstance(lw.qkv_w, torch.Tensor) and isinstance(lw.gate_up_w, torch.Tensor) and lw.conv_in_w is None and
                    lw.cross_q_w is None and lw.ln1_b is None and lw.ln2_b is None and lw.qkv_w.dtype == torch.bfloat16):
                return False
        for lw in self.layers:
            lw.fold_ln1, lw.fold_ln2 = lw.ln1_w, lw.ln2_w
            lw.qkv_w = (lw.qkv_w.float() * lw.ln1_w.float()[None, :]).to(torch.bfloat16)
            lw.gate_up_w = (lw.gate_up_w.float() * lw.ln2_w.float()[None, :]).to(torch.bfloat16)
            lw.ln1_w = torch.ones_like(lw.ln1_w)
            lw.ln2_w = torch.ones_like(lw.ln2_w)
        self.norms_folded = True
        return True

    def _fused_step_ok(self, s: StepInputs) -> bool:
        """Decode-sized steps of a folded model run five kernels per layer: QKV (+ norm, rotary, cache append), attention,
        o_proj (+ residual, + all-reduce), gate/up (+ norm, SiLU * mul), down_proj (+ residual, + all-reduce)."""
        a = self.arch
        lw = self.layers[0]
        return (self.norms_folded and self.fuse_steps and self.active_adapter is None and s.lora_ids is None and
                s.input_ids.shape[0] <= ops.FUSED_MAX_TOKENS and
                (s.inputs_embeds is None or s.inputs_embeds.is_cuda) and a.residual_multiplier == 1.0 and not a.has_linear_layers and not a.attn_output_gate and not a.qk_norm_after_rope and not a.qk_norm_full_width and
                lw.post_attn_norm_w is None and lw.post_ffn_norm_w is None and not s.cross_qk_heads)

    def _forward_fused(self, s: StepInputs, kv: PagedKVCache) -> torch.Tensor:
        a = self.arch
        # the residual stream is updated in place by the projections' epilogues: never the caller's tensor
        h = s.inputs_embeds.clone() if s.inputs_embeds is not None else ops.embedding(s.input_ids, self.embed, a.embed_scale)
        if a.learned_positions:
            h = h + ops.embedding(s.positions, self.pos_embed, 1.0)
        rot = a.applied_rotary_dim
        cos, sin = self.cos, self.sin
        if self.cos_small is not None and s.max_kv_len <= self.rope_original_context:
            cos, sin = self.cos_small, self.sin_small
        for li, lw in enumerate(self.layers):
            kc, vc, windowed = kv.layer(li)
            slots = s.slot_mapping_w if windowed else s.slot_mapping
            table = s.block_table_w if windowed else s.block_table
            lcos, lsin, lrot = self._layer_rope(li, cos, sin, rot)
            if (lw.q_norm_w is None and lw.k_norm_w is None and not a.rotary_interleaved and not a.mrope_section and
                    ops.qkv_fusable(a.head_dim, lrot if lcos is not None else 0, kc)):
                q = ops.qkv_rope_append(h, lw.qkv_w, lw.qkv_b, s.positions, slots, lcos, lsin, kc, vc, self.heads_local,
                                        self.kv_heads_local, a.head_dim, lrot, norm_eps=a.norm_eps)
            else:
                q = ops.linear(h, lw.qkv_w, lw.qkv_b, norm_eps=a.norm_eps)
                ops.rope_kv_append(q, s.positions, slots, lcos, lsin, kc, vc, self.heads_local, self.kv_heads_local, a.head_dim, lrot,
                                   a.rotary_interleaved, lw.q_norm_w, lw.k_norm_w, a.norm_eps,
                                   s.positions3 if a.mrope_section else None, a.mrope_section, a.mrope_interleaved)
            att = self._attention(s, q, kc, vc, table, kv.block_size, lw)
            h = self._row_parallel_residual(att, lw.o_w, lw.o_b, h)
            act = ops.gate_up_act(h, lw.gate_up_w, lw.gate_up_b, a.activation, interleaved=lw.gate_up_interleaved, norm_eps=a.norm_eps)
            h = self._row_parallel_residual(act, lw.down_w, lw.down_b, h)
        x, _ = ops.norm(h, self.final_norm_w, a.norm_eps, None, self.final_norm_b, a.layernorm)
        return self._logits(s, x)

    def _row_parallel_residual(self, x, w, b, residual):
        """residual + (row-parallel projection summed over the tensor-parallel ranks), written over `residual`."""
        tp = self.tp
        bias = b if tp.rank == 0 else None
        if tp.size == 1:
            return ops.linear(x, w, bias, residual=residual, out=residual)
        if isinstance(w, torch.Tensor) and tp.fused_ok(x, w.shape[0]):
            return ops.linear(x, w, bias, residual=residual, out=residual, all_reduce=True)
        return tp.reduce(ops.linear(x, w, bias), residual)

    def _logits(self, s: StepInputs, x: torch.Tensor) -> torch.Tensor:
        a = self.arch
        self.last_hidden = x
        if s.logits_rows is not None:
            x = ops.gather_rows(x, s.logits_rows)
        logits = ops.linear(x, self.lm_head_w, self.lm_head_b, out_fp32=True)
        logits = self.tp.gather_logits(logits)
        if a.logits_scale != 1.0:
            logits = logits * a.logits_scale
        if a.final_logit_softcap > 0:
            logits = torch.tanh(logits / a.final_logit_softcap) * a.final_logit_softcap
        return logits

    # ------------------------------------------------------------------------------------ forward
    # ------------------------------------------------------------------------------------ sequence-parallel form
    def _sp_ok(self, s: StepInputs) -> bool:
        """Prefill-sized steps of a plain dense model under tensor parallelism run in the sequence-parallel form: the
        residual stream is split by token rows between the ranks, the row-parallel projections end in a fused
        reduce-scatter and the column-parallel ones start from a fused all-gather."""
        tp, a = self.tp, self.arch
        comm = getattr(tp, "comm", None)
        if tp.size <= 1 or comm is None or s.inputs_embeds is not None or self.active_adapter is not None or a.qk_norm_after_rope:
            return False
        T = s.input_ids.shape[0]
        lw = self.layers[0]
        plain = (a.num_experts == 0 and not a.layernorm and a.residual_multiplier == 1.0 and a.activation == "silu" and lw.post_attn_norm_w is None and
                 lw.gate_up_interleaved and isinstance(lw.gate_up_w, torch.Tensor) and isinstance(lw.qkv_w, torch.Tensor) and
                 self.embed.dtype == torch.bfloat16)
        return (plain and 0 < tp.sp_min_tokens <= T and T % tp.size == 0 and T * a.hidden_size <= comm.plane_elems and
                T * self.lm_head_w.shape[1] <= comm.plane_elems)

    sp_steps = 0   # forwards that took the sequence-parallel form (diagnostics / tests)

    def _forward_sp(self, s: StepInputs, kv: PagedKVCache) -> torch.Tensor:
        a, tp = self.arch, self.tp
        self.sp_steps += 1
        comm, rank, W = tp.comm, tp.rank, tp.size
        T = s.input_ids.shape[0]
        per = T // W
        rows = slice(rank * per, (rank + 1) * per)
        cos, sin = self.cos, self.sin
        if self.cos_small is not None and s.max_kv_len <= self.rope_original_context:
            cos, sin = self.cos_small, self.sin_small
        # this rank's token rows of the residual stream
        h = ops.embedding(s.input_ids[rows].contiguous(), self.embed, a.embed_scale)
        residual = None
        for li, lw in enumerate(self.layers):
            if residual is None:
                x, _ = ops.norm(h, lw.ln1_w, a.norm_eps)
                residual = h
            else:
                x, residual = ops.norm(h, lw.ln1_w, a.norm_eps, residual)
            comm.all_gather_push(x)                                        # all-gather -> QKV GEMM (one consumer kernel)
            qkv = ops.linear_gathered(T, lw.qkv_w, lw.qkv_b)
            kc, vc, windowed = kv.layer(li)
            slots = s.slot_mapping_w if windowed else s.slot_mapping
            table = s.block_table_w if windowed else s.block_table
            lcos, lsin, lrot = self._layer_rope(li, cos, sin, a.applied_rotary_dim)
            ops.rope_kv_append(qkv, s.positions, slots, lcos, lsin, kc, vc, self.heads_local, self.kv_heads_local,
                               a.head_dim, lrot, a.rotary_interleaved, lw.q_norm_w, lw.k_norm_w, a.norm_eps)
            att = ops.paged_attention(qkv, kc, vc, s.cu_seqlens, s.past_lens, table, kv.block_size, self.heads_local,
                                      self.kv_heads_local, a.head_dim, a.scale, lw.window, lw.sinks, a.softcap,
                                      max_q_len=s.max_q_len, max_kv_len=s.max_kv_len)
            # o_proj GEMM -> reduce-scatter by token rows (one kernel); the bias joins once, on rank 0's partial
            h = ops.linear(att, lw.o_w, lw.o_b if rank == 0 else None, reduce_scatter=(rank, W))
            x, residual = ops.norm(h, lw.ln2_w, a.norm_eps, residual)
            comm.all_gather_push(x)                                        # all-gather -> gate/up GEMM + SiLU*mul
            act = ops.linear_gathered(T, lw.gate_up_w, lw.gate_up_b, act_pair=True)
            h = ops.linear(act, lw.down_w, lw.down_b if rank == 0 else None, reduce_scatter=(rank, W))
        x, residual = ops.norm(h, self.final_norm_w, a.norm_eps, residual)
        x = comm.all_gather(x).reshape(T, -1)                              # every rank needs the rows its logits come from
        self.last_hidden = x
        if s.logits_rows is not None:
            x = ops.gather_rows(x, s.logits_rows)
        logits = tp.gather_logits(ops.linear(x, self.lm_head_w, self.lm_head_b, out_fp32=True))
        if a.logits_scale != 1.0:
            logits = logits * a.logits_scale
        if a.final_logit_softcap > 0:
            logits = torch.tanh(logits / a.final_logit_softcap) * a.final_logit_softcap
        return logits

    def forward(self, s: StepInputs, kv: PagedKVCache) -> torch.Tensor:
        """Returns fp32 logits for `s.logits_rows` (or for every token when it is None)."""
        if s.lora_ids is not None and self._lora_batch is None:
            from .lora import LoraBatch
            self._lora_batch = LoraBatch(s.lora_ids, s.lora_names)
            try:
                return self.forward(s, kv)
            finally:
                self._lora_batch = None
        if native.log_flag("enabled") and not (s.input_ids.is_cuda and torch.cuda.is_current_stream_capturing()):
            # tensor dumps (flags model_input_values / model_output_shapes / model_output_values / model_logits)
            from ..utils import debugging
            if not self._dumping:
                self._dumping = True
                try:
                    debugging.dump_inputs(s)
                    out = self.forward(s, kv)
                    debugging.dump_outputs(out, self.last_hidden if isinstance(getattr(self, "last_hidden", None), torch.Tensor) else None)
                    return out
                finally:
                    self._dumping = False
        a = self.arch
        if self._sp_ok(s):
            return self._forward_sp(s, kv)
        if self._fused_step_ok(s):
            return self._forward_fused(s, kv)
        h = s.inputs_embeds if s.inputs_embeds is not None else ops.embedding(s.input_ids, self.embed, a.embed_scale)
        if a.learned_positions:
            h = h + ops.embedding(s.positions, self.pos_embed, 1.0)
        rot = a.applied_rotary_dim
        residual = None
        cos, sin = self.cos, self.sin
        if self.cos_small is not None and s.max_kv_len <= self.rope_original_context:
            cos, sin = self.cos_small, self.sin_small      # the whole step lies within the original context length
        for li, lw in enumerate(self.layers):
            if not a.pre_norm:
                # blocks whose sub-layers read the residual stream itself (their norms follow the sub-layers)
                x = residual = h if residual is None else self._plain(h) + residual
            elif residual is None:
                x, _ = ops.norm(h, lw.ln1_w, a.norm_eps, None, lw.ln1_b, a.layernorm)
                residual = h
            else:
                x, residual = self._add_norm(h, lw.ln1_w, lw.ln1_b, residual)
            if lw.conv_in_w is not None:
                # ---- gated short convolution instead of attention (hybrid models)
                bcx = self._linear(x, lw.conv_in_w, None, lora=self._lora(lw, "in_proj"))
                y = ops.short_conv(bcx, lw.conv_w, lw.conv_b, kv.conv_layer(li), s.slot_mapping, s.positions, s.cu_seqlens, s.past_lens,
                                   s.block_table, kv.block_size)
                h = self._row_parallel(y, lw.conv_out_w, None, self._lora(lw, "out_proj"))
                x, residual = ops.norm(h, lw.ln2_w, a.norm_eps, residual, lw.ln2_b, a.layernorm)
                h = self._mlp(lw, x)
                continue
            if lw.lin_in_w is not None or lw.mamba_in_w is not None:
                h = self._linear_attention(s, kv, li, lw, x) if lw.lin_in_w is not None else self._mamba(s, kv, li, lw, x)
                if a.residual_multiplier != 1.0:
                    h = (h.float() * a.residual_multiplier).to(h.dtype)
                x, residual = ops.norm(h, lw.ln2_w, a.norm_eps, residual, lw.ln2_b, a.layernorm)
                h = self._mlp(lw, x)
                if a.residual_multiplier != 1.0:
                    h = (h.float() * a.residual_multiplier).to(h.dtype)
                continue
            # ---- attention
            qkv = self._linear(x, lw.qkv_w, lw.qkv_b, lora=self._lora(lw, "qkv_proj"))
            kc, vc, windowed = kv.layer(li)
            slots = s.slot_mapping_w if windowed else s.slot_mapping
            table = s.block_table_w if windowed else s.block_table
            lcos, lsin, lrot = self._layer_rope(li, cos, sin, rot)
            if a.qk_norm_full_width and lw.q_norm_w is not None:
                from ..ops import reference as _ref
                qkv = _ref.full_width_qk_norm(qkv, self.heads_local * a.head_dim, self.kv_heads_local * a.head_dim, lw.q_norm_w, lw.k_norm_w, a.norm_eps)
                ops.rope_kv_append(qkv, s.positions, slots, lcos, lsin, kc, vc, self.heads_local, self.kv_heads_local, a.head_dim, lrot,
                                   a.rotary_interleaved)
            elif a.qk_norm_after_rope and lw.q_norm_w is not None:
                from ..ops import reference as _ref
                qkv = _ref.rope_then_head_norm(qkv, s.positions, lcos, lsin, self.heads_local, self.kv_heads_local, a.head_dim, lrot,
                                               a.rotary_interleaved, lw.q_norm_w, lw.k_norm_w, a.norm_eps)
                ops.rope_kv_append(qkv, s.positions, slots, None, None, kc, vc, self.heads_local, self.kv_heads_local, a.head_dim, 0)
            else:
                ops.rope_kv_append(qkv, s.positions, slots, lcos, lsin, kc, vc, self.heads_local, self.kv_heads_local,
                                   a.head_dim, lrot, a.rotary_interleaved, lw.q_norm_w, lw.k_norm_w, a.norm_eps,
                                   s.positions3 if a.mrope_section else None, a.mrope_section, a.mrope_interleaved)
            att = self._attention(s, qkv, kc, vc, table, kv.block_size, lw)
            if lw.attn_gate_w is not None:
                att = (att.float() * torch.sigmoid(self._linear(x, lw.attn_gate_w, None).float())).to(att.dtype)
            h = self._row_parallel(att, lw.o_w, lw.o_b, self._lora(lw, "o_proj"))
            if lw.cross_q_w is not None:
                if s.cross is None:
                    raise RuntimeError("this model needs encoder inputs (set_inputs with audio_features) before tokens")
                x, residual = ops.norm(h, lw.cross_ln_w, a.norm_eps, residual, lw.cross_ln_b, a.layernorm)
                q = self._linear(x, lw.cross_q_w, lw.cross_q_b)
                ck, cv = s.cross.layer(li)
                att = ops.paged_attention(q, ck, cv, s.cu_seqlens, s.cross_lens, s.cross_table, s.cross.block_size, self.heads_local,
                                          self.heads_local, a.head_dim, a.scale, -1, None, 0.0, max_q_len=s.max_q_len,
                                          max_kv_len=s.max_cross_len)
                if s.cross_qk_heads:
                    self._cross_qk(s, li, q, ck)
                h = self._row_parallel(att, lw.cross_o_w, lw.cross_o_b, None)
            if a.parallel_block:
                h = h + self._mlp(lw, x)      # attention and MLP read the same normalised input; one residual join
                continue
            if lw.post_attn_norm_w is not None:
                h, _ = ops.norm(h, lw.post_attn_norm_w, a.norm_eps)
            if a.residual_multiplier != 1.0:
                h = (h.float() * a.residual_multiplier).to(h.dtype)
            if a.pre_norm:
                x, residual = ops.norm(h, lw.ln2_w, a.norm_eps, residual, lw.ln2_b, a.layernorm)
            else:
                x = residual = h + residual
            # ---- MLP (a mixture-of-experts layer may leave its combine step to the residual add + norm that follows)
            h = self._mlp(lw, x, defer=lw.post_ffn_norm_w is None and a.residual_multiplier == 1.0 and a.pre_norm)
            if lw.post_ffn_norm_w is not None:
                h, _ = ops.norm(h, lw.post_ffn_norm_w, a.norm_eps)
            if a.residual_multiplier != 1.0:
                h = (h.float() * a.residual_multiplier).to(h.dtype)
        x, residual = self._add_norm(h, self.final_norm_w, self.final_norm_b, residual)
        return self._logits(s, x)

    def _cross_qk(self, s: StepInputs, li: int, q: torch.Tensor, ck: torch.Tensor) -> None:
        """Scaled query-key scores (before the softmax) of the listed alignment heads of layer `li` against the encoder keys,
        for word-level timestamps (reference: the decoder's `output_cross_qk` tensors and their gather kernels,
        src/models/whisper.cpp:85-103, src/cuda/model_kernels.cu:289-450).  A handful of heads on a debugging / timestamp
        path: tensor ops, positions past a request's encoder length are -inf."""
        if self.tp.size > 1:
            raise RuntimeError("cross-attention scores of alignment heads are not available under tensor parallelism")
        a = self.arch
        scale = a.scale if a.scale else a.head_dim ** -0.5
        T = q.shape[0]
        qh = q.view(T, self.heads_local, a.head_dim)
        bs = s.cross.block_size
        cu, lens = s.cu_seqlens.tolist(), s.cross_lens.tolist()
        for idx, (layer, head) in enumerate(s.cross_qk_heads):
            if layer != li:
                continue
            out = torch.full((T, s.max_cross_len), float("-inf"), dtype=torch.float32, device=q.device)
            for b in range(len(lens)):
                n = lens[b]
                slots = (s.cross_table[b].long()[:, None] * bs + torch.arange(bs, device=q.device)).reshape(-1)[:n]
                k = ck[slots, head].float()                                           # [frames, D]
                out[cu[b]:cu[b + 1], :n] = (qh[cu[b]:cu[b + 1], head].float() @ k.t()) * scale
            s.cross_qk_out[idx] = out

    def fill_cross_cache(self, cross: CrossKVCache, enc_out: torch.Tensor, slots: torch.Tensor) -> None:
        """Projects encoder output rows [S, encoder_hidden] to every layer's cross-attention keys and values and writes
        them at `slots` of the cross cache (once per request; the decoder steps only read them)."""
        a = self.arch
        for li, lw in enumerate(self.layers):
            kv = self._linear(enc_out, lw.cross_kv_w, lw.cross_kv_b)
            ck, cv = cross.layer(li)
            ops.rope_kv_append(kv, slots, slots, None, None, ck, cv, 0, self.heads_local, a.head_dim, 0)

    # ------------------------------------------------------------------------------------ sizing
    def weight_bytes(self) -> int:
        n = 0
        for t in self._all_tensors():
            n += t.numel() * t.element_size()
        return n

    def _all_tensors(self):
        for t in (self.embed, self.final_norm_w, self.final_norm_b, self.lm_head_w, self.lm_head_b, self.cos, self.sin):
            if t is not None:
                yield t
        for lw in self.layers:
            for v in vars(lw).values():
                if isinstance(v, torch.Tensor):
                    yield v
