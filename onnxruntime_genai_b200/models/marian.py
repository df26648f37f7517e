"""Marian translation models with an SSRU decoder (model type "marian-ssru").

What the reference drives as two opaque ONNX sessions (src/models/marian.cpp:8-310: an encoder session over the source
tokens + attention mask, a decoder session that takes one target token, the encoder states, the encoder mask, a step
counter and `rnn_states_prev`, and returns logits + `rnn_states`; the recurrent states follow the beam indices,
marian.cpp:262-306) is here a model of its own:

  encoder   token embedding * sqrt(d) + sinusoidal positions; post-norm transformer layers
            x = LN(x + SelfAttention(x)),  x = LN(x + W2 act(W1 x + b1) + b2)       (bidirectional, padding masked)
  decoder   per layer, one token at a time (Marian's `--transformer-decoder-autoreg rnn --dec-cell ssru`):
            f = sigmoid(Wf x + bf),  c = f * c_prev + (1 - f) * (W x),  x = LN(x + relu(c))      (the SSRU: no self-attention,
            the state c replaces the key / value cache and its size does not grow with the output)
            x = LN(x + CrossAttention(x, encoder states)),  x = LN(x + FFN(x))
  logits    x E^T + b   with the one embedding matrix E shared by source, target and output

The generator hands the source tokens over as the prompt: the first `run` encodes them, projects the encoder states into
every decoder layer's cross-attention keys / values once, and decodes from the start token; every later `run` is one decoder
step.  Beam search reorders the recurrent states and the (per row) view of the cross-attention cache by the beam indices.

Weights live in `encoder.onnx` / `decoder.onnx` as initializers under the names of `weight_shapes` plus one `MarianEncoder` /
`MarianDecoder` node that carries the configuration; `genai_config.json` names the two files the way the reference's
Marian configs do (model.encoder / model.decoder sections with their inputs and outputs).
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..utils import onnx_proto as op
from .arch import ArchConfig

MODEL_TYPE = "marian-ssru"


@dataclass
class MarianConfig:
    vocab_size: int = 32000
    hidden_size: int = 512
    encoder_layers: int = 6
    decoder_layers: int = 6
    num_heads: int = 8
    ffn_size: int = 2048
    activation: str = "relu"            # relu | swish
    max_positions: int = 512
    norm_eps: float = 1e-6
    scale_embedding: bool = True
    bos_token_id: int = 0               # the decoder starts from this token (reference: marian.cpp:196-201)
    eos_token_id: int = 0
    pad_token_id: int = 1

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def weight_shapes(c: MarianConfig) -> Tuple[Dict[str, tuple], Dict[str, tuple]]:
    """(encoder file, decoder file): name -> shape.  Linear weights are [out, in]."""
    H, Fd, V = c.hidden_size, c.ffn_size, c.vocab_size
    enc: Dict[str, tuple] = {"shared.embed.weight": (V, H)}
    for i in range(c.encoder_layers):
        p = f"encoder.layers.{i}."
        for n in ("q", "k", "v", "o"):
            enc[p + f"self_attn.{n}.weight"], enc[p + f"self_attn.{n}.bias"] = (H, H), (H,)
        enc[p + "attn_norm.weight"], enc[p + "attn_norm.bias"] = (H,), (H,)
        enc[p + "ffn.w1.weight"], enc[p + "ffn.w1.bias"] = (Fd, H), (Fd,)
        enc[p + "ffn.w2.weight"], enc[p + "ffn.w2.bias"] = (H, Fd), (H,)
        enc[p + "ffn_norm.weight"], enc[p + "ffn_norm.bias"] = (H,), (H,)
    dec: Dict[str, tuple] = {"shared.embed.weight": (V, H), "decoder.output.bias": (V,)}
    for i in range(c.decoder_layers):
        p = f"decoder.layers.{i}."
        dec[p + "ssru.w.weight"] = (H, H)
        dec[p + "ssru.wf.weight"], dec[p + "ssru.wf.bias"] = (H, H), (H,)
        dec[p + "ssru_norm.weight"], dec[p + "ssru_norm.bias"] = (H,), (H,)
        for n in ("q", "k", "v", "o"):
            dec[p + f"cross_attn.{n}.weight"], dec[p + f"cross_attn.{n}.bias"] = (H, H), (H,)
        dec[p + "cross_norm.weight"], dec[p + "cross_norm.bias"] = (H,), (H,)
        dec[p + "ffn.w1.weight"], dec[p + "ffn.w1.bias"] = (Fd, H), (Fd,)
        dec[p + "ffn.w2.weight"], dec[p + "ffn.w2.bias"] = (H, Fd), (H,)
        dec[p + "ffn_norm.weight"], dec[p + "ffn_norm.bias"] = (H,), (H,)
    return enc, dec


def random_state_dict(c: MarianConfig, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    enc, dec = weight_shapes(c)
    sd: Dict[str, torch.Tensor] = {}
    for name, shape in {**enc, **dec}.items():
        if name.endswith("norm.weight"):
            sd[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            sd[name] = torch.randn(shape, generator=g) * std
    return sd


def sinusoid_positions(length: int, channels: int) -> torch.Tensor:
    """Marian's position signal: sin in the first half of the channels, cos in the second (timescales 1 .. 10000)."""
    half = channels // 2
    inv = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / max(1, half - 1))
    ang = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([torch.sin(ang), torch.cos(ang)], dim=1)


_DT = {"fp32": (torch.float32, op.FLOAT), "bf16": (torch.bfloat16, op.BFLOAT16), "fp16": (torch.float16, op.FLOAT16)}


def _write(path: str, shapes: Dict[str, tuple], sd: Dict[str, torch.Tensor], node_type: str, attrs: dict, inputs, outputs, prec: str):
    tdt, odt = _DT[prec]
    m = op.Model()
    for name, shape in shapes.items():
        t = sd[name].detach().to(tdt).contiguous()
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
        arr = t.view(torch.int16).numpy() if prec == "bf16" else t.numpy()
        m.initializers[name] = op.Tensor(name=name, dtype=odt, dims=tuple(t.shape), raw=np.ascontiguousarray(arr).tobytes())
    m.nodes.append(op.Node(op_type=node_type, name="/" + node_type, inputs=[i for i, _ in inputs] + list(m.initializers),
                           outputs=[o for o, _ in outputs], domain="ogb200", attrs=attrs))
    m.inputs = [op.ValueInfo(n, op.INT32 if "ids" in n or "mask" in n or "length" in n else odt, s) for n, s in inputs]
    m.outputs = [op.ValueInfo(n, odt, s) for n, s in outputs]
    op.save_model(m, path)


def export_marian(c: MarianConfig, out_dir: str, precision: str = "bf16", execution_provider: str = "cuda",
                  state_dict: Optional[Dict[str, torch.Tensor]] = None, seed: int = 0, search: Optional[dict] = None) -> str:
    """encoder.onnx + decoder.onnx + genai_config.json (model.type "marian-ssru")."""
    os.makedirs(out_dir, exist_ok=True)
    prec = "bf16" if precision == "int4" else precision
    sd = state_dict if state_dict is not None else random_state_dict(c, seed)
    enc, dec = weight_shapes(c)
    attrs = asdict(c)
    H = c.hidden_size
    _write(os.path.join(out_dir, "encoder.onnx"), enc, sd, "MarianEncoder", attrs,
           [("input_ids", ("batch_size", "sequence_length")), ("attention_mask", ("batch_size", "sequence_length"))],
           [("encoder_outputs", ("batch_size", "sequence_length", H))], prec)
    _write(os.path.join(out_dir, "decoder.onnx"), dec, sd, "MarianDecoder", attrs,
           [("input_ids", ("batch_size",)), ("encoder_hidden_states", ("batch_size", "sequence_length", H)),
            ("encoder_attention_mask", ("batch_size", "sequence_length")), ("past_key_values_length", (1,)),
            ("rnn_states_prev", (c.decoder_layers, "batch_size", H))],
           [("logits", ("batch_size", c.vocab_size)), ("rnn_states", (c.decoder_layers, "batch_size", H))], prec)
    prov = [{"cuda": {}}] if execution_provider == "cuda" else []
    s = {"max_length": c.max_positions, "num_beams": 1, "num_return_sequences": 1, "do_sample": False, "early_stopping": True,
         "length_penalty": 1.0, "min_length": 0, "past_present_share_buffer": False, "repetition_penalty": 1.0, "temperature": 1.0,
         "top_k": 1, "top_p": 1.0, "no_repeat_ngram_size": 0, "diversity_penalty": 0.0}
    s.update(search or {})
    cfg = {"model": {"type": MODEL_TYPE, "vocab_size": c.vocab_size, "context_length": c.max_positions, "bos_token_id": c.bos_token_id,
                     "eos_token_id": c.eos_token_id, "pad_token_id": c.pad_token_id, "decoder_start_token_id": c.bos_token_id,
                     "encoder": {"filename": "encoder.onnx", "hidden_size": H, "num_attention_heads": c.num_heads,
                                 "num_hidden_layers": c.encoder_layers, "head_size": c.head_dim,
                                 "session_options": {"provider_options": prov},
                                 "inputs": {"input_ids": "input_ids", "attention_mask": "attention_mask"},
                                 "outputs": {"encoder_outputs": "encoder_outputs"}},
                     "decoder": {"filename": "decoder.onnx", "hidden_size": H, "num_attention_heads": c.num_heads,
                                 "num_key_value_heads": c.num_heads, "num_hidden_layers": c.decoder_layers, "head_size": c.head_dim,
                                 "session_options": {"provider_options": prov},
                                 "inputs": {"input_ids": "input_ids", "encoder_hidden_states": "encoder_hidden_states",
                                            "encoder_attention_mask": "encoder_attention_mask",
                                            "past_key_values_length": "past_key_values_length", "rnn_states_prev": "rnn_states_prev"},
                                 "outputs": {"logits": "logits", "rnn_states": "rnn_states"}}},
           "search": s}
    with open(os.path.join(out_dir, "genai_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return out_dir


def _load_file(path: str, node_type: str) -> Tuple[MarianConfig, Dict[str, torch.Tensor]]:
    from .loader import _np_to_torch
    lm = op.LoadedModel(path)
    node = next((n for n in lm.model.nodes if n.op_type == node_type), None)
    if node is None:
        lm.close()
        raise RuntimeError(f"{path}: no {node_type} node (not a {MODEL_TYPE} file of this framework)")
    defaults, kw = MarianConfig(), {}
    for k, v in node.attrs.items():
        if hasattr(defaults, k):
            v = v.decode() if isinstance(v, bytes) else v
            kw[k] = type(getattr(defaults, k))(v)
    sd = {name: _np_to_torch(lm.array(name), lm.info(name).dtype).clone() for name in lm.names()}
    lm.close()
    return MarianConfig(**kw), sd


class MarianModel:
    """Weights + the two forward passes.  On CUDA the linear layers and the layer norms run through this framework's kernels
    (`ops.linear`, `ops.norm`) in bf16; the attention over a few dozen source tokens and the SSRU's element-wise update are
    tensor operations.  On the CPU everything is fp32 tensor operations."""

    def __init__(self, cfg: MarianConfig, sd: Dict[str, torch.Tensor], device, dtype):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype).contiguous() for k, v in sd.items()}
        self.pos = sinusoid_positions(cfg.max_positions, cfg.hidden_size).to(self.device, dtype)
        self.embed_scale = math.sqrt(cfg.hidden_size) if cfg.scale_embedding else 1.0
        c = cfg
        # what the generator and the telemetry read from a decoder
        self.arch = ArchConfig(model_type=MODEL_TYPE, vocab_size=c.vocab_size, hidden_size=c.hidden_size, num_layers=c.decoder_layers,
                               num_heads=c.num_heads, num_kv_heads=c.num_heads, head_dim=c.head_dim, intermediate_size=c.ffn_size,
                               context_length=c.max_positions, norm_eps=c.norm_eps, layernorm=True, bos_token_id=c.bos_token_id,
                               eos_token_id=c.eos_token_id, pad_token_id=c.pad_token_id)
        self.cos_small = None

    @staticmethod
    def load(model_dir: str, config, device, dtype) -> "MarianModel":
        tree = json.loads(config.to_json()).get("model", {})
        enc_file = (tree.get("encoder") or {}).get("filename", "encoder.onnx")
        dec_file = (tree.get("decoder") or {}).get("filename", "decoder.onnx")
        cfg, sd = _load_file(os.path.join(model_dir, enc_file), "MarianEncoder")
        cfg_d, sd_d = _load_file(os.path.join(model_dir, dec_file), "MarianDecoder")
        if asdict(cfg) != asdict(cfg_d):
            raise RuntimeError("marian: encoder and decoder files describe different models")
        sd.update(sd_d)
        return MarianModel(cfg, sd, device, dtype)

    # ------------------------------------------------------------------------------------------ building blocks
    def _linear(self, x: torch.Tensor, name: str) -> torch.Tensor:
        w, b = self.w[name + ".weight"], self.w.get(name + ".bias")
        if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2:
            from .. import ops
            return ops.linear(x.contiguous(), w, b)
        return F.linear(x, w, b)

    def _ln(self, x: torch.Tensor, name: str) -> torch.Tensor:
        w, b = self.w[name + ".weight"], self.w[name + ".bias"]
        if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0:
            from .. import ops
            return ops.norm(x.contiguous(), w, self.cfg.norm_eps, None, b, True)[0]
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), self.cfg.norm_eps).to(x.dtype)

    def _act(self, x: torch.Tensor) -> torch.Tensor:
        return F.relu(x) if self.cfg.activation == "relu" else F.silu(x)

    def _ffn(self, x: torch.Tensor, prefix: str) -> torch.Tensor:
        return self._linear(self._act(self._linear(x, prefix + "ffn.w1")), prefix + "ffn.w2")

    def _embed(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        e = self.w["shared.embed.weight"][ids.long()]
        return (e.float() * self.embed_scale + self.pos[positions.long()].float()).to(self.dtype)

    def _attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, key_mask: Optional[torch.Tensor]) -> torch.Tensor:
        """q [B, Tq, H], k / v [B, Tk, H], key_mask [B, Tk] (True = a real token) -> [B, Tq, H]; softmax in fp32."""
        c = self.cfg
        B, Tq, _ = q.shape
        Tk = k.shape[1]
        qh = q.view(B, Tq, c.num_heads, c.head_dim).transpose(1, 2).float()
        kh = k.view(B, Tk, c.num_heads, c.head_dim).transpose(1, 2).float()
        vh = v.view(B, Tk, c.num_heads, c.head_dim).transpose(1, 2).float()
        s = qh @ kh.transpose(-1, -2) / math.sqrt(c.head_dim)
        if key_mask is not None:
            s = s.masked_fill(~key_mask[:, None, None, :], float("-inf"))
        out = torch.softmax(s, dim=-1) @ vh
        return out.transpose(1, 2).reshape(B, Tq, c.hidden_size).to(q.dtype)

    # ------------------------------------------------------------------------------------------ encoder
    def encode(self, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        """ids int [B, T] (padded on the right), mask bool [B, T] -> encoder states [B, T, H]."""
        B, T = ids.shape
        if T > self.cfg.max_positions:
            raise RuntimeError(f"marian: {T} source tokens exceed max_positions ({self.cfg.max_positions})")
        pos = torch.arange(T, device=ids.device)[None, :].expand(B, T)
        x = self._embed(ids, pos)
        H = self.cfg.hidden_size
        for i in range(self.cfg.encoder_layers):
            p = f"encoder.layers.{i}."
            flat = x.reshape(B * T, H)
            q, k, v = (self._linear(flat, p + f"self_attn.{n}").view(B, T, H) for n in ("q", "k", "v"))
            a = self._linear(self._attention(q, k, v, mask).reshape(B * T, H), p + "self_attn.o")
            flat = self._ln(flat + a, p + "attn_norm")
            flat = self._ln(flat + self._ffn(flat, p), p + "ffn_norm")
            x = flat.view(B, T, H)
        return x

    def cross_cache(self, enc: torch.Tensor) -> List[Tuple[torch.Tensor, torch.Tensor]]:
        """Keys / values of every decoder layer's cross-attention, [B, T, H] each, computed once per source batch."""
        B, T, H = enc.shape
        flat = enc.reshape(B * T, H)
        return [(self._linear(flat, f"decoder.layers.{i}.cross_attn.k").view(B, T, H),
                 self._linear(flat, f"decoder.layers.{i}.cross_attn.v").view(B, T, H)) for i in range(self.cfg.decoder_layers)]

    # ------------------------------------------------------------------------------------------ decoder step
    def decode_step(self, tokens: torch.Tensor, step: int, rnn: torch.Tensor, cross: List[Tuple[torch.Tensor, torch.Tensor]],
                    mask: torch.Tensor, item_of_row: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """tokens int [R]; step = position of these tokens in the target; rnn fp32 [layers, R, H]; cross / mask per source
        item; item_of_row int64 [R] names the source item of every row -> (logits fp32 [R, V], new rnn)."""
        c = self.cfg
        if step >= c.max_positions:
            raise RuntimeError(f"marian: target position {step} exceeds max_positions ({c.max_positions})")
        R = tokens.shape[0]
        x = self._embed(tokens, torch.full((R,), step, device=tokens.device))
        new_rnn = torch.empty_like(rnn)
        m = mask[item_of_row]
        for i in range(c.decoder_layers):
            p = f"decoder.layers.{i}."
            f = torch.sigmoid(self._linear(x, p + "ssru.wf").float())
            cand = self._linear(x, p + "ssru.w").float()
            cell = f * rnn[i] + (1.0 - f) * cand
            new_rnn[i] = cell
            x = self._ln(x + F.relu(cell).to(x.dtype), p + "ssru_norm")
            q = self._linear(x, p + "cross_attn.q")
            k, v = cross[i]
            a = self._attention(q[:, None, :], k[item_of_row], v[item_of_row], m)[:, 0, :]
            x = self._ln(x + self._linear(a.contiguous(), p + "cross_attn.o"), p + "cross_norm")
            x = self._ln(x + self._ffn(x, p), p + "ffn_norm")
        logits = x.float() @ self.w["shared.embed.weight"].float().t() + self.w["decoder.output.bias"].float()
        return logits, new_rnn


class MarianState:
    """What `Generator` needs from a sequence state (`run`, `reorder_rows`, `rewind`, `graph_ok`), for the encoder-decoder
    flow: the first `run` receives the source tokens of every row, later runs one target token per row."""

    def __init__(self, model: MarianModel, rows: int, max_length: int):
        self.m, self.rows, self.max_length = model, rows, max_length
        self.kv_len = [0] * rows
        self.cross = None
        self._reset()

    def _reset(self):
        self.cross = self.mask = self.item_of_row = None
        self.step = 0
        self.rnn = torch.zeros(self.m.cfg.decoder_layers, self.rows, self.m.cfg.hidden_size, dtype=torch.float32, device=self.m.device)
        self.kv_len = [0] * self.rows

    def graph_ok(self) -> bool:
        return False

    def set_alignment_heads(self, heads) -> None:
        raise RuntimeError("marian: cross_qk outputs are not available")

    def run(self, row_tokens: List[List[int]], want_all_logits: bool = False, inputs_embeds=None, positions3=None):
        if want_all_logits or inputs_embeds is not None:
            raise RuntimeError("marian: only next-token logits from token ids are available")
        m, dev = self.m, self.m.device
        if len(row_tokens) != self.rows:
            raise RuntimeError(f"marian: expected tokens for {self.rows} rows")
        with torch.no_grad():
            if self.cross is None:
                # ---- the prompt is the source text: rows of one batch entry (its beams) carry the same tokens, encode each once
                items, item_of_row = [], []
                for toks in row_tokens:
                    if not items or toks != items[-1]:
                        items.append(list(toks))
                    item_of_row.append(len(items) - 1)
                T = max(len(t) for t in items)
                ids = torch.full((len(items), T), m.cfg.pad_token_id, dtype=torch.int64)
                mask = torch.zeros(len(items), T, dtype=torch.bool)
                for i, t in enumerate(items):
                    ids[i, :len(t)] = torch.tensor(t, dtype=torch.int64)
                    mask[i, :len(t)] = True
                self.mask = mask.to(dev)
                enc = m.encode(ids.to(dev), self.mask)
                self.cross = m.cross_cache(enc)
                self.item_of_row = torch.tensor(item_of_row, dtype=torch.int64, device=dev)
                tokens = torch.full((self.rows,), m.cfg.bos_token_id, dtype=torch.int64, device=dev)
                for r, t in enumerate(row_tokens):
                    self.kv_len[r] = len(t)
            else:
                if any(len(t) != 1 for t in row_tokens):
                    raise RuntimeError("marian: after the source text, one token per row and step")
                tokens = torch.tensor([t[0] for t in row_tokens], dtype=torch.int64, device=dev)
                for r in range(self.rows):
                    self.kv_len[r] += 1
            logits, self.rnn = m.decode_step(tokens, self.step, self.rnn, self.cross, self.mask, self.item_of_row)
            self.step += 1
        return logits, list(range(self.rows))

    def reorder_rows(self, src_rows: List[int]):
        idx = torch.tensor(src_rows, dtype=torch.int64, device=self.m.device)
        self.rnn = self.rnn[:, idx].contiguous()
        if self.item_of_row is not None:
            self.item_of_row = self.item_of_row[idx].contiguous()
        self.kv_len = [self.kv_len[s] for s in src_rows]

    def rewind(self, row: int, length: int):
        if length != 0:
            raise RuntimeError("marian: only rewind_to(0) is supported (the recurrent state cannot be cropped)")
        if row == 0:
            self._reset()
