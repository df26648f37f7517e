"""Speech transducers: an acoustic encoder, a prediction network over the emitted tokens, a joiner, and the greedy
frame-synchronous search that ties them together - RNN-T (model type "nemotron_speech") and TDT, the token-and-duration
transducer (model type "parakeet_tdt").

What the reference runs as three ONNX sessions plus a C++ loop (src/models/parakeet.cpp:395-535 EmitNextToken for TDT,
src/models/nemotron_speech.cpp for RNN-T, src/models/transducer_state.h) is here:

  encoder     `models/encoder.py::TransformerEncoder` (audio kind): log-mel frames -> encoder frames (stride 2)
  predictor   token embedding -> LSTM layers; its output after the tokens emitted so far (it starts from the blank token)
  joiner      out( relu( enc_proj(frame) + pred_proj(predictor output) ) ) -> [vocab logits | duration logits]
  search      at encoder frame t: token = argmax of the vocab logits.  RNN-T: blank -> t += 1; otherwise emit the token, feed it
              to the predictor and stay on the frame, at most `max_symbols_per_step` times.  TDT: the duration head picks how
              many frames to skip (index 0 is forbidden together with blank, which would never advance); a non-blank token is
              emitted and fed to the predictor; a skip of 0 keeps the frame until `max_symbols_per_step` tokens were emitted
              there, then one frame is skipped.  When the audio is used up the blank id is returned: it is the model's
              end-of-sequence id.

The utterance is encoded in chunks of `chunk_frames` log-mel frames with `left_context_frames` of earlier audio re-encoded in
front of every chunk (bounded attention span and memory for long recordings); only the chunk's own frames are searched.

`TransducerState` gives `Generator` what it expects from a sequence state: every `run` emits the next token and returns
logits with all their mass on it, so that the ordinary greedy search commits it; batch 1.  `StreamingSession`
(`streaming.py`) drives the same search over audio that arrives piece by piece.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..utils import onnx_proto as op
from .arch import ArchConfig

MODEL_TYPES = ("parakeet_tdt", "nemotron_speech")


@dataclass
class TransducerConfig:
    vocab_size: int = 1025              # token logits of the joiner, the blank included
    blank_id: int = 1024
    encoder_hidden: int = 512
    pred_hidden: int = 640
    pred_layers: int = 2
    joint_hidden: int = 640
    tdt_durations: str = ""             # "0,1,2,3,4" for TDT; empty: RNN-T
    max_symbols_per_step: int = 10
    chunk_frames: int = 0               # log-mel frames encoded at a time (0: the whole utterance at once)
    left_context_frames: int = 0

    @property
    def durations(self) -> List[int]:
        return [int(v) for v in self.tdt_durations.split(",") if v.strip()]


def weight_shapes(c: TransducerConfig) -> Tuple[Dict[str, tuple], Dict[str, tuple]]:
    """(decoder file = prediction network, joiner file)."""
    P, J = c.pred_hidden, c.joint_hidden
    dec: Dict[str, tuple] = {"predictor.embed.weight": (c.vocab_size, P)}
    for l in range(c.pred_layers):
        p = f"predictor.lstm.{l}."
        dec[p + "w_ih"], dec[p + "w_hh"], dec[p + "b_ih"], dec[p + "b_hh"] = (4 * P, P), (4 * P, P), (4 * P,), (4 * P,)
    join = {"joiner.enc.weight": (J, c.encoder_hidden), "joiner.enc.bias": (J,), "joiner.pred.weight": (J, P), "joiner.pred.bias": (J,),
            "joiner.out.weight": (c.vocab_size + len(c.durations), J), "joiner.out.bias": (c.vocab_size + len(c.durations),)}
    return dec, join


def random_state_dict(c: TransducerConfig, seed: int = 0, std: float = 0.2) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    dec, join = weight_shapes(c)
    return {n: torch.randn(s, generator=g) * std for n, s in {**dec, **join}.items()}


_DT = {"fp32": (torch.float32, op.FLOAT), "bf16": (torch.bfloat16, op.BFLOAT16), "fp16": (torch.float16, op.FLOAT16)}


def _write(path, shapes, sd, node_type, attrs, inputs, outputs, prec):
    tdt, odt = _DT[prec]
    m = op.Model()
    for name, shape in shapes.items():
        t = sd[name].detach().to(tdt).contiguous()
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
        arr = t.view(torch.int16).numpy() if prec == "bf16" else t.numpy()
        m.initializers[name] = op.Tensor(name=name, dtype=odt, dims=tuple(t.shape), raw=np.ascontiguousarray(arr).tobytes())
    m.nodes.append(op.Node(op_type=node_type, name="/" + node_type, inputs=list(inputs) + list(m.initializers), outputs=list(outputs),
                           domain="ogb200", attrs=attrs))
    m.inputs = [op.ValueInfo(n, odt, ("batch_size", "n")) for n in inputs]
    m.outputs = [op.ValueInfo(n, odt, ("batch_size", "n")) for n in outputs]
    op.save_model(m, path)


def export_transducer(c: TransducerConfig, enc, out_dir: str, model_type: str = "parakeet_tdt", precision: str = "bf16",
                      execution_provider: str = "cuda", state_dict=None, encoder_state_dict=None, seed: int = 0, num_mels: int = 80,
                      sample_rate: int = 16000, chunk_samples: int = 8960, vad: Optional[dict] = None) -> str:
    """encoder.onnx (audio encoder of `models/encoder.py`), decoder.onnx (prediction network), joiner.onnx, genai_config.json with
    the reference's sections (model.encoder / decoder / joiner, blank_id, max_symbols_per_step, tdt_durations, sample_rate,
    chunk_samples, optional vad) and audio_processor_config.json for the log-mel front end."""
    from .encoder import export_encoder, random_encoder_state_dict
    if model_type not in MODEL_TYPES:
        raise ValueError(f"model_type must be one of {MODEL_TYPES}")
    if (model_type == "parakeet_tdt") != bool(c.durations):
        raise ValueError("parakeet_tdt needs tdt_durations; nemotron_speech (RNN-T) takes none")
    if enc.hidden_size != c.encoder_hidden:
        raise ValueError("the joiner's encoder projection must match the encoder's hidden size")
    os.makedirs(out_dir, exist_ok=True)
    prec = "bf16" if precision == "int4" else precision
    sd = state_dict if state_dict is not None else random_state_dict(c, seed)
    dec, join = weight_shapes(c)
    export_encoder(enc, out_dir, "encoder.onnx", encoder_state_dict or random_encoder_state_dict(enc, seed), prec)
    _write(os.path.join(out_dir, "decoder.onnx"), dec, sd, "TransducerPredictor", asdict(c), ["targets", "lstm_hidden_state", "lstm_cell_state"],
           ["outputs", "lstm_hidden_state_out", "lstm_cell_state_out"], prec)
    _write(os.path.join(out_dir, "joiner.onnx"), join, sd, "TransducerJoiner", asdict(c), ["encoder_outputs", "decoder_outputs"], ["logits"], prec)
    prov = [{"cuda": {}}] if execution_provider == "cuda" else []
    model = {"type": model_type, "vocab_size": c.vocab_size, "context_length": 4096, "bos_token_id": c.blank_id, "eos_token_id": c.blank_id,
             "pad_token_id": c.blank_id, "blank_id": c.blank_id, "max_symbols_per_step": c.max_symbols_per_step, "sample_rate": sample_rate,
             "chunk_samples": chunk_samples, "num_mels": num_mels,
             "encoder": {"filename": "encoder.onnx", "hidden_size": c.encoder_hidden, "session_options": {"provider_options": prov},
                         "inputs": {"audio_features": "audio_features"}, "outputs": {"encoder_outputs": "encoder_outputs"}},
             "decoder": {"filename": "decoder.onnx", "hidden_size": c.pred_hidden, "num_hidden_layers": c.pred_layers,
                         "session_options": {"provider_options": prov},
                         "inputs": {"targets": "targets", "lstm_hidden_state": "lstm_hidden_state", "lstm_cell_state": "lstm_cell_state"},
                         "outputs": {"outputs": "outputs", "lstm_hidden_state": "lstm_hidden_state_out", "lstm_cell_state": "lstm_cell_state_out"}},
             "joiner": {"filename": "joiner.onnx", "inputs": {"encoder_outputs": "encoder_outputs", "decoder_outputs": "decoder_outputs"},
                        "outputs": {"logits": "logits"}}}
    if c.durations:
        model["tdt_durations"] = c.durations
    if vad:
        model["vad"] = dict(vad)
    cfg = {"model": model, "search": {"max_length": 4096, "num_beams": 1, "num_return_sequences": 1, "do_sample": False, "top_k": 1,
                                      "top_p": 1.0, "temperature": 1.0, "repetition_penalty": 1.0, "min_length": 0, "early_stopping": True,
                                      "length_penalty": 1.0, "no_repeat_ngram_size": 0, "diversity_penalty": 0.0,
                                      "past_present_share_buffer": False}}
    with open(os.path.join(out_dir, "genai_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    with open(os.path.join(out_dir, "audio_processor_config.json"), "w") as f:
        json.dump({"processor": {"name": "log_mel", "sample_rate": sample_rate, "num_mel_bins": num_mels, "n_fft": 400, "hop_length": 160,
                                 "num_frames": 0}}, f, indent=2)
    return out_dir


def _load_file(path: str, node_type: str):
    from .loader import _np_to_torch
    lm = op.LoadedModel(path)
    node = next((n for n in lm.model.nodes if n.op_type == node_type), None)
    if node is None:
        lm.close()
        raise RuntimeError(f"{path}: no {node_type} node (not a transducer file of this framework)")
    defaults, kw = TransducerConfig(), {}
    for k, v in node.attrs.items():
        if hasattr(defaults, k):
            v = v.decode() if isinstance(v, bytes) else v
            kw[k] = type(getattr(defaults, k))(v)
    sd = {name: _np_to_torch(lm.array(name), lm.info(name).dtype).clone() for name in lm.names()}
    lm.close()
    return TransducerConfig(**kw), sd


class TransducerModel:
    def __init__(self, cfg: TransducerConfig, sd: Dict[str, torch.Tensor], encoder, device, dtype):
        self.cfg, self.encoder, self.device, self.dtype = cfg, encoder, torch.device(device), dtype
        # the prediction network and the joiner are a few small matrices applied to single vectors: fp32 tensor operations
        self.w = {k: v.to(self.device, torch.float32).contiguous() for k, v in sd.items()}
        c = cfg
        self.arch = ArchConfig(model_type="transducer", vocab_size=c.vocab_size, hidden_size=c.pred_hidden, num_layers=c.pred_layers,
                               num_heads=1, num_kv_heads=1, head_dim=c.pred_hidden, intermediate_size=c.joint_hidden, context_length=4096,
                               bos_token_id=c.blank_id, eos_token_id=c.blank_id, pad_token_id=c.blank_id)
        self.cos_small = None

    @staticmethod
    def load(model_dir: str, config, device, dtype) -> "TransducerModel":
        from .encoder import TransformerEncoder
        tree = json.loads(config.to_json()).get("model", {})
        name = lambda sec, default: (tree.get(sec) or {}).get("filename", default)
        cfg, sd = _load_file(os.path.join(model_dir, name("decoder", "decoder.onnx")), "TransducerPredictor")
        _, sd_j = _load_file(os.path.join(model_dir, name("joiner", "joiner.onnx")), "TransducerJoiner")
        sd.update(sd_j)
        enc = TransformerEncoder.load(os.path.join(model_dir, name("encoder", "encoder.onnx")), device, dtype)
        return TransducerModel(cfg, sd, enc, device, dtype)

    # ---- the three networks
    def encode(self, features: torch.Tensor) -> torch.Tensor:
        """log-mel [n_mels, frames] -> encoder frames [frames / 2, H] (fp32)."""
        out, lens = self.encoder.encode_audio(features[None])
        return out.view(1, lens[0], -1)[0].float()

    def predictor_start(self):
        P, L = self.cfg.pred_hidden, self.cfg.pred_layers
        z = lambda: torch.zeros(L, P, dtype=torch.float32, device=self.device)
        return self.predictor_step(self.cfg.blank_id, (z(), z()))

    def predictor_step(self, token: int, state):
        """-> (output [P], (h [L, P], c [L, P])) after feeding `token`."""
        h, c = state
        x = self.w["predictor.embed.weight"][token]
        nh, nc = torch.empty_like(h), torch.empty_like(c)
        P = self.cfg.pred_hidden
        for l in range(self.cfg.pred_layers):
            p = f"predictor.lstm.{l}."
            g = self.w[p + "w_ih"] @ x + self.w[p + "b_ih"] + self.w[p + "w_hh"] @ h[l] + self.w[p + "b_hh"]
            i, f, gg, o = torch.sigmoid(g[:P]), torch.sigmoid(g[P:2 * P]), torch.tanh(g[2 * P:3 * P]), torch.sigmoid(g[3 * P:])
            nc[l] = f * c[l] + i * gg
            nh[l] = o * torch.tanh(nc[l])
            x = nh[l]
        return x, (nh, nc)

    def joint(self, frame: torch.Tensor, pred: torch.Tensor) -> torch.Tensor:
        z = F.relu(self.w["joiner.enc.weight"] @ frame + self.w["joiner.enc.bias"] + self.w["joiner.pred.weight"] @ pred + self.w["joiner.pred.bias"])
        return self.w["joiner.out.weight"] @ z + self.w["joiner.out.bias"]


class TransducerSearch:
    """The greedy search over encoder frames that arrive in pieces (`add_frames`); `next_token` returns the next emitted token,
    None when it needs more frames, and the blank id once `finish()` was called and the frames are used up."""

    def __init__(self, model: TransducerModel):
        self.m = model
        self.frames: Optional[torch.Tensor] = None      # encoder frames not yet consumed start at self.t
        self.t = 0
        self.symbols_this_frame = 0
        self.finished = False
        self.pred_out, self.pred_state = model.predictor_start()

    def add_frames(self, frames: torch.Tensor):
        if self.frames is None or self.t >= self.frames.shape[0]:
            self.t = 0 if self.frames is None else self.t - self.frames.shape[0]      # a skip may reach into the next piece
            self.frames = frames
        else:
            self.frames = torch.cat([self.frames[self.t:], frames])
            self.t = 0

    def finish(self):
        self.finished = True

    def next_token(self) -> Optional[int]:
        c = self.m.cfg
        durations = c.durations
        V = c.vocab_size
        with torch.no_grad():
            while True:
                if self.frames is None or self.t >= self.frames.shape[0]:
                    return c.blank_id if self.finished else None
                logits = self.m.joint(self.frames[self.t], self.pred_out)
                token = int(torch.argmax(logits[:V]))
                emitted = token != c.blank_id
                if durations:
                    start = 0 if emitted else 1      # (blank, stay) would neither emit nor advance
                    skip = durations[start + int(torch.argmax(logits[V + start:V + len(durations)]))]
                else:
                    skip = 0 if emitted else 1
                if emitted:
                    self.symbols_this_frame += 1
                    self.pred_out, self.pred_state = self.m.predictor_step(token, self.pred_state)
                if skip > 0:
                    self.symbols_this_frame = 0
                elif self.symbols_this_frame >= c.max_symbols_per_step:
                    self.symbols_this_frame = 0
                    skip = 1
                self.t += skip
                if emitted:
                    return token


def chunked_encode(model: TransducerModel, features: torch.Tensor):
    """Yields the encoder frames of the utterance chunk by chunk: `chunk_frames` log-mel frames at a time, each encoded together
    with `left_context_frames` of the audio before it, whose frames are dropped again."""
    c = model.cfg
    total = features.shape[1]
    if c.chunk_frames <= 0 or total <= c.chunk_frames:
        yield model.encode(features)
        return
    for s in range(0, total, c.chunk_frames):
        e = min(total, s + c.chunk_frames)
        lo = max(0, s - c.left_context_frames)
        lo -= (s - lo) % 2                           # the stride-2 front end keeps the chunk's frames aligned
        lo = max(0, lo)
        out = model.encode(features[:, lo:e])
        yield out[(s - lo) // 2:]


class TransducerState:
    """Sequence state for `Generator` (batch 1): `set_audio` stages the utterance's log-mel features; every `run` emits one token."""

    def __init__(self, model: TransducerModel, rows: int, max_length: int):
        if rows != 1:
            raise RuntimeError("speech transducers decode one utterance at a time (batch_size 1, no beams)")
        self.m, self.rows, self.max_length = model, rows, max_length
        self.kv_len = [0]
        self.search = TransducerSearch(model)
        self._chunks = None

    def set_audio(self, features: torch.Tensor):
        """features [n_mels, frames] (already normalised log-mel)."""
        self.search = TransducerSearch(self.m)
        self._chunks = chunked_encode(self.m, features.to(self.m.device))

    def graph_ok(self) -> bool:
        return False

    def set_alignment_heads(self, heads) -> None:
        raise RuntimeError("transducers have no cross-attention")

    def run(self, row_tokens, want_all_logits: bool = False, inputs_embeds=None, positions3=None, device_ids=None):
        if self._chunks is None:
            raise RuntimeError("set the audio_features input before generating")
        while True:
            tok = self.search.next_token()
            if tok is not None:
                break
            nxt = next(self._chunks, None)
            if nxt is None:
                self.search.finish()
            else:
                self.search.add_frames(nxt)
        self.kv_len[0] += 1
        logits = torch.full((1, self.m.cfg.vocab_size), -1e9, dtype=torch.float32, device=self.m.device)
        logits[0, tok] = 0.0
        return logits, [0]

    def reorder_rows(self, src_rows):
        pass

    def rewind(self, row: int, length: int):
        if length != 0:
            raise RuntimeError("transducers: only rewind_to(0) is supported")
        self.kv_len = [0]
        self._chunks = None
