"""Audio that arrives piece by piece: voice-activity gate, streaming log-mel front end, and a transcription session over a
speech transducer.

Reference behaviour restated here: `src/models/silero_vad.cpp` (a recurrent classifier over windows of 512 samples at 16 kHz -
256 at 8 kHz - each prefixed by the last 64 / 32 samples of the window before it, state carried between windows; a chunk
contains speech when any of its windows reaches the threshold), `src/models/streaming_processor.cpp:13-66` (chunks of
`chunk_samples`; a silent chunk is still kept for context until max(prefix_padding, silence_duration) chunks of silence in a
row, after that silent chunks are dropped), `src/models/nemotron_streaming_processor.cpp` / `parakeet_processor.cpp` (log-mel
features of the kept audio handed to the generator as `audio_features`).

  VoiceActivityDetector   the classifier (one linear layer over context + window, an LSTM cell, a sigmoid output) with its
                          state; weights in `vad.onnx` (`export_vad`)
  StreamingProcessor      `process(samples)` -> the log-mel frames that became complete (or None); `flush()` at the end
  StreamingSession        `feed(samples)` -> tokens emitted for the audio so far; `finish()` -> the rest.  Every batch of new
                          frames is encoded together with `left_context_frames` of the frames before it.

Log-mel frames for streaming are not centred: frame i covers samples [i * hop, i * hop + n_fft), natural log of the mel
energies with a fixed floor - the same frames whether the audio comes in one piece or in many.
"""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional

import numpy as np
import torch

from .utils import onnx_proto as op

VAD_STATE = 128


def log_mel_frames(samples: np.ndarray, n_mels: int = 80, n_fft: int = 400, hop: int = 160, sample_rate: int = 16000) -> np.ndarray:
    """float32 [n_mels, frames] with frames = (len - n_fft) // hop + 1 (0 when the audio is shorter than one window)."""
    from .multimodal import mel_filter_bank
    x = torch.from_numpy(np.ascontiguousarray(samples, dtype=np.float32))
    if x.numel() < n_fft:
        return np.zeros((n_mels, 0), dtype=np.float32)
    spec = torch.stft(x, n_fft, hop, window=torch.hann_window(n_fft), center=False, return_complex=True)
    mel = torch.from_numpy(mel_filter_bank(n_mels, n_fft, sample_rate)) @ (spec.abs() ** 2)
    return torch.log(mel + 2.0 ** -24).numpy().astype(np.float32)


# ------------------------------------------------------------------------------------------------ voice activity
def vad_weight_shapes(sample_rate: int, features: int = 64) -> Dict[str, tuple]:
    factor = sample_rate // 8000
    n_in = (256 + 32) * factor
    return {"vad.in.weight": (features, n_in), "vad.in.bias": (features,), "vad.lstm.w_ih": (4 * VAD_STATE, features),
            "vad.lstm.w_hh": (4 * VAD_STATE, VAD_STATE), "vad.lstm.b": (4 * VAD_STATE,), "vad.out.weight": (1, VAD_STATE), "vad.out.bias": (1,)}


def export_vad(out_dir: str, state_dict: Dict[str, torch.Tensor], sample_rate: int = 16000, filename: str = "vad.onnx") -> str:
    m = op.Model()
    for name, shape in vad_weight_shapes(sample_rate, state_dict["vad.in.weight"].shape[0]).items():
        t = state_dict[name].detach().float().contiguous()
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
        m.initializers[name] = op.Tensor(name=name, dtype=op.FLOAT, dims=tuple(t.shape), raw=t.numpy().tobytes())
    m.nodes.append(op.Node(op_type="SileroVad", name="/vad/SileroVad", inputs=["input", "state", "sr"] + list(m.initializers),
                           outputs=["output", "stateN"], domain="ogb200", attrs={"sample_rate": int(sample_rate)}))
    m.inputs = [op.ValueInfo("input", op.FLOAT, (1, "samples")), op.ValueInfo("state", op.FLOAT, (2, 1, VAD_STATE))]
    m.outputs = [op.ValueInfo("output", op.FLOAT, (1, 1)), op.ValueInfo("stateN", op.FLOAT, (2, 1, VAD_STATE))]
    path = os.path.join(out_dir, filename)
    op.save_model(m, path)
    return path


class VoiceActivityDetector:
    def __init__(self, state_dict: Dict[str, torch.Tensor], sample_rate: int = 16000, threshold: float = 0.5):
        if sample_rate not in (8000, 16000):
            raise RuntimeError("the voice-activity detector runs at 8 kHz or 16 kHz")
        factor = sample_rate // 8000
        self.window, self.context_size, self.threshold = 256 * factor, 32 * factor, float(threshold)
        self.w = {k: v.float() for k, v in state_dict.items()}
        self.reset()

    @staticmethod
    def load(path: str, sample_rate: int, threshold: float) -> "VoiceActivityDetector":
        from .models.loader import _np_to_torch
        lm = op.LoadedModel(path)
        sd = {name: _np_to_torch(lm.array(name), lm.info(name).dtype).clone() for name in lm.names()}
        lm.close()
        return VoiceActivityDetector(sd, sample_rate, threshold)

    def reset(self):
        self.state = torch.zeros(2, VAD_STATE)
        self.context = torch.zeros(self.context_size)

    def process_window(self, samples: np.ndarray) -> float:
        """Speech probability of one window (exactly `window` samples); updates the recurrent state and the context."""
        if len(samples) != self.window:
            raise RuntimeError(f"the detector expects windows of {self.window} samples")
        x = torch.cat([self.context, torch.from_numpy(np.ascontiguousarray(samples, dtype=np.float32))])
        f = torch.relu(self.w["vad.in.weight"] @ x + self.w["vad.in.bias"])
        h, c = self.state[0], self.state[1]
        g = self.w["vad.lstm.w_ih"] @ f + self.w["vad.lstm.w_hh"] @ h + self.w["vad.lstm.b"]
        S = VAD_STATE
        i, fg, gg, o = torch.sigmoid(g[:S]), torch.sigmoid(g[S:2 * S]), torch.tanh(g[2 * S:3 * S]), torch.sigmoid(g[3 * S:])
        c = fg * c + i * gg
        h = o * torch.tanh(c)
        self.state = torch.stack([h, c])
        self.context = x[-self.context_size:].clone()
        return float(torch.sigmoid(self.w["vad.out.weight"] @ h + self.w["vad.out.bias"])[0])

    def contains_speech(self, chunk: np.ndarray) -> bool:
        """True as soon as one of the chunk's non-overlapping windows reaches the threshold (a tail shorter than a window is
        not looked at)."""
        for s in range(0, len(chunk) - self.window + 1, self.window):
            if self.process_window(chunk[s:s + self.window]) >= self.threshold:
                return True
        return False


# ------------------------------------------------------------------------------------------------ streaming front end
class StreamingProcessor:
    """Turns a stream of samples into log-mel frames, chunk by chunk, dropping long silences when the model has a `vad`
    section."""

    def __init__(self, model):
        tree = json.loads(model.config.to_json()).get("model", {})
        self.sample_rate = int(tree.get("sample_rate", 16000))
        self.chunk_samples = int(tree.get("chunk_samples", 8960))
        with open(os.path.join(model.config.config_path, "audio_processor_config.json")) as f:
            p = json.load(f)["processor"]
        self.n_mels, self.n_fft, self.hop = int(p["num_mel_bins"]), int(p["n_fft"]), int(p["hop_length"])
        self.vad = None
        vad = tree.get("vad") or {}
        if vad.get("filename"):
            self.vad = VoiceActivityDetector.load(os.path.join(model.config.config_path, vad["filename"]), self.sample_rate,
                                                  float(vad.get("threshold", 0.5)))
            chunk_ms = self.chunk_samples / self.sample_rate * 1000.0
            self.silence_chunks = max(1, int(float(vad.get("silence_duration_ms", 500)) / chunk_ms))
            self.prefix_chunks = max(1, int(float(vad.get("prefix_padding_ms", 300)) / chunk_ms))
        self.pending = np.zeros(0, dtype=np.float32)     # samples not yet grouped into a chunk
        self.audio = np.zeros(0, dtype=np.float32)       # kept samples whose frames are not complete yet
        self.silent_run = 0
        self.dropped_chunks = 0

    def _should_drop(self, chunk: np.ndarray) -> bool:
        if self.vad is None:
            return False
        if self.vad.contains_speech(chunk):
            self.silent_run = 0
            return False
        self.silent_run += 1
        return self.silent_run >= max(self.prefix_chunks, self.silence_chunks)

    def _frames(self) -> Optional[np.ndarray]:
        n = (len(self.audio) - self.n_fft) // self.hop + 1 if len(self.audio) >= self.n_fft else 0
        if n <= 0:
            return None
        out = log_mel_frames(self.audio[:(n - 1) * self.hop + self.n_fft], self.n_mels, self.n_fft, self.hop, self.sample_rate)
        self.audio = self.audio[n * self.hop:]
        return out

    def process(self, samples) -> Optional[np.ndarray]:
        """Takes mono float samples at the model's rate; returns the log-mel frames [n_mels, n] completed by them, or None."""
        self.pending = np.concatenate([self.pending, np.asarray(samples, dtype=np.float32).reshape(-1)])
        outs = []
        while len(self.pending) >= self.chunk_samples:
            chunk, self.pending = self.pending[:self.chunk_samples], self.pending[self.chunk_samples:]
            if self._should_drop(chunk):
                self.dropped_chunks += 1
                self.audio = np.zeros(0, dtype=np.float32)      # framing restarts at the next kept chunk
                continue
            self.audio = np.concatenate([self.audio, chunk])
            f = self._frames()
            if f is not None:
                outs.append(f)
        return np.concatenate(outs, axis=1) if outs else None

    _OPTIONS = ("threshold", "silence_duration_ms", "prefix_padding_ms")

    def set_option(self, key: str, value: str):
        """Options of the voice-activity gate (reference: OgaStreamingProcessorSetOption): threshold, silence_duration_ms,
        prefix_padding_ms."""
        if key not in self._OPTIONS:
            raise RuntimeError(f"unknown streaming option {key!r} (known: {', '.join(self._OPTIONS)})")
        if self.vad is None:
            raise RuntimeError("this model has no voice-activity detector")
        v = float(value)
        chunk_ms = self.chunk_samples / self.sample_rate * 1000.0
        if key == "threshold":
            if not 0.0 <= v <= 1.0:
                raise RuntimeError("threshold must lie in [0, 1]")
            self.vad.threshold = v
        elif key == "silence_duration_ms":
            self.silence_chunks = max(1, int(v / chunk_ms))
        else:
            self.prefix_chunks = max(1, int(v / chunk_ms))

    def get_option(self, key: str) -> str:
        if key not in self._OPTIONS:
            raise RuntimeError(f"unknown streaming option {key!r} (known: {', '.join(self._OPTIONS)})")
        if self.vad is None:
            raise RuntimeError("this model has no voice-activity detector")
        chunk_ms = self.chunk_samples / self.sample_rate * 1000.0
        if key == "threshold":
            return repr(float(self.vad.threshold))
        return repr(float((self.silence_chunks if key == "silence_duration_ms" else self.prefix_chunks) * chunk_ms))

    def flush(self) -> Optional[np.ndarray]:
        """The frames of the samples that did not fill a chunk (the end of the recording)."""
        if len(self.pending):
            self.audio = np.concatenate([self.audio, self.pending])
            self.pending = np.zeros(0, dtype=np.float32)
        return self._frames()


def frames_as_inputs(frames: np.ndarray):
    """Log-mel frames [n_mels, n] as the generator input {"audio_features": [1, n_mels, n]}."""
    from .api import NamedTensors
    out = NamedTensors()
    out["audio_features"] = np.ascontiguousarray(frames, dtype=np.float32)[None]
    return out


class StreamingSession:
    """Transcribes while the audio arrives: `feed(samples)` returns the tokens the transducer emitted for the audio so far."""

    def __init__(self, model):
        from .models.transducer import TransducerModel, TransducerSearch
        if not isinstance(model.decoder, TransducerModel):
            raise RuntimeError("this model has no streaming audio component")
        self.m = model.decoder
        self.processor = StreamingProcessor(model)
        self.search = TransducerSearch(self.m)
        self.context: Optional[torch.Tensor] = None      # the last left_context_frames log-mel frames
        self.tokens: List[int] = []
        self.done = False

    def _consume(self, frames: Optional[np.ndarray]) -> List[int]:
        if frames is not None and frames.shape[1] >= 2:
            new = torch.from_numpy(frames)
            left = self.m.cfg.left_context_frames
            ctx = self.context if (self.context is not None and left > 0) else new[:, :0]
            ctx = ctx[:, ctx.shape[1] % 2:]                # an even context keeps the stride-2 front end aligned
            enc = self.m.encode(torch.cat([ctx, new], dim=1).to(self.m.device))
            self.search.add_frames(enc[ctx.shape[1] // 2:])
            if left > 0:
                self.context = torch.cat([ctx, new], dim=1)[:, -left:]
        out = []
        while True:
            tok = self.search.next_token()
            if tok is None or tok == self.m.cfg.blank_id:
                break
            out.append(tok)
        self.tokens += out
        return out

    def feed(self, samples) -> List[int]:
        if self.done:
            raise RuntimeError("the session is finished")
        return self._consume(self.processor.process(samples))

    def finish(self) -> List[int]:
        out = self._consume(self.processor.flush())
        self.search.finish()
        self.done = True
        return out
