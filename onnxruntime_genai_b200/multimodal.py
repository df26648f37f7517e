"""Multimodal inputs: `Images`, `Audios` and the `MultiModalProcessor` returned by `Model.create_multimodal_processor()`.

    processor = model.create_multimodal_processor()
    inputs = processor("<|image_1|>\\nWhat is shown here?", images=og.Images.open("cat.png"))
    generator.set_inputs(inputs)                       # runs the vision / audio encoder and the prompt

The processor turns a prompt plus images into `input_ids` (every image placeholder expanded to one image token per
patch) and `pixel_values` (resized, normalised), and a prompt plus audio clips into decoder prompt ids and
`audio_features` (Whisper log-mel frames).  The reference does this work in onnxruntime-extensions
(src/models/processor.cpp:11-120, src/models/whisper_processor.cpp, src/models/phi_image_processor.cpp); the arithmetic
below restates the public definitions (Whisper's log-mel front end, CLIP-style image normalisation).
"""
from __future__ import annotations

import json
import math
import os
import re
import wave
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from .api import NamedTensors


# ------------------------------------------------------------------------------------------------ containers
class Images:
    """A list of RGB images as uint8 arrays [H, W, 3]."""

    def __init__(self, arrays: Sequence[np.ndarray]):
        self.arrays = [np.asarray(a) for a in arrays]

    @staticmethod
    def open(*paths: str) -> "Images":
        if not paths:
            raise RuntimeError("No images provided")
        from PIL import Image
        out = []
        for p in paths:
            if not os.path.exists(p):
                raise RuntimeError(f"Image file not found: {p}")
            with Image.open(p) as im:
                out.append(np.asarray(im.convert("RGB")))
        return Images(out)

    @staticmethod
    def open_bytes(*blobs: bytes) -> "Images":
        import io
        from PIL import Image
        out = []
        for b in blobs:
            with Image.open(io.BytesIO(b)) as im:
                out.append(np.asarray(im.convert("RGB")))
        return Images(out)

    def __len__(self):
        return len(self.arrays)


class Audios:
    """A list of mono float32 waveforms with their sample rates."""

    def __init__(self, waves: Sequence[np.ndarray], sample_rates: Union[int, Sequence[int]] = 16000):
        self.waves = [np.asarray(w, dtype=np.float32).reshape(-1) for w in waves]
        self.rates = [int(sample_rates)] * len(self.waves) if isinstance(sample_rates, int) else [int(r) for r in sample_rates]

    @staticmethod
    def open(*paths: str) -> "Audios":
        if not paths:
            raise RuntimeError("No audios provided")
        waves, rates = [], []
        for p in paths:
            if not os.path.exists(p):
                raise RuntimeError(f"Audio file not found: {p}")
            with wave.open(p, "rb") as w:
                n, ch, width, rate = w.getnframes(), w.getnchannels(), w.getsampwidth(), w.getframerate()
                raw = w.readframes(n)
            if width == 2:
                x = np.frombuffer(raw, dtype="<i2").astype(np.float32) / 32768.0
            elif width == 4:
                x = np.frombuffer(raw, dtype="<i4").astype(np.float32) / 2147483648.0
            elif width == 1:
                x = (np.frombuffer(raw, dtype=np.uint8).astype(np.float32) - 128.0) / 128.0
            else:
                raise RuntimeError(f"unsupported sample width {width} in {p}")
            if ch > 1:
                x = x.reshape(-1, ch).mean(axis=1)
            waves.append(x)
            rates.append(rate)
        return Audios(waves, rates)

    def __len__(self):
        return len(self.waves)


# ------------------------------------------------------------------------------------------------ audio features
def _hz_to_mel(f):
    f = np.asarray(f, dtype=np.float64)
    mel = f / (200.0 / 3)
    log_region = f >= 1000.0
    return np.where(log_region, 15.0 + np.log(np.maximum(f, 1e-10) / 1000.0) / (math.log(6.4) / 27.0), mel)


def _mel_to_hz(m):
    m = np.asarray(m, dtype=np.float64)
    return np.where(m >= 15.0, 1000.0 * np.exp((math.log(6.4) / 27.0) * (m - 15.0)), m * (200.0 / 3))


def mel_filter_bank(n_mels: int, n_fft: int, sample_rate: int) -> np.ndarray:
    """Triangular filters on the Slaney mel scale with area normalisation: [n_mels, n_fft // 2 + 1]."""
    freqs = np.linspace(0, sample_rate / 2, n_fft // 2 + 1)
    pts = _mel_to_hz(np.linspace(_hz_to_mel(0.0), _hz_to_mel(sample_rate / 2), n_mels + 2))
    width = np.diff(pts)
    ramps = pts[:, None] - freqs[None, :]
    lower, upper = -ramps[:-2] / width[:-1, None], ramps[2:] / width[1:, None]
    fb = np.maximum(0.0, np.minimum(lower, upper))
    fb *= (2.0 / (pts[2:n_mels + 2] - pts[:n_mels]))[:, None]
    return fb.astype(np.float32)


def resample_linear(x: np.ndarray, rate: int, target: int) -> np.ndarray:
    if rate == target or x.size == 0:
        return x.astype(np.float32)
    n = int(round(x.size * target / rate))
    return np.interp(np.arange(n) * (rate / target), np.arange(x.size), x).astype(np.float32)


def log_mel_spectrogram(wave_: np.ndarray, n_mels: int = 80, n_fft: int = 400, hop: int = 160, sample_rate: int = 16000,
                        n_frames: int = 3000) -> np.ndarray:
    """Whisper's input features: the clip is padded or cut to n_frames * hop samples; Hann-window STFT, mel filter bank,
    log10 clamped to 8 below the clip's maximum, mapped to about [-1, 1].  Returns float32 [n_mels, n_frames]."""
    want = n_frames * hop
    x = torch.zeros(want, dtype=torch.float32)
    w = torch.from_numpy(np.ascontiguousarray(wave_[:want], dtype=np.float32))
    x[:w.numel()] = w
    spec = torch.stft(x, n_fft, hop, window=torch.hann_window(n_fft), return_complex=True)   # centred, reflect padding
    power = spec[:, :-1].abs() ** 2
    mel = torch.from_numpy(mel_filter_bank(n_mels, n_fft, sample_rate)) @ power
    lg = torch.clamp(mel, min=1e-10).log10()
    lg = torch.maximum(lg, lg.max() - 8.0)
    return ((lg + 4.0) / 4.0).numpy().astype(np.float32)


# ------------------------------------------------------------------------------------------------ image features
def preprocess_image(img: np.ndarray, size: int, mean: Sequence[float], std: Sequence[float]) -> np.ndarray:
    """uint8 [H, W, 3] -> float32 [3, size, size]: bicubic resize to a square, scale to [0, 1], normalise per channel."""
    from PIL import Image
    im = Image.fromarray(np.asarray(img, dtype=np.uint8)).resize((size, size), Image.BICUBIC)
    x = np.asarray(im, dtype=np.float32) / 255.0
    x = (x - np.asarray(mean, dtype=np.float32)) / np.asarray(std, dtype=np.float32)
    return np.ascontiguousarray(x.transpose(2, 0, 1))


# ------------------------------------------------------------------------------------------------ processor
_IMAGE_TAG = re.compile(r"<\|image_\d+\|>")


class MultiModalProcessor:
    def __init__(self, model):
        from .tokenizer import Tokenizer
        self.model = model
        self.tokenizer = Tokenizer(model)
        d = model.config.config_path
        self.image_cfg = self.audio_cfg = None
        mm = model.multimodal
        if mm.get("vision"):
            with open(os.path.join(d, mm["vision"].get("config_filename") or "processor_config.json")) as f:
                self.image_cfg = json.load(f)["processor"]
        if mm.get("audio"):
            name = (mm.get("speech") or {}).get("config_filename") or "audio_processor_config.json"
            with open(os.path.join(d, name)) as f:
                self.audio_cfg = json.load(f)["processor"]

    # -- text
    def decode(self, tokens) -> str:
        return self.tokenizer.decode(tokens)

    def create_stream(self):
        return self.tokenizer.create_stream()

    def _encode_with_images(self, prompt: str, n_images: int) -> np.ndarray:
        c = self.image_cfg
        tag = c.get("image_token", "<|image|>")
        parts = re.split("(" + _IMAGE_TAG.pattern + "|" + re.escape(tag) + ")", prompt)
        ids: List[int] = []
        seen = 0
        per = int(c["num_image_tokens"])
        for part in parts:
            if not part:
                continue
            if _IMAGE_TAG.fullmatch(part) or part == tag:
                ids += [int(c["image_token_id"])] * per
                seen += 1
            else:
                ids += self.tokenizer.encode(part).tolist()
        if seen != n_images:
            raise RuntimeError(f"the prompt has {seen} image placeholders but {n_images} images were given")
        return np.asarray(ids, dtype=np.int32)

    def _qwen_vl_inputs(self, prompt: str, images: "Images") -> "NamedTensors":
        """Qwen2-VL front end (reference: src/models/qwen2_5_vl_image_processor.cpp): every image is resized to its own smart
        size, cut into patches in merge-window order, and its placeholder in the prompt becomes t * h * w / merge^2 image tokens."""
        from .models import qwen_vl
        c = self.image_cfg
        vc = qwen_vl.QwenVisionConfig(patch_size=int(c["patch_size"]), spatial_merge_size=int(c["merge_size"]),
                                      temporal_patch_size=int(c["temporal_patch_size"]), min_pixels=int(c["min_pixels"]),
                                      max_pixels=int(c["max_pixels"]))
        pieces, grids = [], []
        for a in images.arrays:
            p, g = qwen_vl.preprocess_image(a, vc)
            pieces.append(p.numpy())
            grids.append(g)
        tag = c.get("image_token", "<|image_pad|>")
        parts = re.split("(" + _IMAGE_TAG.pattern + "|" + re.escape(tag) + ")", prompt)
        ids: List[int] = []
        seen = 0
        for part in parts:
            if not part:
                continue
            if _IMAGE_TAG.fullmatch(part) or part == tag:
                if seen >= len(grids):
                    raise RuntimeError(f"the prompt has more image placeholders than the {len(grids)} images given")
                t, h, w = grids[seen]
                ids += [int(c["image_token_id"])] * (t * h * w // vc.spatial_merge_size ** 2)
                seen += 1
            else:
                ids += self.tokenizer.encode(part).tolist()
        if seen != len(grids):
            raise RuntimeError(f"the prompt has {seen} image placeholders but {len(grids)} images were given")
        out = NamedTensors()
        out["pixel_values"] = np.concatenate(pieces, axis=0)
        out["image_grid_thw"] = np.asarray(grids, dtype=np.int64)
        out["input_ids"] = np.asarray(ids, dtype=np.int32)[None]
        return out

    def __call__(self, prompt: Union[str, Sequence[str], None] = None, images: Optional[Images] = None,
                 audios: Optional[Audios] = None) -> NamedTensors:
        out = NamedTensors()
        prompts = [prompt] if isinstance(prompt, str) or prompt is None else list(prompt)
        if images is not None and len(images):
            if self.image_cfg is None:
                raise RuntimeError("this model has no vision component")
            if len(prompts) != 1:
                raise RuntimeError("image inputs take one prompt")
            c = self.image_cfg
            if c.get("name") == "qwen2_vl_image_processing":
                return self._qwen_vl_inputs(prompts[0] or "", images)
            out["pixel_values"] = np.stack([preprocess_image(a, int(c["image_size"]), c["image_mean"], c["image_std"]) for a in images.arrays])
            out["image_sizes"] = np.asarray([[a.shape[0], a.shape[1]] for a in images.arrays], dtype=np.int64)
            out["input_ids"] = self._encode_with_images(prompts[0] or "", len(images))[None]
            return out
        if audios is not None and len(audios):
            if self.audio_cfg is None:
                raise RuntimeError("this model has no audio component")
            c = self.audio_cfg
            feats = [log_mel_spectrogram(resample_linear(w, r, int(c["sample_rate"])), int(c["num_mel_bins"]), int(c["n_fft"]),
                                         int(c["hop_length"]), int(c["sample_rate"]), int(c["num_frames"]))
                     for w, r in zip(audios.waves, audios.rates)]
            out["audio_features"] = np.stack(feats)
            if len(prompts) == 1 and len(audios) > 1:
                prompts = prompts * len(audios)
            if len(prompts) != len(audios):
                raise RuntimeError("one decoder prompt per audio clip is required")
            if prompts[0] is not None:
                self.tokenizer.update_options(add_special_tokens="false")
                out["input_ids"] = self.tokenizer.encode_batch([p or "" for p in prompts])
            return out
        if prompts[0] is None:
            raise RuntimeError("a prompt, images or audios are required")
        out["input_ids"] = self.tokenizer.encode_batch(prompts)
        return out
