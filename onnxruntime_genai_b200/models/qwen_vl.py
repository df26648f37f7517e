"""Qwen2-VL vision pipeline: image front end, vision tower, three-component rotary positions.

What the reference splits over `src/models/qwen2_5_vl_image_processor.cpp` (smart resize, normalisation, patch layout,
`image_grid_thw`), `src/models/qwen_vl_vision.cpp` (the vision sessions: patch embedding, attention blocks, patch merger) and
`src/models/qwen_vl_model.cpp` + `position_inputs.cpp` (the [3, batch, sequence] position ids of multimodal RoPE and the
rope delta kept for the decode steps) is one module here:

  preprocess_image   an RGB image -> patches [grid_t * grid_h * grid_w, C * T * P * P] in merge-window order + its (t, h, w) grid
  QwenVisionTower    patches + grids -> image features [patches / merge^2, decoder hidden size]:
                     patch embedding (the 3-D convolution with kernel = stride is a linear map of the flattened patch),
                     pre-norm blocks x += Attn(LN(x)), x += MLP(LN(x)) with a 2-D rotary embedding (row and column of
                     the patch, each on half of the rotary pairs) and attention confined to one frame of one image,
                     quick-GELU MLP, then the merger: LN, 2 x 2 neighbouring patches concatenated, a two-layer MLP
  mrope_positions    token ids + grids -> the three position components of every prompt token (text tokens advance all
                     three together; the tokens of an image keep the temporal component and take the row / column of
                     their merged patch) and the offset of the positions that follow

Weights carry the checkpoint's own names without the `visual.` prefix (`patch_embed.proj.weight`, `blocks.N.attn.qkv.weight`,
`merger.mlp.0.weight`, ...), stored as initializers of `vision.onnx` beside one `QwenVision` node with the configuration.
On CUDA the linear layers and layer norms run through `ops.linear` / `ops.norm`; the attention of a frame is a tensor
operation over that frame's patches.
"""
from __future__ import annotations

import math
import os
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from ..utils import onnx_proto as op

QWEN_VL_TYPES = ("qwen2_vl", "qwen2_5_vl")
IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class QwenVisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584          # width of the decoder the features are spliced into
    num_heads: int = 16
    mlp_ratio: float = 4.0
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2
    norm_eps: float = 1e-6
    min_pixels: int = 56 * 56
    max_pixels: int = 28 * 28 * 1280
    # Qwen2.5-VL: RMS norms, a gated SiLU MLP of `intermediate_size`, and attention inside windows of `window_size` pixels
    # except in the blocks listed (as a comma-separated string) in `fullatt_blocks`
    variant: str = "qwen2_vl"        # qwen2_vl | qwen2_5_vl
    intermediate_size: int = 0
    window_size: int = 112
    fullatt_blocks: str = ""

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def mlp_dim(self) -> int:
        return self.intermediate_size if self.windowed else int(self.embed_dim * self.mlp_ratio)

    @property
    def windowed(self) -> bool:
        return self.variant == "qwen2_5_vl"

    @property
    def full_blocks(self) -> List[int]:
        return [int(v) for v in self.fullatt_blocks.split(",") if v.strip()]

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


def weight_shapes(c: QwenVisionConfig) -> Dict[str, tuple]:
    E, M, P, T = c.embed_dim, c.mlp_dim, c.patch_size, c.temporal_patch_size
    s: Dict[str, tuple] = {"patch_embed.proj.weight": (E, c.in_channels, T, P, P)}
    for i in range(c.depth):
        p = f"blocks.{i}."
        s[p + "norm1.weight"], s[p + "norm2.weight"] = (E,), (E,)
        if not c.windowed:
            s[p + "norm1.bias"], s[p + "norm2.bias"] = (E,), (E,)
        s[p + "attn.qkv.weight"], s[p + "attn.qkv.bias"] = (3 * E, E), (3 * E,)
        s[p + "attn.proj.weight"], s[p + "attn.proj.bias"] = (E, E), (E,)
        if c.windowed:
            for n in ("gate_proj", "up_proj"):
                s[p + f"mlp.{n}.weight"], s[p + f"mlp.{n}.bias"] = (M, E), (M,)
            s[p + "mlp.down_proj.weight"], s[p + "mlp.down_proj.bias"] = (E, M), (E,)
        else:
            s[p + "mlp.fc1.weight"], s[p + "mlp.fc1.bias"] = (M, E), (M,)
            s[p + "mlp.fc2.weight"], s[p + "mlp.fc2.bias"] = (E, M), (E,)
    G = E * c.spatial_merge_size ** 2
    s["merger.ln_q.weight"] = (E,)
    if not c.windowed:
        s["merger.ln_q.bias"] = (E,)
    s["merger.mlp.0.weight"], s["merger.mlp.0.bias"] = (G, G), (G,)
    s["merger.mlp.2.weight"], s["merger.mlp.2.bias"] = (c.hidden_size, G), (c.hidden_size,)
    return s


def random_state_dict(c: QwenVisionConfig, seed: int = 0, std: float = 0.05) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in weight_shapes(c).items():
        if ("norm" in name or "ln_q" in name) and name.endswith("weight"):
            sd[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            sd[name] = torch.randn(shape, generator=g) * std
    return sd


def strip_prefix(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """A checkpoint's `visual.*` / `model.visual.*` tensors under this module's names."""
    out = {}
    for k, v in state_dict.items():
        for pre in ("model.visual.", "visual."):
            if k.startswith(pre):
                out[k[len(pre):]] = v
                break
    return out


# ------------------------------------------------------------------------------------------------ image front end
def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Both sides multiples of `factor`, the pixel count inside [min_pixels, max_pixels], the aspect ratio kept as far as that
    allows (reference: qwen2_5_vl_image_processor.cpp smart-resize step; same rule as the checkpoint's own processor)."""
    if max(height, width) / min(height, width) > 200:
        raise RuntimeError("image aspect ratio above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def patchify(frames: torch.Tensor, c: QwenVisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """frames fp32 [n, C, H, W] (normalised; H and W multiples of patch * merge; n is padded to a multiple of the temporal patch by
    repeating the last frame) -> (patches [t * gh * gw, C * T * P * P], (t, gh, gw)).  Patches are ordered frame group, then
    2 x 2 merge window, then position inside the window - the order the merger concatenates."""
    P, T, m = c.patch_size, c.temporal_patch_size, c.spatial_merge_size
    n, C, H, W = frames.shape
    if n % T:
        frames = torch.cat([frames, frames[-1:].expand(T - n % T, C, H, W)], dim=0)
        n = frames.shape[0]
    gt, gh, gw = n // T, H // P, W // P
    x = frames.reshape(gt, T, C, gh // m, m, P, gw // m, m, P)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return x.reshape(gt * gh * gw, C * T * P * P).contiguous(), (gt, gh, gw)


def preprocess_image(image: np.ndarray, c: QwenVisionConfig) -> Tuple[torch.Tensor, Tuple[int, int, int]]:
    """uint8 [H, W, 3] (or float in 0..1) -> (patches, grid): bicubic resize to the smart size, CLIP normalisation, the still
    image repeated to fill one temporal patch."""
    img = torch.as_tensor(np.asarray(image))
    if img.dtype == torch.uint8:
        img = img.float() / 255.0
    img = img.float().permute(2, 0, 1)[None]
    h, w = smart_resize(img.shape[2], img.shape[3], c.patch_size * c.spatial_merge_size, c.min_pixels, c.max_pixels)
    if (h, w) != tuple(img.shape[2:]):
        img = F.interpolate(img, size=(h, w), mode="bicubic", align_corners=False, antialias=True).clamp(0.0, 1.0)
    mean = torch.tensor(IMAGE_MEAN).view(1, 3, 1, 1)
    std = torch.tensor(IMAGE_STD).view(1, 3, 1, 1)
    return patchify((img - mean) / std, c)


# ------------------------------------------------------------------------------------------------ positions
def mrope_positions(tokens: Sequence[int], image_token_id: int, grids: Sequence[Tuple[int, int, int]], merge: int,
                    start: int = 0) -> Tuple[np.ndarray, int, int]:
    """Three position components [3, len(tokens)] of a prompt whose runs of `image_token_id` stand for the images of `grids`
    in order (run length t * h * w / merge^2 each), the number of grids consumed, and the position the next token takes.
    Text: all three components advance together.  Image: temporal component fixed per frame group, row and column of the
    merged patch, all offset by the position where the image starts; the text after it continues one past the largest
    component used so far."""
    pos = np.zeros((3, len(tokens)), dtype=np.int32)
    nxt, i, used = int(start), 0, 0
    n = len(tokens)
    while i < n:
        if tokens[i] != image_token_id:
            pos[:, i] = nxt
            nxt += 1
            i += 1
            continue
        if used >= len(grids):
            raise RuntimeError("the prompt has more image-token runs than images")
        t, h, w = grids[used]
        gh, gw = h // merge, w // merge
        count = t * gh * gw
        if i + count > n or any(tok != image_token_id for tok in tokens[i:i + count]):
            raise RuntimeError(f"image {used}: expected a run of {count} image tokens")
        idx = np.arange(count)
        pos[0, i:i + count] = nxt + idx // (gh * gw)
        pos[1, i:i + count] = nxt + (idx // gw) % gh
        pos[2, i:i + count] = nxt + idx % gw
        nxt += max(t, gh, gw)
        i += count
        used += 1
    return pos, used, nxt


# ------------------------------------------------------------------------------------------------ export / load
_DT = {"fp32": (torch.float32, op.FLOAT), "bf16": (torch.bfloat16, op.BFLOAT16), "fp16": (torch.float16, op.FLOAT16)}


def export_qwen_vision(c: QwenVisionConfig, out_dir: str, state_dict: Dict[str, torch.Tensor], filename: str = "vision.onnx",
                       precision: str = "bf16") -> str:
    os.makedirs(out_dir, exist_ok=True)
    prec = "bf16" if precision == "int4" else precision
    tdt, odt = _DT[prec]
    m = op.Model()
    for name, shape in weight_shapes(c).items():
        t = state_dict[name].detach().to(tdt).contiguous()
        if tuple(t.shape) != tuple(shape):
            raise RuntimeError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")
        arr = t.view(torch.int16).numpy() if prec == "bf16" else t.numpy()
        m.initializers[name] = op.Tensor(name=name, dtype=odt, dims=tuple(t.shape), raw=np.ascontiguousarray(arr).tobytes())
    m.nodes.append(op.Node(op_type="QwenVision", name="/vision/QwenVision", inputs=["pixel_values", "image_grid_thw"] + list(m.initializers),
                           outputs=["image_features"], domain="ogb200", attrs=asdict(c)))
    m.inputs = [op.ValueInfo("pixel_values", odt, ("num_patches", c.patch_dim)), op.ValueInfo("image_grid_thw", op.INT64, ("num_images", 3))]
    m.outputs = [op.ValueInfo("image_features", odt, ("num_merged_patches", c.hidden_size))]
    path = os.path.join(out_dir, filename)
    op.save_model(m, path)
    return path


class QwenVisionTower:
    def __init__(self, cfg: QwenVisionConfig, sd: Dict[str, torch.Tensor], device, dtype):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w = {k: v.to(self.device, dtype).contiguous() for k, v in sd.items()}
        self.w["patch_embed.proj.weight"] = self.w["patch_embed.proj.weight"].reshape(cfg.embed_dim, cfg.patch_dim).contiguous()
        quarter = cfg.head_dim // 4          # frequencies per axis: the row angles fill one quarter of the head's dimensions, the column angles the next
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, 2 * quarter, 2, dtype=torch.float32) / (2 * quarter)))

    @staticmethod
    def is_file(path: str) -> bool:
        try:
            lm = op.LoadedModel(path)
            ok = any(n.op_type == "QwenVision" for n in lm.model.nodes)
            lm.close()
            return ok
        except Exception:
            return False

    @staticmethod
    def load(path: str, device, dtype) -> "QwenVisionTower":
        from .loader import _np_to_torch
        lm = op.LoadedModel(path)
        node = next(n for n in lm.model.nodes if n.op_type == "QwenVision")
        defaults, kw = QwenVisionConfig(), {}
        for k, v in node.attrs.items():
            if hasattr(defaults, k):
                v = v.decode() if isinstance(v, bytes) else v
                kw[k] = type(getattr(defaults, k))(v)
        sd = {name: _np_to_torch(lm.array(name), lm.info(name).dtype).clone() for name in lm.names()}
        lm.close()
        return QwenVisionTower(QwenVisionConfig(**kw), sd, device, dtype)

    def _linear(self, x, name):
        w, b = self.w[name + ".weight"], self.w.get(name + ".bias")
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            from .. import ops
            return ops.linear(x.contiguous(), w, b)
        return F.linear(x, w, b)

    def _ln(self, x, name):
        """LayerNorm (Qwen2-VL) or RMS norm (Qwen2.5-VL)."""
        w, b = self.w[name + ".weight"], self.w.get(name + ".bias")
        rms = self.cfg.windowed
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            from .. import ops
            return ops.norm(x.contiguous(), w, self.cfg.norm_eps, None, b, not rms)[0]
        if rms:
            xf = x.float()
            return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps) * w.float()).to(x.dtype)
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), self.cfg.norm_eps).to(x.dtype)

    def _window_order(self, grids) -> Tuple[torch.Tensor, List[int]]:
        """Qwen2.5-VL: the merged patches (groups of merge^2 patches) regrouped so that every attention window - a square of
        window_size / (patch * merge) merged patches per side, clipped at the image border - is contiguous.  Returns the
        permutation of the groups and the patch counts of the windows in the new order."""
        c = self.cfg
        m2 = c.spatial_merge_size ** 2
        side = c.window_size // c.spatial_merge_size // c.patch_size
        order, sizes, base = [], [], 0
        for t, h, w in grids:
            gh, gw = h // c.spatial_merge_size, w // c.spatial_merge_size
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            for f in range(t):
                for r0 in range(0, gh, side):
                    for c0 in range(0, gw, side):
                        win = idx[f, r0:r0 + side, c0:c0 + side].reshape(-1)
                        order.append(win + base)
                        sizes.append(int(win.numel()) * m2)
            base += t * gh * gw
        return torch.cat(order), sizes

    def _rotary(self, grids) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos / sin [patches, head_dim]: the first half of the rotary pairs turns with the patch's row, the second half with
        its column; rows / columns are listed in the merge-window order of the patches."""
        m = self.cfg.spatial_merge_size
        rows, cols = [], []
        for t, h, w in grids:
            r = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            c = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            rows.append(r.repeat(t))
            cols.append(c.repeat(t))
        rows, cols = torch.cat(rows).float(), torch.cat(cols).float()
        ang = torch.cat([rows[:, None] * self.inv_freq[None, :], cols[:, None] * self.inv_freq[None, :]], dim=1)   # [N, head_dim / 2]
        ang = torch.cat([ang, ang], dim=1).to(self.device)
        return torch.cos(ang), torch.sin(ang)

    @staticmethod
    def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x [N, heads, D] fp32; pairs (i, i + D/2)."""
        half = x.shape[-1] // 2
        rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
        return x * cos[:, None, :] + rot * sin[:, None, :]

    def forward(self, patches: torch.Tensor, grids: Sequence[Tuple[int, int, int]]) -> torch.Tensor:
        """patches [N, C * T * P * P], grids [(t, h, w)] with sum t*h*w = N -> features [N / merge^2, hidden_size]."""
        c = self.cfg
        grids = [tuple(int(v) for v in g) for g in grids]
        N = sum(t * h * w for t, h, w in grids)
        if patches.shape != (N, c.patch_dim):
            raise RuntimeError(f"pixel_values: expected [{N}, {c.patch_dim}] for these grids, got {tuple(patches.shape)}")
        if any(h % c.spatial_merge_size or w % c.spatial_merge_size for _, h, w in grids):
            raise RuntimeError("image grid sides must be multiples of the spatial merge size")
        with torch.no_grad():
            x = self._linear(patches.to(self.device, self.dtype), "patch_embed.proj")
            cos, sin = self._rotary(grids)
            frames = [h * w for t, h, w in grids for _ in range(t)]            # attention stays inside one frame of one image
            H, D, m2 = c.num_heads, c.head_dim, c.spatial_merge_size ** 2
            windows, perm = frames, None
            if c.windowed:
                perm, windows = self._window_order(grids)
                expand = (perm[:, None] * m2 + torch.arange(m2)[None, :]).reshape(-1).to(self.device)     # groups -> their patches
                x, cos, sin = x[expand], cos[expand], sin[expand]
                # a full-attention block still sees whole frames: in window order a frame's patches stay contiguous
            full = set(c.full_blocks)
            for i in range(c.depth):
                p = f"blocks.{i}."
                qkv = self._linear(self._ln(x, p + "norm1"), p + "attn.qkv").float().view(N, 3, H, D)
                q, k, v = self._rotate(qkv[:, 0], cos, sin), self._rotate(qkv[:, 1], cos, sin), qkv[:, 2]
                out = torch.empty(N, H, D, dtype=torch.float32, device=self.device)
                s = 0
                for n in (frames if (not c.windowed or i in full) else windows):
                    qs, ks, vs = (z[s:s + n].transpose(0, 1) for z in (q, k, v))            # [H, n, D]
                    att = torch.softmax(qs @ ks.transpose(-1, -2) / math.sqrt(D), dim=-1) @ vs
                    out[s:s + n] = att.transpose(0, 1)
                    s += n
                x = x + self._linear(out.reshape(N, H * D).to(self.dtype), p + "attn.proj")
                y = self._ln(x, p + "norm2")
                if c.windowed:
                    hdn = (F.silu(self._linear(y, p + "mlp.gate_proj").float()) * self._linear(y, p + "mlp.up_proj").float()).to(self.dtype)
                    x = x + self._linear(hdn, p + "mlp.down_proj")
                else:
                    hdn = self._linear(y, p + "mlp.fc1").float()
                    hdn = (hdn * torch.sigmoid(1.702 * hdn)).to(self.dtype)                    # quick GELU
                    x = x + self._linear(hdn, p + "mlp.fc2")
            g = self._ln(x, "merger.ln_q").reshape(N // m2, c.embed_dim * m2)
            g = F.gelu(self._linear(g, "merger.mlp.0").float()).to(self.dtype)
            out = self._linear(g, "merger.mlp.2")
            if perm is not None:
                out = out[torch.argsort(perm).to(self.device)]                                 # back to the order of the image tokens
            return out

    # the name `Generator.set_inputs` calls on every vision encoder
    def encode_patches(self, patches, grids) -> Tuple[torch.Tensor, List[int]]:
        m2 = self.cfg.spatial_merge_size ** 2
        feats = self.forward(torch.as_tensor(np.asarray(patches)) if not isinstance(patches, torch.Tensor) else patches, grids)
        return feats, [int(t * h * w) // m2 for t, h, w in grids]
