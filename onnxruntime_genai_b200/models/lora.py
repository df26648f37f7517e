"""Multi-LoRA adapters: `Adapters(model).load(path, name)`, `generator.set_active_adapter(adapters, name)`.

API parity with the reference (src/models/adapters.h/.cpp, src/python/python.cpp:724-729; graph form
in src/python/py/models/builders/base.py:2108-2147: y = W x + B (A x) with the scaling folded into
B).  The reference feeds LoRA A/B as extra graph inputs of an ONNX Runtime session; here they are
extra low-rank GEMMs on the same tcgen05 kernel: t = x A^T (rank r, padded to a multiple of 8 for the
16-byte TMA rule), then y[:, cols] += t B^T through the GEMM's residual epilogue, so the adapter path
adds two small launches per adapted projection and no elementwise kernel.

Adapter files: `.safetensors` or `.npz` with tensors named
`...layers.<i>...<proj>...lora_A...` of shape [in, r] (or [r, in]) and `...lora_B...` of shape
[r, out] (or [out, r]), proj in {q_proj, k_proj, v_proj, qkv_proj, o_proj, gate_proj, up_proj,
gate_up_proj, down_proj}; an optional scalar `...lora_alpha` / `scaling` multiplies B.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Tuple

import numpy as np
import torch

from .. import ops

_PROJ_TARGET = {  # adapter projection -> (runtime projection, which slice of its output)
    "qkv_proj": ("qkv_proj", "all"), "q_proj": ("qkv_proj", "q"), "k_proj": ("qkv_proj", "k"), "v_proj": ("qkv_proj", "v"),
    "o_proj": ("o_proj", "all"), "gate_up_proj": ("gate_up_proj", "all"), "gate_proj": ("gate_up_proj", "gate"),
    "up_proj": ("gate_up_proj", "up"), "down_proj": ("down_proj", "all"),
}


def apply_lora(y: torch.Tensor, x: torch.Tensor, lora: List[Tuple[torch.Tensor, torch.Tensor, int]]) -> torch.Tensor:
    """y[:, off:off+n] += (x @ A^T) @ B^T for every (A [r, K], B [n, r], off) entry."""
    for a, b, off in lora:
        t = ops.linear(x, a)
        view = y[:, off:off + b.shape[0]]
        if y.is_cuda:
            ops.linear(t, b, residual=view, out=view)
        else:
            view += ops.linear(t, b)
    return y


def _read_file(path: str) -> Dict[str, torch.Tensor]:
    if path.endswith(".npz"):
        z = np.load(path)
        return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    raise RuntimeError(f"unsupported adapter file {path} (expected .safetensors or .npz)")


class Adapters:
    def __init__(self, model):
        self.model = model
        self._loaded: Dict[str, int] = {}  # name -> reference count of generators using it

    def load(self, path: str, name: str) -> None:
        if name in self._loaded:
            raise RuntimeError(f"adapter '{name}' is already loaded")
        if not os.path.exists(path):
            raise RuntimeError(f"adapter file not found: {path}")
        tensors = _read_file(str(path))
        dec = self.model.decoder
        arch, tp = dec.arch, dec.tp
        if tp.size > 1:
            raise RuntimeError("LoRA adapters are not supported with tensor parallelism in this build")
        dev, dt = dec.device, dec.dtype
        pairs: Dict[Tuple[int, str], Dict[str, torch.Tensor]] = {}
        scale = 1.0
        for k, v in tensors.items():
            if k.endswith(("lora_alpha", "scaling")):
                scale = float(v)
                continue
            m = re.search(r"layers\.(\d+)\..*?(qkv_proj|gate_up_proj|q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj).*?lora_([AB])", k)
            if not m:
                continue
            pairs.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3)] = v.float()
        if not pairs:
            raise RuntimeError(f"{path} contains no LoRA tensors")
        q, kv, inter = arch.q_size, arch.kv_size, arch.intermediate_size
        offsets = {"all": 0, "q": 0, "k": q, "v": q + kv, "gate": 0, "up": inter}
        in_dim = {"qkv_proj": arch.hidden_size, "o_proj": q, "gate_up_proj": arch.hidden_size, "down_proj": inter}
        for (layer, proj), ab in pairs.items():
            if "A" not in ab or "B" not in ab:
                raise RuntimeError(f"adapter '{name}': layer {layer} {proj} needs both lora_A and lora_B")
            target, part = _PROJ_TARGET[proj]
            K = in_dim[target]
            a, b = ab["A"], ab["B"]
            a = a if a.shape[1] == K else a.t()        # -> [r, K]
            r = a.shape[0]
            b = b if b.shape[1] == r else b.t()        # -> [n, r]
            if a.shape[1] != K or b.shape[1] != r:
                raise RuntimeError(f"adapter '{name}': layer {layer} {proj} has inconsistent shapes {tuple(ab['A'].shape)} / {tuple(ab['B'].shape)}")
            lw_ = dec.layers[layer]
            fold = lw_.fold_ln1 if target == "qkv_proj" else (lw_.fold_ln2 if target == "gate_up_proj" else None)
            if fold is not None:
                # the model's input norms were folded into these projections (their norm weights are ones now): the low-rank
                # path sees rows scaled by 1 / rms only, so A takes the norm's weight as the base weight did
                a = a * fold.float().cpu()[None, :]
            rp = (r + 7) // 8 * 8                       # TMA needs 16-byte rows
            ap = torch.zeros(rp, K)
            ap[:r] = a
            bp = torch.zeros(b.shape[0], rp)
            bp[:, :r] = b * scale
            entry = (ap.to(dev, dt).contiguous(), bp.to(dev, dt).contiguous(), offsets[part])
            dec.layers[layer].lora.setdefault(name, {}).setdefault(target, []).append(entry)
        self._loaded[name] = 0

    def unload(self, name: str) -> None:
        if name not in self._loaded:
            raise RuntimeError(f"adapter '{name}' is not loaded")
        if self._loaded[name] > 0 or self.model.decoder.active_adapter == name:
            raise RuntimeError(f"adapter '{name}' is still in use")
        for lw in self.model.decoder.layers:
            lw.lora.pop(name, None)
        del self._loaded[name]

    def _activate(self, model, name: str) -> None:
        if name not in self._loaded:
            raise RuntimeError(f"adapter '{name}' is not loaded")
        model.decoder.active_adapter = name
