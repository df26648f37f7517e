"""Multi-LoRA adapters: `Adapters(model).load(path, name)`, `generator.set_active_adapter(adapters, name)`.

API parity with the reference (src/models/adapters.h/.cpp, src/python/python.cpp:724-729; graph form
in src/python/py/models/builders/base.py:2108-2147: y = W x + B (A x) with the scaling folded into
B).  The reference feeds LoRA A/B as extra graph inputs of an ONNX Runtime session; here they are
extra low-rank GEMMs on the same tcgen05 kernel: t = x A^T (rank r, padded to a multiple of 8 for the
16-byte TMA rule), then y[:, cols] += t B^T through the GEMM's residual epilogue, so the adapter path
adds two small launches per adapted projection and no elementwise kernel.

Adapter files: `.onnx_adapter` (the reference's container, utils/onnx_adapter.py), `.safetensors` or `.npz` with tensors named
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


class LoraBatch:
    """The adapters of one packed step: `ids[t]` names token t's adapter as an index into `names` (len(names) = no adapter).
    On the GPU the tokens are grouped by adapter once per step with the expert-routing machinery of the MoE layers (adapters play
    the experts, top-1 with weight 1, tokens without an adapter are "not local" and skipped), and every adapted projection then
    costs two grouped low-rank GEMMs and one combine, whatever the number of adapters in the batch."""

    def __init__(self, ids: torch.Tensor, names):
        self.ids, self.names = ids, tuple(names)
        self.plan = None
        if ids.is_cuda:
            T, E = ids.shape[0], len(self.names)
            logits = torch.empty(T, E + 1, dtype=torch.float32, device=ids.device)      # shape carrier only: the selection is given
            self.plan = ops.moe_route(logits, 1, 0, (0, E), topk=(ids.view(T, 1).contiguous(), torch.ones(T, 1, dtype=torch.float32, device=ids.device)))


class GroupedLora:
    """What `apply_lora` needs for one projection of one layer under a LoraBatch: per output slice (offset, width) the stacked
    A [E, r, K] and B [E, n, r] of the batch's adapters (zeros where an adapter does not touch the slice)."""

    def __init__(self, batch: LoraBatch, slices):
        self.batch, self.slices = batch, slices


def grouped_lora(lw, proj: str, batch: LoraBatch):
    cache = lw.__dict__.setdefault("_lora_stacks", {})
    key = (batch.names, proj)
    if key not in cache:
        per = [lw.lora.get(n, {}).get(proj) or [] for n in batch.names]
        slots = sorted({(off, b.shape[0]) for entries in per for (_, b, off) in entries})
        slices = []
        for off, n in slots:
            found = [[(a, b) for (a, b, o) in entries if o == off and b.shape[0] == n] for entries in per]
            ref_a = next(f[0][0] for f in found if f)
            r = max(f[0][0].shape[0] for f in found if f)
            A = torch.zeros(len(per), r, ref_a.shape[1], dtype=ref_a.dtype, device=ref_a.device)
            B = torch.zeros(len(per), n, r, dtype=ref_a.dtype, device=ref_a.device)
            for e, f in enumerate(found):
                for a, b in f:          # several entries of one adapter on the same slice add up only through separate slices
                    A[e, :a.shape[0]] = a
                    B[e, :, :b.shape[1]] = b
            slices.append((A, B, off, n))
        cache[key] = slices
    return GroupedLora(batch, cache[key]) if cache[key] else None


def _apply_grouped(y: torch.Tensor, x: torch.Tensor, g: GroupedLora) -> torch.Tensor:
    batch = g.batch
    if batch.plan is None:
        ids = batch.ids.long()
        for e in range(len(batch.names)):
            rows = (ids == e).nonzero().flatten()
            if rows.numel() == 0:
                continue
            xe = x[rows]
            for A, B, off, n in g.slices:
                y[rows, off:off + n] += ops.linear(ops.linear(xe, A[e]), B[e])
        return y
    xs = ops.gather_rows(x, batch.plan.sorted_token)
    for A, B, off, n in g.slices:
        t = ops.moe_gemm(xs, A, batch.plan)
        u = ops.moe_gemm(t, B, batch.plan)
        view = y[:, off:off + n]
        view.copy_(ops.moe_combine(u, batch.plan, residual=view))
    return y


def apply_lora(y: torch.Tensor, x: torch.Tensor, lora) -> torch.Tensor:
    """y[:, off:off+n] += (x @ A^T) @ B^T for every (A [r, K], B [n, r], off) entry; with a GroupedLora every token takes the
    matrices of its own adapter."""
    if isinstance(lora, GroupedLora):
        return _apply_grouped(y, x, lora)
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
    if path.endswith(".onnx_adapter"):
        from ..utils.onnx_adapter import BFLOAT16, read_adapter
        params, _ = read_adapter(path)
        out = {}
        for k, (arr, dtype) in params.items():
            t = torch.from_numpy(np.array(arr))
            out[k] = t.view(torch.bfloat16) if dtype == BFLOAT16 else t
        return out
    raise RuntimeError(f"unsupported adapter file {path} (expected .onnx_adapter, .safetensors or .npz)")


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
        in_dim = {"qkv_proj": arch.hidden_size, "o_proj": q, "gate_up_proj": arch.hidden_size, "down_proj": inter}
        # Tensor parallelism: column-parallel projections (qkv, gate/up) keep A whole and take this rank's rows of B, part by
        # part; row-parallel ones (o, down) take this rank's columns of A and keep B whole - their low-rank product is a partial
        # sum like the dense one and goes through the same all-reduce.
        R, rk = tp.size, tp.rank
        ql, kvl, il = q // R, kv // R, inter // R
        offsets = {"all": 0, "q": 0, "k": ql, "v": ql + kvl, "gate": 0, "up": il}

        def shard(target, part, a, b):
            if R == 1:
                return a, b
            if target in ("o_proj", "down_proj"):
                w = ql if target == "o_proj" else il
                return a[:, rk * w:(rk + 1) * w], b
            if part == "all":
                widths = (q, kv, kv) if target == "qkv_proj" else (inter, inter)
                rows, base = [], 0
                for wd in widths:
                    rows.append(b[base + rk * (wd // R): base + (rk + 1) * (wd // R)])
                    base += wd
                return a, torch.cat(rows, dim=0)
            wd = {"q": ql, "k": kvl, "v": kvl, "gate": il, "up": il}[part]
            return a, b[rk * wd:(rk + 1) * wd]
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
            a, b = shard(target, part, a, b)
            K = a.shape[1]
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
            lw.__dict__.pop("_lora_stacks", None)
        del self._loaded[name]

    def _activate(self, model, name: str) -> None:
        if name not in self._loaded:
            raise RuntimeError(f"adapter '{name}' is not loaded")
        model.decoder.active_adapter = name
