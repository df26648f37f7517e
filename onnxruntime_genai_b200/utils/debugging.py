"""Tensor dumps for the `model_input_values` / `model_output_shapes` / `model_output_values` / `model_logits` log flags
(reference: src/models/debugging.cpp:9-199 DumpTensor / DumpValues, src/models/model.cpp:115-130): shape and type, the first and
last ten values, and statistics that make a broken tensor obvious at a glance (minimum / maximum with their positions, mean,
standard deviation, the first non-finite value and how many there are)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..native_loader import native

VALUE_COUNT = 10       # values shown at each end of a tensor


def describe(name: str, t: Optional[torch.Tensor], values: bool = True) -> str:
    if t is None:
        return f"{name}: None"
    head = f"{name}: {str(t.dtype).replace('torch.', '')}{list(t.shape)} on {t.device}"
    if not values or t.numel() == 0:
        return head
    flat = t.detach().reshape(-1)
    n = flat.numel()
    if n <= 2 * VALUE_COUNT:
        shown = ", ".join(_fmt(v) for v in flat.tolist())
    else:
        shown = ", ".join(_fmt(v) for v in flat[:VALUE_COUNT].tolist()) + ", ..., " + ", ".join(_fmt(v) for v in flat[-VALUE_COUNT:].tolist())
    lines = [head, f"  values: {shown}"]
    if t.is_floating_point():
        f = flat.float()
        finite = torch.isfinite(f)
        bad = int((~finite).sum())
        g = torch.where(finite, f, torch.zeros_like(f))
        cnt = max(1, n - bad)
        mean = float(g.sum() / cnt)
        var = float((torch.where(finite, (f - mean) ** 2, torch.zeros_like(f))).sum() / cnt)
        lo = torch.where(finite, f, torch.full_like(f, float("inf")))
        hi = torch.where(finite, f, torch.full_like(f, float("-inf")))
        lines.append(f"  min {float(lo.min()):.6g} at [{int(lo.argmin())}]  max {float(hi.max()):.6g} at [{int(hi.argmax())}]  "
                     f"mean {mean:.6g}  stddev {var ** 0.5:.6g}")
        if bad:
            first = int((~finite).nonzero()[0])
            lines.append(f"  NON-FINITE: first at [{first}] = {float(f[first])}, {bad} in total")
    return "\n".join(lines)


def _fmt(v) -> str:
    return f"{v:.6g}" if isinstance(v, float) else str(v)


def dump_inputs(step_inputs) -> None:
    """Called by the model runtime before a forward pass when the flag is on."""
    if not native.log_flag("model_input_values"):
        return
    fields: Dict[str, Optional[torch.Tensor]] = {k: getattr(step_inputs, k, None) for k in
                                                 ("input_ids", "positions", "slot_mapping", "cu_seqlens", "past_lens", "block_table")}
    native.log_write("model_input_values", "\n".join(describe(k, v) for k, v in fields.items() if v is not None))


def dump_outputs(logits: torch.Tensor, hidden: Optional[torch.Tensor] = None) -> None:
    if native.log_flag("model_output_shapes"):
        native.log_write("model_output_shapes", describe("logits", logits, values=False))
    if native.log_flag("model_output_values") or native.log_flag("model_logits"):
        text = describe("logits", logits)
        if hidden is not None and native.log_flag("model_output_values"):
            text += "\n" + describe("hidden_states", hidden)
        native.log_write("model_output_values" if native.log_flag("model_output_values") else "model_logits", text)
