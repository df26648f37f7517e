"""Constrained decoding: JSON schema / regex / Lark grammars -> per-step token bitmasks.

Same contract as the reference's GuidanceLogitsProcessor (src/constrained_logits_processor.cpp:58-295):
one matcher per batch entry, a bitmask of (vocab-1)/32+1 words per row with bit v set when token v
may come next, `commit_tokens` advances the grammar, `reset` starts over, `clone` gives an
independent cursor for speculative look-ahead, fast-forward tokens only with batch size 1.
The grammar engine is llguidance (as in the reference); the mask is applied on the device by
`ops.logits_bitmask` (csrc/elementwise.cu) instead of a separate 1-thread-per-logit kernel.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional

import numpy as np
import torch

from . import ops

_TOKENIZER_CACHE = {}


def _ll_tokenizer(model):
    import llguidance
    cfg = model.config
    d = cfg.tokenizer_path if hasattr(cfg, "tokenizer_path") else (os.path.join(cfg.config_path, cfg.tokenizer_dir) if cfg.tokenizer_dir else cfg.config_path)
    path = os.path.join(d, "tokenizer.json")
    key = (path, cfg.vocab_size)
    tok = _TOKENIZER_CACHE.get(key)
    if tok is None:
        if not os.path.exists(path):
            raise RuntimeError("guidance needs tokenizer.json next to the model to map tokens to bytes")
        with open(path) as f:
            text = f.read()
        eos = list(cfg.eos_token_ids)
        tok = llguidance.LLTokenizer(text, n_vocab=cfg.vocab_size, eos_token=eos if len(eos) > 1 else eos[0])
        _TOKENIZER_CACHE[key] = tok
    return tok


def _grammar(kind: str, data: str) -> str:
    import llguidance
    if kind == "json_schema":
        return llguidance.LLMatcher.grammar_from_json_schema(data)
    if kind == "regex":
        return llguidance.LLMatcher.grammar_from_regex(data)
    if kind == "lark_grammar":
        return llguidance.LLMatcher.grammar_from_lark(data)
    raise RuntimeError(f"Unsupported guidance type: {kind}")


class GuidanceProcessor:
    def __init__(self, model, kind: str, data: str, batch_size: int, enable_ff_tokens: bool = False, _matchers=None):
        import llguidance
        if enable_ff_tokens and batch_size > 1:
            raise RuntimeError("fast-forward tokens are only supported with batch_size 1")
        self.model, self.kind, self.data, self.batch = model, kind, data, batch_size
        self.ff = enable_ff_tokens
        self.vocab = model.config.vocab_size
        self.words = (self.vocab - 1) // 32 + 1
        self._tok = _ll_tokenizer(model)
        self._grammar = _grammar(kind, data)
        if _matchers is None:
            err = llguidance.LLMatcher.validate_grammar(self._grammar, self._tok)
            if err:
                raise RuntimeError(f"invalid {kind} grammar: {err}")
            _matchers = [llguidance.LLMatcher(self._tok, self._grammar) for _ in range(batch_size)]
        self.matchers = _matchers
        self.mask = np.full((batch_size, self.words), -1, dtype=np.int32)

    def commit_prompt(self, prompt_ids) -> None:
        """The grammar constrains generated tokens only; the prompt is not fed to the matcher."""

    def compute_mask(self) -> np.ndarray:
        for i, m in enumerate(self.matchers):
            if m.is_stopped():  # grammar complete: only end-of-sequence may follow
                u = self.mask.view(np.uint32)
                u[i, :] = 0
                for e in self.model.config.eos_token_ids:
                    if 0 <= e < self.vocab:
                        u[i, e >> 5] |= np.uint32(1 << (e & 31))
                continue
            row = self.mask[i]
            m.unsafe_compute_mask_ptr(row.ctypes.data, row.size * row.itemsize)
            if m.is_error():
                raise RuntimeError("grammar matcher error: " + m.get_error())
        return self.mask

    def apply(self, logits: torch.Tensor) -> torch.Tensor:
        """Masks [rows, vocab] fp32 logits in place (rows = batch * beams share their batch entry's mask)."""
        mask = self.compute_mask()
        rows = logits.shape[0]
        per = rows // self.batch
        mrows = torch.arange(self.batch, dtype=torch.int32).repeat_interleave(per)
        return ops.logits_bitmask(logits, torch.from_numpy(mask).to(logits.device), mrows.to(logits.device))

    def commit_tokens(self, tokens) -> None:
        toks = np.asarray(tokens).reshape(-1)
        per = max(1, toks.size // self.batch)
        for i, m in enumerate(self.matchers):
            if m.is_stopped():
                continue
            m.consume_token(int(toks[i * per]))

    def ff_tokens(self) -> List[int]:
        """Tokens the grammar forces next (batch size 1 only)."""
        if not self.ff:
            return []
        return list(self.matchers[0].compute_ff_tokens())

    def is_accepting(self, i: int = 0) -> bool:
        return self.matchers[i].is_accepting()

    def reset(self) -> None:
        for m in self.matchers:
            m.reset()

    def clone(self) -> "GuidanceProcessor":
        return GuidanceProcessor(self.model, self.kind, self.data, self.batch, self.ff, _matchers=[m.deep_copy() for m in self.matchers])
