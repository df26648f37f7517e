"""Tokenizer, streaming detokenizer and chat templates.

API parity with the reference's Python binding (src/python/python.cpp:493-541): `encode`, `decode`,
`encode_batch`, `decode_batch`, `to_token_id`, `apply_chat_template`, `create_stream`, the
`bos_token_id / eos_token_ids / pad_token_id` properties and `update_options`.  The reference
delegates to onnxruntime-extensions; here the Hugging Face `tokenizers` library reads the same
`tokenizer.json`, and chat templates (Jinja) come from `tokenizer_config.json` or
`chat_template.jinja`.
"""
from __future__ import annotations

import json
import os
from typing import List, Optional, Sequence

import numpy as np


class Tokenizer:
    def __init__(self, model):
        from tokenizers import Tokenizer as HFTokenizer
        cfg = model.config
        self._dir = cfg.tokenizer_path if hasattr(cfg, "tokenizer_path") else (os.path.join(cfg.config_path, cfg.tokenizer_dir) if cfg.tokenizer_dir else cfg.config_path)
        path = os.path.join(self._dir, "tokenizer.json")
        if not os.path.exists(path):
            raise RuntimeError(f"tokenizer.json not found in {self._dir}")
        self._tok = HFTokenizer.from_file(path)
        self._cfg = {}
        tc = os.path.join(self._dir, "tokenizer_config.json")
        if os.path.exists(tc):
            with open(tc) as f:
                self._cfg = json.load(f)
        self._template = self._cfg.get("chat_template")
        jt = os.path.join(self._dir, "chat_template.jinja")
        if os.path.exists(jt):
            with open(jt) as f:
                self._template = f.read()
        self.bos_token_id = cfg.bos_token_id
        self.eos_token_ids = np.asarray(cfg.eos_token_ids, dtype=np.int32)
        self.pad_token_id = cfg.pad_token_id
        self._add_special = True
        self._skip_special = True

    def update_options(self, **kw):
        for k, v in kw.items():
            if k == "add_special_tokens":
                self._add_special = str(v).lower() in ("1", "true")
            elif k == "skip_special_tokens":
                self._skip_special = str(v).lower() in ("1", "true")
            else:
                raise RuntimeError(f"Unknown tokenizer option: {k}")

    def encode(self, text: str) -> np.ndarray:
        return np.asarray(self._tok.encode(text, add_special_tokens=self._add_special).ids, dtype=np.int32)

    def decode(self, tokens) -> str:
        return self._tok.decode([int(t) for t in np.asarray(tokens).reshape(-1)], skip_special_tokens=self._skip_special)

    def encode_batch(self, texts: Sequence[str]) -> np.ndarray:
        """Returns a right-padded [batch, max_len] int32 array (pad_token_id fills)."""
        enc = [self._tok.encode(t, add_special_tokens=self._add_special).ids for t in texts]
        n = max(len(e) for e in enc) if enc else 0
        out = np.full((len(enc), n), self.pad_token_id, dtype=np.int32)
        for i, e in enumerate(enc):
            out[i, :len(e)] = e
        return out

    def decode_batch(self, tokens) -> List[str]:
        return [self.decode(row) for row in np.asarray(tokens)]

    def to_token_id(self, text: str) -> int:
        tid = self._tok.token_to_id(text)
        if tid is None:
            raise RuntimeError(f"'{text}' is not a single token in the vocabulary")
        return tid

    def apply_chat_template(self, messages: str, *, template_str: Optional[str] = None, tools: Optional[str] = None,
                            add_generation_prompt: bool = True) -> str:
        import jinja2
        tpl = template_str or self._template
        if not tpl:
            raise RuntimeError("no chat template: pass template_str or provide tokenizer_config.json / chat_template.jinja")
        msgs = json.loads(messages) if isinstance(messages, str) else messages
        tool_list = json.loads(tools) if isinstance(tools, str) and tools else tools
        env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True, extensions=["jinja2.ext.loopcontrols"])
        env.globals["raise_exception"] = lambda m: (_ for _ in ()).throw(RuntimeError(m))
        env.filters["tojson"] = lambda v, indent=None: json.dumps(v, indent=indent, ensure_ascii=False)

        def tok(name):
            v = self._cfg.get(name)
            return v.get("content") if isinstance(v, dict) else (v or "")

        return env.from_string(tpl).render(messages=msgs, tools=tool_list, add_generation_prompt=add_generation_prompt,
                                           bos_token=tok("bos_token"), eos_token=tok("eos_token"), pad_token=tok("pad_token"))

    def create_stream(self) -> "TokenizerStream":
        return TokenizerStream(self)

    # Byte-level vocabulary for grammar engines: token id -> bytes.
    def token_bytes(self, vocab_size: int) -> List[bytes]:
        vocab = self._tok.get_vocab(with_added_tokens=True)
        inv = {i: s for s, i in vocab.items()}
        byte_dec = _byte_decoder()
        out = []
        for i in range(vocab_size):
            s = inv.get(i)
            if s is None:
                out.append(b"")
                continue
            try:
                out.append(bytes(byte_dec[c] for c in s))
            except KeyError:
                out.append(s.replace("▁", " ").encode("utf-8"))
        return out


def _byte_decoder():
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("\xa1"), ord("\xac") + 1)) + list(range(ord("\xae"), ord("\xff") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {chr(c): b for b, c in zip(bs, cs)}


class TokenizerStream:
    """Incremental detokenizer: returns the newly completed text for each token (holds back bytes that
    do not yet form a complete UTF-8 sequence)."""

    def __init__(self, tokenizer: Tokenizer):
        self._t = tokenizer
        self._ids: List[int] = []
        self._emitted = ""
        self._prefix_start = 0

    def decode(self, token: int) -> str:
        self._ids.append(int(token))
        text = self._t._tok.decode(self._ids[self._prefix_start:], skip_special_tokens=self._t._skip_special)
        if text.endswith("�"):
            return ""
        new = text[len(self._emitted):]
        self._emitted = text
        if len(self._ids) - self._prefix_start > 64 and new.endswith(("\n", " ")):
            self._prefix_start = len(self._ids)
            self._emitted = ""
        return new
