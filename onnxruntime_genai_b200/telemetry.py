"""Usage events to a local sink.

The reference ships events (model load, generation: time to first token, token counts, device information, with
redaction of anything user-derived) to a remote collector (src/telemetry/*, CMakeLists.txt:95-99).  Nothing leaves the
machine here: events are appended as JSON lines to the file named by ORTGENAI_TELEMETRY_FILE (or `enable(path)`), and
with neither set nothing is recorded.  Redaction keeps the reference's rule: no prompt text, token ids or paths; a model
directory appears only as the first 16 hex digits of its SHA-256.

    ModelLoad   {model_type, device, layers, hidden_size, vocab_size, dtype, load_ms, model_dir_hash}
    Generation  {model_type, device, batch_size, prompt_tokens, generated_tokens, ttft_ms, tokens_per_s}
"""
from __future__ import annotations

import hashlib
import json
import os
import threading
import time
from typing import Any, Callable, Dict, Optional

_lock = threading.Lock()
_path: Optional[str] = os.environ.get("ORTGENAI_TELEMETRY_FILE") or None
_callback: Optional[Callable[[str, Dict[str, Any]], None]] = None
_SESSION = hashlib.sha256(f"{os.getpid()}:{time.time_ns()}".encode()).hexdigest()[:16]
_ALLOWED_TYPES = (int, float, bool, str, type(None))


def enable(path: Optional[str] = None, callback: Optional[Callable[[str, Dict[str, Any]], None]] = None) -> None:
    """Records events to `path` (JSON lines) and / or hands them to `callback(name, fields)`."""
    global _path, _callback
    with _lock:
        _path, _callback = path, callback


def disable() -> None:
    enable(None, None)


def enabled() -> bool:
    return _path is not None or _callback is not None


def redact_path(path: str) -> str:
    return hashlib.sha256(os.path.abspath(path).encode()).hexdigest()[:16]


def log_event(name: str, fields: Dict[str, Any]) -> None:
    """Scalar fields only; anything else is dropped (a tensor or a token list can never end up in an event)."""
    if not enabled():
        return
    clean = {k: v for k, v in fields.items() if isinstance(v, _ALLOWED_TYPES)}
    rec = {"event": name, "time_unix_ms": int(time.time() * 1000), "session": _SESSION, **clean}
    with _lock:
        if _callback is not None:
            _callback(name, dict(rec))
        if _path is not None:
            with open(_path, "a") as f:
                f.write(json.dumps(rec) + "\n")


class GenerationTimer:
    """Per-generator bookkeeping for the Generation event: prompt tokens, first-token latency, generated tokens."""

    def __init__(self):
        self.t_prompt = None
        self.t_first = None
        self.prompt_tokens = 0
        self.generated = 0
        self.sent = False

    def on_prompt(self, n_tokens: int) -> None:
        if self.t_prompt is None:
            self.t_prompt = time.perf_counter()
        self.prompt_tokens += int(n_tokens)

    def on_token(self) -> None:
        if self.t_first is None:
            self.t_first = time.perf_counter()
        self.generated += 1

    def finish(self, model_type: str, device: str, batch_size: int) -> None:
        if self.sent or self.t_prompt is None or not enabled():
            return
        self.sent = True
        now = time.perf_counter()
        decode_s = now - (self.t_first or now)
        log_event("Generation", {"model_type": model_type, "device": device, "batch_size": int(batch_size),
                                 "prompt_tokens": self.prompt_tokens, "generated_tokens": self.generated * int(batch_size),
                                 "ttft_ms": round(((self.t_first or now) - self.t_prompt) * 1e3, 3),
                                 "tokens_per_s": round((self.generated - 1) * batch_size / decode_s, 2) if decode_s > 0 and self.generated > 1 else None})
