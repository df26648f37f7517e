"""Imports the C++ runtime core (`_og_native`), building it in-tree on first use."""
from __future__ import annotations

import importlib


def load():
    try:
        return importlib.import_module("onnxruntime_genai_b200._og_native")
    except ImportError:
        from .build_native import build_native
        build_native()
        importlib.invalidate_caches()
        return importlib.import_module("onnxruntime_genai_b200._og_native")


native = load()
