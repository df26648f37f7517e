"""Model packages: a directory with a top-level `manifest.json` that bundles several build variants of one model
(reference: docs/model_package.md, src/models/model_package.cpp).

    my-model.ortpackage/
      manifest.json                  {"schema_version": "1.0", "components": {"model": {"variants": {name: {ep, device, ...}}}}}
      <variant>/genai_config.json    one complete model directory per variant (or `variant_directory`)
      shared_assets/sha256-<hex>/    files shared by the variants, referenced as "sha256:<hex>[/tail]"

`resolve_package(path)` picks the variant for this machine — this runtime has two back ends, so the choice is by
execution provider: CUDA variants when a GPU is present, CPU variants otherwise, the first declared variant among equals
(the reference delegates the ranking to each provider's compatibility-string scoring) — and `resolve_asset` turns a
`model.tokenizer_dir` value into a directory with the portable-layout confinement the flat layout has (no absolute paths,
no `..`).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Optional, Tuple

_EP_ALIASES = {
    "cuda": ("cudaexecutionprovider", "cuda", "nvtensorrtrtxexecutionprovider"),
    "cpu": ("cpuexecutionprovider", "cpu", ""),
}


def is_package(path: str) -> bool:
    return os.path.isdir(path) and os.path.isfile(os.path.join(path, "manifest.json")) and \
        not os.path.isfile(os.path.join(path, "genai_config.json"))


def _confined(base: str, rel: str, what: str) -> str:
    if os.path.isabs(rel) or rel.startswith(("/", "\\")) or ".." in rel.replace("\\", "/").split("/") or (len(rel) > 1 and rel[1] == ":"):
        raise RuntimeError(f"{what}: '{rel}' must be a relative path inside the package (no absolute paths, no '..')")
    return os.path.normpath(os.path.join(base, rel))


def load_manifest(path: str) -> dict:
    with open(os.path.join(path, "manifest.json")) as f:
        m = json.load(f)
    comps = m.get("components") or {}
    if "model" not in comps or not (comps["model"].get("variants") or {}):
        raise RuntimeError("manifest.json: expected an inline component named 'model' with at least one variant")
    return m


def resolve_package(path: str, provider: Optional[str] = None) -> Tuple[str, dict]:
    """Returns (variant directory, manifest) for the variant that matches `provider` ("cuda" / "cpu"; default: cuda when
    a GPU is visible, else cpu).  Raises when no variant targets that provider."""
    m = load_manifest(path)
    variants: Dict[str, dict] = m["components"]["model"]["variants"]
    if provider is None:
        import torch
        provider = "cuda" if torch.cuda.is_available() else "cpu"
    wanted = _EP_ALIASES[provider]
    order = [provider] if provider == "cpu" else [provider, "cpu"]     # a GPU machine can still run a CPU variant
    for prov in order:
        for name, v in variants.items():
            if str(v.get("ep", "")).lower() in _EP_ALIASES[prov]:
                d = _confined(path, v.get("variant_directory") or name, f"variant '{name}'")
                if not os.path.isfile(os.path.join(d, "genai_config.json")):
                    raise RuntimeError(f"variant '{name}': {d} has no genai_config.json")
                return d, m
    eps = sorted({str(v.get("ep", "")) for v in variants.values()})
    raise RuntimeError(f"model package has no variant for execution provider '{provider}' (declared: {', '.join(eps)}; wanted one of {wanted})")


def resolve_asset(variant_dir: str, value: str, package_root: Optional[str], manifest: Optional[dict]) -> str:
    """Directory named by a `model.tokenizer_dir` value: empty -> the variant directory; `sha256:<hex>[/tail]` -> the
    shared asset (only inside a package; manifest `shared_assets` overrides honoured); anything else -> a confined
    relative path under the variant directory."""
    if not value:
        return variant_dir
    if value.startswith("sha256:"):
        if package_root is None:
            raise RuntimeError("the sha256: path scheme is only valid when the model is loaded from a model package")
        digest, _, tail = value[len("sha256:"):].partition("/")
        if not digest or any(c not in "0123456789abcdefABCDEF" for c in digest):
            raise RuntimeError(f"malformed shared-asset reference '{value}'")
        override = ((manifest or {}).get("shared_assets") or {}).get(f"sha256:{digest}") or ((manifest or {}).get("shared_assets") or {}).get(digest)
        base = override if override else os.path.join(package_root, "shared_assets", f"sha256-{digest}")
        if override and not os.path.isabs(base):
            base = _confined(package_root, base, "shared_assets override")
        if not os.path.isdir(base):
            raise RuntimeError(f"shared asset sha256:{digest} not found under {package_root}")
        return _confined(base, tail, "shared asset tail") if tail else base
    return _confined(variant_dir, value, "model.tokenizer_dir")
