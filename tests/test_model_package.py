"""Model packages: manifest.json + variant directories + content-addressed shared assets (docs/model_package.md of the reference)."""
import copy
import json
import os
import shutil

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200 import model_package
from onnxruntime_genai_b200.models.arch import PRESETS
from onnxruntime_genai_b200.models.builder import export_model


@pytest.fixture(scope="module")
def package(tmp_path_factory):
    root = tmp_path_factory.mktemp("pkg") / "tiny.ortpackage"
    arch = copy.deepcopy(PRESETS["tiny-llama"])
    arch.num_layers, arch.vocab_size = 1, 300
    for name, ep in (("cpu-1", "cpu"), ("cuda-1", "cuda")):
        export_model(copy.deepcopy(arch), str(root / name), "fp32" if ep == "cpu" else "bf16", ep, seed=3)
    digest = "ab" * 32
    shared = root / "shared_assets" / f"sha256-{digest}"
    os.makedirs(shared / "tok")
    # a minimal word-level tokenizer
    vocab = {f"w{i}": i for i in range(300)}
    tok = {"version": "1.0", "truncation": None, "padding": None, "added_tokens": [], "normalizer": None,
           "pre_tokenizer": {"type": "Whitespace"}, "post_processor": None, "decoder": None,
           "model": {"type": "WordLevel", "vocab": vocab, "unk_token": "w0"}}
    (shared / "tok" / "tokenizer.json").write_text(json.dumps(tok))
    for name in ("cpu-1", "cuda-1"):
        cfgp = root / name / "genai_config.json"
        cfg = json.loads(cfgp.read_text())
        cfg["model"]["tokenizer_dir"] = f"sha256:{digest}/tok"
        cfgp.write_text(json.dumps(cfg))
    manifest = {"schema_version": "1.0", "components": {"model": {"variants": {
        "cuda-1": {"ep": "CUDAExecutionProvider", "device": "gpu"},
        "cpu-1": {"ep": "CPUExecutionProvider", "device": "cpu"}}}}}
    (root / "manifest.json").write_text(json.dumps(manifest))
    return str(root), digest


def test_package_selects_the_variant_of_the_provider(package):
    root, digest = package
    assert model_package.is_package(root)
    d, _ = model_package.resolve_package(root, "cpu")
    assert d.endswith("cpu-1")
    d, _ = model_package.resolve_package(root, "cuda")
    assert d.endswith("cuda-1")
    cfg = og.Config(root, provider="cpu")
    assert cfg.config_path.endswith("cpu-1")
    assert cfg.tokenizer_path == os.path.join(root, "shared_assets", f"sha256-{digest}", "tok")
    model = og.Model(cfg)
    tok = og.Tokenizer(model)
    ids = tok.encode("w5 w17 w250")
    assert list(ids) == [5, 17, 250]
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=12)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([ids], dtype=np.int32))
    g.generate_next_token()
    assert 0 <= int(g.get_next_tokens()[0]) < 300


def test_package_errors(package, tmp_path):
    root, digest = package
    other = tmp_path / "p2"
    shutil.copytree(root, other)
    m = json.loads((other / "manifest.json").read_text())
    del m["components"]["model"]["variants"]["cpu-1"]
    m["components"]["model"]["variants"]["cuda-1"]["ep"] = "OpenVINOExecutionProvider"
    (other / "manifest.json").write_text(json.dumps(m))
    with pytest.raises(RuntimeError, match="no variant for execution provider"):
        model_package.resolve_package(str(other), "cpu")
    m["components"]["model"]["variants"]["cuda-1"] = {"ep": "cpu", "variant_directory": "../escape"}
    (other / "manifest.json").write_text(json.dumps(m))
    with pytest.raises(RuntimeError, match="relative path inside the package"):
        model_package.resolve_package(str(other), "cpu")
    # shared assets: unknown digest, traversal in the tail, scheme outside a package
    d, man = model_package.resolve_package(root, "cpu")
    with pytest.raises(RuntimeError, match="not found"):
        model_package.resolve_asset(d, "sha256:" + "cd" * 32, root, man)
    with pytest.raises(RuntimeError, match="no '..'"):
        model_package.resolve_asset(d, f"sha256:{digest}/../x", root, man)
    with pytest.raises(RuntimeError, match="only valid when"):
        model_package.resolve_asset(d, f"sha256:{digest}", None, None)
    assert model_package.resolve_asset(d, "", root, man) == d
    # a manifest override remaps the digest to another directory of the package
    man2 = dict(man, shared_assets={f"sha256:{digest}": "cpu-1"})
    assert model_package.resolve_asset(d, f"sha256:{digest}", root, man2) == os.path.join(root, "cpu-1")
