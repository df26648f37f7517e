"""Strict genai_config.json parsing (reference behaviour: src/config.cpp:1497-1671, 1931-2148)."""
import json
import os

import pytest

from onnxruntime_genai_b200.native_loader import native

BASE = {
    "model": {"bos_token_id": 1, "context_length": 4096,
              "decoder": {"session_options": {"log_id": "onnxruntime-genai", "provider_options": [{"cuda": {"enable_cuda_graph": "1"}}]},
                          "filename": "model.onnx", "head_size": 128, "hidden_size": 4096,
                          "inputs": {"input_ids": "input_ids", "attention_mask": "attention_mask",
                                     "past_key_names": "past_key_values.%d.key", "past_value_names": "past_key_values.%d.value"},
                          "outputs": {"logits": "logits", "present_key_names": "present.%d.key", "present_value_names": "present.%d.value"},
                          "num_attention_heads": 32, "num_hidden_layers": 32, "num_key_value_heads": 8},
              "eos_token_id": [128001, 128008], "pad_token_id": 128001, "type": "llama", "vocab_size": 128256},
    "search": {"do_sample": False, "max_length": 0, "top_k": 50, "top_p": 1.0, "temperature": 1.0, "num_beams": 1},
}


def cfg(**over):
    d = json.loads(json.dumps(BASE))
    for k, v in over.items():
        d[k] = v
    return json.dumps(d)


def test_parses_reference_layout_and_defaults():
    c = native.Config.from_json(cfg())
    assert c.model_type == "llama" and c.vocab_size == 128256 and c.context_length == 4096
    assert c.eos_token_ids == [128001, 128008] and c.pad_token_id == 128001
    assert c.search["max_length"] == 4096, "max_length 0 defaults to context_length"
    assert c.search["top_k"] == 50 and c.search["num_beams"] == 1 and c.search["early_stopping"] is True
    d = c.decoder
    assert d["num_key_value_heads"] == 8 and d["inputs"]["past_key_names"] == "past_key_values.%d.key"
    assert d["provider_options"][0][0] == "cuda" and d["graph_capture"] is True
    assert c.speculative == {"max_draft_tokens": 4, "ngram_size": 0, "ngram_chained_lookup": False, "min_adaptive_k": 0, "cooldown": False}


def test_scalar_eos_and_missing_eos():
    d = json.loads(cfg())
    d["model"]["eos_token_id"] = 7
    assert native.Config.from_json(json.dumps(d)).eos_token_ids == [7]
    del d["model"]["eos_token_id"]
    assert native.Config.from_json(json.dumps(d)).eos_token_ids == [128001], "falls back to pad_token_id"


@pytest.mark.parametrize("path,key", [(["model"], "typo_key"), (["model", "decoder"], "hiden_size"), (["search"], "beam_width"),
                                      ([], "extra_root"), (["model", "decoder", "inputs"], "not_an_input")])
def test_unknown_key_is_an_error_with_its_path(path, key):
    d = json.loads(cfg())
    node = d
    for p in path:
        node = node[p]
    node[key] = 1 if path != ["model", "decoder", "inputs"] else "x"
    with pytest.raises(RuntimeError, match=key):
        native.Config.from_json(json.dumps(d))


def test_type_errors_and_non_integers():
    d = json.loads(cfg())
    d["search"]["top_k"] = 2.5
    with pytest.raises(RuntimeError, match="top_k"):
        native.Config.from_json(json.dumps(d))
    d = json.loads(cfg())
    d["model"]["vocab_size"] = "big"
    with pytest.raises(RuntimeError, match="vocab_size"):
        native.Config.from_json(json.dumps(d))
    with pytest.raises(RuntimeError, match="parse error"):
        native.Config.from_json("{ \"model\": ")


def test_context_length_required():
    d = json.loads(cfg())
    del d["model"]["context_length"]
    with pytest.raises(RuntimeError, match="context_length"):
        native.Config.from_json(json.dumps(d))


def test_overlay_and_provider_edits():
    c = native.Config.from_json(cfg())
    c.overlay(json.dumps({"search": {"top_k": 7, "do_sample": True}, "model": {"decoder": {"num_hidden_layers": 2}}}))
    assert c.search["top_k"] == 7 and c.search["do_sample"] is True and c.decoder["num_hidden_layers"] == 2
    assert c.decoder["head_size"] == 128, "overlay merges, it does not replace"
    with pytest.raises(RuntimeError):
        c.overlay(json.dumps({"search": {"nope": 1}}))
    assert c.search["top_k"] == 7, "a rejected overlay leaves the config untouched"
    c.clear_providers()
    assert c.decoder["provider_options"] == [] and c.decoder["graph_capture"] is False
    c.append_provider("CUDAExecutionProvider")
    c.set_provider_option("cuda", "enable_cuda_graph", "1")
    assert c.decoder["provider_options"][0][0] == "cuda" and c.decoder["graph_capture"] is True


def test_speculative_and_engine_ranges():
    for bad in ({"max_draft_tokens": 0}, {"max_draft_tokens": 17}, {"ngram_size": 1}, {"ngram_size": 17}, {"min_adaptive_k": 17}):
        with pytest.raises(RuntimeError):
            native.Config.from_json(cfg(speculative=bad))
    c = native.Config.from_json(cfg(speculative={"max_draft_tokens": 16, "ngram_size": 3, "cooldown": True}))
    assert c.speculative["ngram_size"] == 3 and c.speculative["cooldown"] is True
    for bad in ({"block_size": 0}, {"gpu_utilization_factor": 1.5}, {"max_batch_size": -1}, {"num_blocks": 0}):
        with pytest.raises(Exception):
            native.Config.from_json(cfg(engine={"dynamic_batching": bad}))
    c = native.Config.from_json(cfg(engine={"dynamic_batching": {"block_size": 16}}))
    assert c.engine["dynamic_batching"] == {"block_size": 16, "max_batch_size": 16, "max_scheduled_tokens": 2048,
                                            "num_blocks": None, "gpu_utilization_factor": None}
    both = native.Config.from_json(cfg(engine={"dynamic_batching": {"block_size": 4}, "static_batching": {"max_batch_size": 2}}))
    assert "dynamic_batching" not in both.engine and both.engine["static_batching"]["max_batch_size"] == 2


@pytest.mark.parametrize("bad", ["/etc/passwd", "../model.onnx", "sub/../../x.onnx", "\\\\share\\x", "C:\\x.onnx"])
def test_config_paths_must_stay_inside_the_model_dir(bad):
    with pytest.raises(RuntimeError):
        native.validate_config_path(bad, "model.decoder.filename")
    d = json.loads(cfg())
    d["model"]["decoder"]["filename"] = bad
    with pytest.raises(RuntimeError):
        native.Config.from_json(json.dumps(d))


def test_relative_paths_are_fine():
    for ok in ("model.onnx", "sub/model.onnx", "a..b/model.onnx", ""):
        native.validate_config_path(ok)


def test_search_option_validation():
    native.validate_search_option("top_k", 5)
    native.validate_search_option("do_sample", True)
    with pytest.raises(RuntimeError):
        native.validate_search_option("top_k", 1.5)
    with pytest.raises(RuntimeError):
        native.validate_search_option("not_an_option", 1)
    with pytest.raises(RuntimeError):
        native.validate_speculative_option("ngram_size", 1)


def test_load_from_directory(tmp_path):
    (tmp_path / "genai_config.json").write_text(cfg())
    c = native.Config(str(tmp_path), json.dumps({"search": {"max_length": 99}}))
    assert c.search["max_length"] == 99 and c.config_path == str(tmp_path)
    with pytest.raises(RuntimeError):
        native.Config(str(tmp_path / "missing"))
