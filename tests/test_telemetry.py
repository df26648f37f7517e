"""Usage events go to a local sink only, with nothing user-derived in them (reference: src/telemetry/*)."""
import copy
import json

import numpy as np

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200 import telemetry
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model


def test_model_load_and_generation_events(tmp_path):
    arch = ArchConfig(model_type="llama", vocab_size=64, hidden_size=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=16,
                      intermediate_size=32, context_length=64, bos_token_id=0, eos_token_id=1, pad_token_id=0)
    d = str(tmp_path / "m")
    export_model(copy.deepcopy(arch), d, "fp32", "cpu")
    assert not telemetry.enabled()
    og.Model(d)                                             # nothing is recorded unless a sink is set
    sink = str(tmp_path / "events.jsonl")
    seen = []
    telemetry.enable(sink, lambda name, rec: seen.append(name))
    try:
        model = og.Model(d)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=12)
        g = og.Generator(model, p)
        prompt = np.asarray([[5, 6, 7, 8]], dtype=np.int32)
        g.append_tokens(prompt)
        while not g.is_done():
            g.generate_next_token()
    finally:
        telemetry.disable()
    events = [json.loads(line) for line in open(sink)]
    assert [e["event"] for e in events] == ["ModelLoad", "Generation"] == seen
    load, gen = events
    assert load["model_type"] == "llama" and load["layers"] == 1 and load["device"] == "cpu" and load["load_ms"] >= 0
    assert load["model_dir_hash"] == telemetry.redact_path(d) and d not in json.dumps(events)      # paths only as a hash
    assert gen["prompt_tokens"] == 4 and 1 <= gen["generated_tokens"] <= 8 and gen["ttft_ms"] >= 0
    # only scalars pass: a token list handed to log_event is dropped
    telemetry.enable(sink)
    telemetry.log_event("X", {"tokens": [1, 2, 3], "n": 3})
    telemetry.disable()
    last = json.loads(open(sink).read().splitlines()[-1])
    assert last["event"] == "X" and "tokens" not in last and last["n"] == 3
    og.Model(d)
    assert len(open(sink).read().splitlines()) == 3          # disabled again


def test_tensor_dumps_follow_the_log_flags(tmp_path):
    """model_input_values / model_output_shapes / model_output_values: shapes, first and last values and statistics of the step's
    tensors go to the log callback (reference: src/models/debugging.cpp, src/models/model.cpp:115-130)."""
    import numpy as np
    import torch
    import onnxruntime_genai_b200 as og
    from helpers import tiny_model_dir
    from onnxruntime_genai_b200.utils.debugging import describe
    text = describe("x", torch.tensor([1.0, float("nan"), -3.0, 2.0]))
    assert "float32[4]" in text and "NON-FINITE: first at [1]" in text and "min -3 at [2]" in text and "max 2 at [3]" in text
    d, _ = tiny_model_dir(str(tmp_path / "m"), std=0.3)
    model = og.Model(d)
    lines = []
    og.set_log_callback(lines.append)
    og.set_log_options(enabled=True, model_input_values=True, model_output_shapes=True, model_output_values=True)
    try:
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=12, do_sample=False)
        g = og.Generator(model, p)
        g.append_tokens(np.asarray([[5, 6, 7]], dtype=np.int32))
        g.generate_next_token()
    finally:
        og.set_log_options(enabled=False, model_input_values=False, model_output_shapes=False, model_output_values=False)
        og.set_log_callback(None)
    joined = "\n".join(lines)
    assert "input_ids: int32[3]" in joined and "values: 5, 6, 7" in joined
    import re
    assert re.search(r"logits: float32\[1, \d+\] on cpu", joined) and "stddev" in joined
