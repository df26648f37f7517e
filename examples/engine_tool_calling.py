"""Tool calling through the continuous-batching engine (counterpart of the reference's
examples/python/engine/tool-calling.py): several conversations run concurrently; each answer is constrained to a JSON object
that names one of the offered tools and its arguments, and every turn continues the same request (the cached prefix of
the conversation is reused).

    python examples/engine_tool_calling.py -m <model_dir> -q "Weather in Paris?" "What is 17 * 23?"
"""
import argparse
import json

import onnxruntime_genai_b200 as og

TOOLS = [
    {"name": "get_weather", "description": "Current weather for a city", "parameters": {
        "type": "object", "properties": {"city": {"type": "string"}}, "required": ["city"], "additionalProperties": False}},
    {"name": "calculator", "description": "Evaluate an arithmetic expression", "parameters": {
        "type": "object", "properties": {"expression": {"type": "string"}}, "required": ["expression"], "additionalProperties": False}},
]


def call_schema(tools):
    """One JSON object {"name": <tool>, "arguments": {...}} for exactly one of the tools."""
    return {"anyOf": [{"type": "object", "properties": {"name": {"const": t["name"]}, "arguments": t["parameters"]},
                       "required": ["name", "arguments"], "additionalProperties": False} for t in tools]}


def run_tool(call):
    if call["name"] == "get_weather":
        return {"city": call["arguments"]["city"], "temperature_c": 21, "sky": "clear"}
    try:
        return {"value": eval(call["arguments"]["expression"], {"__builtins__": {}}, {})}   # toy calculator
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-q", "--questions", nargs="*", default=["What is the weather in Paris?", "What is 17 * 23?"])
    ap.add_argument("--max_new_tokens", type=int, default=96)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    cfg = og.Config(a.model)
    if a.cpu:
        cfg.clear_providers()
    model = og.Model(cfg)
    tok = og.Tokenizer(model)
    engine = og.Engine(model)
    schema = json.dumps(call_schema(TOOLS))
    state = {}
    for q in a.questions:
        msgs = [{"role": "system", "content": "Answer with one tool call."}, {"role": "user", "content": q}]
        ids = tok.encode(tok.apply_chat_template(json.dumps(msgs), tools=json.dumps(TOOLS), add_generation_prompt=True))
        params = og.GeneratorParams(model)
        params.set_search_options(max_length=len(ids) + 2 * a.max_new_tokens + 64)
        params.set_guidance("json_schema", schema)
        req = og.Request(params)
        req.add_tokens(ids)
        req.set_opaque_data(q)
        engine.add_request(req)
        state[id(req)] = {"text": [], "turn": 0}
    while engine.has_pending_requests():
        req = engine.step()
        if req is None:
            continue
        st = state[id(req)]
        while req.has_unseen_tokens():
            st["text"].append(req.get_unseen_token())
        if not req.is_turn_complete():
            continue
        answer = tok.decode(st["text"])
        print(f"[{req.get_opaque_data()!r}] turn {st['turn']}: {answer}")
        call = None
        if st["turn"] == 0:
            try:
                call = json.loads(answer)
            except ValueError:
                print("  (the answer ran into the length limit before the JSON object was closed)")
        if call is None:
            engine.remove_request(req)
            continue
        follow = tok.apply_chat_template(json.dumps([{"role": "tool", "content": json.dumps(run_tool(call))}]), add_generation_prompt=True)
        st["text"], st["turn"] = [], 1
        req.continue_with(tok.encode(follow))      # next turn of the same request: the conversation so far stays cached


if __name__ == "__main__":
    main()
