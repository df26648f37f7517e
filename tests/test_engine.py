"""Engine contracts with scripted doubles on the host (modelled on the reference's engine_unit_tests and
test_onnxruntime_genai_engine.py: closed-form model, isolated == simultaneous, staggered admission, EOS /
max_length, continuation, capacity, transaction rollback, fatal failure, invariants)."""
import copy

import numpy as np
import pytest

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.engine.engine import Engine, EngineStepError, ExecutionFailure, FailureKind, Request, StepOutcome
from onnxruntime_genai_b200.native_loader import native

VOCAB, EOS = 64, 1


class ClosedFormExecutor:
    """next = (first_prompt_token + current_token + current_length) % vocab — no model math at all."""

    def __init__(self):
        self.calls = []
        self.script = []  # failures to raise, consumed front to back

    def execute(self, plan, edits=None, masks=None):
        self.calls.append([(e.request.id, e.num_tokens, e.processed_before, e.is_prefill) for e in plan.entries])
        if self.script:
            f = self.script.pop(0)
            if f is not None:
                raise f
        out = []
        for e in plan.entries:
            toks = e.request.tokens()
            cur = int(toks[e.processed_before + e.num_tokens - 1])
            out.append((int(toks[0]) + cur + e.processed_before + e.num_tokens) % VOCAB)
        return np.asarray(out, dtype=np.int32)


def closed_form(prompt, max_length):
    seq = list(prompt)
    out = []
    while len(seq) < max_length:
        t = (seq[0] + seq[-1] + len(seq)) % VOCAB
        seq.append(t)
        out.append(t)
        if t == EOS:      # the end-of-sequence token is streamed, then the turn ends
            break
    return out


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    from onnxruntime_genai_b200.models.arch import ArchConfig
    from onnxruntime_genai_b200.models.builder import export_model
    arch = ArchConfig(model_type="llama", vocab_size=VOCAB, hidden_size=32, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=16,
                      intermediate_size=32, context_length=128, bos_token_id=0, eos_token_id=EOS, pad_token_id=0)
    d = str(tmp_path_factory.mktemp("synthetic_paged"))
    export_model(arch, d, "fp32", "cpu", paged=True, block_size=4, num_blocks=128, max_batch_size=8, max_scheduled_tokens=32)
    return og.Model(d)


def make_engine(model, **kw):
    ex = ClosedFormExecutor()
    return Engine(model, executor=ex, **kw), ex


def request(model, prompt, max_length=40, **opts):
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=max_length, **opts)
    r = Request(p)
    r.add_tokens(np.asarray(prompt, dtype=np.int32))
    return r


def run_all(engine, reqs, check=True):
    outs = {id(r): [] for r in reqs}
    guard = 0
    while engine.has_pending_requests():
        guard += 1
        assert guard < 5000
        r = engine.step()
        if check:
            engine.core.check_invariants()
        if r is None:
            continue
        while r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r.is_turn_complete():
            engine.remove_request(r)
    return [outs[id(r)] for r in reqs]


def test_single_request_matches_closed_form(model):
    engine, _ = make_engine(model)
    r = request(model, [5, 9, 3])
    engine.add_request(r)
    assert run_all(engine, [r]) == [closed_form([5, 9, 3], 40)]
    assert engine.core.free_blocks == 128


def test_isolated_equals_simultaneous_and_staggered(model):
    prompts = [[5, 9, 3], [7], [2, 2, 2, 2, 2, 2, 2, 2, 2], [11, 60], [33] * 17]
    want = [closed_form(p, 40) for p in prompts]
    engine, _ = make_engine(model)
    reqs = [request(model, p) for p in prompts]
    for r in reqs:
        engine.add_request(r)
    assert run_all(engine, reqs) == want
    # staggered admission: add a request every few steps
    engine, _ = make_engine(model)
    reqs = [request(model, p) for p in prompts]
    outs = {id(r): [] for r in reqs}
    pending = list(reqs)
    steps = 0
    while pending or engine.has_pending_requests():
        if pending and steps % 3 == 0:
            engine.add_request(pending.pop(0))
        steps += 1
        r = engine.step()
        engine.core.check_invariants()
        if r is None:
            continue
        while r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r.is_turn_complete():
            engine.remove_request(r)
    assert [outs[id(r)] for r in reqs] == want


def test_eos_ends_the_turn_and_is_streamed_and_max_length_is_respected(model):
    # first=1, current=62, length 2 -> (1 + 62 + 2) % 64 == 1 == EOS immediately.  The sampled EOS is appended to the
    # sequence and reaches the caller (reference: src/engine/request.cpp CommitStep + src/search.cpp:266-296), then the turn ends.
    engine, _ = make_engine(model)
    r = request(model, [1, 62])
    engine.add_request(r)
    assert run_all(engine, [r]) == [[EOS]] and r.status == native.RequestStatus.Closed
    assert list(r.tokens()) == [1, 62, EOS]
    engine, _ = make_engine(model)
    r = request(model, [5, 9, 3], max_length=6)
    engine.add_request(r)
    out = run_all(engine, [r])[0]
    assert len(out) == 3 and len(r.tokens()) == 6


def test_decode_first_schedule_and_token_budget(model):
    engine, ex = make_engine(model)
    a, b = request(model, [3] * 40, max_length=60), request(model, [4] * 30, max_length=60)
    engine.add_request(a)
    engine.step()   # a prefill, budget 32
    assert ex.calls[0] == [(a._native.id, 32, 0, True)]
    engine.add_request(b)
    engine.step()
    # a still prefilling (8 left) comes first as a resident, then b gets the rest of the 32-token budget
    assert ex.calls[1] == [(a._native.id, 8, 32, True), (b._native.id, 24, 0, True)]
    engine.step()
    # a is now decoding: decodes are planned before prefills
    assert ex.calls[2][0] == (a._native.id, 1, 40, False) and ex.calls[2][1] == (b._native.id, 6, 24, True)


def test_chunk_size_caps_prefill_per_request(model):
    engine, ex = make_engine(model)
    r = request(model, [3] * 20, chunk_size=8)
    engine.add_request(r)
    engine.step(); engine.step(); engine.step()
    assert [c[0][1] for c in ex.calls[:3]] == [8, 8, 4]


def test_capacity_deferral_and_handle_release(model):
    engine, ex = make_engine(model, num_blocks=6)      # 24 slots
    a, b = request(model, [3] * 14, max_length=20), request(model, [4] * 14, max_length=20)
    engine.add_request(a)
    engine.add_request(b)
    engine.step()
    assert [c[0] for c in ex.calls[0]] == [a._native.id], "b does not fit while a holds 4 of 6 blocks"
    assert engine.last_outcome == StepOutcome.Committed
    outs = run_all(engine, [a, b])
    assert outs == [closed_form([3] * 14, 20), closed_form([4] * 14, 20)]
    assert engine.core.free_blocks == 6


def test_unserviceable_request_is_rejected(model):
    engine, _ = make_engine(model, num_blocks=2)
    r = request(model, [3] * 20, max_length=30)
    engine.add_request(r)
    with pytest.raises(EngineStepError, match="UnserviceableRequest"):
        engine.step()
    assert not engine.has_pending_requests()
    engine.core.check_invariants()


@pytest.mark.parametrize("kind,outcome", [(FailureKind.RetryableBeforeExecution, StepOutcome.RetryableBatchAbort),
                                          (FailureKind.RetryableDuringExecution, StepOutcome.RetryableBatchAbort),
                                          (FailureKind.CapacityExceeded, StepOutcome.ExecutionCapacityExceeded)])
def test_retryable_failure_rolls_the_step_back(model, kind, outcome):
    engine, ex = make_engine(model)
    reqs = [request(model, [5, 9, 3]), request(model, [7] * 9)]
    for r in reqs:
        engine.add_request(r)
    engine._run_model_step()
    free_before = engine.core.free_blocks
    tokens_before = [r.tokens().tolist() for r in reqs]
    ex.script = [ExecutionFailure(kind, "scripted")]
    engine._run_model_step()
    assert engine.last_outcome == outcome
    assert engine.core.free_blocks == free_before and [r.tokens().tolist() for r in reqs] == tokens_before
    assert engine.metrics["steps_aborted"] == 1 and not engine.core.transaction_open
    engine.core.check_invariants()
    # the retried step and everything after it produce exactly what an undisturbed run produces
    run_all(engine, reqs)
    assert [r.tokens().tolist() for r in reqs] == [[5, 9, 3] + closed_form([5, 9, 3], 40), [7] * 9 + closed_form([7] * 9, 40)]


def test_fatal_failure_marks_engine_unhealthy(model):
    engine, ex = make_engine(model)
    r = request(model, [5, 9, 3])
    engine.add_request(r)
    ex.script = [ExecutionFailure(FailureKind.Fatal, "device lost")]
    with pytest.raises(EngineStepError, match="FatalExecutionFailure"):
        engine.step()
    assert not engine.core.healthy
    with pytest.raises(RuntimeError, match="unhealthy"):
        engine.step()
    with pytest.raises(RuntimeError, match="unhealthy"):
        engine.add_request(request(model, [1, 2]))
    engine.core.check_invariants()


def test_post_processing_failure_is_a_contract_failure(model):
    engine, ex = make_engine(model)
    r = request(model, [5, 9, 3])
    engine.add_request(r)
    ex.script = [ExecutionFailure(FailureKind.PostProcessing, "bad logits shape")]
    with pytest.raises(EngineStepError, match="ExecutionContractFailure"):
        engine.step()
    assert engine.core.healthy and r.tokens().tolist() == [5, 9, 3]


def test_multi_turn_continuation_reuses_the_cache(model):
    engine, ex = make_engine(model)
    r = request(model, [5, 9, 3], max_length=8)
    engine.add_request(r)
    first = run_all_keep(engine, r)
    assert r.is_turn_complete() and len(r.tokens()) == 8
    with pytest.raises(RuntimeError):
        r.continue_with([4])                     # max_length is cumulative across turns
    r2 = request(model, [5, 9, 3], max_length=30)
    engine.add_request(r2)
    while not r2.is_turn_complete() or r2.has_unseen_tokens():
        x = engine.step()
        while x is not None and x.has_unseen_tokens():
            x.get_unseen_token()
        if len(r2.tokens()) >= 7:
            break
    n_calls = len(ex.calls)
    # finish the turn by hitting max_length, then continue
    r3 = request(model, [6, 6], max_length=5)
    engine.add_request(r3)
    run_all_keep(engine, r3)
    assert r3.is_turn_complete()
    p = r3._native.processed
    r3.params.search["max_length"] = 5
    with pytest.raises(RuntimeError):
        r3.continue_with([1, 2, 3])


def run_all_keep(engine, r):
    out = []
    guard = 0
    while not r.is_turn_complete() or r.has_unseen_tokens():
        guard += 1
        assert guard < 1000
        x = engine.step()
        engine.core.check_invariants()
        while x is not None and x.has_unseen_tokens():
            out.append(x.get_unseen_token())
    return out


def test_continue_with_only_processes_the_new_tokens(model):
    engine, ex = make_engine(model)
    r = request(model, [5, 9, 3], max_length=40)
    # stop the turn early through EOS: craft so that the next token is EOS
    engine.add_request(r)
    for _ in range(3):
        engine.step()
    r.get_unseen_token() if r.has_unseen_tokens() else None
    # cannot continue an active turn
    with pytest.raises(RuntimeError):
        r.continue_with([4, 4])
    engine.remove_request(r)
    q = request(model, [1, 62], max_length=40)      # EOS at once -> turn complete with processed == 2
    engine.add_request(q)
    run_all_keep(engine, q)
    assert q.is_turn_complete() and q._native.processed == 2
    ex.calls.clear()
    q.continue_with([10, 11, 12])
    assert q.status == native.RequestStatus.Assigned
    engine.step()
    # the end-of-turn token of the first turn was sampled but never fed: it leads the next turn's prefill (4 tokens)
    assert ex.calls[0] == [(q._native.id, 4, 2, True)], "only the unprocessed tokens are fed; the cached prefix is reused"


def test_remove_request_reclaims_blocks_and_teardown(model):
    engine, _ = make_engine(model)
    reqs = [request(model, [i + 2] * 10) for i in range(4)]
    for r in reqs:
        engine.add_request(r)
    engine.step()
    assert engine.core.free_blocks < 128
    for r in reqs:
        engine.remove_request(r)
    assert engine.core.free_blocks == 128 and not engine.has_pending_requests()
    engine.core.check_invariants()
    del engine
    engine, _ = make_engine(model)                  # recreate after teardown
    r = request(model, [5, 9, 3])
    engine.add_request(r)
    assert run_all(engine, [r]) == [closed_form([5, 9, 3], 40)]


def test_request_validation(model):
    engine, _ = make_engine(model)
    with pytest.raises(RuntimeError):
        engine.add_request(request(model, [1] * 50, max_length=40))          # prompt leaves no room
    p = og.GeneratorParams(model)
    p.set_search_options(num_beams=2)
    r = Request(p)
    r.add_tokens(np.asarray([1, 2], dtype=np.int32))
    with pytest.raises(RuntimeError, match="beam"):
        engine.add_request(r)
    r = request(model, [1, 2])
    engine.add_request(r)
    with pytest.raises(RuntimeError):
        engine.add_request(r)
    with pytest.raises(RuntimeError):
        r.add_tokens([3])


def test_block_pool_unit():
    pool = native.BlockPool(4)
    a = pool.reserve(3)
    assert a == [0, 1, 2] and pool.free_count == 1
    assert pool.reserve(2) is None and pool.free_count == 1, "reservation is all-or-nothing"
    pool.commit(0); pool.release(1); pool.release(2)
    assert pool.free_count == 3
    with pytest.raises(Exception):
        pool.free(1)                                 # not committed
    pool.free(0)
    assert pool.reserve(4) == [0, 1, 2, 3]


def test_sampling_args_resolution():
    o = native.RequestOptions()
    o.do_sample = False
    assert o.resolve() == (1, 0.0, 1.0)
    o.do_sample, o.top_k, o.top_p, o.temperature = True, 40, 0.0, 0.7
    assert o.resolve()[0] == 40 and o.resolve()[1] == 1.0
    o.top_k, o.top_p = 0, 0.9
    k, p, t = o.resolve()
    assert k == -1 and abs(p - 0.9) < 1e-6 and abs(t - 0.7) < 1e-6
    o.top_k = 1
    assert o.resolve() == (1, 0.0, 1.0)


# ------------------------------------------------------------------------------------------------ decode look-ahead
class AheadExecutor(ClosedFormExecutor):
    """The asynchronous executor seam with a stand-in for the device: `enqueue_next` computes the following step from the
    PREVIOUS handle's ids and its own copy of positions (never from the requests, whose new ids have not been committed
    yet), as the device-side advance does."""

    def __init__(self):
        super().__init__()
        self.ahead_calls = 0

    def execute_async(self, plan, edits=None, masks=None):
        toks = self.execute(plan, edits, masks)
        state = None
        if plan.graph_eligible:
            state = [(int(e.request.tokens()[0]), e.processed_before + 1) for e in plan.entries]   # (first token, length after)
        return {"toks": toks, "state": state}

    def enqueue_next(self, plan, handle):
        if handle["state"] is None or not plan.lookahead_ok:
            return None
        self.ahead_calls += 1
        toks, state = [], []
        for (first, length), cur in zip(handle["state"], handle["toks"].tolist()):
            toks.append((first + cur + length + 1) % VOCAB)
            state.append((first, length + 1))
        return {"toks": np.asarray(toks, dtype=np.int32), "state": state}

    def refresh_inputs(self, plan):
        self.refreshed = getattr(self, "refreshed", 0) + 1      # the device copy of the inputs of a step that is already running

    def collect(self, handle):
        return handle["toks"]


def test_lookahead_steps_match_the_synchronous_engine(model):
    prompts = [[5, 9, 2], [7], [11, 3, 4, 8, 15, 16, 23], [2, 2]]
    sync, _ = make_engine(model)
    sreqs = [request(model, p, max_length=30 + i) for i, p in enumerate(prompts)]
    for r in sreqs:
        sync.add_request(r)
    want = run_all(sync, sreqs)
    ex = AheadExecutor()
    engine = Engine(model, executor=ex, lookahead=True)
    assert engine.options.lookahead == 1
    reqs = [request(model, p, max_length=30 + i) for i, p in enumerate(prompts)]
    for r in reqs[:3]:
        engine.add_request(r)
    outs = {id(r): [] for r in reqs}
    steps = 0
    while engine.has_pending_requests():
        steps += 1
        assert steps < 2000
        if steps == 9:
            engine.add_request(reqs[3])          # a new request arrives while a step enqueued ahead is pending: it is dropped
        r = engine.step()
        if r is None:
            continue
        while r.has_unseen_tokens():
            outs[id(r)].append(r.get_unseen_token())
        if r.is_turn_complete():
            engine.remove_request(r)
    assert [outs[id(r)] for r in reqs] == want
    assert engine.lookahead_hits > 10 and ex.ahead_calls >= engine.lookahead_hits and ex.refreshed == engine.lookahead_hits
    engine.core.check_invariants()
    assert engine.core.free_blocks == engine.options.num_blocks


def test_lookahead_plan_reserves_the_next_block_and_predicts_the_next_signature():
    o = native.EngineOptions()
    o.block_size, o.num_blocks, o.max_batch_size, o.max_scheduled_tokens, o.vocab_size, o.eos_ids, o.lookahead = 4, 16, 4, 16, VOCAB, [EOS], 1
    core = native.EngineCore(o)
    ro = native.RequestOptions()
    ro.max_length = 12
    r = core.create_request(ro)
    r.add_tokens(np.asarray([3, 4, 5], dtype=np.int32))
    core.add_request(r)
    plan = core.plan()                               # prefill of 3 tokens: no look-ahead for prefill entries
    assert not plan.lookahead_ok and plan.entries[0].is_prefill
    core.commit(np.asarray([7], dtype=np.int32))
    held = lambda: o.num_blocks - core.free_blocks
    assert held() == 1
    plan = core.plan()                               # decode of token 4 (position 3): position 4 opens block 1 -> reserved now
    assert plan.lookahead_ok and plan.graph_eligible
    nxt = plan.next_signature
    core.commit(np.asarray([8], dtype=np.int32))
    assert held() == 2
    plan = core.plan()
    assert plan.signature == nxt and plan.lookahead_ok
    core.commit(np.asarray([9], dtype=np.int32))
    # a different request set gives a different signature
    r2 = core.create_request(ro)
    r2.add_tokens(np.asarray([1, 2], dtype=np.int32))
    core.add_request(r2)
    nxt = plan.next_signature
    plan = core.plan()
    assert plan.signature != nxt and not plan.lookahead_ok
    core.abort(native.FailureKind.RetryableBeforeExecution, "test")
    core.check_invariants()


def test_static_batching_runs_fixed_batches_to_completion():
    """engine.static_batching (reference: src/engine/scheduler.cpp:57-113): up to four waiting requests are admitted together
    with the blocks of their whole max_length, nothing joins while the batch runs, the batch size halves (4, 2, 1) until the
    cache holds it, and search.chunk_size is refused."""
    o = native.EngineOptions()
    o.block_size, o.num_blocks, o.max_batch_size, o.max_scheduled_tokens, o.vocab_size, o.eos_ids = 4, 12, 8, 64, VOCAB, [EOS]
    o.static_batching = True
    core = native.EngineCore(o)

    def request(n_prompt, max_length, chunk=0):
        ro = native.RequestOptions()
        ro.max_length, ro.chunk_size = max_length, chunk
        r = core.create_request(ro)
        r.add_tokens(np.arange(3, 3 + n_prompt, dtype=np.int32))
        return r

    with pytest.raises(RuntimeError, match="chunk_size requires dynamic batching"):
        core.add_request(request(3, 8, chunk=2))
    reqs = [request(3, 8) for _ in range(6)]          # 2 blocks each at full length: 12 blocks hold 6, a batch is 4
    for r in reqs:
        core.add_request(r)
    plan = core.plan()
    assert [e.request.id for e in plan.entries] == [r.id for r in reqs[:4]] and all(e.is_prefill for e in plan.entries)
    assert core.free_blocks == 12 - 4 * 2              # the whole max_length is owned from the first step
    core.commit(np.full(4, 9, dtype=np.int32))
    late = request(2, 6)
    core.add_request(late)                             # arrives while the batch runs: waits for the next batch
    for _ in range(4):                                 # 3 prompt tokens + 5 generated = max_length 8; one came with the prefill
        plan = core.plan()
        assert [e.request.id for e in plan.entries] == [r.id for r in reqs[:4]] and not any(e.newly_admitted for e in plan.entries)
        core.commit(np.full(4, 9, dtype=np.int32))
    # the finished batch keeps its blocks until its requests are removed: only one full-length request fits beside it
    plan = core.plan()
    assert [e.request.id for e in plan.entries] == [reqs[4].id] and plan.entries[0].newly_admitted
    core.commit(np.asarray([EOS], dtype=np.int32))
    for r in reqs[:5]:
        core.remove_request(r)
    plan = core.plan()                                 # two are waiting: the last of the first wave and the late arrival
    assert [e.request.id for e in plan.entries] == [reqs[5].id, late.id]
    core.commit(np.full(2, EOS, dtype=np.int32))
    core.check_invariants()

    # halving: a pool that cannot hold four full-length requests takes two
    o.num_blocks = 5
    small = native.EngineCore(o)
    core = small
    rs = [request(3, 8) for _ in range(4)]
    for r in rs:
        small.add_request(r)
    plan = small.plan()
    assert [e.request.id for e in plan.entries] == [rs[0].id, rs[1].id] and small.free_blocks == 1
    small.commit(np.full(2, EOS, dtype=np.int32))      # both finish at once
    plan = small.plan()                                # their blocks are still held: nothing fits, the step is deferred
    assert not plan.entries and plan.deferred == 1
    small.remove_request(rs[0])
    small.remove_request(rs[1])
    plan = small.plan()
    assert [e.request.id for e in plan.entries] == [rs[2].id, rs[3].id]
    small.commit(np.full(2, EOS, dtype=np.int32))
    small.remove_request(rs[2])
    small.remove_request(rs[3])
    small.check_invariants()
    assert small.free_blocks == 5


def test_engine_with_a_static_batching_config(model, tmp_path):
    """`engine.static_batching` in genai_config.json selects the fixed-batch policy; outputs equal the closed form and no
    request joins a running batch."""
    import json
    import os
    import shutil
    d = str(tmp_path / "static")
    shutil.copytree(model.config.config_path, d)
    cfg_path = os.path.join(d, "genai_config.json")
    with open(cfg_path) as f:
        cfg = json.load(f)
    cfg["engine"] = {"static_batching": {"max_batch_size": 4}}
    with open(cfg_path, "w") as f:
        json.dump(cfg, f)
    m = og.Model(d)
    engine, ex = make_engine(m, num_blocks=64)
    assert engine.options.static_batching
    prompts = [[3 + i, 9, 4 + i] for i in range(6)]
    reqs = [request(m, p, max_length=12) for p in prompts]
    for r in reqs:
        engine.add_request(r)
    outs = run_all(engine, reqs)
    assert outs == [closed_form(p, 12) for p in prompts]
    first = {c[0] for c in ex.calls[0]}
    assert len(first) == 4                              # four requests start together ...
    started = set()
    for call in ex.calls:
        ids = {c[0] for c in call}
        if ids & first:
            assert ids <= first                         # ... and nobody joins while any of them still runs
        started |= ids
    assert len(started) == 6


def test_decode_advance_reference():
    import torch
    from onnxruntime_genai_b200 import ops
    table = torch.tensor([[5, 9, -1], [2, 7, 3]], dtype=torch.int32)
    ids, pos = torch.tensor([1, 2], dtype=torch.int32), torch.tensor([3, 7], dtype=torch.int32)
    past, slots, spos = pos.clone(), torch.tensor([5 * 4 + 3, 7 * 4 + 3], dtype=torch.int32), torch.tensor([4, 8], dtype=torch.int32)
    ops.decode_advance(torch.tensor([40, 41], dtype=torch.int32), ids, pos, past, slots, spos, table, 4)
    assert ids.tolist() == [40, 41] and pos.tolist() == [4, 8] and past.tolist() == [4, 8] and spos.tolist() == [5, 9]
    assert slots.tolist() == [9 * 4 + 0, 3 * 4 + 0]
    ops.decode_advance(torch.tensor([1, 1], dtype=torch.int32), ids, pos, past, slots, spos, table[:, :2], 4)
    assert slots.tolist() == [9 * 4 + 1, -1]       # position 9 lies in column 2, which this table does not have


def test_attention_split_choice():
    from onnxruntime_genai_b200 import ops
    # 64 requests x 8 / 4 / 2 / 1 kv heads per GPU, requests issued longest first: 1 / 2 / 4 / 4 even parts (no fixed chunk)
    for hkv, want in ((8, 1), (4, 2), (2, 4), (1, 4)):
        assert ops.choose_kv_splits(64, hkv, 1, 4096, group=4, ordered=True) == (want, 0)
        assert ops.choose_kv_splits(64, hkv, 1, 1 << 24, group=4, ordered=True) == (want, 0)     # independent of the bound
    assert ops.choose_kv_splits(64, 2, 1, 300, group=4, ordered=True) == (1, 0)                   # pieces would be too short
    # unordered small batches keep fixed chunks sized for the GPU; big batches and prefill-sized steps do not split
    s, chunk = ops.choose_kv_splits(1, 8, 1, 8192, group=4)
    assert s > 1 and chunk % 64 == 0 and s * chunk >= 8192
    assert ops.choose_kv_splits(64, 8, 1, 4096, group=4) == (1, 0)
    assert ops.choose_kv_splits(4, 8, 512, 4096, group=4) == (1, 0)


def test_abandoned_request_is_reclaimed_at_the_next_boundary(tmp_path):
    """Dropping the last reference to a submitted request (no remove_request) frees its blocks before the next step
    (reference: src/engine/engine.cpp:107-136, abandoned-handle reclamation)."""
    import gc
    import onnxruntime_genai_b200 as og
    from helpers import tiny_model_dir
    d, _ = tiny_model_dir(str(tmp_path / "m"), std=0.3)
    model = og.Model(d)
    eng = og.Engine(model)
    free0 = eng.core.free_blocks

    def submit(n):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=n + 40, do_sample=False)
        r = og.Request(p)
        r.add_tokens(np.arange(3, 3 + n, dtype=np.int32))
        eng.add_request(r)
        return r

    def drain(r):
        while r.has_unseen_tokens():
            r.get_unseen_token()

    keep, drop = submit(20), submit(33)
    for _ in range(3):
        eng.step()
        drain(keep)
        drain(drop)
    assert eng.core.free_blocks < free0
    used_both = free0 - eng.core.free_blocks
    del drop
    gc.collect()
    eng.step()                                   # the boundary: the abandoned request goes
    drain(keep)
    assert eng.reclaimed == 1
    assert free0 - eng.core.free_blocks < used_both
    for _ in range(200):
        if not eng.has_pending_requests():
            break
        eng.step()
        drain(keep)
    assert keep.is_turn_complete()
    eng.remove_request(keep)
    assert eng.core.free_blocks == free0 and eng.reclaimed == 1
