"""Continuous-batching engine: `Engine.add_request / step / remove_request / has_pending_requests`
and `Request` (reference API: src/python/python.cpp:731-768; canonical loop:
examples/python/engine/continuous-batching.py:80-113).

One `step()` is a transaction driven by the native core (native/engine_core.cpp):
plan + reserve blocks + checkpoint -> pack the step inputs into ONE pinned staging buffer -> one
H2D copy -> forward over the packed tokens (CUDA graph replay for pure-decode steps, bucketed by
batch and block-table width) -> logits edits / grammar masks -> one sampler launch with per-row
parameters -> one small D2H of the sampled ids -> commit.  A failure while executing aborts the
transaction: every request and every reserved block returns to its state before the step; a fatal
failure marks the engine unhealthy (reference: src/engine/engine.cpp:227-478).

The executor is injectable (`Engine(model, executor=...)`), which is how the tests script
retryable / capacity / fatal failures on the host without touching a GPU.
"""
from __future__ import annotations

import os
import time
import weakref
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..api import GeneratorParams, Model, _Trace
from ..models.decoder import PagedKVCache, StepInputs
from ..native_loader import native

FailureKind = native.FailureKind
StepOutcome = native.StepOutcome


class EngineStepError(RuntimeError):
    def __init__(self, outcome, message):
        super().__init__(f"{outcome.name}: {message}")
        self.outcome = outcome


class ExecutionFailure(Exception):
    """Raised by an executor to classify a failure (kind: native.FailureKind)."""

    def __init__(self, kind, message=""):
        super().__init__(message or kind.name)
        self.kind = kind


class Request:
    def __init__(self, params: GeneratorParams):
        self.params = params
        self._pending_tokens: List[int] = []
        self._native = None
        self._engine = None
        self._opaque = None
        self._adapter: Optional[str] = None
        self.t_added = self.t_first = None

    # tokens ------------------------------------------------------------------------------------
    def add_tokens(self, ids):
        arr = np.asarray(ids, dtype=np.int32).reshape(-1)
        if self._native is not None:
            self._native.add_tokens(arr)  # raises: already assigned
        if arr.size == 0:
            raise RuntimeError("add_tokens: empty token list")
        self._pending_tokens.extend(arr.tolist())

    def continue_with(self, ids, max_length: Optional[int] = None):
        """Queues another turn on the request's resident state.  max_length: a new (larger) cumulative limit for the turns to
        come - a turn that ended by reaching max_length can only be continued with one; bounded by the model's context."""
        if self._native is None:
            raise RuntimeError("continue_with: the request has not been added to an engine")
        if max_length is not None:
            limit = int(self._engine.model.config.context_length)
            if max_length > limit:
                raise RuntimeError(f"continue_with: max_length {max_length} exceeds the model's context length {limit}")
            self.params.search["max_length"] = int(max_length)
        self._native.continue_with(np.asarray(ids, dtype=np.int32).reshape(-1), int(max_length or 0))

    def has_unseen_tokens(self) -> bool:
        return self._native is not None and self._native.has_unseen_tokens()

    def get_unseen_token(self) -> int:
        if self._native is None:
            raise RuntimeError("get_unseen_token: no unseen tokens")
        return self._native.get_unseen_token()

    def is_turn_complete(self) -> bool:
        return self._native is not None and self._native.is_turn_complete()

    def is_done(self) -> bool:
        return self.is_turn_complete()

    def set_active_adapter(self, adapters, name: Optional[str]):
        """This request's tokens run with the named LoRA adapter (None: the base model).  Requests with different adapters, and
        with none, share engine steps: the low-rank products are grouped by adapter inside each step."""
        if name is not None and name not in adapters._loaded:
            raise RuntimeError(f"adapter '{name}' is not loaded")
        self._adapter = name
        if self._engine is not None:
            self._engine._adapter_requests = sum(1 for r in self._engine._by_native.values() if r._adapter is not None)

    def set_opaque_data(self, obj):
        self._opaque = obj

    def get_opaque_data(self):
        return self._opaque

    @property
    def status(self):
        return self._native.status if self._native is not None else native.RequestStatus.Unassigned

    def tokens(self) -> np.ndarray:
        return self._native.tokens() if self._native is not None else np.asarray(self._pending_tokens, dtype=np.int32)

    def _options(self):
        s = self.params.search
        o = native.RequestOptions()
        o.max_length, o.min_length, o.do_sample = int(s["max_length"]), int(s["min_length"]), bool(s["do_sample"])
        o.top_k, o.top_p, o.temperature = int(s["top_k"]), float(s["top_p"]), float(s["temperature"])
        o.repetition_penalty, o.no_repeat_ngram_size = float(s["repetition_penalty"]), int(s["no_repeat_ngram_size"])
        o.random_seed, o.chunk_size = int(s["random_seed"]), int(s.get("chunk_size") or 0)
        o.num_beams, o.batch_size = int(s["num_beams"]), int(s["batch_size"])
        if self.params.guidance_type and self.params.guidance_ff_tokens:
            raise RuntimeError("Engine requests do not support guidance ff_tokens")
        return o


# ------------------------------------------------------------------------------------------------ staging
class _Staging:
    """All per-step inputs in one pinned host buffer with a device mirror (one H2D copy per step)."""

    FIELDS_TOK = ["input_ids", "positions", "token_row", "slot_mapping", "slot_mapping_w"]
    FIELDS_ROW = ["past_lens", "logits_rows", "top_k", "sample_pos", "attn_order"]

    def __init__(self, max_tokens: int, max_batch: int, table_cols: int, device: torch.device, windowed: bool):
        self.max_tokens, self.max_batch, self.table_cols = max_tokens, max_batch, table_cols
        lay, off = {}, 0

        def add(name, n_words):
            nonlocal off
            lay[name] = (off, n_words)
            off += (n_words + 3) // 4 * 4  # 16-byte alignment
        for f in self.FIELDS_TOK:
            add(f, max_tokens)
        add("cu_seqlens", max_batch + 1)
        for f in self.FIELDS_ROW:
            add(f, max_batch)
        add("state_slots", max_batch)     # recurrent models: slot of every request in the state pool (filled by the executor, not the core)
        add("top_p", max_batch)
        add("temperature", max_batch)
        add("seeds", 2 * max_batch)
        add("block_table", max_batch * table_cols)
        if windowed:
            add("block_table_w", max_batch * table_cols)
        self.layout, self.words = lay, off
        pin = device.type == "cuda"
        # Two pinned host images used in turn: with decode look-ahead the copy of one step's inputs may still be queued
        # behind the running step when the host packs the next one.
        self._hosts = [torch.zeros(off, dtype=torch.int32, pin_memory=pin) for _ in range(2 if pin else 1)]
        self._addrs = []
        self.host = self._hosts[0]
        self.dev = torch.zeros(off, dtype=torch.int32, device=device) if pin else self.host
        self.tokens_host = torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin)
        # asynchronous steps land their ids in a ring of pinned buffers (a step's ids are read while the next step runs)
        self.tokens_ring = [torch.zeros(max_batch, dtype=torch.int32, pin_memory=pin) for _ in range(4)]
        self.ring_next = 0
        for h in self._hosts:
            a = {k: h.data_ptr() + 4 * o for k, (o, _) in lay.items() if k != "state_slots"}
            if not windowed:
                a.pop("slot_mapping_w", None)
            self._addrs.append(a)
        self.addr = self._addrs[0]
        self._cur = 0

    def host_np(self) -> np.ndarray:
        """The current pinned host image as a numpy array (shares memory)."""
        if not hasattr(self, "_np"):
            self._np = [h.numpy() for h in self._hosts]
        return self._np[self._cur]

    def flip(self):
        """Switches to the other pinned host image (call before packing a step)."""
        self._cur = (self._cur + 1) % len(self._hosts)
        self.host, self.addr = self._hosts[self._cur], self._addrs[self._cur]

    def view(self, name, n=None, dtype=torch.int32, host=False):
        o, w = self.layout[name]
        t = (self.host if host else self.dev)[o:o + w]
        if dtype != torch.int32:
            t = t.view(dtype)
        return t if n is None else t[:n]

    def upload(self):
        if self.dev is not self.host:
            self.dev.copy_(self.host, non_blocking=True)

    @property
    def h2d_bytes(self):
        return self.words * 4


# ------------------------------------------------------------------------------------------------ executor
class ModelExecutor:
    """Runs the model for a planned step and returns the sampled token per plan entry."""

    def __init__(self, model: Model, core, staging: _Staging, kv: PagedKVCache, use_graphs: bool):
        self.model, self.core, self.staging, self.kv = model, core, staging, kv
        self.decoder = model.decoder
        self.use_graphs = use_graphs and model.device.type == "cuda"
        self.graphs: Dict[Any, Any] = {}
        self.windowed = kv.win is not None
        self.graph_launches: Dict[Any, int] = {}
        self.last_key = None       # graph key of the step enqueued last (None: it did not run from a graph)
        self._unsplit: Dict[int, bool] = {}
        # decode steps issue the attention CTAs of long requests first (OGB_ATTN_ORDER=0: in batch order)
        self.order_attention = self.use_graphs and os.environ.get("OGB_ATTN_ORDER", "1") != "0"
        self.lora_of = None          # set by the engine: plan -> (per-token adapter ids on the device, adapter names) or None
        self.state_slots_of = None   # set by the engine for models with linear-attention layers: plan -> [B] int32 state slots
        self._graph_state_slots = False   # building the inputs of a graph step: the state slots are read from the staging buffer

    def _step_inputs(self, T: int, B: int, cols: int, max_q: int, max_kv: int, ordered: bool = False) -> StepInputs:
        st = self.staging
        table = st.view("block_table").view(st.max_batch, st.table_cols)[:B, :cols]
        s = StepInputs(input_ids=st.view("input_ids", T), positions=st.view("positions", T), slot_mapping=st.view("slot_mapping", T),
                       cu_seqlens=st.view("cu_seqlens", B + 1), past_lens=st.view("past_lens", B), block_table=table,
                       logits_rows=st.view("logits_rows", B), max_q_len=max_q, max_kv_len=max_kv)
        if self.state_slots_of is not None and self._graph_state_slots:
            s.state_slots = st.view("state_slots", B)
        if self.windowed:
            s.slot_mapping_w = st.view("slot_mapping_w", T)
            s.block_table_w = st.view("block_table_w").view(st.max_batch, st.table_cols)[:B, :cols]
        if ordered:
            s.attn_order = st.view("attn_order", B)
        return s

    @staticmethod
    def _bucket(n: int, lo: int = 1) -> int:
        b = lo
        while b < n:
            b *= 2
        return b

    def forward(self, plan) -> torch.Tensor:
        B, T = len(plan.entries), plan.token_count
        st = self.staging
        lora = self.lora_of(plan) if self.lora_of is not None else None
        if self.use_graphs and plan.graph_eligible and lora is None:
            key = self.upload_graph_inputs(plan)
            g = self.graphs.get(key)
            if g is None:
                g = self._capture(*key)
                self.graphs[key] = g
            graph, logits = g
            graph.replay()
            self.last_key = key
            return logits[:B]
        st.upload()
        s = self._step_inputs(T, B, st.table_cols, plan.max_query_len, plan.max_kv_len)
        if plan.max_query_len > 1:
            # decode-first schedule: the requests that feed one token lead the batch
            nd = 0
            for e in plan.entries:
                if e.num_tokens != 1:
                    break
                nd += 1
            s.num_decode = nd
        if lora is not None:
            s.lora_ids, s.lora_names = lora
        if self.state_slots_of is not None:
            s.state_slots = self.state_slots_of(plan)
        return self.decoder.forward(s, self.kv)

    def upload_graph_inputs(self, plan):
        """Pads the packed inputs of a one-token-per-request step to the graph's batch bucket, copies them to the device
        and returns the graph key (batch bucket, block-table column bucket)."""
        B, T = len(plan.entries), plan.token_count
        st = self.staging
        bb = min(self._bucket(B), st.max_batch)
        cb = min(self._bucket(plan.block_table_columns, 8), st.table_cols)
        if bb not in self._unsplit:
            # The column bucket only bounds the key range that the attention launch splits; a batch whose split choice does not
            # depend on the length (no split, or an even division) has one graph for every length (no capture in the middle of
            # a long decode).  Not for long-context RoPE models, whose step bound also selects the cache pair.
            dec = self.decoder
            g_ = dec.heads_local // dec.kv_heads_local
            far = ops.choose_kv_splits(bb, dec.kv_heads_local, 1, 1 << 24, group=g_, ordered=self.order_attention)
            near = ops.choose_kv_splits(bb, dec.kv_heads_local, 1, 4096, group=g_, ordered=self.order_attention)
            self._unsplit[bb] = dec.cos_small is None and far == near and far[1] == 0
        if self._unsplit[bb]:
            cb = st.table_cols
        key = (bb, cb)
        if bb > B:  # padded rows: zero-length requests that append nothing
            h = st.host
            o, _ = st.layout["cu_seqlens"]
            h[o + B + 1:o + bb + 1] = int(h[o + B])
            for f, val in (("past_lens", 0), ("logits_rows", 0)):
                o, _ = st.layout[f]
                h[o + B:o + bb] = val
            for f, val in (("input_ids", 0), ("positions", 0), ("slot_mapping", -1)):
                o, _ = st.layout[f]
                h[o + T:o + bb] = val
            if self.windowed:
                o, _ = st.layout["slot_mapping_w"]
                h[o + T:o + bb] = -1
        if self.state_slots_of is not None:
            # recurrent models: the requests' state slots travel with the other inputs (padded rows feed no token and touch no state)
            o, _ = st.layout["state_slots"]
            hn = st.host_np()
            hn[o:o + B] = self.state_slots_of(plan, host=True)
            hn[o + B:o + bb] = 0
        if self.order_attention:
            # requests by cached length, longest first: the order in which the attention kernel issues its CTAs
            hn = st.host_np()
            o, _ = st.layout["past_lens"]
            oo, _ = st.layout["attn_order"]
            hn[oo:oo + bb] = np.argsort(-hn[o:o + bb], kind="stable")
        st.upload()
        return key

    def _capture(self, bb: int, cb: int):
        st = self.staging
        self._graph_state_slots = True
        s = self._step_inputs(bb, bb, st.table_cols, 1, cb * self.kv.block_size, ordered=self.order_attention)
        self._graph_state_slots = False
        # the warm-up runs really execute the step: appending keys and values again is harmless, advancing a recurrent state is
        # not, so the states are copied aside and put back before the first replay
        saved = self.kv.state.clone() if (self.state_slots_of is not None and self.kv.state is not None) else None
        tp = self.decoder.tp
        if tp.size > 1:
            tp.barrier()   # ranks enter warm-up and capture together (peer waits in the fused kernels are bounded)
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for _ in range(2):  # warm-up: tensor maps, attribute set-up, allocator
                self.decoder.forward(s, self.kv)
        torch.cuda.current_stream().wait_stream(stream)
        if saved is not None:
            self.kv.state.copy_(saved)
            del saved
        torch.cuda.synchronize()
        from ..ops import _lib
        before = _lib.LAUNCH_COUNT
        graph = torch.cuda.CUDAGraph()
        with ops.graph_capture(graph):
            logits = self.decoder.forward(s, self.kv)
        self.graph_launches[(bb, cb)] = _lib.LAUNCH_COUNT - before
        return graph, logits

    def execute(self, plan, edits=None, masks=None) -> np.ndarray:
        st = self.staging
        B = len(plan.entries)
        with torch.no_grad():
            logits = self.forward(plan)
            for e in edits or ():  # penalties first, then bans (separate launches: no write race on a token)
                ops.logits_edit(logits, *e)
            if masks is not None:
                ops.logits_bitmask(logits, *masks)
            toks = ops.sample(logits, st.view("top_k", B), st.view("top_p", B, torch.float32), st.view("temperature", B, torch.float32),
                              st.view("seeds", None, torch.int64)[:B], st.view("sample_pos", B))
        if toks.is_cuda:
            st.tokens_host[:B].copy_(toks, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return st.tokens_host[:B].numpy()
        return toks.numpy()

    def execute_speculative(self, plan, spec, edits=None, masks=None):
        """A step whose decoding entries may carry proposed tokens: one packed forward with logits for every row that needs a
        prediction (all 1 + K rows of an entry with K drafts, the last row of any other sampling entry), verification, and
        the per-entry (accepted, next token) pair for EngineCore.commit_speculative.  Synchronous."""
        st = self.staging
        B, T = len(plan.entries), plan.token_count
        rows, row_of = [], []
        any_plain = False
        for e in plan.entries:
            row_of.append(len(rows))
            if not e.samples:
                any_plain = True
                continue
            k = e.request.draft_count if not e.is_prefill else 0
            any_plain = any_plain or k == 0
            rows.extend(range(e.packed_offset + e.num_tokens - 1 - k, e.packed_offset + e.num_tokens))
        with torch.no_grad():
            st.upload()
            s = self._step_inputs(T, B, st.table_cols, plan.max_query_len, plan.max_kv_len)
            dev = self.model.device
            s.logits_rows = torch.tensor(rows or [0], dtype=torch.int32, device=dev)
            nd = 0
            for e in plan.entries:
                if e.num_tokens != 1:
                    break
                nd += 1
            s.num_decode = nd
            logits = self.decoder.forward(s, self.kv)
            if any_plain:
                spec.mirror_prefill(s)         # the draft model's cache follows prompt chunks and plain decode tokens
            if edits or masks is not None:
                ro = torch.tensor(row_of, dtype=torch.int64, device=dev)
                for (r_, t_, o_, v_) in edits or ():
                    ops.logits_edit(logits, ro[r_.long()].to(torch.int32), t_, o_, v_)
                if masks is not None:
                    words, mrows = masks
                    per_row = torch.full((logits.shape[0],), -1, dtype=torch.int32, device=dev)
                    sel = torch.nonzero(mrows >= 0).flatten()
                    per_row[ro[sel]] = mrows[sel]
                    ops.logits_bitmask(logits, words, per_row)
            return spec.verify(plan, logits, row_of)

    def _sample_async(self, logits, B: int):
        st = self.staging
        toks = ops.sample(logits, st.view("top_k", B), st.view("top_p", B, torch.float32), st.view("temperature", B, torch.float32),
                          st.view("seeds", None, torch.int64)[:B], st.view("sample_pos", B))
        buf = st.tokens_ring[st.ring_next % len(st.tokens_ring)]
        st.ring_next += 1
        buf[:B].copy_(toks, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        return ev, B, buf, toks

    def execute_async(self, plan, edits=None, masks=None):
        """Enqueues the step (input copy, model, sampler, copy of the ids to pinned memory) and returns a handle for
        `collect`; the host does not wait."""
        return self.finish_async(plan, self.begin_async(plan), edits, masks)

    def begin_async(self, plan) -> torch.Tensor:
        """First half of execute_async: enqueues the input copy and the model.  The caller may compute logits edits and grammar
        masks on the host while the device runs it, then call finish_async."""
        self.last_key = None
        with torch.no_grad():
            return self.forward(plan)

    def finish_async(self, plan, logits, edits=None, masks=None):
        B = len(plan.entries)
        with torch.no_grad():
            for e in edits or ():
                ops.logits_edit(logits, *e)
            if masks is not None:
                ops.logits_bitmask(logits, *masks)
            return self._sample_async(logits, B)

    def enqueue_next(self, plan, handle):
        """Decode look-ahead: enqueues the step that follows `plan` (a graph step whose ids, `handle`, are still on their
        way) with inputs derived on the device - sampled ids become input ids, positions and cache slots move on by one -
        and returns its handle, or None when that step cannot reuse the captured graph of this one."""
        key = self.last_key
        if key is None or key not in self.graphs or not plan.lookahead_ok or plan.max_kv_len + 1 > key[1] * self.kv.block_size:
            return None
        st = self.staging
        B = len(plan.entries)
        with torch.no_grad():
            table = st.view("block_table").view(st.max_batch, st.table_cols)
            ops.decode_advance(handle[3], st.view("input_ids", B), st.view("positions", B), st.view("past_lens", B),
                               st.view("slot_mapping", B), st.view("sample_pos", B), table[:B], self.kv.block_size)
            graph, logits = self.graphs[key]
            graph.replay()
            return self._sample_async(logits[:B], B)

    def refresh_inputs(self, plan):
        """Copies the packed inputs of a step that was enqueued ahead of time (see Engine._launch_inner)."""
        self.last_key = self.upload_graph_inputs(plan)

    def collect(self, handle) -> np.ndarray:
        ev, B, buf, _ = handle
        ev.synchronize()
        return buf[:B].numpy().copy()   # the pinned buffer is reused by a later step


# ------------------------------------------------------------------------------------------------ engine
class Engine:
    def __init__(self, model: Model, executor=None, num_blocks: Optional[int] = None, lookahead: Optional[bool] = None):
        self.model = model
        cfg = model.config
        eng = cfg.engine.get("dynamic_batching")
        static = False
        if eng is None:
            sb = cfg.engine.get("static_batching")
            static = sb is not None     # fixed batches of up to 4 requests that run to completion, on the paged cache
            eng = {"block_size": 16, "num_blocks": None, "gpu_utilization_factor": None,
                   "max_batch_size": sb["max_batch_size"] if sb else 16, "max_scheduled_tokens": 2048}
        arch = model.arch
        self.block_size = int(eng["block_size"])
        dec = model.decoder
        nb = num_blocks or eng.get("num_blocks")
        if not nb:
            nb = self._blocks_from_memory(eng.get("gpu_utilization_factor") or 0.9)
        o = native.EngineOptions()
        o.block_size, o.num_blocks = self.block_size, int(nb)
        o.max_batch_size, o.max_scheduled_tokens = int(eng["max_batch_size"]), int(eng["max_scheduled_tokens"])
        o.static_batching = static
        o.vocab_size, o.pad_token_id, o.eos_ids = cfg.vocab_size, cfg.pad_token_id, list(cfg.eos_token_ids)
        windowed = arch.sliding_window > 0 and arch.sliding_layers is not None
        if windowed:
            o.window_size = arch.sliding_window
        # Decode look-ahead: with the built-in executor on a GPU, pure decode steps are enqueued one step before their
        # input ids reach the host (OGB_ENGINE_LOOKAHEAD=0 turns it off); the core then also reserves the block of every
        # request's next position so that the device can compute the next cache slots by itself.
        # (`lookahead=True` forces it for an executor that has execute_async / enqueue_next / collect.)
        self.lookahead = (executor is None and model.device.type == "cuda" and not windowed and
                          os.environ.get("OGB_ENGINE_LOOKAHEAD", "1") != "0" and os.environ.get("OGB_ENGINE_RUN_AHEAD", "1") != "0")
        if lookahead is not None:
            self.lookahead = bool(lookahead) and not windowed
        recurrent = model.arch.has_linear_layers
        if recurrent:
            self.lookahead = False        # steps of recurrent models run eagerly, one at a time
        # Speculative decoding (a draft model in the checkpoint, or speculative.ngram_size > 0 in genai_config.json): decoding
        # requests carry proposed tokens that one packed forward of the target verifies for the whole batch (engine/speculative.py).
        # The block look-ahead then reserves room for the proposals instead of serving the enqueue-ahead of plain decode steps.
        spec_cfg = dict(getattr(cfg, "speculative", None) or {})
        want_spec = (executor is None and not windowed and not static and not recurrent and      # (a rejected draft cannot be taken out of a recurrent state)
                     (getattr(model, "draft", None) is not None or int(spec_cfg.get("ngram_size", 0) or 0) > 0) and
                     os.environ.get("OGB_ENGINE_SPECULATIVE", "1") != "0")
        if want_spec:
            self.lookahead = False
            o.lookahead = max(1, min(16, int(spec_cfg.get("max_draft_tokens", 4)))) + 1
            o.lookahead_execution = False
        else:
            o.lookahead = 1 if self.lookahead else 0
        self.core = native.EngineCore(o)
        self.options = o
        n_win = self.core.ring_blocks_per_request * o.max_batch_size if windowed else 0
        self.kv = PagedKVCache(arch, o.num_blocks, self.block_size, model.device, model.dtype, kv_heads=dec.kv_heads_local,
                               num_window_blocks=n_win, conv_channels=dec.conv_channels_local, kv_bits=getattr(model, "kv_bits", 16))
        max_ctx = min(cfg.context_length, o.num_blocks * self.block_size)
        cols = (max_ctx + self.block_size - 1) // self.block_size
        self.staging = _Staging(o.max_scheduled_tokens + o.max_batch_size, o.max_batch_size, cols, model.device, windowed)
        self.executor = executor or ModelExecutor(model, self.core, self.staging, self.kv, use_graphs=True)
        self.spec = None
        if want_spec:
            from .speculative import EngineSpeculator
            self.spec = EngineSpeculator(self, spec_cfg)
        # Requests are held weakly: when the caller drops its last reference to a submitted request, the request is abandoned and
        # reclaimed at the next add_request / step boundary (reference: src/engine/engine.cpp:107-136)
        self._by_native: "weakref.WeakValueDictionary[int, Request]" = weakref.WeakValueDictionary()
        self._natives: Dict[int, Any] = {}
        self._abandoned: List[int] = []
        self.reclaimed = 0               # abandoned requests reclaimed so far
        self._adapter_requests = 0       # requests with a LoRA adapter: their steps run eagerly (no graphs, no look-ahead)
        if hasattr(self.executor, "lora_of"):
            self.executor.lora_of = self._lora_of
        self._state_slot: Dict[int, int] = {}      # request id -> slot of the recurrent-state pool (linear-attention models)
        self._free_slots: List[int] = []
        if model.arch.has_linear_layers and hasattr(self.executor, "state_slots_of"):
            self.kv.ensure_state_slots(o.max_batch_size)
            self._free_slots = list(range(o.max_batch_size - 1, -1, -1))
            self.executor.state_slots_of = self._state_slots_of
        self._guidance: Dict[int, Any] = {}
        self.last_outcome = StepOutcome.NoWork
        self.step_count = 0
        self._with_processors = set()   # ids of requests with min_length / repetition penalty / no-repeat-ngram
        self._need_first = set()        # ids of requests that have not produced a token yet (time to first token)
        self._inflight = None
        self._ahead = None              # (signature of the plan it belongs to, handle) of a step enqueued ahead of time
        self.lookahead_hits = 0
        # one step ahead of the caller: only with the built-in executor on a GPU (OGB_ENGINE_RUN_AHEAD=0 turns it off)
        # host time spent planning / packing / enqueueing steps, and time spent waiting for the device to finish one
        self.host_stats = {"launch_s": 0.0, "wait_s": 0.0, "launches": 0}
        self.run_ahead = (executor is None and model.device.type == "cuda" and os.environ.get("OGB_ENGINE_RUN_AHEAD", "1") != "0") or self.lookahead

    def _blocks_from_memory(self, utilization: float) -> int:
        arch, dec = self.model.arch, self.model.decoder
        per_block = PagedKVCache.bytes_per_block(arch, self.block_size, self.model.dtype, dec.kv_heads_local, dec.conv_channels_local,
                                                 getattr(self.model, "kv_bits", 16))
        if self.model.device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(self.model.device)
            budget = int(free * 0.9 * utilization)
        else:
            budget = 256 << 20
        return max(16, budget // per_block)

    # ------------------------------------------------------------------ API
    def _reclaim_abandoned(self):
        """Requests whose last external reference is gone: removed from the scheduler, their blocks freed."""
        while self._abandoned:
            rid = self._abandoned.pop()
            nat = self._natives.pop(rid, None)
            if nat is None:
                continue            # removed explicitly before it was dropped
            if self._inflight is not None and any(e.request.id == rid for e in self._inflight[0].entries):
                self._drain()
            self.core.remove_request(nat)
            self._release_state_slot(rid)
            self._guidance.pop(rid, None)
            self._with_processors.discard(rid)
            self._need_first.discard(rid)
            if self.spec is not None:
                self.spec.forget(rid)
            self.reclaimed += 1
        self._adapter_requests = sum(1 for r in self._by_native.values() if r._adapter is not None)

    def add_request(self, request: Request):
        self._reclaim_abandoned()
        if request._native is not None:
            raise RuntimeError("add_request: request was already added to an engine")
        nat = self.core.create_request(request._options())
        nat.add_tokens(np.asarray(request._pending_tokens, dtype=np.int32))
        self.core.add_request(nat)
        request._native, request._engine = nat, self
        request.t_added = time.perf_counter()
        self._by_native[nat.id] = request
        self._natives[nat.id] = nat
        weakref.finalize(request, self._abandoned.append, nat.id)
        self._adapter_requests = sum(1 for r in self._by_native.values() if r._adapter is not None)
        self._need_first.add(nat.id)
        so = request.params.search
        if so.get("min_length", 0) > 0 or so.get("repetition_penalty", 1.0) != 1.0 or so.get("no_repeat_ngram_size", 0) > 0:
            self._with_processors.add(nat.id)
        if request.params.guidance_type:
            from ..guidance import GuidanceProcessor
            self._guidance[nat.id] = GuidanceProcessor(self.model, request.params.guidance_type, request.params.guidance_data, 1, False)
            self._guidance[nat.id].commit_prompt(np.asarray(request._pending_tokens, dtype=np.int32).reshape(1, -1))

    def _state_slots_of(self, plan, host: bool = False):
        """Slot of every request of the step in the recurrent-state pool; a request gets one when it first runs (its state starts
        from zero because its past length is 0 then) and gives it back when it leaves the engine."""
        out = np.empty(len(plan.entries), dtype=np.int32)
        for i, e in enumerate(plan.entries):
            rid = e.request.id
            slot = self._state_slot.get(rid)
            if slot is None:
                if not self._free_slots:
                    n = self.kv.state_slots
                    self.kv.ensure_state_slots(2 * n)
                    self._free_slots = list(range(2 * n - 1, n - 1, -1))
                    if hasattr(self.executor, "graphs"):
                        self.executor.graphs.clear()      # captured steps hold the address of the old pool
                slot = self._free_slots.pop()
                self._state_slot[rid] = slot
            out[i] = slot
        return out if host else torch.from_numpy(out).to(self.model.device)

    def _release_state_slot(self, rid: int) -> None:
        slot = self._state_slot.pop(rid, None)
        if slot is not None:
            self._free_slots.append(slot)

    def _lora_of(self, plan):
        """(per-token adapter index on the device, names of the adapters present) for a step that holds at least one request with
        an adapter, else None.  Tokens of requests without an adapter carry the index len(names)."""
        if not self._adapter_requests:
            return None
        names: List[str] = []
        per_entry = []
        for e in plan.entries:
            rq = self._by_native.get(e.request.id)
            name = rq._adapter if rq is not None else None
            if name is not None and name not in names:
                names.append(name)
            per_entry.append(name)
        if not names:
            return None
        ids = np.empty(plan.token_count, dtype=np.int32)
        for e, name in zip(plan.entries, per_entry):
            ids[e.packed_offset:e.packed_offset + e.num_tokens] = names.index(name) if name is not None else len(names)
        return torch.from_numpy(ids).to(self.model.device), tuple(names)

    def remove_request(self, request: Request):
        if request._native is None:
            return
        if self._inflight is not None and any(e.request.id == request._native.id for e in self._inflight[0].entries):
            self._drain()     # the request is part of the step in flight: let that step commit first
        self.core.remove_request(request._native)
        self._by_native.pop(request._native.id, None)
        self._natives.pop(request._native.id, None)
        self._release_state_slot(request._native.id)
        self._adapter_requests = sum(1 for r in self._by_native.values() if r._adapter is not None)
        self._guidance.pop(request._native.id, None)
        self._with_processors.discard(request._native.id)
        self._need_first.discard(request._native.id)
        if self.spec is not None:
            self.spec.forget(request._native.id)

    def has_pending_requests(self) -> bool:
        return self.core.has_pending_requests()

    def step(self) -> Optional[Request]:
        """Returns one request that has unseen tokens (or just finished its turn), running the model when
        no such request is waiting; returns None when there is nothing to do.

        On CUDA the engine runs one step ahead: as soon as the ids of a step are committed the next step is planned,
        packed and enqueued, and only then are the ready requests handed out, so the GPU computes step n + 1 while the
        caller consumes the tokens of step n."""
        if self._abandoned:
            self._reclaim_abandoned()
        nat = self.core.next_ready()
        if nat is None:
            self._advance()
            nat = self.core.next_ready()
        return self._by_native.get(nat.id) if nat is not None else None

    # ------------------------------------------------------------------ internals
    def _advance(self):
        if self._inflight is None:
            self._launch()
        if self._inflight is not None:
            self._finish()
            if self.run_ahead and self.last_outcome == StepOutcome.Committed:
                self._launch()

    def _drain(self):
        """Completes the step in flight, if any (before the set of requests changes under it)."""
        if self._inflight is not None:
            self._finish()

    def _run_model_step(self):
        """One synchronous step: plan, execute, commit."""
        self._drain()
        self._launch()
        if self._inflight is not None:
            self._finish()

    def _fail(self, e: Exception):
        self._ahead = None      # a step enqueued ahead of the failed one is never used
        if isinstance(e, ExecutionFailure):
            outcome = self.core.abort(e.kind, str(e))
            self.last_outcome = outcome
            if outcome in (StepOutcome.FatalExecutionFailure, StepOutcome.ExecutionContractFailure):
                raise EngineStepError(outcome, str(e)) from e
            return
        if isinstance(e, torch.cuda.OutOfMemoryError):
            self.last_outcome = self.core.abort(FailureKind.CapacityExceeded, str(e))
            return
        kind = FailureKind.CapacityExceeded if "out of memory" in str(e).lower() else FailureKind.Fatal
        self.last_outcome = self.core.abort(kind, str(e))
        if kind == FailureKind.Fatal:
            raise EngineStepError(self.last_outcome, str(e)) from e

    def _launch(self):
        """Plans and packs a step and hands it to the executor; leaves it in `_inflight` (with its ids already there
        when the executor is synchronous)."""
        t0 = time.perf_counter()
        try:
            self._launch_inner()
        finally:
            self.host_stats["launch_s"] += time.perf_counter() - t0
            self.host_stats["launches"] += 1

    def _launch_inner(self):
        with _Trace("engine", "launch"):
            if self.spec is not None:
                try:
                    self.spec.propose()
                except Exception as e:      # proposing touches no engine state: a failure here is a failed step without a plan
                    raise EngineStepError(StepOutcome.FatalExecutionFailure, f"speculative proposal failed: {e}") from e
            plan = self.core.plan()
            self.last_outcome = plan.outcome
            if plan.unserviceable:
                for nat in plan.unserviceable:
                    self._by_native.pop(nat.id, None)
                    self._natives.pop(nat.id, None)
                if plan.outcome != StepOutcome.Planned:
                    raise EngineStepError(StepOutcome.UnserviceableRequest, "a request needs more KV-cache blocks than the engine owns")
            if plan.outcome != StepOutcome.Planned:
                return
            st = self.staging
            ahead, self._ahead = self._ahead, None
            plain = not self._with_processors and not self._guidance and not self._adapter_requests
            try:
                st.flip()
                if ahead is not None and plain and ahead[0] == plan.signature:
                    # This very step is already running: it was enqueued while the previous one was in flight.  Its packed
                    # inputs are copied to the device all the same (behind the running kernels, which read identical values):
                    # they carry the block-table columns that the step after this one needs.
                    handle = ahead[1]
                    self.lookahead_hits += 1
                    self._inflight = (plan, handle, None)
                    self.core.pack(st.addr, st.max_tokens, st.max_batch, st.table_cols)
                    self.executor.refresh_inputs(plan)
                elif self.spec is not None:
                    self.core.pack(st.addr, st.max_tokens, st.max_batch, st.table_cols)
                    edits, masks = self._logits_processors(plan)
                    self._inflight = (plan, None, self.executor.execute_speculative(plan, self.spec, edits, masks))
                    return
                else:
                    self.core.pack(st.addr, st.max_tokens, st.max_batch, st.table_cols)
                    if self.run_ahead and hasattr(self.executor, "begin_async"):
                        # the model is enqueued first: penalties and grammar masks (host work: llguidance walks the grammar for
                        # every constrained request) are computed while the device runs the forward pass
                        logits = self.executor.begin_async(plan)
                        edits, masks = self._logits_processors(plan)
                        handle = self.executor.finish_async(plan, logits, edits, masks)
                        self._inflight = (plan, handle, None)
                    elif self.run_ahead:
                        edits, masks = self._logits_processors(plan)
                        handle = self.executor.execute_async(plan, edits, masks)
                        self._inflight = (plan, handle, None)
                    else:
                        edits, masks = self._logits_processors(plan)
                        self._inflight = (plan, None, self.executor.execute(plan, edits, masks))
                if self.lookahead and plain and plan.lookahead_ok:
                    nxt = self.executor.enqueue_next(plan, handle)
                    if nxt is not None:
                        self._ahead = (plan.next_signature, nxt)
            except Exception as e:
                self._ahead = None
                self._fail(e)

    def _finish(self):
        with _Trace("engine", "finish"):
            plan, handle, toks = self._inflight
            self._inflight = None
            accepted = None
            if isinstance(toks, tuple):       # a speculative step: (accepted drafts per entry, token after them)
                accepted, toks = toks
            if handle is not None:
                t0 = time.perf_counter()
                try:
                    toks = self.executor.collect(handle)
                except Exception as e:
                    self._fail(e)
                    return
                finally:
                    self.host_stats["wait_s"] += time.perf_counter() - t0
            now = time.perf_counter()
            if self._need_first or self._guidance:      # steady-state decode has neither: no per-entry work on the host
                for i, e in enumerate(plan.entries):
                    if not e.samples:
                        continue
                    rid = e.request.id
                    if rid in self._need_first:
                        self._need_first.discard(rid)
                        rq = self._by_native.get(rid)
                        if rq is not None:
                            rq.t_first = now
                    gp = self._guidance.get(rid)
                    if gp is not None:
                        committed = [int(toks[i])]
                        if accepted is not None and int(accepted[i]) > 0:
                            # the accepted drafts still sit at the tail of the request's tokens (the commit below trims the rest)
                            k = e.request.draft_count
                            all_toks = e.request.tokens()
                            committed = [int(t) for t in all_toks[len(all_toks) - k: len(all_toks) - k + int(accepted[i])]] + committed
                        for t in committed:           # (commit_tokens takes one token per batch row)
                            gp.commit_tokens(np.asarray([t], dtype=np.int32))
            self.t_last_step = now
            if accepted is not None:
                self.last_outcome = self.core.commit_speculative(np.ascontiguousarray(accepted, dtype=np.int32),
                                                                 np.ascontiguousarray(toks, dtype=np.int32))
            else:
                self.last_outcome = self.core.commit(np.ascontiguousarray(toks, dtype=np.int32))
            self.step_count += 1

    def _logits_processors(self, plan):
        """Sparse logits edits (min_length, repetition penalty, no-repeat-ngram) and grammar masks."""
        if not self._with_processors and not self._guidance:
            return [], None        # no admitted request edits its logits: nothing to look at per entry
        rows, toks, opsl, vals = [], [], [], []
        mask_rows, mask_list = [], []
        V = self.model.config.vocab_size
        eos = list(self.model.config.eos_token_ids)
        any_mask = False
        for i, e in enumerate(plan.entries):
            if not e.samples:
                mask_rows.append(-1)
                continue
            o = e.request.options
            seq = None
            if o.min_length > 0 and e.request.num_tokens < o.min_length:
                for t in eos:
                    rows.append(i); toks.append(t); opsl.append(0); vals.append(0.0)
            if o.repetition_penalty != 1.0:
                seq = e.request.tokens()
                for t in np.unique(seq).tolist():
                    rows.append(i); toks.append(t); opsl.append(1); vals.append(float(o.repetition_penalty))
            if o.no_repeat_ngram_size > 0:
                seq = e.request.tokens() if seq is None else seq
                for t in native.no_repeat_ngram_banned(seq, o.no_repeat_ngram_size, V):
                    rows.append(i); toks.append(t); opsl.append(0); vals.append(0.0)
            gp = self._guidance.get(e.request.id)
            if gp is not None:
                mask_rows.append(len(mask_list))
                mask_list.append(gp)
                any_mask = True
            else:
                mask_rows.append(-1)
        dev = self.model.device
        edits = []
        for want in (1, 0):  # penalties before bans
            sel = [j for j, o_ in enumerate(opsl) if o_ == want]
            if sel:
                g = lambda x, dt: torch.tensor([x[j] for j in sel], dtype=dt, device=dev)
                edits.append((g(rows, torch.int32), g(toks, torch.int32), g(opsl, torch.int32), g(vals, torch.float32)))
        masks = None
        if any_mask:
            masks = (torch.from_numpy(self._grammar_masks(mask_list)).to(dev), torch.tensor(mask_rows, dtype=torch.int32, device=dev))
        return edits, masks

    def _grammar_masks(self, procs) -> np.ndarray:
        """One bitmask row per constrained request of the step.  The grammar walks of the requests are independent: llguidance's
        thread pool fills all rows at once (the step's host time is the slowest request's mask, not their sum), while the
        device runs the forward pass of the same step."""
        words = procs[0].words
        out = np.empty((len(procs), words), dtype=np.int32)
        live = [(gp.matchers[0], i) for i, gp in enumerate(procs) if not gp.matchers[0].is_stopped()]
        if len(live) > 1:
            import llguidance
            import llguidance.numpy as llnp
            if getattr(self, "_ll_exec", None) is None:
                self._ll_exec = llguidance.LLExecutor(num_threads=min(16, max(2, (os.cpu_count() or 4) // 2)))
            llnp.fill_next_token_bitmask_par(self._ll_exec, live, out)
            done = {i for _, i in live}
            for m, i in live:
                if m.is_error():
                    raise RuntimeError("grammar matcher error: " + m.get_error())
        else:
            done = set()
        for i, gp in enumerate(procs):
            if i not in done:
                out[i] = gp.compute_mask()[0]      # a single live request, or a finished grammar (only end-of-sequence may follow)
        return out

    @property
    def metrics(self) -> Dict[str, int]:
        return dict(self.core.metrics)
