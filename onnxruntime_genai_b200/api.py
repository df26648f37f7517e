"""Public Python API: Config, Model, GeneratorParams, Generator, Tensor, NamedTensors.

Surface and behaviour follow the reference binding (src/python/python.cpp:444-835) and the
Generator it wraps (src/generators.cpp:564-1008): `append_tokens` runs the prompt (prefill, chunked
by `search.chunk_size`), `generate_next_token` runs one decode step when the logits are stale, then
applies guidance mask -> min_length -> repetition penalty -> no-repeat-ngram -> greedy / top-k /
top-p / beam selection (src/standard_decoding_strategy.cpp:12-62); `rewind_to` drops tokens and their
KV entries; `get_logits` / `set_logits` expose the fp32 scores of the next position.

Differences by design: the model math runs in this process as PyTorch modules over sm_100a kernels
(no ONNX Runtime session); the static-batch Generator uses the same paged KV cache and packed
variable-length forward as the continuous-batching Engine, with one contiguous run of blocks per
batch row, so padded prompts are handled by simply not feeding the pad tokens.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from . import ops, telemetry
from .models.decoder import PagedKVCache, StepInputs
from .native_loader import native

_cuda_device_id = 0


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


def set_current_gpu_device_id(i: int) -> None:
    global _cuda_device_id
    _cuda_device_id = int(i)
    if torch.cuda.is_available():
        torch.cuda.set_device(_cuda_device_id)


def get_current_gpu_device_id() -> int:
    return _cuda_device_id


def set_log_options(**kw) -> None:
    for k, v in kw.items():
        if isinstance(v, bool):
            native.log_set_bool(k, v)
        else:
            native.log_set_string(k, str(v))


def set_log_callback(fn) -> None:
    native.log_set_callback(fn)


class _Trace:
    """RAII-style scope that writes a Chrome trace event when tracing is enabled and, with OGB_NVTX=1, an NVTX range of the
    same name (so the scopes line up with the kernels in a CUDA profiler's timeline)."""
    nvtx = os.environ.get("OGB_NVTX", "0") == "1"

    def __init__(self, cat: str, name: str):
        self.cat, self.name = cat, name
        self._pushed = False

    def __enter__(self):
        self.t0 = native.trace_now_us() if native.trace_enabled() else -1
        if _Trace.nvtx and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(f"{self.cat}:{self.name}")
            self._pushed = True
        return self

    def __exit__(self, *exc):
        if self._pushed:
            torch.cuda.nvtx.range_pop()
        if self.t0 >= 0:
            native.trace_complete(self.cat, self.name, self.t0, native.trace_now_us() - self.t0)
        return False


# ------------------------------------------------------------------------------------------------ Config
class Config:
    def __init__(self, path: str, overlay: str = "", provider: Optional[str] = None):
        """path: a model directory (genai_config.json + graph) or a model package (manifest.json + one directory per
        build variant); for a package the variant matching `provider` ("cuda" / "cpu"; default: what this machine has) is
        loaded."""
        from . import model_package
        self._package_root, self._manifest = None, None
        path = str(path)
        if model_package.is_package(path):
            self._package_root = path
            path, self._manifest = model_package.resolve_package(path, provider)
        self._c = native.Config(path, overlay)
        self._model_data: Dict[str, bytes] = {}

    @property
    def tokenizer_path(self) -> str:
        """Directory of the tokenizer files: the model directory, a relative `model.tokenizer_dir` under it, or a shared
        asset of the package (`sha256:<hex>[/tail]`)."""
        from . import model_package
        return model_package.resolve_asset(self._c.config_path, self._c.tokenizer_dir, self._package_root, self._manifest)

    def __getattr__(self, name):
        return getattr(self._c, name)

    def append_provider(self, name: str):
        self._c.append_provider(name)

    def set_provider_option(self, provider: str, key: str, value: str):
        self._c.set_provider_option(provider, key, value)

    def clear_providers(self):
        self._c.clear_providers()

    def overlay(self, json_text: str):
        self._c.overlay(json_text)

    def add_model_data(self, filename: str, data: bytes):
        self._model_data[filename] = bytes(data)

    def remove_model_data(self, filename: str):
        self._model_data.pop(filename, None)


# ------------------------------------------------------------------------------------------------ Tensor
class Tensor:
    """A named-less n-d array handed to / returned from the runtime (wraps numpy or torch)."""

    def __init__(self, array):
        self._t = array if isinstance(array, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(array))

    def shape(self):
        return list(self._t.shape)

    def type(self):
        return str(self._t.dtype)

    def as_numpy(self):
        return self._t.detach().float().cpu().numpy() if self._t.dtype == torch.bfloat16 else self._t.detach().cpu().numpy()

    def torch(self):
        return self._t


class NamedTensors(dict):
    pass


# ------------------------------------------------------------------------------------------------ Model
class Model:
    def __init__(self, config_or_path, tp=None):
        self.config = config_or_path if isinstance(config_or_path, Config) else Config(str(config_or_path))
        c = self.config
        provs = [p for p, _ in c.decoder["provider_options"]]
        want_cuda = "cuda" in provs
        if want_cuda and not torch.cuda.is_available():
            raise RuntimeError("the model config selects the cuda provider but no CUDA device is available "
                               "(use Config.clear_providers() to run the CPU path)")
        self.device_type = "cuda" if want_cuda else "cpu"
        self.device = torch.device("cuda", torch.cuda.current_device()) if want_cuda else torch.device("cpu")
        self.type = c.model_type
        from .models.arch import ALM_TYPES, LLM_TYPES, VLM_TYPES
        from .models import marian, transducer
        if self.type not in LLM_TYPES + VLM_TYPES + ALM_TYPES + [marian.MODEL_TYPE] + list(transducer.MODEL_TYPES):
            raise RuntimeError(f"Unsupported model type: {self.type}")
        self.dtype = torch.bfloat16 if want_cuda else torch.float32
        from .models.loader import load_decoder
        t_load = time.perf_counter()
        with _Trace("model", "load"):
            if self.type == marian.MODEL_TYPE:
                # encoder-decoder translation model with a recurrent (SSRU) decoder: its own weights, forward passes and state
                if tp is not None and getattr(tp, "size", 1) > 1:
                    raise RuntimeError("marian-ssru models run on one GPU")
                self.decoder, self.draft = marian.MarianModel.load(c.config_path, c, self.device, self.dtype), None
            elif self.type in transducer.MODEL_TYPES:
                # speech transducer (RNN-T / TDT): acoustic encoder + prediction network + joiner and their frame-synchronous search
                self.decoder, self.draft = transducer.TransducerModel.load(c.config_path, c, self.device, self.dtype), None
            else:
                self.decoder = load_decoder(c.config_path, c, self.device, self.dtype, tp)
                self.draft = load_decoder(c.config_path, c, self.device, self.dtype, tp, decoder=c.draft) if c.draft else None
        if telemetry.enabled():
            a = self.decoder.arch
            telemetry.log_event("ModelLoad", {"model_type": self.type, "device": self.device_type, "layers": a.num_layers,
                                              "hidden_size": a.hidden_size, "vocab_size": a.vocab_size, "dtype": str(self.dtype).replace("torch.", ""),
                                              "load_ms": round((time.perf_counter() - t_load) * 1e3, 1),
                                              "model_dir_hash": telemetry.redact_path(c.config_path)})
        # Multimodal components (reference: src/models/multi_modal.cpp:104-160, src/models/whisper.cpp:19-60): the audio or
        # vision encoder named by the config's `encoder` / `vision` section.
        tree = json.loads(c.to_json()).get("model", {})
        self.multimodal: Dict[str, Any] = {}
        self.encoder = self.vision = None
        if self.type in ALM_TYPES or self.type in VLM_TYPES:
            from .models.encoder import TransformerEncoder
            if self.type in ALM_TYPES:
                sec = tree.get("encoder") or {}
                self.encoder = TransformerEncoder.load(os.path.join(c.config_path, sec.get("filename", "encoder.onnx")), self.device, self.dtype)
                self.multimodal["audio"] = sec
                self.multimodal["speech"] = tree.get("speech") or {}
            if tree.get("vision"):
                sec = tree["vision"]
                self.vision = TransformerEncoder.load(os.path.join(c.config_path, sec["filename"]), self.device, self.dtype)
                self.multimodal["vision"] = sec
                self.image_token_id = int(tree.get("image_token_id", -1))
        from .models import qwen_vl
        if self.type in qwen_vl.QWEN_VL_TYPES and tree.get("vision"):
            # Qwen2-VL: patches + (t, h, w) grids in, merged image features out; the decoder takes three position components per token
            sec = tree["vision"]
            self.vision = qwen_vl.QwenVisionTower.load(os.path.join(c.config_path, sec["filename"]), self.device, self.dtype)
            self.multimodal["vision"] = sec
            self.image_token_id = int(tree.get("image_token_id", -1))
        self.arch = self.decoder.arch
        # KV-cache quantisation is a provider option of the decoder session (reference: src/config_utils.cpp:13-45)
        self.kv_bits = 16
        for _, opts in c.decoder["provider_options"]:
            bits = str(dict(opts).get("kvCacheQuantizationBits", "0"))
            if bits not in ("0", "8"):
                raise RuntimeError(f"kvCacheQuantizationBits={bits} is not supported (0 or 8)")
            if bits == "8":
                self.kv_bits = 8
        self.graph_capture = bool(c.decoder.get("graph_capture", False))
        if self.draft is not None and self.draft.arch.vocab_size != self.arch.vocab_size:
            raise RuntimeError("speculative decoding: draft and target vocabularies differ")

    def create_multimodal_processor(self):
        if not self.multimodal:
            raise RuntimeError("this model has no vision or speech component")
        from .multimodal import MultiModalProcessor
        return MultiModalProcessor(self)

    def create_streaming_processor(self):
        """Streaming front end of a speech transducer: samples in, log-mel frames out, long silences dropped when the model has a
        `vad` section (reference: src/models/streaming_processor.cpp, nemotron_streaming_processor.cpp)."""
        from .models.transducer import TransducerModel
        if not isinstance(self.decoder, TransducerModel):
            raise RuntimeError("this model has no streaming audio component")
        from .streaming import StreamingProcessor
        return StreamingProcessor(self)

    def create_streaming_session(self):
        """`feed(samples)` -> tokens emitted so far, `finish()` -> the rest (speech transducers)."""
        from .streaming import StreamingSession
        return StreamingSession(self)


# ------------------------------------------------------------------------------------------------ params
_SEARCH_BOOLS = {"do_sample", "past_present_share_buffer", "early_stopping"}


class GeneratorParams:
    def __init__(self, model: Model):
        self.model = model
        self.search: Dict[str, Any] = dict(model.config.search)
        self.speculative: Dict[str, Any] = dict(model.config.speculative)
        self.guidance_type: Optional[str] = None
        self.guidance_data: Optional[str] = None
        self.guidance_ff_tokens = False

    def set_search_options(self, **kw):
        for k, v in kw.items():
            if k in _SEARCH_BOOLS:
                v = bool(v)
            native.validate_search_option(k, v)  # throws on unknown names / non-integers
            self.search[k] = v

    def get_search_options(self) -> Dict[str, Any]:
        return dict(self.search)

    def set_speculative_options(self, **kw):
        for k, v in kw.items():
            native.validate_speculative_option(k, v)
            self.speculative[k] = v

    def get_speculative_options(self) -> Dict[str, Any]:
        return dict(self.speculative)

    def set_guidance(self, type: str, data: str, enable_ff_tokens: bool = False):
        if type not in ("json_schema", "regex", "lark_grammar"):
            raise RuntimeError(f"Unsupported guidance type: {type} (json_schema, regex, lark_grammar)")
        self.guidance_type, self.guidance_data, self.guidance_ff_tokens = type, data, bool(enable_ff_tokens)


def _sampling_method(search: Dict[str, Any], vocab: int):
    """(method, k, p, t) following src/generators.cpp:661-682."""
    do_sample, k, p, t = search["do_sample"], int(search["top_k"]), float(search["top_p"]), float(search["temperature"])
    if not do_sample or k == 1 or t == 0:
        return "greedy", 1, 0.0, 1.0
    if search["num_beams"] > 1:
        raise RuntimeError("sampling (do_sample=True) is not supported with beam search")
    if not (0.0 <= p <= 1.0):
        raise RuntimeError("top_p must be between 0.0 and 1.0")
    if k < 0 or k > vocab:
        raise RuntimeError("top_k must be between 0 and vocab_size")
    if 0.0 < p < 1.0 and k > 1:
        return "top_k_top_p", k, p, t
    if k > 1:
        return "top_k", k, 1.0, t
    return "top_p", 0, p if p > 0 else 1.0, t


# ------------------------------------------------------------------------------------------------ Generator
class SequenceState:
    """Device state of a static batch: paged KV with one contiguous run of blocks per row."""

    def __init__(self, decoder, rows: int, max_length: int, block_size: int = 16, kv_bits: int = 16):
        self.decoder = decoder
        self.rows = rows
        self.block_size = block_size
        self.blocks_per_row = (max_length + block_size - 1) // block_size
        dev = decoder.device
        self.kv = PagedKVCache(decoder.arch, rows * self.blocks_per_row, block_size, dev, decoder.dtype,
                               kv_heads=decoder.kv_heads_local, conv_channels=decoder.conv_channels_local, kv_bits=kv_bits)
        self.block_table = (torch.arange(rows * self.blocks_per_row, dtype=torch.int32).view(rows, self.blocks_per_row)).to(dev)
        self.kv.ensure_state_slots(rows)             # linear-attention layers: row r keeps its recurrent state in slot r
        self.kv_len = [0] * rows
        # Beam search shares cache blocks between rows (copy-on-write at block granularity).  Until the first reorder every
        # row owns one contiguous run of blocks and none of this is active (`_tbl` is None).
        self._tbl: Optional[np.ndarray] = None     # host mirror of the block table once rows share blocks
        self._ref: Optional[np.ndarray] = None     # references per physical block
        self._free: List[int] = []
        self._moves: List[tuple] = []              # (src block, dst block) copies to do before the next forward
        self._tbl_dirty = False
        self.rope_delta = [0] * rows                 # multimodal RoPE: offset of a row's rotary position from its cache position
        self.cross = None                            # encoder keys / values of an encoder-decoder model (set_cross)
        self.cross_table = self.cross_lens = None
        self.max_cross_len = 0

    def set_cross(self, enc_out: torch.Tensor, enc_lens: List[int], rows_per_item: int):
        """Projects the encoder output of each batch item into the decoder layers' cross-attention keys / values once;
        the item's rows (beams) all point at the same blocks."""
        from .models.decoder import CrossKVCache
        dec, dev, bs = self.decoder, self.decoder.device, self.block_size
        if len(enc_lens) * rows_per_item != self.rows:
            raise RuntimeError(f"encoder inputs for {len(enc_lens)} items do not match the batch ({self.rows // rows_per_item})")
        nblk = [(n + bs - 1) // bs for n in enc_lens]
        self.cross = CrossKVCache(dec.arch, sum(nblk), bs, dev, dec.dtype, dec.heads_local)
        table = torch.full((self.rows, max(nblk)), -1, dtype=torch.int32)
        slots, b0 = [], 0
        for i, n in enumerate(enc_lens):
            table[i * rows_per_item:(i + 1) * rows_per_item, :nblk[i]] = torch.arange(b0, b0 + nblk[i], dtype=torch.int32)
            slots.append(torch.arange(n, dtype=torch.int32) + b0 * bs)
            b0 += nblk[i]
        with torch.no_grad():
            dec.fill_cross_cache(self.cross, enc_out, torch.cat(slots).to(dev))
        self.cross_table = table.to(dev)
        self.cross_lens = torch.tensor([n for n in enc_lens for _ in range(rows_per_item)], dtype=torch.int32, device=dev)
        self.max_cross_len = max(enc_lens)
        self._graphs = {}     # captured steps hold the previous cross cache

    def _cross_fields(self, rows_used=None) -> dict:
        if self.cross is None:
            return {}
        sel = rows_used is not None and len(rows_used) != self.rows
        return dict(cross=self.cross, cross_table=self.cross_table[rows_used].contiguous() if sel else self.cross_table,
                    cross_lens=self.cross_lens[rows_used].contiguous() if sel else self.cross_lens, max_cross_len=self.max_cross_len)

    def run(self, row_tokens: List[List[int]], want_all_logits: bool = False, inputs_embeds=None, positions3=None,
            device_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Feeds row_tokens[r] (possibly empty) after the cached prefix of row r; returns fp32 logits of the last
        fed token of every non-empty row (or of every token).  positions3[r]: [3, len(row_tokens[r])] rotary position
        components of the fed tokens (multimodal RoPE); later tokens continue one past the largest component.
        device_ids: int32 device tensor with the ids of all fed tokens in row order - the values in row_tokens are then only
        counted, so a token chosen on the device (a draft model's argmax) is fed without a round trip through the host."""
        dev = self.decoder.device
        mrope = self.decoder.arch.mrope_section is not None and (positions3 is not None or any(self.rope_delta))
        p3: List[np.ndarray] = []
        ids, pos, slots, cu, past, rows_used, last = [], [], [], [0], [], [], []
        for r, toks in enumerate(row_tokens):
            if not toks:
                continue
            base = self.kv_len[r]
            if base + len(toks) > self.blocks_per_row * self.block_size:
                raise RuntimeError("sequence exceeds the allocated KV cache (max_length)")
            if self._tbl is not None:
                self._own_blocks(r, base, len(toks))
            for j, t in enumerate(toks):
                p = base + j
                ids.append(t)
                pos.append(p)
                slots.append(self._slot(r, p))
            if mrope:
                if positions3 is not None and positions3[r] is not None:
                    comp = np.asarray(positions3[r], dtype=np.int32).reshape(3, len(toks))
                    self.rope_delta[r] = int(comp.max()) + 1 - (base + len(toks))
                else:
                    comp = np.tile(np.arange(base, base + len(toks), dtype=np.int32) + self.rope_delta[r], (3, 1))
                p3.append(comp)
            cu.append(len(ids))
            past.append(base)
            rows_used.append(r)
            last.append(len(ids) - 1)
            self.kv_len[r] = base + len(toks)
        self._flush_block_moves()
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        if device_ids is not None and (device_ids.dtype != torch.int32 or device_ids.numel() != len(ids) or device_ids.device != dev):
            raise RuntimeError("device_ids must be an int32 tensor on the model's device with one id per fed token")
        s = StepInputs(input_ids=device_ids.reshape(-1) if device_ids is not None else i32(ids), positions=i32(pos), slot_mapping=i32(slots),
                       cu_seqlens=i32(cu), past_lens=i32(past),
                       block_table=self.block_table[rows_used].contiguous() if len(rows_used) != self.rows else self.block_table,
                       logits_rows=None if want_all_logits else i32(last),
                       max_q_len=max(len(t) for t in row_tokens if t), max_kv_len=max(self.kv_len), inputs_embeds=inputs_embeds,
                       min_q_len=min(len(t) for t in row_tokens if t),
                       state_slots=i32(rows_used) if self.decoder.arch.has_linear_layers else None,
                       **self._cross_fields(rows_used))
        if mrope:
            s.positions3 = torch.from_numpy(np.ascontiguousarray(np.concatenate(p3, axis=1))).to(dev)
        heads = getattr(self, "alignment_heads", None)
        if heads and self.cross is not None:
            s.cross_qk_heads, s.cross_qk_out = heads, [None] * len(heads)
        out = self.decoder.forward(s, self.kv)
        if s.cross_qk_out:
            # per row: one [heads, frames] slab per token fed so far (prompt tokens included)
            qk = torch.stack(s.cross_qk_out, dim=1).cpu()                           # [tokens, heads, frames]
            for j, r in enumerate(rows_used):
                self.cross_qk_rows[r].extend(qk[cu[j]:cu[j + 1]])
        return out, rows_used

    def set_alignment_heads(self, heads) -> None:
        """heads: [(layer, head)] whose cross-attention scores are recorded from now on (`Generator.get_output("cross_qk")`)."""
        self.alignment_heads = [(int(l), int(h)) for l, h in heads]
        self.cross_qk_rows = [[] for _ in range(self.rows)]

    # ---- single-token decode steps replayed from CUDA graphs (one graph per power-of-two bound on the KV length)
    def graph_ok(self) -> bool:
        dec = self.decoder
        if dec.device.type != "cuda" or os.environ.get("OGB_GENERATOR_GRAPH", "1") == "0":
            return False
        if dec.arch.num_experts > 0 and not all(lw.exp_blocked for lw in dec.layers):
            return False   # the unfused expert loop reads counts back to the host
        if any(self.rope_delta):
            return False   # rotary positions differ from the cache positions (multimodal RoPE after an image)
        if getattr(self, "alignment_heads", None):
            return False   # the recorded cross-attention scores are gathered with host-side shapes
        return dec.tp.size == 1

    def run_decode_graph(self, last_tokens: List[int]) -> torch.Tensor:
        """One token per row through a captured forward.  Returns the (static) fp32 logits buffer [rows, vocab]."""
        dev = self.decoder.device
        R = self.rows
        cap = self.blocks_per_row * self.block_size
        if max(self.kv_len) + 1 > cap:
            raise RuntimeError("sequence exceeds the allocated KV cache (max_length)")
        if not hasattr(self, "_g_host"):
            self._g_host = torch.empty(4 * R, dtype=torch.int32).pin_memory()
            self._g_dev = torch.empty(4 * R, dtype=torch.int32, device=dev)
            self._g_cu = torch.arange(R + 1, dtype=torch.int32, device=dev)
            self._g_rows = torch.arange(R, dtype=torch.int32, device=dev)
            self._g_np = self._g_host.numpy()
            self._g_pool = torch.cuda.graph_pool_handle()
            self._graphs: Dict[Any, Any] = {}
        h = self._g_np
        span = cap
        for r in range(R):
            p = self.kv_len[r]
            if self._tbl is not None:
                self._own_blocks(r, p, 1)
            h[r], h[R + r], h[2 * R + r], h[3 * R + r] = int(last_tokens[r]), p, self._slot(r, p), p
        self._flush_block_moves()
        self._g_dev.copy_(self._g_host, non_blocking=True)
        bound = 256
        while bound < max(self.kv_len) + 1:
            bound *= 2
        bound = min(bound, cap)
        if self.decoder.cos_small is not None and max(self.kv_len) + 1 <= self.decoder.rope_original_context:
            bound = min(bound, self.decoder.rope_original_context)   # the bound also selects the RoPE cache pair
        key = (bound, self.decoder.active_adapter)
        d = self._g_dev
        if key not in self._graphs:
            recurrent = self.decoder.arch.has_linear_layers
            s = StepInputs(input_ids=d[:R], positions=d[R:2 * R], slot_mapping=d[2 * R:3 * R], cu_seqlens=self._g_cu, past_lens=d[3 * R:],
                           block_table=self.block_table, logits_rows=self._g_rows, max_q_len=1, max_kv_len=bound,
                           state_slots=self._g_rows if recurrent else None, **self._cross_fields())
            with torch.no_grad():
                # the warm-up run really executes the step: appending keys and values twice is harmless, advancing a recurrent
                # state twice is not, so those states are put back before the replay
                saved = self.kv.state.clone() if recurrent and self.kv.state is not None else None
                self.decoder.forward(s, self.kv)   # warm-up: allocator, tensor maps, scratch
                if saved is not None:
                    self.kv.state.copy_(saved)
                    del saved
                torch.cuda.synchronize(dev)
                g = torch.cuda.CUDAGraph()
                with ops.graph_capture(g, pool=self._g_pool):   # graphs are replayed one at a time: they may share memory
                    out = self.decoder.forward(s, self.kv)
            self._graphs[key] = (g, out)
        g, out = self._graphs[key]
        g.replay()
        for r in range(R):
            self.kv_len[r] += 1
        return out

    def snapshot_recurrent(self) -> None:
        """Saves the recurrent states of every row (linear-attention layers) so that `restore_recurrent` can put them back
        after tokens were fed that are not kept (reference: the snapshot slots of src/models/recurrent_state.h:12-66)."""
        if self.kv.state is None:
            return
        if self._state_snapshot is None or self._state_snapshot.shape != self.kv.state.shape:
            self._state_snapshot = torch.empty_like(self.kv.state)
        rows = list(range(self.rows))
        ops.copy_state_slots(self.kv.state, self._state_snapshot, rows, rows)

    def restore_recurrent(self) -> None:
        if self.kv.state is None:
            return
        if self._state_snapshot is None or self._state_snapshot.shape != self.kv.state.shape:
            raise RuntimeError("restore_recurrent without a snapshot")
        rows = list(range(self.rows))
        ops.copy_state_slots(self._state_snapshot, self.kv.state, rows, rows)

    _state_snapshot = None

    def rewind(self, row: int, length: int):
        if self.decoder.arch.has_linear_layers and 0 < length < self.kv_len[row]:
            # a recurrent state cannot be cropped to an earlier position: callers restart from the empty state and feed the kept
            # tokens again (`Generator.rewind_to`), or restore a snapshot taken before the tokens were fed (speculative rounds)
            raise RuntimeError("models with linear-attention layers can only be rewound to length 0")
        self.kv_len[row] = min(self.kv_len[row], length)
        if length == 0:
            self.rope_delta[row] = 0
        if self._tbl is not None:
            self._recount()

    def _slot(self, row: int, pos: int) -> int:
        if self._tbl is None:
            return row * self.blocks_per_row * self.block_size + pos
        return int(self._tbl[row, pos // self.block_size]) * self.block_size + pos % self.block_size

    def _used_blocks(self, row: int) -> int:
        return (self.kv_len[row] + self.block_size - 1) // self.block_size

    def _recount(self):
        ref = np.zeros(self.rows * self.blocks_per_row, dtype=np.int32)
        for r in range(self.rows):
            np.add.at(ref, self._tbl[r, :self._used_blocks(r)], 1)
        self._ref = ref
        self._free = np.nonzero(ref == 0)[0][::-1].tolist()

    def _own_blocks(self, row: int, start: int, count: int):
        """Makes the blocks that positions [start, start + count) of `row` fall into writable by this row alone: a
        shared block that already holds tokens is copied to a fresh one, a block past the cached tokens is taken from
        the free list."""
        bs = self.block_size
        for j in range(start // bs, (start + count - 1) // bs + 1):
            holds_tokens = j * bs < start
            blk = int(self._tbl[row, j])
            if holds_tokens and self._ref[blk] == 1:
                continue
            new = self._free.pop()
            if holds_tokens:
                self._ref[blk] -= 1
                self._moves.append((blk, new))
            self._tbl[row, j] = new
            self._ref[new] = 1
            self._tbl_dirty = True

    def _flush_block_moves(self):
        if self._moves:
            bs = self.block_size
            dev = self.kv.full.device
            src = torch.tensor([m[0] for m in self._moves], dtype=torch.int64, device=dev)
            dst = torch.tensor([m[1] for m in self._moves], dtype=torch.int64, device=dev)
            ar = torch.arange(bs, device=dev)
            s_idx, d_idx = (src[:, None] * bs + ar).reshape(-1), (dst[:, None] * bs + ar).reshape(-1)
            self.kv.full[:, :, d_idx] = self.kv.full[:, :, s_idx]
            if self.kv.conv is not None:
                self.kv.conv[:, d_idx] = self.kv.conv[:, s_idx]
            self._moves = []
        if self._tbl_dirty:
            self.block_table.copy_(torch.from_numpy(self._tbl))
            self._tbl_dirty = False

    def _reorder_cross_qk(self, src_rows: List[int]):
        if getattr(self, "alignment_heads", None):
            self.cross_qk_rows = [list(self.cross_qk_rows[s]) for s in src_rows]

    def reorder_rows(self, src_rows: List[int]):
        """Beam search: row r continues from the cache of row src_rows[r].  Only the block table is permuted; blocks are
        shared between the rows that descend from the same hypothesis and copied when one of them writes into a shared
        block (`_own_blocks`), so a step moves at most one block per row instead of whole caches."""
        self._reorder_cross_qk(src_rows)
        if self._tbl is None:
            if all(r == s for r, s in enumerate(src_rows)):
                return
            self._tbl = self.block_table.cpu().numpy().copy()
        self._tbl = self._tbl[np.asarray(src_rows, dtype=np.int64)].copy()
        if self.kv.state is not None:       # recurrent states follow their hypotheses
            self.kv.state = self.kv.state[:, torch.as_tensor(src_rows, dtype=torch.long, device=self.kv.state.device)].contiguous()
        self.kv_len = [self.kv_len[s] for s in src_rows]
        self._recount()
        self._tbl_dirty = True


class Generator:
    def __init__(self, model: Model, params: GeneratorParams):
        self.model = model
        self.params = params
        s = dict(params.search)
        cfg = model.config
        if s["max_length"] > cfg.context_length:
            raise RuntimeError(f"max_length ({s['max_length']}) cannot be greater than model context_length ({cfg.context_length})")
        if not (1 <= s["batch_size"] <= 32 * 64):
            raise RuntimeError("batch_size must be >= 1")
        if not (1 <= s["num_beams"] <= 32):
            raise RuntimeError("num_beams must be between 1 and 32")
        if s["num_return_sequences"] > s["num_beams"] and s["num_beams"] > 1:
            raise RuntimeError("num_return_sequences cannot exceed num_beams")
        self.search_opts = s
        self.method, self.k, self.p, self.t = _sampling_method(s, cfg.vocab_size)
        sp = native.SearchParams()
        sp.batch_size, sp.num_beams, sp.num_return_sequences = s["batch_size"], s["num_beams"], s["num_return_sequences"]
        sp.max_length, sp.min_length, sp.vocab_size = s["max_length"], s["min_length"], cfg.vocab_size
        sp.pad_token_id, sp.eos_token_ids = cfg.pad_token_id, list(cfg.eos_token_ids)
        sp.repetition_penalty, sp.no_repeat_ngram_size = s["repetition_penalty"], s["no_repeat_ngram_size"]
        sp.length_penalty, sp.early_stopping, sp.random_seed = s["length_penalty"], s["early_stopping"], s["random_seed"]
        self._sp = sp
        self.search = native.Search(sp)
        self._beam_dev = None                                                   # device-side beam scorer, made at the first beam step
        self._beam_dev_ok = os.environ.get("OGB_DEVICE_BEAM_SCORER", "1") != "0"   # 0: candidates cross to the host scorer
        self.rows = s["batch_size"] * s["num_beams"]
        if model.type == "marian-ssru":
            from .models.marian import MarianState
            self.state = MarianState(model.decoder, self.rows, s["max_length"])
        elif model.type in ("parakeet_tdt", "nemotron_speech"):
            from .models.transducer import TransducerState
            self.state = TransducerState(model.decoder, self.rows, s["max_length"])
        else:
            self.state = SequenceState(model.decoder, self.rows, s["max_length"], kv_bits=model.kv_bits)
        self._logits: Optional[torch.Tensor] = None
        self._fresh = False
        self._started = False
        self._telemetry = telemetry.GenerationTimer()
        self._seed = s["random_seed"] if s["random_seed"] >= 0 else int.from_bytes(os.urandom(4), "little")
        self._guidance = None
        if params.guidance_type:
            from .guidance import GuidanceProcessor
            self._guidance = GuidanceProcessor(model, params.guidance_type, params.guidance_data, s["batch_size"],
                                               params.guidance_ff_tokens)
        self._strategy = None
        spec = params.speculative
        if model.draft is not None or spec.get("ngram_size", 0) > 0:
            from .speculative import make_strategy
            self._strategy = make_strategy(self, spec)
        self._runtime_options: Dict[str, str] = {}
        self._terminated = False

    # ------------------------------------------------------------------ tokens in
    def append_tokens(self, tokens):
        with _Trace("generator", "append_tokens"):
            if isinstance(tokens, Tensor):
                tokens = tokens.as_numpy()
            if telemetry.enabled():
                self._telemetry.on_prompt(np.asarray(tokens).size)
            arr = np.asarray(tokens, dtype=np.int32)
            if arr.ndim == 1:
                arr = arr.reshape(1, -1)
            B = self.search_opts["batch_size"]
            if arr.shape[0] != B:
                raise RuntimeError(f"append_tokens: expected {B} rows, got {arr.shape[0]}")
            if arr.shape[1] == 0:
                raise RuntimeError("append_tokens: empty token list")
            if self._started and B > 1:
                raise RuntimeError("continuous decoding (append after generate) requires batch_size 1")
            if native.log_flag("append_next_tokens"):
                native.log_write("append_next_tokens", str(arr.tolist()))
            self.search.append_tokens(arr)
            pad = self.model.config.pad_token_id
            nb = self.search_opts["num_beams"]
            row_tokens: List[List[int]] = []
            for b in range(B):
                toks = arr[b].tolist()
                if not self._started and B > 1:  # padded batch: pad tokens are not fed to the model
                    while len(toks) > 1 and toks[-1] == pad:
                        toks.pop()
                    while len(toks) > 1 and toks[0] == pad:
                        toks.pop(0)
                for _ in range(nb):
                    row_tokens.append(list(toks))
            if self._started and self._unfed_last:
                # the last generated token has not been through the model yet
                last = self.search.next_tokens().tolist()
                row_tokens = [[last[r]] + row_tokens[r] for r in range(self.rows)]
                self._unfed_last = False
            if self._guidance is not None:
                self._guidance.commit_prompt(arr)
            if self._strategy is not None:
                self._strategy.on_append(arr)
            self._compute_logits(row_tokens)
            self._started = True

    _unfed_last = False  # True while the newest token has not been run through the model

    def _compute_logits(self, row_tokens: List[List[int]]):
        dec = self.model.decoder
        if dec.cos_small is not None:
            # Long-context RoPE: the cache of a sequence that grows past the original context length was filled with the
            # short-factor rotation; rebuild it from the whole sequence with the long-factor caches
            # (reference: src/standard_decoding_strategy.cpp:64-76).
            cur = max(self.state.kv_len)
            if 0 < cur <= dec.rope_original_context < cur + max(len(t) for t in row_tokens):
                for r in range(self.rows):
                    self.state.rewind(r, 0)
                row_tokens = [self.search.sequence(r).tolist() for r in range(self.rows)]
        chunk = int(self.search_opts.get("chunk_size") or 0)
        with _Trace("model", "run"), torch.no_grad():
            if chunk > 0 and self._image_features is None:
                longest = max(len(t) for t in row_tokens)
                logits = None
                for c0 in range(0, longest, chunk):
                    part = [t[c0:c0 + chunk] for t in row_tokens]
                    out, used = self.state.run(part)
                    if logits is None:
                        logits = torch.empty(self.rows, out.shape[1], dtype=torch.float32, device=out.device)
                    logits[used] = out
            elif all(len(t) == 1 for t in row_tokens) and self._started and self.state.graph_ok():
                logits = self.state.run_decode_graph([t[0] for t in row_tokens])
            else:
                logits, used = self.state.run(row_tokens, inputs_embeds=self._embeds_with_images(row_tokens),
                                              positions3=self._take_position_ids(row_tokens))
                if len(used) != self.rows:
                    full = torch.empty(self.rows, logits.shape[1], dtype=torch.float32, device=logits.device)
                    full[used] = logits
                    logits = full
        self._logits = logits
        self._fresh = True

    # ------------------------------------------------------------------ one step
    def generate_next_token(self):
        with _Trace("generator", "generate_next_token"):
            if self._terminated:
                raise RuntimeError("session terminated")
            if self.search.is_done:
                return
            if not self._started:
                raise RuntimeError("generate_next_token called before append_tokens")
            if self._strategy is not None:
                self._strategy.step()
            else:
                self._standard_step()
        if telemetry.enabled():
            self._telemetry.on_token()
            if self.search.is_done:
                self._telemetry.finish(self.model.type, self.model.device_type, self.search_opts.get("batch_size", 1) if isinstance(self.search_opts, dict) else 1)

    def _ensure_logits(self):
        if not self._fresh:
            last = self.search.next_tokens().tolist()
            self._compute_logits([[t] for t in last])
            self._unfed_last = False

    def _standard_step(self):
        self._ensure_logits()
        logits = self._logits
        so = self.search_opts
        if self._guidance is not None:
            logits = self._guidance.apply(logits)
        on_cpu = not logits.is_cuda
        if on_cpu:
            arr = np.ascontiguousarray(logits.float().numpy())
            self.search.score(arr, "beam" if so["num_beams"] > 1 else self.method, self.k, self.p, self.t)
            if so["num_beams"] > 1:
                self.state.reorder_rows(self.search.beam_rows().tolist())
        else:
            self._device_step(logits)
        self._fresh = False
        self._unfed_last = True
        toks = self.search.next_tokens()
        if self._guidance is not None:
            self._guidance.commit_tokens(toks)
        if native.log_flag("generate_next_token"):
            native.log_write("generate_next_token", str(toks.tolist()))
        if self.search.is_done and native.log_flag("hit_eos"):
            native.log_write("hit_eos", "generation finished")

    def _device_step(self, logits: torch.Tensor):
        so = self.search_opts
        dev = logits.device
        need_edit = so["min_length"] > 0 or so["repetition_penalty"] != 1.0 or so["no_repeat_ngram_size"] > 0
        if need_edit:
            logits = logits.clone() if logits is self._logits else logits
            self._apply_penalties_device(logits)
        if so["num_beams"] > 1:
            from . import beam_device
            if self._beam_dev is None and self._beam_dev_ok and beam_device.supported(so["num_beams"], self._sp.eos_token_ids):
                seqs = np.stack([self.search.sequence(r) for r in range(self.rows)]).astype(np.int32)
                self._beam_dev = beam_device.DeviceBeamScorer(seqs, so["batch_size"], so["num_beams"], so["max_length"], self._sp.pad_token_id,
                                                              list(self._sp.eos_token_ids), so["length_penalty"], so["early_stopping"], dev)
            if self._beam_dev is not None:
                # scorer, hypotheses and sequences on the device: one small copy back (tokens, source rows, open entries)
                cs, ct, cb = ops.beam_candidates(logits, self._beam_dev.beam_scores(), so["batch_size"], so["num_beams"])
                toks, rows, all_done = self._beam_dev.step(cs, ct, cb)
                self.search.commit_beam_result(toks, rows, all_done)
                self.state.reorder_rows(rows.tolist())
                return
            scores = torch.from_numpy(self.search.beam_scores()).to(dev)
            cs, ct, cb = ops.beam_candidates(logits, scores, so["batch_size"], so["num_beams"])
            self.search.commit_beam_step(cs.cpu().numpy(), ct.cpu().numpy(), cb.cpu().numpy())
            self.state.reorder_rows(self.search.beam_rows().tolist())
            return
        R = self.rows
        if self.method == "greedy":
            toks = ops.argmax(logits)
        else:
            k = torch.full((R,), self.k if self.k > 0 else -1, dtype=torch.int32, device=dev)
            p = torch.full((R,), self.p, dtype=torch.float32, device=dev)
            t = torch.full((R,), self.t, dtype=torch.float32, device=dev)
            seeds = (torch.arange(R, dtype=torch.int64, device=dev) * 0x9E3779B97F4A7C15 % (1 << 62)) + self._seed
            pos = torch.full((R,), self.search.length, dtype=torch.int32, device=dev)
            toks = ops.sample(logits, k, p, t, seeds, pos)
        self.search.commit_tokens(toks.cpu().numpy())

    def _apply_penalties_device(self, logits: torch.Tensor):
        """Builds the sparse edit list on the host from the sequences and applies it in one kernel."""
        so = self.search_opts
        rows, toks, opsl, vals = [], [], [], []
        cur = self.search.length
        eos = list(self.model.config.eos_token_ids)
        for r in range(self.rows):
            seq = self.search.sequence(r)
            if cur < so["min_length"]:
                for e in eos:
                    rows.append(r); toks.append(e); opsl.append(0); vals.append(0.0)
            if so["repetition_penalty"] != 1.0:
                for tkn in np.unique(seq).tolist():
                    rows.append(r); toks.append(tkn); opsl.append(1); vals.append(float(so["repetition_penalty"]))
            if so["no_repeat_ngram_size"] > 0:
                for tkn in native.no_repeat_ngram_banned(seq, so["no_repeat_ngram_size"], logits.shape[1]):
                    rows.append(r); toks.append(tkn); opsl.append(0); vals.append(0.0)
        if not rows:
            return
        dev = logits.device
        # repetition penalty first, then bans: order inside one launch is irrelevant because a ban wins anyway
        order = np.argsort(np.asarray(opsl), kind="stable")[::-1]
        i32 = lambda x: torch.tensor(np.asarray(x)[order], dtype=torch.int32, device=dev)
        pen = [i for i in range(len(opsl)) if opsl[i] == 1]
        ban = [i for i in range(len(opsl)) if opsl[i] == 0]
        for sel in (pen, ban):
            if sel:
                ops.logits_edit(logits, torch.tensor([rows[i] for i in sel], dtype=torch.int32, device=dev),
                                torch.tensor([toks[i] for i in sel], dtype=torch.int32, device=dev),
                                torch.tensor([opsl[i] for i in sel], dtype=torch.int32, device=dev),
                                torch.tensor([vals[i] for i in sel], dtype=torch.float32, device=dev))

    # ------------------------------------------------------------------ accessors
    def is_done(self) -> bool:
        return bool(self.search.is_done)

    def get_next_tokens(self) -> np.ndarray:
        return self.search.next_tokens()

    def get_sequence(self, index: int) -> np.ndarray:
        so = self.search_opts
        if so["num_beams"] > 1 and self.search.is_done:
            if self._beam_dev is not None and not self._beam_dev.finalized:
                for b, ranked in enumerate(self._beam_dev.finalize()):
                    for rank, (toks, score) in enumerate(ranked):
                        self.search.set_hypothesis(b, rank, toks.astype(np.int32), score)
            self.search.finalize()
            b, rank = divmod(index, so["num_return_sequences"])
            return self.search.hypothesis(b, rank)[0]
        return self.search.sequence(index)

    def token_count(self) -> int:
        return int(self.search.length)

    def get_logits(self) -> np.ndarray:
        self._ensure_logits()
        return self._logits.detach().float().cpu().numpy().reshape(self.rows, 1, -1)

    def set_logits(self, new_logits):
        arr = np.asarray(new_logits, dtype=np.float32).reshape(self.rows, -1)
        if arr.shape[1] != self.model.config.vocab_size:
            raise RuntimeError("set_logits: last dimension must equal vocab_size")
        self._logits = torch.from_numpy(arr.copy()).to(self.model.device)
        self._fresh = True

    def rewind_to(self, length: int):
        if self.search_opts["batch_size"] > 1 and length != 0:
            raise RuntimeError("rewind_to a non-zero length requires batch_size 1")
        if length > self.search.length:
            raise RuntimeError("rewind_to: length exceeds the current sequence length")
        recurrent = getattr(getattr(self.model, "arch", None), "has_linear_layers", False) and 0 < length < self.search.length
        self.search.rewind_to(int(length))
        if recurrent:
            # a recurrent state cannot be cropped: restart from the empty state and feed the kept tokens again
            for r in range(self.rows):
                self.state.rewind(r, 0)
            self._fresh = False
            self._unfed_last = False
            self._compute_logits([self.search.sequence(r).tolist() for r in range(self.rows)])
            if self._guidance is not None:
                self._guidance.reset()
            if self._strategy is not None:
                self._strategy.on_rewind(int(length))
            return
        if self._beam_dev is not None:
            # the host scorer cannot take over a search the device scorer began: later steps stay on the device, from the
            # rewound sequences with fresh beam scores
            self._beam_dev = None
        for r in range(self.rows):
            self.state.rewind(r, int(length))
        self._fresh = False
        self._unfed_last = False
        if length == 0:
            self._started = False
        else:
            # the token at position length-1 must be fed again to produce logits
            self.state.rewind(0, int(length) - 1)
            last = int(self.search.sequence(0)[-1])
            self._compute_logits([[last]])
        if self._guidance is not None:
            self._guidance.reset()
        if self._strategy is not None:
            self._strategy.on_rewind(int(length))

    def get_input(self, name: str):
        if name == "input_ids":
            return self.search.next_tokens()
        if name in getattr(self, "_extra_inputs", {}):
            v = self._extra_inputs[name]
            return v.as_numpy() if isinstance(v, Tensor) else np.asarray(v)
        raise RuntimeError(f"unknown model input: {name}")

    def get_output(self, name: str):
        if name == "logits":
            return self.get_logits()
        if name == "hidden_states":
            return self.model.decoder.last_hidden.detach().float().cpu().numpy()
        if name == "cross_qk":
            # [rows, alignment heads, tokens fed so far, encoder frames]: scaled query-key scores before the softmax
            rows = getattr(self.state, "cross_qk_rows", None)
            if not rows or not rows[0]:
                raise RuntimeError("cross_qk: set the alignment_heads input (an int32 [n, 2] tensor of (layer, head)) before the tokens")
            n = min(len(r) for r in rows)
            return torch.stack([torch.stack(r[:n], dim=1) for r in rows]).numpy()
        raise RuntimeError(f"unknown model output: {name}")

    def set_inputs(self, named: NamedTensors):
        """Inputs produced by the multimodal processor: `audio_features` run the audio encoder and fill the decoder's
        cross-attention cache, `pixel_values` run the vision encoder (its features replace the image-token embeddings of
        the prompt), `input_ids` are appended as the prompt (reference: src/generators.cpp:700-711 SetInputs)."""
        named = dict(named)
        self._extra_inputs = named
        m = self.model
        arr = lambda v: v.as_numpy() if isinstance(v, Tensor) else v
        if "audio_features" in named and hasattr(self.state, "set_audio"):
            # speech transducer: the log-mel features of one utterance; decoding starts from the blank token
            feats = torch.as_tensor(np.asarray(arr(named["audio_features"]), dtype=np.float32))
            if feats.dim() == 3:
                if feats.shape[0] != 1:
                    raise RuntimeError("speech transducers take one utterance at a time")
                feats = feats[0]
            self.state.set_audio(feats)
            if not self._started:
                self.append_tokens(np.asarray([[m.decoder.cfg.blank_id]], dtype=np.int32))
            return
        if "audio_features" in named:
            if m.encoder is None:
                raise RuntimeError("this model has no audio encoder")
            feats = torch.as_tensor(np.asarray(arr(named["audio_features"])))
            if feats.shape[0] != self.search_opts["batch_size"]:
                raise RuntimeError(f"audio_features: expected {self.search_opts['batch_size']} clips, got {feats.shape[0]}")
            with _Trace("model", "encoder"):
                enc_out, lens = m.encoder.encode_audio(feats)
                self.state.set_cross(enc_out, lens, self.search_opts["num_beams"])
        if "pixel_values" in named:
            if m.vision is None:
                raise RuntimeError("this model has no vision encoder")
            with _Trace("model", "vision"):
                if hasattr(m.vision, "encode_patches"):
                    # Qwen2-VL: pixel_values are flattened patches, image_grid_thw says how they tile every image
                    if "image_grid_thw" not in named:
                        raise RuntimeError("this vision encoder needs image_grid_thw beside pixel_values")
                    grids = [tuple(int(v) for v in g) for g in np.asarray(arr(named["image_grid_thw"])).reshape(-1, 3)]
                    feats, lens = m.vision.encode_patches(np.asarray(arr(named["pixel_values"]), dtype=np.float32), grids)
                    self._image_grids = grids
                else:
                    feats, lens = m.vision.encode_images(torch.as_tensor(np.asarray(arr(named["pixel_values"]))))
            self._image_features = feats
        if "input_ids" in named:
            self.append_tokens(arr(named["input_ids"]))

    _image_features: Optional[torch.Tensor] = None
    _image_grids = None      # (t, h, w) of the images whose features are pending (Qwen2-VL)

    def _take_position_ids(self, row_tokens: List[List[int]]):
        """A staged `position_ids` input of shape [3, batch, sequence] (multimodal RoPE, reference:
        src/models/position_inputs.cpp, the Qwen2-VL branch) applies to the next tokens fed: per row the three components of
        its tokens."""
        extra = getattr(self, "_extra_inputs", {})
        if self.model.arch.mrope_section is not None and "position_ids" not in extra and self._image_grids:
            # positions derived here from the image grids (reference: src/models/qwen_vl_model.cpp computes them the same way
            # when the caller supplies none): every batch entry consumes its images in order, its beams share them
            from .models.qwen_vl import mrope_positions
            nb = self.search_opts["num_beams"]
            merge = self.model.vision.cfg.spatial_merge_size
            out, grids = [], list(self._image_grids)
            for r, toks in enumerate(row_tokens):
                if r % nb == 0:
                    start = self.state.kv_len[r] + self.state.rope_delta[r]
                    comp, used, _ = mrope_positions(toks, self.model.image_token_id, grids, merge, start) if toks else (None, 0, 0)
                    grids = grids[used:]
                out.append(comp)
            self._image_grids = grids or None
            return out
        if self.model.arch.mrope_section is None or "position_ids" not in extra:
            return None
        v = extra.pop("position_ids")
        arr = np.asarray(v.as_numpy() if isinstance(v, Tensor) else v)
        if arr.ndim != 3 or arr.shape[0] != 3:
            raise RuntimeError("position_ids for multimodal RoPE must have shape [3, batch, sequence]")
        nb = self.search_opts["num_beams"]
        out = []
        for r, toks in enumerate(row_tokens):
            comp = arr[:, r // nb, :]
            if comp.shape[1] < len(toks):
                raise RuntimeError("position_ids are shorter than the tokens they describe")
            out.append(comp[:, comp.shape[1] - len(toks):] if toks else None)
        return out

    def _embeds_with_images(self, row_tokens: List[List[int]]) -> Optional[torch.Tensor]:
        """Token embeddings of the packed step with the rows at image-token positions replaced, in order, by the pending
        image features (each batch item's beams read the same features)."""
        feats = self._image_features
        if feats is None:
            return None
        dec, m = self.model.decoder, self.model
        nb = self.search_opts["num_beams"]
        ids = torch.tensor([t for toks in row_tokens for t in toks], dtype=torch.int32, device=dec.device)
        emb = ops.embedding(ids, dec.embed, dec.arch.embed_scale)
        src, used = [], 0
        for r, toks in enumerate(row_tokens):
            n = sum(1 for t in toks if t == m.image_token_id)
            if r % nb == 0:
                start, used = used, used + n
            src.append(torch.arange(start, start + n))
        src = torch.cat(src) if src else torch.zeros(0, dtype=torch.long)
        if used > feats.shape[0]:
            raise RuntimeError(f"the prompt has {used} image tokens but the images give {feats.shape[0]} features")
        if src.numel():
            emb[(ids == m.image_token_id).nonzero().flatten()] = feats[src.to(dec.device)].to(emb.dtype)
        self._image_features = feats[used:] if used < feats.shape[0] else None
        return emb

    def set_model_input(self, name: str, tensor):
        self._extra_inputs = getattr(self, "_extra_inputs", {})
        self._extra_inputs[name] = tensor
        if name == "alignment_heads":
            arr = np.asarray(tensor.as_numpy() if isinstance(tensor, Tensor) else tensor).reshape(-1, 2)
            a = self.model.arch
            if arr.size and (arr[:, 0].max() >= a.num_layers or arr[:, 1].max() >= a.num_heads or arr.min() < 0):
                raise RuntimeError("alignment_heads: (layer, head) out of range")
            self.state.set_alignment_heads(arr.tolist())

    def snapshot_state(self):
        """Marks the current state as a point speculative decoding may roll back to (reference:
        src/generators.h:135, recurrent models copy their state to a snapshot slot).  Every cache of this runtime - keys /
        values and the convolution inputs of hybrid layers - is addressed by position through block tables, so `rewind_to`
        restores any earlier length without a copy; the call only records the length."""
        self._snapshot_length = self.token_count()
        return self._snapshot_length

    def set_hidden_states(self, hidden_states):
        """Stages a `hidden_states` input for the next model run (the input of a multi-token-prediction head, reference:
        src/generators.h:141); read back with get_input("hidden_states")."""
        arr = hidden_states.as_numpy() if isinstance(hidden_states, Tensor) else np.asarray(hidden_states)
        self.set_model_input("hidden_states", arr)

    def set_active_adapter(self, adapters, name: str):
        adapters._activate(self.model, name)

    def set_runtime_option(self, key: str, value: str):
        if key == "terminate_session":
            self._terminated = value in ("1", "true", True)
        elif key == "enable_profiling":
            if value not in ("0", "", False):
                native.trace_enable("" if value in ("1", True) else str(value))
            else:
                native.trace_disable()
        else:
            raise RuntimeError(f"Unknown runtime option: {key}")
        self._runtime_options[key] = str(value)

    def get_speculative_stats(self) -> Dict[str, Any]:
        if self._strategy is None:
            return {}
        return self._strategy.stats()
