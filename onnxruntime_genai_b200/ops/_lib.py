"""ctypes binding of libogb200_kernels.so (the sm_100a kernel library).

The library is built in-tree by `onnxruntime_genai_b200.build_native`.  On a machine with a CUDA
device the library MUST load: ops on CUDA tensors never fall back to PyTorch silently.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libogb200_kernels.so")

_lib = None
_initialised_devices = set()

_P = c_void_p


class GemmFused(ctypes.Structure):
    """OgbGemmFused of csrc/kernels.h: the decode-step fusions of ogb_gemm_bf16_fused."""
    _fields_ = [("norm_eps", c_float), ("positions", _P), ("slots", _P), ("cos", _P), ("sin", _P), ("k_cache", _P), ("v_cache", _P),
                ("Hq", c_int), ("Hkv", c_int), ("D", c_int), ("rot", c_int), ("max_pos", c_int)]


_SIGS = {
    "ogb_runtime_init": (c_int, [c_int]),
    "ogb_status_device_ptr": (_P, [c_int]),
    "ogb_status_read_and_clear": (c_int, [c_int]),
    "ogb_sm_count": (c_int, [c_int]),
    "ogb_last_cuda_error": (ctypes.c_char_p, []),
    "ogb_gemm_token_tile": (c_int, [c_int, c_int]),
    "ogb_gemm_auto_splits": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "ogb_gemm_max_active_clusters": (c_int, [c_int, c_int]),
    "ogb_gemm_bf16": (c_int, [_P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P, c_int, c_int, c_int, c_int, _P, c_int, _P]),
    "ogb_gemm_bf16_fused": (c_int, [_P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, _P, _P, c_int, c_int, c_int, c_int, _P, c_int, _P, _P]),
    "ogb_comm_register": (c_int, [c_int, c_int, c_int, _P, _P, c_longlong]),
    "ogb_comm_register_nvls": (c_int, [c_int, _P, _P, _P, _P, _P, _P, _P, c_longlong]),
    "ogb_comm_has_nvls": (c_int, [c_int]),
    "ogb_comm_set_options": (c_int, [c_int, c_longlong, c_int]),
    "ogb_comm_capacity": (c_longlong, [c_int]),
    "ogb_w4_packed_bytes": (c_longlong, [c_int, c_int]),
    "ogb_gemm_w4": (c_int, [_P, c_int, _P, _P, c_int, c_int, c_int, c_int, _P, _P, c_int, c_int, c_int, _P, c_int, _P]),
    "ogb_moe_gemm": (c_int, [_P, c_int, _P, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P, c_int, c_int, c_float, c_float, _P, _P, _P,
                             _P, c_int, c_int, _P, _P]),
    "ogb_fp4_packed_bytes": (c_longlong, [c_int, c_int, c_int]),
    "ogb_moe_gemm_fp4": (c_int, [_P, c_int, _P, _P, c_int, c_int, c_int, c_int, c_int, _P, c_int, c_int, c_float, c_float, _P, _P, _P,
                                 _P, c_int, c_int, c_int, _P, _P, _P]),
    "ogb_moe_fp4_reads_row_map": (c_int, [c_int, c_int, c_int]),
    "ogb_collective": (c_int, [c_int, _P, _P, _P, c_longlong, c_int, _P, c_int, _P]),
    "ogb_moe_topk": (c_int, [_P, c_int, c_int, c_int, c_int, c_int, _P, _P, _P]),
    "ogb_moe_max_tiles": (c_int, [c_int, c_int, c_int]),
    "ogb_moe_sort": (c_int, [_P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, c_int, _P]),
    "ogb_moe_combine": (c_int, [_P, c_int, _P, _P, c_int, c_int, c_int, _P, c_int, _P, c_int, _P]),
    "ogb_embedding": (c_int, [_P, _P, _P, c_int, c_int, c_int, c_float, _P]),
    "ogb_norm": (c_int, [_P, _P, _P, _P, _P, _P, c_int, c_int, c_float, c_int, _P]),
    "ogb_norm_moe_combine": (c_int, [_P, c_int, _P, _P, c_int, _P, _P, _P, _P, _P, c_int, c_int, c_float, c_int, _P]),
    "ogb_rope_kv_append": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, _P]),
    "ogb_rope_kv_append_bits": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_int, _P, c_int, c_int, _P]),
    "ogb_embedding_q4": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, c_int, c_float, _P]),
    "ogb_act_mul": (c_int, [_P, _P, c_int, c_int, c_int, _P]),
    "ogb_act": (c_int, [_P, _P, c_longlong, c_int, _P]),
    "ogb_causal_conv": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "ogb_short_conv": (c_int, [_P, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, c_int, c_int, c_int, _P]),
    "ogb_decode_advance": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P]),
    "ogb_logits_edit": (c_int, [_P, c_int, _P, _P, _P, _P, c_int, _P]),
    "ogb_logits_bitmask": (c_int, [_P, c_int, c_int, _P, _P, _P]),
    "ogb_bf16_to_f32": (c_int, [_P, _P, c_longlong, _P]),
    "ogb_gather_rows": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "ogb_gather_rows_f16": (c_int, [_P, _P, _P, c_int, c_int, _P]),
    "ogb_attention_scratch_bytes": (c_longlong, [c_int, c_int, c_int, c_int]),
    "ogb_paged_attention": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, _P, c_float, c_float, c_int, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_longlong, c_int, _P, _P, _P]),
    "ogb_paged_attention_skip": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, _P, c_float, c_float, c_int, c_int,
                                         c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_longlong, c_int, _P, _P, _P, c_int]),
    "ogb_attention_tc_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "ogb_attention_tc": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, _P, c_float, c_float, c_int, c_int, c_int,
                                 c_int, c_int, c_int, c_int, c_int, _P, _P]),
    "ogb_paged_attention_kv8": (c_int, [_P, c_int, _P, _P, _P, _P, _P, c_int, c_int, _P, c_int, _P, c_float, c_float, c_int, c_int,
                                    c_int, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_longlong, c_int, _P, _P, _P]),
    "ogb_gated_delta_fused": (c_int, [_P, c_longlong, c_longlong, c_longlong, c_longlong, _P, c_longlong, c_longlong, c_longlong, _P, _P, c_float,
                                      _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "ogb_gdn_gate_norm": (c_int, [_P, _P, c_longlong, _P, c_float, _P, c_int, c_int, c_int, _P]),
    "ogb_gated_delta": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "ogb_mamba2_scan_fused": (c_int, [_P, c_longlong, _P, c_longlong, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "ogb_mamba_gate_norm": (c_int, [_P, _P, c_longlong, _P, c_float, _P, c_int, c_int, _P]),
    "ogb_mamba2_scan": (c_int, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, _P]),
    "ogb_copy_state_slots": (c_int, [_P, _P, c_int, c_int, c_longlong, _P, _P, c_int, _P]),
    "ogb_sample": (c_int, [_P, c_longlong, c_int, c_int, _P, _P, _P, _P, _P, _P, _P]),
    "ogb_argmax": (c_int, [_P, c_longlong, c_int, c_int, _P, _P]),
    "ogb_topk": (c_int, [_P, c_longlong, c_int, c_int, c_int, c_int, _P, _P, _P, _P]),
    "ogb_beam_merge": (c_int, [_P, _P, c_int, c_int, c_int, _P, _P, _P, _P]),
    "ogb_beam_scorer_step": (c_int, [_P, _P, _P, _P, _P, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float,
                                     _P, c_int, _P]),
    "ogb_beam_scorer_finalize": (c_int, [_P, _P, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, _P,
                                         c_int, _P]),
    "ogb_verify_sampled": (c_int, [_P, c_longlong, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, _P, _P, _P, _P]),
    "ogb_verify_greedy": (c_int, [_P, _P, c_int, _P, _P, _P]),
}

_OPTIONAL = set()


def lib():
    """Returns the loaded kernel library, building it first when the sources are newer."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        from ..build_native import build_kernels
        build_kernels()
    handle = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _SIGS.items():
        try:
            fn = getattr(handle, name)
        except AttributeError:
            if name in _OPTIONAL:
                continue
            raise RuntimeError(f"{LIB_PATH} is stale (missing {name}); rebuild with python -m onnxruntime_genai_b200.build_native")
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def bind(name: str, restype, argtypes):
    """Registers the signature of an extra entry point (used by optional kernel files)."""
    fn = getattr(lib(), name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def init_device(index: int) -> None:
    if index in _initialised_devices:
        return
    rc = lib().ogb_runtime_init(index)
    if rc != 0:
        raise RuntimeError(f"ogb_runtime_init({index}) failed with {rc}")
    _initialised_devices.add(index)


STATUS_NAMES = {0: "ok", 1: "TMA pipeline wait ran out", 2: "accumulator wait ran out", 3: "peer wait ran out", 4: "bad argument"}


def check_status(index: int) -> None:
    """Synchronises the device and raises if a kernel reported a bounded wait that ran out."""
    code = lib().ogb_status_read_and_clear(index)
    if code != 0:
        raise RuntimeError(f"sm_100a kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown')}")


LAUNCH_COUNT = 0  # launcher calls so far (one kernel each; split-KV attention adds its combine kernel)


def check(rc: int, what: str) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += 1
    if rc != 0:
        why = ""
        if rc == -4:     # a launch (or the configuration call before it) was refused by the CUDA runtime
            try:
                why = ": " + lib().ogb_last_cuda_error().decode()
            except Exception:
                pass
        raise RuntimeError(f"{what} failed with code {rc}{why}")
