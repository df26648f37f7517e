"""The allocation-free attention entry point (csrc/noalloc.h), called through its exported C symbol.

Some callers of the kernel library cannot allocate device memory at all (a plug-in inside a foreign
process, a serving thread that must not touch the allocator, a fixed memory budget).  For them
`ogb_paged_attention_noalloc` keeps the split-KV scratch inside the library.  It must give the same
result as the regular entry point, call after call, even though every call reuses the same scratch.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = -7


def _symbol():
    from onnxruntime_genai_b200.ops import _lib
    P, I, F, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
    fn = _lib.bind("ogb_paged_attention_noalloc", I, [P, I, P, P, P, P, P, I, I, P, I, P, F, F, I, I, I, I, I, I, I, I, P])
    need = _lib.bind("ogb_paged_attention_noalloc_required_bytes", LL, [I, I, I, I])
    return fn, need


def _case(seed, B, past, Hq, Hkv, D, bs):
    g = torch.Generator().manual_seed(seed)
    cols = max((p + 1 + bs - 1) // bs for p in past)
    nblocks = B * cols + 2
    perm = torch.randperm(nblocks, generator=g)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    used = 0
    for b in range(B):
        n = (past[b] + 1 + bs - 1) // bs
        table[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()
    return dict(q=mk(B, (Hq + 2 * Hkv) * D), kc=mk(nblocks * bs, Hkv, D), vc=mk(nblocks * bs, Hkv, D),
                cu=torch.arange(B + 1, dtype=torch.int32).cuda(), pl=torch.tensor(past, dtype=torch.int32).cuda(), table=table.cuda())


def test_noalloc_attention_matches_regular_entry_point_twice():
    from onnxruntime_genai_b200 import ops
    fn, need = _symbol()
    Hq, Hkv, D, bs, splits = 32, 8, 128, 16, 4
    stream = torch.cuda.current_stream().cuda_stream
    for seed, past in ((1, [700, 45, 1300, 16]), (2, [90, 2047, 5, 512])):   # two calls in a row share the scratch
        c = _case(seed, 4, past, Hq, Hkv, D, bs)
        want = ops.paged_attention(c["q"], c["kc"], c["vc"], c["cu"], c["pl"], c["table"], bs, Hq, Hkv, D, 1 / math.sqrt(D),
                                   max_q_len=1, max_kv_len=max(past) + 1, splits=splits)
        out = torch.empty(4, Hq * D, dtype=torch.bfloat16, device="cuda")
        assert need(4, Hq, D, splits) <= 8 << 20
        rc = fn(c["q"].data_ptr(), c["q"].stride(0), c["kc"].data_ptr(), c["vc"].data_ptr(), c["cu"].data_ptr(), c["pl"].data_ptr(),
                c["table"].data_ptr(), c["table"].stride(0), bs, out.data_ptr(), out.stride(0), None, 1 / math.sqrt(D), 0.0, 0, 4, 4, 1,
                Hq, Hkv, D, splits, stream)
        assert rc == 0
        torch.cuda.synchronize()
        # same kernel, same split plan: the two entry points agree bit for bit
        assert torch.equal(out, want), f"no-alloc entry point differs from the regular one by {(out.float() - want.float()).abs().max().item()}"
        _against_oracle(c, out, Hq, Hkv, D, bs)


def _against_oracle(c, out, Hq, Hkv, D, bs):
    from onnxruntime_genai_b200.ops import reference as ref
    want = ref.paged_attention(c["q"].cpu(), c["kc"].cpu(), c["vc"].cpu(), c["cu"].cpu(), c["pl"].cpu(), c["table"].cpu(), bs, Hq, Hkv, D,
                               1 / math.sqrt(D))
    err = (out.float().cpu() - want.float()).abs().max().item()
    assert err <= 3e-2, f"no-alloc entry point differs from the fp32 reference by {err}"


@pytest.mark.parametrize("D,splits", [(64, 3), (96, 1), (128, 1)])
def test_noalloc_attention_other_head_dims_and_single_split(D, splits):
    """head_dim 64 / 96 and a call that needs no scratch at all (splits = 1), against the fp32 reference."""
    fn, need = _symbol()
    Hq, Hkv, bs = 8, 2, 16
    past = [300, 17, 1023]
    c = _case(7 + D, 3, past, Hq, Hkv, D, bs)
    out = torch.empty(3, Hq * D, dtype=torch.bfloat16, device="cuda")
    assert need(3, Hq, D, splits) == (0 if splits == 1 else splits * 3 * Hq * (D + 2) * 4)
    rc = fn(c["q"].data_ptr(), c["q"].stride(0), c["kc"].data_ptr(), c["vc"].data_ptr(), c["cu"].data_ptr(), c["pl"].data_ptr(),
            c["table"].data_ptr(), c["table"].stride(0), bs, out.data_ptr(), out.stride(0), None, 1 / math.sqrt(D), 0.0, 0, 3, 3, 1,
            Hq, Hkv, D, splits, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    _against_oracle(c, out, Hq, Hkv, D, bs)


def test_noalloc_attention_refuses_oversized_requests():
    fn, need = _symbol()
    Hq, D, splits, tokens = 64, 128, 16, 4096
    assert need(tokens, Hq, D, splits) > 8 << 20
    rc = fn(None, 0, None, None, None, None, None, 0, 16, None, 0, None, 1.0, 0.0, 0, 1, tokens, 1, Hq, 8, D, splits, None)
    assert rc == TOO_LARGE
