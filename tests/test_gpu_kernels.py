"""Each sm_100a kernel against the plain PyTorch fp32 restatement of the same op."""
import math

import numpy as np
import pytest
import torch

from onnxruntime_genai_b200 import ops
from onnxruntime_genai_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, std=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


def _close(a, b, rtol, atol):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (tol {tol.flatten()[err.argmax()].item():.4g}), mean err {err.mean().item():.4g}"


def test_library_loaded():
    from onnxruntime_genai_b200.ops import _lib
    assert _lib.lib() is not None
    ws = ops.workspace(torch.device("cuda", 0))
    assert ws.sm_count >= 100


# ------------------------------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (7, 256, 256), (64, 4096, 4096), (64, 6144, 4096), (33, 1000, 2880),
                                   (128, 512, 1024), (300, 384, 512), (1024, 2048, 1024), (16, 128256, 256)])
def test_gemm_matches_fp32(M, N, K):
    x = _rand(M, K, std=1.0, seed=1)
    w = _rand(N, K, std=0.05, seed=2)
    y = ops.linear(x, w)
    ops.check_kernel_status()
    want = ref.linear(x.cpu(), w.cpu())
    _close(y, want, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.05)


@pytest.mark.parametrize("splits", [1, 2, 3, 4, 5, 7, 8])
def test_gemm_split_k(splits):
    M, N, K = 48, 512, 2048
    x, w = _rand(M, K, seed=3), _rand(N, K, std=0.05, seed=4)
    y = ops.linear(x, w, splits=splits)
    ops.check_kernel_status()
    _close(y, ref.linear(x.cpu(), w.cpu()), rtol=2e-2, atol=0.05)
    y2 = ops.linear(x, w, splits=splits)
    assert torch.equal(y, y2), "split-K reduction must be deterministic and the tile counters self-cleaning"


def test_gemm_epilogues():
    M, N, K = 40, 768, 512
    x, w = _rand(M, K, seed=5), _rand(N, K, std=0.05, seed=6)
    bias, res = _rand(N, seed=7), _rand(M, N, seed=8)
    y = ops.linear(x, w, bias=bias, residual=res)
    _close(y, ref.linear(x.cpu(), w.cpu(), bias.cpu(), res.cpu()), rtol=2e-2, atol=0.05)
    y32 = ops.linear(x, w, out_fp32=True)
    assert y32.dtype == torch.float32
    _close(y32, ref.linear(x.cpu(), w.cpu(), out_fp32=True), rtol=1e-2, atol=0.02)
    ops.check_kernel_status()


@pytest.mark.parametrize("M,I,K,splits", [(5, 256, 256, 1), (64, 1024, 512, 1), (64, 1024, 2048, 4), (200, 384, 256, 1), (33, 128, 512, 3)])
def test_gemm_gate_up_silu(M, I, K, splits):
    x = _rand(M, K, seed=9)
    w = _rand(2 * I, K, std=0.05, seed=10)
    b = _rand(2 * I, std=0.5, seed=11)
    want = ref.gate_up_act(x.cpu(), w.cpu(), b.cpu())
    wi, bi = ops.interleave_gate_up(w), ops.interleave_gate_up(b)
    _close(ref.gate_up_act(x.cpu(), wi.cpu(), bi.cpu(), interleaved=True), want, rtol=1e-3, atol=1e-3)
    y = ops.gate_up_act(x, wi, bi, splits=splits, interleaved=True)
    ops.check_kernel_status()
    _close(y, want, rtol=3e-2, atol=0.05)
    # stacked (not interleaved) weights take the unfused route and must agree too
    _close(ops.gate_up_act(x, w, b), want, rtol=3e-2, atol=0.05)


@pytest.mark.parametrize("M,N,K,splits", [(64, 4096, 512, 0), (17, 256, 2048, 4), (130, 384, 256, 1)])
def test_gemm_fused_allreduce_world_of_one(M, N, K, splits):
    """The fused GEMM + all-reduce protocol (peer push, arrival counters, parity) with a single rank."""
    from onnxruntime_genai_b200.parallel.symm import LocalComm
    comm = LocalComm(torch.device("cuda", 0))
    try:
        x, w = _rand(M, K, seed=12), _rand(N, K, std=0.05, seed=13)
        res = _rand(M, N, seed=14)
        want = ref.linear(x.cpu(), w.cpu(), None, res.cpu())
        for _ in range(3):   # consecutive uses alternate the buffer parity and advance the counters
            y = ops.linear(x, w, residual=res, splits=splits, all_reduce=True)
            ops.check_kernel_status()
            _close(y, want, rtol=3e-2, atol=0.06)
            z = ops.linear(x, w, residual=res, splits=splits, reduce_scatter=(0, 1))   # scatter over one rank: every row stays
            _close(z, want, rtol=3e-2, atol=0.06)
    finally:
        comm.close()


def test_standalone_collectives_world_of_one():
    """all-reduce / all-gather / reduce-scatter kernels over the symmetric buffers with a single rank (push, stamp,
    wait, combine, epoch) interleaved with the fused GEMM on the same buffers."""
    from onnxruntime_genai_b200.parallel.symm import LocalComm
    comm = LocalComm(torch.device("cuda", 0))
    try:
        x = _rand(64, 4096, seed=21)
        r = _rand(64, 4096, seed=22)
        w = _rand(256, 4096, std=0.05, seed=23)
        for i in range(3):
            assert torch.equal(comm.all_reduce(x), x)
            _close(comm.all_reduce(x, residual=r), x.float() + r.float(), rtol=1e-2, atol=1e-2)
            y = ops.linear(x, w, all_reduce=True)     # same buffers, different slice-to-slot mapping
            assert torch.equal(comm.all_gather(x.float()), x.float()[None])
            assert torch.equal(comm.reduce_scatter(x[None].contiguous()), x)
            _close(y, ref.linear(x.cpu(), w.cpu()), rtol=3e-2, atol=0.06)
            small = _rand(8, seed=24 + i)
            assert torch.equal(comm.all_reduce(small), small)
        ops.check_kernel_status()
        assert not comm.fits(_rand(4096, 4096, seed=25))
    finally:
        comm.close()


@pytest.mark.parametrize("M,N,K,pair", [(64, 512, 1024, False), (5, 256, 4096, False), (200, 384, 512, False), (48, 512, 256, True)])
def test_gemm_all_gather_fused_world_of_one(M, N, K, pair):
    """all-gather -> GEMM: activations pushed as flagged lines, tiles assembled inside the GEMM (swizzled layout,
    row / k tails, split-K clusters), against the plain GEMM on the same data."""
    from onnxruntime_genai_b200.parallel.symm import LocalComm
    comm = LocalComm(torch.device("cuda", 0))
    try:
        x, w = _rand(M, K, seed=71), _rand(N, K, std=0.05, seed=72)
        if pair:
            w = ops.interleave_gate_up(w)
        for _ in range(3):
            comm.all_gather_push(x)
            y = ops.linear_gathered(M, w, act_pair=pair)
            want = ops.gate_up_act(x, w, interleaved=True) if pair else ops.linear(x, w)
            ops.check_kernel_status()
            assert torch.equal(y, want), f"max diff {(y.float() - want.float()).abs().max().item()}"
            assert torch.equal(comm.all_reduce(x), x)     # a waiting call between two pushes
    finally:
        comm.close()


def test_gemm_persistent_prefill_kernel():
    """Prefill-sized problems (at least one 128 x 256 tile per SM) take the persistent kernel with the double-buffered
    accumulator: several tiles per CTA, token and feature tails, every epilogue, against fp32."""
    x = _rand(1000, 512, seed=81)
    w, b, r = _rand(6144, 512, std=0.05, seed=82), _rand(6144, seed=83), _rand(1000, 6144, seed=84)
    _close(ops.linear(x, w, b, r), ref.linear(x.cpu(), w.cpu(), b.cpu(), r.cpu()), rtol=2e-2, atol=0.06)
    w2 = _rand(20000, 256, std=0.05, seed=85)          # 157 feature tiles with a tail, fp32 output (LM-head form)
    x2 = _rand(300, 256, seed=86)
    _close(ops.linear(x2, w2, out_fp32=True), ref.linear(x2.cpu(), w2.cpu(), out_fp32=True), rtol=1e-2, atol=0.03)
    w3, b3 = _rand(8192, 384, std=0.05, seed=87), _rand(8192, seed=88)     # gate/up pairs, 600 tokens: 64 x 3 tiles
    x3 = _rand(600, 384, seed=89)
    want = ref.gate_up_act(x3.cpu(), w3.cpu(), b3.cpu())
    _close(ops.gate_up_act(x3, ops.interleave_gate_up(w3), ops.interleave_gate_up(b3), interleaved=True), want, rtol=3e-2, atol=0.05)
    # many k-blocks per tile and many tiles per CTA
    x4, w4 = _rand(2048, 4096, seed=90), _rand(4096, 4096, std=0.02, seed=91)
    _close(ops.linear(x4, w4), ref.linear(x4.cpu(), w4.cpu()), rtol=2e-2, atol=0.08)
    ops.check_kernel_status()


def test_gemm_strided_activation():
    M, K, N = 20, 256, 256
    big = _rand(M, 3 * K, seed=11)
    x = big[:, K:2 * K]
    w = _rand(N, K, std=0.05, seed=12)
    _close(ops.linear(x, w), ref.linear(x.cpu(), w.cpu()), rtol=2e-2, atol=0.05)


# ------------------------------------------------------------------------------------------- decode-step fusions
@pytest.mark.parametrize("T,N,K,splits", [(1, 512, 256, 0), (5, 6144, 4096, 0), (64, 6144, 4096, 0), (64, 768, 4096, 0), (100, 1024, 512, 1),
                                           (64, 4096, 1792, 4), (33, 1000, 4100 // 8 * 8, 0), (300, 1024, 1024, 0)])
def test_gemm_with_folded_rms_norm(T, N, K, splits):
    """ops.linear(x, W * g, norm_eps=eps) against the fp32 definition linear(rmsnorm(x, g), W): the kernel sums the squares of
    every row from the activation tiles in shared memory (over the split-K cluster) and scales in the epilogue; steps beyond
    the decode tile sizes normalise with a unit-weight norm kernel first."""
    eps = 1e-5
    x, w, g = _rand(T, K, std=1.5, seed=201), _rand(N, K, std=0.03, seed=202), (1.0 + _rand(K, std=0.2, seed=203).float()).to(torch.bfloat16)
    b, r = _rand(N, seed=204), _rand(T, N, seed=205)
    wf = (w.float() * g.float()[None, :]).to(torch.bfloat16)
    xn = ref.norm(x.cpu(), g.cpu(), eps)[0]
    tol = dict(rtol=3e-2, atol=3e-2 * math.sqrt(K) * 0.03 + 0.03)
    _close(ops.linear(x, wf, norm_eps=eps, splits=splits), ref.linear(xn, w.cpu()), **tol)
    _close(ops.linear(x, wf, b, r, norm_eps=eps, splits=splits), ref.linear(xn, w.cpu(), b.cpu(), r.cpu()), **tol)
    y32 = ops.linear(x, wf, norm_eps=eps, out_fp32=True, splits=splits)
    _close(y32, ref.linear(xn, w.cpu(), out_fp32=True), **tol)
    # against the exact statement of what the kernel computes (folded weight, fp32 row scale): tight
    exact = (x.float().cpu() @ wf.float().cpu().t()) * torch.rsqrt((x.float().cpu() ** 2).mean(-1, keepdim=True) + eps)
    if T <= ops.FUSED_MAX_TOKENS:     # larger steps round the normalised rows to bf16 first
        _close(y32, exact, rtol=2e-3, atol=2e-3 * math.sqrt(K) * 0.03 + 1e-3)
    if N % 128 == 0:
        wi, bi = ops.interleave_gate_up(wf), ops.interleave_gate_up(b)
        _close(ops.gate_up_act(x, wi, bi, interleaved=True, norm_eps=eps, splits=splits), ref.gate_up_act(xn, w.cpu(), b.cpu()), rtol=4e-2, atol=0.08)
    ops.check_kernel_status()


@pytest.mark.parametrize("T,Hq,Hkv,D,rot,K,bias,eps", [(64, 32, 8, 128, 128, 4096, False, 1e-5), (7, 4, 1, 128, 128, 4096, True, 0.0),
                                                        (33, 8, 2, 64, 64, 512, True, 1e-5), (1, 16, 2, 128, 64, 1024, False, 1e-6),
                                                        (128, 6, 2, 32, 32, 256, False, 1e-5), (16, 4, 4, 128, 0, 256, True, 0.0)])
def test_qkv_projection_with_fused_rope_and_cache_append(T, Hq, Hkv, D, rot, K, bias, eps):
    """One kernel (GEMM + rotary embedding + KV-cache append, optionally + folded norm) against the fp32 restatement of the
    three separate steps: rotated queries, and the cache rows at every token's slot (negative slots store nothing)."""
    N = (Hq + 2 * Hkv) * D
    x, w = _rand(T, K, std=1.0, seed=211), _rand(N, K, std=0.04, seed=212)
    b = _rand(N, std=0.5, seed=213) if bias else None
    max_pos = 300
    pos = torch.randint(0, max_pos, (T,), generator=torch.Generator().manual_seed(1), dtype=torch.int32)
    slots = torch.randperm(T + 9, generator=torch.Generator().manual_seed(2))[:T].to(torch.int32)
    if T > 3:
        slots[2] = -1
    half = max(rot // 2, 1)
    ang = torch.arange(max_pos)[:, None].float() * (1.0 / (10000 ** (torch.arange(half).float() / half)))[None, :]
    cos, sin = (torch.cos(ang), torch.sin(ang)) if rot else (None, None)
    kc_ref, vc_ref = torch.zeros(T + 9, Hkv, D), torch.zeros(T + 9, Hkv, D)
    xn = ref.rms_scale(x.cpu(), eps) if eps > 0 else x.cpu()
    qkv_ref = ref.linear(xn, w.cpu(), b.cpu() if bias else None, out_fp32=True)
    ref.rope_kv_append(qkv_ref, pos, slots, cos, sin, kc_ref, vc_ref, Hq, Hkv, D, rot)
    kc, vc = torch.zeros(T + 9, Hkv, D, dtype=torch.bfloat16, device=DEV), torch.zeros(T + 9, Hkv, D, dtype=torch.bfloat16, device=DEV)
    q = ops.qkv_rope_append(x, w, b, pos.to(DEV), slots.to(DEV), cos.to(DEV) if rot else None, sin.to(DEV) if rot else None, kc, vc,
                            Hq, Hkv, D, rot, norm_eps=eps)
    assert q.shape == (T, Hq * D), "the fused kernel writes the query columns only"
    tol = dict(rtol=3e-2, atol=3e-2 * math.sqrt(K) * 0.04 + 0.03)
    _close(q, qkv_ref[:, :Hq * D], **tol)
    _close(kc, kc_ref, **tol)
    _close(vc, vc_ref, **tol)
    ops.check_kernel_status()


# ------------------------------------------------------------------------------------------- norm / rope / misc
@pytest.mark.parametrize("H", [256, 3072, 4096, 8192])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(H, with_res):
    x, w = _rand(9, H, seed=13), _rand(H, seed=14)
    res = _rand(9, H, seed=15) if with_res else None
    res_ref = res.cpu().clone() if with_res else None
    y, r = ops.norm(x, w, 1e-5, res)
    yr, rr = ref.norm(x.cpu(), w.cpu(), 1e-5, res_ref)
    _close(y, yr, rtol=2e-2, atol=2e-2)
    if with_res:
        _close(r, rr, rtol=1e-2, atol=1e-2)


def test_layernorm_bias():
    H = 2560
    x, w, b = _rand(5, H, seed=16), _rand(H, seed=17), _rand(H, seed=18)
    y, _ = ops.norm(x, w, 1e-5, None, b, layernorm=True)
    yr, _ = ref.norm(x.cpu(), w.cpu(), 1e-5, None, b.cpu(), layernorm=True)
    _close(y, yr, rtol=2e-2, atol=3e-2)


@pytest.mark.parametrize("D,rot,inter,qk_norm", [(128, 128, False, False), (64, 64, False, True), (96, 96, False, False),
                                                   (128, 64, True, False), (64, 32, False, False)])
def test_rope_kv_append(D, rot, inter, qk_norm):
    T, Hq, Hkv, slots_n = 11, 8, 2, 64
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=19)
    pos = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    slots = torch.randperm(slots_n)[:T].to(torch.int32).to(DEV)
    slots[2] = -1
    freqs = torch.outer(torch.arange(64).float(), 1.0 / (10000 ** (torch.arange(0, rot, 2).float() / rot)))
    cos, sin = freqs.cos().to(DEV), freqs.sin().to(DEV)
    kc, vc = torch.zeros(slots_n, Hkv, D, dtype=torch.bfloat16, device=DEV), torch.zeros(slots_n, Hkv, D, dtype=torch.bfloat16, device=DEV)
    qn = _rand(D, seed=20) if qk_norm else None
    kn = _rand(D, seed=21) if qk_norm else None
    q2, kc2, vc2 = qkv.cpu().clone(), kc.cpu().clone(), vc.cpu().clone()
    ops.rope_kv_append(qkv, pos, slots, cos, sin, kc, vc, Hq, Hkv, D, rot, inter, qn, kn, 1e-6)
    ref.rope_kv_append(q2, pos.cpu(), slots.cpu(), cos.cpu(), sin.cpu(), kc2, vc2, Hq, Hkv, D, rot, inter,
                       qn.cpu() if qk_norm else None, kn.cpu() if qk_norm else None, 1e-6)
    _close(qkv[:, :Hq * D], q2[:, :Hq * D], rtol=2e-2, atol=3e-2)
    _close(kc, kc2, rtol=2e-2, atol=3e-2)
    _close(vc, vc2, rtol=0, atol=0)


@pytest.mark.parametrize("interleaved_sections", [False, True])
@pytest.mark.parametrize("kv8", [False, True])
def test_rope_multimodal_positions(kv8, interleaved_sections):
    """Three position components per token, rotary pairs split into sections (Qwen2-VL) or alternating t h w (Qwen3-VL); bf16 and int8 caches."""
    T, Hq, Hkv, D, slots_n = 9, 4, 2, 128, 32
    qkv = _rand(T, (Hq + 2 * Hkv) * D, seed=29)
    rng = np.random.RandomState(1)
    p3 = torch.from_numpy(rng.randint(0, 60, size=(3, T)).astype(np.int32))
    pos = torch.arange(T, dtype=torch.int32)
    slots = torch.randperm(slots_n)[:T].to(torch.int32)
    freqs = torch.outer(torch.arange(64).float(), 1.0 / (10000 ** (torch.arange(0, D, 2).float() / D)))
    cos, sin = freqs.cos(), freqs.sin()
    row = D + 16 if kv8 else D
    dt = torch.int8 if kv8 else torch.bfloat16
    kc, vc = torch.zeros(slots_n, Hkv, row, dtype=dt, device=DEV), torch.zeros(slots_n, Hkv, row, dtype=dt, device=DEV)
    q2, kc2, vc2 = qkv.cpu().clone(), kc.cpu().clone(), vc.cpu().clone()
    sec = [16, 24, 24]
    il = interleaved_sections
    ops.rope_kv_append(qkv, pos.to(DEV), slots.to(DEV), cos.to(DEV), sin.to(DEV), kc, vc, Hq, Hkv, D, D, False, None, None, 1e-6, p3.to(DEV), sec, il)
    ref.rope_kv_append(q2, pos, slots, cos, sin, kc2, vc2, Hq, Hkv, D, D, False, None, None, 1e-6, p3, sec, il)
    if il:
        other = qkv.cpu().clone().copy_(_rand(T, (Hq + 2 * Hkv) * D, seed=29).cpu())
        ref.rope_kv_append(other, pos, None, cos, sin, None, None, Hq, Hkv, D, D, False, None, None, 1e-6, p3, sec, False)
        assert (other[:, :Hq * D].float() - q2[:, :Hq * D].float()).abs().max() > 0.05   # the two layouts really differ
    _close(qkv[:, :Hq * D], q2[:, :Hq * D], rtol=2e-2, atol=3e-2)
    if kv8:
        _close(ref.kv8_load(kc.cpu(), Hkv, D), ref.kv8_load(kc2, Hkv, D), rtol=3e-2, atol=3e-2)
    else:
        _close(kc, kc2, rtol=2e-2, atol=3e-2)
    plain = q2.clone()
    ref.rope_kv_append(plain.copy_(_rand(T, (Hq + 2 * Hkv) * D, seed=29).cpu()), pos, None, cos, sin, None, None, Hq, Hkv, D, D)
    assert (plain[:, :Hq * D].float() - q2[:, :Hq * D].float()).abs().max() > 0.05      # the components really differ


def test_embedding_gather_actmul_cast():
    table = _rand(1000, 512, seed=22)
    ids = torch.tensor([0, 5, 999, 17], dtype=torch.int32, device=DEV)
    assert torch.equal(ops.embedding(ids, table), table[ids.long()])
    _close(ops.embedding(ids, table, 3.0), ref.embedding(ids.cpu(), table.cpu(), 3.0), rtol=1e-2, atol=1e-2)
    x = _rand(6, 512, seed=23)
    assert torch.equal(ops.gather_rows(x, torch.tensor([5, 0, 3], dtype=torch.int32, device=DEV)), x[[5, 0, 3]])
    _close(ops.act_mul(x), ref.act_mul(x.cpu()), rtol=2e-2, atol=2e-2)
    _close(ops.act_mul(x, "gelu"), ref.act_mul(x.cpu(), "gelu"), rtol=2e-2, atol=2e-2)
    for act in ("silu", "gelu", "relu", "gelu_erf"):
        _close(ops.activation(x * 4, act), ref.activation((x * 4).cpu().float(), act), rtol=1e-2, atol=1e-2)
    assert torch.equal(ops.to_float32(x), x.float())


@pytest.mark.parametrize("sym", [False, True])
def test_embedding_q4_gather_matches_dequantised_rows(sym):
    from onnxruntime_genai_b200.models.builder import quantize_int4_block32
    from onnxruntime_genai_b200.ops.w4 import QuantizedEmbedding
    V, K = 777, 320
    w = torch.randn(V, K, generator=torch.Generator().manual_seed(3)) * 0.1
    q, s, zp = quantize_int4_block32(w, symmetric=sym)
    qe = QuantizedEmbedding(q.reshape(V, -1).to(DEV), s.to(torch.float16).view(V, -1).to(DEV), zp.reshape(V, -1).to(DEV) if zp is not None else None, V, K)
    ids = torch.tensor([0, 5, 776, 17, 5, 900], dtype=torch.int32, device=DEV)     # the last id is clamped
    table = qe.dequantize()
    want = table[ids.long().clamp(max=V - 1)]
    assert torch.equal(ops.embedding(ids, qe).float(), want)
    _close(ops.embedding(ids, qe, 3.0), want * 3.0, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("L,bias", [(3, False), (4, True)])
def test_short_conv_matches_reference(L, bias):
    """Prefill chunks, single-token rows and a chunk continuing a cached prefix in one packed launch; the paged cache after
    the launch must hold b * x of the new positions."""
    rng = np.random.RandomState(5)
    C, bs = 256, 16
    q_lens, past = [19, 1, 5, 1], [0, 37, 14, 2]
    B, T = len(q_lens), sum(q_lens)
    cols = max((p_ + q_ + bs - 1) // bs for p_, q_ in zip(past, q_lens))
    perm = rng.permutation(B * cols + 2)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    used = 0
    for b in range(B):
        need = (past[b] + q_lens[b] + bs - 1) // bs
        table[b, :need] = torch.from_numpy(perm[used:used + need].astype(np.int32))
        used += need
    cache = _rand((B * cols + 2) * bs, C, std=1.0, seed=40)
    bcx = _rand(T, 3 * C, std=1.0, seed=41)
    w = _rand(C, L, std=0.5, seed=42)
    bvec = _rand(C, std=0.5, seed=43) if bias else None
    pos, slots = [], []
    for b in range(B):
        for j in range(q_lens[b]):
            p_ = past[b] + j
            pos.append(p_)
            slots.append(int(table[b, p_ // bs]) * bs + p_ % bs)
    pos, slots = torch.tensor(pos, dtype=torch.int32), torch.tensor(slots, dtype=torch.int32)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    c_cpu = cache.cpu().clone()
    want = ref.short_conv(bcx.cpu(), w.cpu(), bvec.cpu() if bias else None, c_cpu, slots, pos, cu, pl, table, bs)
    got = ops.short_conv(bcx, w, bvec, cache, slots.to(DEV), pos.to(DEV), cu.to(DEV), pl.to(DEV), table.to(DEV), bs)
    _close(got, want, rtol=3e-2, atol=3e-2)
    assert torch.equal(cache.cpu(), c_cpu)


@pytest.mark.parametrize("bias", [False, True])
def test_causal_conv_plain_mode_matches_the_gated_form_with_unit_gates(bias):
    """The convolution of the recurrent layer kinds: x is a column slice of a wider projection, no gates, SiLU on the output; the same
    packed launch shapes as the gated test, against the CPU restatement fed with unit gates."""
    rng = np.random.RandomState(6)
    C, bs, L = 192, 16, 4
    q_lens, past = [19, 1, 5, 1], [0, 37, 14, 2]
    B, T = len(q_lens), sum(q_lens)
    cols = max((p_ + q_ + bs - 1) // bs for p_, q_ in zip(past, q_lens))
    perm = rng.permutation(B * cols + 2)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    used = 0
    for b in range(B):
        need = (past[b] + q_lens[b] + bs - 1) // bs
        table[b, :need] = torch.from_numpy(perm[used:used + need].astype(np.int32))
        used += need
    cache = _rand((B * cols + 2) * bs, C, std=1.0, seed=50)
    wide = _rand(T, 64 + C + 40, std=1.0, seed=51)
    x = wide[:, 64:64 + C]                       # 128-byte offset, row stride of the wider tensor
    w = _rand(C, L, std=0.5, seed=52)
    bvec = _rand(C, std=0.5, seed=53) if bias else None
    pos, slots = [], []
    for b in range(B):
        for j in range(q_lens[b]):
            p_ = past[b] + j
            pos.append(p_)
            slots.append(int(table[b, p_ // bs]) * bs + p_ % bs)
    pos, slots = torch.tensor(pos, dtype=torch.int32), torch.tensor(slots, dtype=torch.int32)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    c_cpu = cache.cpu().clone()
    xc = x.cpu().contiguous()
    ones = torch.ones_like(xc)
    want = ref.short_conv(torch.cat([ones, ones, xc], 1), w.cpu(), bvec.cpu() if bias else None, c_cpu, slots, pos, cu, pl, table, bs)
    want = torch.nn.functional.silu(want.float())
    got = ops.causal_conv(x, w, bvec, cache, slots.to(DEV), pos.to(DEV), cu.to(DEV), pl.to(DEV), table.to(DEV), bs, silu=True)
    _close(got, want.to(torch.bfloat16), rtol=3e-2, atol=3e-2)
    assert torch.equal(cache.cpu(), c_cpu)


def test_gated_delta_layer_matches_the_tensor_form():
    """ops.gated_delta_layer (normalisation, gates, recurrence, gated output norm in two kernels) against the same arithmetic written
    with tensor operations around the plain recurrence restatement."""
    torch.manual_seed(3)
    Hk, Hv, dk, dv = 2, 4, 64, 64
    kd, vd = Hk * dk, Hv * dv
    cd = 2 * kd + vd
    lens, past = [9, 1, 1, 21], [0, 5, 1, 16]
    T = sum(lens)
    conv = torch.nn.functional.silu(torch.randn(T, cd, device=DEV)).to(torch.bfloat16)
    proj = torch.randn(T, cd + vd + 2 * Hv, device=DEV).to(torch.bfloat16)
    neg_exp_a = -(torch.rand(Hv, device=DEV) * 2 + 0.1)
    dt_bias = torch.randn(Hv, device=DEV) * 0.5
    norm_w = 1 + 0.1 * torch.randn(dv, device=DEV)
    state = torch.randn(6, Hv, dk, dv, device=DEV) * 0.1
    slots = torch.tensor([4, 1, 5, 0], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    pl = torch.tensor(past, dtype=torch.int32, device=DEV)
    st_ref = state.clone().cpu()
    c, pr = conv.float().cpu(), proj.float().cpu()
    q = torch.nn.functional.normalize(c[:, :kd].view(T, Hk, dk), dim=-1, eps=1e-6) * dk ** -0.5
    k = torch.nn.functional.normalize(c[:, kd:2 * kd].view(T, Hk, dk), dim=-1, eps=1e-6)
    v = c[:, 2 * kd:].view(T, Hv, dv)
    z, b_, a_ = pr[:, cd:cd + vd], pr[:, cd + vd:cd + vd + Hv], pr[:, cd + vd + Hv:]
    g = neg_exp_a.cpu() * torch.nn.functional.softplus(a_ + dt_bias.cpu())
    o = ref.gated_delta(q, k, v, g, torch.sigmoid(b_), st_ref, slots.cpu(), cu.cpu(), pl.cpu()).float()
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.cpu()
    want = o.view(T, vd) * torch.nn.functional.silu(z)
    got = ops.gated_delta_layer(conv, proj, cd, vd, Hk, Hv, dk, dv, neg_exp_a, dt_bias, norm_w, 1e-6, state, slots, cu, pl)
    _close(got, want.to(torch.bfloat16), rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(state.cpu(), st_ref, rtol=2e-3, atol=2e-3)


def test_mamba2_layer_matches_the_tensor_form():
    """ops.mamba2_layer (step sizes, scan over column ranges of the convolved projection, gated norm over the whole width) against the
    same arithmetic written with tensor operations around the plain scan restatement."""
    torch.manual_seed(4)
    heads, groups, P, N = 8, 2, 32, 64
    I, GN = heads * P, groups * N
    cd = I + 2 * GN
    lens, past = [9, 1, 1, 21], [0, 5, 1, 16]
    T = sum(lens)
    conv = torch.nn.functional.silu(torch.randn(T, cd, device=DEV)).to(torch.bfloat16)
    proj = torch.randn(T, I + cd + heads, device=DEV).to(torch.bfloat16)
    dt_bias = torch.randn(heads, device=DEV) * 0.5
    neg_a = -(torch.rand(heads, device=DEV) * 2 + 0.1)
    Dv = torch.randn(heads, device=DEV)
    norm_w = 1 + 0.1 * torch.randn(I, device=DEV)
    state = torch.randn(6, heads, N, P, device=DEV) * 0.1
    slots = torch.tensor([4, 1, 5, 0], dtype=torch.int32, device=DEV)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device=DEV)
    pl = torch.tensor(past, dtype=torch.int32, device=DEV)
    st_ref = state.clone().cpu()
    c, pr = conv.float().cpu(), proj.float().cpu()
    step = torch.nn.functional.softplus(pr[:, I + cd:] + dt_bias.cpu())
    y = ref.mamba2_scan(c[:, :I].reshape(T, heads, P), step, neg_a.cpu(), c[:, I:I + GN].reshape(T, groups, N), c[:, I + GN:].reshape(T, groups, N),
                        Dv.cpu(), st_ref, slots.cpu(), cu.cpu(), pl.cpu()).float().view(T, I)
    y = y * torch.nn.functional.silu(pr[:, :I])
    want = y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + 1e-5) * norm_w.cpu()
    got = ops.mamba2_layer(conv, proj, heads, groups, P, N, dt_bias, neg_a, Dv, norm_w, 1e-5, state, slots, cu, pl)
    _close(got, want.to(torch.bfloat16), rtol=4e-2, atol=4e-2)
    torch.testing.assert_close(state.cpu(), st_ref, rtol=2e-3, atol=2e-3)


def test_decode_advance_matches_reference():
    rng = np.random.RandomState(3)
    B, cols, bs = 37, 9, 16
    table = torch.from_numpy(rng.randint(0, 500, size=(B, cols)).astype(np.int32))
    table[::5, 6:] = -1
    pos = torch.from_numpy(rng.randint(0, cols * bs - 1, size=(B,)).astype(np.int32))
    fields = [torch.from_numpy(rng.randint(0, 1000, size=(B,)).astype(np.int32)) for _ in range(4)]   # ids, past, slots, sample_pos
    sampled = torch.from_numpy(rng.randint(0, 32000, size=(B,)).astype(np.int32))
    cpu = [f.clone() for f in (fields[0], pos, fields[1], fields[2], fields[3])]
    gpu = [f.clone().to(DEV) for f in (fields[0], pos, fields[1], fields[2], fields[3])]
    ops.decode_advance(sampled, *cpu, table, bs)
    big = torch.full((64, cols + 3), -7, dtype=torch.int32, device=DEV)      # a strided view, as in the engine's staging buffer
    big[:B, :cols] = table.to(DEV)
    ops.decode_advance(sampled.to(DEV), *gpu, big[:B, :cols], bs)
    for a, b in zip(cpu, gpu):
        assert torch.equal(a, b.cpu())


# ------------------------------------------------------------------------------------------- attention
def _attention_case(B, q_lens, past, Hq, Hkv, D, bs, window=0, sinks=False, softcap=0.0, splits=None, seed=30, order=False):
    rng = np.random.RandomState(seed)
    T = sum(q_lens)
    cols = max((p + q + bs - 1) // bs for p, q in zip(past, q_lens))
    nblocks = B * cols + 3
    perm = rng.permutation(nblocks)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    k_cache = _rand(nblocks * bs, Hkv, D, std=1.0, seed=seed + 1)
    v_cache = _rand(nblocks * bs, Hkv, D, std=1.0, seed=seed + 2)
    used = 0
    for b in range(B):
        need = (past[b] + q_lens[b] + bs - 1) // bs
        table[b, :need] = torch.from_numpy(perm[used:used + need].astype(np.int32))
        used += need
    q = _rand(T, (Hq + 2 * Hkv) * D, std=1.0, seed=seed + 3)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    sk = (torch.randn(Hq, generator=torch.Generator().manual_seed(seed)) * 2).float() if sinks else None
    scale = 1.0 / math.sqrt(D)
    out = ops.paged_attention(q, k_cache, v_cache, cu.to(DEV), pl.to(DEV), table.to(DEV), bs, Hq, Hkv, D, scale, window,
                              sk.to(DEV) if sinks else None, softcap, max_q_len=max(q_lens), max_kv_len=max(p + q for p, q in zip(past, q_lens)),
                              splits=splits, order=torch.argsort(-pl.long(), stable=True).to(torch.int32).to(DEV) if order else None)
    want = ref.paged_attention(q.cpu(), k_cache.cpu(), v_cache.cpu(), cu, pl, table, bs, Hq, Hkv, D, scale, window, sk, softcap)
    _close(out, want, rtol=3e-2, atol=3e-2)


def test_attention_tcgen05_prefill_kernel():
    """Requests with at least 128 query rows run on the tcgen05 kernel (S, P and O in tensor memory, P V with its A operand read
    from tensor memory, V as an MN-major operand); the short requests of the same call stay on the other kernel."""
    assert ops.TC_ATTENTION_MIN_ROWS == 128
    n0 = ops._lib.LAUNCH_COUNT
    _attention_case(B=1, q_lens=[256], past=[0], Hq=8, Hkv=2, D=128, bs=16)                       # causal, 8 row tiles, diagonal masks
    assert ops._lib.LAUNCH_COUNT - n0 == 2      # the launch for short requests (all of its CTAs leave at once) + the tensor-core launch
    _attention_case(B=2, q_lens=[300, 50], past=[100, 700], Hq=8, Hkv=2, D=128, bs=16)            # cached prefixes, a partial row tile
    _attention_case(B=3, q_lens=[20, 200, 1], past=[64, 0, 333], Hq=8, Hkv=2, D=128, bs=16)       # short requests beside a long one
    _attention_case(B=1, q_lens=[200], past=[37], Hq=8, Hkv=8, D=64, bs=16)                       # head_dim 64, no grouping
    _attention_case(B=1, q_lens=[400], past=[300], Hq=8, Hkv=2, D=128, bs=16, window=128, sinks=True)
    _attention_case(B=1, q_lens=[130], past=[0], Hq=8, Hkv=2, D=128, bs=16, softcap=30.0)
    _attention_case(B=2, q_lens=[70, 200], past=[70, 200], Hq=8, Hkv=8, D=64, bs=16, window=-1)   # bidirectional over cached keys
    _attention_case(B=1, q_lens=[256], past=[31], Hq=8, Hkv=2, D=128, bs=32)                      # 32-token cache blocks
    _attention_case(B=1, q_lens=[1100], past=[0], Hq=4, Hkv=1, D=128, bs=16)                      # more tiles than S buffers and K/V stages
    _attention_case(B=2, q_lens=[150, 160], past=[2000, 5], Hq=32, Hkv=8, D=128, bs=16, splits=3, order=True)
    ops.check_kernel_status()


@pytest.mark.parametrize("splits", [None, 3])
def test_attention_bidirectional_over_cached_keys(splits):
    """window < 0: every query sees exactly the `past` cached keys (encoder self-attention after its keys were appended,
    cross-attention over encoder keys) - prefill-sized and single-query rows."""
    _attention_case(B=3, q_lens=[70, 9, 33], past=[70, 150, 1500], Hq=8, Hkv=8, D=64, bs=16, window=-1, splits=splits)
    _attention_case(B=4, q_lens=[1] * 4, past=[1, 64, 333, 1500], Hq=12, Hkv=12, D=64, bs=16, window=-1, splits=splits)
    _attention_case(B=2, q_lens=[40, 17], past=[40, 17], Hq=8, Hkv=2, D=128, bs=16, window=-1, splits=splits)


def _attention_case_kv8(B, q_lens, past, Hq, Hkv, D, bs, splits=None, seed=50, window=0):
    """The same problem over an 8-bit cache filled by the append kernel: compared with the reference attention over the
    reference's own quantised cache (bit-identical rows are not required, close outputs are)."""
    rng = np.random.RandomState(seed)
    cols = max((p + q + bs - 1) // bs for p, q in zip(past, q_lens))
    nblocks = B * cols + 3
    perm = rng.permutation(nblocks)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    used = 0
    for b in range(B):
        need = (past[b] + q_lens[b] + bs - 1) // bs
        table[b, :need] = torch.from_numpy(perm[used:used + need].astype(np.int32))
        used += need
    kc_g = torch.zeros(nblocks * bs, Hkv, D + 16, dtype=torch.int8, device=DEV)
    vc_g = torch.zeros_like(kc_g)
    kc_c, vc_c = kc_g.cpu().clone(), vc_g.cpu().clone()
    # fill every request's cached prefix and this step's tokens through the append path (rot = 0: plain append)
    for b in range(B):
        n = past[b] + q_lens[b]
        rows = _rand(n, 2 * Hkv * D, std=1.0, seed=seed + 10 + b)
        pos = torch.arange(n, dtype=torch.int32)
        slots = (table[b, (pos // bs).long()] * bs + pos % bs).to(torch.int32)
        ops.rope_kv_append(rows.clone(), pos.to(DEV), slots.to(DEV), None, None, kc_g, vc_g, 0, Hkv, D, 0)
        ref.rope_kv_append(rows.cpu().clone(), pos, slots, None, None, kc_c, vc_c, 0, Hkv, D, 0)
    # the two append paths agree on the stored rows (scales equal, values within one step)
    d = (kc_g.cpu()[..., :D].int() - kc_c[..., :D].int()).abs().max()
    assert d <= 1 and torch.equal(kc_g.cpu()[..., D:D + 4], kc_c[..., D:D + 4])
    T = sum(q_lens)
    q = _rand(T, Hq * D, std=1.0, seed=seed + 3)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    out = ops.paged_attention(q, kc_g, vc_g, cu.to(DEV), pl.to(DEV), table.to(DEV), bs, Hq, Hkv, D, scale, window,
                              max_q_len=max(q_lens), max_kv_len=max(p + q_ for p, q_ in zip(past, q_lens)), splits=splits)
    want = ref.paged_attention(q.cpu(), kc_g.cpu(), vc_g.cpu(), cu, pl, table, bs, Hq, Hkv, D, scale, window)
    _close(out, want, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("D", [64, 96, 128])
def test_attention_int8_cache(D):
    _attention_case_kv8(B=4, q_lens=[1] * 4, past=[0, 15, 200, 1023], Hq=8, Hkv=2, D=D, bs=16)           # decode mode
    _attention_case_kv8(B=3, q_lens=[70, 1, 9], past=[0, 130, 64], Hq=8, Hkv=2, D=D, bs=16)               # prefill / mixed rows
    _attention_case_kv8(B=2, q_lens=[1, 1], past=[700, 2047], Hq=32, Hkv=8, D=D, bs=16, splits=(8, 256))  # split keys
    _attention_case_kv8(B=2, q_lens=[1, 30], past=[500, 100], Hq=8, Hkv=2, D=D, bs=16, window=128)


def test_attention_mixed_step_as_two_launches():
    """Single-token requests first, prompt chunks after: the decoder runs them as a decode-tile launch (with its own split
    choice and a scratch sized for the leading rows only) and a 64-row-tile launch writing into one output."""
    rng = np.random.RandomState(7)
    q_lens, past = [1, 1, 1, 40, 17], [900, 5, 2047, 0, 64]
    B, nd, Hq, Hkv, D, bs = 5, 3, 8, 2, 128, 16
    cols = max((p_ + q_ + bs - 1) // bs for p_, q_ in zip(past, q_lens))
    nblocks = B * cols + 3
    perm = rng.permutation(nblocks)
    table = torch.full((B, cols), -1, dtype=torch.int32)
    used = 0
    for b in range(B):
        need = (past[b] + q_lens[b] + bs - 1) // bs
        table[b, :need] = torch.from_numpy(perm[used:used + need].astype(np.int32))
        used += need
    kc, vc = _rand(nblocks * bs, Hkv, D, std=1.0, seed=61), _rand(nblocks * bs, Hkv, D, std=1.0, seed=62)
    T = sum(q_lens)
    q = _rand(T, (Hq + 2 * Hkv) * D, std=1.0, seed=63)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    pl = torch.tensor(past, dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    cu_d, pl_d, tb_d = cu.to(DEV), pl.to(DEV), table.to(DEV)
    out = torch.zeros(T, Hq * D, dtype=torch.bfloat16, device=DEV)
    ops.paged_attention(q, kc, vc, cu_d[:nd + 1], pl_d[:nd], tb_d[:nd], bs, Hq, Hkv, D, scale, max_q_len=1, max_kv_len=2048, out=out,
                        total_tokens=nd)
    ops.paged_attention(q, kc, vc, cu_d[nd:], pl_d[nd:], tb_d[nd:], bs, Hq, Hkv, D, scale, max_q_len=40, max_kv_len=2048, out=out)
    want = ref.paged_attention(q.cpu(), kc.cpu(), vc.cpu(), cu, pl, table, bs, Hq, Hkv, D, scale)
    _close(out, want, rtol=3e-2, atol=3e-2)
    assert ops.choose_kv_splits(nd, Hkv, 1, 2048, group=Hq // Hkv)[0] > 1      # the leading launch really used the split path


@pytest.mark.parametrize("splits", [None, 3])
def test_attention_longest_first_issue_order(splits):
    """A permutation of the requests only changes which CTA serves which request."""
    _attention_case(B=7, q_lens=[1] * 7, past=[5, 900, 64, 2047, 130, 0, 333], Hq=32, Hkv=8, D=128, bs=16, splits=splits, order=True)
    _attention_case(B=3, q_lens=[33, 1, 8], past=[0, 700, 40], Hq=8, Hkv=2, D=64, bs=16, splits=splits, order=True)


@pytest.mark.parametrize("D", [64, 96, 128])
def test_attention_decode(D):
    _attention_case(B=5, q_lens=[1] * 5, past=[0, 15, 16, 200, 1023], Hq=8, Hkv=2, D=D, bs=16)


@pytest.mark.parametrize("splits", [2, 4, 7])
def test_attention_decode_split_kv(splits):
    _attention_case(B=3, q_lens=[1, 1, 1], past=[5, 700, 2047], Hq=32, Hkv=8, D=128, bs=16, splits=splits)


@pytest.mark.parametrize("splits", [(8, 256), (5, 512), (33, 64), (3, 128)])
def test_attention_decode_fixed_chunks(splits):
    """Fixed key ranges per split: short requests leave most splits empty, long ones may end inside a chunk, and a
    chunk count that does not cover the longest request must still be refused by nobody (the last chunk is clipped)."""
    _attention_case(B=4, q_lens=[1, 1, 1, 1], past=[5, 700, 2047, 255], Hq=32, Hkv=8, D=128, bs=16, splits=splits)
    _attention_case(B=3, q_lens=[1, 2, 1], past=[300, 64, 1], Hq=8, Hkv=2, D=64, bs=16, window=128, sinks=True, splits=splits)


def test_attention_prefill_and_mixed():
    _attention_case(B=3, q_lens=[70, 1, 33], past=[0, 90, 17], Hq=8, Hkv=2, D=128, bs=16)
    _attention_case(B=2, q_lens=[257, 5], past=[0, 300], Hq=4, Hkv=4, D=64, bs=256)


def test_attention_mha_and_wide_group():
    _attention_case(B=2, q_lens=[20, 1], past=[3, 50], Hq=4, Hkv=4, D=96, bs=16)
    _attention_case(B=2, q_lens=[9, 1], past=[40, 333], Hq=16, Hkv=2, D=64, bs=16)


def test_attention_decode_mode_shapes():
    # decode mode = at most 16 (token, head) rows per kv head: full 16-wide group, multi-token verify rows, MHA
    _attention_case(B=3, q_lens=[1, 1, 1], past=[0, 63, 64], Hq=32, Hkv=2, D=128, bs=16)
    _attention_case(B=3, q_lens=[3, 4, 1], past=[10, 200, 65], Hq=8, Hkv=2, D=64, bs=16)
    _attention_case(B=2, q_lens=[1, 1], past=[129, 1], Hq=4, Hkv=4, D=96, bs=16, splits=2)
    _attention_case(B=4, q_lens=[1] * 4, past=[1500, 31, 32, 700], Hq=32, Hkv=8, D=128, bs=16, splits=3)


def test_attention_window_sinks_softcap():
    _attention_case(B=3, q_lens=[1, 1, 40], past=[500, 30, 100], Hq=8, Hkv=2, D=64, bs=16, window=128, sinks=True)
    _attention_case(B=2, q_lens=[1, 1], past=[500, 130], Hq=8, Hkv=2, D=64, bs=16, window=128, sinks=True, splits=3)
    _attention_case(B=2, q_lens=[1, 19], past=[77, 0], Hq=8, Hkv=4, D=128, bs=16, softcap=30.0)


# ------------------------------------------------------------------------------------------- sampling
def test_argmax_and_greedy_rows():
    x = _rand(7, 32000, dtype=torch.float32, seed=40)
    want = x.argmax(-1).to(torch.int32)
    assert torch.equal(ops.argmax(x), want)
    ones = torch.ones(7, dtype=torch.int32, device=DEV)
    f = torch.ones(7, dtype=torch.float32, device=DEV)
    z = torch.zeros(7, dtype=torch.int64, device=DEV)
    assert torch.equal(ops.sample(x, ones, f, f, z, ones), want)


def test_sampling_distribution_matches_reference():
    """Empirical token frequencies of the device sampler vs the exact truncated distribution."""
    V, n = 512, 20000
    g = torch.Generator().manual_seed(41)
    row = (torch.randn(V, generator=g) * 2.5).float()
    for k, p, t in [(50, 0.9, 0.7), (8, 1.0, 1.0), (0, 0.8, 1.3), (0, 1.0, 1.0)]:
        logits = row.to(DEV).repeat(n, 1).contiguous()
        tk = torch.full((n,), k if k > 0 else -1, dtype=torch.int32, device=DEV)
        tp = torch.full((n,), p, dtype=torch.float32, device=DEV)
        tt = torch.full((n,), t, dtype=torch.float32, device=DEV)
        seeds = torch.full((n,), 1234, dtype=torch.int64, device=DEV)
        pos = torch.arange(n, dtype=torch.int32, device=DEV)
        toks = ops.sample(logits, tk, tp, tt, seeds, pos).cpu().long()
        ids, probs = ref.sampled_distribution(row, k if k > 1 else None, p if 0 < p < 1 else None, t)
        allowed = set(ids.tolist())
        assert set(toks.tolist()) <= allowed, "sampled a token outside the truncated support"
        freq = torch.bincount(toks, minlength=V).double() / n
        expect = torch.zeros(V, dtype=torch.double)
        expect[ids] = probs
        # total variation distance; for n=20000 and support <= 512 the noise floor is ~0.05
        tv = 0.5 * (freq - expect).abs().sum().item()
        assert tv < 0.06, f"(k={k}, p={p}, t={t}) total variation {tv:.3f}"


def test_sampling_reproducible_and_batch_independent():
    V = 32000
    x = _rand(16, V, dtype=torch.float32, seed=42) * 3
    tk = torch.full((16,), 40, dtype=torch.int32, device=DEV)
    tp = torch.full((16,), 0.95, dtype=torch.float32, device=DEV)
    tt = torch.full((16,), 0.8, dtype=torch.float32, device=DEV)
    seeds = torch.arange(16, dtype=torch.int64, device=DEV) + 99
    pos = torch.full((16,), 7, dtype=torch.int32, device=DEV)
    a = ops.sample(x, tk, tp, tt, seeds, pos)
    b = ops.sample(x, tk, tp, tt, seeds, pos)
    assert torch.equal(a, b)
    one = ops.sample(x[5:6].contiguous(), tk[5:6], tp[5:6], tt[5:6], seeds[5:6], pos[5:6])
    assert int(one[0]) == int(a[5]), "a row must sample the same token alone or inside a batch"


def test_sampling_ties_and_masked_rows():
    V = 1000
    x = torch.zeros(4, V, dtype=torch.float32, device=DEV)           # every logit ties
    tk = torch.full((4,), 10, dtype=torch.int32, device=DEV)
    f1 = torch.ones(4, dtype=torch.float32, device=DEV)
    seeds = torch.arange(4, dtype=torch.int64, device=DEV)
    toks = ops.sample(x, tk, f1, f1, seeds, torch.zeros(4, dtype=torch.int32, device=DEV))
    assert bool((toks < 10).all()), "ties at the top-k threshold keep the lowest indices"
    y = torch.full((2, V), torch.finfo(torch.float32).min, device=DEV)
    y[0, 77] = 0.0
    y[1, 5] = 1.0
    y[1, 6] = 1.0
    toks = ops.sample(y, torch.tensor([50, 50], dtype=torch.int32, device=DEV), f1[:2] * 0.9, f1[:2], seeds[:2],
                      torch.zeros(2, dtype=torch.int32, device=DEV))
    assert int(toks[0]) == 77 and int(toks[1]) in (5, 6)


def test_topk_and_beam_candidates():
    x = _rand(6, 5000, dtype=torch.float32, seed=43)
    for k in (1, 8, 64):
        v, i = ops.topk(x, k)
        rv, ri = ref.topk(x.cpu(), k)
        assert torch.equal(i.cpu(), ri)
        _close(v, rv, 0, 0)
    add = _rand(6, dtype=torch.float32, seed=44)
    v, i = ops.topk(x, 8, log_softmax=True, add=add)
    rv, ri = ref.topk(x.cpu(), 8, log_softmax=True, add=add.cpu())
    assert torch.equal(i.cpu(), ri)
    _close(v, rv, rtol=1e-4, atol=1e-4)
    s, t, b = ops.beam_candidates(x, add, batch=2, beams=3)
    rs, rt, rb = ops.beam_candidates(x.cpu(), add.cpu(), batch=2, beams=3)
    assert torch.equal(t.cpu(), rt) and torch.equal(b.cpu(), rb)
    _close(s, rs, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("rows,n", [(1, 201088), (3, 50000), (20, 32064), (40, 128256), (100, 16384)])
def test_topk_long_rows_cluster_kernel(rows, n):
    """Long rows take the candidate-list kernel: 8 / 4 / 2 / 1 CTAs per row depending on the row count, ties at the cut."""
    x = _rand(rows, n, dtype=torch.float32, seed=46)
    x[:, ::7] = x[:, 3:4]            # many equal values, some of them inside the top-k set
    for k in (1, 50, 128):
        v, i = ops.topk(x, k)
        rv, ri = ref.topk(x.cpu(), k)
        assert torch.equal(i.cpu(), ri)
        _close(v, rv, 0, 0)
    add = _rand(rows, dtype=torch.float32, seed=47)
    v, i = ops.topk(x, 8, log_softmax=True, add=add)
    rv, ri = ref.topk(x.cpu(), 8, log_softmax=True, add=add.cpu())
    assert torch.equal(i.cpu(), ri)
    _close(v, rv, rtol=1e-4, atol=1e-4)
    ops.check_kernel_status()


def test_logits_mask_and_edit():
    V = 1003
    x = _rand(3, V, dtype=torch.float32, seed=45)
    xr = x.cpu().clone()
    words = (V - 1) // 32 + 1
    mask = torch.randint(-2**31, 2**31 - 1, (2, words), dtype=torch.int64).to(torch.int32)
    rows = torch.tensor([1, -1, 0], dtype=torch.int32)
    ops.logits_bitmask(x, mask.to(DEV), rows.to(DEV))
    ref.logits_bitmask(xr, mask, rows)
    assert torch.equal(x.cpu(), xr)
    x = _rand(3, V, dtype=torch.float32, seed=46)
    xr = x.cpu().clone()
    r = torch.tensor([0, 0, 2], dtype=torch.int32)
    t = torch.tensor([5, 9, 1000], dtype=torch.int32)
    o = torch.tensor([1, 0, 1], dtype=torch.int32)
    v = torch.tensor([1.3, 0.0, 2.0])
    ops.logits_edit(x, r.to(DEV), t.to(DEV), o.to(DEV), v.to(DEV))
    ref.logits_edit(xr, r, t, o, v)
    _close(x, xr, rtol=1e-6, atol=1e-6)


# ------------------------------------------------------------------------------------------- int4 dequant GEMM
def _w4_case(N, K, seed, symmetric=False):
    from onnxruntime_genai_b200.models.builder import quantize_int4_block32
    from onnxruntime_genai_b200.ops.w4 import W4Weight, unpack_ort_q4
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * 0.05
    qw, s, zp = quantize_int4_block32(w, symmetric=symmetric)
    q, z = unpack_ort_q4(qw, zp, N, K)
    return W4Weight.from_quantized(q, s.to(torch.float16).float(), z, DEV), w


@pytest.mark.parametrize("M,N,K,splits", [(1, 128, 64, 1), (5, 3072, 3072, 0), (64, 1000, 512, 1), (16, 256, 4096, 4), (130, 384, 256, 1),
                                          (300, 512, 1024, 1), (33, 9216, 3072, 0)])
def test_gemm_w4_matches_dequantised_fp32(M, N, K, splits):
    w4, w = _w4_case(N, K, seed=50)
    x = _rand(M, K, seed=51)
    y = ops.linear(x, w4, splits=splits)
    ops.check_kernel_status()
    want = ref.linear(x.cpu(), w4.dequantize())
    _close(y, want, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.05)
    assert (w4.dequantize() - w).abs().max() < 0.02, "the kernel-side dequantisation formula stays close to the original weights"


def test_gemm_w4_epilogues_and_symmetric():
    w4, _ = _w4_case(512, 256, seed=52, symmetric=True)
    x, bias, res = _rand(20, 256, seed=53), _rand(512, seed=54), _rand(20, 512, seed=55)
    y = ops.linear(x, w4, bias=bias, residual=res)
    _close(y, ref.linear(x.cpu(), w4.dequantize(), bias.cpu(), res.cpu()), rtol=2e-2, atol=0.05)
    y32 = ops.linear(x, w4, out_fp32=True)
    _close(y32, ref.linear(x.cpu(), w4.dequantize(), out_fp32=True), rtol=1e-2, atol=0.02)
    ops.check_kernel_status()


def test_gemm_w4_gate_up_pair():
    from onnxruntime_genai_b200.models.builder import quantize_int4_block32
    from onnxruntime_genai_b200.ops.w4 import W4Weight, unpack_ort_q4
    I, K, M = 256, 512, 24
    w = torch.randn(2 * I, K, generator=torch.Generator().manual_seed(56)) * 0.05
    qw, s, zp = quantize_int4_block32(w)
    q, z = unpack_ort_q4(qw, zp, 2 * I, K)
    plain = W4Weight.from_quantized(q, s, z, DEV)
    il = W4Weight.from_quantized(ops.interleave_gate_up(q), ops.interleave_gate_up(s), ops.interleave_gate_up(z), DEV, interleaved=True)
    x = _rand(M, K, seed=57)
    want = ref.gate_up_act(x.cpu(), plain.dequantize())
    _close(ops.gate_up_act(x, il), want, rtol=3e-2, atol=0.05)
    _close(ops.gate_up_act(x, plain), want, rtol=3e-2, atol=0.05)
    ops.check_kernel_status()


_GEMV_CASES = {}


@pytest.mark.parametrize("M", [1, 2, 3, 4, 7, 8, 11, 16])
def test_gemv_w4_few_tokens(M):
    """One to four tokens take the weight-streaming GEMV, more the tensor-core kernel with its smallest token tile: all epilogues, uneven k splits, rows past N, many k-blocks per
    CTA, against the dequantised fp32 product."""
    for N, K, splits in ((1152, 768, 0), (1000, 512, 3), (128, 64, 1), (256, 4096, 2)):
        if (N, K) not in _GEMV_CASES:      # quantising on the host is the slow part: once per shape
            w4, _ = _w4_case(N, K, seed=60)
            _GEMV_CASES[(N, K)] = (w4, w4.dequantize())
        w4, wd = _GEMV_CASES[(N, K)]
        x, bias, res = _rand(M, K, seed=61), _rand(N, seed=62), _rand(M, N, seed=63)
        want = ref.linear(x.cpu(), wd, bias.cpu(), res.cpu())
        y = ops.linear(x, w4, bias=bias, residual=res, splits=splits)
        _close(y, want, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.05)
        y32 = ops.linear(x, w4, out_fp32=True, splits=splits)
        _close(y32, ref.linear(x.cpu(), wd, out_fp32=True), rtol=1e-2, atol=1e-2 * math.sqrt(K) * 0.05)
    ops.check_kernel_status()
    # paired SiLU*mul epilogue
    from onnxruntime_genai_b200.models.builder import quantize_int4_block32
    from onnxruntime_genai_b200.ops.w4 import W4Weight, unpack_ort_q4
    I, K = 256, 512
    w = torch.randn(2 * I, K, generator=torch.Generator().manual_seed(64)) * 0.05
    qw, s, zp = quantize_int4_block32(w)
    q, z = unpack_ort_q4(qw, zp, 2 * I, K)
    plain = W4Weight.from_quantized(q, s, z, DEV)
    il = W4Weight.from_quantized(ops.interleave_gate_up(q), ops.interleave_gate_up(s), ops.interleave_gate_up(z), DEV, interleaved=True)
    x = _rand(M, K, seed=65)
    _close(ops.gate_up_act(x, il), ref.gate_up_act(x.cpu(), plain.dequantize()), rtol=3e-2, atol=0.05)
    ops.check_kernel_status()


# ------------------------------------------------------------------------------------------- mixture of experts
@pytest.mark.parametrize("T,E,k,mode", [(1, 8, 2, 0), (37, 32, 4, 0), (64, 128, 8, 2), (300, 60, 4, 1)])
def test_moe_topk_matches_torch(T, E, k, mode):
    logits = _rand(T, E, std=2.0, dtype=torch.float32, seed=31)
    plan = ops.moe_route(logits, k, mode)
    v, i = torch.topk(logits, k, dim=-1)
    if mode == 0:
        w = torch.softmax(v, dim=-1)
    else:
        w = torch.softmax(logits, dim=-1).gather(1, i)
        if mode == 2:
            w = w / w.sum(-1, keepdim=True)
    assert plan.topk_idx.cpu().tolist() == i.cpu().tolist()
    _close(plan.topk_w, w, 1e-4, 1e-6)
    # grouping: every assignment appears once, rows of an expert are contiguous, tiles cover exactly those rows
    off = plan.expert_offsets.cpu().tolist()
    inv = plan.inv_pos.cpu().reshape(-1).tolist()
    src = plan.sorted_token.cpu().tolist()
    flat = i.cpu().reshape(-1).tolist()
    assert sorted(inv) == list(range(T * k)) and off[-1] == T * k
    for a, pos in enumerate(inv):
        assert off[flat[a]] <= pos < off[flat[a] + 1] and src[pos] == a // k
    nt = int(plan.num_tiles.cpu()[0])
    covered = []
    for t in range(nt):
        e, r0, n = int(plan.tile_expert[t]), int(plan.tile_row0[t]), int(plan.tile_rows[t])
        assert off[e] <= r0 and r0 + n <= off[e + 1] and 0 < n <= plan.bt
        covered += list(range(r0, r0 + n))
    assert sorted(covered) == list(range(T * k)) and nt <= plan.max_tiles


def _moe_reference(x, router_w, router_b, gu_w, gu_b, dn_w, dn_b, k, alpha, limit, lo=0, hi=None):
    """fp32 loop over experts; gu_w [E, 2I, H] rows even = gate, odd = up."""
    x = x.float()
    logits = x @ router_w.float().t() + router_b.float()
    v, i = torch.topk(logits, k, dim=-1)
    w = torch.softmax(v, dim=-1)
    out = torch.zeros_like(x)
    hi = gu_w.shape[0] if hi is None else hi
    for e in range(lo, hi):
        tok, slot = (i == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        gu = x[tok].to(torch.bfloat16).float() @ gu_w[e].float().t() + gu_b[e].float()
        g, u = gu[:, 0::2].clamp(max=limit), gu[:, 1::2].clamp(-limit, limit)
        act = (g * torch.sigmoid(alpha * g) * (u + 1)).to(torch.bfloat16).float()
        y = (act @ dn_w[e].float().t() + dn_b[e].float()).to(torch.bfloat16).float()
        out.index_add_(0, tok, y * w[tok, slot][:, None])
    return out, logits


@pytest.mark.parametrize("T,E,k,H,I", [(3, 4, 2, 128, 64), (64, 32, 4, 256, 192), (700, 8, 2, 320, 128), (130, 16, 4, 2880, 64)])
def test_moe_grouped_gemm_matches_expert_loop(T, E, k, H, I):
    x = _rand(T, H, std=1.0, seed=41)
    router_w, router_b = _rand(E, H, std=0.1, seed=42), _rand(E, std=0.1, seed=43)
    gu_w, gu_b = _rand(E, 2 * I, H, std=0.05, seed=44), _rand(E, 2 * I, std=0.1, seed=45)
    dn_w, dn_b = _rand(E, H, I, std=0.05, seed=46), _rand(E, H, std=0.1, seed=47)
    alpha, limit = 1.702, 7.0
    want, logits_ref = _moe_reference(x, router_w, router_b, gu_w, gu_b, dn_w, dn_b, k, alpha, limit)
    logits = ops.linear(x, router_w, router_b, out_fp32=True)
    # near-ties in the router would legitimately pick different experts: require a clear margin in this test's data
    v = torch.topk(logits_ref, k + 1, dim=-1).values
    assert float((v[:, k - 1] - v[:, k]).min()) > 1e-3 or T > 100
    gw, gb = ops.interleave_experts_gate_up(gu_w), ops.interleave_experts_gate_up(gu_b)
    for lo, hi in ((0, E), (E // 2, E)):
        plan = ops.moe_route(logits, k, 0, (lo, hi))
        xs = ops.gather_rows(x, plan.sorted_token)
        h = ops.moe_gemm(xs, gw[lo:hi].contiguous(), plan, gb[lo:hi].contiguous(), act_kind=2, alpha=alpha, limit=limit)
        y = ops.moe_gemm(h, dn_w[lo:hi].contiguous(), plan, dn_b[lo:hi].contiguous())
        got = ops.moe_combine(y, plan)
        ops.check_kernel_status()
        ref_out = want if (lo, hi) == (0, E) else _moe_reference(x, router_w, router_b, gu_w, gu_b, dn_w, dn_b, k, alpha, limit, lo, hi)[0]
        bad = ((got.float() - ref_out.to(got.device)).abs() > 0.03 + 0.03 * ref_out.abs().to(got.device)).float().mean().item()
        assert bad < (0.002 if T <= 100 else 0.02), f"{bad:.4f} of the outputs differ (experts {lo}..{hi})"


def _random_fp4(E, N, K, seed):
    """Random MXFP4 experts: codes [E, N, K] (every e2m1 value, both signs), scale codes [E, N, K/32]."""
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 16, (E, N, K), generator=g, dtype=torch.uint8)
    scales = torch.randint(117, 123, (E, N, K // 32), generator=g, dtype=torch.uint8)
    return codes, scales


@pytest.mark.parametrize("rows", [64, 4])          # 4 rows of the fp16 form: the streaming kernel for tiles of up to 8 rows
@pytest.mark.parametrize("half", [False, True])
def test_fp4_expansion_is_exact_for_every_code(half, rows):
    """One expert whose rows hold every e2m1 code against an identity activation: the grouped FP4 GEMM returns the
    weights themselves, so every code (the subnormal 0.5 and both zeros included) times several block scales is
    checked bit for bit."""
    from onnxruntime_genai_b200.ops.fp4 import Fp4Experts
    N, K = 128, 64
    codes = (torch.arange(N * K, dtype=torch.int64).view(1, N, K) * 7 % 16).to(torch.uint8)
    codes[0, :, :16] = torch.arange(16, dtype=torch.uint8)
    # bf16 form 2^-112 .. 2^1, fp16 form 2^-14 .. 2^9 (times 6 still below the fp16 maximum divided by the fp32 round trip):
    # every product is a normal bf16 (the kernels are built with flush-to-zero fp32 arithmetic)
    if half:
        scales = (torch.arange(N * 2, dtype=torch.int64).view(1, N, 2) % 24 + 113).to(torch.uint8)
    else:
        scales = (torch.arange(N * 2, dtype=torch.int64).view(1, N, 2) % 114 + 15).to(torch.uint8)
    scales[0, :8] = 127
    fe = Fp4Experts.from_codes(codes, scales, DEV, half=half)
    x = torch.eye(K, dtype=torch.float16 if half else torch.bfloat16, device=DEV)[:rows].contiguous()
    logits = torch.zeros(rows, 1, dtype=torch.float32, device=DEV)
    plan = ops.moe_route(logits, 1, 0, (0, 1))
    xs = x[plan.sorted_token.long()].contiguous()
    y = ops.moe_gemm(xs, fe, plan, None)
    ops.check_kernel_status()
    got = torch.empty_like(y)
    got[plan.sorted_token.long()] = y
    want = fe.dequantize(0).t().to(torch.bfloat16)[:rows]   # [rows, N]: row k of the output is column k of the weight
    assert torch.equal(got.cpu(), want), f"{(got.cpu() != want).sum().item()} of {want.numel()} weights differ"


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("T,E,k,H,I", [(3, 4, 2, 128, 64), (64, 32, 4, 256, 192), (700, 8, 2, 320, 128), (40, 8, 4, 2880, 64),
                                       (2, 8, 2, 2880, 192), (4, 8, 4, 320, 2880), (24, 32, 4, 320, 128), (7, 4, 2, 448, 256)])
def test_moe_fp4_grouped_gemm_matches_expert_loop(T, E, k, H, I, half):
    """Packed MXFP4 experts through the grouped FP4 GEMM (clamped SwiGLU epilogue, then the down projection whose
    row count is not a multiple of the 128-row tile) against the fp32 loop over the dequantised experts."""
    from onnxruntime_genai_b200.ops.fp4 import Fp4Experts
    x = _rand(T, H, std=1.0, seed=51)
    router_w, router_b = _rand(E, H, std=0.1, seed=52), _rand(E, std=0.1, seed=53)
    gu_c, gu_s = _random_fp4(E, 2 * I, H, 54)
    dn_c, dn_s = _random_fp4(E, H, I, 55)
    gu_b, dn_b = _rand(E, 2 * I, std=0.1, seed=56), _rand(E, H, std=0.1, seed=57)
    gu_w = Fp4Experts.from_codes(gu_c, gu_s, "cpu").dequantize().to(DEV)
    dn_w = Fp4Experts.from_codes(dn_c, dn_s, "cpu").dequantize().to(DEV)
    alpha, limit = 1.702, 7.0
    want, _ = _moe_reference(x, router_w, router_b, gu_w, gu_b, dn_w, dn_b, k, alpha, limit)
    logits = ops.linear(x, router_w, router_b, out_fp32=True)
    gb = ops.interleave_experts_gate_up(gu_b)
    for lo, hi in ((0, E), (E // 2, E)):
        gw = Fp4Experts.from_codes(ops.interleave_experts_gate_up(gu_c[lo:hi]), ops.interleave_experts_gate_up(gu_s[lo:hi]), DEV, half=half)
        dw = Fp4Experts.from_codes(dn_c[lo:hi].contiguous(), dn_s[lo:hi].contiguous(), DEV, half=half)
        plan = ops.moe_route(logits, k, 0, (lo, hi))
        mapped = ops.moe_fp4_reads_rows(gw, plan)      # decode-sized steps of the fp16 form read the rows through the plan's map
        xs = x if mapped else ops.gather_rows(x, plan.sorted_token, f16=half)
        h = ops.moe_gemm(xs, gw, plan, gb[lo:hi].contiguous(), act_kind=2, alpha=alpha, limit=limit,
                         out_dtype=torch.float16 if half else torch.bfloat16, row_map=mapped)
        if mapped:   # the same through a gathered fp16 copy
            h2 = ops.moe_gemm(ops.gather_rows(x, plan.sorted_token, f16=True), gw, plan, gb[lo:hi].contiguous(), act_kind=2, alpha=alpha,
                              limit=limit, out_dtype=torch.float16)
            n_rows = int(plan.expert_offsets[-1].item())
            assert torch.equal(h[:n_rows], h2[:n_rows])
        y = ops.moe_gemm(h, dw, plan, dn_b[lo:hi].contiguous())
        got = ops.moe_combine(y, plan)
        ops.check_kernel_status()
        ref_out = want if (lo, hi) == (0, E) else _moe_reference(x, router_w, router_b, gu_w, gu_b, dn_w, dn_b, k, alpha, limit, lo, hi)[0]
        bad = ((got.float() - ref_out.to(got.device)).abs() > 0.03 + 0.03 * ref_out.abs().to(got.device)).float().mean().item()
        assert bad < (0.002 if T <= 100 else 0.02), f"{bad:.4f} of the outputs differ (experts {lo}..{hi})"


@pytest.mark.parametrize("T,E,k,H", [(1, 32, 4, 2880), (7, 8, 2, 320), (40, 16, 4, 4096)])
def test_norm_moe_combine_equals_combine_then_norm(T, E, k, H):
    """The combine step folded into the residual add + norm: same bits as moe_combine followed by norm, also with experts
    that are not local (rows skipped)."""
    logits = torch.randn(T, E, device=DEV, generator=torch.Generator(device=DEV).manual_seed(5))
    w = _rand(H, std=1.0, seed=71)
    for rng in ((0, E), (E // 2, E)):
        plan = ops.moe_route(logits, k, 0, rng)
        y = _rand(T * k, H, std=1.0, seed=72)
        r1, r2 = _rand(T, H, std=1.0, seed=73), _rand(T, H, std=1.0, seed=73)
        a, ra = ops.norm(ops.moe_combine(y, plan), w, 1e-5, r1)
        b, rb = ops.norm_moe_combine(ops.PendingCombine(y, plan), w, 1e-5, r2)
        ops.check_kernel_status()
        assert torch.equal(a, b) and torch.equal(ra, rb)


def test_copy_state_slots_between_pools():
    """Recurrent-state snapshots: dst[:, dst_slots] = src[:, src_slots] over all layers, other slots untouched."""
    g = torch.Generator(device=DEV).manual_seed(3)
    src = torch.randn(3, 6, 4, 16, 8, device=DEV, generator=g)
    dst = torch.randn(3, 6, 4, 16, 8, device=DEV, generator=g)
    want = dst.clone()
    want[:, [5, 0, 2]] = src[:, [1, 4, 2]]
    ops.copy_state_slots(src, dst, [1, 4, 2], [5, 0, 2])
    assert torch.equal(dst, want)
    same = src.clone()
    ops.copy_state_slots(same, same, [0], [3])               # inside one pool
    assert torch.equal(same[:, 3], src[:, 0]) and torch.equal(same[:, :3], src[:, :3])


# ------------------------------------------------------------------------------------------- beam scorer on the device
@pytest.mark.parametrize("batch,beams,lp,early,p_eos", [(1, 2, 1.0, False, 0.2), (3, 4, 1.0, True, 0.25), (2, 8, 0.6, False, 0.15),
                                                          (4, 3, 1.7, False, 0.3), (2, 5, 1.0, False, 0.0)])
def test_device_beam_scorer_follows_the_host_scorer(batch, beams, lp, early, p_eos):
    """The same stream of candidates (random scores, tokens with end-of-sequence ids mixed in, random source beams) through the
    device scorer and through the host scorer: same tokens, source rows and verdict every step, same sequences, same ranked
    hypotheses at the end."""
    from onnxruntime_genai_b200.beam_device import DeviceBeamScorer
    from onnxruntime_genai_b200.native_loader import native
    vocab, L, prompt_len, eos = 60, 24, 5, [1, 7]
    sp = native.SearchParams()
    sp.batch_size, sp.num_beams, sp.num_return_sequences, sp.vocab_size, sp.max_length = batch, beams, beams, vocab, L
    sp.eos_token_ids, sp.pad_token_id, sp.length_penalty, sp.early_stopping, sp.random_seed = eos, 0, lp, early, 1
    host = native.Search(sp)
    rng = np.random.RandomState(100 * batch + beams)
    prompt = rng.randint(8, vocab, size=(batch, prompt_len)).astype(np.int32)
    host.append_tokens(prompt)
    rows = batch * beams
    seqs = np.stack([host.sequence(r) for r in range(rows)]).astype(np.int32)
    dev = DeviceBeamScorer(seqs, batch, beams, L, 0, eos, lp, early, torch.device(DEV))
    cand = 2 * beams
    running = np.zeros((batch, beams), dtype=np.float32)
    steps = 0
    while not host.is_done:
        cs = np.zeros((batch, cand), dtype=np.float32)
        ct = np.zeros((batch, cand), dtype=np.int32)
        cb = rng.randint(0, beams, size=(batch, cand)).astype(np.int32)
        for b in range(batch):
            cs[b] = np.sort(running[b].max() - rng.rand(cand).astype(np.float32) * 3.0 - 0.1)[::-1]
            toks = rng.randint(8, vocab, size=cand)
            is_eos = rng.rand(cand) < p_eos
            is_eos[np.flatnonzero(is_eos)[beams:]] = False          # at least num_beams candidates continue
            toks[is_eos] = rng.choice(eos, size=int(is_eos.sum()))
            ct[b] = toks
        host.commit_beam_step(cs.copy(), ct.copy(), cb.copy())
        t_d, r_d, done_d = dev.step(torch.from_numpy(cs).to(DEV), torch.from_numpy(ct).to(DEV), torch.from_numpy(cb).to(DEV))
        assert t_d.tolist() == host.next_tokens().tolist(), f"step {steps}"
        assert r_d.tolist() == host.beam_rows().tolist(), f"step {steps}"
        np.testing.assert_allclose(dev.beam_scores().cpu().numpy(), host.beam_scores(), rtol=0, atol=0)
        dseq = dev.sequences().cpu().numpy()
        for r in range(rows):
            assert dseq[r].tolist() == host.sequence(r).tolist()
        if host.length < L:
            assert done_d == bool(host.is_done), f"step {steps}"
        running = host.beam_scores().reshape(batch, beams)
        steps += 1
    host.finalize()
    ranked = dev.finalize()
    for b in range(batch):
        assert len(ranked[b]) >= 1
        for rank, (toks, score) in enumerate(ranked[b]):
            h_toks, h_score = host.hypothesis(b, rank)
            assert toks.tolist() == h_toks.tolist(), f"entry {b} rank {rank}"
            assert abs(score - h_score) <= 1e-5 * max(1.0, abs(h_score))
    assert steps >= 3


# ------------------------------------------------------------------------------------------- sampled speculative verify
def test_verify_sampled_preserves_the_target_distribution():
    """Rejection sampling theorem: whatever the proposal, the first committed token follows the target's sampled
    distribution; and the accept probability is min(1, p(x)/q(x))."""
    V, n, k, p, t = 300, 3000, 20, 0.9, 0.8
    g = torch.Generator().manual_seed(7)
    rows = (torch.randn(2, V, generator=g) * 2.0).float()
    ids, probs = ref.sampled_distribution(rows[0], k, p, t)
    expect = torch.zeros(V, dtype=torch.double)
    expect[ids] = probs
    logits = rows.to(DEV).contiguous()
    top = int(ids[0])
    second = int(ids[1])
    # (a) deterministic proposal of the most likely token, (b) a sparse proposal distribution that over-weights the second token
    q_sparse = (np.asarray([top, second, int(ids[2])], dtype=np.int32), np.asarray([0.2, 0.7, 0.1], dtype=np.float32))
    for draft_tok, q in ((top, None), (second, q_sparse)):
        counts = torch.zeros(V, dtype=torch.double)
        acc = 0
        for s in range(n):
            a, commit, ap = ops.verify_sampled(logits, [draft_tok], [q], k, p, t, seed=1000 + s, first_position=5)
            assert len(commit) == a + 1 and (a == 0 or commit[0] == draft_tok)
            counts[commit[0]] += 1
            acc += a
        px = float(expect[draft_tok])
        qx = 1.0 if q is None else float(q[1][list(q[0]).index(draft_tok)])
        assert abs(ap[0] - min(1.0, px / qx)) < 1e-4
        assert abs(acc / n - min(1.0, px / qx)) < 0.04
        if q is None:
            # one-hot proposal: committed token ~ p exactly (accept w.p. p(x), else residual p without x)
            tv = 0.5 * (counts / n - expect).abs().sum().item()
            assert tv < 0.06, f"total variation {tv:.3f}"
        else:
            # the draft token itself was drawn by us, not from q, so only the conditional law is checked:
            # given rejection the replacement follows max(0, p - q) renormalised
            resid = (expect - torch.zeros(V, dtype=torch.double).index_put((torch.tensor(q[0]).long(),), torch.tensor(q[1]).double())).clamp(min=0)
            resid = resid / resid.sum()
            rej = counts.clone()
            rej[draft_tok] -= acc
            tv = 0.5 * (rej / rej.sum() - resid).abs().sum().item()
            assert tv < 0.08, f"residual total variation {tv:.3f}"


def test_verify_sampled_multi_token_and_bonus():
    V, k = 1000, 50
    x = _rand(5, V, dtype=torch.float32, seed=77) * 3
    # proposals equal to each row's arg max with sharp logits are accepted; the bonus token equals the plain sampler's draw
    sharp = x.clone()
    am = sharp.argmax(-1)
    sharp[torch.arange(5), am] += 60.0
    draft = am[:4].cpu().tolist()
    a, commit, ap = ops.verify_sampled(sharp, draft, [None] * 4, k, 0.95, 0.7, seed=11, first_position=30)
    assert a == 4 and commit[:4] == draft and all(v > 0.999 for v in ap)
    tk = torch.full((1,), k, dtype=torch.int32, device=DEV)
    one = ops.sample(sharp[4:5].contiguous(), tk, torch.full((1,), 0.95, device=DEV), torch.full((1,), 0.7, device=DEV),
                     torch.full((1,), 11, dtype=torch.int64, device=DEV), torch.full((1,), 34, dtype=torch.int32, device=DEV))
    assert commit[4] == int(one[0])
    # a proposal outside the target's top-k is rejected at once and replaced by a token of the target's support
    worst = int(x[0].argmin())
    a, commit, ap = ops.verify_sampled(x, [worst, draft[1], draft[2], draft[3]], [None] * 4, k, 0.95, 0.7, seed=12, first_position=30)
    assert a == 0 and len(commit) == 1 and ap[0] == 0.0
    assert commit[0] in torch.topk(x[0], k).indices.cpu().tolist()
    # twice in a row: the kernel's completion counter resets itself
    b = ops.verify_sampled(x, [worst, draft[1], draft[2], draft[3]], [None] * 4, k, 0.95, 0.7, seed=12, first_position=30)
    assert b[0] == a and b[1] == commit


@pytest.mark.parametrize("Hk,Hv,dk,dv", [(2, 4, 16, 16), (4, 4, 64, 64), (2, 8, 128, 128), (1, 2, 32, 96)])
def test_gated_delta_rule_kernel(Hk, Hv, dk, dv):
    """The recurrence of a linear-attention layer: prompt chunks, single tokens, a fresh request (state reset) and requests that
    continue from their slot's state, against the fp32 restatement."""
    torch.manual_seed(3)
    q_lens, past = [7, 1, 19, 1], [0, 5, 12, 0]
    T, B = sum(q_lens), len(q_lens)
    q = torch.nn.functional.normalize(torch.randn(T, Hk, dk), dim=-1).to(torch.bfloat16).to(DEV)
    k = torch.nn.functional.normalize(torch.randn(T, Hk, dk), dim=-1).to(torch.bfloat16).to(DEV)
    v = torch.randn(T, Hv, dv).to(torch.bfloat16).to(DEV)
    g = (-torch.rand(T, Hv) * 0.5).to(DEV)
    beta = torch.rand(T, Hv).to(DEV)
    state = torch.randn(6, Hv, dk, dv, device=DEV) * 0.1
    slots = torch.tensor([4, 0, 2, 5], dtype=torch.int32, device=DEV)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32, device=DEV)
    pl = torch.tensor(past, dtype=torch.int32, device=DEV)
    want_state = state.cpu().clone()
    want = ref.gated_delta(q.cpu(), k.cpu(), v.cpu(), g.cpu(), beta.cpu(), want_state, slots.cpu(), cu.cpu(), pl.cpu())
    got = ops.gated_delta(q, k, v, g, beta, state, slots, cu, pl)
    _close(got, want, rtol=2e-2, atol=2e-2)
    _close(state, want_state, rtol=1e-3, atol=1e-3)
    assert torch.equal(state[1].cpu(), want_state[1]) and torch.equal(state[3].cpu(), want_state[3])     # untouched slots
    ops.check_kernel_status()
