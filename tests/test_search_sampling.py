"""Host search / sampling math (reference behaviour: src/search.cpp, src/sampling_distribution.h,
src/beam_search_scorer.cpp; tests modelled on test/sampling_tests.cpp and sampling_distribution_tests.cpp)."""
import math

import numpy as np
import pytest

from onnxruntime_genai_b200.native_loader import native


def params(batch=1, beams=1, vocab=16, max_length=12, **kw):
    p = native.SearchParams()
    p.batch_size, p.num_beams, p.vocab_size, p.max_length = batch, beams, vocab, max_length
    p.eos_token_ids, p.pad_token_id = kw.pop("eos", [0]), kw.pop("pad", 15)
    p.random_seed = kw.pop("seed", 42)
    for k, v in kw.items():
        setattr(p, k, v)
    return p


def onehotish(rows, vocab, winners, hi=5.0):
    x = np.zeros((rows, vocab), dtype=np.float32)
    for r, w in enumerate(winners):
        x[r, w] = hi
    return x


def test_greedy_appends_argmax_and_stops_at_max_length():
    s = native.Search(params(batch=2, max_length=5))
    s.append_tokens(np.array([[3, 4], [5, 6]], dtype=np.int32))
    for step in range(3):
        s.score(onehotish(2, 16, [7 + step, 9]), "greedy")
    assert s.sequence(0).tolist() == [3, 4, 7, 8, 9] and s.sequence(1).tolist() == [5, 6, 9, 9, 9]
    assert s.is_done


def test_eos_pads_finished_rows_and_finishes_when_all_done():
    s = native.Search(params(batch=2, max_length=10))
    s.append_tokens(np.array([[3], [5]], dtype=np.int32))
    s.score(onehotish(2, 16, [0, 7]), "greedy")      # row 0 hits EOS
    assert s.next_tokens().tolist() == [0, 7] and not s.is_done
    s.score(onehotish(2, 16, [9, 8]), "greedy")      # row 0 now emits pad
    assert s.next_tokens().tolist() == [15, 8]
    s.score(onehotish(2, 16, [9, 0]), "greedy")
    assert s.is_done and s.sequence(0).tolist() == [3, 0, 15, 15]


def test_min_length_masks_eos():
    s = native.Search(params(max_length=10, min_length=3))
    s.append_tokens(np.array([[3]], dtype=np.int32))
    x = onehotish(1, 16, [0])
    x[0, 4] = 1.0
    s.score(x.copy(), "greedy")
    assert s.next_tokens().tolist() == [4], "EOS is masked while the sequence is shorter than min_length"
    s.score(x.copy(), "greedy")
    s.score(x.copy(), "greedy")
    assert s.next_tokens().tolist() == [0]


def test_repetition_penalty_sign_convention():
    x = np.array([2.0, -2.0, 1.0, 3.0], dtype=np.float32)
    native.apply_repetition_penalty(x, np.array([0, 1, 1, 0], dtype=np.int32), 2.0)
    np.testing.assert_allclose(x, [1.0, -4.0, 1.0, 3.0])


def test_no_repeat_ngram_bans_completions():
    prefix = np.array([1, 2, 3, 1, 2], dtype=np.int32)
    assert native.no_repeat_ngram_banned(prefix, 3, 8) == [3]
    assert native.no_repeat_ngram_banned(prefix, 2, 8) == [3]
    assert native.no_repeat_ngram_banned(np.array([1, 2], dtype=np.int32), 3, 8) == []


def _exact_dist(logits, k, p, t):
    x = logits.astype(np.float64) / t
    order = np.argsort(-x, kind="stable")
    if k > 1:
        order = order[:k]
    pr = np.exp(x[order] - x[order].max())
    pr /= pr.sum()
    if 0 < p < 1:
        keep = int(np.searchsorted(np.cumsum(pr), p)) + 1
        order, pr = order[:keep], pr[:keep] / pr[:keep].sum()
    return order, pr


@pytest.mark.parametrize("k,p,t", [(5, 0.0, 1.0), (0, 0.7, 1.0), (8, 0.6, 0.5), (0, 0.0, 2.0), (50, 0.95, 0.7)])
def test_sampled_distribution_matches_definition(k, p, t):
    rng = np.random.RandomState(0)
    logits = (rng.randn(300) * 3).astype(np.float32)
    ids, probs = native.sampled_distribution(logits, k, p, t)
    want_ids, want_p = _exact_dist(logits, k, p, t)
    assert ids.tolist() == want_ids.tolist()
    np.testing.assert_allclose(probs, want_p, rtol=1e-4, atol=1e-6)
    assert abs(probs.sum() - 1) < 1e-5


def test_sampling_statistics_top_k_top_p():
    """Empirical frequencies of the host sampler follow the truncated distribution."""
    vocab, n = 32, 6000
    rng = np.random.RandomState(1)
    logits = (rng.randn(vocab) * 2).astype(np.float32)
    want_ids, want_p = _exact_dist(logits, 10, 0.9, 0.8)
    counts = np.zeros(vocab)
    s = native.Search(params(vocab=vocab, max_length=n + 2, eos=[vocab + 5], seed=7))
    s.append_tokens(np.array([[1]], dtype=np.int32))
    for _ in range(n):
        s.score(logits.reshape(1, -1).copy(), "top_k_top_p", 10, 0.9, 0.8)
        counts[s.next_tokens()[0]] += 1
    assert set(np.nonzero(counts)[0]) <= set(want_ids.tolist())
    expect = np.zeros(vocab)
    expect[want_ids] = want_p
    assert 0.5 * np.abs(counts / n - expect).sum() < 0.03


def test_seed_reproducibility_and_checkpoint_restore():
    logits = np.random.RandomState(2).randn(1, 64).astype(np.float32)

    def run(seed, n):
        s = native.Search(params(vocab=64, max_length=40, eos=[99], seed=seed))
        s.append_tokens(np.array([[1]], dtype=np.int32))
        for _ in range(n):
            s.score(logits.copy(), "top_k", 20, 0.0, 1.0)
        return s
    a, b, c = run(5, 10), run(5, 10), run(6, 10)
    assert a.sequence(0).tolist() == b.sequence(0).tolist() != c.sequence(0).tolist()
    s = run(5, 4)
    cp = s.save()
    s.score(logits.copy(), "top_k", 20, 0.0, 1.0)
    first = s.next_tokens()[0]
    s.restore(cp)
    assert s.length == 5
    s.score(logits.copy(), "top_k", 20, 0.0, 1.0)
    assert s.next_tokens()[0] == first, "restoring a checkpoint also restores the RNG"


def test_beam_search_matches_bruteforce():
    """Fixed per-step distribution: beams must find the best 3-token continuation by total log-probability."""
    vocab, beams = 6, 3
    rng = np.random.RandomState(3)
    table = rng.randn(vocab, vocab).astype(np.float32) * 2     # next-token logits depend on the last token
    table[:, 0] = -30                                         # EOS (0) is never attractive
    s = native.Search(params(batch=1, beams=beams, vocab=vocab, max_length=4, length_penalty=1.0, num_return_sequences=3, eos=[0]))
    s.append_tokens(np.array([[2]], dtype=np.int32))
    while not s.is_done:
        last = [int(s.sequence(r)[-1]) for r in range(beams)]
        s.score(np.stack([table[t] for t in last]).copy(), "beam")
    s.finalize()
    lsm = table - np.log(np.exp(table).sum(-1, keepdims=True))
    best = sorted(((lsm[2, a] + lsm[a, b] + lsm[b, c], [2, a, b, c]) for a in range(vocab) for b in range(vocab) for c in range(vocab)),
                  key=lambda x: -x[0])
    got, score = s.hypothesis(0, 0)
    assert got.tolist() == best[0][1]
    assert abs(score - best[0][0] / 4 ** 1.0) < 1e-4, "hypotheses are ranked by sum_logprobs / len^length_penalty"


def test_beam_search_eos_hypotheses_and_early_stopping():
    vocab = 5
    s = native.Search(params(batch=1, beams=2, vocab=vocab, max_length=8, eos=[0], early_stopping=True, num_return_sequences=2))
    s.append_tokens(np.array([[3]], dtype=np.int32))
    step1 = np.log(np.array([[0.05, 0.6, 0.3, 0.025, 0.025]] * 2, dtype=np.float32))
    s.score(step1.copy(), "beam")
    assert sorted(s.next_tokens().tolist()) == [1, 2]
    eos_now = np.log(np.array([[0.9, 0.04, 0.03, 0.02, 0.01]] * 2, dtype=np.float32))
    s.score(eos_now.copy(), "beam")
    s.score(eos_now.copy(), "beam")
    assert s.is_done, "two finished hypotheses with early_stopping end the search"
    s.finalize()
    h0, sc0 = s.hypothesis(0, 0)
    h1, sc1 = s.hypothesis(0, 1)
    assert sc0 >= sc1 and h0.tolist()[0] == 3


def test_sampling_with_beams_is_rejected():
    s = native.Search(params(beams=2, vocab=8, max_length=6))
    s.append_tokens(np.array([[1]], dtype=np.int32))
    with pytest.raises(RuntimeError):
        s.score(np.zeros((2, 8), dtype=np.float32), "top_k", 3, 0.0, 1.0)


def test_device_path_commit_tokens_mirrors_host_rules():
    s = native.Search(params(batch=2, max_length=6))
    s.append_tokens(np.array([[3], [4]], dtype=np.int32))
    s.commit_tokens(np.array([0, 5], dtype=np.int32))
    s.commit_tokens(np.array([9, 0], dtype=np.int32))
    assert s.sequence(0).tolist() == [3, 0, 15] and s.sequence(1).tolist() == [4, 5, 0] and s.is_done


def test_append_validation():
    s = native.Search(params(batch=2, max_length=4))
    with pytest.raises(RuntimeError):
        s.append_tokens(np.zeros((3, 2), dtype=np.int32))
    with pytest.raises(RuntimeError):
        s.append_tokens(np.zeros((2, 9), dtype=np.int32))


def test_debug_bounds_mode_names_the_bad_index(monkeypatch):
    """OGB_DEBUG_BOUNDS: an out-of-range id / slot / row raises before any kernel (or reference op) touches memory."""
    import torch
    from onnxruntime_genai_b200 import ops
    monkeypatch.setattr(ops, "DEBUG_BOUNDS", True)
    table = torch.zeros(10, 8)
    ops.embedding(torch.tensor([0, 9], dtype=torch.int32), table)
    with pytest.raises(IndexError, match="embedding: ids holds 10"):
        ops.embedding(torch.tensor([0, 10], dtype=torch.int32), table)
    with pytest.raises(IndexError, match="gather_rows: rows holds -1"):
        ops.gather_rows(torch.zeros(4, 8), torch.tensor([-1], dtype=torch.int32))
    logits = torch.zeros(2, 16)
    with pytest.raises(IndexError, match="logits_edit: tokens holds 16"):
        ops.logits_edit(logits, torch.tensor([0], dtype=torch.int32), torch.tensor([16], dtype=torch.int32),
                        torch.tensor([0], dtype=torch.int32), torch.tensor([0.0]))
