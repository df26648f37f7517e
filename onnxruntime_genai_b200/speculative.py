"""Speculative decoding strategies: draft-model and n-gram proposers with one multi-token verify.

Behaviour follows the reference (src/speculative_decoding_strategy.cpp:142-938,
src/base_speculative_strategy.cpp:44-140, src/n_gram_decoding_strategy.cpp:70-189,
docs/SpeculativeDecoding.md): batch size 1, no beams; a round proposes K tokens (K from the
adaptive controller), verifies them with ONE target forward over [last token, d1..dK], accepts the
longest valid prefix (greedy: equal to the target argmax; sampling: u < min(1, p_t/p_d)), appends
the target's correction token at the first rejection or a bonus token when everything was
accepted, and rewinds both KV caches to the accepted length.  `generate_next_token` still yields
one token per call: extra accepted tokens are drained on the following calls.  After three rounds
that accepted nothing one round is skipped when `cooldown` is set.

What differs by design: the paged KV cache makes the rewind a length update (no copy); the greedy
accept scan runs on the device (`ogb_verify_greedy`), so a greedy round reads back K+2 integers
instead of K+1 rows of logits; the host-side controllers (adaptive K, cooldown, n-gram index,
sampled accept/correct math) are the C++ ones in native/speculative.h.
"""
from __future__ import annotations

import time
from collections import deque
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from . import ops
from .native_loader import native


class _SpecBase:
    def __init__(self, gen, spec: Dict[str, Any]):
        so = gen.search_opts
        if so["batch_size"] != 1:
            raise RuntimeError("speculative decoding requires batch_size 1")
        if so["num_beams"] != 1:
            raise RuntimeError("speculative decoding does not support beam search")
        if gen._guidance is not None and gen._guidance.ff:
            raise RuntimeError("speculative decoding cannot be combined with guidance fast-forward tokens")
        self.gen = gen
        self.max_k = int(spec.get("max_draft_tokens", 4))
        self.adaptive = native.AdaptiveK(self.max_k, int(spec.get("min_adaptive_k", 0)))
        self.cooldown = native.ZeroAcceptCooldown(bool(spec.get("cooldown", False)))
        self.pending: deque = deque()
        self._grammar_synced = False     # True while a plain step commits its token to the grammar itself
        self.s = dict(rounds=0, proposed=0, evaluated=0, accepted=0, committed=0, bonus=0, corrections=0, standard_steps=0,
                      cooldown_skips=0, empty_proposals=0, propose_ms=0.0, verify_ms=0.0)

    # hooks ------------------------------------------------------------------------------------
    def on_append(self, arr):
        self.pending.clear()

    def on_rewind(self, length: int):
        self.pending.clear()
        self.adaptive.reset()

    def stats(self) -> Dict[str, Any]:
        d = dict(self.s)
        d["effective_k"] = self.adaptive.k
        d["acceptance_rate"] = d["accepted"] / d["evaluated"] if d["evaluated"] else 0.0
        d["tokens_per_round"] = d["committed"] / d["rounds"] if d["rounds"] else 0.0
        d["k_increases"], d["k_decreases"] = self.adaptive.increases, self.adaptive.decreases
        return d

    # proposer interface -----------------------------------------------------------------------
    def propose(self, k: int):
        """Returns (tokens, dists): dists[i] is (ids, probs) of the distribution token i was drawn from, or
        None for a deterministic proposal."""
        raise NotImplementedError

    def after_round(self, committed: List[int], accepted: int, k: int):
        pass

    # one API call -----------------------------------------------------------------------------
    def _surface(self, token: int):
        g = self.gen
        g.search.commit_tokens(np.asarray([token], dtype=np.int32))
        if g._guidance is not None and not self._grammar_synced:
            g._guidance.commit_tokens(np.asarray([token], dtype=np.int32))
        if g.search.is_done:
            self.pending.clear()

    def step(self):
        g = self.gen
        if self.pending:
            self._surface(self.pending.popleft())
            return
        if g._fresh:                      # logits of the prompt are already there: plain step
            self._plain_step()
            return
        if self.cooldown.should_skip_round():
            self.s["cooldown_skips"] += 1
            self._plain_step()
            return
        room = g.search_opts["max_length"] - g.search.length
        k = min(self.adaptive.k, room - 1)
        if k < 1:
            self._plain_step()
            return
        t0 = time.perf_counter()
        draft, dists = self.propose(k)
        t1 = time.perf_counter()
        if not draft:
            self.s["empty_proposals"] += 1
            self._plain_step()
            return
        accepted, commit = self._verify(draft, dists)
        t2 = time.perf_counter()
        n_prop = len(draft)
        self.s["rounds"] += 1
        self.s["proposed"] += n_prop
        self.s["evaluated"] += min(n_prop, accepted + 1)
        self.s["accepted"] += accepted
        self.s["committed"] += len(commit)
        self.s["bonus" if accepted == n_prop else "corrections"] += 1
        self.s["propose_ms"] += (t1 - t0) * 1e3
        self.s["verify_ms"] += (t2 - t1) * 1e3
        self.adaptive.record(k, min(n_prop, accepted + 1), accepted, len(commit), n_prop == k, (t2 - t0) * 1e3)
        self.cooldown.record(min(n_prop, accepted + 1), accepted)
        self.after_round(commit, accepted, n_prop)
        self.pending.extend(commit[1:])
        self._surface(commit[0])

    def _plain_step(self):
        g = self.gen
        g._standard_step()                # (applies the grammar mask and advances the grammar itself)
        self.s["standard_steps"] += 1
        self.after_round([int(g.search.next_tokens()[0])], 0, 0)

    def _verify(self, draft: List[int], dists):
        g = self.gen
        st = g.state
        seq = g.search.sequence(0)
        n = len(seq)
        k = len(draft)
        base = st.kv_len[0]                       # == n - 1: the last committed token has not been fed
        recurrent = st.decoder.arch.has_linear_layers
        if recurrent:
            st.snapshot_recurrent()               # the verification pass feeds the drafts into the recurrent states as well
        with torch.no_grad():
            logits, _ = st.run([[int(seq[-1])] + list(draft)], want_all_logits=True)
        fed = list(draft)
        so = g.search_opts
        penalties = so["min_length"] > 0 or so["repetition_penalty"] != 1.0 or so["no_repeat_ngram_size"] > 0
        if g._guidance is not None:
            # Constrained decoding inside the round (reference: src/speculative_decoding_strategy.cpp:532, 944-1270): a CLONE of
            # the grammar cursor walks the draft; row i is masked with what the grammar allows after the prefix + draft[:i].  A draft
            # token the grammar forbids ends the walk: its row's mask rejects it, the rows after it are never consulted.  The
            # real cursor only advances when the committed tokens are surfaced.
            cursor = g._guidance.clone()
            logits = logits.float().clone()
            for i in range(k + 1):
                mask = cursor.compute_mask()                      # [1, words]
                row = logits[i:i + 1]
                if row.is_cuda:
                    ops.logits_bitmask(row, torch.from_numpy(mask).to(row.device))
                else:
                    bits = np.unpackbits(mask.view(np.uint8), bitorder="little")[:row.shape[1]].astype(bool)
                    row[0, torch.from_numpy(~bits)] = float("-inf")
                if i == k:
                    break
                allowed = bool((int(mask[0, draft[i] >> 5]) >> (draft[i] & 31)) & 1)
                if not allowed:
                    k = i                                          # rows beyond i belong to a continuation the grammar excludes
                    draft, dists = draft[:i + 1], dists[:i + 1]
                    logits = logits[:i + 1]
                    # verification sees k = i + 1 drafts with i + 1 rows: give it a last row (never reached: draft i is rejected)
                    logits = torch.cat([logits, logits[-1:]], dim=0)
                    k = i + 1
                    break
                cursor.commit_tokens(np.asarray([draft[i]], dtype=np.int32))
        if g.method == "greedy" and not penalties:
            if logits.is_cuda:
                am = ops.argmax(logits)
                acc = torch.empty(1, dtype=torch.int32, device=logits.device)
                com = torch.empty(k + 1, dtype=torch.int32, device=logits.device)
                d = torch.tensor(draft, dtype=torch.int32, device=logits.device)
                from .ops import _lib
                _lib.check(_lib.lib().ogb_verify_greedy(d.data_ptr(), am.data_ptr(), k, acc.data_ptr(), com.data_ptr(),
                                                        torch.cuda.current_stream().cuda_stream), "verify_greedy")
                accepted = int(acc.item())
                commit = com[:accepted + 1].tolist()
            else:
                accepted, commit, _ = native.verify_greedy(np.asarray(draft, dtype=np.int32), logits.float().numpy())
        elif logits.is_cuda and g.method != "greedy" and not penalties and 1 < g.k <= 1024 and g.t > 0:
            # rejection sampling on the device: one launch over the K + 1 rows, stateless randomness keyed by position
            accepted, commit, _ = ops.verify_sampled(logits.float(), draft, list(dists), g.k, g.p if 0 < g.p < 1 else 0.0, g.t,
                                                     g._seed, n)
        else:
            rows = np.ascontiguousarray(logits.float().cpu().numpy())
            if penalties:
                prefix = seq.tolist()
                eos = list(g.model.config.eos_token_ids)
                for i in range(k + 1):
                    cur = np.asarray(prefix + list(draft[:i]), dtype=np.int32)
                    native.apply_min_length(rows[i], len(cur), so["min_length"], eos)
                    native.apply_repetition_penalty(rows[i], cur, so["repetition_penalty"])
                    native.apply_no_repeat_ngram(rows[i], cur, so["no_repeat_ngram_size"])
            if g.method == "greedy":
                accepted, commit, _ = native.verify_greedy(np.asarray(draft, dtype=np.int32), rows)
            else:
                accepted, commit, _ = native.verify_sampled(np.asarray(draft, dtype=np.int32), list(dists), rows,
                                                            g.k if g.k > 1 else 0, g.p if 0 < g.p < 1 else 0.0, g.t, g.search)
        # keep the accepted prefix in the cache: [.., last, d1..d_accepted]; the correction / bonus token is unfed
        if recurrent and accepted < len(fed):
            # rejected drafts went through the recurrent states: put the saved states back and feed the kept tokens again (their
            # keys / values are rewritten with the same values)
            st.restore_recurrent()
            st.kv_len[0] = base
            with torch.no_grad():
                st.run([[int(seq[-1])] + fed[:accepted]])
        st.kv_len[0] = base + 1 + accepted
        g._fresh = False
        g._unfed_last = True
        return accepted, [int(t) for t in commit]


class NGramStrategy(_SpecBase):
    def __init__(self, gen, spec):
        super().__init__(gen, spec)
        if gen.search_opts["no_repeat_ngram_size"] > 0:
            raise RuntimeError("n-gram speculative decoding cannot be combined with no_repeat_ngram_size")
        self.index = native.NGramIndex(int(spec["ngram_size"]))
        self.chained = bool(spec.get("ngram_chained_lookup", False))
        self._synced = 0

    def _sync(self):
        seq = self.gen.search.sequence(0)
        if len(seq) < self._synced:
            self.index.reset(seq)
        else:
            self.index.append(seq[self._synced:])
        self._synced = len(seq)

    def on_rewind(self, length):
        super().on_rewind(length)
        self.index.reset(self.gen.search.sequence(0))
        self._synced = length

    def propose(self, k):
        self._sync()
        toks = self.index.propose(k, self.chained)
        return list(toks), [None] * len(toks)

    def stats(self):
        d = super().stats()
        d["ngram_hits"], d["ngram_misses"] = self.index.hits, self.index.misses
        return d


class DraftModelStrategy(_SpecBase):
    def __init__(self, gen, spec):
        super().__init__(gen, spec)
        if gen.search_opts["no_repeat_ngram_size"] > 0:
            raise RuntimeError("draft-model speculative decoding cannot be combined with no_repeat_ngram_size")
        from .api import SequenceState
        if gen.model.draft.arch.has_linear_layers:
            raise RuntimeError("the draft model's cache is cropped every round: a draft model with linear-attention layers is not supported")
        self.draft_state = SequenceState(gen.model.draft, 1, gen.search_opts["max_length"])

    def on_rewind(self, length):
        super().on_rewind(length)
        self.draft_state.rewind(0, max(0, length - 1))

    def propose(self, k):
        g, ds = self.gen, self.draft_state
        seq = g.search.sequence(0).tolist()
        toks: List[int] = []
        dists = []
        feed = seq[ds.kv_len[0]:]                 # catch up with the committed sequence (includes the unfed last token)
        sample = g.method != "greedy"
        if not sample and k > 0 and ds.decoder.device.type == "cuda":
            # greedy proposals never leave the device between draft steps: each step's argmax is the next step's input id,
            # and the k tokens come back in one copy
            picked = []
            with torch.no_grad():
                logits, _ = ds.run([feed])
                for i in range(k):
                    tok = ops.argmax(logits).to(torch.int32).reshape(1)
                    picked.append(tok)
                    if i + 1 < k:
                        logits, _ = ds.run([[0]], device_ids=tok)
            return torch.cat(picked).cpu().tolist(), [None] * k
        for _ in range(k):
            with torch.no_grad():
                logits, _ = ds.run([feed])
            if sample:
                row = logits[0].float().cpu().numpy()
                ids, probs = native.sampled_distribution(row, g.k if g.k > 1 else 0, g.p if 0 < g.p < 1 else 0.0, g.t)
                u = g.search.uniform()
                j = int(np.searchsorted(np.cumsum(probs), u, side="right"))
                t = int(ids[min(j, len(ids) - 1)])
                dists.append((ids, probs))
            else:
                t = int(ops.argmax(logits)[0]) if logits.is_cuda else int(torch.argmax(logits[0]))
                dists.append(None)
            toks.append(t)
            feed = [t]
        return toks, dists

    def after_round(self, committed, accepted, k):
        # the draft cache holds [.., last, d1..d_{k-1}]; keep what is still a prefix of the committed sequence
        n = self.gen.search.length + len(self.pending)  # not yet surfaced tokens count as committed
        valid = self.gen.state.kv_len[0]
        self.draft_state.kv_len[0] = min(self.draft_state.kv_len[0], valid)


def make_strategy(gen, spec: Dict[str, Any]):
    if gen.model.draft is not None:
        return DraftModelStrategy(gen, spec)
    if int(spec.get("ngram_size", 0)) > 0:
        return NGramStrategy(gen, spec)
    return None
