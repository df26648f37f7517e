"""Speculative decoding inside the continuous-batching engine: every decoding request of a step may carry K proposed
tokens, the target model verifies all proposals of the batch in ONE packed forward (each request contributes the rows
[pending token, d1..dK]), and the step transaction commits, per request, the accepted prefix plus the target's correction
or bonus token.

Reference behaviour (batch 1 only there): src/speculative_decoding_strategy.cpp:460-792 (round: propose, multi-token
verify, accept loop, correction / bonus token), src/base_speculative_strategy.cpp:44-140 (draft-model proposer),
src/n_gram_decoding_strategy.cpp:70-189 (n-gram proposer), src/speculative_sampling.h:39-177 (accept / correction
math).  What is different here:

  * batched: proposals are staged in the native request (`Request.set_draft`), the scheduler counts them against the token
    budget, the paged cache keeps the slots of accepted drafts and rejected ones are simply overwritten later
    (`EngineCore.commit_speculative`); a failed step rolls back like any other;
  * proposals are deterministic (n-gram continuation, or the draft model's argmax), so sampled verification is the
    deterministic-proposal form: accept d with probability p_target(d), otherwise draw from p_target without d;
  * the draft model shares the target's block tables: its own (smaller) paged cache is addressed by the same block ids and
    slots, so there is no second block manager; it re-feeds the last two committed tokens at the start of a round, which
    repairs its cache after a fully accepted round without per-request bookkeeping;
  * greedy verification reads back one argmax id per row, never logits;
  * under tensor parallelism every rank proposes and verifies identically (same gathered logits, same Philox keys).
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..models.decoder import PagedKVCache, StepInputs
from ..native_loader import native


class EngineSpeculator:
    def __init__(self, engine, spec: Dict[str, Any]):
        self.engine = engine
        self.model = engine.model
        self.max_k = max(1, min(16, int(spec.get("max_draft_tokens", 4))))
        self.ngram_size = int(spec.get("ngram_size", 0))
        self.chained = bool(spec.get("ngram_chained_lookup", False))
        self.draft = self.model.draft
        self.stats = dict(rounds=0, proposed=0, accepted=0, committed=0, requests=0)
        self._ngram: Dict[int, Any] = {}          # request id -> (NGramIndex, tokens indexed so far)
        self.draft_kv: Optional[PagedKVCache] = None
        if self.draft is not None:
            kv = engine.kv
            self.draft_kv = PagedKVCache(self.draft.arch, kv.num_blocks, kv.block_size, self.model.device, self.model.dtype,
                                         kv_heads=self.draft.kv_heads_local, conv_channels=self.draft.conv_channels_local)
        elif self.ngram_size <= 0:
            raise RuntimeError("speculative decoding needs a draft model (model.draft) or speculative.ngram_size > 0")

    @property
    def acceptance_rate(self) -> float:
        return self.stats["accepted"] / self.stats["proposed"] if self.stats["proposed"] else 0.0

    def forget(self, request_id: int) -> None:
        self._ngram.pop(request_id, None)

    # ------------------------------------------------------------------------------------------ proposals
    def _eligible(self, nat) -> bool:
        """Decoding requests with exactly one pending token whose owned blocks already cover the draft positions (the engine
        runs with a block look-ahead of max_k + 1; a request fresh out of prefill gets there after one plain step)."""
        if nat.is_prefill or nat.pending != 1 or nat.draft_count or nat.status not in (native.RequestStatus.Active, native.RequestStatus.Assigned):
            return False
        eng = self.engine
        if nat.id in eng._with_processors:
            return False
        need = nat.num_tokens + self.max_k
        return len(nat.blocks()) * eng.block_size >= need and nat.num_tokens + 1 < nat.options.max_length

    def propose(self) -> None:
        """Stages proposals on every eligible request (before the step is planned)."""
        reqs = [r._native for r in self.engine._by_native.values() if r._native is not None and self._eligible(r._native)]
        if not reqs:
            return
        if self.draft is not None:
            drafts = self._propose_draft(reqs)
        else:
            drafts = [self._propose_ngram(nat) for nat in reqs]
        for nat, d in zip(reqs, drafts):
            if len(d):
                nat.set_draft(np.asarray(d, dtype=np.int32))

    def _propose_ngram(self, nat) -> List[int]:
        idx, seen = self._ngram.get(nat.id, (None, 0))
        toks = nat.tokens()
        if idx is None:
            idx = native.NGramIndex(self.ngram_size)
        if len(toks) < seen:
            idx.reset(toks)
        else:
            idx.append(toks[seen:])
        self._ngram[nat.id] = (idx, len(toks))
        return list(idx.propose(self.max_k, self.chained))

    def _propose_draft(self, reqs) -> List[List[int]]:
        """K greedy draft steps over the eligible requests, on the device: the first step feeds each request's last two
        committed tokens (positions n - 2 and n - 1), the following ones the previous argmax; one readback at the end."""
        dev, K, bs = self.model.device, self.max_k, self.engine.block_size
        B = len(reqs)
        ids, pos, slots, past, cu = [], [], [], [], [0]
        cols = max(len(r.blocks()) for r in reqs)
        table = np.full((B, cols), -1, dtype=np.int32)
        for i, r in enumerate(reqs):
            toks, blocks = r.tokens(), r.blocks()
            n = len(toks)
            first = max(0, n - 2)
            table[i, :len(blocks)] = blocks
            for p in range(first, n):
                ids.append(int(toks[p])); pos.append(p); slots.append(blocks[p // bs] * bs + p % bs)
            past.append(first)
            cu.append(len(ids))
        t = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)
        table_d = torch.from_numpy(table).to(dev)
        s = StepInputs(input_ids=t(ids), positions=t(pos), slot_mapping=t(slots), cu_seqlens=t(cu), past_lens=t(past), block_table=table_d,
                       logits_rows=t([c - 1 for c in cu[1:]]), max_q_len=2, max_kv_len=max(len(r.tokens()) for r in reqs) + K)
        out = torch.empty(K, B, dtype=torch.int32, device=dev)
        with torch.no_grad():
            logits = self.draft.forward(s, self.draft_kv)
            out[0].copy_(ops.argmax(logits))
            if K > 1:
                # one token per request from here on; the inputs move on by one position on the device
                n_tok = [len(r.tokens()) for r in reqs]
                cur = StepInputs(input_ids=out[0].clone(), positions=t(n_tok), slot_mapping=t([r.blocks()[n // bs] * bs + n % bs for r, n in zip(reqs, n_tok)]),
                                 cu_seqlens=t(list(range(B + 1))), past_lens=t(n_tok), block_table=table_d, logits_rows=t(list(range(B))),
                                 max_q_len=1, max_kv_len=s.max_kv_len)
                scratch = torch.zeros(B, dtype=torch.int32, device=dev)
                for k in range(1, K):
                    logits = self.draft.forward(cur, self.draft_kv)
                    out[k].copy_(ops.argmax(logits))
                    if k + 1 < K:
                        ops.decode_advance(out[k], cur.input_ids, cur.positions, cur.past_lens, cur.slot_mapping, scratch, table_d, bs)
        host = out.t().contiguous().cpu().numpy()
        return [host[i].tolist() for i in range(B)]

    def mirror_prefill(self, s: StepInputs) -> None:
        """The draft model processes the same packed step as the target (prompt chunks and plain decode tokens), so that its
        cache, addressed by the same slots, follows the committed sequences."""
        if self.draft is None:
            return
        with torch.no_grad():
            self.draft.forward(s, self.draft_kv)

    # ------------------------------------------------------------------------------------------ verification
    def verify(self, plan, logits: torch.Tensor, row_of: List[int]):
        """logits: one fp32 row per (entry, fed token that needs a prediction), in plan order; row_of[i]: first row of entry i
        (entries that do not sample have none).  Returns (accepted[], next_token[]) for core.commit_speculative."""
        n = len(plan.entries)
        accepted = np.zeros(n, dtype=np.int32)
        nxt = np.zeros(n, dtype=np.int32)
        def is_greedy(o):
            return (not o.do_sample) or o.top_k == 1 or o.temperature == 0
        # Constrained requests: row 0 of an entry was masked by the engine with the grammar's current state; rows 1..k take the
        # masks of a cloned cursor that walks the drafts (a draft the grammar forbids is masked in its own row, hence rejected
        # there, and the rows after it are never consulted)
        guided = self.engine._guidance
        if guided:
            for i, e in enumerate(plan.entries):
                gp = guided.get(e.request.id) if e.samples else None
                k = e.request.draft_count if (gp is not None and not e.is_prefill) else 0
                if k == 0:
                    continue
                toks = e.request.tokens()
                drafts = [int(x) for x in toks[len(toks) - k:]]
                cursor = gp.clone()
                for j in range(1, k + 1):
                    prev = cursor.compute_mask()
                    d = drafts[j - 1]
                    if not (int(prev[0, d >> 5]) >> (d & 31)) & 1:
                        break
                    cursor.commit_tokens(np.asarray([d], dtype=np.int32))
                    mask = cursor.compute_mask()
                    row = logits[row_of[i] + j: row_of[i] + j + 1]
                    if row.is_cuda:
                        ops.logits_bitmask(row, torch.from_numpy(mask.copy()).to(row.device))
                    else:
                        bits = np.unpackbits(mask.view(np.uint8), bitorder="little")[:row.shape[1]].astype(bool)
                        row[0, torch.from_numpy(~bits)] = float("-inf")
        greedy = [i for i, e in enumerate(plan.entries) if e.samples and is_greedy(e.request.options)]
        sampled = [i for i, e in enumerate(plan.entries) if e.samples and not is_greedy(e.request.options)]
        am = None
        if greedy:
            am = ops.argmax(logits).cpu().numpy() if logits.is_cuda else torch.argmax(logits.float(), dim=-1).numpy()
        for i in greedy:
            e = plan.entries[i]
            k = e.request.draft_count if not e.is_prefill else 0
            toks = e.request.tokens()
            drafts = toks[len(toks) - k:] if k else []
            a = 0
            while a < k and int(am[row_of[i] + a]) == int(drafts[a]):
                a += 1
            accepted[i], nxt[i] = a, int(am[row_of[i] + a])
        for i in sampled:
            e = plan.entries[i]
            k = e.request.draft_count if not e.is_prefill else 0
            o = e.request.options
            toks = e.request.tokens()
            drafts = [int(x) for x in toks[len(toks) - k:]] if k else []
            rows = logits[row_of[i]:row_of[i] + k + 1]
            tk, tp_, tt = o.resolve()
            first_pos = len(toks) - k
            if rows.is_cuda and 1 < tk <= 1024 and tt > 0:
                a, commit, _ = ops.verify_sampled(rows.float(), drafts, [None] * k, int(tk), float(tp_) if 0 < tp_ < 1 else 0.0, float(tt),
                                                  int(e.request.seed), first_pos)
            else:
                a, commit = _verify_sampled_host(rows.float().cpu().numpy(), drafts, int(tk), float(tp_), float(tt), int(e.request.seed), first_pos)
            accepted[i], nxt[i] = a, int(commit[-1])
        st = self.stats
        for i, e in enumerate(plan.entries):
            k = e.request.draft_count if (e.samples and not e.is_prefill) else 0
            if k:
                st["rounds"] += 1
                st["proposed"] += k
                st["accepted"] += int(accepted[i])
                st["committed"] += int(accepted[i]) + 1
        return accepted, nxt


def _verify_sampled_host(rows: np.ndarray, drafts: List[int], top_k: int, top_p: float, temperature: float, seed: int, first_pos: int):
    """Deterministic-proposal rejection sampling on the host (CPU models): accept draft d at row i with probability p_i(d), else
    draw the correction from p_i without d; after K acceptances the bonus token comes from the last row.  Randomness is keyed by
    (seed, position) like the device sampler."""
    commit: List[int] = []
    a = 0
    for i in range(len(drafts) + 1):
        ids, probs = native.sampled_distribution(rows[i], top_k if top_k > 1 else 0, top_p if 0 < top_p < 1 else 0.0, temperature)
        rng = np.random.Generator(np.random.Philox(key=seed & ((1 << 64) - 1), counter=[first_pos + i, 0x5BEC, 0, 0]))
        if i < len(drafts):
            d = drafts[i]
            where = np.nonzero(ids == d)[0]
            p_d = float(probs[where[0]]) if len(where) else 0.0
            if rng.random() < p_d:
                commit.append(d)
                a += 1
                continue
            probs = probs.copy()
            if len(where):
                probs[where[0]] = 0.0
            tot = probs.sum()
            if tot <= 0:
                commit.append(int(ids[0]))
                break
            probs = probs / tot
        j = int(np.searchsorted(np.cumsum(probs), rng.random(), side="right"))
        commit.append(int(ids[min(j, len(ids) - 1)]))
        break
    return a, commit
