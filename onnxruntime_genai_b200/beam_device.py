"""Beam-search scorer that lives on the GPU (`csrc/beam_scorer.cu`).

`Generator` hands it the best 2 * num_beams candidates of every batch entry (still on the device, from
`ops.beam_candidates`); one kernel chooses the live continuations, files finished hypotheses, decides which entries are done
and appends the new column to the device-side token sequences.  What comes back per step is one small copy: a token and a
source row per beam plus the number of entries still open - the host needs the source rows to reorder the block tables of
the paged cache, and mirrors the tokens into its own `Sequences`.  The running beam scores never leave the device.

Reference: src/cuda/beam_search_scorer_cuda.cu:79-230 (Process / Finalize / AppendNextTokenToSequences) and its host driver
src/search_cuda.cpp (BeamSearch_Cuda::SelectTop); the host restatement of the same rules is native/search.cpp::BeamScorer.
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import numpy as np
import torch

from .ops import _lib

MAX_BEAMS, MAX_EOS = 32, 8


def supported(num_beams: int, eos_ids) -> bool:
    return 1 < num_beams <= MAX_BEAMS and len(eos_ids) <= MAX_EOS


class DeviceBeamScorer:
    def __init__(self, sequences: np.ndarray, batch: int, num_beams: int, max_length: int, pad_token_id: int, eos_ids, length_penalty: float,
                 early_stopping: bool, device: torch.device):
        """sequences: int32 [batch * num_beams, length] - the rows generated so far (the prompt, repeated for every beam)."""
        rows, length = sequences.shape
        assert rows == batch * num_beams and 1 <= length <= max_length and supported(num_beams, eos_ids)
        self.batch, self.nb, self.rows, self.L = batch, num_beams, rows, max_length
        self.pad, self.lp, self.early = int(pad_token_id), float(length_penalty), int(bool(early_stopping))
        self.eos = (ctypes.c_int32 * max(1, len(eos_ids)))(*[int(e) for e in eos_ids])
        self.n_eos = len(eos_ids)
        self.device = device
        i32 = dict(dtype=torch.int32, device=device)
        self.seq = torch.zeros(2, rows, max_length, **i32)
        self.seq[0, :, :length] = torch.from_numpy(np.ascontiguousarray(sequences, dtype=np.int32)).to(device)
        self.cur, self.length = 0, length
        # only the first beam of an entry starts live, so that identical beams do not all pick the same token
        self.scores = torch.full((batch, num_beams), -1e9, dtype=torch.float32, device=device)
        self.scores[:, 0] = 0.0
        self.scores = self.scores.reshape(rows).contiguous()
        self.hyp_tokens = torch.zeros(batch, num_beams, max_length, **i32)
        self.hyp_len = torch.zeros(batch, num_beams, **i32)
        self.hyp_order = torch.zeros(batch, num_beams, **i32)
        self.hyp_score = torch.zeros(batch, num_beams, dtype=torch.float32, device=device)
        self.hyp_count = torch.zeros(batch, **i32)
        self.done = torch.zeros(batch, **i32)
        self.out = torch.zeros(2 * rows + 2, **i32)
        self.out[2 * rows] = batch
        self.host_out = torch.zeros(2 * rows + 2, dtype=torch.int32).pin_memory()
        self.finalized = False

    def _state_args(self):
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        return (p(self.scores), p(self.hyp_tokens), p(self.hyp_len), p(self.hyp_score), p(self.hyp_order), p(self.hyp_count), p(self.done),
                p(self.out), self.batch, self.nb, self.L, self.pad, self.early, self.lp, self.eos, self.n_eos,
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))

    def step(self, cand_scores: torch.Tensor, cand_tokens: torch.Tensor, cand_beams: torch.Tensor) -> Tuple[np.ndarray, np.ndarray, bool]:
        """Candidates [batch, 2 * num_beams] (fp32, int32, int32; best first) -> (next token per row, source row per row, all
        entries done)."""
        if self.length >= self.L:
            raise RuntimeError("beam search: the sequences are already at max_length")
        assert cand_scores.is_cuda and cand_scores.dtype == torch.float32 and cand_scores.is_contiguous()
        assert cand_tokens.dtype == torch.int32 and cand_beams.dtype == torch.int32 and cand_tokens.is_contiguous() and cand_beams.is_contiguous()
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = _lib.lib().ogb_beam_scorer_step(p(cand_scores), p(cand_tokens), p(cand_beams), p(self.seq[0]), p(self.seq[1]), self.cur, self.length,
                                             *self._state_args())
        _lib.check(rc, "beam_scorer_step")
        self.cur ^= 1
        self.length += 1
        self.host_out.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        h = self.host_out.numpy()
        if h[2 * self.rows + 1]:
            raise RuntimeError("beam search: fewer than num_beams live candidates")
        return h[:self.rows].copy(), h[self.rows:2 * self.rows].copy(), int(h[2 * self.rows]) == 0

    def beam_scores(self) -> torch.Tensor:
        return self.scores

    def sequences(self) -> torch.Tensor:
        """The device copy of the running sequences, int32 [rows, length]."""
        return self.seq[self.cur, :, :self.length]

    def finalize(self) -> List[List[Tuple[np.ndarray, float]]]:
        """Ranked hypotheses of every batch entry, best first: [(tokens, score), ...]."""
        if not self.finalized:
            p = lambda t: ctypes.c_void_p(t.data_ptr())
            rc = _lib.lib().ogb_beam_scorer_finalize(p(self.seq[0]), p(self.seq[1]), self.cur, self.length, *self._state_args())
            _lib.check(rc, "beam_scorer_finalize")
            self.finalized = True
        order, count = self.hyp_order.cpu().numpy(), self.hyp_count.cpu().numpy()
        lens, scores, toks = self.hyp_len.cpu().numpy(), self.hyp_score.cpu().numpy(), self.hyp_tokens.cpu().numpy()
        out = []
        for b in range(self.batch):
            ranked = []
            for rank in range(int(count[b])):
                slot = int(order[b, rank])
                ranked.append((toks[b, slot, :int(lens[b, slot])].copy(), float(scores[b, slot])))
            out.append(ranked)
        return out
