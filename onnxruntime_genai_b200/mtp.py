"""Multi-token-prediction (MTP) self-speculation: `og.MtpGenerator(model, head_dir, params)`.

Reference: src/mtp_generator.{h,cpp} and examples/python/qwen-3.6-mtp.md — the main model exposes its
last hidden state, a one-layer MTP head takes (embedding of the newest token, hidden state of the
position before it) and drafts the token after it; drafted tokens are verified by one main forward over
[newest token, drafts...] and the longest matching prefix plus the main model's own next token is kept.

Head checkpoint (`export_mtp_head`): a one-layer decoder graph (same naming contract as the main
exporter) plus three initializers: `mtp.enorm.weight`, `mtp.hnorm.weight` (RMSNorm of the token
embedding and of the incoming hidden state) and `mtp.fc.MatMul.weight` `[2H, H]` (projection of their
concatenation).  Embedding table and LM head are shared with the main model.

The head is a regular `DecoderModel` with one layer fed through `inputs_embeds`; its KV cache is a
second paged cache that is rewound together with the main one.  Greedy verification uses the device
accept kernel (`ogb_verify_greedy`).
"""
from __future__ import annotations

import copy
import os
from typing import Any, Dict, List, Optional

import numpy as np
import torch

from . import ops
from .api import Config, Generator, GeneratorParams, Model, SequenceState
from .models.arch import ArchConfig
from .models.decoder import StepInputs
from .speculative import _SpecBase


def export_mtp_head(arch: ArchConfig, out_dir: str, precision: str = "bf16", execution_provider: str = "cuda", seed: int = 1,
                    std: float = 0.02, state_dict: Optional[Dict[str, torch.Tensor]] = None) -> str:
    """Writes `mtp.onnx` (+ data) and its genai_config.json into out_dir (random weights unless state_dict is given;
    extra keys: mtp.enorm.weight [H], mtp.hnorm.weight [H], mtp.fc.weight [H, 2H])."""
    from .models.builder import export_model, random_tensor
    from .utils import onnx_proto as op
    head = copy.deepcopy(arch)
    head.num_layers = 1
    head.tie_embeddings = False
    if head.layer_types is not None:
        head.layer_types = ["full_attention"]      # the head's one layer attends, whatever mix the main stack has
    head.sliding_layers = None if head.sliding_layers is None else []
    head.no_rope_layers = None
    export_model(head, out_dir, precision, execution_provider, state_dict=state_dict, seed=seed, std=std, filename="mtp.onnx")
    H = arch.hidden_size
    extra = {"mtp.enorm.weight": (H,), "mtp.hnorm.weight": (H,), "mtp.fc.weight": (H, 2 * H)}
    tensors = {}
    for name, shape in extra.items():
        t = state_dict[name] if state_dict is not None and name in state_dict else (
            torch.ones(shape) if name.endswith("norm.weight") else random_tensor(name, shape, seed, std))
        tensors[name] = t.float()
    np.savez(os.path.join(out_dir, "mtp_extra.npz"), **{k: v.numpy() for k, v in tensors.items()})
    return out_dir


def mtp_state_dict_from_hf(arch: ArchConfig, sd: Dict[str, torch.Tensor]) -> Optional[Dict[str, torch.Tensor]]:
    """The multi-token-prediction tensors of a Hugging Face checkpoint (`mtp.fc`, `mtp.pre_fc_norm_embedding`, `mtp.pre_fc_norm_hidden`,
    `mtp.layers.0.*`, `mtp.norm`; reference: src/python/py/models/builders/qwen_mtp.py) under the names `export_mtp_head` reads.  The
    embedding table and the LM head are the main model's.  None when the checkpoint has no such tensors."""
    if not any(k.startswith("mtp.") for k in sd):
        return None
    out = {}
    for k, v in sd.items():
        if k.startswith("mtp.layers.0."):
            out["model.layers.0." + k[len("mtp.layers.0."):]] = v
        elif k == "mtp.norm.weight":
            out["model.norm.weight"] = v
        elif k == "mtp.fc.weight":
            out[k] = v
        elif k == "mtp.pre_fc_norm_embedding.weight":
            out["mtp.enorm.weight"] = v.float() + arch.norm_offset      # zero-centred norms store the offset from one
        elif k == "mtp.pre_fc_norm_hidden.weight":
            out["mtp.hnorm.weight"] = v.float() + arch.norm_offset
        elif k in ("model.embed_tokens.weight", "lm_head.weight"):
            out[k] = v
    if "lm_head.weight" not in out and "model.embed_tokens.weight" in out:
        out["lm_head.weight"] = out["model.embed_tokens.weight"]
    return out


class MtpHead:
    def __init__(self, main: Model, head_dir: str):
        cfg = Config(head_dir)
        if main.device_type == "cpu":
            cfg.clear_providers()
        self.model = Model(cfg)
        if self.model.arch.hidden_size != main.arch.hidden_size or self.model.arch.vocab_size != main.arch.vocab_size:
            raise RuntimeError("MTP head does not match the main model (hidden size / vocabulary)")
        z = np.load(os.path.join(head_dir, "mtp_extra.npz"))
        dev, dt = main.device, main.dtype
        self.enorm = torch.from_numpy(z["mtp.enorm.weight"]).to(dev, dt)
        self.hnorm = torch.from_numpy(z["mtp.hnorm.weight"]).to(dev, dt)
        self.fc = torch.from_numpy(z["mtp.fc.weight"]).to(dev, dt).contiguous()
        dec = self.model.decoder
        dec.embed = main.decoder.embed            # shared embedding table and LM head
        dec.lm_head_w, dec.lm_head_b = main.decoder.lm_head_w, main.decoder.lm_head_b
        self.main = main

    def inputs(self, tokens: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
        a = self.main.arch
        e = ops.embedding(tokens, self.main.decoder.embed, a.embed_scale)
        e, _ = ops.norm(e, self.enorm, a.norm_eps)
        h, _ = ops.norm(hidden.contiguous(), self.hnorm, a.norm_eps)
        return ops.linear(torch.cat([e, h], dim=-1).contiguous(), self.fc)


class _MtpStrategy(_SpecBase):
    """Proposer that drafts with the MTP head; plugged into the Generator like the other speculative strategies."""

    def __init__(self, gen: Generator, head: MtpHead, spec):
        super().__init__(gen, spec)
        self.head = head
        self.hstate = SequenceState(head.model.decoder, 1, gen.search_opts["max_length"])
        self.last_hidden: Optional[torch.Tensor] = None   # main hidden state of the newest position in the main cache

    def on_rewind(self, length):
        super().on_rewind(length)
        self.hstate.rewind(0, 0)
        self.last_hidden = None

    def _head_step(self, token: int, hidden: torch.Tensor):
        """Feeds (token, hidden) at the head's next position; returns (logits [1, V], head hidden [1, H])."""
        st = self.hstate
        dev = self.head.main.device
        emb = self.head.inputs(torch.tensor([token], dtype=torch.int32, device=dev), hidden.view(1, -1))
        p = st.kv_len[0]
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
        s = StepInputs(input_ids=i32([token]), positions=i32([p]), slot_mapping=i32([p]), cu_seqlens=i32([0, 1]), past_lens=i32([p]),
                       block_table=st.block_table, logits_rows=i32([0]), max_q_len=1, max_kv_len=p + 1, inputs_embeds=emb)
        with torch.no_grad():
            logits = st.decoder.forward(s, st.kv)
        st.kv_len[0] = p + 1
        return logits, st.decoder.last_hidden

    def propose(self, k):
        g = self.gen
        if self.last_hidden is None:
            return [], []
        seq = g.search.sequence(0)
        # The head keeps its own compact cache: entry j of a round pairs a token with the hidden state that
        # preceded it (main hidden state for the first entry, the head's own output afterwards).
        self._round_base = self.hstate.kv_len[0]
        toks: List[int] = []
        tok, hid = int(seq[-1]), self.last_hidden
        for _ in range(k):
            logits, hid = self._head_step(tok, hid)
            tok = int(ops.argmax(logits)[0]) if logits.is_cuda else int(torch.argmax(logits[0]))
            toks.append(tok)
        return toks, [None] * len(toks)

    def _verify(self, draft, dists):
        accepted, commit = super()._verify(draft, dists)
        # the main hidden state of the last position that stays in the main cache feeds the next round
        self.last_hidden = self.gen.model.decoder.last_hidden[accepted].detach().clone()
        # head entries whose token turned out right stay: the first one plus one per accepted draft
        self.hstate.kv_len[0] = self._round_base + min(accepted + 1, len(draft))
        return accepted, commit

    def after_round(self, committed, accepted, k):
        if k == 0:   # plain step: the main model ran the prompt or one token; remember its newest hidden state
            self.last_hidden = self.gen.model.decoder.last_hidden[-1].detach().clone()


class MtpGenerator(Generator):
    """Generator whose proposals come from an MTP head.  The head proposes its argmax; verification is greedy, or with
    do_sample the deterministic-proposal form of rejection sampling (accept d with probability p_target(d), otherwise draw the
    correction from p_target without d; reference: src/mtp_generator.cpp:638, 891)."""

    def __init__(self, model: Model, head_dir: str, params: GeneratorParams):
        super().__init__(model, params)
        so = self.search_opts
        if so["batch_size"] != 1 or so["num_beams"] != 1:
            raise RuntimeError("MtpGenerator requires batch_size 1 and num_beams 1")
        self.head = MtpHead(model, head_dir)
        spec = dict(params.speculative)
        self._strategy = _MtpStrategy(self, self.head, spec)
