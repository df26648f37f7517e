"""Marian translation model with an SSRU decoder (reference: src/models/marian.cpp: encoder session over the source tokens,
decoder session fed one token + the recurrent states per step, states reordered by the beam indices).

The oracle below restates the model from its formulas one source sentence and one target token at a time, with none of the
implementation's batching, padding, caches or kernels."""
import math

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200.models.marian import MarianConfig, export_marian, random_state_dict, sinusoid_positions

CFG = MarianConfig(vocab_size=53, hidden_size=32, encoder_layers=2, decoder_layers=3, num_heads=4, ffn_size=48, activation="swish",
                   max_positions=40, bos_token_id=0, eos_token_id=0, pad_token_id=1)


def _ln(x, w, b, eps):
    mu = x.mean()
    var = ((x - mu) ** 2).mean()
    return (x - mu) / math.sqrt(var + eps) * w + b


def _attend(q, keys, values, heads):
    """q [H], keys / values [T, H] -> [H], head by head."""
    H = q.shape[0]
    d = H // heads
    out = torch.zeros(H, dtype=torch.float64)
    for h in range(heads):
        sl = slice(h * d, (h + 1) * d)
        s = keys[:, sl] @ q[sl] / math.sqrt(d)
        p = torch.softmax(s, dim=0)
        out[sl] = p @ values[:, sl]
    return out


class Oracle:
    def __init__(self, cfg, sd):
        self.c = cfg
        self.w = {k: v.double() for k, v in sd.items()}
        self.pos = sinusoid_positions(cfg.max_positions, cfg.hidden_size).double()

    def lin(self, x, name):
        y = self.w[name + ".weight"] @ x
        return y + self.w[name + ".bias"] if name + ".bias" in self.w else y

    def act(self, x):
        return torch.relu(x) if self.c.activation == "relu" else x * torch.sigmoid(x)

    def ffn(self, x, p):
        return self.lin(self.act(self.lin(x, p + "ffn.w1")), p + "ffn.w2")

    def embed(self, tok, pos):
        return self.w["shared.embed.weight"][tok] * math.sqrt(self.c.hidden_size) + self.pos[pos]

    def encode(self, src):
        c = self.c
        xs = [self.embed(t, i) for i, t in enumerate(src)]
        for l in range(c.encoder_layers):
            p = f"encoder.layers.{l}."
            K = torch.stack([self.lin(x, p + "self_attn.k") for x in xs])
            V = torch.stack([self.lin(x, p + "self_attn.v") for x in xs])
            nxt = []
            for x in xs:
                a = self.lin(_attend(self.lin(x, p + "self_attn.q"), K, V, c.num_heads), p + "self_attn.o")
                y = _ln(x + a, self.w[p + "attn_norm.weight"], self.w[p + "attn_norm.bias"], c.norm_eps)
                nxt.append(_ln(y + self.ffn(y, p), self.w[p + "ffn_norm.weight"], self.w[p + "ffn_norm.bias"], c.norm_eps))
            xs = nxt
        return torch.stack(xs)

    def step(self, tok, t, cells, enc):
        c = self.c
        x = self.embed(tok, t)
        new_cells = []
        for l in range(c.decoder_layers):
            p = f"decoder.layers.{l}."
            f = torch.sigmoid(self.lin(x, p + "ssru.wf"))
            cell = f * cells[l] + (1 - f) * self.lin(x, p + "ssru.w")
            new_cells.append(cell)
            x = _ln(x + torch.relu(cell), self.w[p + "ssru_norm.weight"], self.w[p + "ssru_norm.bias"], c.norm_eps)
            K = torch.stack([self.lin(e, p + "cross_attn.k") for e in enc])
            V = torch.stack([self.lin(e, p + "cross_attn.v") for e in enc])
            a = self.lin(_attend(self.lin(x, p + "cross_attn.q"), K, V, c.num_heads), p + "cross_attn.o")
            x = _ln(x + a, self.w[p + "cross_norm.weight"], self.w[p + "cross_norm.bias"], c.norm_eps)
            x = _ln(x + self.ffn(x, p), self.w[p + "ffn_norm.weight"], self.w[p + "ffn_norm.bias"], c.norm_eps)
        return self.w["shared.embed.weight"] @ x + self.w["decoder.output.bias"], new_cells

    def greedy(self, src, n):
        enc = self.encode(src)
        cells = [torch.zeros(self.c.hidden_size, dtype=torch.float64) for _ in range(self.c.decoder_layers)]
        tok, out, all_logits = self.c.bos_token_id, [], []
        for t in range(n):
            logits, cells = self.step(tok, t, cells, enc)
            all_logits.append(logits)
            tok = int(torch.argmax(logits))
            out.append(tok)
            if tok == self.c.eos_token_id:
                break
        return out, all_logits


@pytest.fixture(scope="module")
def marian_dir(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("marian"))
    sd = random_state_dict(CFG, seed=3, std=0.25)
    sd["decoder.output.bias"][CFG.eos_token_id] = -4.0       # keep random weights from ending the sentence at once
    export_marian(CFG, d, "fp32", "cpu", state_dict=sd)
    return d, sd


def test_marian_greedy_matches_the_per_token_oracle(marian_dir):
    d, sd = marian_dir
    model = og.Model(d)
    assert model.type == "marian-ssru"
    oracle = Oracle(CFG, sd)
    rng = np.random.RandomState(0)
    for n_src in (1, 7, 12):
        src = rng.randint(2, CFG.vocab_size, size=n_src).astype(np.int32)
        want, want_logits = oracle.greedy(src.tolist(), 9)
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=n_src + 9)
        g = og.Generator(model, p)
        g.append_tokens(src[None, :])
        got = []
        for t in range(len(want)):
            np.testing.assert_allclose(g.get_logits()[0, 0], want_logits[t].float().numpy(), rtol=2e-4, atol=2e-4)
            g.generate_next_token()
            got.append(int(g.get_next_tokens()[0]))
        assert got == want
        assert g.get_sequence(0).tolist() == src.tolist() + want


def test_marian_batch_with_padding_and_beams(marian_dir):
    """A padded batch decodes every sentence as it decodes alone; beam search returns ranked hypotheses whose best is at least
    as likely as greedy decoding, and a second search over the same generator after rewind_to(0) repeats the first."""
    d, sd = marian_dir
    model = og.Model(d)
    oracle = Oracle(CFG, sd)
    rng = np.random.RandomState(1)
    a, b = rng.randint(2, CFG.vocab_size, size=9).astype(np.int32), rng.randint(2, CFG.vocab_size, size=4).astype(np.int32)
    batch = np.full((2, 9), CFG.pad_token_id, dtype=np.int32)
    batch[0], batch[1, :4] = a, b
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=9 + 8, batch_size=2)
    g = og.Generator(model, p)
    g.append_tokens(batch)
    while not g.is_done():
        g.generate_next_token()
    for i, src in enumerate((a, b)):
        want, _ = oracle.greedy(src.tolist(), 8)
        got = g.get_sequence(i).tolist()[9:]
        assert got[:len(want)] == want

    def beam():
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=9 + 8, num_beams=3, num_return_sequences=3, length_penalty=1.0, early_stopping=False)
        g = og.Generator(model, p)
        g.append_tokens(a[None, :])
        while not g.is_done():
            g.generate_next_token()
        first = [g.get_sequence(i).tolist() for i in range(3)]
        return g, first

    g, first = beam()
    assert len({tuple(s) for s in first}) == 3 and all(s[:9] == a.tolist() for s in first)

    def loglik(seq):
        enc = oracle.encode(a.tolist())
        cells = [torch.zeros(CFG.hidden_size, dtype=torch.float64) for _ in range(CFG.decoder_layers)]
        tok, total = CFG.bos_token_id, 0.0
        for t, nxt in enumerate(seq):
            logits, cells = oracle.step(tok, t, cells, enc)
            total += float(torch.log_softmax(logits, dim=0)[nxt])
            tok = nxt
        return total

    greedy, _ = oracle.greedy(a.tolist(), 8)
    best = first[0][9:]
    assert loglik(best) / len(best) >= loglik(greedy) / len(greedy) - 1e-6
    _, again = beam()
    assert again == first


def test_marian_refuses_what_it_cannot_do(marian_dir):
    d, _ = marian_dir
    model = og.Model(d)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=20)
    g = og.Generator(model, p)
    g.append_tokens(np.asarray([[5, 6, 7]], dtype=np.int32))
    g.generate_next_token()
    with pytest.raises(RuntimeError):
        g.rewind_to(2)
    g.rewind_to(0)
    g.append_tokens(np.asarray([[8, 9]], dtype=np.int32))
    g.generate_next_token()
    assert g.token_count() == 3
