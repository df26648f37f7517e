"""Speech transducers (reference: src/models/parakeet.cpp EmitNextToken for TDT, nemotron_speech.cpp for RNN-T, silero_vad.cpp,
streaming_processor.cpp).  The oracles restate the greedy searches and the recurrent cells with torch's own LSTM cell."""
import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
from onnxruntime_genai_b200 import streaming
from onnxruntime_genai_b200.models.encoder import EncoderConfig, random_encoder_state_dict
from onnxruntime_genai_b200.models.transducer import TransducerConfig, export_transducer, random_state_dict

ENC = EncoderConfig(kind="audio", hidden_size=32, num_layers=2, num_heads=4, intermediate_size=64, num_mel_bins=16, max_source_positions=400)


def _cfg(tdt: bool, **kw):
    return TransducerConfig(vocab_size=21, blank_id=20, encoder_hidden=32, pred_hidden=24, pred_layers=2, joint_hidden=28,
                            tdt_durations="0,1,2,4" if tdt else "", max_symbols_per_step=3, **kw)


def _export(tmp_path, tdt, seed=0, vad=None, **kw):
    cfg = _cfg(tdt, **kw)
    sd = random_state_dict(cfg, seed=seed, std=0.6)
    esd = random_encoder_state_dict(ENC, seed=seed, std=0.2)
    d = str(tmp_path)
    export_transducer(cfg, ENC, d, "parakeet_tdt" if tdt else "nemotron_speech", "fp32", "cpu", state_dict=sd, encoder_state_dict=esd,
                      num_mels=16, chunk_samples=3200, vad=vad)
    return d, cfg, sd


class Oracle:
    """Greedy RNN-T / TDT over given encoder frames, with torch.nn.LSTMCell as the prediction network."""

    def __init__(self, cfg, sd):
        self.c, self.sd = cfg, {k: v.double() for k, v in sd.items()}
        self.cells = []
        for l in range(cfg.pred_layers):
            cell = torch.nn.LSTMCell(cfg.pred_hidden, cfg.pred_hidden).double()
            p = f"predictor.lstm.{l}."
            with torch.no_grad():
                cell.weight_ih.copy_(self.sd[p + "w_ih"]); cell.weight_hh.copy_(self.sd[p + "w_hh"])
                cell.bias_ih.copy_(self.sd[p + "b_ih"]); cell.bias_hh.copy_(self.sd[p + "b_hh"])
            self.cells.append(cell)

    def predict(self, tok, state):
        x = self.sd["predictor.embed.weight"][tok][None]
        new = []
        with torch.no_grad():
            for cell, (h, c) in zip(self.cells, state):
                h, c = cell(x, (h, c))
                new.append((h, c))
                x = h
        return x[0], new

    def joint(self, frame, pred):
        z = torch.relu(self.sd["joiner.enc.weight"] @ frame + self.sd["joiner.enc.bias"] + self.sd["joiner.pred.weight"] @ pred + self.sd["joiner.pred.bias"])
        return self.sd["joiner.out.weight"] @ z + self.sd["joiner.out.bias"]

    def decode(self, frames):
        c = self.c
        zero = lambda: torch.zeros(1, c.pred_hidden, dtype=torch.float64)
        pred, state = self.predict(c.blank_id, [(zero(), zero()) for _ in range(c.pred_layers)])
        durs, V = c.durations, c.vocab_size
        t, count, out = 0, 0, []
        while t < frames.shape[0]:
            lg = self.joint(frames[t].double(), pred)
            tok = int(torch.argmax(lg[:V]))
            if durs:
                lo = 1 if tok == c.blank_id else 0
                skip = durs[lo + int(torch.argmax(lg[V + lo:]))]
            else:
                skip = 1 if tok == c.blank_id else 0
            if tok != c.blank_id:
                out.append(tok)
                count += 1
                pred, state = self.predict(tok, state)
            if skip > 0:
                count = 0
            elif count >= c.max_symbols_per_step:
                count, skip = 0, 1
            t += skip
        return out


def _generate(model, feats):
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=400)
    g = og.Generator(model, p)
    g.set_inputs({"audio_features": feats[None]})
    while not g.is_done():
        g.generate_next_token()
    seq = g.get_sequence(0).tolist()
    blank = model.decoder.cfg.blank_id
    assert seq[0] == blank and seq[-1] == blank          # starts from the blank token, ends with it as the end-of-sequence id
    return seq[1:-1]


@pytest.mark.parametrize("tdt", [True, False])
def test_greedy_transducer_search_matches_the_oracle(tmp_path, tdt):
    d, cfg, sd = _export(tmp_path, tdt, seed=3)
    model = og.Model(d)
    assert model.type == ("parakeet_tdt" if tdt else "nemotron_speech")
    feats = np.random.RandomState(0).randn(16, 120).astype(np.float32)
    got = _generate(model, feats)
    frames = model.decoder.encode(torch.from_numpy(feats))
    want = Oracle(cfg, sd).decode(frames)
    assert got == want and len(got) >= 5
    if not tdt:      # RNN-T never emits more than max_symbols_per_step tokens on one frame
        assert len(got) <= cfg.max_symbols_per_step * frames.shape[0]


def test_chunked_encoding_searches_every_frame_once(tmp_path):
    """chunk_frames / left_context_frames: every chunk is encoded with the audio before it as context, the search walks the
    chunk's own frames; the oracle runs over the same frames put together by hand."""
    d, cfg, sd = _export(tmp_path, True, seed=5, chunk_frames=40, left_context_frames=20)
    model = og.Model(d)
    feats = np.random.RandomState(1).randn(16, 130).astype(np.float32)
    got = _generate(model, feats)
    f = torch.from_numpy(feats)
    pieces = []
    for s in range(0, 130, 40):
        lo = max(0, s - 20)
        pieces.append(model.decoder.encode(f[:, lo:min(130, s + 40)])[(s - lo) // 2:])
    assert sum(p.shape[0] for p in pieces) == 65
    assert got == Oracle(cfg, sd).decode(torch.cat(pieces))


def test_streaming_front_end_and_session(tmp_path):
    d, cfg, sd = _export(tmp_path, True, seed=7)
    model = og.Model(d)
    rng = np.random.RandomState(2)
    audio = (rng.randn(3200 * 6) * 0.1).astype(np.float32)
    # the frames do not depend on how the samples are cut up
    whole = streaming.log_mel_frames(audio, 16)
    proc = model.create_streaming_processor()
    parts = []
    for s in range(0, len(audio), 1234):
        f = proc.process(audio[s:s + 1234])
        if f is not None:
            parts.append(f)
    tail = proc.flush()
    if tail is not None:
        parts.append(tail)
    np.testing.assert_allclose(np.concatenate(parts, axis=1), whole, rtol=1e-5, atol=1e-5)
    # one feed of everything equals the generator over the same frames
    sess = model.create_streaming_session()
    toks = sess.feed(audio) + sess.finish()
    n = (3200 * 6 - 400) // 160 + 1
    assert whole.shape[1] == n
    assert toks == _generate(model, whole) and len(toks) >= 3
    # piecewise feeding emits tokens as the audio arrives
    sess = model.create_streaming_session()
    counts = [len(sess.feed(audio[s:s + 3200])) for s in range(0, len(audio), 3200)]
    rest = sess.finish()
    assert sum(counts) + len(rest) == len(sess.tokens) and sum(1 for c in counts if c) >= 2
    with pytest.raises(RuntimeError):
        sess.feed(audio[:10])


def test_voice_activity_gate(tmp_path):
    """The detector's cell against torch's LSTM cell, and the chunk rule: silence is kept for context until
    max(prefix_padding, silence_duration) chunks of it in a row, then dropped until speech comes back."""
    g = torch.Generator().manual_seed(1)
    vsd = {n: torch.randn(s, generator=g) * 0.3 for n, s in streaming.vad_weight_shapes(16000, 12).items()}
    streaming.export_vad(str(tmp_path), vsd)
    d, cfg, sd = _export(tmp_path, True, seed=9, vad={"filename": "vad.onnx", "threshold": 0.5, "silence_duration_ms": 400, "prefix_padding_ms": 200})
    model = og.Model(d)
    det = streaming.VoiceActivityDetector.load(str(tmp_path / "vad.onnx"), 16000, 0.5)
    cell = torch.nn.LSTMCell(12, 128)
    with torch.no_grad():
        cell.weight_ih.copy_(vsd["vad.lstm.w_ih"]); cell.weight_hh.copy_(vsd["vad.lstm.w_hh"])
        cell.bias_ih.copy_(vsd["vad.lstm.b"]); cell.bias_hh.zero_()
    rng = np.random.RandomState(3)
    h, c, ctx = torch.zeros(1, 128), torch.zeros(1, 128), torch.zeros(64)
    for _ in range(4):
        win = rng.randn(512).astype(np.float32)
        x = torch.cat([ctx, torch.from_numpy(win)])
        with torch.no_grad():
            h, c = cell(torch.relu(vsd["vad.in.weight"] @ x + vsd["vad.in.bias"])[None], (h, c))
            want = float(torch.sigmoid(vsd["vad.out.weight"] @ h[0] + vsd["vad.out.bias"])[0])
        assert abs(det.process_window(win) - want) < 1e-5
        ctx = x[-64:]
    with pytest.raises(RuntimeError):
        det.process_window(win[:100])

    proc = model.create_streaming_processor()
    assert proc.vad is not None and proc.silence_chunks == 2 and proc.prefix_chunks == 1      # 200 ms chunks
    speech = iter([True, False, False, False, False, True, False])
    proc.vad.contains_speech = lambda chunk: next(speech)
    kept = []
    for i in range(7):
        before = proc.dropped_chunks
        proc.process(np.zeros(3200, dtype=np.float32))
        kept.append(proc.dropped_chunks == before)
    assert kept == [True, True, False, False, False, True, True]
