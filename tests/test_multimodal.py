"""Multimodal models: a Whisper-style encoder-decoder (audio encoder -> cross-attention decoder) and a vision-language
model (ViT encoder + projector -> image features spliced into the prompt embeddings), through the processor and the
Generator API, against the independent dense references in tests/dense_reference.py."""
import copy
import json
import os
import wave

import numpy as np
import pytest
import torch

import onnxruntime_genai_b200 as og
import dense_reference as dense
from helpers import make_tokenizer
from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import (export_vision_language, export_whisper, random_state_dict, whisper_decoder_arch)
from onnxruntime_genai_b200.models.encoder import EncoderConfig, random_encoder_state_dict
from onnxruntime_genai_b200.multimodal import log_mel_spectrogram, mel_filter_bank


def _whisper_dir(d, provider="cpu", precision="fp32", hidden=64, heads=4, vocab=None):
    vocab = vocab or make_tokenizer(d)
    enc = EncoderConfig(kind="audio", hidden_size=hidden, num_layers=2, num_heads=heads, intermediate_size=2 * hidden, num_mel_bins=16,
                        max_source_positions=50)
    arch = whisper_decoder_arch(vocab, hidden, 2, heads, 2 * hidden, encoder_hidden_size=hidden, context_length=64,
                                bos_token_id=0, eos_token_id=1, pad_token_id=1)
    dsd, esd = random_state_dict(arch, seed=2, std=0.1), random_encoder_state_dict(enc, seed=3, std=0.1)
    export_whisper(copy.deepcopy(arch), enc, d, precision, provider, decoder_state_dict=dsd, encoder_state_dict=esd, num_frames=100)
    return arch, enc, dsd, esd


def _tone_wav(path, seconds=0.4, rate=16000, freq=440.0):
    t = np.arange(int(seconds * rate)) / rate
    x = (0.3 * np.sin(2 * np.pi * freq * t) * 32767).astype("<i2")
    with wave.open(path, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(rate)
        w.writeframes(x.tobytes())


def test_mel_filter_bank_and_log_mel_shapes():
    fb = mel_filter_bank(80, 400, 16000)
    assert fb.shape == (80, 201) and (fb >= 0).all()
    # every filter is a single triangle: one rise, one fall; neighbouring centres increase
    peaks = fb.argmax(1)
    assert (np.diff(peaks) >= 0).all() and peaks[0] > 0
    # Slaney normalisation: area of each triangle is about 1 Hz^-1 * bin width
    widths = fb.sum(1) * (8000 / 200)
    assert np.allclose(widths, 1.0, atol=0.35)
    t = np.arange(16000) / 16000
    m = log_mel_spectrogram(np.sin(2 * np.pi * 1000 * t).astype(np.float32), n_frames=120)
    assert m.shape == (80, 120) and m.max() <= 1.6 and m.max() - m.min() <= 2.0 + 1e-5
    loud = m[:, :90].mean(1).argmax()
    assert abs(_centre_hz(fb[loud]) - 1000) < 120        # the 1 kHz tone lands in the filter centred near 1 kHz
    assert m[:, 110:].max() < m[:, :90].max()            # the zero padding after the clip is quieter


def _centre_hz(row):
    return row.argmax() * 8000 / 200


def test_whisper_generate_matches_dense_reference(tmp_path):
    d = str(tmp_path)
    arch, enc, dsd, esd = _whisper_dir(d)
    wav1, wav2 = os.path.join(d, "a.wav"), os.path.join(d, "b.wav")
    _tone_wav(wav1, freq=440.0)
    _tone_wav(wav2, freq=1200.0, seconds=0.25, rate=8000)       # resampled to 16 kHz by the processor
    model = og.Model(d)
    assert model.type == "whisper" and model.arch.cross_attention and model.arch.learned_positions
    proc = model.create_multimodal_processor()
    inputs = proc(["<s>hello", "<s>hello"], audios=og.Audios.open(wav1, wav2))
    feats = inputs["audio_features"]
    assert feats.shape == (2, 16, 100) and inputs["input_ids"].shape[0] == 2
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=24, batch_size=2)
    g = og.Generator(model, p)
    g.set_inputs(inputs)
    lg = g.get_logits()[:, 0, :]
    seqs = [inputs["input_ids"][b].tolist() for b in range(2)]
    encs = [dense.whisper_encoder(enc, esd, torch.from_numpy(feats[b])) for b in range(2)]
    for b in range(2):
        want = dense.logits(arch, dsd, seqs[b], encoder_hidden=encs[b])[-1].numpy()
        np.testing.assert_allclose(lg[b], want, rtol=2e-3, atol=3e-4)
    assert np.abs(lg[0] - lg[1]).max() > 1e-3, "the two clips must give different logits"
    for _ in range(5):
        g.generate_next_token()
        nxt = g.get_next_tokens()
        for b in range(2):
            seqs[b].append(int(nxt[b]))
        if g.is_done():
            break
        lg = g.get_logits()[:, 0, :]
        for b in range(2):
            want = dense.logits(arch, dsd, seqs[b], encoder_hidden=encs[b])[-1].numpy()
            np.testing.assert_allclose(lg[b], want, rtol=2e-3, atol=4e-4)
    assert isinstance(proc.decode(g.get_sequence(0)), str)


def test_whisper_beam_search_shares_the_encoder_cache(tmp_path):
    d = str(tmp_path)
    _whisper_dir(d)
    model = og.Model(d)
    feats = np.random.RandomState(0).randn(1, 16, 100).astype(np.float32)
    outs = []
    for beams in (1, 3):
        p = og.GeneratorParams(model)
        p.set_search_options(max_length=16, num_beams=beams, num_return_sequences=1, batch_size=1, length_penalty=1.0)
        g = og.Generator(model, p)
        g.set_inputs(og.NamedTensors(audio_features=feats, input_ids=np.array([[0, 5, 9]], dtype=np.int32)))
        assert g.state.cross.pool.shape[2] == 64          # one copy of the 50 encoder positions, shared by the beams
        while not g.is_done():
            g.generate_next_token()
        outs.append(g.get_sequence(0).tolist())
    assert outs[0][:3] == outs[1][:3] == [0, 5, 9] and len(outs[1]) > 3


def test_decoder_without_audio_inputs_is_refused(tmp_path):
    d = str(tmp_path)
    _whisper_dir(d)
    model = og.Model(d)
    g = og.Generator(model, og.GeneratorParams(model))
    with pytest.raises(RuntimeError, match="encoder inputs"):
        g.append_tokens(np.array([[0, 3]], dtype=np.int32))


def _vlm_dir(d, provider="cpu", precision="fp32", hidden=64):
    vocab = make_tokenizer(d)
    arch = ArchConfig(model_type="phi3", vocab_size=vocab, hidden_size=hidden, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=hidden // 4,
                      intermediate_size=2 * hidden, context_length=256, bos_token_id=0, eos_token_id=1, pad_token_id=1)
    vis = EncoderConfig(kind="vision", hidden_size=48, num_layers=2, num_heads=4, intermediate_size=96, image_size=28, patch_size=7,
                        projection_size=hidden)
    dsd, vsd = random_state_dict(arch, seed=4, std=0.1), random_encoder_state_dict(vis, seed=5, std=0.1)
    export_vision_language(copy.deepcopy(arch), vis, d, image_token_id=vocab - 1, precision=precision, execution_provider=provider,
                           decoder_state_dict=dsd, vision_state_dict=vsd)
    return arch, vis, dsd, vsd


def test_vision_language_prompt_matches_dense_reference(tmp_path):
    from PIL import Image
    d = str(tmp_path)
    arch, vis, dsd, vsd = _vlm_dir(d)
    rng = np.random.RandomState(1)
    paths = []
    for i, shape in enumerate([(40, 52, 3), (31, 28, 3)]):
        paths.append(os.path.join(d, f"im{i}.png"))
        Image.fromarray(rng.randint(0, 255, size=shape, dtype=np.uint8)).save(paths[-1])
    model = og.Model(d)
    assert model.type == "phi3v" and model.vision is not None
    proc = model.create_multimodal_processor()
    inputs = proc("<|image_1|>\nhello <|image_2|> world", images=og.Images.open(*paths))
    ids = inputs["input_ids"][0].tolist()
    tok = model.image_token_id
    assert ids.count(tok) == 2 * vis.num_patches and inputs["pixel_values"].shape == (2, 3, 28, 28)
    with pytest.raises(RuntimeError, match="placeholders"):
        proc("no image here", images=og.Images.open(paths[0]))
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=len(ids) + 8)
    g = og.Generator(model, p)
    g.set_inputs(inputs)
    feats = torch.cat([dense.vision_encoder(vis, vsd, torch.from_numpy(inputs["pixel_values"][i])) for i in range(2)])
    emb = dsd["model.embed_tokens.weight"].float()[torch.tensor(ids)]
    emb[torch.tensor(ids) == tok] = feats
    want = dense.logits(arch, dsd, ids, inputs_embeds=emb)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=3e-4)
    # decode continues from the mixed prompt with ordinary token embeddings
    g.generate_next_token()
    ids.append(int(g.get_next_tokens()[0]))
    emb = torch.cat([emb, dsd["model.embed_tokens.weight"].float()[ids[-1]][None]])
    want = dense.logits(arch, dsd, ids, inputs_embeds=emb)[-1].numpy()
    np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=2e-3, atol=4e-4)


def test_text_only_model_has_no_processor(tmp_path):
    from helpers import tiny_model_dir
    d, _ = tiny_model_dir(str(tmp_path))
    with pytest.raises(RuntimeError, match="no vision or speech"):
        og.Model(d).create_multimodal_processor()


def test_encoder_head_padding_is_exact():
    """Head sizes the attention kernel does not have run zero-padded to the next supported size: same output."""
    from onnxruntime_genai_b200.models.encoder import TransformerEncoder
    cfg = EncoderConfig(kind="vision", hidden_size=48, num_layers=2, num_heads=4, intermediate_size=96, image_size=28, patch_size=7,
                        projection_size=32)
    sd = random_encoder_state_dict(cfg, seed=7, std=0.1)
    px = torch.randn(2, 3, 28, 28)
    a, _ = TransformerEncoder(cfg, sd, "cpu", torch.float32).encode_images(px)
    padded = TransformerEncoder(cfg, sd, "cpu", torch.float32, pad_heads=True)
    assert padded.head_pad == 64 and padded.layers[0].qkv_w.shape[0] == 3 * 4 * 64
    b, _ = padded.encode_images(px)
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    want = torch.cat([dense.vision_encoder(cfg, sd, px[i]) for i in range(2)])
    torch.testing.assert_close(a, want, rtol=2e-4, atol=2e-4)


def test_whisper_alignment_heads_record_cross_attention_scores(tmp_path):
    """`alignment_heads` (an int32 [n, 2] input of (layer, head) pairs) makes the generator record the scaled query-key
    scores of those cross-attention heads for every token fed: [rows, n, tokens, frames], readable as the `cross_qk` output
    (word-level timestamps are computed from them).  Token-by-token decoding and one prefill of the same tokens agree."""
    d = str(tmp_path)
    arch, enc, dsd, esd = _whisper_dir(d)
    model = og.Model(d)
    feats = np.random.RandomState(0).randn(2, 16, 100).astype(np.float32)
    heads = np.array([[0, 1], [1, 0], [1, 3]], dtype=np.int32)
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=12, batch_size=2)
    g = og.Generator(model, p)
    g.set_model_input("alignment_heads", heads)
    g.set_inputs(og.NamedTensors(audio_features=feats, input_ids=np.array([[0, 5, 9], [0, 7, 3]], dtype=np.int32)))
    for _ in range(4):
        g.generate_next_token()
    g.get_logits()                                            # runs the newest token
    qk = g.get_output("cross_qk")
    frames = g.state.max_cross_len
    n_tok = g.token_count()
    assert qk.shape == (2, 3, n_tok, frames) and np.isfinite(qk).all() and np.abs(qk).max() > 0
    # the same tokens as one prompt: identical scores (the recorded rows do not depend on how the tokens were fed)
    g2 = og.Generator(model, p)
    g2.set_model_input("alignment_heads", heads)
    g2.set_inputs(og.NamedTensors(audio_features=feats, input_ids=np.stack([g.get_sequence(0), g.get_sequence(1)]).astype(np.int32)))
    qk2 = g2.get_output("cross_qk")
    np.testing.assert_allclose(qk2, qk, rtol=1e-4, atol=1e-5)
    assert np.abs(qk[0] - qk[1]).max() > 1e-3                 # the two clips differ
    with pytest.raises(RuntimeError, match="out of range"):
        g2.set_model_input("alignment_heads", np.array([[9, 0]], dtype=np.int32))
    g3 = og.Generator(model, p)
    with pytest.raises(RuntimeError, match="alignment_heads"):
        g3.get_output("cross_qk")


def test_hf_whisper_checkpoint_directory(tmp_path):
    """A `WhisperForConditionalGeneration` directory through create_model: encoder.onnx + decoder.onnx, and the decoder's logits over
    log-mel features against the family's implementation in `transformers` (reference: src/python/py/models/builders/whisper.py)."""
    import json
    transformers = pytest.importorskip("transformers")
    from safetensors.torch import save_file
    from onnxruntime_genai_b200.models.builder import create_model
    cfg = transformers.WhisperConfig(vocab_size=120, d_model=64, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4, decoder_attention_heads=4,
                                     encoder_ffn_dim=128, decoder_ffn_dim=96, num_mel_bins=16, max_source_positions=50, max_target_positions=40,
                                     decoder_start_token_id=3, bos_token_id=1, eos_token_id=2, pad_token_id=2, suppress_tokens=None, begin_suppress_tokens=None)
    torch.manual_seed(0)
    m = transformers.WhisperForConditionalGeneration(cfg).float().eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "embed_positions" in n and "encoder" in n:
                continue                       # the fixed sinusoid table
            p.copy_(1 + 0.1 * torch.randn_like(p) if ("layer_norm" in n and n.endswith("weight")) else torch.randn_like(p) * 0.1)
    src = tmp_path / "hf"
    src.mkdir()
    sd = {k: v.detach().clone().contiguous() for k, v in m.state_dict().items() if k != "proj_out.weight"}
    save_file(sd, str(src / "model.safetensors"))
    d = cfg.to_dict()
    d["architectures"] = ["WhisperForConditionalGeneration"]
    (src / "config.json").write_text(json.dumps(d))
    out = str(tmp_path / "out")
    create_model(str(src), out, "fp32", "cpu")
    model = og.Model(out)
    assert model.type == "whisper" and model.arch.num_layers == 2 and model.arch.intermediate_size == 96
    feats = np.random.RandomState(0).randn(1, 16, 100).astype(np.float32)
    ids = [3, 7, 9, 11]
    p = og.GeneratorParams(model)
    p.set_search_options(max_length=20, batch_size=1)
    g = og.Generator(model, p)
    g.set_inputs(og.NamedTensors(audio_features=feats, input_ids=np.array([ids], dtype=np.int32)))
    seq = list(ids)
    for _ in range(4):
        with torch.no_grad():
            want = m(input_features=torch.from_numpy(feats), decoder_input_ids=torch.tensor([seq])).logits[0, -1].numpy()
        np.testing.assert_allclose(g.get_logits().reshape(-1), want, rtol=3e-3, atol=4e-4)
        g.generate_next_token()
        seq.append(int(g.get_next_tokens()[0]))
        if g.is_done():
            break
