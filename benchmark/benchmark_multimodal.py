"""Multimodal benchmark (counterpart of the reference's benchmark/python/benchmark_multimodal.py): image or audio
pre-processing time, encoder time, time to first token and generation rate through the public API.

    python benchmark/benchmark_multimodal.py -i <model_dir> --image a.png [b.png ...] -p "<|image_1|>\\nDescribe." -g 64
    python benchmark/benchmark_multimodal.py --synthetic whisper-base -g 64          # random weights, 30 s of noise
    python benchmark/benchmark_multimodal.py --synthetic vit-llm -g 64               # ViT-L/14-sized tower on a 1B-sized decoder

Wall clock around the API calls with a device synchronisation on both sides; one JSON object per run.
"""
import argparse
import json
import os
import statistics
import sys
import tempfile
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def synthetic_dir(kind: str, provider: str):
    from onnxruntime_genai_b200.models.arch import ArchConfig
    from onnxruntime_genai_b200.models.builder import export_vision_language, export_whisper, whisper_decoder_arch
    from onnxruntime_genai_b200.models.encoder import EncoderConfig
    d = tempfile.mkdtemp(prefix="ogb_mm_")
    prec = "bf16" if provider == "cuda" else "fp32"
    if kind == "whisper-base":
        enc = EncoderConfig(kind="audio", hidden_size=512, num_layers=6, num_heads=8, intermediate_size=2048, num_mel_bins=80,
                            max_source_positions=1500)
        arch = whisper_decoder_arch(51865, 512, 6, 8, 2048, encoder_hidden_size=512, context_length=448, bos_token_id=50257,
                                    eos_token_id=-1, pad_token_id=50256)
        export_whisper(arch, enc, d, prec, provider)
    else:
        arch = ArchConfig(model_type="llama", vocab_size=32064, hidden_size=2048, num_layers=16, num_heads=32, num_kv_heads=8, head_dim=64,
                          intermediate_size=8192, context_length=4096, bos_token_id=1, eos_token_id=-1, pad_token_id=0)
        vis = EncoderConfig(kind="vision", hidden_size=1024, num_layers=24, num_heads=16, intermediate_size=4096, image_size=336,
                            patch_size=14, projection_size=2048)
        export_vision_language(arch, vis, d, image_token_id=32000, precision=prec, execution_provider=provider)
    return d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-i", "--input_folder", default="")
    ap.add_argument("--synthetic", default="", choices=["", "whisper-base", "vit-llm"])
    ap.add_argument("-e", "--execution_provider", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--image", nargs="*", default=[])
    ap.add_argument("--audio", nargs="*", default=[])
    ap.add_argument("-p", "--prompt", default="")
    ap.add_argument("-g", "--generation_length", type=int, default=64)
    ap.add_argument("-r", "--repetitions", type=int, default=3)
    ap.add_argument("-w", "--warmup", type=int, default=1)
    a = ap.parse_args()
    import torch
    import onnxruntime_genai_b200 as og
    model_dir = a.input_folder or synthetic_dir(a.synthetic or "vit-llm", a.execution_provider)
    cfg = og.Config(model_dir)
    if a.execution_provider == "cpu":
        cfg.clear_providers()
    model = og.Model(cfg)
    sync = (lambda: torch.cuda.synchronize()) if model.device_type == "cuda" else (lambda: None)
    rng = np.random.RandomState(0)
    audio = model.encoder is not None
    runs = []
    for it in range(a.warmup + a.repetitions):
        t0 = time.perf_counter()
        if a.input_folder:
            proc = model.create_multimodal_processor()
            inputs = (proc([a.prompt] * len(a.audio), audios=og.Audios.open(*a.audio)) if audio
                      else proc(a.prompt, images=og.Images.open(*a.image)))
        elif audio:
            from onnxruntime_genai_b200.multimodal import log_mel_spectrogram
            feats = log_mel_spectrogram(rng.randn(30 * 16000).astype(np.float32) * 0.1)
            inputs = og.NamedTensors(audio_features=feats[None], input_ids=np.asarray([[50258, 50259, 50359, 50363]], dtype=np.int32))
        else:
            from onnxruntime_genai_b200.multimodal import preprocess_image
            px = preprocess_image(rng.randint(0, 255, size=(480, 640, 3), dtype=np.uint8), 336, [0.5] * 3, [0.5] * 3)
            ids = [1] + [32000] * 576 + rng.randint(3, 30000, size=32).tolist()
            inputs = og.NamedTensors(pixel_values=px[None], input_ids=np.asarray([ids], dtype=np.int32))
        t_pre = time.perf_counter()
        p = og.GeneratorParams(model)
        n_prompt = int(np.asarray(inputs["input_ids"]).shape[1])
        p.set_search_options(max_length=n_prompt + a.generation_length + 1, batch_size=int(np.asarray(inputs["input_ids"]).shape[0]))
        gen = og.Generator(model, p)
        sync()
        t1 = time.perf_counter()
        gen.set_inputs(inputs)          # encoder + prompt
        gen.generate_next_token()
        sync()
        t2 = time.perf_counter()
        n = 1
        while n < a.generation_length and not gen.is_done():
            gen.generate_next_token()
            n += 1
        sync()
        t3 = time.perf_counter()
        if it >= a.warmup:
            runs.append({"preprocess_s": t_pre - t0, "ttft_s": t2 - t1, "decode_s": t3 - t2, "tokens": n})
    med = lambda k: statistics.median(r[k] for r in runs)
    print(json.dumps({"model": a.input_folder or a.synthetic or "vit-llm", "modality": "audio" if audio else "vision", "prompt_tokens": n_prompt,
                      "preprocess_ms_p50": round(med("preprocess_s") * 1e3, 3), "ttft_ms_p50": round(med("ttft_s") * 1e3, 3),
                      "tpot_ms_p50": round(med("decode_s") / max(1, runs[0]["tokens"] - 1) * 1e3, 4),
                      "decode_tokens_per_s": round((runs[0]["tokens"] - 1) / med("decode_s"), 1), "repetitions": len(runs),
                      "device": str(model.device)}))


if __name__ == "__main__":
    main()
