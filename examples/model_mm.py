"""Vision-language and speech models through the multimodal processor (counterpart of the reference's
examples/python/model-mm.py and whisper.py).

    python examples/model_mm.py -m <vlm_dir> --image cat.png -p "<|image_1|>\nWhat is in this picture?"
    python examples/model_mm.py -m <whisper_dir> --audio clip.wav -p "<|startoftranscript|><|en|><|transcribe|><|notimestamps|>"
"""
import argparse

import onnxruntime_genai_b200 as og


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("-m", "--model", required=True)
    ap.add_argument("-p", "--prompt", default="")
    ap.add_argument("--image", nargs="*", default=[])
    ap.add_argument("--audio", nargs="*", default=[])
    ap.add_argument("--max_length", type=int, default=448)
    ap.add_argument("--num_beams", type=int, default=1)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    cfg = og.Config(a.model)
    if a.cpu:
        cfg.clear_providers()
    model = og.Model(cfg)
    processor = model.create_multimodal_processor()
    if a.audio:
        audios = og.Audios.open(*a.audio)
        inputs = processor([a.prompt] * len(audios), audios=audios)
        batch = len(audios)
    else:
        inputs = processor(a.prompt, images=og.Images.open(*a.image) if a.image else None)
        batch = 1
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=a.max_length, batch_size=batch, num_beams=a.num_beams, num_return_sequences=1)
    gen = og.Generator(model, params)
    gen.set_inputs(inputs)
    if batch == 1 and a.num_beams == 1:
        stream = processor.create_stream()
        while not gen.is_done():
            gen.generate_next_token()
            print(stream.decode(int(gen.get_next_tokens()[0])), end="", flush=True)
        print()
    else:
        while not gen.is_done():
            gen.generate_next_token()
        for i in range(batch):
            print(f"[{i}] {processor.decode(gen.get_sequence(i * a.num_beams))}")


if __name__ == "__main__":
    main()
