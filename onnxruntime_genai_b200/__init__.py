"""onnxruntime_genai_b200: a Blackwell-native (B200, sm_100a) generative-inference runtime with the
public API of onnxruntime-genai.

    import onnxruntime_genai_b200 as og
    model = og.Model("path/to/model_dir")           # genai_config.json + model.onnx (+ .data)
    tokenizer = og.Tokenizer(model)
    params = og.GeneratorParams(model)
    params.set_search_options(max_length=256, do_sample=True, top_k=50, top_p=0.9, temperature=0.7)
    generator = og.Generator(model, params)
    generator.append_tokens(tokenizer.encode("Hello"))
    while not generator.is_done():
        generator.generate_next_token()
    print(tokenizer.decode(generator.get_sequence(0)))
"""
__version__ = "0.1.0"

from .api import (Config, Generator, GeneratorParams, Model, NamedTensors, Tensor, get_current_gpu_device_id,  # noqa: F401
                  is_cuda_available, set_current_gpu_device_id, set_log_callback, set_log_options)
from .tokenizer import Tokenizer, TokenizerStream  # noqa: F401
from . import streaming  # noqa: F401  (StreamingProcessor, StreamingSession, VoiceActivityDetector)


def __getattr__(name):
    # Heavier subsystems are imported on first use.
    if name in ("Engine", "Request"):
        from .engine import engine as _e
        return getattr(_e, name)
    if name == "Adapters":
        from .models.lora import Adapters
        return Adapters
    if name in ("Images", "Audios", "MultiModalProcessor"):
        from . import multimodal as _m
        return getattr(_m, name)
    if name == "MtpGenerator":
        from .mtp import MtpGenerator
        return MtpGenerator
    raise AttributeError(name)
