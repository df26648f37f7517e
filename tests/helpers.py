"""Shared test helpers: a small byte-level BPE tokenizer and model directories that carry it."""
import copy
import json
import os

from onnxruntime_genai_b200.models.arch import ArchConfig
from onnxruntime_genai_b200.models.builder import export_model

CORPUS = [
    '{"name": "Alice", "age": 30, "city": "Paris"}', '{"name": "Bob", "age": 7, "tags": ["a", "b"]}',
    "The quick brown fox jumps over the lazy dog. 0123456789", "yes no maybe true false null [] {} : , \" \\ ",
    "hello world, hello tokens, hello grammar", "abcdefghijklmnopqrstuvwxyz ABCDEFGHIJKLMNOPQRSTUVWXYZ",
]


def make_tokenizer(out_dir: str, vocab_size: int = 384):
    """Trains a byte-level BPE tokenizer (all 256 bytes in the alphabet) and writes tokenizer.json + config."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=vocab_size - 2, special_tokens=["<s>", "</s>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(CORPUS * 4, trainer)
    os.makedirs(out_dir, exist_ok=True)
    tok.save(os.path.join(out_dir, "tokenizer.json"))
    with open(os.path.join(out_dir, "tokenizer_config.json"), "w") as f:
        json.dump({"bos_token": "<s>", "eos_token": "</s>",
                   "chat_template": "{% for m in messages %}<|{{ m['role'] }}|>{{ m['content'] }}\n{% endfor %}"
                                    "{% if add_generation_prompt %}<|assistant|>{% endif %}"}, f)
    return tok.get_vocab_size()


def tiny_model_dir(out_dir: str, provider: str = "cpu", precision: str = "fp32", seed: int = 0, std: float = 0.05, **arch_kw):
    """A 2-layer Llama-style model whose vocabulary is the test tokenizer's."""
    vocab = make_tokenizer(out_dir)
    kw = dict(model_type="llama", vocab_size=vocab, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
              intermediate_size=128, context_length=512, bos_token_id=0, eos_token_id=1, pad_token_id=1)
    kw.update(arch_kw)
    arch = ArchConfig(**kw)
    export_model(arch, out_dir, precision, provider, seed=seed, std=std, paged=True, block_size=16, num_blocks=256, max_batch_size=8)
    return out_dir, arch
