"""Shared pieces of the example command lines: model presets, device choice, tokenizer fallback."""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from tesseract_b200.models import LlamaConfig  # noqa: E402


def pick_device(name: str) -> torch.device:
    if name == "cuda":
        if not torch.cuda.is_available():
            raise SystemExit("error: --device cuda but no CUDA device is visible")
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    if name != "cpu":
        raise SystemExit(f"error: unknown --device '{name}'")
    return torch.device("cpu")


def preset(name: str, dtype: torch.dtype, max_pos: int) -> LlamaConfig:
    if name == "tiny":        # the reference's llama_train config (examples/llama_train.cpp:117-125)
        return LlamaConfig(vocab_size=64, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                           num_key_value_heads=4, intermediate_size=128, max_position_embeddings=max(max_pos, 128),
                           dtype=dtype)
    if name == "small":       # test-bed size with 128-wide heads (runs every native kernel)
        return LlamaConfig(vocab_size=4096, hidden_size=512, num_hidden_layers=4, num_attention_heads=4,
                           num_key_value_heads=2, intermediate_size=1024, max_position_embeddings=max(max_pos, 256),
                           dtype=dtype)
    if name == "llama3-8b":
        return LlamaConfig.llama_3_8b(dtype=dtype, max_position_embeddings=max_pos)
    if name == "llama3.2-1b":
        cfg = LlamaConfig.llama_3_2_1b()
        cfg.dtype, cfg.max_position_embeddings = dtype, max_pos
        return cfg
    raise SystemExit(f"error: unknown --model '{name}' (tiny | small | llama3.2-1b | llama3-8b)")


class ByteTokenizer:
    """Fallback when no tokenizer.json is given: one token per UTF-8 byte (ids 0..255)."""

    def encode(self, text: str, add_special_tokens: bool = True):
        return list(text.encode("utf-8"))

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(int(i) & 0xFF for i in ids).decode("utf-8", errors="replace")


def load_tokenizer(path: str):
    if not path:
        return ByteTokenizer()
    from tesseract_b200.io.tokenizer import BpeTokenizer
    return BpeTokenizer.from_file(path)
