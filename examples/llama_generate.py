#!/usr/bin/env python
"""Text generation from a Hugging Face Llama directory or a random-weight preset (the reference's
examples/llama_generate.cpp, same flags).

    python examples/llama_generate.py --model-dir /path/to/Llama-3.2-1B --prompt "Hello" --max-new-tokens 64
    python examples/llama_generate.py --config c.json --safetensors m.safetensors --tokenizer tokenizer.json --prompt hi
    python examples/llama_generate.py --model small --prompt abc --sample --top-p 0.9 --temperature 0.8 --kv-int8
    python examples/llama_generate.py --model small --prompt 12 --grammar-regex "[0-9]+"
"""
from __future__ import annotations

import argparse
import os
import sys

from _common import load_tokenizer, pick_device, preset, torch


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model-dir", default="")
    ap.add_argument("--config", default="")
    ap.add_argument("--safetensors", default="")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--model", default="", help="random-weight preset instead of files: tiny | small | llama3-8b")
    ap.add_argument("--prompt", default="Hello")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eos", type=int, default=None)
    ap.add_argument("--kv-int8", action="store_true")
    ap.add_argument("--grammar-regex", default="")
    ap.add_argument("--no-stream", action="store_true")
    a = ap.parse_args()

    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.sampler import SamplingParams
    dev = pick_device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if a.model_dir:
        a.config = a.config or os.path.join(a.model_dir, "config.json")
        a.safetensors = a.safetensors or os.path.join(a.model_dir, "model.safetensors")
        a.tokenizer = a.tokenizer or os.path.join(a.model_dir, "tokenizer.json")
    if a.config and a.safetensors:
        cfg = LlamaConfig.from_json(open(a.config).read())
        cfg.dtype = dtype
        model = LlamaModel.from_pretrained(a.safetensors, cfg, device=dev)
    elif a.model:
        cfg = preset(a.model, dtype, 2048)
        model = LlamaModel(cfg, device=dev, init_std=0.02, seed=a.seed)
    else:
        print("error: pass --model-dir, or --config with --safetensors, or a --model preset. See --help.", file=sys.stderr)
        return 1
    tok = load_tokenizer(a.tokenizer)
    ids = [i % cfg.vocab_size for i in tok.encode(a.prompt)]
    if not ids:
        print("error: the prompt encodes to no tokens", file=sys.stderr)
        return 1
    gen = GenerateConfig(max_new_tokens=a.max_new_tokens, eos_token_id=cfg.eos_token_id if a.eos is None else a.eos,
                         do_sample=a.sample, seed=a.seed, kv_int8=a.kv_int8,
                         sampling=SamplingParams(temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                                                 repetition_penalty=a.repetition_penalty))
    model.eval()
    with torch.no_grad():
        if a.grammar_regex:
            from tesseract_b200.models.structured import generate_structured
            out = generate_structured(model, ids, tok, a.grammar_regex, gen)
        else:
            out = model.generate(ids, gen)
    new = out[len(ids):]
    if a.no_stream:
        print(tok.decode(out))
    else:
        print(a.prompt, end="", flush=True)
        for t in new:
            print(tok.decode([t]), end="", flush=True)
        print()
    print(f"[{len(ids)} prompt tokens, {len(new)} new tokens]", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
