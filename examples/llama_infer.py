#!/usr/bin/env python
"""Full-model forward on a prompt or on random ids with synthetic or safetensors weights: prints the logits' shape,
the finite count and the top-k next-token candidates, or generates with ``--generate`` (the reference's
examples/llama_infer.cpp:118-298, same flags).

    python examples/llama_infer.py --synthetic --vocab 512 --hidden 64 --layers 2 --heads 4 --kv-heads 2 --ff 128
    python examples/llama_infer.py --synthetic --prompt "hello" --generate --max-new-tokens 8 --sample --top-k 20
    python examples/llama_infer.py --safetensors m.safetensors --tokenizer tokenizer.json --prompt "Hi" --generate
"""
from __future__ import annotations

import argparse

from _common import load_tokenizer, pick_device, torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--safetensors", default="")
    ap.add_argument("--tokenizer", default="")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--generate", action="store_true")
    ap.add_argument("--max-new-tokens", type=int, default=16)
    ap.add_argument("--sample", action="store_true")
    ap.add_argument("--temperature", type=float, default=1.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=512)
    ap.add_argument("--hidden", type=int, default=64)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--heads", type=int, default=4)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--ff", type=int, default=128)
    ap.add_argument("--max-seq", type=int, default=256)
    ap.add_argument("--rope-theta", type=float, default=10000.0)
    ap.add_argument("--tie", default="false")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq", type=int, default=8)
    ap.add_argument("--topk", type=int, default=5)
    a = ap.parse_args(argv)
    if not a.synthetic and not a.safetensors:
        raise SystemExit("error: pass --synthetic or --safetensors PATH. See --help.")

    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.sampler import SamplingParams
    dev = pick_device(a.device)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    cfg = LlamaConfig(vocab_size=a.vocab, hidden_size=a.hidden, num_hidden_layers=a.layers,
                      num_attention_heads=a.heads, num_key_value_heads=a.kv_heads, intermediate_size=a.ff,
                      max_position_embeddings=a.max_seq, rope_theta=a.rope_theta,
                      tie_word_embeddings=(a.tie != "false"), dtype=dtype)
    print(f"[llama_infer] config:\n  vocab={cfg.vocab_size} hidden={cfg.hidden_size} layers={cfg.num_hidden_layers} "
          f"heads={cfg.num_attention_heads} kv_heads={cfg.num_key_value_heads} ff={cfg.intermediate_size} "
          f"max_seq={cfg.max_position_embeddings} tie={cfg.tie_word_embeddings} device={dev} dtype={dtype}")
    if a.synthetic:
        print("[llama_infer] using synthetic (random-init) weights")
        model = LlamaModel(cfg, device=dev, init_std=0.02, seed=a.seed)
    else:
        print(f"[llama_infer] loading {a.safetensors}")
        model = LlamaModel.from_pretrained(a.safetensors, cfg, device=dev)
        print(f"[llama_infer] loaded {sum(p.numel() for p in model.parameters())} parameters")
    model.eval()
    tok = load_tokenizer(a.tokenizer)

    if a.prompt:
        ids = [i % cfg.vocab_size for i in tok.encode(a.prompt)]
        print(f'[llama_infer] prompt = "{a.prompt}"\n[llama_infer] ids = ' + " ".join(str(i) for i in ids))
        print(f'[llama_infer] decoded = "{tok.decode(ids)}"')
        if not ids:
            raise SystemExit("error: the prompt encodes to no tokens")
    else:
        g = torch.Generator().manual_seed(a.seed)
        ids = None
        batch_ids = torch.randint(0, cfg.vocab_size, (a.batch, a.seq), generator=g).to(dev)

    if a.generate:
        if ids is None:
            raise SystemExit("error: --generate needs --prompt")
        mode = "sampling" if a.sample else "greedy"
        extra = f" (T={a.temperature}, top_k={a.top_k}, top_p={a.top_p}, rep={a.repetition_penalty}, seed={a.seed})" \
            if a.sample else ""
        print(f"[llama_infer] decoding = {mode}{extra}")
        gen = GenerateConfig(max_new_tokens=a.max_new_tokens, eos_token_id=cfg.eos_token_id, do_sample=a.sample,
                             seed=a.seed, sampling=SamplingParams(temperature=a.temperature, top_k=a.top_k,
                                                                  top_p=a.top_p,
                                                                  repetition_penalty=a.repetition_penalty))
        with torch.no_grad():
            out = model.generate(ids, gen)
        print(f"[llama_infer] generated {len(out) - len(ids)} tokens: " + " ".join(str(i) for i in out))
        print(f'[llama_infer] decoded text = "{tok.decode(out)}"')
        print("[llama_infer] done.")
        return 0

    if ids is not None:
        batch_ids = torch.tensor([ids], dtype=torch.long, device=dev)
    with torch.no_grad():
        logits = model(batch_ids)
    host = logits.float().cpu()
    print(f"[llama_infer] logits.shape = {list(logits.shape)}")
    print(f"[llama_infer] finite = {int(torch.isfinite(host).sum())} / {host.numel()}")
    k = max(1, min(a.topk, cfg.vocab_size))
    score, idx = host[0, -1].topk(k)
    print(f"[llama_infer] top-{k} for b=0, last position:")
    for s, i in zip(score.tolist(), idx.tolist()):
        print(f"  id={i}  logit={s:.6f}")
    print("[llama_infer] done.")
    return 0 if bool(torch.isfinite(host).all()) else 2


if __name__ == "__main__":
    raise SystemExit(main())
