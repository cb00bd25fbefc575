"""Token generation from the command line for any registered architecture.

    generate --model DIR [--dtype bfloat16|float32|int4|int8] --prompt-ids 5,17,3 [--prompt-ids ...] --max-new 32
             [--temperature 0] [--top-k 0] [--top-p 1] [--seed 0] [--eos -1] [--max-tokens N] [--max-seqs 4] [--step-tokens 512]

DIR holds config.json and model.safetensors; config.json's "architecture" picks the model class (turboinfer_b200.models).  Prompts
are token ids (the library has no tokenizer).  A model of the layered sequence engine runs all prompts through its continuous-
batching loop (SeqModel.generate); the quantized Llama-style decoder generates them one after the other.  One JSON line per
prompt goes to standard output: {"prompt": index, "tokens": [new token ids]}."""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str):
    return [int(t) for t in text.replace(",", " ").split()]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "int4", "int8"])
    ap.add_argument("--prompt-ids", action="append", required=True, help="token ids of one prompt, comma or space separated; repeatable")
    ap.add_argument("--max-new", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eos", type=int, default=-1)
    ap.add_argument("--max-tokens", type=int, default=0, help="tokens the cache pool holds (0: enough for all prompts at once)")
    ap.add_argument("--max-seqs", type=int, default=4)
    ap.add_argument("--step-tokens", type=int, default=512)
    a = ap.parse_args(argv)
    prompts = [_ids(p) for p in a.prompt_ids]
    if any(not p for p in prompts):
        ap.error("an empty prompt")
    from . import seq
    from .models import load_model
    live = min(len(prompts), a.max_seqs)
    longest = sorted((len(p) + a.max_new + 63) // 64 * 64 for p in prompts)[-live:]
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens or sum(longest), max_seqs=a.max_seqs)
    if isinstance(model, seq.SeqModel):
        outs = model.generate(prompts, a.max_new, step_tokens=a.step_tokens, temperature=a.temperature, top_k=a.top_k, top_p=a.top_p,
                              seed=a.seed, eos=a.eos)
    else:
        outs = []
        for p in prompts:
            if a.temperature > 0:
                toks, _, _ = model.generate_sampled(p, a.max_new, temperature=a.temperature, top_k=a.top_k or 50, top_p=a.top_p, seed=a.seed,
                                                    stop_on_eos=a.eos >= 0)
            else:
                toks, _, _ = model.generate_greedy(p, a.max_new, stop_on_eos=a.eos >= 0)
            outs.append([int(t) for t in toks])
    for i, o in enumerate(outs):
        sys.stdout.write(json.dumps({"prompt": i, "tokens": o}) + "\n")
    model.free()
    return 0


if __name__ == "__main__":
    sys.exit(main())
