"""Trace replay: feeds given token ids through a model step by step and writes the logits that are asked for.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--max-seqs 4]

Standard input carries one JSON object per line,
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
Every entry brings a request's next tokens (a request is admitted at its first entry); all entries of a line run as ONE step of
the engine (turboinfer_b200.seq.SeqModel.step -- the step the generation loop uses).  For a step with wanted places the logits
[wanted, vocab] go to DIR/<step>.f32 (little-endian fp32, in the order of the entries and of `want`); after every step a line
`done <step>` is printed.  Requests named in "end" give their pages and state slot back after the step."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-seqs", type=int, default=4)
    a = ap.parse_args(argv)
    from .models import load_model
    model = load_model(a.model, a.dtype, max_tokens=a.max_tokens, max_seqs=a.max_seqs)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries, want = [], []
        for e in msg.get("entries", []):
            if e["id"] not in live:
                live[e["id"]] = model.open()
            if not e.get("tokens"):
                continue   # admitted, nothing to run for it in this step
            entries.append((live[e["id"]], [int(t) for t in e["tokens"]]))
            want.append([int(w) for w in (e.get("want") or [])])
        if entries:
            logits = model.step(entries, want)
            if logits.shape[0]:
                tmp = os.path.join(a.out, ".%s.part" % msg["step"])
                with open(tmp, "wb") as f:
                    f.write(logits.astype("<f4").tobytes())
                os.replace(tmp, os.path.join(a.out, "%s.f32" % msg["step"]))
        for rid in msg.get("end", []):
            if rid in live:
                model.close(live.pop(rid))
        sys.stdout.write("done %s\n" % msg["step"])
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
