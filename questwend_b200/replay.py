"""Trace replay: feed given token ids through a model step by step and write the logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries`` gives each request its next tokens and the places among them whose logits
are wanted; ``end`` names requests that are finished after the step, whose slots and
pages are given back.  For a step with wanted logits, ``<out>/<step>.f32`` holds them
as little-endian float32 [wanted, vocab], in the order of the entries and of ``want``.
After every step a line ``done <step>`` is printed and flushed.  Nothing is sampled.
This program has no model code of its own: it drives ``Engine.step``, the step
function that generation uses.  (The reference's nearest tool compares one whole
prompt with token-by-token feeding, cli/main.cpp:313-337.)
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    from .engine.engine import Engine, StepEntry     # after parsing: --help needs no GPU
    os.makedirs(args.out, exist_ok=True)
    # every live request holds at least one page of 64 tokens, so there are never more of them than pages
    engine = Engine.from_folder(args.model, dtype=args.dtype, device=args.device, max_tokens=args.max_tokens,
                                max_batch=max(1, -(-args.max_tokens // 64)))
    slot_of: dict = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in slot_of:
                slot_of[rid] = engine.open_sequences(1)[0]
            entries.append(StepEntry(slot_of[rid], list(e["tokens"]), list(e.get("want", []))))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                host = logits.to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f"{step}.f32.tmp")
                host.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        ended = [slot_of.pop(rid) for rid in rec.get("end", []) if rid in slot_of]
        if ended:
            engine.close_sequences(ended)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
