"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
A request that appears for the first time starts a sequence (it gets a cache slot); later
entries continue it; `end` lists requests that are finished after the step, whose slots and
pages go back to the cache.  For a step in which something is wanted the logits at the wanted
places, in the order of the entries and of `want`, are written to OUT/<step>.f32 as little-endian
float32 [wanted, vocab].  After every step a line `done <step>` is printed and flushed.

Nothing is sampled and nothing is computed here: the program drives `Engine.step`, the same
step function, cache and kernels that generation uses.  It is the analogue of the reference's
`--bench`, which feeds synthetic tokens step by step through `forward` (src/main.zig:669-699).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
TOKEN_UNIT = 64          # --max-tokens counts each request rounded up to this many tokens


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    args = ap.parse_args(argv)

    from .engine.engine import Engine
    from .weights.loader import load_model

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    dtype = DTYPES[args.dtype]
    model = load_model(args.model, dtype=dtype, device="cuda")
    max_tokens = max(TOKEN_UNIT, -(-args.max_tokens // TOKEN_UNIT) * TOKEN_UNIT)
    engine = Engine(model, max_batch=max_tokens // TOKEN_UNIT, max_seq_len=max_tokens, max_tokens=max_tokens,
                    page_size=TOKEN_UNIT)
    slot_of: dict[str, int] = {}

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        new = [e["id"] for e in entries if e["id"] not in slot_of]
        if new:
            for rid, slot in zip(new, engine.start(len(new))):
                slot_of[rid] = slot
        if entries:
            slots = [slot_of[e["id"]] for e in entries]
            tokens = [list(e["tokens"]) for e in entries]
            want = [list(e.get("want", [])) for e in entries]
            logits = engine.step(slots, tokens, want)
            if logits is not None:
                arr = logits.to(torch.float32).cpu().numpy().astype("<f4", copy=False)
                arr.tofile(out_dir / f"{step}.f32")
        ended = [rid for rid in rec.get("end", []) if rid in slot_of]
        if ended:
            engine.finish([slot_of.pop(rid) for rid in ended])
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
