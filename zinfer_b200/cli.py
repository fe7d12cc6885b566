"""Command line in the manner of the reference's `zinfer -m MODEL [options]`
(src/main.zig:14-63, parsed at src/main.zig:141-248): the same option names and meanings where
the reference has them.  The reference reads text and a GGUF file; this library starts from
token ids and a model folder, so `-p` takes comma-separated ids and `-m` a folder.

    zinfer_b200 -m FOLDER -p 1,2,3 -n 32 --temp 0
    zinfer_b200 -m FOLDER -f prompts.txt --temp 0.8 --top-k 40 --seed 7
    zinfer_b200 --random-weights CONFIG.json --write FOLDER --seed-weights 3
    zinfer_b200 -m FOLDER --bench 512,64 --batch-sizes 1,8
    zinfer_b200 -m FOLDER -p 1,2,3 -n 8 --dump-logits logits.f32

Ctrl-C ends a running generation at its next step and prints what was generated so far
(src/main.zig:297-299, src/gen.zig:476-479); a second Ctrl-C ends the program.
"""
from __future__ import annotations

import argparse
import json
import signal
import sys
import time
from pathlib import Path


def parse_ids(text: str) -> list[int]:
    return [int(t) for t in text.replace(",", " ").split()]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="zinfer_b200", description="LFM2 generation on one B200")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("-p", "--prompt", help="prompt as token ids, comma or space separated")
    ap.add_argument("-f", "--file", help="file with one prompt (token ids) per line")
    ap.add_argument("-n", "--predict", type=int, default=256,
                    help="max tokens to generate (default 256; -1 or 0 = until the context is full)")
    ap.add_argument("-c", "--ctx", type=int, default=0, help="context length (default: min(4096, trained))")
    ap.add_argument("-b", "--batch", type=int, default=8192, help="prompt tokens per step (longer prompts are chunked)")
    ap.add_argument("--max-batch", type=int, default=64, help="sequences that run together")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "fp32", "float32"])
    g = ap.add_argument_group("sampling (defaults as shown)")
    g.add_argument("--temp", type=float, default=0.8, help="temperature, 0 = greedy (0.8)")
    g.add_argument("--top-k", type=int, default=40, help="0 = off (40)")
    g.add_argument("--top-p", type=float, default=0.95, help="(0.95)")
    g.add_argument("--min-p", type=float, default=0.05, help="(0.05)")
    g.add_argument("--repeat-penalty", type=float, default=1.0, help="penalize the last 64 tokens, 1 = off (1.0)")
    g.add_argument("--dry-multiplier", type=float, default=0.0)
    g.add_argument("--dry-base", type=float, default=1.75)
    g.add_argument("--dry-allowed-length", type=int, default=2)
    g.add_argument("--dry-range", type=int, default=1024)
    g.add_argument("--xtc-probability", type=float, default=0.0)
    g.add_argument("--xtc-threshold", type=float, default=0.1)
    g.add_argument("--xtc-min-keep", type=int, default=1)
    g.add_argument("--seed", type=int, default=None, help="RNG seed (default: time)")
    ap.add_argument("--stop", default=None, help="stop token ids (default: the model's eos ids)")
    ap.add_argument("--bench", default=None, metavar="PP,TG",
                    help="time a prompt of PP synthetic tokens and TG generated tokens (src/main.zig:669-699)")
    ap.add_argument("--batch-sizes", default="1", metavar="B1,B2,...",
                    help="with --bench: run it for each of these numbers of equal sequences (default 1)")
    ap.add_argument("--dump-logits", metavar="PATH",
                    help="write the logits at the last token of every prompt as little-endian float32 "
                         "[prompts, vocab] before generating")
    ap.add_argument("--random-weights", metavar="CONFIG.json", help="write a model folder with random weights")
    ap.add_argument("--write", metavar="FOLDER", help="where --random-weights writes")
    ap.add_argument("--seed-weights", type=int, default=0)
    ap.add_argument("-v", "--verbose", action="store_true", help="print model info")
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import zinfer_b200 as z
    from zinfer_b200.sampling import SamplingParams

    if args.random_weights:
        if not args.write:
            print("--random-weights needs --write FOLDER", file=sys.stderr)
            return 2
        cfg = z.config_from_dict(json.loads(Path(args.random_weights).read_text()))
        z.write_random_model(args.write, cfg, args.seed_weights)
        print(f"wrote {args.write}")
        if not args.model:
            return 0
    if not args.model:
        print("error: -m MODEL is required", file=sys.stderr)        # src/main.zig:246
        return 2

    t0 = time.perf_counter()
    model = z.load(args.model, dtype=args.dtype)
    cfg = model.config
    ctx = args.ctx or min(4096, cfg.max_position_embeddings)          # src/main.zig:324-326
    engine = z.Engine(model, max_batch=args.max_batch, max_seq_len=ctx, max_step_tokens=args.batch)
    if args.verbose:
        print(f"model: {cfg.architecture} | dtype {args.dtype} | ctx {ctx} | vocab {cfg.vocab_size} | "
              f"load {1e3 * (time.perf_counter() - t0):.0f} ms", file=sys.stderr)

    def on_sigint(signum, frame):
        if engine.interrupt.is_set():
            raise KeyboardInterrupt
        engine.interrupt.set()

    signal.signal(signal.SIGINT, on_sigint)

    if args.bench:
        pp, tg = (int(x) for x in args.bench.split(","))
        for b in parse_ids(args.batch_sizes):
            if b > args.max_batch:
                print(f"error: --batch-sizes {b} exceeds --max-batch {args.max_batch}", file=sys.stderr)
                return 2
            toks = [[(i * 7919 + 13 + 31 * s) % cfg.vocab_size for i in range(pp)] for s in range(b)]   # src/main.zig:673
            engine.generate(toks, max_new_tokens=tg, temp=0.0, stop_ids=[])
            print(f"batch {b}: " + engine.stats.report())
        return 0

    prompts = []
    if args.prompt:
        prompts.append(parse_ids(args.prompt))
    if args.file:
        prompts += [parse_ids(l) for l in Path(args.file).read_text().splitlines() if l.strip()]
    if not prompts:
        print("error: give a prompt with -p or -f", file=sys.stderr)
        return 2
    seed = args.seed if args.seed is not None else time.time_ns() & 0xFFFFFFFF     # src/main.zig:330
    params = SamplingParams(temp=args.temp, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                            repeat_penalty=args.repeat_penalty, seed=seed, dry_multiplier=args.dry_multiplier,
                            dry_base=args.dry_base, dry_allowed_length=args.dry_allowed_length,
                            dry_range=args.dry_range, xtc_probability=args.xtc_probability,
                            xtc_threshold=args.xtc_threshold, xtc_min_keep=args.xtc_min_keep)
    stop = parse_ids(args.stop) if args.stop is not None else None
    if args.dump_logits:
        import numpy as np
        rows = []
        for i in range(0, len(prompts), args.max_batch):
            slots = engine.start(len(prompts[i:i + args.max_batch]))
            try:
                rows.append(engine.step(slots, prompts[i:i + args.max_batch]).float().cpu().numpy())
            finally:
                engine.finish(slots)
        np.concatenate(rows).astype("<f4").tofile(args.dump_logits)
    results = engine.generate(prompts, max_new_tokens=args.predict, sampling=params, stop_ids=stop)
    for r in results:
        print(" ".join(str(t) for t in r.tokens) + f"  [{r.finish_reason}]")
    print(engine.stats.report(), file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
