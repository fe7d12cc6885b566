"""Benchmark of zinfer_b200: decode tokens per second of an LFM2-1.2B-shaped model with random
weights on one B200, with the prefill rate, the decode roofline and batch-1/64 points beside it.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step: one new token for each of the batch's sequences.  After W warm-up
steps exactly K steps are timed with CUDA events on the launching stream.  The step reads 2.3 GB
of weights and the live requests' cache, far more than the 126 MB L2, so no flush is needed
between iterations.  The line printed is one JSON object; `value` is device-timed, `e2e` is the
same metric through `Engine.generate` with token ids going in from and coming back to the host
every step.  The reference engine (a Zig program for CPUs) cannot be installed as a Python
package, so `--impl reference` prints an `unavailable` line.  This library runs on one GPU: for
--gpus > 1 the program says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

# LFM2-1.2B: the sizes of the published checkpoint's config.json
LFM2_1_2B = dict(
    architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=65536, hidden_size=2048, num_hidden_layers=16,
    num_attention_heads=32, num_key_value_heads=8, max_position_embeddings=128000,
    layer_types=["conv", "conv", "full_attention", "conv", "conv", "full_attention", "conv", "conv", "full_attention",
                 "conv", "full_attention", "conv", "full_attention", "conv", "full_attention", "conv"],
    block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256,
    conv_L_cache=3, conv_bias=False, rope_theta=1000000.0, norm_eps=1e-5, tie_word_embeddings=True, eos_token_id=7)


def _lfm2(hidden, layers, attn_at, heads, ffn):
    """An LFM2 configuration of the given sizes with the effective SwiGLU width `ffn`."""
    d = dict(LFM2_1_2B, hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
             layer_types=["full_attention" if i in attn_at else "conv" for i in range(layers)],
             block_ff_dim=ffn, block_auto_adjust_ff_dim=False)
    return d


# The secondary workloads: (configuration, batch, prompt lengths, decode steps, longest sequence)
SECONDARY = {
    "2.6b": (_lfm2(2048, 30, {2, 6, 10, 14, 18, 21, 24, 27}, 32, 10752), 16, (64, 4096), 256, 4096 + 512),
    "350m": (_lfm2(1024, 16, {2, 5, 8, 10, 12, 14}, 16, 4608), 64, (1024, 32768), 128, 32768 + 256),
}
CONTEXT = 4096
PROMPT_RANGE = (512, 2048)
PREFILL_TOKENS = 2048
POINT_STEPS = 64            # the batch-1 and batch-64 points are timed over at least this many steps
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except (KeyError, ValueError, json.JSONDecodeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines: list[str] = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 6 or not f[0].isdigit():
                continue
            sm.append(int(f[0]))
            mx = max(mx, int(f[1]) if f[1].isdigit() else 0)
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": int(statistics.median(sm)) if sm else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(sm)}


def model_numbers(cfg, n_layers_run: int) -> dict:
    """Weight bytes a decode step reads and FLOPs a prefill needs, from the configuration."""
    D, F, Q, KV, V = cfg.hidden_size, cfg.ffn_dim, cfg.q_dim, cfg.kv_dim, cfg.vocab_size
    kinds = cfg.layer_types[:n_layers_run]
    conv = 3 * D * D + D * D
    attn = (Q + 2 * KV) * D + D * Q
    ffn = 3 * D * F
    layer_params = sum((conv if k == "conv" else attn) + ffn for k in kinds)
    n_attn = sum(k != "conv" for k in kinds)
    return {"layer_params": layer_params, "head_params": V * D, "n_attn": n_attn, "n_conv": len(kinds) - n_attn,
            "kv_bytes_per_token": n_attn * 2 * KV * 2, "conv_state_bytes": (len(kinds) - n_attn) * (cfg.conv_L_cache - 1) * D * 4}


def time_decode(engine, torch, rng, batch: int, steps: int, warmup: int, vocab: int, prompt_range=None):
    """Prefills `batch` prompts of lengths uniform in `prompt_range` (default PROMPT_RANGE), then times
    `steps` decode steps.  Every CUDA graph the timed steps replay is recorded before the timing
    starts; `captures` counts the steps that had to record one all the same (expected: 0).
    Returns (ms per step, total cached tokens at the middle of the timed region, launches per step,
    captures)."""
    from zinfer_b200 import kernels
    lo, hi = prompt_range or PROMPT_RANGE
    lens = rng.integers(lo, hi + 1, size=batch).tolist()
    prompts = [rng.integers(0, vocab, size=n).tolist() for n in lens]
    slots = engine.start(batch)
    try:
        engine.step(slots, prompts, want=[[] for _ in prompts])
        toks = rng.integers(0, vocab, size=(warmup + steps, batch))
        launches = None
        for i in range(warmup):
            before = kernels.launch_count
            engine.decode(slots, toks[i].tolist())
            if launches is None:
                launches = kernels.launch_count - before
        longest = max(lens) + warmup
        engine.prepare_decode(batch, longest, longest + steps + 1)
        torch.cuda.synchronize()
        captures = engine.graph_captures
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(warmup, warmup + steps):
            engine.decode(slots, toks[i].tolist())
        stop.record()
        torch.cuda.synchronize()
        engine.check_status()
        ms = start.elapsed_time(stop) / steps
        cached = sum(lens) + batch * (warmup + steps // 2)
        captures = engine.graph_captures - captures
    finally:
        engine.finish(slots)
    return ms, cached, launches, captures


def time_prefill(engine, torch, rng, cfg, warmup: int, num: dict, pk: dict, tokens: int = PREFILL_TOKENS) -> dict:
    """One sequence of `tokens` tokens in one step; median of 5 after the warm-up."""
    toks = rng.integers(0, cfg.vocab_size, size=tokens).tolist()
    times = []
    for i in range(warmup + 5):
        slot = engine.start(1)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step(slot, [toks], check=False)
        stop.record()
        torch.cuda.synchronize()
        engine.finish(slot)
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    pre_ms = statistics.median(times)
    T = tokens
    flops = 2 * T * num["layer_params"] + 2 * num["head_params"] + num["n_attn"] * 2 * T * T * cfg.q_dim
    return {"value": round(T / (pre_ms * 1e-3), 1), "tokens": T, "ms": round(pre_ms, 3),
            "frac": round(flops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}


def secondary_arm(args) -> dict:
    """One of the secondary workloads: unequal long prompts, then `steps` timed decode steps."""
    import numpy as np
    import torch
    import zinfer_b200 as z
    from zinfer_b200 import kernels

    kernels.require_cuda()
    pk = peaks()
    cfg_dict, batch, prompt_range, steps, longest = SECONDARY[args.model]
    cfg = z.config_from_dict(cfg_dict)
    model = z.random(cfg, seed=0, dtype="bf16", fill_on_device=True)
    rng = np.random.default_rng(0)
    lens = np.random.default_rng(0).integers(prompt_range[0], prompt_range[1] + 1, size=batch)   # as time_decode draws them
    page = 64
    room = int(sum(-(-(int(n) + args.warmup + steps + 1) // page) * page for n in lens))
    engine = z.Engine(model, max_batch=batch, max_seq_len=longest, max_tokens=room, page_size=page)
    num = model_numbers(cfg, cfg.num_hidden_layers)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with ClockSampler() as clocks:
        ms, cached, launches, captures = time_decode(engine, torch, rng, batch, steps, args.warmup, cfg.vocab_size,
                                                     prompt_range=prompt_range)
    wall = time.perf_counter() - t0
    weight_bytes = 2 * (num["layer_params"] + num["head_params"])
    step_bytes = weight_bytes + cached * num["kv_bytes_per_token"] + batch * num["conv_state_bytes"] * 2
    achieved = step_bytes / (ms * 1e-3) / 1e9
    return {"metric": f"decode tokens/s at batch {batch} (LFM2-{args.model.upper()} shape, random weights)",
            "value": round(batch / (ms * 1e-3), 1), "unit": "tokens/s", "ms_per_step": round(ms, 4), "steps": steps,
            "warmup": args.warmup, "dtype": "bf16", "impl": "zinfer_b200",
            "config": {"model": f"LFM2-{args.model.upper()}", "global_batch": batch, "layers": cfg.num_hidden_layers,
                       "hidden": cfg.hidden_size, "ffn": cfg.ffn_dim, "prompt_lens": f"uniform[{prompt_range[0]},{prompt_range[1]}]",
                       "cached_tokens": int(cached), "peaks": pk["source"]},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4), "weight_gb": round(weight_bytes / 1e9, 3),
                         "cache_gb": round(cached * num["kv_bytes_per_token"] / 1e9, 3)},
            "clocks": clocks.summary(), "gpu_launches": int(launches or 0) * steps,
            "graph_captures_in_timed_steps": captures, "wall_s_with_prompts": round(wall, 1)}


def own_arm(args) -> dict:
    import numpy as np
    import torch

    sys.path.insert(0, str(ROOT))
    import zinfer_b200 as z
    from zinfer_b200 import kernels

    kernels.require_cuda()
    pk = peaks()
    cfg_dict = dict(LFM2_1_2B)
    layers_cfg = cfg_dict["num_hidden_layers"]
    if args.layers and args.layers < layers_cfg:
        cfg_dict["num_hidden_layers"] = args.layers
        cfg_dict["layer_types"] = cfg_dict["layer_types"][:args.layers]
    cfg = z.config_from_dict(cfg_dict)
    model = z.random(cfg, seed=0, dtype="bf16", fill_on_device=True)
    B = args.batch
    engine = z.Engine(model, max_batch=64, max_seq_len=max(CONTEXT, args.prefill_tokens), page_size=64,
                      max_tokens=max(64 * CONTEXT, args.prefill_tokens), max_step_tokens=max(8192, args.prefill_tokens),
                      use_graphs=not args.no_graphs)
    if args.only == "prefill":
        return {"prefill": time_prefill(engine, torch, np.random.default_rng(0), cfg, args.warmup,
                                        model_numbers(cfg, cfg.num_hidden_layers), pk, args.prefill_tokens)}
    rng = np.random.default_rng(0)
    num = model_numbers(cfg, cfg.num_hidden_layers)
    weight_bytes = 2 * (num["layer_params"] + num["head_params"])

    # decode at the headline batch, device-timed, with the clocks sampled meanwhile
    with ClockSampler() as clocks:
        ms, cached, launches, captures = time_decode(engine, torch, rng, B, args.steps, args.warmup, cfg.vocab_size)
    value = B / (ms * 1e-3)
    step_bytes = weight_bytes + cached * num["kv_bytes_per_token"] + B * num["conv_state_bytes"] * 2
    achieved = step_bytes / (ms * 1e-3) / 1e9

    if args.only == "decode":
        return {"value": round(value, 1), "ms_per_step": round(ms, 4), "launches_per_step": launches,
                "roofline_frac": round(achieved / pk["hbm_gbs"], 4)}

    # other batch sizes, each over at least POINT_STEPS steps whatever --steps says
    points = {}
    for b in (1, 64):
        pms, pcached, _, pcap = time_decode(engine, torch, rng, b, max(POINT_STEPS, args.steps), args.warmup,
                                            cfg.vocab_size)
        captures += pcap
        pbytes = weight_bytes + pcached * num["kv_bytes_per_token"] + b * num["conv_state_bytes"] * 2
        points[f"decode_b{b}"] = round(b / (pms * 1e-3), 1)
        points[f"decode_b{b}_hbm_frac"] = round(pbytes / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    prefill = time_prefill(engine, torch, rng, cfg, args.warmup, num, pk)
    T = PREFILL_TOKENS

    # the same metric end to end through the public entry point: host token ids in and out every step
    prompts = [rng.integers(0, cfg.vocab_size, size=int(n)).tolist()
               for n in rng.integers(PROMPT_RANGE[0], PROMPT_RANGE[1] + 1, size=B)]
    n_new = max(POINT_STEPS, args.steps) + 1       # at least 64 steps, as the other points
    # warm-up: the same generation once, so that every graph the timed one replays is captured
    engine.generate(prompts, max_new_tokens=n_new, temp=0.0, stop_ids=[])
    engine.generate(prompts, max_new_tokens=n_new, temp=0.0, stop_ids=[])
    st = engine.stats
    e2e_value = B * st.n_decode_steps / st.t_gen_s
    from zinfer_b200.engine.context import batch_layout
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch_layout(B, B)["_total"][0],
           "d2h_bytes_per_step": 4 * (B + 1)}

    return {
        "metric": "decode tokens/s at batch 8 (LFM2-1.2B shape, random weights, context 4096)" if B == 8
        else f"decode tokens/s at batch {B} (LFM2-1.2B shape, random weights, context 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic token ids, random-init weights N(0, 0.02)", "impl": "zinfer_b200",
        "config": {"model": "LFM2-1.2B", "global_batch": B, "seq_len": CONTEXT, "parallelism": "none",
                   "vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "layers": cfg.num_hidden_layers,
                   "layers_of_config": layers_cfg, "attn_layers": num["n_attn"], "heads": cfg.num_attention_heads,
                   "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "ffn": cfg.ffn_dim,
                   "conv_window": cfg.conv_L_cache, "prompt_lens": "uniform[512,2048]", "prefill_tokens": T,
                   "l2": "inputs larger than L2 (2.3 GB of weights per step)", "peaks": pk["source"]},
        "clocks": clocks.summary(),
        "e2e": e2e,
        "gpu_launches": int(launches or 0) * args.steps,
        "graph_captures_in_timed_steps": captures,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="own", choices=["own", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="run only the first L layers (named in `config`)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure one part only (for profiling); the JSON line then lacks the other parts")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="with --only prefill: the prompt's length (the headline line always uses 2,048)")
    ap.add_argument("--model", default="1.2b", choices=["1.2b"] + sorted(SECONDARY),
                    help="1.2b: the headline benchmark; 2.6b, 350m: the secondary workloads (decode only)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "pylypenko99/zinfer is a Zig program for CPUs: pip cannot install it "
                                         "(no setup.py or pyproject.toml) and no Zig compiler is on this image"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: zinfer_b200 runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    print(json.dumps(own_arm(args) if args.model == "1.2b" else secondary_arm(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
