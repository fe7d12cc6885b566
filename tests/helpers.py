"""Tiny LFM2 configurations for the tests and helpers to build, replay and compare them.

tiny_a and tiny_b are the two configurations that differ in every size and option (first layer
kind, head counts and group size, head size, feed-forward rule, conv window and bias, rope
base, eps, tied or untied head, norm-weight init, vocabulary); tiny_c adds a windowed
attention group next to a full one, a width and vocabulary that are no power of two, a
two-tap convolution and a float32 weight file; tiny_d and tiny_e have the head size 64 that the
tensor-core attention kernels take, and differ in the rest.

Each of them comes a second time as loud_a ... loud_e: the same sizes with weights N(0, 1/hidden)
and norm weights 1 + N.  With the standard deviation 0.02 that the tiny configurations are
specified with, a contraction over 64 to 256 inputs shrinks its input some tenfold, so that the
logits are the token's own embedding plus small corrections, and a fault in a mixer moves them by
less than the bfloat16 tolerance.  In the loud variants every contraction keeps the size of its
input, every layer changes the residual stream by as much as it holds, and a wrong mixer output,
cache slot or state row changes the logits as a whole.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]

TINY = {
    "tiny_a": dict(
        config=dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=256, hidden_size=64,
                    num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
                    layer_types=["conv", "full_attention", "conv", "full_attention"], block_ff_dim=128,
                    block_auto_adjust_ff_dim=False, conv_L_cache=3, conv_bias=False, rope_theta=10000.0,
                    norm_eps=1e-5, tie_word_embeddings=True, eos_token_id=7),
        seed=11, norm_init="one_plus_normal", storage="bfloat16"),
    "tiny_b": dict(
        config=dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=512, hidden_size=96,
                    num_hidden_layers=6, num_attention_heads=3, num_key_value_heads=1, max_position_embeddings=256,
                    layer_types=["full_attention", "conv", "conv", "full_attention", "conv", "full_attention"],
                    block_ff_dim=288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
                    block_multiple_of=64, conv_L_cache=4, conv_bias=True, rope_theta=1000000.0, norm_eps=1e-6,
                    tie_word_embeddings=False, eos_token_id=[3, 5]),
        seed=23, norm_init="normal", storage="bfloat16"),
    "tiny_c": dict(
        config=dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=331, hidden_size=80,
                    num_hidden_layers=5, num_attention_heads=5, num_key_value_heads=5, head_dim=48,
                    max_position_embeddings=512,
                    layer_types=["sliding_attention", "conv", "full_attention", "sliding_attention", "conv"],
                    sliding_window=24, block_ff_dim=200, block_auto_adjust_ff_dim=True, block_multiple_of=8,
                    conv_L_cache=2, conv_bias=False, rope_theta=50000.0, norm_eps=3e-6,
                    tie_word_embeddings=True, eos_token_id=2),
        seed=37, norm_init="one_plus_normal", storage="float32"),
    # head size 64 with four heads per KV head and sizes in multiples of 16: the shapes for which the
    # tensor-core attention kernels, the fused epilogues and the tcgen05 contractions are chosen
    "tiny_d": dict(
        config=dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=1000, hidden_size=256,
                    num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2, head_dim=64,
                    max_position_embeddings=1024,
                    layer_types=["conv", "full_attention", "conv", "full_attention"],
                    block_ff_dim=768, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0,
                    block_multiple_of=256, conv_L_cache=3, conv_bias=False, rope_theta=1000000.0, norm_eps=1e-5,
                    tie_word_embeddings=True, eos_token_id=7),
        seed=41, norm_init="one_plus_normal", storage="bfloat16"),
    # head size 64 again, otherwise unlike tiny_d: two heads per KV head, a windowed layer first, four
    # taps with a bias, an untied head over a vocabulary that is no power of two, a width of 192
    "tiny_e": dict(
        config=dict(architectures=["Lfm2ForCausalLM"], model_type="lfm2", vocab_size=777, hidden_size=192,
                    num_hidden_layers=5, num_attention_heads=6, num_key_value_heads=3, head_dim=64,
                    max_position_embeddings=512,
                    layer_types=["sliding_attention", "conv", "conv", "full_attention", "sliding_attention"],
                    sliding_window=40, block_ff_dim=320, block_auto_adjust_ff_dim=False, conv_L_cache=4,
                    conv_bias=True, rope_theta=10000.0, norm_eps=1e-6, tie_word_embeddings=False, eos_token_id=[1, 9]),
        seed=53, norm_init="normal", storage="bfloat16"),
}


for _name in list(TINY):
    _spec = TINY[_name]
    TINY["loud_" + _name[-1]] = dict(_spec, seed=_spec["seed"] + 100, norm_init="one_plus_normal",
                                     std=float(_spec["config"]["hidden_size"]) ** -0.5)
QUIET = [n for n in TINY if n.startswith("tiny_")]
LOUD = [n for n in TINY if n.startswith("loud_")]


def make_model_folder(folder, name: str) -> Path:
    import torch
    import zinfer_b200 as z

    spec = TINY[name]
    cfg = z.config_from_dict(spec["config"])
    return z.write_random_model(folder, cfg, spec["seed"], std=spec.get("std", 0.02), norm_init=spec["norm_init"],
                                storage_dtype=getattr(torch, spec["storage"]))


def random_tokens(seed: int, n: int, vocab: int) -> list[int]:
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def rel_err(got: np.ndarray, ref: np.ndarray) -> float:
    """Largest absolute difference relative to the largest reference magnitude."""
    scale = float(np.max(np.abs(ref)))
    assert scale > 0, "reference logits are all zero: the comparison would be empty"
    return float(np.max(np.abs(got.astype(np.float64) - ref.astype(np.float64)))) / scale


# Tolerances: largest absolute error relative to max |logit| of the plain float64 implementation.
# TOL holds for the tiny_* configurations as specified (weights N(0, 0.02)).  The loud variants,
# and any model whose contractions keep the size of their input (the LFM2-1.2B shape with
# N(0, 0.02) at width 2048 is one), have a higher floor in bfloat16: rounding nothing but the
# inputs of the contractions, the cache and the probabilities to bfloat16, with exact
# arithmetic otherwise, already gives 1.2e-2 to 2.8e-2 (test_plain.py measures it with
# PlainLfm2(round_activations=...)), most of it from the normalised rows that enter every
# contraction.  A wrong row, slot, chunk or state moves these models' logits by 0.3 or more.
TOL = {"float32": 5e-5, "bfloat16": 2e-2}
TOL_LOUD = {"float32": 5e-5, "bfloat16": 4e-2}


def tol(name: str, dtype: str) -> float:
    return (TOL_LOUD if name.startswith("loud_") else TOL)[dtype]


def run_trace(model_dir, dtype: str, steps: list[dict], max_tokens: int, out_dir) -> dict[int, np.ndarray]:
    """Runs bin/trace_run on `steps`; returns step -> float32 array [wanted, vocab]."""
    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out",
                           str(out_dir), "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True,
                          timeout=900, env=dict(os.environ, ZINFER_PYTHON=sys.executable))
    assert proc.returncode == 0, f"trace_run failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], proc.stdout[-2000:]
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    out = {}
    for s in steps:
        f = out_dir / f"{s['step']}.f32"
        wanted = sum(len(e.get("want", [])) for e in s["entries"])
        if wanted:
            out[s["step"]] = np.fromfile(f, dtype="<f4").reshape(wanted, vocab)
        else:
            assert not f.exists()
    return out
