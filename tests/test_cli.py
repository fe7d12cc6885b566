"""The command line without a GPU: option names and defaults in the manner of the reference's
`zinfer` (src/main.zig:14-63), the parsing of token ids, the random-weights mode that writes a
model folder, and the errors that come before any device work."""
import json

import numpy as np
import pytest

import helpers
import plain_lfm2 as P
from zinfer_b200 import cli


def test_option_names_and_defaults_follow_the_reference():
    ap = cli.build_parser()
    a = ap.parse_args(["-m", "folder"])
    # the reference's defaults: -n 256, --temp 0.8, --top-k 40, --top-p 0.95, --min-p 0.05,
    # --repeat-penalty 1.0 (src/main.zig:20-43); DRY and XTC off
    assert (a.model, a.predict, a.temp, a.top_k, a.top_p, a.min_p, a.repeat_penalty) == ("folder", 256, 0.8, 40, 0.95, 0.05, 1.0)
    assert (a.dry_multiplier, a.dry_base, a.dry_allowed_length, a.dry_range) == (0.0, 1.75, 2, 1024)
    assert (a.xtc_probability, a.xtc_threshold, a.xtc_min_keep) == (0.0, 0.1, 1)
    assert a.seed is None and a.stop is None and a.ctx == 0 and a.dtype == "bf16"
    b = ap.parse_args(["--model", "f", "--prompt", "1,2", "--predict", "7", "--ctx", "512", "--batch", "64", "--temp", "0",
                       "--top-k", "0", "--top-p", "1", "--min-p", "0", "--repeat-penalty", "1.3", "--seed", "9",
                       "--dry-multiplier", "0.8", "--xtc-probability", "0.5", "--stop", "3 5", "--dtype", "float32", "-v"])
    assert (b.prompt, b.predict, b.ctx, b.batch, b.temp, b.top_k, b.seed, b.dtype, b.verbose) == \
        ("1,2", 7, 512, 64, 0.0, 0, 9, "float32", True)
    assert (b.repeat_penalty, b.dry_multiplier, b.xtc_probability, b.stop) == (1.3, 0.8, 0.5, "3 5")
    short = ap.parse_args(["-m", "f", "-p", "4", "-n", "3", "-c", "128", "-b", "32", "-f", "prompts.txt"])
    assert (short.prompt, short.predict, short.ctx, short.batch, short.file) == ("4", 3, 128, 32, "prompts.txt")


def test_help_lists_the_options(capsys):
    with pytest.raises(SystemExit) as e:
        cli.build_parser().parse_args(["--help"])
    assert e.value.code == 0
    text = capsys.readouterr().out
    for name in ("--model", "--prompt", "--predict", "--temp", "--top-k", "--top-p", "--min-p", "--repeat-penalty",
                 "--seed", "--dry-multiplier", "--xtc-probability", "--bench", "--random-weights", "--write"):
        assert name in text


@pytest.mark.parametrize("text,ids", [("1,2,3", [1, 2, 3]), ("5 17  3", [5, 17, 3]), (" 7, 8 ,9 ", [7, 8, 9]), ("", [])])
def test_token_ids_are_split_at_commas_and_blanks(text, ids):
    assert cli.parse_ids(text) == ids
    with pytest.raises(ValueError):
        cli.parse_ids("1,x")


def test_errors_before_any_model_is_loaded(capsys, tmp_path):
    assert cli.main([]) == 2
    assert "-m MODEL is required" in capsys.readouterr().err
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(helpers.TINY["tiny_a"]["config"]))
    assert cli.main(["--random-weights", str(cfg)]) == 2
    assert "--write" in capsys.readouterr().err


def test_random_weights_mode_writes_a_folder_that_the_plain_reader_takes(capsys, tmp_path):
    """`--random-weights CONFIG --write FOLDER --seed-weights S` needs no GPU: config.json and
    model.safetensors appear, the same seed gives the same bytes, another seed other ones."""
    conf = dict(helpers.TINY["tiny_b"]["config"])
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(conf))
    out = [tmp_path / n for n in ("m1", "m2", "m3")]
    for folder, seed in zip(out, ("3", "3", "4")):
        assert cli.main(["--random-weights", str(cfg), "--write", str(folder), "--seed-weights", seed]) == 0
        assert f"wrote {folder}" in capsys.readouterr().out
    written = json.loads((out[0] / "config.json").read_text())
    for key in ("architectures", "vocab_size", "hidden_size", "layer_types", "norm_eps", "conv_bias"):
        assert written[key] == conf[key]
    w = [P.read_safetensors(f / "model.safetensors") for f in out]
    assert set(w[0]) == set(w[1]) == set(w[2])
    assert "lm_head.weight" in w[0] and any(n.endswith("conv.conv.bias") for n in w[0])
    assert all(np.array_equal(w[0][n], w[1][n]) for n in w[0])
    assert any(not np.array_equal(w[0][n], w[2][n]) for n in w[0])
    D, V = conf["hidden_size"], conf["vocab_size"]
    assert w[0]["model.embed_tokens.weight"].shape == (V, D)
