"""The command line run to the end on a GPU, as a user runs it: `bin/zinfer_b200 -m DIR -p IDS -n N
--temp 0` prints the tokens the plain implementation's greedy decoding gives; `-f FILE` serves
several prompts; `--dump-logits` writes the logits at each prompt's last token; `--bench PP,TG
--batch-sizes ...` reports both rates (src/main.zig:309-667, 669-699)."""
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import helpers
from plain_lfm2 import PlainLfm2

pytestmark = pytest.mark.gpu


def run_cli(*args):
    proc = subprocess.run([str(helpers.ROOT / "bin" / "zinfer_b200"), *map(str, args)], capture_output=True, text=True,
                          timeout=600, env=dict(os.environ, ZINFER_PYTHON=sys.executable))
    assert proc.returncode == 0, f"zinfer_b200 {args} failed ({proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}"
    return proc


def parse_line(line):
    m = re.fullmatch(r"([\d ]*?)\s*\[(\w+)\]", line.strip())
    assert m, line
    return [int(t) for t in m.group(1).split()], m.group(2)


@pytest.mark.parametrize("name", ["loud_a", "loud_e"])
def test_greedy_tokens_of_the_command_line_are_the_plain_ones(model_folders, tmp_path, name):
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    prompts = [helpers.random_tokens(600 + i, n, vocab) for i, n in enumerate([9, 1, 30])]
    want = [plain.greedy(p, 8) for p in prompts]

    one = run_cli("-m", folder, "-p", ",".join(map(str, prompts[0])), "-n", 8, "--temp", 0, "--stop", "", "--dtype", "fp32", "-v")
    assert parse_line(one.stdout.strip().splitlines()[-1]) == (want[0][0], "length")
    assert "prompt: 9 tokens" in one.stderr and "gen: 8 tokens" in one.stderr and "model:" in one.stderr

    listing = tmp_path / "prompts.txt"
    listing.write_text("".join(" ".join(map(str, p)) + "\n" for p in prompts))
    dump = tmp_path / "last.f32"
    many = run_cli("-m", folder, "-f", listing, "-n", 8, "--temp", 0, "--stop", "", "--dtype", "fp32", "--max-batch", 2,
                   "--dump-logits", dump)
    lines = [parse_line(l) for l in many.stdout.strip().splitlines()]
    assert lines == [(w[0], "length") for w in want]
    got = np.fromfile(dump, dtype="<f4").reshape(3, vocab)
    for i, p in enumerate(prompts):
        ref = plain.logits(p)
        assert np.abs(got[i] - ref[-1]).max() <= helpers.tol(name, "float32") * np.abs(ref).max()

    # a stop token: the model's greedy third token of the first prompt ends it, unprinted
    stopped = run_cli("-m", folder, "-p", " ".join(map(str, prompts[0])), "-n", 8, "--temp", 0, "--stop", want[0][0][2],
                      "--dtype", "fp32")
    toks, why = parse_line(stopped.stdout.strip().splitlines()[-1])
    assert why == "stop" and toks == want[0][0][:want[0][0].index(want[0][0][2])]


def test_bench_mode_reports_prompt_and_generation_rates(model_folders):
    out = run_cli("-m", model_folders["tiny_d"], "--bench", "64,8", "--batch-sizes", "1,3").stdout.strip().splitlines()
    assert len(out) == 2
    for line, b in zip(out, (1, 3)):
        m = re.fullmatch(rf"batch {b}: prompt: (\d+) tokens, ([\d.]+) tok/s \| gen: (\d+) tokens, ([\d.]+) tok/s \| 1 batches, 7 decode steps", line)
        assert m, line
        assert int(m.group(1)) == 64 * b and int(m.group(3)) == 8 * b and float(m.group(2)) > 0 and float(m.group(4)) > 0
