"""The two plain implementations against each other: tests/plain_lfm2.py (NumPy, whole sequences,
no cache) and tests/forward_ref.cpp (C++, 32-bit floats, one sequence with a position counter, a
key/value cache and a convolution state, in the shape of the reference's State.forwardBatch,
src/model.zig:2347-2516).  They were written from the reference's lines independently, share no
code, read the model file with readers of their own, and must agree to 1e-5 of max |logit| on
every tiny configuration: whole prompts, and the same tokens fed in pieces and one by one (which
only the C++ one can do: it is also a check of what a cache and a state must hold).
Neither is anchored on a run of zinfer: no Zig compiler is available where this was written."""
import ctypes
import json
import shutil
import subprocess

import numpy as np
import pytest

import helpers
from plain_lfm2 import PlainLfm2


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    gxx = shutil.which("g++") or shutil.which("c++")
    if gxx is None:
        pytest.skip("no C++ compiler")
    out = tmp_path_factory.mktemp("forward_ref") / "forward_ref.so"
    subprocess.run([gxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-ffp-contract=off", "-o", str(out),
                    str(helpers.ROOT / "tests" / "forward_ref.cpp")], check=True)
    lib = ctypes.CDLL(str(out))
    lib.ref_open.argtypes = [ctypes.c_char_p, ctypes.c_float, ctypes.c_float, ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    lib.ref_open.restype = ctypes.c_void_p
    lib.ref_forward.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.POINTER(ctypes.c_float)]
    lib.ref_forward.restype = ctypes.c_int
    for name in ("ref_close", "ref_reset"):
        getattr(lib, name).argtypes = [ctypes.c_void_p]
        getattr(lib, name).restype = None
    for name in ("ref_vocab", "ref_layers"):
        getattr(lib, name).argtypes = [ctypes.c_void_p]
        getattr(lib, name).restype = ctypes.c_int
    lib.ref_error.restype = ctypes.c_char_p
    return lib


class Ref:
    def __init__(self, lib, folder):
        cfg = json.loads((folder / "config.json").read_text())
        kinds = cfg["layer_types"]
        windows = (ctypes.c_int * len(kinds))(*[int(cfg.get("sliding_window") or 0) if k == "sliding_attention" else 0
                                                 for k in kinds])
        self.lib = lib
        self.st = lib.ref_open(str(folder / "model.safetensors").encode(), cfg.get("norm_eps", 1e-5),
                               cfg.get("rope_theta", 10000.0), windows, cfg["max_position_embeddings"])
        assert self.st, lib.ref_error().decode()
        assert lib.ref_layers(self.st) == cfg["num_hidden_layers"] and lib.ref_vocab(self.st) == cfg["vocab_size"]
        self.vocab = cfg["vocab_size"]

    def forward(self, tokens):
        toks = (ctypes.c_int * len(tokens))(*tokens)
        out = np.empty((len(tokens), self.vocab), dtype=np.float32)
        rc = self.lib.ref_forward(self.st, toks, len(tokens), out.ctypes.data_as(ctypes.POINTER(ctypes.c_float)))
        assert rc == 0, self.lib.ref_error().decode()
        return out

    def reset(self):
        self.lib.ref_reset(self.st)

    def close(self):
        self.lib.ref_close(self.st)


@pytest.mark.parametrize("name", list(helpers.TINY))
def test_the_two_plain_implementations_agree(ref, model_folders, name):
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    r = Ref(ref, folder)
    try:
        for seed, n in ((1, 70), (2, 33), (3, 1)):
            toks = helpers.random_tokens(2000 + seed, n, vocab)
            want = plain.logits(toks)
            whole = r.forward(toks)
            assert helpers.rel_err(whole, want) <= 1e-5, f"{name}: whole prompt of {n}"
            r.reset()
            # the same tokens in pieces: 5, then 2, then one by one; the cache and the state carry over
            cuts = [c for c in (5, 7) if c < n] + list(range(8, n)) + [n]
            pieces, a = [], 0
            for b in cuts:
                if b > a:
                    pieces.append(r.forward(toks[a:b]))
                    a = b
            assert helpers.rel_err(np.concatenate(pieces), want) <= 1e-5, f"{name}: prompt of {n} in pieces"
            r.reset()
    finally:
        r.close()


def test_the_cached_implementation_refuses_what_it_cannot_hold(ref, model_folders):
    r = Ref(ref, model_folders["tiny_a"])
    try:
        r.forward([1] * 128)
        toks = (ctypes.c_int * 1)(1)
        out = np.empty((1, 256), dtype=np.float32)
        assert ref.ref_forward(r.st, toks, 1, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))) == -1
        assert b"context full" in ref.ref_error()
        r.reset()
        bad = (ctypes.c_int * 1)(256)
        assert ref.ref_forward(r.st, bad, 1, out.ctypes.data_as(ctypes.POINTER(ctypes.c_float))) == -1
    finally:
        r.close()
