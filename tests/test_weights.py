"""Weights: lookup by name, kept dtypes, the one error that lists everything wrong, malformed
containers, the random-weights folder."""
import json
import struct

import numpy as np
import pytest
import torch

import helpers
from plain_lfm2 import read_safetensors
from zinfer_b200.config import config_from_dict
from zinfer_b200.weights import (SafetensorsFile, WeightError, WeightFileError, load_model, write_random_model,
                                 write_safetensors)


@pytest.fixture(scope="module")
def folder_b(tmp_path_factory):
    return helpers.make_model_folder(tmp_path_factory.mktemp("wb") / "m", "tiny_b")


def rewrite(folder, dst, edit):
    """Copies a model folder with its tensors passed through `edit(dict) -> dict`."""
    dst.mkdir(parents=True, exist_ok=True)
    (dst / "config.json").write_text((folder / "config.json").read_text())
    with SafetensorsFile(folder / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    write_safetensors(dst / "model.safetensors", edit(tensors))
    return dst


def test_loads_by_name_with_kept_dtypes(folder_b):
    for dtype in (torch.bfloat16, torch.float32):
        m = load_model(folder_b, dtype=dtype, device="cpu")
        blk = m.layers[1]
        assert blk.mixer.w_in.dtype == dtype and blk.mixer.w_in.shape == (3 * 96, 96)
        assert blk.mixer.taps.dtype == torch.float32 and blk.mixer.taps.shape == (4, 96)
        assert blk.mixer.conv_bias.dtype == torch.float32
        assert blk.mixer_norm.weight.dtype == torch.float32
        assert m.layers[0].mixer.w_qkv.shape == ((3 + 2) * 32, 96)
        assert m.layers[0].ffn.w_gate_up.shape == (2 * 192, 96)
        assert m.head.weight is not None and m.head.weight.shape == (512, 96)
    plain = read_safetensors(folder_b / "model.safetensors")
    got = load_model(folder_b, dtype=torch.float32, device="cpu")
    assert np.array_equal(got.layers[1].mixer.taps.numpy(), plain["model.layers.1.conv.conv.weight"].reshape(96, 4).T)
    assert np.array_equal(got.layers[0].mixer.w_qkv[:96].numpy(), plain["model.layers.0.self_attn.q_proj.weight"])
    # gate and up are stacked in groups of 16 rows: 16 of w1, the same 16 of w3, ...
    gu = got.layers[0].ffn.w_gate_up.numpy().reshape(12, 2, 16, 96)
    assert np.array_equal(gu[:, 0].reshape(192, 96), plain["model.layers.0.feed_forward.w1.weight"])
    assert np.array_equal(gu[:, 1].reshape(192, 96), plain["model.layers.0.feed_forward.w3.weight"])
    bcx = got.layers[1].mixer.w_in.numpy().reshape(6, 3, 16, 96)
    assert np.array_equal(bcx[:, 2].reshape(96, 96), plain["model.layers.1.conv.in_proj.weight"][192:])


def test_tied_head_uses_the_embedding(tmp_path):
    f = helpers.make_model_folder(tmp_path / "a", "tiny_a")
    m = load_model(f, dtype=torch.float32, device="cpu")
    assert m.head.weight is None and m.head.embedding is m.embedding
    with SafetensorsFile(f / "model.safetensors") as sf:
        assert "lm_head.weight" not in sf


def test_one_error_lists_missing_unexpected_and_wrong_shapes(folder_b, tmp_path):
    def edit(t):
        t.pop("model.layers.1.conv.conv.bias")
        t.pop("model.layers.3.self_attn.k_layernorm.weight")
        t["model.layers.9.extra.weight"] = torch.zeros(2)
        t["model.layers.0.feed_forward.w2.weight"] = torch.zeros(96, 191, dtype=torch.bfloat16)
        t["model.embedding_norm.weight"] = torch.zeros(96, dtype=torch.int32)
        return t

    bad = rewrite(folder_b, tmp_path / "bad", edit)
    with pytest.raises(WeightError) as e:
        load_model(bad, dtype=torch.float32, device="cpu")
    msg = str(e.value)
    assert e.value.missing == ["model.layers.1.conv.conv.bias", "model.layers.3.self_attn.k_layernorm.weight"]
    assert e.value.unexpected == ["model.layers.9.extra.weight"]
    assert "feed_forward.w2.weight' has shape [96, 191], expected [96, 192]" in msg
    assert "embedding_norm.weight' has dtype torch.int32" in msg
    for name in e.value.missing + e.value.unexpected:
        assert name in msg


def test_stored_float32_vector_stays_float32_and_matrix_follows_the_run_dtype(tmp_path):
    f = helpers.make_model_folder(tmp_path / "c", "tiny_c")          # stored in float32
    m = load_model(f, dtype=torch.bfloat16, device="cpu")
    plain = read_safetensors(f / "model.safetensors")
    assert m.final_norm.weight.dtype == torch.float32
    assert np.array_equal(m.final_norm.weight.numpy(), plain["model.embedding_norm.weight"])
    assert m.embedding.weight.dtype == torch.bfloat16
    m32 = load_model(f, dtype=torch.float32, device="cpu")
    assert np.array_equal(m32.embedding.weight.numpy(), plain["model.embed_tokens.weight"])


def test_optional_projection_biases_are_taken_when_present(folder_b, tmp_path):
    def edit(t):
        t["model.layers.1.conv.in_proj.bias"] = torch.ones(288)
        return t

    m = load_model(rewrite(folder_b, tmp_path / "pb", edit), dtype=torch.float32, device="cpu")
    assert m.layers[1].mixer.in_bias is not None and m.layers[1].mixer.out_bias is None
    assert m.layers[2].mixer.in_bias is None


def test_every_prefix_of_a_file_fails_cleanly(folder_b, tmp_path):
    raw = (folder_b / "model.safetensors").read_bytes()
    (tmp_path / "config.json").write_text((folder_b / "config.json").read_text())
    (hlen,) = struct.unpack("<Q", raw[:8])
    cuts = sorted(set([0, 1, 7, 8, 9, 8 + hlen // 2, 8 + hlen - 1, 8 + hlen, 8 + hlen + 1, len(raw) // 2, len(raw) - 1]))
    for n in cuts:
        (tmp_path / "model.safetensors").write_bytes(raw[:n])
        with pytest.raises((WeightFileError, WeightError)):
            load_model(tmp_path, dtype=torch.float32, device="cpu")


@pytest.mark.parametrize("header,match", [
    (b"[1, 2]", "JSON object"),
    (b"{not json", "not valid JSON"),
    (json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode(), "needs 16 bytes"),
    (json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 1 << 40]}}).encode(), "outside the file"),
    (json.dumps({"t": {"dtype": "Q4_0", "shape": [4], "data_offsets": [0, 16]}}).encode(), "unsupported dtype"),
    (json.dumps({"t": {"dtype": "F32", "shape": [-4], "data_offsets": [0, 16]}}).encode(), "negative"),
    (json.dumps({"t": {"dtype": "F32"}}).encode(), "malformed"),
])
def test_malformed_headers(tmp_path, header, match):
    p = tmp_path / "x.safetensors"
    p.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 16)
    with pytest.raises(WeightFileError, match=match):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 62) + b"{}")
    with pytest.raises(WeightFileError, match="header length"):
        SafetensorsFile(p)


def test_random_folder_is_seeded_and_independent_of_order(tmp_path):
    cfg = config_from_dict(helpers.TINY["tiny_a"]["config"])
    a = read_safetensors(write_random_model(tmp_path / "a", cfg, 5) / "model.safetensors")
    b = read_safetensors(write_random_model(tmp_path / "b", cfg, 5) / "model.safetensors")
    c = read_safetensors(write_random_model(tmp_path / "c", cfg, 6) / "model.safetensors")
    assert a.keys() == b.keys() and all(np.array_equal(a[k], b[k]) for k in a)
    assert not np.array_equal(a["model.embed_tokens.weight"], c["model.embed_tokens.weight"])
    assert a["model.layers.0.conv.conv.weight"].shape == (64, 1, 3)
    w = a["model.layers.1.feed_forward.w1.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(w.mean())) < 0.002
    assert abs(float(a["model.layers.0.operator_norm.weight"].mean()) - 1.0) < 0.02
    cfg_json = json.loads((tmp_path / "a" / "config.json").read_text())
    assert cfg_json["architectures"] == ["Lfm2ForCausalLM"] and cfg_json["vocab_size"] == 256
    from zinfer_b200.weights import random_model
    mem = random_model(cfg, 5, dtype=torch.float32, device="cpu")
    assert np.array_equal(mem.embedding.weight.numpy(), a["model.embed_tokens.weight"])


def test_sharded_folder(folder_b, tmp_path):
    with SafetensorsFile(folder_b / "model.safetensors") as f:
        tensors = {n: f.tensor(n) for n in f.names()}
    names = list(tensors)
    half = len(names) // 2
    write_safetensors(tmp_path / "s1.safetensors", {n: tensors[n] for n in names[:half]})
    write_safetensors(tmp_path / "s2.safetensors", {n: tensors[n] for n in names[half:]})
    index = {"weight_map": {n: ("s1.safetensors" if i < half else "s2.safetensors") for i, n in enumerate(names)}}
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(index))
    (tmp_path / "config.json").write_text((folder_b / "config.json").read_text())
    m = load_model(tmp_path, dtype=torch.float32, device="cpu")
    assert m.embedding.weight.shape == (512, 96)
