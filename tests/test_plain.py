"""The plain implementation checks itself: each part against a second, independent formulation
(loops instead of matrices, a recurrence instead of a window), and properties that any correct
decoder has (causality, rotation keeps the norm)."""
import math

import numpy as np
import pytest

import helpers
import plain_lfm2 as P


def rnd(shape, seed, scale=1.0):
    return (np.random.default_rng(seed).standard_normal(shape) * scale).astype(np.float64)


def test_rms_norm_against_the_definition():
    x, w = rnd((3, 10), 1), rnd((10,), 2)
    y = P.rms_norm(x, w, 1e-5, np.float64)
    for i in range(3):
        ms = sum(v * v for v in x[i]) / 10
        assert np.allclose(y[i], [x[i, j] / math.sqrt(ms + 1e-5) * w[j] for j in range(10)], rtol=1e-12)


def test_rope_keeps_norms_and_depends_on_relative_positions():
    f = P.rope_inv_freq(10000.0, 16)
    assert f[0] == 1.0 and all(f[i] > f[i + 1] for i in range(7))            # src/rope.zig:69-108
    q, k = rnd((1, 1, 16), 3), rnd((1, 1, 16), 4)
    dots = []
    for p0 in (0, 5, 100):
        qr = P.apply_rope(q, np.array([p0 + 7]), f, np.float64)
        kr = P.apply_rope(k, np.array([p0]), f, np.float64)
        assert abs(np.linalg.norm(qr) - np.linalg.norm(q)) < 1e-6
        dots.append(float((qr * kr).sum()))
    assert max(dots) - min(dots) < 1e-4
    assert np.array_equal(P.apply_rope(q, np.array([0]), f, np.float64), q)


def test_short_conv_against_a_token_by_token_recurrence():
    T, D, K = 9, 6, 4
    xn, w_in, w_out = rnd((T, D), 5), rnd((3 * D, D), 6, 0.3), rnd((D, D), 7, 0.3)
    cw, cb = rnd((D, K), 8), rnd((D,), 9)
    whole = P.short_conv(xn, w_in, cw, w_out, conv_b=cb, dtype=np.float64)
    state = np.zeros((K - 1, D))
    for t in range(T):
        bcx = w_in @ xn[t]
        u = bcx[:D] * bcx[2 * D:]
        hist = np.vstack([state, u[None]])
        c = np.array([sum(cw[ch, k] * hist[k, ch] for k in range(K)) for ch in range(D)]) + cb
        y = w_out @ (bcx[D:2 * D] * c)
        assert np.allclose(y, whole[t], atol=1e-12)
        state = hist[1:]


def test_attention_against_loops_with_window_and_groups():
    T, D, H, Hkv, hd = 7, 12, 4, 2, 6
    xn = rnd((T, D), 10)
    wq, wk, wv, wo = rnd((H * hd, D), 11, 0.3), rnd((Hkv * hd, D), 12, 0.3), rnd((Hkv * hd, D), 13, 0.3), rnd((D, H * hd), 14, 0.3)
    qn, kn = 1 + rnd((hd,), 15, 0.1), 1 + rnd((hd,), 16, 0.1)
    f = P.rope_inv_freq(100.0, hd)
    for window in (0, 3):
        got = P.gqa_attention(xn, wq, wk, wv, wo, qn, kn, H, Hkv, hd, 1e-6, f, window=window, dtype=np.float64)
        q = P.apply_rope(P.rms_norm((xn @ wq.T).reshape(T, H, hd), qn, 1e-6, np.float64), np.arange(T), f, np.float64)
        k = P.apply_rope(P.rms_norm((xn @ wk.T).reshape(T, Hkv, hd), kn, 1e-6, np.float64), np.arange(T), f, np.float64)
        v = (xn @ wv.T).reshape(T, Hkv, hd)
        for t in range(T):
            heads = []
            for h in range(H):
                lo = max(0, t + 1 - window) if window else 0
                s = np.array([q[t, h] @ k[j, h // 2] / math.sqrt(hd) for j in range(lo, t + 1)])
                p = np.exp(s - s.max())
                p /= p.sum()
                heads.append(sum(p[j - lo] * v[j, h // 2] for j in range(lo, t + 1)))
            assert np.allclose(wo @ np.concatenate(heads), got[t], atol=1e-12)


def test_attention_takes_another_position_encoding_in_the_place_of_the_rotation():
    """The `encode` hook runs where the rotation runs: given the rotation itself it reproduces the
    built-in path, and given nothing the scores are position-free."""
    T, D, H, Hkv, hd = 6, 8, 2, 1, 4
    xn = rnd((T, D), 30)
    wq, wk, wv, wo = rnd((H * hd, D), 31, 0.3), rnd((Hkv * hd, D), 32, 0.3), rnd((Hkv * hd, D), 33, 0.3), rnd((D, H * hd), 34, 0.3)
    qn, kn = 1 + rnd((hd,), 35, 0.1), 1 + rnd((hd,), 36, 0.1)
    f = P.rope_inv_freq(50.0, hd)
    built_in = P.gqa_attention(xn, wq, wk, wv, wo, qn, kn, H, Hkv, hd, 1e-6, f, dtype=np.float64)
    rotate = lambda q, k, pos: (P.apply_rope(q, pos, f, np.float64), P.apply_rope(k, pos, f, np.float64))
    hooked = P.gqa_attention(xn, wq, wk, wv, wo, qn, kn, H, Hkv, hd, 1e-6, None, dtype=np.float64, encode=rotate)
    assert np.array_equal(built_in, hooked)
    bare = P.gqa_attention(xn, wq, wk, wv, wo, qn, kn, H, Hkv, hd, 1e-6, None, dtype=np.float64)
    assert not np.allclose(bare, built_in)


def test_swiglu_against_scalars():
    xn, w1, w3, w2 = rnd((2, 5), 17), rnd((7, 5), 18), rnd((7, 5), 19), rnd((5, 7), 20)
    got = P.swiglu(xn, w1, w3, w2, np.float64)
    for t in range(2):
        g, u = w1 @ xn[t], w3 @ xn[t]
        h = np.array([gi / (1 + math.exp(-gi)) * ui for gi, ui in zip(g, u)])
        assert np.allclose(w2 @ h, got[t], atol=1e-12)
    assert abs(float(P.swiglu(np.ones((1, 1)), np.ones((1, 1)), np.ones((1, 1)), np.ones((1, 1)), np.float64)[0, 0]) - 0.7310585786) < 1e-9


@pytest.mark.parametrize("name", list(helpers.TINY))
def test_whole_model_is_causal_and_float32_agrees_with_float64(model_folders, name):
    m64 = P.PlainLfm2(model_folders[name], dtype=np.float64)
    m32 = P.PlainLfm2(model_folders[name], dtype=np.float32)
    toks = helpers.random_tokens(3, 40, m64.cfg["vocab_size"])
    full = m64.logits(toks)
    assert full.shape == (40, m64.cfg["vocab_size"]) and np.abs(full).max() > 0
    assert np.allclose(m64.logits(toks[:17]), full[:17], atol=1e-6 * np.abs(full).max())
    changed = list(toks)
    changed[30] = (changed[30] + 1) % m64.cfg["vocab_size"]
    assert np.array_equal(m64.logits(changed)[:30], full[:30]) and not np.allclose(m64.logits(changed)[30:], full[30:])
    assert helpers.rel_err(m32.logits(toks), full) < 2e-5


def test_window_changes_logits_only_beyond_the_window(model_folders):
    m = P.PlainLfm2(model_folders["tiny_c"], dtype=np.float64)
    toks = helpers.random_tokens(4, 60, m.cfg["vocab_size"])
    a = m.logits(toks)
    m.window = 0
    m.kinds = ["full_attention" if k == "sliding_attention" else k for k in m.kinds]
    b = m.logits(toks)
    assert np.allclose(a[:24], b[:24], atol=1e-9) and not np.allclose(a[40:], b[40:], atol=1e-6)


def test_feed_forward_width_and_kinds():
    assert P.ffn_dim(dict(block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256)) == 8192
    assert P.ffn_dim(dict(block_ff_dim=288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=64)) == 192
    assert P.ffn_dim(dict(block_ff_dim=128)) == 128
    assert P.layer_kinds(dict(num_hidden_layers=3, full_attn_idxs=[1])) == ["conv", "full_attention", "conv"]


def test_sampling_reference_functions():
    l = np.array([1.0, 3.0, 2.0, 3.0, -1.0, 0.5])
    p = P.filtered_probs(l, temp=1.0, top_k=3)
    assert set(np.nonzero(p)[0]) == {1, 2, 3} and abs(p.sum() - 1) < 1e-12
    p = P.filtered_probs(l, temp=1.0, top_k=1)
    assert np.nonzero(p)[0].tolist() == [1]                      # first of the tied maxima
    p = P.filtered_probs(l, temp=0.5, top_p=0.6)
    assert set(np.nonzero(p)[0]) == {1, 3}
    p = P.filtered_probs(l, temp=1.0, min_p=0.2)
    assert set(np.nonzero(p)[0]) == {1, 2, 3}                    # exp(-1) = 0.37 stays, exp(-2) = 0.14 goes
    assert np.allclose(P.repeat_penalty(np.array([2.0, -2.0, 1.0]), [0, 1, 0], 2.0), [1.0, -4.0, 1.0])


@pytest.mark.parametrize("name,low,high", [("tiny_b", 5e-4, 4e-3), ("loud_a", 1e-2, 3e-2), ("loud_b", 1e-2, 3e-2),
                                           ("loud_d", 8e-3, 3e-2)])
def test_error_floor_of_a_bfloat16_pipeline(model_folders, name, low, high):
    """What bfloat16 costs when nothing else is inexact: float64 arithmetic with only the inputs
    and outputs of the contractions, the cache and the probabilities rounded.  On the configurations
    as specified the floor is a tenth of the tolerance; on the loud ones it is above the 2e-2 that
    holds there, which is why they have a tolerance of their own (helpers.TOL_LOUD)."""
    exact = P.PlainLfm2(model_folders[name], dtype=np.float64)
    rounded = P.PlainLfm2(model_folders[name], dtype=np.float64, round_activations=P.to_bf16)
    toks = helpers.random_tokens(1004, 64, exact.cfg["vocab_size"])
    floor = helpers.rel_err(rounded.logits(toks), exact.logits(toks))
    assert low <= floor <= high, floor
    assert floor < helpers.tol(name, "bfloat16")
