"""Plain, slow LFM2 in NumPy: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It shares no code with the package
under test: it has its own config reading, its own safetensors reader and its
own arithmetic.  It restates the formulas of pylypenko99/zinfer's CPU engine for
the `lfm2` architecture; every function cites the file and lines it restates
(paths inside that project).  zinfer's own code cannot be compiled on the build
machine (it needs a Zig 0.17 compiler, which is not installed and cannot be
installed offline), so this file rests on the formulas, not on a run of zinfer.

Deliberate differences from zinfer's arithmetic, both making this file more exact:
`exp` is the exact library function instead of the degree-6 polynomial
(src/ffn.zig:12-28) and no softmax tile is skipped (src/attention.zig:493).

Everything is computed in `dtype` (float32 by default, float64 on request).

`act` (a function, usually `to_bf16`) makes the parts round what a reduced-precision pipeline
has to round even with exact arithmetic: the inputs and outputs of the contractions, what goes
into the cache, and the probabilities.  It measures the error floor of such a pipeline; no
comparison with the engine uses it as the expected value.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- files

def read_safetensors(path) -> dict[str, np.ndarray]:
    """Reads every tensor of a safetensors file into float32 / int arrays.

    The container replaces zinfer's GGUF reader (src/gguf.zig:140-255): an
    8-byte little-endian header length, a JSON header {name: {dtype, shape,
    data_offsets}}, then raw little-endian data.
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = raw[base + a:base + b]
        dt = info["dtype"]
        if dt == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float32)
        elif dt == "BF16":
            u = np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32)
        elif dt == "F16":
            arr = np.frombuffer(buf, dtype="<f2").astype(np.float32)
        elif dt == "I32":
            arr = np.frombuffer(buf, dtype="<i4").copy()
        elif dt == "I64":
            arr = np.frombuffer(buf, dtype="<i8").copy()
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = arr.reshape(info["shape"])
    return out


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Rounds float32 values to the nearest bfloat16 (ties to even), kept as float32."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return rounded.astype(np.uint32).view(np.float32).reshape(x.shape)


# --------------------------------------------------------------------------- config

def ffn_dim(cfg: dict) -> int:
    """Effective SwiGLU width.  zinfer reads the effective width from the file
    (src/model.zig:423-440); a config.json carries `block_ff_dim` and the rule
    2/3 -> multiplier -> round up to `block_multiple_of`."""
    f = int(cfg.get("block_ff_dim", cfg.get("intermediate_size")))
    if cfg.get("block_auto_adjust_ff_dim", False):
        f = int(2 * f / 3)
        mult = cfg.get("block_ffn_dim_multiplier", None)
        if mult is not None:
            f = int(mult * f)
        mo = int(cfg.get("block_multiple_of", 256))
        f = mo * ((f + mo - 1) // mo)
    return f


def layer_kinds(cfg: dict) -> list[str]:
    """Mixer kind per layer: zinfer takes it from the per-layer KV-head array, 0 = conv
    (src/model.zig:492-508); config.json lists `layer_types` or `full_attn_idxs`."""
    n = int(cfg["num_hidden_layers"])
    if cfg.get("layer_types") is not None:
        return list(cfg["layer_types"])
    idx = set(cfg.get("full_attn_idxs") or range(n))
    return ["full_attention" if i in idx else "conv" for i in range(n)]


def rope_theta(cfg: dict) -> float:
    if "rope_theta" in cfg:
        return float(cfg["rope_theta"])
    rp = cfg.get("rope_parameters") or {}
    return float(rp.get("rope_theta", 10000.0))  # src/model.zig:446


# --------------------------------------------------------------------------- parts

def rms_norm(x: np.ndarray, w: np.ndarray, eps: float, dtype=np.float32) -> np.ndarray:
    """y = x * 1/sqrt(mean(x^2) + eps) * w over the last axis; scale first, weight second
    (src/model.zig:1166-1181)."""
    x = x.astype(dtype)
    ss = np.sum(x * x, axis=-1, keepdims=True, dtype=dtype)
    scale = (dtype(1.0) / np.sqrt(ss / dtype(x.shape[-1]) + dtype(eps))).astype(dtype)
    return (x * scale * w.astype(dtype)).astype(dtype)


def rope_inv_freq(theta: float, n_rot: int) -> np.ndarray:
    """f_i = theta^(-2i/n_rot) in float64, cast to float32 (src/rope.zig:8-16)."""
    i = np.arange(n_rot // 2, dtype=np.float64)
    return np.power(np.float64(theta), -2.0 * i / np.float64(n_rot)).astype(np.float32)


def apply_rope(x: np.ndarray, positions: np.ndarray, inv_freq: np.ndarray, dtype=np.float32) -> np.ndarray:
    """NeoX pairing (i, i + n_rot/2) on x[T, heads, hd]; angle = float32(pos) * f_i in
    float32 (src/rope.zig:34-45, 50-64; NeoX because arch != llama, src/model.zig:449)."""
    half = inv_freq.shape[0]
    ang = positions.astype(np.float32)[:, None] * inv_freq[None, :]          # float32 product
    cos = np.cos(ang.astype(np.float64)).astype(dtype)[:, None, :]
    sin = np.sin(ang.astype(np.float64)).astype(dtype)[:, None, :]
    x = x.astype(dtype)
    a = x[..., :half]
    b = x[..., half:2 * half]
    out = x.copy()
    out[..., :half] = a * cos - b * sin
    out[..., half:2 * half] = a * sin + b * cos
    return out


def _act(act, x, dtype):
    return x if act is None else act(np.asarray(x, dtype=np.float32)).astype(dtype)


def short_conv(xn, w_in, conv_w, w_out, conv_b=None, b_in=None, b_out=None, dtype=np.float32, act=None):
    """Gated short convolution of a whole sequence starting from a zero state
    (src/model.zig:1994-2028): [B, C, X] = xn W_in^T; u = B*X;
    c_t = sum_k w[:, k] u_{t-(K-1)+k} (tap K-1 on the current token); y = C*c; y W_out^T.
    `conv_w` is [D, K] (channel, tap).  Biases are this build's extension (zinfer has none)."""
    T, D = xn.shape
    K = conv_w.shape[-1]
    bcx = xn.astype(dtype) @ w_in.astype(dtype).T
    if b_in is not None:
        bcx = bcx + b_in.astype(dtype)
    bcx = _act(act, bcx, dtype)
    Bg, Cg, X = bcx[:, :D], bcx[:, D:2 * D], bcx[:, 2 * D:]
    u = Bg * X
    hist = np.concatenate([np.zeros((K - 1, D), dtype=dtype), u], axis=0)
    c = np.zeros((T, D), dtype=dtype)
    for k in range(K):                                  # tap 0 first, as the FMA chain does
        c = c + conv_w[:, k].astype(dtype)[None, :] * hist[k:k + T]
    if conv_b is not None:
        c = c + conv_b.astype(dtype)[None, :]
    y = _act(act, Cg * c, dtype)
    out = y @ w_out.astype(dtype).T
    if b_out is not None:
        out = out + b_out.astype(dtype)
    return out.astype(dtype)


def gqa_attention(xn, wq, wk, wv, wo, q_norm_w, k_norm_w, n_heads, n_kv, hd, eps, inv_freq,
                  window=0, dtype=np.float32, cache_round=None, encode=None, act=None):
    """Grouped-query attention over a whole sequence (src/model.zig:1715-1991):
    q,k,v projections; per-head RMSNorm of q and k with the layer eps
    (src/model.zig:1741-1744, 1760-1763); RoPE; causal scores (q.k)*1/sqrt(hd)
    (src/attention.zig:486); softmax; PV; query head h reads KV head h // (H/Hkv)
    (src/model.zig:1330, 1360); keys [max(0, p+1-window), p] (src/model.zig:1362-1363).
    `cache_round` (a function) rounds q, k and v the way a reduced-precision cache would.
    `encode` (a function (q, k, positions) -> (q, k)) stands for another position encoding, run
    where the rotation runs; tests of parts that are not the reference's use it."""
    T, _ = xn.shape
    xn = xn.astype(dtype)
    q = _act(act, xn @ wq.astype(dtype).T, dtype).reshape(T, n_heads, hd)
    k = _act(act, xn @ wk.astype(dtype).T, dtype).reshape(T, n_kv, hd)
    v = _act(act, xn @ wv.astype(dtype).T, dtype).reshape(T, n_kv, hd)
    if act is not None and cache_round is None:
        cache_round = act
    pos = np.arange(T)
    if q_norm_w is not None:
        q = rms_norm(q, q_norm_w, eps, dtype)
        k = rms_norm(k, k_norm_w, eps, dtype)
    if inv_freq is not None:
        q = apply_rope(q, pos, inv_freq, dtype)
        k = apply_rope(k, pos, inv_freq, dtype)
    if encode is not None:
        q, k = encode(q, k, pos)
    if cache_round is not None:
        q, k, v = cache_round(q).astype(dtype), cache_round(k).astype(dtype), cache_round(v).astype(dtype)
    g = n_heads // n_kv
    scale = dtype(1.0 / math.sqrt(hd))
    out = np.zeros((T, n_heads, hd), dtype=dtype)
    for h in range(n_heads):
        kh = h // g
        s = (q[:, h, :] @ k[:, kh, :].T) * scale                       # [T, T]
        i = pos[:, None]
        j = pos[None, :]
        mask = j <= i
        if window and window > 0:
            mask &= j >= (i + 1 - window)
        s = np.where(mask, s, -np.inf)
        m = np.max(s, axis=-1, keepdims=True)
        p = np.exp(s - m)
        out[:, h, :] = (_act(act, p, dtype) @ v[:, kh, :]) / np.sum(p, axis=-1, keepdims=True)
    return (_act(act, out.reshape(T, n_heads * hd), dtype) @ wo.astype(dtype).T).astype(dtype)


def swiglu(xn, w1, w3, w2, dtype=np.float32, act=None):
    """h = silu(xn W1^T) * (xn W3^T); out = h W2^T; silu(g) = g / (1 + exp(-g))
    (src/model.zig:1085-1117, 2411-2422; src/ffn.zig:31-33, 49-57)."""
    xn = xn.astype(dtype)
    g = xn @ w1.astype(dtype).T
    u = xn @ w3.astype(dtype).T
    h = _act(act, g / (dtype(1.0) + np.exp(-g)) * u, dtype)
    return (h @ w2.astype(dtype).T).astype(dtype)


# --------------------------------------------------------------------------- model

class PlainLfm2:
    """Whole-sequence LFM2 forward from a model folder (config.json + model.safetensors)."""

    def __init__(self, folder, dtype=np.float32, round_weights_bf16=False, round_activations=None):
        folder = Path(folder)
        self.cfg = json.loads((folder / "config.json").read_text())
        self.w = read_safetensors(folder / "model.safetensors")
        if round_weights_bf16:
            self.w = {k: (to_bf16(v) if v.dtype == np.float32 and v.ndim >= 2 else v) for k, v in self.w.items()}
        self.dtype = dtype
        self.act = round_activations
        c = self.cfg
        self.D = int(c["hidden_size"])
        self.H = int(c["num_attention_heads"])
        self.Hkv = int(c["num_key_value_heads"])
        self.hd = int(c.get("head_dim") or self.D // self.H)
        self.eps = float(c.get("norm_eps", 1e-5))                      # src/model.zig:445
        self.kinds = layer_kinds(c)
        self.window = int(c.get("sliding_window") or 0)
        self.inv_freq = rope_inv_freq(rope_theta(c), self.hd)
        self.tied = bool(c.get("tie_word_embeddings", c.get("tie_embedding", True)))

    def layer(self, i, x, cache_round=None):
        """x += Mixer(RMSNorm(x, operator_norm)); x += FFN(RMSNorm(x, ffn_norm))
        (src/model.zig:2395-2422)."""
        w, dt, p = self.w, self.dtype, f"model.layers.{i}."
        xn = _act(self.act, rms_norm(x, w[p + "operator_norm.weight"], self.eps, dt), dt)
        kind = self.kinds[i]
        if kind == "conv":
            cw = w[p + "conv.conv.weight"]
            cw = cw.reshape(cw.shape[0], cw.shape[-1])
            y = short_conv(xn, w[p + "conv.in_proj.weight"], cw, w[p + "conv.out_proj.weight"],
                           conv_b=w.get(p + "conv.conv.bias"), b_in=w.get(p + "conv.in_proj.bias"),
                           b_out=w.get(p + "conv.out_proj.bias"), dtype=dt, act=self.act)
        else:
            y = gqa_attention(xn, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
                              w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
                              w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
                              self.H, self.Hkv, self.hd, self.eps, self.inv_freq,
                              window=self.window if kind == "sliding_attention" else 0,
                              dtype=dt, cache_round=cache_round, act=self.act)
        x = x + y
        xn = _act(self.act, rms_norm(x, w[p + "ffn_norm.weight"], self.eps, dt), dt)
        x = x + swiglu(xn, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
                       w[p + "feed_forward.w2.weight"], dt, act=self.act)
        return x

    def hidden(self, tokens, cache_round=None):
        x = self.w["model.embed_tokens.weight"][np.asarray(tokens)].astype(self.dtype)   # src/model.zig:2352-2358
        for i in range(len(self.kinds)):
            x = self.layer(i, x, cache_round)
        return x

    def logits(self, tokens, cache_round=None) -> np.ndarray:
        """Logits [T, V] at every position of one sequence.  Final norm is the embedding norm
        (src/model.zig:599-600, 2484-2486); the head is lm_head or the tied embedding
        (src/model.zig:595-598, 2490)."""
        x = self.hidden(tokens, cache_round)
        xn = _act(self.act, rms_norm(x, self.w["model.embedding_norm.weight"], self.eps, self.dtype), self.dtype)
        head = self.w["model.embed_tokens.weight"] if self.tied else self.w["lm_head.weight"]
        return (xn @ head.astype(self.dtype).T).astype(np.float32)

    def greedy(self, prompt, max_new, stop_ids=()):
        """Greedy generation by recomputing the whole sequence for every token
        (src/gen.zig:434-537: the stop token is returned but not appended)."""
        toks = list(prompt)
        out = []
        for _ in range(max_new):
            nxt = int(np.argmax(self.logits(toks)[-1]))              # first maximum wins, src/sampler.zig:532-610
            if nxt in stop_ids:
                return out, "stop"
            out.append(nxt)
            toks.append(nxt)
        return out, "length"


# --------------------------------------------------------------------------- sampling

def softmax_temperature(logits: np.ndarray, temp: float) -> np.ndarray:
    """p ~ exp((l - l_max)/T) (src/sampler.zig:236-242)."""
    l = logits.astype(np.float64)
    e = np.exp((l - l.max()) / temp)
    return e / e.sum()


def filtered_probs(logits, temp, top_k=0, top_p=1.0, min_p=0.0):
    """Probabilities after zinfer's filter chain: top-k, top-p and min-p on untempered
    probabilities relative to the best, then temperature on the survivors
    (src/sampler.zig:190-242).  Returns a dense vector over the vocabulary."""
    l = logits.astype(np.float64)
    order = np.argsort(-l, kind="stable")
    k = len(l) if top_k == 0 or top_k > len(l) else top_k
    cand = order[:k]
    mx = l[cand[0]]
    keep = k
    if top_p < 1:
        e = np.exp(l[cand] - mx)
        acc = np.cumsum(e)
        keep = int(np.argmax(acc >= top_p * e.sum())) + 1
    if min_p > 0:
        e = np.exp(l[cand[:keep]] - mx)
        bad = np.nonzero(e < min_p)[0]
        if len(bad):
            keep = max(int(bad[0]), 1)
    p = np.zeros_like(l)
    e = np.exp((l[cand[:keep]] - mx) / temp)
    p[cand[:keep]] = e / e.sum()
    return p


def repeat_penalty(logits, recent, penalty):
    """Each distinct token among the last 64 once: l>0 ? l/F : l*F (src/sampler.zig:91-100)."""
    out = logits.copy()
    for t in dict.fromkeys(recent[-64:]):
        out[t] = out[t] / penalty if out[t] > 0 else out[t] * penalty
    return out
