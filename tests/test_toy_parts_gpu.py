"""The framework takes parts and architectures it has never seen, without a change to its files:
a toy mixer with fixed-size state of its own (an exponential moving average), registered from
this test together with a toy architecture that uses it beside the library's attention; a
schedule that runs a layer twice and lets one entry read another entry's cache; a toy norm
written to the base interface alone; and a toy mixer whose growing cache is ONE vector per token.
All are built from a config.json, filled with random weights, loaded by name and stepped whole and
token by token against a plain NumPy restatement written here.  The toy mixers read their batch
on the host, so they cannot be recorded in a CUDA graph: the engine, asked for graphs, runs their
single-token steps one by one instead."""
import json
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import helpers
import plain_lfm2 as P

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------- the toy mixer

def make_toy():
    from zinfer_b200.config import Lfm2Config, register_architecture, unregister_architecture
    from zinfer_b200.models import LayerCall, Model
    from zinfer_b200.parts import (MIXERS, NORMS, GqaAttention, KVRequest, LMHead, Mixer, Norm, PreNormBlock, RMSNorm,
                                   RotaryEncoding, StateRequest, SwiGLU, TokenEmbedding, WeightSpec, linear)

    class MeanAbsNorm(Norm):
        """y = x / (mean |x| + eps) * w, written to the base interface alone: forward(ctx, x, rows)."""

        def __init__(self, dim, eps, weight_name):
            self.dim, self.eps, self.weight_name = dim, eps, weight_name

        def weight_specs(self):
            return [WeightSpec(self.weight_name, (self.dim,), role="vector", init="norm")]

        def load(self, weights, dtype, device):
            self.weight = weights[self.weight_name]

        def forward(self, ctx, x, rows=None):
            if rows is not None:
                x = x[rows.long()]
            return (x / (x.abs().mean(-1, keepdim=True) + self.eps) * self.weight).to(ctx.dtype)

    class LatentMixer(Mixer):
        """c_t = xn_t W_c^T is the one vector a token leaves in the cache; out += mean(c_0..c_t) W_o^T."""

        def __init__(self, hidden, rank, c_name, o_name):
            self.hidden, self.rank, self.c_name, self.o_name = hidden, rank, c_name, o_name

        def weight_specs(self):
            return [WeightSpec(self.c_name, (self.rank, self.hidden)), WeightSpec(self.o_name, (self.hidden, self.rank))]

        def load(self, weights, dtype, device):
            self.w_c, self.w_o = weights[self.c_name], weights[self.o_name]

        def kv_request(self):
            return KVRequest(1, self.rank, value_dim=0)

        def forward(self, ctx, call, xn, out, accumulate):
            kv = call.kv
            assert kv.v is None and kv.k.shape[1:] == (1, kv.page_size, self.rank)
            c = linear(xn, self.w_c)
            cu, slots, starts = ctx.cu_q.tolist(), ctx.seq_slot.tolist(), ctx.seq_start.tolist()
            table = kv.page_table.cpu()
            means = torch.empty(c.shape, dtype=torch.float32, device=c.device)
            for b, slot in enumerate(slots):
                for t in range(cu[b], cu[b + 1]):
                    pos = starts[b] + t - cu[b]
                    kv.k[table[slot, pos // kv.page_size], 0, pos % kv.page_size] = c[t]
                    pages = table[slot, :pos // kv.page_size + 1].long().to(c.device)
                    seen = kv.k[pages, 0].reshape(-1, self.rank)[:pos + 1]
                    means[t] = seen.float().mean(0)
            linear(means.to(xn.dtype), self.w_o, out=out, accumulate=accumulate)

    class EmaMixer(Mixer):
        """s_t = decay * s_{t-1} + xn_t (per channel, float32 state per sequence); out += s_t W^T."""

        def __init__(self, hidden, decay, out_name):
            self.hidden, self.decay, self.out_name = hidden, decay, out_name

        def weight_specs(self):
            return [WeightSpec(self.out_name, (self.hidden, self.hidden))]

        def load(self, weights, dtype, device):
            self.w = weights[self.out_name]

        def state_request(self):
            return StateRequest((self.hidden,), torch.float32)

        def forward(self, ctx, call, xn, out, accumulate):
            cu, slots = ctx.cu_q.tolist(), ctx.seq_slot.tolist()
            s_all = torch.empty(xn.shape, dtype=torch.float32, device=xn.device)
            for b, slot in enumerate(slots):
                s = call.state[slot]
                for t in range(cu[b], cu[b + 1]):
                    s = self.decay * s + xn[t].float()
                    s_all[t] = s
                call.state[slot] = s
            linear(s_all.to(xn.dtype), self.w, out=out, accumulate=accumulate)

    @dataclass
    class ToyConfig(Lfm2Config):
        ema_decay: float = 0.5
        run_order: tuple = ()
        share: tuple = ()
        latent_rank: int = 0
        toy_norm: bool = False

        @classmethod
        def from_json_dict(cls, d):
            base = Lfm2Config.from_json_dict(dict(d, layer_types=["conv" if k in ("ema", "latent") else k
                                                                  for k in d["layer_types"]]))
            cfg = cls(**{f: getattr(base, f) for f in base.__dataclass_fields__})
            cfg.layer_types = tuple(d["layer_types"])
            cfg.ema_decay = float(d["ema_decay"])
            cfg.run_order = tuple(d.get("run_order") or range(len(cfg.layer_types)))
            cfg.share = tuple(tuple(p) for p in d.get("share", ()))
            cfg.latent_rank = int(d.get("latent_rank", 0))
            cfg.toy_norm = bool(d.get("toy_norm", False))
            return cfg

        def to_json_dict(self):
            return dict(super().to_json_dict(), ema_decay=self.ema_decay, run_order=list(self.run_order),
                        share=[list(p) for p in self.share], latent_rank=self.latent_rank, toy_norm=self.toy_norm)

    def build(cfg):
        D = cfg.hidden_size
        emb = TokenEmbedding(cfg.vocab_size, D, "model.embed_tokens.weight")
        rope = RotaryEncoding(cfg.head_dim, cfg.rope_theta)
        layers = []
        for i, kind in enumerate(cfg.layer_types):
            p = f"model.layers.{i}."
            if kind == "ema":
                mixer = MIXERS.get("toy_ema")(D, cfg.ema_decay, p + "ema.out.weight")
            elif kind == "latent":
                mixer = MIXERS.get("toy_latent")(D, cfg.latent_rank, p + "latent.c.weight", p + "latent.o.weight")
            else:
                a = p + "self_attn."
                mixer = GqaAttention(D, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                     a + "q_proj.weight", a + "k_proj.weight", a + "v_proj.weight", a + "out_proj.weight",
                                     a + "q_layernorm.weight", a + "k_layernorm.weight", cfg.norm_eps, rope)
            norm = NORMS.get("toy_mean_abs") if cfg.toy_norm else RMSNorm
            layers.append(PreNormBlock(norm(D, cfg.norm_eps, p + "operator_norm.weight"), mixer,
                                       norm(D, cfg.norm_eps, p + "ffn_norm.weight"),
                                       SwiGLU(D, cfg.ffn_dim, p + "feed_forward.w1.weight", p + "feed_forward.w3.weight",
                                              p + "feed_forward.w2.weight")))
        share = dict(cfg.share)
        schedule = [LayerCall(l, share.get(c)) for c, l in enumerate(cfg.run_order)]
        return Model(cfg, emb, layers, RMSNorm(D, cfg.norm_eps, "model.embedding_norm.weight"),
                     LMHead(cfg.vocab_size, D, None, emb), schedule=schedule)

    MIXERS.register("toy_ema", EmaMixer, replace=True)
    MIXERS.register("toy_latent", LatentMixer, replace=True)
    NORMS.register("toy_mean_abs", MeanAbsNorm, replace=True)
    register_architecture("ToyEmaForCausalLM", ToyConfig, build, replace=True)

    def cleanup():
        MIXERS.unregister("toy_ema")
        MIXERS.unregister("toy_latent")
        NORMS.unregister("toy_mean_abs")
        unregister_architecture("ToyEmaForCausalLM")

    return cleanup


TOY = dict(architectures=["ToyEmaForCausalLM"], vocab_size=97, hidden_size=48, num_hidden_layers=3,
           num_attention_heads=3, num_key_value_heads=1, max_position_embeddings=128,
           layer_types=["ema", "full_attention", "ema"], block_ff_dim=64, rope_theta=1000.0, norm_eps=1e-5,
           ema_decay=0.75)


def plain_toy(folder, tokens, run_order=None, share=()):
    """Whole-sequence logits of the toy architecture, from the plain parts."""
    cfg = json.loads((folder / "config.json").read_text())
    w = P.read_safetensors(folder / "model.safetensors")
    D, H, Hkv = cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd, eps, dt = D // H, cfg["norm_eps"], np.float64
    f = P.rope_inv_freq(cfg["rope_theta"], hd)
    x = w["model.embed_tokens.weight"][np.asarray(tokens)].astype(dt)
    order = run_order or range(len(cfg["layer_types"]))
    share = dict(share)
    kv_of_call = {}

    def norm(v, weight):
        if cfg.get("toy_norm"):
            return v / (np.abs(v).mean(-1, keepdims=True) + eps) * weight.astype(dt)
        return P.rms_norm(v, weight, eps, dt)

    for c, i in enumerate(order):
        p = f"model.layers.{i}."
        xn = norm(x, w[p + "operator_norm.weight"])
        if cfg["layer_types"][i] == "latent":
            cvec = xn @ w[p + "latent.c.weight"].astype(dt).T
            means = np.cumsum(cvec, axis=0) / np.arange(1, len(tokens) + 1)[:, None]
            y = means @ w[p + "latent.o.weight"].astype(dt).T
        elif cfg["layer_types"][i] == "ema":
            s = np.zeros(D)
            rows = []
            for t in range(len(tokens)):
                s = cfg["ema_decay"] * s + xn[t]
                rows.append(s)
            y = np.stack(rows) @ w[p + "ema.out.weight"].astype(dt).T
        else:
            a = p + "self_attn."
            T = len(tokens)
            q = (xn @ w[a + "q_proj.weight"].astype(dt).T).reshape(T, H, hd)
            q = P.apply_rope(P.rms_norm(q, w[a + "q_layernorm.weight"], eps, dt), np.arange(T), f, dt)
            if c in share:
                k, v = kv_of_call[share[c]]
            else:
                k = (xn @ w[a + "k_proj.weight"].astype(dt).T).reshape(T, Hkv, hd)
                k = P.apply_rope(P.rms_norm(k, w[a + "k_layernorm.weight"], eps, dt), np.arange(T), f, dt)
                v = (xn @ w[a + "v_proj.weight"].astype(dt).T).reshape(T, Hkv, hd)
                kv_of_call[c] = (k, v)
            att = np.zeros((T, H, hd))
            for h in range(H):
                sc = q[:, h] @ k[:, h // (H // Hkv)].T / np.sqrt(hd)
                sc = np.where(np.tril(np.ones((T, T), bool)), sc, -np.inf)
                pr = np.exp(sc - sc.max(-1, keepdims=True))
                att[:, h] = (pr / pr.sum(-1, keepdims=True)) @ v[:, h // (H // Hkv)]
            y = att.reshape(T, H * hd) @ w[a + "out_proj.weight"].astype(dt).T
        x = x + y
        xn = norm(x, w[p + "ffn_norm.weight"])
        x = x + P.swiglu(xn, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"], w[p + "feed_forward.w2.weight"], dt)
    xn = P.rms_norm(x, w["model.embedding_norm.weight"], eps, dt)
    return xn @ w["model.embed_tokens.weight"].astype(dt).T


def run_cuts(z, folder, seqs, ref, dtype="fp32", tol=helpers.TOL["float32"]):
    model = z.load(folder, dtype=dtype)
    eng = z.Engine(model, max_batch=2, max_seq_len=128, page_size=16)         # graphs asked for (the default)
    assert not eng.use_graphs, "a mixer that is not capture_safe must keep the engine from recording steps"
    for round_ in range(2):                      # twice: the second round reuses slots and state rows
        slots = eng.start(2)
        heads = [5, 1]
        out = eng.step(slots, [s[:h] for s, h in zip(seqs, heads)], want=[list(range(h)) for h in heads]).cpu().numpy()
        rows = [(i, p) for i, h in enumerate(heads) for p in range(h)]
        for r, (i, p) in enumerate(rows):
            assert np.abs(out[r] - ref[i][p]).max() <= tol * np.abs(ref[i]).max(), (round_, i, p)
        fed = list(heads)
        while any(f < len(s) for f, s in zip(fed, seqs)):
            live = [i for i in range(2) if fed[i] < len(seqs[i])]
            out = eng.decode([slots[i] for i in live], [seqs[i][fed[i]] for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                assert np.abs(out[r] - ref[i][fed[i]]).max() <= tol * np.abs(ref[i]).max(), (round_, i, fed[i])
                fed[i] += 1
        eng.finish(slots)
    eng.cache.check_consistency()
    return model, eng


def test_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    import zinfer_b200 as z
    cleanup = make_toy()
    try:
        cfg = z.config_from_dict(TOY)
        folder = z.write_random_model(tmp_path / "toy", cfg, 3, storage_dtype=torch.float32)
        assert "model.layers.0.ema.out.weight" in P.read_safetensors(folder / "model.safetensors")
        seqs = [helpers.random_tokens(1, 40, 97), helpers.random_tokens(2, 23, 97)]
        ref = [plain_toy(folder, s) for s in seqs]
        model, eng = run_cuts(z, folder, seqs, ref)
        assert type(model.layers[0].mixer).__name__ == "EmaMixer"
        assert len(eng.cache.state_tensors) == 1 and eng.cache.state_tensors[0].shape == (2, 2, 48)
        assert len(eng.cache.groups) == 1 and eng.cache.groups[0].n_layers == 1
        run_cuts(z, folder, seqs, ref, dtype="bf16", tol=helpers.TOL["bfloat16"])
    finally:
        cleanup()


def test_schedule_runs_a_layer_twice_and_shares_a_cache(tmp_path):
    """Order [0, 1, 0, 1]: layer 0 (state) and layer 1 (attention) run twice.  The second run of
    layer 0 has a state row of its own; the second run of layer 1 reads the keys and values
    that its first run wrote."""
    import zinfer_b200 as z
    cleanup = make_toy()
    try:
        d = dict(TOY, num_hidden_layers=2, layer_types=["ema", "full_attention"], run_order=[0, 1, 0, 1], share=[[3, 1]])
        folder = z.write_random_model(tmp_path / "toy2", z.config_from_dict(d), 4, storage_dtype=torch.float32)
        seqs = [helpers.random_tokens(5, 37, 97), helpers.random_tokens(6, 18, 97)]
        ref = [plain_toy(folder, s, run_order=[0, 1, 0, 1], share=[(3, 1)]) for s in seqs]
        model, eng = run_cuts(z, folder, seqs, ref)
        assert len(model.schedule) == 4 and eng.cache.state_tensors[0].shape[0] == 2
        assert eng.cache.groups[0].n_layers == 1 and not eng.calls[3].writes_kv and eng.calls[1].writes_kv
        unshared = [plain_toy(folder, s, run_order=[0, 1, 0, 1]) for s in seqs]
        assert np.abs(unshared[0] - ref[0]).max() > 1e-3 * np.abs(ref[0]).max(), "sharing must change the result"
    finally:
        cleanup()


def test_toy_norm_and_a_mixer_with_one_cached_vector_per_token(tmp_path):
    """A norm that knows only the base signature (no pending form: the parts behind it get a
    tensor), and a mixer that asks the cache for ONE tensor of its own width per token."""
    import zinfer_b200 as z
    cleanup = make_toy()
    try:
        d = dict(TOY, layer_types=["latent", "full_attention", "latent"], latent_rank=24, toy_norm=True)
        folder = z.write_random_model(tmp_path / "toy3", z.config_from_dict(d), 6, std=0.1, storage_dtype=torch.float32)
        seqs = [helpers.random_tokens(7, 40, 97), helpers.random_tokens(8, 23, 97)]
        ref = [plain_toy(folder, s) for s in seqs]
        model, eng = run_cuts(z, folder, seqs, ref)
        assert type(model.layers[0].mixer_norm).__name__ == "MeanAbsNorm"
        latent = [g for g in eng.cache.groups if g.v is None]
        assert len(latent) == 1 and latent[0].n_layers == 2 and latent[0].k.shape[-1] == 24
        assert len(eng.cache.groups) == 2 and not eng.cache.state_tensors
        run_cuts(z, folder, seqs, ref, dtype="bf16", tol=helpers.TOL["bfloat16"])
    finally:
        cleanup()
