"""Each part a layer is put together from, alone: built from its constructor parameters, given
random weights by name, run on a hand-made step context and cache, and compared with the plain
function of the same part.  Sizes differ from the tiny models': widths that are no multiple of
16 next to widths that are, group sizes 1, 2 and 3, a window, a rotation narrower than the
head, a scaled rotation table, two to five convolution taps.  The mixers run a prompt step of
unequal sequences and then single tokens, so that the cache and the state they leave are part
of what is compared."""
import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.5e-2


def close(got, ref, dtype, what=""):
    got = np.asarray(got.detach().double().cpu())
    ref = np.asarray(ref, dtype=np.float64)
    scale = np.abs(ref).max()
    assert scale > 0, f"{what}: empty reference"
    err = np.abs(got - ref).max() / scale
    assert err <= tol(dtype), f"{what}: error {err:.3e} of max |ref| {scale:.3e}"


def rnd(shape, seed, dtype, scale=1.0):
    """Random values that the run dtype holds exactly, as a float32 host tensor."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).float()


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


def load(part, tensors, dtype):
    """Hands a part its tensors the way the loader does: matrices in the run dtype, vectors in
    float32, on the device, by the names the part asks for."""
    given = {}
    for spec in part.weight_specs():
        if spec.name not in tensors:
            assert spec.optional, f"the test forgot {spec.name}"
            continue
        t = tensors[spec.name]
        assert tuple(t.shape) in ((spec.shape,) + tuple(spec.alt_shapes)), spec.name
        given[spec.name] = t.to(dtype if spec.role == "matrix" else torch.float32).cuda().contiguous()
    part.load(given, dtype, torch.device("cuda"))
    for sub in part.parts():
        load(sub, tensors, dtype)
    return part


class Bench:
    """A cache for ONE schedule entry and the step contexts to drive a mixer through it."""

    def __init__(self, k, mixer, dtype, n_slots=3, max_seq=256, page=16):
        from zinfer_b200.cache import CacheManager, CallCacheSpec
        from zinfer_b200.engine.context import CallContext
        self.dtype, self.dev = dtype, torch.device("cuda")
        self.cache = CacheManager([CallCacheSpec(kv=mixer.kv_request(), state=mixer.state_request())], n_slots,
                                  n_slots * max_seq, max_seq, page, dtype, self.dev)
        self.status = k.status_word(self.dev)
        self.call = CallContext(0, 0, self.cache.kv_view(0), self.cache.writes_kv(0), self.cache.state_view(0))

    def step(self, slots, rows_per_seq):
        from zinfer_b200.engine.context import StepContext, pack_batch
        lens = [int(n) for n in rows_per_seq]
        starts = [int(self.cache.lengths[s]) for s in slots]
        self.cache.reserve(slots, lens)
        self.cache.sync()
        buf = torch.from_numpy(pack_batch(slots, starts, [[0] * n for n in lens])).to(self.dev)
        ctx = StepContext(self.dtype, self.dev, self.status, buf, sum(lens), len(slots), lens,
                          max(s + n for s, n in zip(starts, lens)))
        return ctx

    def done(self, slots, rows_per_seq):
        self.cache.advance(slots, rows_per_seq)
        assert int(self.status.item()) == 0


def run_mixer(k, mixer, dtype, xs, prompt_lens, page=16):
    """Runs `mixer` over the sequences `xs` (float32 [T_b, D] each): the first prompt_lens[b] rows
    in one packed step, the rest one row per sequence and step; shorter sequences leave the batch
    earlier.  Slots are taken in reverse so that slot and batch index differ.  Returns out[b]
    [T_b, D] (float32, the mixer's own output without a residual)."""
    bench = Bench(k, mixer, dtype, n_slots=len(xs) + 1, page=page)
    held = bench.cache.alloc_slots(len(xs) + 1)
    slots = held[1:][::-1]
    D = xs[0].shape[1]
    outs = [torch.zeros(x.shape[0], D) for x in xs]
    ctx = bench.step(slots, prompt_lens)
    xn = torch.cat([x[:n] for x, n in zip(xs, prompt_lens)]).to(dtype).cuda()
    out = torch.full((xn.shape[0], D), 7.0, device="cuda")
    mixer.forward(ctx, bench.call, xn, out, False)            # overwrite: the 7s must be gone
    bench.done(slots, prompt_lens)
    o = 0
    for b, n in enumerate(prompt_lens):
        outs[b][:n] = out[o:o + n].cpu()
        o += n
    t = list(prompt_lens)
    while True:
        live = [b for b, x in enumerate(xs) if t[b] < x.shape[0]]
        if not live:
            break
        ctx = bench.step([slots[b] for b in live], [1] * len(live))
        xn = torch.stack([xs[b][t[b]] for b in live]).to(dtype).cuda()
        base = torch.full((len(live), D), 0.5, device="cuda")
        out = base.clone()
        mixer.forward(ctx, bench.call, xn, out, True)         # accumulate: the 0.5 stays under it
        bench.done([slots[b] for b in live], [1] * len(live))
        for i, b in enumerate(live):
            outs[b][t[b]] = (out[i] - base[i]).cpu()
            t[b] += 1
    bench.cache.free_slots(held)
    bench.cache.check_consistency()
    return outs


# ------------------------------------------------------------------------------- norm, rotation, tables

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,eps", [(72, 1e-5), (1000, 3e-6), (2048, 1e-6)])
def test_rmsnorm_part(k, dtype, dim, eps):
    from zinfer_b200.parts import RMSNorm
    from zinfer_b200.parts.linear import NormedRows
    norm = load(RMSNorm(dim, eps, "n.weight"), {"n.weight": 1.0 + rnd((dim,), 1, dtype, 0.3)}, dtype)
    x = rnd((9, dim), 2, torch.float32, 3.0)
    ref = P.rms_norm(x.numpy().astype(np.float64), norm.weight.cpu().numpy(), eps, np.float64)
    bench = Bench(k, norm_free_mixer(), dtype)
    ctx = bench.step(bench.cache.alloc_slots(1), [9])
    got = norm.forward(ctx, x.cuda())
    assert got.dtype == dtype
    close(got, ref, dtype, "all rows")
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    close(norm.forward(ctx, x.cuda(), rows), ref[[7, 0, 3]], dtype, "chosen rows")
    lazy = norm.pending(ctx, x.cuda())
    assert isinstance(lazy, NormedRows) and torch.equal(lazy.tensor(), got)


def norm_free_mixer():
    """A mixer that asks for nothing, to give `Bench` a schedule entry."""
    from zinfer_b200.parts import Mixer
    return Mixer()


@pytest.mark.parametrize("hd,n_rot,theta,scale", [(48, 48, 10000.0, 1.0), (64, 32, 1e6, 0.25), (16, 16, 500.0, 1.0)])
def test_rotary_part_gives_the_plain_table(hd, n_rot, theta, scale):
    from zinfer_b200.parts import RotaryEncoding
    rope = RotaryEncoding(hd, theta, n_rot=n_rot, scale=scale)
    rope.load({}, torch.float32, torch.device("cuda"))
    params = rope.rotary()
    ref = (P.rope_inv_freq(theta, n_rot).astype(np.float64) * scale).astype(np.float32)
    assert params.n_rot == n_rot and not params.interleaved
    assert np.array_equal(params.inv_freq.cpu().numpy(), ref)
    with pytest.raises(ValueError):
        RotaryEncoding(hd, theta, n_rot=hd + 2)
    with pytest.raises(ValueError):
        RotaryEncoding(hd, theta, n_rot=7)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,dim,tied", [(331, 72, True), (1000, 200, False)])
def test_embedding_and_head_parts(k, dtype, vocab, dim, tied):
    from zinfer_b200.parts import LMHead, TokenEmbedding
    tensors = {"emb": rnd((vocab, dim), 3, dtype, 0.5), "head": rnd((vocab, dim), 4, dtype, 0.5)}
    emb = load(TokenEmbedding(vocab, dim, "emb", scale=1.5), tensors, dtype)
    head = load(LMHead(vocab, dim, None if tied else "head", emb), tensors, dtype)
    assert [s.name for s in head.weight_specs()] == ([] if tied else ["head"])
    bench = Bench(k, norm_free_mixer(), dtype)
    ctx = bench.step(bench.cache.alloc_slots(1), [6])
    tokens = torch.tensor([0, vocab - 1, 5, 5, 17, vocab // 2], dtype=torch.int32, device="cuda")
    x = emb.forward(ctx, tokens)
    assert x.dtype == torch.float32
    assert torch.equal(x.cpu(), tensors["emb"][tokens.cpu().long()] * 1.5)
    xn = rnd((6, dim), 5, dtype)
    logits = head.forward(ctx, xn.to(dtype).cuda())
    assert logits.dtype == torch.float32 and logits.shape == (6, vocab)
    close(logits, xn.double().numpy() @ tensors["emb" if tied else "head"].double().numpy().T, dtype, "logits")
    with pytest.raises(ValueError):
        LMHead(vocab, dim, None, None)


# ------------------------------------------------------------------------------- feed-forward

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,F", [(72, 200), (96, 208), (256, 1024)])
@pytest.mark.parametrize("rows", [1, 5, 20, 70])
def test_swiglu_part(k, dtype, D, F, rows):
    """1 and 5 rows take the few-row kernels, 20 the tensor-core kernel for few rows and 70 the
    prompt kernels; F = 200 is no multiple of 16 and keeps the unfused activation."""
    from zinfer_b200.parts import RMSNorm, SwiGLU
    tensors = {"w1": rnd((F, D), 6, dtype, 0.2), "w3": rnd((F, D), 7, dtype, 0.2), "w2": rnd((D, F), 8, dtype, 0.2),
               "n": 1.0 + rnd((D,), 9, dtype, 0.2)}
    ffn = load(SwiGLU(D, F, "w1", "w3", "w2"), tensors, dtype)
    bench = Bench(k, norm_free_mixer(), dtype)
    ctx = bench.step(bench.cache.alloc_slots(1), [rows])
    xn = rnd((rows, D), 10, dtype)
    ref = P.swiglu(xn.numpy(), tensors["w1"].numpy(), tensors["w3"].numpy(), tensors["w2"].numpy(), np.float64)
    out = torch.full((rows, D), 3.0, device="cuda")
    ffn.forward(ctx, xn.to(dtype).cuda(), out, False)
    close(out, ref, dtype, "overwrite")
    ffn.forward(ctx, xn.to(dtype).cuda(), out, True)
    close(out, 2 * ref, dtype, "accumulate")
    # the norm still pending, as a block hands it over
    x = rnd((rows, D), 11, torch.float32, 2.0)
    norm = load(RMSNorm(D, 1e-5, "n"), tensors, dtype)
    eager = norm.forward(ctx, x.cuda())
    ref = P.swiglu(eager.float().cpu().numpy(), tensors["w1"].numpy(), tensors["w3"].numpy(), tensors["w2"].numpy(),
                   np.float64)
    out = torch.zeros((rows, D), device="cuda")
    ffn.forward(ctx, norm.pending(ctx, x.cuda()), out, False)
    close(out, ref, dtype, "pending norm")


# ------------------------------------------------------------------------------- mixers

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,K,bias,proj_bias", [(72, 2, False, False), (96, 5, True, False), (208, 3, True, True)])
def test_short_conv_part(k, dtype, D, K, bias, proj_bias):
    """Three sequences of unequal length: a prompt step (one prompt shorter than the taps), then
    single tokens from the state the prompt left; compared with the convolution of each whole
    sequence."""
    from zinfer_b200.parts import ShortConv
    tensors = {"in": rnd((3 * D, D), 12, dtype, 0.3), "conv": rnd((D, 1, K), 13, dtype, 0.5),
               "out": rnd((D, D), 14, dtype, 0.3)}
    if bias:
        tensors["cb"] = rnd((D,), 15, dtype, 0.3)
    if proj_bias:
        tensors["ib"], tensors["ob"] = rnd((3 * D,), 16, dtype, 0.3), rnd((D,), 17, dtype, 0.3)
    mixer = load(ShortConv(D, K, "in", "conv", "out", "cb" if bias else None, "ib" if proj_bias else None,
                           "ob" if proj_bias else None), tensors, dtype)
    assert mixer.kv_request() is None and mixer.state_request().shape == (K - 1, D)
    xs = [rnd((n, D), 20 + n, dtype) for n in (23, 9, 14)]
    outs = run_mixer(k, mixer, dtype, xs, [11, 1, 14 - 6])
    f = lambda name: tensors[name].numpy() if name in tensors else None
    for b, x in enumerate(xs):
        ref = P.short_conv(x.numpy(), f("in"), f("conv").reshape(D, K), f("out"), f("cb"), f("ib"), f("ob"), np.float64)
        close(outs[b], ref, dtype, f"sequence {b}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,H,Hkv,hd,n_rot,window,qk_norm,page", [
    (72, 3, 1, 48, 48, 0, True, 16),        # three heads on one KV head
    (96, 4, 2, 32, 16, 0, False, 32),       # half of the head rotated, no q/k norm
    (80, 5, 5, 16, 16, 12, True, 16),       # a window shorter than the prompt
    (128, 4, 2, 64, 64, 0, True, 64),       # the shape the tensor-core kernels take
    (64, 2, 2, 64, 0, 20, True, 64),        # no position encoding at all
])
def test_gqa_attention_part(k, dtype, D, H, Hkv, hd, n_rot, window, qk_norm, page):
    from zinfer_b200.parts import GqaAttention, RotaryEncoding
    theta, eps = 5000.0, 2e-6
    tensors = {"q": rnd((H * hd, D), 30, dtype, 0.3), "k": rnd((Hkv * hd, D), 31, dtype, 0.3),
               "v": rnd((Hkv * hd, D), 32, dtype, 0.3), "o": rnd((D, H * hd), 33, dtype, 0.3),
               "qn": 1.0 + rnd((hd,), 34, dtype, 0.3), "kn": 1.0 + rnd((hd,), 35, dtype, 0.3)}
    rope = RotaryEncoding(hd, theta, n_rot=n_rot) if n_rot else None
    mixer = load(GqaAttention(D, H, Hkv, hd, "q", "k", "v", "o", "qn" if qk_norm else None, "kn" if qk_norm else None,
                              eps, rope, window), tensors, dtype)
    req = mixer.kv_request()
    assert (req.n_kv_heads, req.head_dim, req.window) == (Hkv, hd, window) and mixer.state_request() is None
    xs = [rnd((n, D), 40 + n, dtype) for n in (70, 37, 45)]
    outs = run_mixer(k, mixer, dtype, xs, [70 - 5, 37 - 20, 1], page=page)
    f = lambda name: tensors[name].numpy()
    inv = P.rope_inv_freq(theta, n_rot) if n_rot else None
    for b, x in enumerate(xs):
        ref = plain_attention(x.numpy(), f, H, Hkv, hd, eps, inv, n_rot, window, qk_norm)
        close(outs[b], ref, dtype, f"sequence {b}")


def plain_attention(x, f, H, Hkv, hd, eps, inv, n_rot, window, qk_norm):
    """`P.gqa_attention` rotates the first 2 * len(inv) elements of a head, which is the partial
    rotation when `inv` has n_rot / 2 entries."""
    return P.gqa_attention(x, f("q"), f("k"), f("v"), f("o"), f("qn") if qk_norm else None, f("kn") if qk_norm else None,
                           H, Hkv, hd, eps, inv, window, np.float64)


# ------------------------------------------------------------------------------- block

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mixer_kind", ["attention", "conv"])
def test_prenorm_block_part(k, dtype, mixer_kind):
    """x += mixer(norm(x)); x += ffn(norm(x)) on the float32 stream, for a prompt step and for
    single tokens, with either mixer in the block."""
    from zinfer_b200.parts import GqaAttention, PreNormBlock, RMSNorm, RotaryEncoding, ShortConv, SwiGLU
    D, F, H, Hkv, hd, K, eps = 96, 176, 3, 1, 32, 3, 1e-5
    tensors = {"q": rnd((H * hd, D), 50, dtype, 0.2), "k": rnd((Hkv * hd, D), 51, dtype, 0.2),
               "v": rnd((Hkv * hd, D), 52, dtype, 0.2), "o": rnd((D, H * hd), 53, dtype, 0.2),
               "qn": 1.0 + rnd((hd,), 54, dtype, 0.2), "kn": 1.0 + rnd((hd,), 55, dtype, 0.2),
               "in": rnd((3 * D, D), 56, dtype, 0.2), "conv": rnd((D, K), 57, dtype, 0.5), "out": rnd((D, D), 58, dtype, 0.2),
               "w1": rnd((F, D), 59, dtype, 0.2), "w3": rnd((F, D), 60, dtype, 0.2), "w2": rnd((D, F), 61, dtype, 0.2),
               "n1": 1.0 + rnd((D,), 62, dtype, 0.2), "n2": 1.0 + rnd((D,), 63, dtype, 0.2)}
    if mixer_kind == "attention":
        mixer = GqaAttention(D, H, Hkv, hd, "q", "k", "v", "o", "qn", "kn", eps, RotaryEncoding(hd, 1e4))
    else:
        mixer = ShortConv(D, K, "in", "conv", "out")
    block = load(PreNormBlock(RMSNorm(D, eps, "n1"), mixer, RMSNorm(D, eps, "n2"), SwiGLU(D, F, "w1", "w3", "w2")),
                 tensors, dtype)
    f = lambda name: tensors[name].numpy()
    T, prompt = 26, 19
    x = rnd((T, D), 64, torch.float32)
    h = x.numpy().astype(np.float64)
    xn = P.rms_norm(h, f("n1"), eps, np.float64)
    if mixer_kind == "attention":
        h = h + P.gqa_attention(xn, f("q"), f("k"), f("v"), f("o"), f("qn"), f("kn"), H, Hkv, hd, eps,
                                P.rope_inv_freq(1e4, hd), 0, np.float64)
    else:
        h = h + P.short_conv(xn, f("in"), f("conv"), f("out"), dtype=np.float64)
    ref = h + P.swiglu(P.rms_norm(h, f("n2"), eps, np.float64), f("w1"), f("w3"), f("w2"), np.float64)

    bench = Bench(k, mixer, dtype)
    slot = bench.cache.alloc_slots(2)[1:]
    got = torch.zeros(T, D)
    ctx = bench.step(slot, [prompt])
    stream = x[:prompt].cuda().clone()
    block.forward(ctx, bench.call, stream)
    bench.done(slot, [prompt])
    got[:prompt] = stream.cpu()
    for t in range(prompt, T):
        ctx = bench.step(slot, [1])
        stream = x[t:t + 1].cuda().clone()
        block.forward(ctx, bench.call, stream)
        bench.done(slot, [1])
        got[t] = stream[0].cpu()
    close(got, ref, dtype, "stream after the block")


# ------------------------------------------------------------------------------- parts of the test's own

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hkv,hd,page", [(3, 1, 48, 16), (4, 2, 64, 64)])
def test_attention_takes_a_position_encoding_of_another_kind(k, dtype, H, Hkv, hd, page):
    """A position encoding defined here that is no rotation table: learned vectors per absolute
    position, added to the normalised q and k.  The attention part runs it between its norm and
    its cache write, in prompt steps and in single-token steps."""
    from zinfer_b200.parts import POSITION_ENCODINGS, GqaAttention, PositionEncoding, WeightSpec

    class LearnedPositions(PositionEncoding):
        def __init__(self, head_dim, n_pos, q_name, k_name):
            self.head_dim, self.n_pos, self.q_name, self.k_name = head_dim, n_pos, q_name, k_name

        def weight_specs(self):
            return [WeightSpec(self.q_name, (self.n_pos, self.head_dim)), WeightSpec(self.k_name, (self.n_pos, self.head_dim))]

        def load(self, weights, dtype, device):
            self.tq, self.tk = weights[self.q_name], weights[self.k_name]

        def apply(self, ctx, q, k):
            pos = ctx.tok_pos.long()
            q.unflatten(1, (-1, self.head_dim)).add_(self.tq[pos][:, None, :])
            k.unflatten(1, (-1, self.head_dim)).add_(self.tk[pos][:, None, :])

    POSITION_ENCODINGS.register("toy_learned", LearnedPositions, replace=True)
    try:
        D, eps = 80, 1e-5
        tensors = {"q": rnd((H * hd, D), 70, dtype, 0.3), "k": rnd((Hkv * hd, D), 71, dtype, 0.3),
                   "v": rnd((Hkv * hd, D), 72, dtype, 0.3), "o": rnd((D, H * hd), 73, dtype, 0.3),
                   "qn": 1.0 + rnd((hd,), 74, dtype, 0.3), "kn": 1.0 + rnd((hd,), 75, dtype, 0.3),
                   "pq": rnd((96, hd), 76, dtype, 0.7), "pk": rnd((96, hd), 77, dtype, 0.7)}
        enc = POSITION_ENCODINGS.get("toy_learned")(hd, 96, "pq", "pk")
        assert enc.rotary() is None
        mixer = load(GqaAttention(D, H, Hkv, hd, "q", "k", "v", "o", "qn", "kn", eps, enc), tensors, dtype)
        xs = [rnd((n, D), 80 + n, dtype) for n in (70, 33)]
        outs = run_mixer(k, mixer, dtype, xs, [52, 33 - 4], page=page)
        f = lambda name: tensors[name].numpy().astype(np.float64)
        encode = lambda q, kk, pos: (q + f("pq")[pos][:, None, :], kk + f("pk")[pos][:, None, :])
        for b, x in enumerate(xs):
            ref = P.gqa_attention(x.numpy(), f("q"), f("k"), f("v"), f("o"), f("qn"), f("kn"), H, Hkv, hd, eps, None, 0,
                                  np.float64, encode=encode)
            close(outs[b], ref, dtype, f"sequence {b}")
        bare = P.gqa_attention(xs[1].numpy(), f("q"), f("k"), f("v"), f("o"), f("qn"), f("kn"), H, Hkv, hd, eps, None, 0,
                               np.float64)
        assert np.abs(bare - ref).max() > 1e-2 * np.abs(ref).max(), "the encoding must change the result"
    finally:
        POSITION_ENCODINGS.unregister("toy_learned")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 7, 40])
def test_feed_forward_with_routing_of_the_tests_own(k, dtype, rows):
    """A feed-forward defined here that routes: router logits in float32, the best two of four
    experts per row, their softmax as weights; the experts are the library's SwiGLU parts, nested
    so that their weights are found through `parts()`.  Registered, built by name, run alone and
    inside a block."""
    from zinfer_b200.parts import FEED_FORWARDS, FeedForward, PreNormBlock, RMSNorm, ShortConv, SwiGLU, WeightSpec

    class TopTwo(FeedForward):
        def __init__(self, hidden, ffn_dim, n_experts, prefix):
            self.hidden, self.n_experts, self.router_name = hidden, n_experts, prefix + "router"
            self.experts = [SwiGLU(hidden, ffn_dim, f"{prefix}{e}.w1", f"{prefix}{e}.w3", f"{prefix}{e}.w2")
                            for e in range(n_experts)]

        def parts(self):
            return list(self.experts)

        def weight_specs(self):
            return [WeightSpec(self.router_name, (self.n_experts, self.hidden))]

        def load(self, weights, dtype, device):
            self.router = weights[self.router_name]

        def forward(self, ctx, xn, out, accumulate):
            logits = xn.float() @ self.router.float().t()
            top, idx = logits.topk(2, dim=-1)
            gate = torch.softmax(top, dim=-1)
            total = torch.zeros_like(out)
            for e, expert in enumerate(self.experts):
                hit = (idx == e)
                rows_e = hit.any(-1).nonzero().flatten()
                if rows_e.numel() == 0:
                    continue
                y = torch.empty((rows_e.numel(), self.hidden), dtype=torch.float32, device=out.device)
                expert.forward(ctx, xn[rows_e].contiguous(), y, False)
                total[rows_e] += y * (gate * hit)[rows_e].sum(-1, keepdim=True)
            if accumulate:
                out += total
            else:
                out.copy_(total)

    FEED_FORWARDS.register("toy_top_two", TopTwo, replace=True)
    try:
        D, F, E = 96, 112, 4
        tensors = {"f.router": rnd((E, D), 90, dtype, 1.0), "n1": 1.0 + rnd((D,), 91, dtype, 0.2),
                   "n2": 1.0 + rnd((D,), 92, dtype, 0.2), "in": rnd((3 * D, D), 93, dtype, 0.2),
                   "conv": rnd((D, 3), 94, dtype, 0.5), "out": rnd((D, D), 95, dtype, 0.2)}
        for e in range(E):
            tensors.update({f"f.{e}.w1": rnd((F, D), 100 + e, dtype, 0.2), f"f.{e}.w3": rnd((F, D), 110 + e, dtype, 0.2),
                            f"f.{e}.w2": rnd((D, F), 120 + e, dtype, 0.2)})
        ffn = load(FEED_FORWARDS.get("toy_top_two")(D, F, E, "f."), tensors, dtype)
        f = lambda name: tensors[name].numpy().astype(np.float64)

        def plain(xn):
            logits = xn @ f("f.router").T
            out = np.zeros_like(xn)
            used = set()
            for t in range(xn.shape[0]):
                best = np.argsort(-logits[t])[:2]
                assert logits[t][best[1]] - np.sort(logits[t])[-3] > 1e-3, "routing too close to call"
                g = np.exp(logits[t][best] - logits[t][best[0]])
                g /= g.sum()
                for w, e in zip(g, best):
                    out[t] += w * P.swiglu(xn[t:t + 1], f(f"f.{e}.w1"), f(f"f.{e}.w3"), f(f"f.{e}.w2"), np.float64)[0]
                    used.add(int(e))
            return out, used

        bench = Bench(k, norm_free_mixer(), dtype)
        ctx = bench.step(bench.cache.alloc_slots(1), [rows])
        xn = rnd((rows, D), 130, dtype)
        ref, used = plain(xn.numpy().astype(np.float64))
        assert rows < 7 or len(used) == E
        out = torch.full((rows, D), 2.0, device="cuda")
        ffn.forward(ctx, xn.to(dtype).cuda(), out, False)
        close(out, ref, dtype, "alone")

        # inside a block, after a mixer: the routing then sees the block's own normalised rows, so the
        # reference takes them from the norm part and only the feed-forward is compared
        mixer = ShortConv(D, 3, "in", "conv", "out")
        block = load(PreNormBlock(RMSNorm(D, 1e-5, "n1"), mixer, RMSNorm(D, 1e-5, "n2"), ffn), tensors, dtype)
        bench = Bench(k, mixer, dtype)
        slot = bench.cache.alloc_slots(1)
        ctx = bench.step(slot, [rows])
        x = rnd((rows, D), 131, torch.float32).cuda()
        after_mixer = x.clone()
        block.mixer.forward(ctx, bench.call, block.mixer_norm.pending(ctx, after_mixer), after_mixer, True)
        xn2 = block.ffn_norm.forward(ctx, after_mixer).float().cpu().numpy().astype(np.float64)
        ref2, _ = plain(xn2)
        bench.call.state.zero_()                  # the same step again through the block, from an empty state
        block.forward(ctx, bench.call, x)
        close(x - after_mixer, ref2, dtype, "in a block")
    finally:
        FEED_FORWARDS.unregister("toy_top_two")
