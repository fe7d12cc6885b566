"""The single-token step as one kernel launch: each operation of its program alone against a
plain reference at other sizes than the tiny models', then whole steps through the engine
against the plain implementation and against the engine's separate kernels."""
import math

import numpy as np
import pytest
import torch

import helpers
from plain_lfm2 import PlainLfm2
from test_kernels_gpu import PagedSetup, attn_ref, close, rnd, rope_ref

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


def run_program(k, ops, M, tokens=None, seq_start=None, seq_slot=None):
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    raw = b"".join(bytes(o) for o in ops)
    dev = torch.frombuffer(bytearray(raw), dtype=torch.uint8).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    barrier = torch.zeros(1, dtype=torch.int32).cuda()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    k.fused_decode(dev, len(ops), M, i32(tokens or [0] * M), i32(seq_start or [0] * M),
                   i32(seq_slot or list(range(M))), barrier, status, sms)
    torch.cuda.synchronize()
    return status.item()


def gemm_op(k, xin, epi, rg, x, w, out, n_out, norm_w=None, eps=0.0, bias=None):
    op = k.FusedOp()
    op.kind, op.xin, op.epi, op.rg = k.FUSED_OP_GEMM, xin, epi, rg
    op.N, op.K, op.ldw, op.ldx, op.ldc = n_out, w.shape[1], w.stride(0), x.stride(0), out.stride(0)
    op.W, op.X, op.C = w.data_ptr(), x.data_ptr(), out.data_ptr()
    if norm_w is not None:
        op.norm_w, op.eps = norm_w.data_ptr(), eps
    if bias is not None:
        op.bias = bias.data_ptr()
    return op


def test_operation_record_layout(k):
    assert k.fused_decode_limits()["max_rows"] == 16


@pytest.mark.parametrize("M,N,K,rg,epi,bias", [(1, 40, 96, 1, "f32", False), (5, 331, 160, 2, "f32", True),
                                               (8, 2048, 2048, 1, "acc", False), (13, 100, 6656, 2, "bf16", True),
                                               (16, 48, 32, 1, "acc", True), (9, 1000, 2048, 2, "f32", False)])
def test_plain_contraction(k, M, N, K, rg, epi, bias):
    """Rows and columns that fill no tile, a K with fewer slabs than warps, a K staged in pieces
    (6656 at 13 rows), each way of storing."""
    x = rnd((M, K), 1, BF).cuda()
    w = rnd((N, K), 2, BF, 0.1).cuda()
    b = rnd((N,), 3, torch.float32).cuda() if bias else None
    ref = x.double() @ w.double().T + (b.double() if bias else 0)
    if epi == "bf16":
        out = torch.zeros((M, N), dtype=BF).cuda()
        code = k.FUSED_EPI_BF16
    else:
        out = rnd((M, N), 4, torch.float32).cuda()
        if epi == "acc":
            ref = ref + out.double()
        code = k.FUSED_EPI_ACC_F32 if epi == "acc" else k.FUSED_EPI_F32
    assert run_program(k, [gemm_op(k, k.FUSED_XIN_BF16, code, rg, x, w, out, N, bias=b)], M) == 0
    close(out, ref, BF, f"fused contraction {M}x{N}x{K}")


@pytest.mark.parametrize("M,F,K", [(3, 48, 96), (8, 1024, 2048), (12, 208, 2016), (7, 64, 4096)])
def test_norm_prologue_and_swiglu_epilogue(k, M, F, K):
    from zinfer_b200.parts.linear import interleave_rows
    x = rnd((M, K), 1, torch.float32, 3.0).cuda()
    nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
    g, u = rnd((F, K), 3, BF, 0.05).cuda(), rnd((F, K), 4, BF, 0.05).cuda()
    w = interleave_rows([g, u])
    eps = 1e-6
    xn = (x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * nw.double()).bfloat16().double()
    gate, up = xn @ g.double().T, xn @ u.double().T
    out = torch.zeros((M, F), dtype=BF).cuda()
    op = gemm_op(k, k.FUSED_XIN_NORM, k.FUSED_EPI_SWIGLU, 2, x, w, out, F, nw, eps)
    assert run_program(k, [op], M) == 0
    close(out, gate / (1 + torch.exp(-gate)) * up, BF, "norm + gate/up + activation")


@pytest.mark.parametrize("M,D,taps,bias", [(1, 96, 2, False), (8, 2048, 3, False), (13, 160, 4, True), (16, 64, 7, True)])
def test_convolution_epilogue_equals_the_separate_kernels(k, M, D, taps, bias):
    """Three steps of in_proj + gated convolution with state, against gemm_skinny + conv_decode."""
    w_in = rnd((3 * D, D), 3, BF, 0.2).cuda()
    tw = rnd((taps, D), 4, torch.float32).cuda()
    in_b = rnd((3 * D,), 5, torch.float32).cuda() if bias else None
    cb = rnd((D,), 6, torch.float32).cuda() if bias else None
    nw = (1 + rnd((D,), 2, torch.float32, 0.1)).cuda()
    slots = torch.randperm(M + 3, generator=torch.Generator().manual_seed(1))[:M].to(torch.int32).cuda()
    st_a = rnd((M + 3, taps - 1, D), 7, torch.float32).cuda()
    st_b = st_a.clone()
    y = torch.zeros((M, D), dtype=BF).cuda()
    for step in range(3):
        x = rnd((M, D), 10 + step, torch.float32, 2.0).cuda()
        op = gemm_op(k, k.FUSED_XIN_NORM, k.FUSED_EPI_CONV, 3, x, w_in, y, D, nw, 1e-5, in_b)
        op.conv_state, op.state_stride, op.conv_taps, op.taps = st_a.data_ptr(), st_a.stride(0), tw.data_ptr(), taps
        if cb is not None:
            op.conv_bias = cb.data_ptr()
        assert run_program(k, [op], M, seq_slot=slots.cpu().tolist()) == 0
        bcx = k.gemm_skinny(k.rmsnorm(x, nw, 1e-5, BF), w_in, bias=in_b)
        y_ref = k.conv_decode(bcx, st_b, tw, cb, slots, interleave=16)
        close(y, y_ref.double(), BF, f"fused conv step {step}")
        close(st_a, st_b.double(), BF, f"fused conv state {step}")
    untouched = [i for i in range(M + 3) if i not in slots.cpu().tolist()]
    assert torch.equal(st_a[untouched], rnd((M + 3, taps - 1, D), 7, torch.float32).cuda()[untouched])


def attn_op(k, qkv, out, setup, H, Hkv, hd, window, scale, qw=None, kw=None, inv_freq=None, n_rot=0, eps=1e-5):
    op = k.FusedOp()
    op.kind = k.FUSED_OP_ATTN
    op.H, op.Hkv, op.hd, op.page_size, op.window = H, Hkv, hd, setup.page_size, window
    op.pt_stride, op.eps, op.scale = setup.table_dev.stride(0), eps, scale
    op.X, op.C = qkv.data_ptr(), out.data_ptr()
    op.k_cache, op.v_cache, op.page_table = setup.k.data_ptr(), setup.v.data_ptr(), setup.table_dev.data_ptr()
    if qw is not None:
        op.q_norm, op.k_norm = qw.data_ptr(), kw.data_ptr()
    if inv_freq is not None:
        op.inv_freq, op.n_rot = inv_freq.data_ptr(), n_rot
    return op


@pytest.mark.parametrize("H,Hkv,page", [(4, 4, 32), (6, 3, 64), (8, 2, 32), (32, 8, 64)])
def test_attention_operation_with_norm_rotation_and_cache_write(k, H, Hkv, page):
    """Sequences of unequal lengths in NaN-filled shuffled pages; the step's own key and value are
    written at each sequence's position and used."""
    hd, eps = 64, 1e-5
    lens = [0, 1, 37, 70, 5, 511, 64, 31, 32]
    slots = [3, 0, 5, 1, 4, 9, 7, 2, 8]
    M = len(lens)
    scale = 1 / math.sqrt(hd)
    setup = PagedSetup([l + 1 for l in lens], slots, 10, page, Hkv, hd, BF)
    qw = (1 + rnd((hd,), 1, torch.float32, 0.1)).cuda()
    kw = (1 + rnd((hd,), 2, torch.float32, 0.1)).cuda()
    inv_freq = torch.from_numpy(np.power(10000.0, -2.0 * np.arange(hd // 2) / hd).astype(np.float32)).cuda()
    width = (H + 2 * Hkv) * hd
    seqs = [rnd((l + 1, width), 50 + i, BF) for i, l in enumerate(lens)]
    status = torch.zeros(1, dtype=torch.int32).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    # earlier positions reach the cache through the separate kernel
    if sum(lens):
        rows = torch.cat([s[:-1] for s in seqs]).cuda()
        tok_seq = i32(np.repeat(np.arange(M), lens).tolist())
        tok_pos = i32(np.concatenate([np.arange(l) for l in lens]).tolist())
        k.qk_prepare(rows, setup.k, setup.v, qw, kw, inv_freq, tok_seq, tok_pos, i32(slots), setup.table_dev, H, Hkv,
                     hd, hd, False, eps, status)
    last = torch.stack([s[-1] for s in seqs]).cuda()
    out = torch.zeros((M, H * hd), dtype=BF).cuda()
    op = attn_op(k, last, out, setup, H, Hkv, hd, 0, scale, qw, kw, inv_freq, hd, eps)
    assert run_program(k, [op], M, seq_start=lens, seq_slot=slots) == 0
    ref = []
    nrm = lambda t, w: t / torch.sqrt((t ** 2).mean(-1, keepdim=True) + eps) * w.double().cpu()
    for i, l in enumerate(lens):
        x = seqs[i].double()
        q = x[:, :H * hd].reshape(l + 1, H, hd)
        kk = x[:, H * hd:(H + Hkv) * hd].reshape(l + 1, Hkv, hd)
        v = x[:, (H + Hkv) * hd:].reshape(l + 1, Hkv, hd)
        pos = torch.arange(l + 1)
        q = rope_ref(nrm(q, qw), pos, inv_freq.cpu()).bfloat16().double()
        kk = rope_ref(nrm(kk, kw), pos, inv_freq.cpu()).bfloat16().double()
        ref.append(attn_ref(q[-1:], kk, v, l, 0, scale).reshape(1, H * hd))
        pg = setup.table[slots[i], l // page]
        close(setup.k[pg, :, l % page], kk[-1], BF, f"key written for sequence {i}")
        close(setup.v[pg, :, l % page], v[-1], BF, f"value written for sequence {i}")
    close(out, torch.cat(ref), BF, "fused attention operation")
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("window", [0, 24, 64])
def test_attention_operation_far_key_and_window_edge(k, window):
    """One key among hundreds must win the softmax; with a window it sits on the window's first
    position for one sequence and one position outside it for the other."""
    H, Hkv, hd, page = 4, 2, 64, 32
    T = 300
    scale = 1 / math.sqrt(hd)
    far = 7 if window == 0 else T - 2 - window + 1
    kk = rnd((T, Hkv, hd), 1, BF, 0.3)
    v = rnd((T, Hkv, hd), 2, BF)
    q = rnd((T, H, hd), 3, BF, 0.3)
    kk[far] = 0
    kk[far, :, 0] = 12.0
    q[:, :, 0] = 12.0
    # two sequences with the same history: one is at position T-2, the other at T-1
    lens = [T - 2, T - 1]
    setup = PagedSetup([T, T], [2, 0], 4, page, Hkv, hd, BF, seed=3)
    pad = (-T) % page
    kp = torch.cat([kk, torch.zeros(pad, Hkv, hd, dtype=BF)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
    vp = torch.cat([v, torch.zeros(pad, Hkv, hd, dtype=BF)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
    for slot in (2, 0):
        pages = torch.from_numpy(setup.table[slot, :-(-T // page)].astype(np.int64)).cuda()
        setup.k[pages] = kp.cuda()
        setup.v[pages] = vp.cuda()
    rows = torch.stack([torch.cat([q[p].reshape(-1), kk[p].reshape(-1), v[p].reshape(-1)]) for p in lens]).cuda()
    out = torch.zeros((2, H * hd), dtype=BF).cuda()
    op = attn_op(k, rows, out, setup, H, Hkv, hd, window, scale)
    assert run_program(k, [op], 2, seq_start=lens, seq_slot=[2, 0]) == 0
    ref = attn_ref(q[-2:].double(), kk.double(), v.double(), T - 2, window, scale).reshape(2, H * hd)
    close(out, ref, BF, f"far key, window {window}")
    g = H // Hkv
    winner = v[far].float()[[h // g for h in range(H)]]
    assert torch.allclose(out[0].float().cpu().reshape(H, hd), winner, atol=0.05), "the far key did not win"
    if window:
        assert not torch.allclose(out[1].float().cpu().reshape(H, hd), winner, atol=0.05), \
            "a key outside the window was seen"


def test_a_row_length_that_is_no_multiple_of_32_is_refused(k):
    x, w, out = rnd((2, 104), 1, BF).cuda(), rnd((16, 104), 2, BF).cuda(), torch.zeros((2, 16), dtype=BF).cuda()
    assert run_program(k, [gemm_op(k, k.FUSED_XIN_BF16, k.FUSED_EPI_BF16, 1, x, w, out, 16)], 2) == 22
    assert out.abs().max().item() == 0


def test_a_normalised_row_too_long_to_stage_is_refused(k):
    M, K = 12, k.fused_decode_limits(12)["max_staged_k"] + 32
    x = rnd((M, K), 1, torch.float32).cuda()
    w = rnd((16, K), 2, BF).cuda()
    out = torch.zeros((M, 16), dtype=BF).cuda()
    op = gemm_op(k, k.FUSED_XIN_NORM, k.FUSED_EPI_BF16, 1, x, w, out, 16, torch.ones(K).cuda(), 1e-5)
    assert run_program(k, [op], M) == 22
    assert out.abs().max().item() == 0


def test_bad_token_and_missing_page_are_reported(k):
    table = rnd((50, 64), 1, BF).cuda()
    x = torch.zeros((2, 64), dtype=torch.float32).cuda()
    op = k.FusedOp()
    op.kind, op.K, op.vocab, op.scale = k.FUSED_OP_EMBED, 64, 50, 1.0
    op.table, op.C = table.data_ptr(), x.data_ptr()
    assert run_program(k, [op], 2, tokens=[3, 49]) == 0
    assert torch.equal(x.cpu(), table.float().cpu()[[3, 49]])
    assert run_program(k, [op], 2, tokens=[3, 50]) == 1
    assert x[1].abs().max().item() == 0


# ------------------------------------------------------------------------------- whole steps

@pytest.mark.parametrize("name,n_seqs", [("tiny_d", 3), ("tiny_e", 5), ("tiny_d", 12), ("tiny_e", 16)])
def test_fused_steps_against_the_plain_implementation(model_folders, name, n_seqs):
    """Unequal prompts, then 150 single tokens each through the one-kernel step (past page edges
    and past the window), then the slots are given back and used again by a second batch."""
    import zinfer_b200 as z
    folder = model_folders[name]
    plain = PlainLfm2(folder, dtype=np.float64)
    vocab = plain.cfg["vocab_size"]
    model = z.load(folder, dtype="bfloat16")
    eng = z.Engine(model, max_batch=16, max_seq_len=512, page_size=32, fused_decode=True)
    other = z.Engine(model, max_batch=16, max_seq_len=512, page_size=32)
    for batch in range(2):
        n = n_seqs if batch == 0 else max(1, n_seqs - 2)
        heads = [1 + (7 * i + 13 * batch) % 40 for i in range(n)]
        steps = 150 if batch == 0 else 20
        seqs = [helpers.random_tokens(900 + 50 * batch + i, h + steps, vocab) for i, h in enumerate(heads)]
        ref = [plain.logits(s) for s in seqs]
        slots, slots_o = eng.start(n), other.start(n)
        for e, sl in ((eng, slots), (other, slots_o)):
            e.step(sl, [s[:h] for s, h in zip(seqs, heads)], want=[[] for _ in seqs])
        err = gap = 0.0
        for p in range(steps):
            toks = [s[h + p] for s, h in zip(seqs, heads)]
            logits = eng.decode(slots, toks).cpu().numpy()
            separate = other.decode(slots_o, toks).cpu().numpy()
            for i in range(n):
                scale = np.abs(ref[i]).max()
                err = max(err, np.abs(logits[i] - ref[i][heads[i] + p]).max() / scale)
                gap = max(gap, np.abs(logits[i] - separate[i]).max() / scale)
        eng.check_status()
        assert eng._fused[n].plan, "the model was not fused"
        if batch == 1:
            rows = eng._fused[n].plan.trace(eng.last_fused_ctx, repeats=1)
            assert len(rows) == eng._fused[n].plan.n_ops and all(r["work_us"] >= 0 for r in rows)
            assert rows[0]["op"] == "embed" and rows[-1]["op"].startswith("gemm")
        assert not other._fused
        assert err <= helpers.TOL["bfloat16"], (batch, err)
        assert gap <= helpers.TOL["bfloat16"], (batch, gap)
        eng.finish(slots)
        other.finish(slots_o)
        eng.cache.check_consistency()


def test_models_the_kernel_does_not_take_keep_the_separate_kernels(model_folders):
    """Head size 16 (tiny_a) and float32 are not fused; the engine says so and decodes all the same."""
    import zinfer_b200 as z
    for name, dtype in (("tiny_a", "bfloat16"), ("tiny_d", "float32")):
        model = z.load(model_folders[name], dtype=dtype)
        eng = z.Engine(model, max_batch=2, max_seq_len=64, page_size=16, fused_decode=True)
        slots = eng.start(1)
        eng.step(slots, [[1, 2, 3]])
        for t in (4, 5, 6):
            eng.decode(slots, [t])
        eng.check_status()
        assert eng._fused[1].plan is False
        assert eng._graphs


def test_long_sequences_leave_the_fused_step(model_folders):
    """Beyond fused_decode_max_context the step goes back to the kernels that split a sequence's
    keys over blocks; logits stay those of the plain implementation across the change."""
    import zinfer_b200 as z
    folder = model_folders["tiny_d"]
    plain = PlainLfm2(folder, dtype=np.float64)
    seq = helpers.random_tokens(77, 60, plain.cfg["vocab_size"])
    ref = plain.logits(seq)
    model = z.load(folder, dtype="bfloat16")
    eng = z.Engine(model, max_batch=2, max_seq_len=128, page_size=32, fused_decode=True, fused_decode_max_context=40)
    slots = eng.start(1)
    eng.step(slots, [seq[:20]], want=[[]])
    err = 0.0
    for p in range(20, 60):
        logits = eng.decode(slots, [seq[p]]).cpu().numpy()
        err = max(err, np.abs(logits[0] - ref[p]).max() / np.abs(ref).max())
    assert eng._fused[1].plan and eng._graphs
    assert err <= helpers.TOL["bfloat16"], err
