"""Each kernel alone against a plain float64 reference, at sizes other than the tiny models':
widths and vocabularies that are no power of two, head sizes in steps of 16, odd group sizes,
page edges, and inputs made so that a fault shows (one far key that must win the softmax, a
window's edge)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype == torch.float32 else 1.5e-2


def close(got, ref, dtype, what=""):
    got = got.detach().double().cpu()
    ref = ref.detach().double().cpu()
    scale = ref.abs().max().item()
    assert scale > 0, f"{what}: empty reference"
    err = (got - ref).abs().max().item() / scale
    assert err <= tol(dtype), f"{what}: error {err:.3e} of max |ref| {scale:.3e}"


def rnd(shape, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.fixture(scope="module")
def k():
    from zinfer_b200 import kernels
    kernels.require_cuda()
    return kernels


# ------------------------------------------------------------------------------- row kernels

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim", [48, 2048 + 16, 7])
def test_embed_and_status(k, dtype, dim):
    vocab = 331
    table = rnd((vocab, dim), 1, dtype).cuda()
    toks = torch.tensor([0, 330, 17, 5, 17], dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    x = k.embed(toks, table, status)
    assert x.dtype == torch.float32 and status.item() == 0
    assert torch.equal(x.cpu(), table.float().cpu()[toks.cpu().long()])
    bad = torch.tensor([3, vocab], dtype=torch.int32).cuda()
    x = k.embed(bad, table, status)
    assert status.item() == 1 and x[1].abs().max().item() == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,dim,eps", [(5, 80, 1e-5), (3, 2048, 1e-6), (2, 1000, 3e-6), (1, 16, 1e-5),
                                       (300, 2048, 1e-5), (261, 200, 1e-6), (257, 2052, 1e-5)])
def test_rmsnorm(k, dtype, n, dim, eps):
    """Few rows (a block per row) and 256 rows and more (a warp per row up to a width of 2048; the row
    count no multiple of the 8 rows of a block)."""
    x = rnd((n, dim), 2, torch.float32, 3.0).cuda()
    x[n // 2] *= 50.0                                   # rows of different sizes: a row's scale is its own
    w = (1 + rnd((dim,), 3, torch.float32, 0.1)).cuda()
    ref = x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * w.double()
    got = k.rmsnorm(x, w, eps, dtype)
    for r in (0, n // 2, n - 1):
        close(got[r], ref[r], dtype, f"rmsnorm row {r}")
    close(got, ref, dtype, "rmsnorm")
    rows = torch.tensor([n - 1, 0], dtype=torch.int32).cuda()
    close(k.rmsnorm(x, w, eps, dtype, rows), ref[[n - 1, 0]], dtype, "rmsnorm rows")


def interleaved(parts, group=16):
    from zinfer_b200.parts.linear import interleave_rows
    return interleave_rows(parts, group)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(k, dtype):
    n, F = 7, 208
    gu = rnd((n, 2 * F), 4, dtype, 2.0).cuda()
    g, u = gu[:, :F].double(), gu[:, F:].double()
    ref = g / (1 + torch.exp(-g)) * u
    close(k.silu_mul(gu), ref, dtype, "silu_mul")
    mixed = interleaved([gu[:, :F].T.contiguous(), gu[:, F:].T.contiguous()]).T.contiguous()
    close(k.silu_mul(mixed, interleave=16), ref, dtype, "silu_mul, groups of 16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (5, 64, 64), (70, 200, 96), (130, 257, 1000), (64, 128, 2048)])
def test_gemm_simt(k, dtype, M, N, K):
    a = rnd((M, K), 5, dtype).cuda()
    w = rnd((N, K), 6, dtype, 0.1).cuda()
    bias = rnd((N,), 7, torch.float32).cuda()
    ref = a.double() @ w.double().T
    close(k.gemm_simt(a, w), ref, dtype, "gemm")
    close(k.gemm_simt(a, w, out_dtype=torch.float32), ref, dtype, "gemm f32 out")
    close(k.gemm_simt(a, w, bias=bias, out_dtype=torch.float32), ref + bias.double(), dtype, "gemm bias")
    res = rnd((M, N), 8, torch.float32).cuda()
    res0 = res.clone()
    k.gemm_simt(a, w, out=res, accumulate=True)
    close(res, ref + res0.double(), dtype, "gemm accumulate")


@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (8, 6144, 2048), (5, 100, 8200), (16, 2048, 512), (9, 48, 64),
                                   (33, 257, 1000), (64, 1030, 2048), (3, 65536 + 8, 256)])
def test_gemm_skinny(k, M, N, K):
    a = rnd((M, K), 5, torch.bfloat16).cuda()
    w = rnd((N, K), 6, torch.bfloat16, 0.1).cuda()
    bias = rnd((N,), 7, torch.float32).cuda()
    ref = a.double() @ w.double().T
    assert k.gemm_skinny_takes(a, w)
    close(k.gemm_skinny(a, w), ref, torch.bfloat16, "skinny")
    close(k.gemm_skinny(a, w, out_dtype=torch.float32), ref, torch.float32, "skinny f32 out")
    close(k.gemm_skinny(a, w, bias=bias, out_dtype=torch.float32), ref + bias.double(), torch.float32, "skinny bias")
    res = rnd((M, N), 8, torch.float32).cuda()
    res0 = res.clone()
    k.gemm_skinny(a, w, out=res, accumulate=True)
    close(res, ref + res0.double(), torch.float32, "skinny accumulate")
    assert not k.gemm_skinny_takes(rnd((65, K), 1, torch.bfloat16).cuda(), w)
    assert not k.gemm_skinny_takes(rnd((2, 12), 1, torch.bfloat16).cuda(), rnd((4, 12), 1, torch.bfloat16).cuda())


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 331 * 8, 2048), (2048, 6144, 2048), (130, 264, 8200),
                                   (65, 16, 72), (300, 2048, 8192), (2500, 4096, 128), (4200, 2304, 192)])
def test_gemm_tc_prompt_shapes(k, M, N, K):
    """One tile per block, and (many tiles, N a multiple of 256: the last three) persistent blocks with
    128 x 256 tiles; row tails, K tails, every way of storing."""
    a = rnd((M, K), 5, torch.bfloat16).cuda()
    w = rnd((N, K), 6, torch.bfloat16, 0.1).cuda()
    bias = rnd((N,), 7, torch.float32).cuda()
    ref = a.double() @ w.double().T
    assert k.gemm_tc_takes(a, w)
    close(k.gemm_tc(a, w, out_dtype=torch.float32), ref, torch.float32, "tc f32 out")
    close(k.gemm_tc(a, w), ref, torch.bfloat16, "tc bf16 out")
    close(k.gemm_tc(a, w, bias=bias, out_dtype=torch.float32), ref + bias.double(), torch.float32, "tc bias")
    res = rnd((M, N), 8, torch.float32).cuda()
    res0 = res.clone()
    k.gemm_tc(a, w, out=res, accumulate=True)
    close(res, ref + res0.double(), torch.float32, "tc accumulate")
    assert k.status_word("cuda").item() == 0


@pytest.mark.parametrize("form", [0, 256, 512])
@pytest.mark.parametrize("M,N,K,swiglu", [(256, 256, 64, False), (2048, 2048, 2048, False), (700, 1024, 520, False),
                                          (130, 768, 8200, False), (1100, 512, 192, True), (2048, 4096, 1024, True)])
def test_gemm_tc_forms_agree(k, form, M, N, K, swiglu):
    """The three forms of a prompt-step product (one tile per block, persistent blocks, persistent
    pairs of blocks with tcgen05.mma.cta_group::2) each against the plain product: row tails that
    leave the second block of a pair without rows, K tails, every way of storing."""
    a = rnd((M, K), 15, torch.bfloat16).cuda()
    w = rnd((N, K), 16, torch.bfloat16, 0.1).cuda()
    ref = a.double() @ w.double().T
    k.gemm_tc_force_form(form)
    try:
        if swiglu:
            g = ref.reshape(M, N // 32, 2, 16)
            act = (g[:, :, 0] / (1 + torch.exp(-g[:, :, 0])) * g[:, :, 1]).reshape(M, N // 2)
            close(k.gemm_tc(a, w, swiglu=True), act, torch.bfloat16, "swiglu")
        else:
            close(k.gemm_tc(a, w, out_dtype=torch.float32), ref, torch.float32, "f32 out")
            close(k.gemm_tc(a, w), ref, torch.bfloat16, "bf16 out")
            res = rnd((M, N), 18, torch.float32).cuda()
            res0 = res.clone()
            k.gemm_tc(a, w, out=res, accumulate=True)
            close(res, ref + res0.double(), torch.float32, "accumulate")
        torch.cuda.synchronize()
        assert k.status_word("cuda").item() == 0
    finally:
        k.gemm_tc_force_form(-1)


@pytest.mark.parametrize("M,N,K,splits", [(1, 128, 64, 1), (8, 6144, 2048, 1), (8, 2048, 8192, 8), (16, 331 * 8, 2048, 3),
                                          (17, 2048, 2048, 4), (33, 100, 520, 2), (64, 16384, 2048, 2), (5, 65536, 256, 1)])
def test_gemm_tc_single_token_shapes(k, M, N, K, splits):
    a = rnd((M, K), 5, torch.bfloat16).cuda()
    w = rnd((N, K), 6, torch.bfloat16, 0.1).cuda()
    bias = rnd((N,), 7, torch.float32).cuda()
    ref = a.double() @ w.double().T
    close(k.gemm_tc(a, w, out_dtype=torch.float32, splits=splits), ref, torch.float32, "tc swapped")
    close(k.gemm_tc(a, w, splits=splits, bias=bias), ref + bias.double(), torch.bfloat16, "tc swapped bf16 + bias")
    res = rnd((M, N), 8, torch.float32).cuda()
    res0 = res.clone()
    k.gemm_tc(a, w, out=res, accumulate=True, splits=splits)
    close(res, ref + res0.double(), torch.float32, "tc swapped accumulate")
    again = res0.clone()
    k.gemm_tc(a, w, out=again, accumulate=True, splits=splits)
    assert torch.equal(again, res), "the same launch gave other bits"
    assert k.status_word("cuda").item() == 0


def norm_ref(x, w, eps):
    return (x.double() / torch.sqrt((x.double() ** 2).mean(-1, keepdim=True) + eps) * w.double())


@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (8, 6144, 2048), (16, 100, 1000), (11, 48, 64)])
def test_gemm_skinny_with_fused_norm(k, M, N, K):
    x = rnd((M, K), 1, torch.float32, 3.0).cuda()
    nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
    w = rnd((N, K), 3, torch.bfloat16, 0.1).cuda()
    ref = norm_ref(x, nw, 1e-5).bfloat16().double() @ w.double().T
    inp = k.NormInput(x, nw, 1e-5)
    assert k.gemm_skinny_takes(inp, w)
    close(k.gemm_skinny(inp, w, out_dtype=torch.float32), ref, torch.bfloat16, "skinny + norm")
    unfused = k.gemm_skinny(k.rmsnorm(x, nw, 1e-5, torch.bfloat16), w, out_dtype=torch.float32)
    close(k.gemm_skinny(inp, w, out_dtype=torch.float32), unfused.double(), torch.bfloat16, "fused vs unfused norm")
    assert not k.gemm_skinny_takes(k.NormInput(rnd((17, K), 1, torch.float32).cuda(), nw, 1e-5), w)


@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (8, 2048, 8192), (5, 5000, 64), (8, 16 * 148 * 6 + 24, 32), (3, 16, 8),
                                   (9, 331, 80), (16, 2048, 8192), (13, 5000, 64), (16, 16 * 148 * 6 + 24, 32)])
def test_gemm_skinny_writes_the_next_norms_inputs(k, M, N, K):
    """The accumulating contraction into float32 rows also writes bfloat16(rows * norm weight) and the
    rows' sums of squares per 16 columns: all three kernel shapes (few, some, many blocks), a ragged
    last group of columns."""
    a = rnd((M, K), 1, torch.bfloat16).cuda()
    w = rnd((N, K), 2, torch.bfloat16, 0.1).cuda()
    nw = (1 + rnd((N,), 3, torch.float32, 0.2)).cuda()
    res0 = rnd((M, N), 4, torch.float32, 2.0).cuda()
    res, plain = res0.clone(), res0.clone()
    emit = k.NormEmit(nw)
    assert k.gemm_skinny_emits(a, res)
    k.gemm_skinny(a, w, out=res, accumulate=True, emit=emit)
    k.gemm_skinny(a, w, out=plain, accumulate=True)
    assert torch.equal(res, plain)                       # the sum itself is the same bits
    assert emit.xw.shape == (M, N) and emit.ssq.shape == (M, -(-N // 16))
    assert torch.equal(emit.xw, (res * nw).bfloat16())
    sq = torch.zeros((M, emit.ssq.shape[1] * 16), dtype=torch.float64, device="cuda")
    sq[:, :N] = res.double() ** 2
    close(emit.ssq, sq.reshape(M, -1, 16).sum(-1), torch.float32, "sums of squares per 16 columns")
    with pytest.raises(k.KernelError):
        k.gemm_skinny(rnd((17, K), 1, torch.bfloat16).cuda(), w, out=rnd((17, N), 4, torch.float32).cuda(),
                      accumulate=True, emit=k.NormEmit(nw))
    with pytest.raises(k.KernelError):
        k.gemm_skinny(a, w, out=res.bfloat16(), accumulate=True, emit=k.NormEmit(nw))


def scaled_input(k, x, nw, eps, parts_of=16):
    """What a contraction that summed into x would have left for the norm (nw, eps)."""
    M, K = x.shape
    sq = torch.zeros((M, -(-K // parts_of) * parts_of), dtype=torch.float32, device=x.device)
    sq[:, :K] = x * x
    return k.ScaledInput((x * nw).bfloat16(), sq.reshape(M, -1, parts_of).sum(-1).contiguous(), eps)


@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (8, 6144, 2048), (16, 100, 1000), (7, 65536 + 16, 72)])
def test_gemm_skinny_with_prepared_norm(k, M, N, K):
    x = rnd((M, K), 1, torch.float32, 3.0).cuda()
    x[M - 1] *= 40.0                                    # a row whose scale differs much from the others'
    nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
    w = rnd((N, K), 3, torch.bfloat16, 0.1).cuda()
    ref = norm_ref(x, nw, 1e-5).bfloat16().double() @ w.double().T
    inp = scaled_input(k, x, nw, 1e-5)
    assert k.gemm_skinny_takes(inp, w)
    close(k.gemm_skinny(inp, w, out_dtype=torch.float32), ref, torch.bfloat16, "skinny + prepared norm")
    for m in range(M):     # each row against its own size: a wrong row's scale would show
        close(k.gemm_skinny(inp, w, out_dtype=torch.float32)[m], ref[m], torch.bfloat16, f"row {m}")
    bias = rnd((N,), 5, torch.float32).cuda()
    res0 = rnd((M, N), 4, torch.float32).cuda()
    res = res0.clone()
    k.gemm_skinny(inp, w, out=res, accumulate=True, bias=bias)
    close(res, ref + bias.double() + res0.double(), torch.bfloat16, "prepared norm, bias, accumulate")
    assert not k.gemm_skinny_takes(scaled_input(k, rnd((17, K), 1, torch.float32).cuda(), nw, 1e-5), w)


@pytest.mark.parametrize("M,F,K,norm", [(1, 208, 80, False), (8, 8192, 2048, True), (16, 144, 96, True), (5, 32, 64, False),
                                        (8, 8192, 2048, "prepared"), (3, 48, 72, "prepared"), (13, 144, 96, "prepared")])
def test_gemm_skinny_swiglu(k, M, F, K, norm):
    halves = rnd((2 * F, K), 3, torch.bfloat16, 0.3).cuda()
    w_mixed = interleaved([halves[:F], halves[F:]])
    w = halves
    if norm:
        x = rnd((M, K), 1, torch.float32, 2.0).cuda()
        nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
        inp = scaled_input(k, x, nw, 1e-6) if norm == "prepared" else k.NormInput(x, nw, 1e-6)
        a = norm_ref(x, nw, 1e-6).bfloat16().double()
    else:
        inp = rnd((M, K), 1, torch.bfloat16).cuda()
        a = inp.double()
    g, u = a @ w[:F].double().T, a @ w[F:].double().T
    close(k.gemm_skinny_swiglu(inp, w_mixed), g / (1 + torch.exp(-g)) * u, torch.bfloat16, "skinny swiglu")
    with pytest.raises(k.KernelError):
        k.gemm_skinny_swiglu(inp, w_mixed[:48])        # 24 outputs: not whole groups of 16


@pytest.mark.parametrize("M,F,K", [(65, 64, 64), (300, 8192, 2048), (130, 208, 520), (64, 8192, 2048), (17, 208, 520),
                                   (40, 64, 64), (1, 32, 64), (700, 8192, 256), (2100, 2304, 96)])
def test_gemm_tc_with_swiglu_epilogue(k, M, F, K):
    """Normal mode (more than 64 rows) and swapped mode (the weights on the 128-row side; K whole, and
    cut into 2, 4 and 8 parts over a cluster)."""
    a = rnd((M, K), 1, torch.bfloat16).cuda()
    halves = rnd((2 * F, K), 3, torch.bfloat16, 0.3).cuda()
    g, u = a.double() @ halves[:F].double().T, a.double() @ halves[F:].double().T
    for splits in (1, 2, 4, 8) if M <= 64 else (1,):
        h = k.gemm_tc(a, interleaved([halves[:F], halves[F:]]), swiglu=True, splits=splits)
        assert h.shape == (M, F)
        close(h, g / (1 + torch.exp(-g)) * u, torch.bfloat16, f"tcgen05 contraction with SwiGLU epilogue, K in {splits}")
    assert k.status_word("cuda").item() == 0


@pytest.mark.parametrize("M,N,K", [(9, 328, 80), (64, 2048, 8192), (33, 5000, 64), (16, 136, 520), (64, 2048, 2048)])
@pytest.mark.parametrize("splits", [1, 2, 4, 8])
def test_gemm_tc_writes_the_next_norms_inputs(k, M, N, K, splits):
    """Up to 64 rows (the weights on the 128-row side): the accumulating contraction into float32 rows
    also writes bfloat16(rows * norm weight) and the rows' sums of squares per 32 columns, with K whole
    and cut over a cluster; a ragged last tile of weight rows."""
    a = rnd((M, K), 1, torch.bfloat16).cuda()
    w = rnd((N, K), 2, torch.bfloat16, 0.1).cuda()
    nw = (1 + rnd((N,), 3, torch.float32, 0.2)).cuda()
    bias = rnd((N,), 5, torch.float32).cuda()
    res0 = rnd((M, N), 4, torch.float32, 2.0).cuda()
    res, plain = res0.clone(), res0.clone()
    emit = k.NormEmit(nw)
    assert k.gemm_tc_emits(a, res)
    k.gemm_tc(a, w, out=res, accumulate=True, bias=bias, splits=splits, emit=emit)
    k.gemm_tc(a, w, out=plain, accumulate=True, bias=bias, splits=splits)
    assert torch.equal(res, plain)                       # the sum itself is the same bits
    close(res, a.double() @ w.double().T + bias.double() + res0.double(), torch.bfloat16, "the sum")
    assert emit.xw.shape == (M, N) and emit.ssq.shape == (M, -(-N // 32))
    assert torch.equal(emit.xw, (res * nw).bfloat16())
    sq = torch.zeros((M, emit.ssq.shape[1] * 32), dtype=torch.float64, device="cuda")
    sq[:, :N] = res.double() ** 2
    close(emit.ssq, sq.reshape(M, -1, 32).sum(-1), torch.float32, "sums of squares per 32 columns")
    assert k.status_word("cuda").item() == 0
    with pytest.raises(k.KernelError):
        k.gemm_tc(a, w, out=res.bfloat16(), accumulate=True, emit=k.NormEmit(nw))


@pytest.mark.parametrize("M,N,K", [(9, 328, 80), (64, 6144, 2048), (33, 65536 + 32, 72), (20, 136, 520)])
@pytest.mark.parametrize("splits", [1, 2, 8])
def test_gemm_tc_with_prepared_norm(k, M, N, K, splits):
    x = rnd((M, K), 1, torch.float32, 3.0).cuda()
    x[M - 1] *= 40.0                                    # a row whose scale differs much from the others'
    x[0] *= 0.01
    nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
    w = rnd((N, K), 3, torch.bfloat16, 0.1).cuda()
    ref = norm_ref(x, nw, 1e-5).bfloat16().double() @ w.double().T
    inp = scaled_input(k, x, nw, 1e-5, parts_of=32)
    assert k.gemm_tc_takes(inp, w)
    got = k.gemm_tc(inp, w, out_dtype=torch.float32, splits=splits)
    for m in range(M):     # each row against its own size: a wrong row's scale would show
        close(got[m], ref[m], torch.bfloat16, f"row {m}")
    bias = rnd((N,), 5, torch.float32).cuda()
    res0 = rnd((M, N), 4, torch.float32).cuda()
    res = res0.clone()
    k.gemm_tc(inp, w, out=res, accumulate=True, bias=bias, splits=splits)
    close(res, ref + bias.double() + res0.double(), torch.bfloat16, "prepared norm, bias, accumulate")
    if N % 32 == 0:
        F = N // 2
        g, u = ref[:, :F], ref[:, F:]
        h = k.gemm_tc(inp, interleaved([w[:F], w[F:]]), swiglu=True, splits=splits)
        close(h, g / (1 + torch.exp(-g)) * u, torch.bfloat16, "prepared norm with the SwiGLU epilogue")
    assert k.status_word("cuda").item() == 0
    assert not k.gemm_tc_takes(scaled_input(k, rnd((65, K), 1, torch.float32).cuda(), nw, 1e-5), w)


@pytest.mark.parametrize("M,D,K,taps,bias,norm", [(1, 80, 80, 2, False, False), (8, 2048, 2048, 3, False, True),
                                                  (13, 96, 96, 4, True, True), (16, 48, 64, 7, True, False),
                                                  (8, 2048, 2048, 3, False, "prepared"), (5, 96, 104, 4, True, "prepared")])
def test_gemm_skinny_conv_equals_the_unfused_step(k, M, D, K, taps, bias, norm):
    """Three fused single-token steps against in_proj + conv_decode, state included; in_proj's rows
    are stored as groups of 16 B, 16 C, 16 X rows for both paths."""
    w_in = rnd((3 * D, K), 3, torch.bfloat16, 0.2).cuda()
    tw = rnd((taps, D), 4, torch.float32).cuda()
    in_b = rnd((3 * D,), 5, torch.float32).cuda() if bias else None
    cb = rnd((D,), 6, torch.float32).cuda() if bias else None
    nw = (1 + rnd((K,), 2, torch.float32, 0.1)).cuda()
    slots = torch.randperm(M + 3, generator=torch.Generator().manual_seed(1))[:M].to(torch.int32).cuda()
    st_a = rnd((M + 3, taps - 1, D), 7, torch.float32).cuda()
    st_b = st_a.clone()
    for step in range(3):
        x = rnd((M, K), 10 + step, torch.float32, 2.0).cuda()
        if norm:
            inp = scaled_input(k, x, nw, 1e-5) if norm == "prepared" else k.NormInput(x, nw, 1e-5)
            xn = k.rmsnorm(x, nw, 1e-5, torch.bfloat16)
        else:
            inp = xn = x.bfloat16()
        y_fused = k.gemm_skinny_conv(inp, w_in, in_b, st_a, tw, cb, slots)
        bcx = k.gemm_skinny(xn, w_in, bias=in_b)
        y_ref = k.conv_decode(bcx, st_b, tw, cb, slots, interleave=16)
        close(y_fused, y_ref.double(), torch.bfloat16, f"fused conv step {step}")
        close(st_a, st_b.double(), torch.bfloat16, f"fused conv state {step}")
    untouched = [i for i in range(M + 3) if i not in slots.cpu().tolist()]
    assert torch.equal(st_a[untouched], rnd((M + 3, taps - 1, D), 7, torch.float32).cuda()[untouched])


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_rows_do_not_depend_on_the_batch(k, dtype):
    """A row's contraction is the same bits alone, in a batch, and at another place of it, as long
    as the same kernel runs: in float32 always; in bfloat16 among batches of up to 16 rows (the
    mma.sync kernel, whose warps split K the same way for 8 and for 16 rows) and among batches of 17
    to 64 rows (the tcgen05 kernel with split K)."""
    from zinfer_b200.parts.linear import linear
    a = rnd((70, 96), 9, dtype).cuda()
    w = rnd((200, 96), 10, dtype, 0.1).cuda()
    if dtype == torch.float32:
        full = linear(a, w, out_dtype=torch.float32)
        one = linear(a[33:34].contiguous(), w, out_dtype=torch.float32)
        moved = linear(a[30:40].contiguous(), w, out_dtype=torch.float32)
        assert torch.equal(full[33], one[0]) and torch.equal(full[33], moved[3])
        return
    small = linear(a[28:36].contiguous(), w, out_dtype=torch.float32)            # 8 rows
    one = linear(a[33:34].contiguous(), w, out_dtype=torch.float32)
    moved = linear(a[30:35].contiguous(), w, out_dtype=torch.float32)
    more = linear(a[22:38].contiguous(), w, out_dtype=torch.float32)             # 16 rows
    assert torch.equal(small[5], one[0]) and torch.equal(small[5], moved[3]) and torch.equal(small[5], more[11])
    wide = rnd((2048, 96), 11, dtype, 0.1).cuda()                               # enough rows for a split of K
    big = linear(a[:64].contiguous(), wide, out_dtype=torch.float32)
    mid = linear(a[20:40].contiguous(), wide, out_dtype=torch.float32)          # 20 rows
    few = linear(a[30:47].contiguous(), wide, out_dtype=torch.float32)          # 17 rows
    assert torch.equal(big[33], mid[13]) and torch.equal(big[33], few[3])


# ------------------------------------------------------------------------------- short convolution

def conv_ref(bcx, taps, bias, state):
    """bcx [T, 3D] of one sequence, taps [K, D], state [K-1, D] -> (y [T, D], new state)."""
    T, D = bcx.shape[0], bcx.shape[1] // 3
    K = taps.shape[0]
    u = bcx[:, :D] * bcx[:, 2 * D:]
    hist = torch.cat([state, u], 0)
    c = torch.zeros(T, D, dtype=torch.float64)
    for j in range(K):
        c += taps[j] * hist[j:j + T]
    if bias is not None:
        c += bias
    return bcx[:, D:2 * D] * c, hist[T:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D,K,use_bias", [(80, 2, False), (96, 4, True), (200, 3, False), (64, 7, True)])
def test_short_conv_packed_and_stepwise(k, dtype, D, K, use_bias):
    lens = [1, 2, 9, K - 1, 33]
    slots = [4, 0, 2, 5, 1]
    n_slots = 6
    taps = rnd((K, D), 11, torch.float32).cuda()
    bias = rnd((D,), 12, torch.float32).cuda() if use_bias else None
    seqs = [rnd((l, 3 * D), 20 + i, dtype) for i, l in enumerate(lens)]
    state = rnd((n_slots, K - 1, D), 13, torch.float32).cuda()     # junk in every slot ...
    state[slots] = 0                                               # ... but zero where a sequence starts
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    tok_seq = torch.from_numpy(np.repeat(np.arange(len(lens)), lens).astype(np.int32)).cuda()
    cu_q = torch.from_numpy(cu).cuda()
    seq_slot = torch.tensor(slots, dtype=torch.int32).cuda()
    bcx = torch.cat(seqs).cuda()
    y = k.conv_forward(bcx, state, taps, bias, tok_seq, cu_q, seq_slot)
    if D % 16 == 0:      # the same step with the columns stored as groups of 16 B, 16 C, 16 X
        mixed = interleaved([bcx[:, :D].T.contiguous(), bcx[:, D:2 * D].T.contiguous(), bcx[:, 2 * D:].T.contiguous()]).T.contiguous()
        y_mixed = k.conv_forward(mixed, state, taps, bias, tok_seq, cu_q, seq_slot, interleave=16)
        assert torch.equal(y_mixed, y)
        state_mixed = state.clone()
        k.conv_state_update(mixed, state_mixed, cu_q, seq_slot, len(lens), K, interleave=16)
    k.conv_state_update(bcx, state, cu_q, seq_slot, len(lens), K)
    if D % 16 == 0:
        assert torch.equal(state_mixed, state)
    refs = [conv_ref(s.double(), taps.double().cpu(), None if bias is None else bias.double().cpu(),
                     torch.zeros(K - 1, D, dtype=torch.float64)) for s in seqs]
    close(y, torch.cat([r[0] for r in refs]), dtype, "conv prefill y")
    for s, r in zip(slots, refs):
        close(state[s], r[1], torch.float32, "conv state after prefill") if r[1].abs().max() > 0 else None
    assert torch.equal(state[3].cpu(), rnd((n_slots, K - 1, D), 13, torch.float32)[3]), "a slot not in the batch changed"
    # three more single-token steps for every sequence, compared with the whole sequence at once
    more = [rnd((3, 3 * D), 40 + i, dtype) for i in range(len(lens))]
    for t in range(3):
        step = torch.stack([m[t] for m in more]).cuda()
        yd = k.conv_decode(step, state, taps, bias, seq_slot)
        for i in range(len(lens)):
            whole = conv_ref(torch.cat([seqs[i], more[i][:t + 1]]).double(), taps.double().cpu(),
                             None if bias is None else bias.double().cpu(), torch.zeros(K - 1, D, dtype=torch.float64))
            close(yd[i], whole[0][-1], dtype, f"conv decode step {t} seq {i}")
    # a second packed step (continuation of a prompt) must equal the decode path
    state2 = torch.zeros_like(state)
    k.conv_state_update(bcx, state2, cu_q, seq_slot, len(lens), K)
    cont = torch.cat(more).cuda()
    cu2 = torch.from_numpy(np.arange(0, 3 * len(lens) + 1, 3).astype(np.int32)).cuda()
    ts2 = torch.from_numpy(np.repeat(np.arange(len(lens)), 3).astype(np.int32)).cuda()
    y2 = k.conv_forward(cont, state2, taps, bias, ts2, cu2, seq_slot)
    for i in range(len(lens)):
        whole = conv_ref(torch.cat([seqs[i], more[i]]).double(), taps.double().cpu(),
                         None if bias is None else bias.double().cpu(), torch.zeros(K - 1, D, dtype=torch.float64))
        close(y2[3 * i:3 * i + 3], whole[0][-3:], dtype, f"conv continued prompt seq {i}")


@pytest.mark.parametrize("D,K,use_bias,il", [(96, 3, False, 16), (200, 2, True, 0), (64, 4, True, 16), (2048, 3, False, 16)])
def test_short_conv_of_many_packed_tokens(k, D, K, use_bias, il):
    """Prompt steps of 256 tokens and more in bfloat16 (runs of tokens per thread): sequences of unequal
    lengths whose borders fall inside a run, states that are not zero (continued prompts); against the
    reference, and the same bits as each sequence alone in a step of few tokens (the other kernel)."""
    lens = [1, 2, 131, K - 1, 77, 3, 202, 5]
    slots = [4, 0, 2, 7, 1, 8, 3, 6]
    n_slots = 9
    taps = rnd((K, D), 11, torch.float32).cuda()
    bias = rnd((D,), 12, torch.float32).cuda() if use_bias else None
    seqs = [rnd((l, 3 * D), 20 + i, torch.bfloat16) for i, l in enumerate(lens)]
    state = rnd((n_slots, K - 1, D), 13, torch.float32).cuda()
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    assert cu[-1] >= 256
    tok_seq = torch.from_numpy(np.repeat(np.arange(len(lens)), lens).astype(np.int32)).cuda()
    seq_slot = torch.tensor(slots, dtype=torch.int32).cuda()

    def stored(rows):      # the column order the kernel is told about
        if not il:
            return rows.cuda()
        return interleaved([rows[:, :D].T.contiguous(), rows[:, D:2 * D].T.contiguous(),
                            rows[:, 2 * D:].T.contiguous()]).T.contiguous().cuda()

    y = k.conv_forward(stored(torch.cat(seqs)), state, taps, bias, tok_seq, torch.from_numpy(cu).cuda(), seq_slot,
                       interleave=il)
    for i, sq in enumerate(seqs):
        ref, _ = conv_ref(sq.double(), taps.double().cpu(), None if bias is None else bias.double().cpu(),
                          state[slots[i]].double().cpu())
        close(y[cu[i]:cu[i + 1]], ref, torch.bfloat16, f"sequence {i} of the packed step")
        if lens[i] < 256:
            alone = k.conv_forward(stored(sq), state, taps, bias, torch.zeros(lens[i], dtype=torch.int32).cuda(),
                                   torch.tensor([0, lens[i]], dtype=torch.int32).cuda(), seq_slot[i:i + 1], interleave=il)
            assert torch.equal(alone, y[cu[i]:cu[i + 1]]), f"sequence {i}: packed and alone differ"


# ------------------------------------------------------------------------------- attention

def rope_ref(x, pos, inv_freq, interleaved=False):
    """x [T, heads, hd] float64; NeoX or interleaved pairing."""
    half = inv_freq.shape[0]
    ang = (pos.float()[:, None] * inv_freq.float()[None, :]).double()
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = a * cos - b * sin
        out[..., 1:2 * half:2] = a * sin + b * cos
    else:
        a, b = x[..., :half], x[..., half:2 * half]
        out[..., :half] = a * cos - b * sin
        out[..., half:2 * half] = a * sin + b * cos
    return out


def attn_ref(q, kk, v, starts_q, window, scale):
    """q [Tq, H, hd] at positions starts_q.., keys kk, v [Tk, Hkv, hd] at positions 0..Tk-1."""
    Tq, H, hd = q.shape
    Hkv = kk.shape[1]
    g = H // Hkv
    out = torch.zeros_like(q)
    for h in range(H):
        s = (q[:, h] @ kk[:, h // g].T) * scale
        i = (starts_q + torch.arange(Tq))[:, None]
        j = torch.arange(kk.shape[0])[None, :]
        mask = j <= i
        if window > 0:
            mask &= j >= i + 1 - window
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // g]
    return out


class PagedSetup:
    """A small paged cache with shuffled pages for sequences of given lengths."""

    def __init__(self, lens, slots, n_slots, page_size, Hkv, hd, dtype, seed=0):
        self.page_size = page_size
        pages_per = [-(-l // page_size) for l in lens]
        n_pages = sum(pages_per) + 3
        perm = np.random.default_rng(seed).permutation(n_pages)
        self.table = np.full((n_slots, max(pages_per) + 1), -1, dtype=np.int32)
        it = iter(perm)
        for s, n in zip(slots, pages_per):
            for i in range(n):
                self.table[s, i] = next(it)
        self.k = torch.full((n_pages, Hkv, page_size, hd), float("nan"), dtype=dtype).cuda()
        self.v = torch.full((n_pages, Hkv, page_size, hd), float("nan"), dtype=dtype).cuda()
        self.table_dev = torch.from_numpy(self.table).cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Hkv,hd,page,n_rot,inter", [(4, 2, 16, 16, 16, False), (3, 1, 32, 32, 32, False),
                                                       (5, 5, 48, 64, 48, False), (8, 2, 80, 16, 40, True),
                                                       (6, 2, 128, 64, 128, False), (20, 1, 64, 32, 64, False),
                                                       (32, 8, 64, 64, 64, False), (7, 7, 96, 32, 96, False),
                                                       (16, 2, 32, 64, 32, False), (6, 2, 64, 128, 64, False),
                                                       (5, 1, 128, 64, 64, True), (16, 1, 64, 64, 64, False)])
def test_qk_prepare_then_attention(k, dtype, H, Hkv, hd, page, n_rot, inter):
    """Prompt step of unequal lengths into NaN-filled shuffled pages, then a single-token step
    with and without key splits, against whole-sequence references."""
    from zinfer_b200.parts.attention import query_tiles as attn_tiles_host
    lens = [1, 2, 37, 70, 5]
    slots = [3, 0, 5, 1, 4]
    eps = 1e-5
    scale = 1 / math.sqrt(hd)
    setup = PagedSetup([l + 1 for l in lens], slots, 6, page, Hkv, hd, dtype)
    qw = (1 + rnd((hd,), 1, torch.float32, 0.1)).cuda()
    kw = (1 + rnd((hd,), 2, torch.float32, 0.1)).cuda()
    inv_freq = torch.from_numpy(np.power(10000.0, -2.0 * np.arange(n_rot // 2) / n_rot).astype(np.float32)).cuda()
    status = torch.zeros(1, dtype=torch.int32).cuda()
    width = (H + 2 * Hkv) * hd
    seqs = [rnd((l + 1, width), 50 + i, dtype) for i, l in enumerate(lens)]   # last row = the decode token

    def reference(i, upto):
        x = seqs[i][:upto].double()
        q = x[:, :H * hd].reshape(upto, H, hd)
        kk = x[:, H * hd:(H + Hkv) * hd].reshape(upto, Hkv, hd)
        v = x[:, (H + Hkv) * hd:].reshape(upto, Hkv, hd)
        nrm = lambda t, w: t / torch.sqrt((t ** 2).mean(-1, keepdim=True) + eps) * w.double().cpu()
        pos = torch.arange(upto)
        q = rope_ref(nrm(q, qw), pos, inv_freq.cpu(), inter)
        kk = rope_ref(nrm(kk, kw), pos, inv_freq.cpu(), inter)
        if dtype == torch.bfloat16:      # the cache and q hold bfloat16
            q, kk, v = q.bfloat16().double(), kk.bfloat16().double(), v.bfloat16().double()
        return q, kk, v

    def run(step_lens, starts, rows, num_splits=1, split_keys=0, single_token=False, kind=None):
        cu = np.concatenate([[0], np.cumsum(step_lens)]).astype(np.int32)
        tok_seq = torch.from_numpy(np.repeat(np.arange(len(step_lens)), step_lens).astype(np.int32)).cuda()
        tok_pos = torch.from_numpy(np.concatenate([np.arange(s, s + l) for s, l in zip(starts, step_lens)]).astype(np.int32)).cuda()
        seq_slot = torch.tensor(slots, dtype=torch.int32).cuda()
        seq_start = torch.tensor(starts, dtype=torch.int32).cuda()
        cu_q = torch.from_numpy(cu).cuda()
        q = k.qk_prepare(rows.cuda(), setup.k, setup.v, qw, kw, inv_freq, tok_seq, tok_pos, seq_slot, setup.table_dev,
                         H, Hkv, hd, n_rot, inter, eps, status)
        bq, _ = k.attn_tile_shape(H, Hkv)
        if kind == "prompt_tc":
            bq = k._fn("attention_prefill", "zk_attn_prefill_tile_tokens")(H, Hkv)
        if kind == "prompt_tc5":
            bq = k._fn("attention_prefill_tc5", "zk_attn_prefill_tc5_tile_tokens")(H, Hkv)
        tiles = torch.from_numpy(attn_tiles_host(step_lens, bq)).cuda()
        return k.attention(q, setup.k, setup.v, tiles[0].contiguous(), tiles[1].contiguous(), cu_q, seq_start,
                           seq_slot, setup.table_dev, H, Hkv, hd, scale, 0, num_splits, split_keys, single_token, kind)

    out = run(lens, [0] * len(lens), torch.cat([s[:-1] for s in seqs]))
    assert status.item() == 0
    ref = []
    for i, l in enumerate(lens):
        q, kk, v = reference(i, l)
        ref.append(attn_ref(q, kk, v, 0, 0, scale).reshape(l, H * hd))
    close(out, torch.cat(ref), dtype, "prefill attention")
    if dtype == torch.bfloat16 and k._takes("attention_prefill", "zk_attn_prefill_takes", H, Hkv, hd, page):
        again = run(lens, [0] * len(lens), torch.cat([s[:-1] for s in seqs]), kind="prompt_tc")
        close(again, torch.cat(ref), dtype, "prefill attention on the tensor cores")
        assert not torch.isnan(again.float()).any()
    if k.attention_plan(dtype, H, Hkv, hd, page, False)[0] == "prompt_tc5":
        again = run(lens, [0] * len(lens), torch.cat([s[:-1] for s in seqs]), kind="prompt_tc5")
        assert status.item() == 0 and k.status_word("cuda").item() == 0
        close(again, torch.cat(ref), dtype, "prefill attention with tcgen05")
        assert not torch.isnan(again.float()).any()
    last = torch.stack([s[-1] for s in seqs])
    ref = []
    for i, l in enumerate(lens):
        q, kk, v = reference(i, l + 1)
        ref.append(attn_ref(q[-1:], kk, v, l, 0, scale).reshape(1, H * hd))
    ref = torch.cat(ref)
    close(run([1] * len(lens), lens, last), ref, dtype, "decode attention")
    close(run([1] * len(lens), lens, last, num_splits=3, split_keys=32), ref, dtype, "decode attention, 3 key chunks")
    close(run([1] * len(lens), lens, last, single_token=True), ref, dtype, "single-token kernel")
    close(run([1] * len(lens), lens, last, 2, 64, single_token=True), ref, dtype, "single-token kernel, 2 key chunks")
    assert not torch.isnan(out).any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 24, 64])
def test_attention_far_key_and_window_edge(k, dtype, window):
    """One key among hundreds is made to win the softmax; with a window the winner sits exactly
    on the window's first position for one query and one position outside it for the next."""
    from zinfer_b200.parts.attention import query_tiles as attn_tiles_host
    H, Hkv, hd, page = 4, 2, 32, 32
    T = 300
    scale = 1 / math.sqrt(hd)
    far = 7 if window == 0 else T - 2 - window + 1     # position of the key that must win
    kk = rnd((T, Hkv, hd), 1, dtype, 0.3)
    v = rnd((T, Hkv, hd), 2, dtype)
    q = rnd((T, H, hd), 3, dtype, 0.3)
    kk[far] = 0
    kk[far, :, 0] = 12.0
    q[:, :, 0] = 12.0               # every query scores 144 * scale on the far key
    setup = PagedSetup([T], [2], 4, page, Hkv, hd, dtype, seed=3)
    pages = torch.from_numpy(setup.table[2, :-(-T // page)].astype(np.int64)).cuda()
    pad = (-T) % page
    kp = torch.cat([kk, torch.zeros(pad, Hkv, hd, dtype=dtype)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
    vp = torch.cat([v, torch.zeros(pad, Hkv, hd, dtype=dtype)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
    setup.k[pages] = kp.cuda()
    setup.v[pages] = vp.cuda()
    # the last two queries as one step continuing at position T-2
    starts = T - 2
    bq, _ = k.attn_tile_shape(H, Hkv)
    tiles = torch.from_numpy(attn_tiles_host([2], bq)).cuda()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    out = k.attention(q[-2:].reshape(2, H * hd).cuda(), setup.k, setup.v, tiles[0].contiguous(),
                      tiles[1].contiguous(), i32([0, 2]), i32([starts]), i32([2]), setup.table_dev, H, Hkv, hd, scale,
                      window)
    ref = attn_ref(q[-2:].double(), kk.double(), v.double(), starts, window, scale).reshape(2, H * hd)
    close(out, ref, dtype, f"far key, window {window}")
    g = H // Hkv
    won = torch.allclose(out[0].float().cpu().reshape(H, hd), v[far].float()[[h // g for h in range(H)]], atol=0.05)
    assert won, "the far key did not win for the query that sees it"
    if window:
        lost = torch.allclose(out[1].float().cpu().reshape(H, hd), v[far].float()[[h // g for h in range(H)]], atol=0.05)
        assert not lost, "a key outside the window was seen"
    # the same two queries as single-token steps of two sequences that share the pages
    table2 = setup.table_dev[[2, 2]].contiguous()
    for splits, keys in ((1, 0), (4, 96)):
        o2 = k.attention(q[-2:].reshape(2, H * hd).cuda(), setup.k, setup.v, i32([0, 1]), i32([0, 0]), i32([0, 1, 2]),
                         i32([T - 2, T - 1]), i32([0, 1]), table2, H, Hkv, hd, scale, window, splits, keys,
                         single_token=True)
        close(o2, ref, dtype, f"single-token far key, window {window}, {splits} chunks")


@pytest.mark.parametrize("H,Hkv,hd,page,window", [(32, 8, 64, 64, 0), (16, 8, 64, 128, 0), (6, 2, 128, 64, 0),
                                                  (16, 1, 64, 64, 0), (3, 3, 64, 64, 0), (8, 2, 64, 64, 100),
                                                  (5, 1, 128, 64, 70)])
def test_single_token_attention_on_tensor_cores(k, H, Hkv, hd, page, window):
    """The tensor-core single-token kernel against whole-sequence references: lengths around tile,
    page and chunk edges, shuffled NaN-filled pages, one far key that must win (scaled so that
    its score stands out), a window whose edge cuts a tile, and key chunks with empty ones."""
    dtype = torch.bfloat16
    assert k.attention_plan(dtype, H, Hkv, hd, page, True)[0] == "single_token_tc"
    lens = [1, 63, 64, 65, 127, 300, 1029, 512]
    slots = [3, 0, 5, 1, 4, 7, 2, 6]
    scale = 1 / math.sqrt(hd)
    setup = PagedSetup(lens, slots, 8, page, Hkv, hd, dtype, seed=5)
    g = H // Hkv
    qs, refs = [], []
    for i, (L, slot) in enumerate(zip(lens, slots)):
        kk = rnd((L, Hkv, hd), 10 + i, dtype, 0.3)
        v = rnd((L, Hkv, hd), 30 + i, dtype)
        q = rnd((1, H, hd), 50 + i, dtype, 0.3)
        far = 0 if window == 0 else max(L - window, 0)        # the first key the query may see
        if L > 3:
            kk[far] = 0
            kk[far, :, 0] = 12.0
            q[:, :, 0] = 12.0
            if window and far > 0:
                kk[far - 1] = 0
                kk[far - 1, :, 0] = 14.0      # one position outside the window: would win if it were seen
        pages = torch.from_numpy(setup.table[slot, :-(-L // page)].astype(np.int64)).cuda()
        pad = (-L) % page
        kp = torch.cat([kk, torch.zeros(pad, Hkv, hd, dtype=dtype)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
        vp = torch.cat([v, torch.zeros(pad, Hkv, hd, dtype=dtype)]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3)
        setup.k[pages] = kp.cuda()
        setup.v[pages] = vp.cuda()
        if pad:      # what lies behind the sequence's end in its last page must not matter
            setup.k[pages[-1], :, page - pad:] = float("nan")
            setup.v[pages[-1], :, page - pad:] = float("nan")
        qs.append(q.reshape(1, H * hd))
        refs.append(attn_ref(q.double(), kk.double(), v.double(), L - 1, window, scale).reshape(1, H * hd))
        if L > 3:
            won = torch.allclose(refs[-1].float().reshape(H, hd), v[far].float()[[h // g for h in range(H)]], atol=0.05)
            assert won, "the reference itself does not pick the far key"
    q_all, ref = torch.cat(qs).cuda(), torch.cat(refs)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    n = len(lens)
    for splits, keys in ((1, 0), (3, 384), (9, 128), (2, 1024)):
        out = k.attention(q_all, setup.k, setup.v, i32(list(range(n))), i32([0] * n), i32(list(range(n + 1))),
                          i32([L - 1 for L in lens]), i32(slots), setup.table_dev, H, Hkv, hd, scale, window, splits,
                          keys, single_token=True, kind="single_token_tc")
        assert not torch.isnan(out.float()).any()
        close(out, ref, dtype, f"tensor-core single-token attention, {splits} chunks of {keys}")
    if k.attention_plan(dtype, H, Hkv, hd, 32, True)[0] == "single_token":
        other = k.attention(q_all, setup.k, setup.v, i32(list(range(n))), i32([0] * n), i32(list(range(n + 1))),
                            i32([L - 1 for L in lens]), i32(slots), setup.table_dev, H, Hkv, hd, scale, window, 3, 384,
                            single_token=True, kind="single_token")
        close(other, ref, dtype, "the one-lane-per-key kernel on the same cache")


def test_size_predicates_known_to_python_agree_with_the_libraries(k):
    """`kernels._may_take` lets a model skip compiling a library that cannot serve it; it must never
    say no where the library says yes."""
    libs = {"attention_decode": "zk_attn_decode_takes", "attention_decode_tc": "zk_attn_decode_tc_takes",
            "attention_prefill": "zk_attn_prefill_takes"}
    for lib, fn in libs.items():
        for H, Hkv in ((4, 2), (3, 1), (32, 8), (16, 1), (24, 1), (9, 1), (5, 5)):
            for hd in (16, 32, 48, 64, 80, 96, 128, 256):
                for page in (16, 32, 64, 96, 128):
                    assert bool(k._fn(lib, fn)(H, Hkv, hd, page)) == k._may_take(lib, H, Hkv, hd, page), (lib, H, Hkv, hd, page)


@pytest.mark.parametrize("H,Hkv,page", [(32, 8, 64), (6, 2, 128), (16, 1, 64), (5, 5, 64)])
def test_tcgen05_prompt_attention_far_key_and_continued_prompt(k, H, Hkv, page):
    """The tcgen05 prompt kernel on a prompt cut in two steps (the second continues at position
    500 and ends in the middle of a key tile), with one far key that must win for every query
    that sees it, NaN in every cache row that no token has written, and a second short sequence
    in the same batch."""
    from zinfer_b200.parts.attention import query_tiles as attn_tiles_host
    dtype, hd = torch.bfloat16, 64
    assert k.attention_plan(dtype, H, Hkv, hd, page, False)[0] == "prompt_tc5"
    T, cut, far = 731, 500, 37
    scale = 1 / math.sqrt(hd)
    kk = rnd((T, Hkv, hd), 1, dtype, 0.3)
    v = rnd((T, Hkv, hd), 2, dtype)
    q = rnd((T, H, hd), 3, dtype, 0.3)
    kk[far] = 0
    kk[far, :, 0] = 12.0
    q[:, :, 0] = 12.0
    k2, v2, q2 = rnd((9, Hkv, hd), 4, dtype, 0.3), rnd((9, Hkv, hd), 5, dtype), rnd((9, H, hd), 6, dtype, 0.3)
    setup = PagedSetup([T, 9], [2, 0], 4, page, Hkv, hd, dtype, seed=3)
    for slot, (kx, vx) in ((2, (kk, v)), (0, (k2, v2))):
        n = kx.shape[0]
        pages = torch.from_numpy(setup.table[slot, :-(-n // page)].astype(np.int64)).cuda()
        pad = (-n) % page
        fill = torch.full((pad, Hkv, hd), float("nan"), dtype=dtype)
        setup.k[pages] = torch.cat([kx, fill]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3).cuda()
        setup.v[pages] = torch.cat([vx, fill]).reshape(-1, page, Hkv, hd).permute(0, 2, 1, 3).cuda()
    bq = k._fn("attention_prefill_tc5", "zk_attn_prefill_tc5_tile_tokens")(H, Hkv)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    g = H // Hkv
    ref1 = attn_ref(q.double(), kk.double(), v.double(), 0, 0, scale)
    ref2 = attn_ref(q2.double(), k2.double(), v2.double(), 0, 0, scale)
    # step 1: the first 500 tokens of the long sequence and the whole short one
    lens, starts = [cut, 9], [0, 0]
    tiles = torch.from_numpy(attn_tiles_host(lens, bq)).cuda()
    rows = torch.cat([q[:cut].reshape(cut, H * hd), q2.reshape(9, H * hd)]).cuda()
    out = k.attention(rows, setup.k, setup.v, tiles[0].contiguous(), tiles[1].contiguous(), i32([0, cut, cut + 9]),
                      i32(starts), i32([2, 0]), setup.table_dev, H, Hkv, hd, scale, kind="prompt_tc5")
    assert k.status_word("cuda").item() == 0 and not torch.isnan(out.float()).any()
    close(out[:cut], ref1[:cut].reshape(cut, H * hd), dtype, "first step of the long prompt")
    close(out[cut:], ref2.reshape(9, H * hd), dtype, "the short prompt beside it")
    # step 2: the long sequence goes on at position 500
    n2 = T - cut
    tiles = torch.from_numpy(attn_tiles_host([n2], bq)).cuda()
    out2 = k.attention(q[cut:].reshape(n2, H * hd).cuda(), setup.k, setup.v, tiles[0].contiguous(), tiles[1].contiguous(),
                       i32([0, n2]), i32([cut]), i32([2]), setup.table_dev, H, Hkv, hd, scale, kind="prompt_tc5")
    assert k.status_word("cuda").item() == 0 and not torch.isnan(out2.float()).any()
    close(out2, ref1[cut:].reshape(n2, H * hd), dtype, "continued prompt")
    winner = v[far].float()[[h // g for h in range(H)]]
    for t in (far, far + 1, cut - 1):
        assert torch.allclose(out[t].float().cpu().reshape(H, hd), winner, atol=0.05), f"query {t} did not pick the far key"
    assert torch.allclose(out2[-1].float().cpu().reshape(H, hd), winner, atol=0.05)
    assert not torch.allclose(out[far - 1].float().cpu().reshape(H, hd), winner, atol=0.05), "a later key was seen"


# ------------------------------------------------------------------------------- dependent launches

@pytest.mark.parametrize("rows", [1, 8, 40, 300])
def test_dependent_launches_keep_the_order_of_a_chain(k, rows):
    """The kernels of a step start while the kernel before them still runs and wait for it by
    themselves.  A chain in which every kernel reads what the one before wrote and overwrites what the
    one before read (norm -> contraction with a fused norm -> contraction that adds into the stream),
    launched back to back, gives the same bits as the chain with the device drained after every
    kernel, where nothing can overlap; 1 and 8 rows take the few-row kernels, 40 the tcgen05 kernel
    for few rows, 300 the persistent pairs with their TMA reduce-add."""
    from zinfer_b200.parts.linear import NormedRows, linear
    D, F, eps = 1024, 2048, 1e-5
    up = rnd((F, D), 61, torch.bfloat16, 0.03).cuda()
    down = rnd((D, F), 62, torch.bfloat16, 0.03).cuda()
    nw = (1.0 + rnd((D,), 63, torch.float32, 0.1)).cuda()
    x0 = rnd((rows, D), 64, torch.float32).cuda()

    def chain(drain):
        x = x0.clone()
        torch.cuda.synchronize()
        for _ in range(24):
            h = linear(NormedRows(x, nw, eps, torch.bfloat16), up)       # reads x
            if drain:
                torch.cuda.synchronize()
            linear(h, down, out=x, accumulate=True)                      # writes x, which the kernel before read
            if drain:
                torch.cuda.synchronize()
            xn = k.rmsnorm(x, nw, eps, torch.bfloat16)                   # reads x again
            if drain:
                torch.cuda.synchronize()
            linear(xn, up, out=h)                                        # overwrites h, which a kernel before read
            if drain:
                torch.cuda.synchronize()
            linear(h, down, out=x, accumulate=True)
            if drain:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return x

    a, b = chain(False), chain(True)
    assert torch.isfinite(a).all() and a.abs().max() > 0
    assert torch.equal(a, b)
    assert k.status_word("cuda").item() == 0
