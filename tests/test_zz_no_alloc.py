"""The entry point that allocates nothing (csrc/attention_decode_noalloc.h), called through its
exported C symbol: calls in a row with different batches must equal the regular, allocating
entry point and a float64 evaluation of the same attention on the host, row by row; the device
memory in use is the same before and after a call; a call too large for the built-in scratch is
refused with a message.

Who needs it: a host that cannot call cudaMalloc when attention has to run -- in a real-time
loop that must not take the allocator's lock, or after its memory budget has been closed."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE, EINVAL = -7, -22


@pytest.fixture(scope="module")
def lib():
    from zinfer_b200 import kernels
    from zinfer_b200.csrc.build import load_library
    kernels.require_cuda()
    lib = load_library("attention_decode_noalloc")
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.zk_attn_decode_noalloc.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P]
    lib.zk_attn_decode_noalloc.restype = I
    lib.zk_attn_decode_noalloc_bytes.argtypes = [I, I, I, I]
    lib.zk_attn_decode_noalloc_bytes.restype = ctypes.c_longlong
    lib.zk_attn_decode_noalloc_error.argtypes = []
    lib.zk_attn_decode_noalloc_error.restype = ctypes.c_char_p
    return lib


def make_case(seed, lens, H, Hkv, hd, page):
    """Random q and a shuffled paged cache holding `lens[b]` keys for sequence b."""
    g = torch.Generator().manual_seed(seed)
    B = len(lens)
    pages_per = [-(-l // page) for l in lens]
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages, generator=g).tolist()
    table = np.full((B + 1, max(pages_per)), -1, dtype=np.int32)
    slots = torch.randperm(B + 1, generator=g)[:B].tolist()
    it = iter(perm)
    for s, n in zip(slots, pages_per):
        for i in range(n):
            table[s, i] = next(it)
    k = (torch.randn(n_pages, Hkv, page, hd, generator=g) * 0.5).bfloat16().cuda()
    v = torch.randn(n_pages, Hkv, page, hd, generator=g).bfloat16().cuda()
    q = (torch.randn(B, H * hd, generator=g) * 0.5).bfloat16().cuda()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    return dict(q=q, k=k, v=v, table=torch.from_numpy(table).cuda(), seq_start=i32([l - 1 for l in lens]),
                seq_slot=i32(slots), B=B)


def call(lib, c, H, Hkv, hd, page, window, scale, splits, keys):
    out = torch.empty_like(c["q"])
    rc = lib.zk_attn_decode_noalloc(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), out.data_ptr(),
                                    c["seq_start"].data_ptr(), c["seq_slot"].data_ptr(), c["table"].data_ptr(),
                                    c["table"].stride(0), c["B"], H, Hkv, hd, page, window, scale, splits, keys,
                                    torch.cuda.current_stream().cuda_stream)
    return rc, out


def regular(c, H, Hkv, hd, window, scale, splits, keys):
    from zinfer_b200 import kernels
    B = c["B"]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32).cuda()
    return kernels.attention(c["q"], c["k"], c["v"], i32(list(range(B))), i32([0] * B), i32(list(range(B + 1))),
                             c["seq_start"], c["seq_slot"], c["table"], H, Hkv, hd, scale, window, splits, keys,
                             single_token=True)


def exact(c, lens, H, Hkv, hd, page, window, scale):
    """The same attention in float64 on the host: row b of the result is sequence b's [H * hd]."""
    q, k, v = c["q"].double().cpu(), c["k"].double().cpu(), c["v"].double().cpu()
    table, slots = c["table"].cpu(), c["seq_slot"].cpu().tolist()
    out = torch.zeros(len(lens), H * hd, dtype=torch.float64)
    for b, L in enumerate(lens):
        pages = table[slots[b], :-(-L // page)].long()
        lo = max(0, L - window) if window > 0 else 0
        for h in range(H):
            keys = k[pages, h // (H // Hkv)].reshape(-1, hd)[lo:L]
            vals = v[pages, h // (H // Hkv)].reshape(-1, hd)[lo:L]
            p = torch.softmax(keys @ q[b, h * hd:(h + 1) * hd] * scale, dim=0)
            out[b, h * hd:(h + 1) * hd] = p @ vals
    return out


def test_calls_in_a_row_equal_the_allocating_entry_point_and_float64(lib):
    H, Hkv, hd, page = 32, 8, 64, 64
    scale = hd ** -0.5
    cases = [([700, 33, 1500, 64, 1], 0, 6, 256),
             ([90, 300], 128, 3, 128),          # smaller: stale partials of the call before lie behind it
             ([257], 0, 1, 0)]                  # one chunk: no scratch at all
    for seed, (lens, window, splits, keys) in enumerate(cases):
        c = make_case(seed + 1, lens, H, Hkv, hd, page)
        ref = regular(c, H, Hkv, hd, window, scale, splits, keys)
        f64 = exact(c, lens, H, Hkv, hd, page, window, scale)
        torch.cuda.synchronize()
        out = torch.empty_like(c["q"])                 # the caller's output; counted before the call
        in_use = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
        rc = lib.zk_attn_decode_noalloc(c["q"].data_ptr(), c["k"].data_ptr(), c["v"].data_ptr(), out.data_ptr(),
                                        c["seq_start"].data_ptr(), c["seq_slot"].data_ptr(), c["table"].data_ptr(),
                                        c["table"].stride(0), c["B"], H, Hkv, hd, page, window, scale, splits, keys,
                                        torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert rc == 0, lib.zk_attn_decode_noalloc_error().decode()
        if seed > 0:       # the first call on a device may load the library's kernels
            assert (torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]) == in_use, "the call changed the memory in use"
        assert torch.isfinite(out.float()).all()
        # row by row: a long sequence's output is an average of many values and much smaller than
        # a short one's, so each row is measured against its own size
        for b in range(len(lens)):
            for name, want in (("the allocating entry point", ref[b].double().cpu()), ("float64", f64[b])):
                err = (out[b].double().cpu() - want).abs().max().item() / want.abs().max().item()
                assert err <= 1.5e-2, f"sequence {b} of {lens}, window {window}, {splits} chunks, against {name}: error {err:.3e}"


def test_sizes_beyond_the_scratch_are_refused_with_a_message(lib):
    H, Hkv, hd, page = 32, 8, 64, 64
    assert lib.zk_attn_decode_noalloc_bytes(5, H, hd, 6) == 6 * 5 * H * (hd + 2) * 4
    assert lib.zk_attn_decode_noalloc_bytes(5, H, hd, 1) == 0
    c = make_case(4, [40] * 64, H, Hkv, hd, page)
    rc, _ = call(lib, c, H, Hkv, hd, page, 0, 0.125, 64, 32)           # 64 x 64 x 32 x 66 x 4 bytes = 34 MB
    msg = lib.zk_attn_decode_noalloc_error().decode()
    assert rc == TOO_LARGE and "bytes of scratch" in msg and "8388608" in msg
    rc, _ = call(lib, c, H, Hkv, hd, page, 0, 0.125, 2, 48)            # chunk size not a multiple of 32
    assert rc == EINVAL and "multiples of 32" in lib.zk_attn_decode_noalloc_error().decode()
    rc, out = call(lib, c, H, Hkv, hd, page, 0, 0.125, 2, 32)          # and the library still works
    assert rc == 0 and lib.zk_attn_decode_noalloc_error().decode() == ""
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
