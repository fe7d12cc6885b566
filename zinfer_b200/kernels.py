"""Python face of the hand-written sm_100a kernels in `csrc/`.

Every function checks its tensors (device, dtype, layout, sizes), launches one kernel on the
current CUDA stream through the library's C entry point and raises `KernelError` if the
launcher refuses the sizes or CUDA reports an error.  There is no other implementation behind
these functions: without a CUDA device, a compiler or a loadable library they raise.
"""
from __future__ import annotations

import ctypes
import functools
from typing import Optional

import torch

from .csrc.build import KernelBuildError, load_library

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_C = {"p": ctypes.c_void_p, "i": ctypes.c_int, "f": ctypes.c_float, "l": ctypes.c_longlong}

# library -> function -> argument kinds (p pointer, i int, f float, l long long); the last
# pointer of every launcher is the stream
_SIGNATURES = {
    "elementwise": {
        "zk_embed": "pppiiifipp",
        "zk_rmsnorm": "ppppiifip",
        "zk_silu_mul": "ppiiiip",
        "zk_fill_normal": "pllffip",
    },
    "gemm_simt": {
        "zk_gemm_simt": "ppppiiiiiiiiip",
    },
    "gemm_skinny": {
        "zk_gemm_skinny": "pppfpppiiiiiiii" + "pippp" + "p",
        "zk_gemm_skinny_swiglu": "pppfppiiiiii" + "pi" + "p",
        "zk_gemm_skinny_conv": "pppfppppppp" + "iiiiiiil" + "pi" + "p",
        "zk_gemm_skinny_max_m": "",
        "zk_gemm_skinny_fused_max_m": "",
    },
    "gemm_tc": {
        "zk_gemm_tc": "ppppiiiiiiiiii" + "pifppp" + "pp",
        "zk_gemm_tc_force_form": "i",
    },
    "shortconv": {
        "zk_conv_forward": "ppppppppiiiliip",
        "zk_conv_state_update": "ppppiiiliip",
        "zk_conv_decode": "ppppppiiiliip",
    },
    "attention_decode": {
        "zk_attn_decode": "ppppppppp" + "iiiiiiifiip",
        "zk_attn_decode_takes": "iiii",
    },
    "attention_decode_noalloc": {      # for C callers that must not allocate; see csrc/attention_decode_noalloc.h
        "zk_attn_decode_noalloc": "ppppppp" + "iiiiiiifiip",
        "zk_attn_decode_noalloc_bytes": "iiii",
    },
    "attention_prefill": {
        "zk_attn_prefill": "pppppppppp" + "iiiiiiifp",
        "zk_attn_prefill_takes": "iiii",
        "zk_attn_prefill_tile_tokens": "ii",
    },
    "attention_prefill_tc5": {
        "zk_attn_prefill_tc5": "pppppppppp" + "iii" + "l" + "iiii" + "f" + "pp",
        "zk_attn_prefill_tc5_takes": "iiiii",
        "zk_attn_prefill_tc5_tile_tokens": "ii",
    },
    "attention_decode_tc": {
        "zk_attn_decode_tc": "pppppppppiiiiiiifiip",
        "zk_attn_decode_tc_takes": "iiii",
    },
    "sampling": {
        "zk_apply_penalties": "piipifppip",
        "zk_recent_window": "",
        "zk_penalize_recent": "piipppfp",
        "zk_recent_append": "pipppp",
        "zk_argmax": "piipppp" + "pip" + "p",
        "zk_sample": "piififfffip" + "lpp" + "pp",
    },
    "attention": {
        "zk_qk_prepare": "pppppppppppp" + "iiiiiiifiiipp",
        "zk_attn_fwd": "pppppp" + "pppppp" + "iiiiiiiifiiiiip",
        "zk_attn_merge": "pppiiiip",
        "zk_attn_rows_per_block": "",
        "zk_attn_max_head_dim": "",
    },
}


_RESTYPES = {"zk_attn_decode_noalloc_bytes": ctypes.c_longlong}


class KernelError(RuntimeError):
    """A kernel refused its arguments or CUDA reported a failure."""


_funcs: dict[str, object] = {}


def _fn(lib_name: str, fn_name: str):
    f = _funcs.get(fn_name)
    if f is None:
        lib = load_library(lib_name)
        for name, sig in _SIGNATURES[lib_name].items():
            g = getattr(lib, name)
            g.argtypes = [_C[c] for c in sig]
            g.restype = _RESTYPES.get(name, ctypes.c_int)
            _funcs[name] = g
        f = _funcs[fn_name]
    return f


def _error_name(code: int) -> str:
    lib = load_library("elementwise")
    lib.zk_error_name.argtypes = [ctypes.c_int]
    lib.zk_error_name.restype = ctypes.c_char_p
    s = lib.zk_error_name(code)
    return s.decode() if s else f"status {code}"


# Number of kernel launches made through this module since import (the benchmark reports it).
launch_count = 0

_device_state: dict = {}


def _check(code: int, what: str) -> None:
    global launch_count
    if code != 0:
        raise KernelError(f"{what}: {_error_name(code)} (status {code})")
    launch_count += 1


def require_cuda() -> None:
    """Raises unless a CUDA device is usable; the product path has no CPU implementation."""
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device: zinfer_b200 runs on sm_100a GPUs only and has no CPU path")


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device; launch plans size their grids by it."""
    dev = torch.device("cuda" if device is None else device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    n = _device_state.setdefault(("sm_count", idx), None)
    if n is None:
        n = _device_state[("sm_count", idx)] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


# The current stream's handle, asked for at every launch.  torch.cuda.current_stream() builds a Stream
# object each time (some 5 us, a fifth of the host's time per launch of an unrecorded step); the
# raw getter behind it returns the handle itself.  Where a torch build lacks it the public call does.
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None, contiguous=True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor")
    if dtype is not None:
        ok = t.dtype in dtype if isinstance(dtype, (tuple, list)) else t.dtype == dtype
        if not ok:
            raise KernelError(f"{name}: dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if shape is not None:
        if t.dim() != len(shape) or any(s is not None and s != d for s, d in zip(shape, t.shape)):
            raise KernelError(f"{name}: shape {tuple(t.shape)}, expected {tuple(shape)}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DT[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not a run dtype (float32, bfloat16)") from None


# ------------------------------------------------------------------------------- row kernels

def embed(tokens: torch.Tensor, table: torch.Tensor, status: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """x[t] = float32(table[tokens[t]]) * scale; bad ids set status to 1."""
    _need(tokens, "tokens", torch.int32)
    _need(table, "table", (torch.float32, torch.bfloat16), (None, None))
    _need(status, "status", torch.int32)
    n, (vocab, dim) = tokens.numel(), table.shape
    x = torch.empty((n, dim), dtype=torch.float32, device=table.device)
    _check(_fn("elementwise", "zk_embed")(_ptr(tokens), _ptr(table), _ptr(x), n, dim, vocab, scale,
                                          dtype_code(table.dtype), _ptr(status), _stream()), "embed")
    return x


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm of float32 rows (all, or those listed in `rows`) into `out_dtype`."""
    _need(x, "x", torch.float32, (None, None))
    dim = x.shape[1]
    _need(weight, "weight", torch.float32, (dim,))
    n_out = x.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n_out = rows.numel()
    y = torch.empty((n_out, dim), dtype=out_dtype, device=x.device)
    _check(_fn("elementwise", "zk_rmsnorm")(_ptr(x), _ptr(rows), _ptr(weight), _ptr(y), n_out, dim, eps,
                                            dtype_code(out_dtype), _stream()), "rmsnorm")
    return y


def silu_mul(gu: torch.Tensor, interleave: int = 0) -> torch.Tensor:
    """h = silu(gate) * up.  A row of gu is [gate (F) | up (F)], or with `interleave` = g groups of
    g gates followed by their g ups."""
    _need(gu, "gu", (torch.float32, torch.bfloat16), (None, None))
    n, two_f = gu.shape
    if two_f % 2 or (interleave and (two_f // 2) % interleave):
        raise KernelError(f"silu_mul: width {two_f} does not split into gate and up (groups of {interleave})")
    h = torch.empty((n, two_f // 2), dtype=gu.dtype, device=gu.device)
    _check(_fn("elementwise", "zk_silu_mul")(_ptr(gu), _ptr(h), n, two_f // 2, interleave, dtype_code(gu.dtype),
                                             _stream()), "silu_mul")
    return h


def fill_normal(out: torch.Tensor, seed: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    """Fills `out` with mean + std * N(0, 1), a function of (seed, element index) only."""
    _need(out, "out", (torch.float32, torch.bfloat16))
    _check(_fn("elementwise", "zk_fill_normal")(_ptr(out), out.numel(), seed & 0x7FFFFFFFFFFFFFFF, mean, std,
                                                dtype_code(out.dtype), _stream()), "fill_normal")
    return out


# ------------------------------------------------------------------------------- contractions

def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
              accumulate: bool = False, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) with float32 FMA on the CUDA cores.  a [M, K], w [N, K] share a
    dtype; out is that dtype or float32; accumulate needs a float32 or same-dtype `out`."""
    _need(a, "a", (torch.float32, torch.bfloat16), (None, None))
    _need(w, "w", a.dtype, (None, a.shape[1]))
    M, K = a.shape
    N = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    _need(out, "out", (torch.float32, a.dtype), (M, N))
    if a.dtype == torch.float32 and out.dtype != torch.float32:
        raise KernelError("gemm: float32 inputs need a float32 output")
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    _check(_fn("gemm_simt", "zk_gemm_simt")(_ptr(a), _ptr(w), _ptr(out), _ptr(bias), M, N, K, a.stride(0), w.stride(0),
                                            out.stride(0), dtype_code(a.dtype), dtype_code(out.dtype),
                                            1 if accumulate else 0, _stream()), "gemm_simt")
    return out


def status_word(device) -> torch.Tensor:
    """The int32 status word of a device: kernels that can detect a fault of their inputs or give
    up a bounded wait write a code here; `Engine.check_status` reads and clears it."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    st = _device_state.setdefault(dev, {})
    if "status" not in st:
        st["status"] = torch.zeros(1, dtype=torch.int32, device=dev)
    return st["status"]


GEMM_TC_SWAPPED_MAX_M = 64     # up to this many rows the weights take the 128-row side of the tiles


def gemm_tc_takes(a, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> bool:
    """Whether the tcgen05 kernel takes this contraction: bfloat16, K a multiple of 8, rows and
    output 16-byte aligned.  `a` is a bfloat16 tensor, or a ScaledInput of up to 64 rows."""
    if isinstance(a, ScaledInput):
        if a.xw.shape[0] > GEMM_TC_SWAPPED_MAX_M or not a.ssq.is_contiguous():
            return False
        a = a.xw
    ok = (isinstance(a, torch.Tensor) and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.dim() == 2
          and w.dim() == 2 and a.shape[1] == w.shape[1] and a.shape[1] % 8 == 0 and a.stride(1) == 1
          and w.stride(1) == 1 and a.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0
          and w.data_ptr() % 16 == 0 and w.shape[0] <= 4096 * 128)
    if ok and out is not None:
        ok = out.stride(1) == 1 and out.data_ptr() % 16 == 0
    return ok


def gemm_tc_emits(a, out: Optional[torch.Tensor]) -> bool:
    """Whether `gemm_tc` can write a NormEmit beside `out` for this input."""
    return (a.shape[0] <= GEMM_TC_SWAPPED_MAX_M and out is not None and out.dtype == torch.float32
            and out.is_contiguous())


def gemm_tc(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
            accumulate: bool = False, bias: Optional[torch.Tensor] = None, splits: int = 1,
            swiglu: bool = False, emit: Optional["NormEmit"] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) with TMA-fed tcgen05 MMAs and the accumulator in tensor memory.
    More than 64 rows: persistent blocks on 256-wide tiles when N is a multiple of 256 (pairs of
    blocks with tcgen05.mma.cta_group::2 above 128 rows, TMA stores), else one 128 x 128 tile of
    tokens x weight rows per block.  Up to 64 rows: the weights take
    the 128-row side and K is cut into `splits` (1, 2, 4 or 8) parts, one per block of a cluster,
    that are added in order.  With `swiglu` w holds groups of 16 gate rows and
    their 16 up rows and the result is silu(gate) * up, [M, N/2].  Up to 64 rows `a` may be a
    ScaledInput (the sums are scaled by the rows' 1/rms) and `emit` (see `gemm_tc_emits`) is filled
    for the norm that reads `out` next."""
    if not gemm_tc_takes(a, w, out):
        raise KernelError(f"gemm_tc: a {tuple(a.shape)} / w {tuple(w.shape)} need bfloat16, K a multiple of 8 and "
                          "16-byte aligned rows")
    ssq, ssq_parts, eps = None, 0, 0.0
    if isinstance(a, ScaledInput):
        ssq, ssq_parts, eps, a = _ptr(a.ssq), a.ssq.shape[1], a.eps, a.xw
    M, K = a.shape
    N = w.shape[0]
    if swiglu and (N % 32 or accumulate or bias is not None):
        raise KernelError("gemm_tc: the SwiGLU epilogue needs N a multiple of 32, no bias and no accumulation")
    n_out = N // 2 if swiglu else N
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
    _need(out, "out", (torch.float32, torch.bfloat16), (M, n_out))
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    if emit is not None:
        if not gemm_tc_emits(a, out) or swiglu:
            raise KernelError("gemm_tc: the norm's inputs are written for at most 64 rows summed into contiguous "
                              "float32 rows")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        emit.xw = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
        emit.ssq = torch.empty((M, -(-N // 32)), dtype=torch.float32, device=w.device)
    _check(_fn("gemm_tc", "zk_gemm_tc")(_ptr(a), _ptr(w), _ptr(out), _ptr(bias), M, N, K, a.stride(0), w.stride(0),
                                        out.stride(0), dtype_code(out.dtype), 1 if accumulate else 0, splits,
                                        1 if swiglu else 0, ssq, ssq_parts, eps,
                                        _ptr(emit.weight) if emit else None, _ptr(emit.xw) if emit else None,
                                        _ptr(emit.ssq) if emit else None, _ptr(status_word(a.device)), _stream()),
           "gemm_tc")
    return out


def gemm_tc_force_form(form: int) -> None:
    """For measurements and tests: the form that products of more than 64 rows with N a multiple of
    256 take.  0 = one 128 x 128 tile per block, 256 = persistent blocks with 128 x 256 tiles, 512 =
    persistent pairs of blocks with 256 x 256 tiles (tcgen05.mma.cta_group::2); -1 = the library chooses."""
    _check(_fn("gemm_tc", "zk_gemm_tc_force_form")(int(form)), "gemm_tc_force_form")


_constants: dict[str, int] = {}     # what the libraries say about themselves, asked once


def _constant(lib_name: str, fn_name: str) -> int:
    v = _constants.get(fn_name)
    if v is None:
        v = _constants[fn_name] = _fn(lib_name, fn_name)()
    return v


def gemm_skinny_max_m() -> int:
    return _constant("gemm_skinny", "zk_gemm_skinny_max_m")


def gemm_skinny_fused_max_m() -> int:
    """Most rows for which the skinny kernels fuse RMSNorm, SwiGLU or the short convolution."""
    return _constant("gemm_skinny", "zk_gemm_skinny_fused_max_m")


class NormInput:
    """Rows of the float32 residual stream with an RMSNorm still to be applied: x [M, K], weight
    [K], eps.  The skinny kernels take it in place of a bfloat16 input and normalise themselves."""

    def __init__(self, x: torch.Tensor, weight: torch.Tensor, eps: float):
        _need(x, "x", torch.float32, (None, None))
        _need(weight, "norm weight", torch.float32, (x.shape[1],))
        self.x, self.weight, self.eps = x, weight, float(eps)

    @property
    def shape(self):
        return self.x.shape


class ScaledInput:
    """Rows of the residual stream as the kernel that summed them left them for the next RMSNorm:
    xw [M, K] = bfloat16(x * norm weight) and ssq [M, parts] float32, partial sums of x^2 whose
    sum over `parts` is the row's.  The skinny kernels take it in place of a bfloat16 input and
    scale their sums by 1 / sqrt(sum(ssq) / K + eps)."""

    def __init__(self, xw: torch.Tensor, ssq: torch.Tensor, eps: float):
        _need(xw, "xw", torch.bfloat16, (None, None))
        _need(ssq, "ssq", torch.float32, (xw.shape[0], None))
        self.xw, self.ssq, self.eps = xw, ssq, float(eps)

    @property
    def shape(self):
        return self.xw.shape


class NormEmit:
    """What an accumulating contraction into the residual rows writes for the norm that reads them
    next: `weight` [N] of that norm; after the call `xw` [M, N] = bfloat16(rows * weight) and `ssq`
    [M, parts], partial sums of the rows' squares (how many parts is the kernel's business)."""

    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.xw: Optional[torch.Tensor] = None
        self.ssq: Optional[torch.Tensor] = None


GEMM_SKINNY_EMIT_MAX_M = 16


def _skinny_input(a):
    """(X pointer, Xf pointer, norm weight pointer, eps, M, K, ldx, ssq pointer, ssq parts) of a
    bfloat16 tensor, a NormInput or a ScaledInput."""
    if isinstance(a, NormInput):
        return None, _ptr(a.x), _ptr(a.weight), a.eps, a.x.shape[0], a.x.shape[1], a.x.stride(0), None, 0
    if isinstance(a, ScaledInput):
        return _ptr(a.xw), None, None, a.eps, a.xw.shape[0], a.xw.shape[1], a.xw.stride(0), _ptr(a.ssq), a.ssq.shape[1]
    return _ptr(a), None, None, 0.0, a.shape[0], a.shape[1], a.stride(0), None, 0


def gemm_skinny_takes(a, w: torch.Tensor) -> bool:
    """Whether the skinny kernels take this contraction: bfloat16 weights, few rows, 16-byte
    aligned rows.  `a` is a bfloat16 tensor [M <= 64, K], a NormInput or a ScaledInput [M <= 16, K]."""
    if not (w.dtype == torch.bfloat16 and w.dim() == 2 and w.stride(1) == 1 and w.stride(0) % 8 == 0
            and w.data_ptr() % 16 == 0 and w.shape[1] % 8 == 0):
        return False
    if isinstance(a, NormInput):
        x = a.x
        return (x.shape[0] <= gemm_skinny_fused_max_m() and x.shape[1] == w.shape[1] and x.stride(1) == 1
                and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0 and a.weight.data_ptr() % 16 == 0)
    if isinstance(a, ScaledInput):
        if a.xw.shape[0] > gemm_skinny_fused_max_m() or not a.ssq.is_contiguous():
            return False
        a = a.xw
    return (a.dtype == torch.bfloat16 and a.dim() == 2 and a.shape[0] <= gemm_skinny_max_m()
            and a.shape[1] == w.shape[1] and a.stride(1) == 1 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0)


def gemm_skinny_fused_takes(a, w: torch.Tensor) -> bool:
    """Whether the fused SwiGLU / short-convolution variants take this input (at most 16 rows)."""
    return gemm_skinny_takes(a, w) and a.shape[0] <= gemm_skinny_fused_max_m()


def gemm_skinny_emits(a, out: Optional[torch.Tensor]) -> bool:
    """Whether `gemm_skinny` can write a NormEmit beside `out` for this input."""
    return (isinstance(a, torch.Tensor) and a.shape[0] <= GEMM_SKINNY_EMIT_MAX_M and out is not None
            and out.dtype == torch.float32 and out.is_contiguous())


def gemm_skinny(a, w: torch.Tensor, out: Optional[torch.Tensor] = None, out_dtype=None,
                accumulate: bool = False, bias: Optional[torch.Tensor] = None,
                emit: Optional[NormEmit] = None) -> torch.Tensor:
    """out (+)= a @ w.T (+ bias) for a [M <= 64, K] on the tensor cores, every weight read once.
    With a NormInput the RMSNorm of the rows is applied inside the kernel; with a ScaledInput the
    sums are scaled by the rows' 1/rms.  `emit` (see `gemm_skinny_emits`) is filled for the norm
    that reads `out` next."""
    if not gemm_skinny_takes(a, w):
        raise KernelError(f"gemm_skinny: a {tuple(a.shape)} / w {tuple(w.shape)} need few rows, "
                          "K a multiple of 8 and 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    N = w.shape[0]
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=w.device)
    _need(out, "out", (torch.float32, torch.bfloat16), (M, N))
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    if emit is not None:
        if not gemm_skinny_emits(a, out):
            raise KernelError("gemm_skinny: the norm's inputs are written for at most 16 bfloat16 rows "
                              "summed into contiguous float32 rows")
        _need(emit.weight, "norm weight", torch.float32, (N,))
        emit.xw = torch.empty((M, N), dtype=torch.bfloat16, device=w.device)
        emit.ssq = torch.empty((M, -(-N // 16)), dtype=torch.float32, device=w.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny")(X, Xf, nw, eps, _ptr(w), _ptr(out), _ptr(bias), M, N, K, ldx,
                                                w.stride(0), out.stride(0), dtype_code(out.dtype),
                                                1 if accumulate else 0, ssq, ssq_parts,
                                                _ptr(emit.weight) if emit else None, _ptr(emit.xw) if emit else None,
                                                _ptr(emit.ssq) if emit else None, _stream()), "gemm_skinny")
    return out


def gemm_skinny_swiglu(a, w_gate_up: torch.Tensor) -> torch.Tensor:
    """h = silu(a W_gate^T) * (a W_up^T) in one kernel; w_gate_up [2F, K] holds groups of 16 gate
    rows followed by their 16 up rows."""
    if not gemm_skinny_fused_takes(a, w_gate_up) or w_gate_up.shape[0] % 32:
        raise KernelError("gemm_skinny_swiglu: at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    F = w_gate_up.shape[0] // 2
    h = torch.empty((M, F), dtype=torch.bfloat16, device=w_gate_up.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny_swiglu")(X, Xf, nw, eps, _ptr(w_gate_up), _ptr(h), M, F, K, ldx,
                                                       w_gate_up.stride(0), h.stride(0), ssq, ssq_parts,
                                                       _stream()),
           "gemm_skinny_swiglu")
    return h


def gemm_skinny_conv(a, w_in: torch.Tensor, in_bias, state: torch.Tensor, taps: torch.Tensor, conv_bias,
                     seq_slot: torch.Tensor) -> torch.Tensor:
    """Single-token step of the gated short convolution fused with its in_proj: row m of `a` is
    sequence m; `state` [slots, K-1, D] is shifted by one; returns y [M, D].  w_in [3D, K] and
    in_bias [3D] hold groups of 16 B rows, 16 C rows, 16 X rows."""
    if not gemm_skinny_fused_takes(a, w_in) or w_in.shape[0] % 48:
        raise KernelError("gemm_skinny_conv: at most 16 rows, K a multiple of 8, 16-byte aligned rows")
    X, Xf, nw, eps, M, K, ldx, ssq, ssq_parts = _skinny_input(a)
    D = w_in.shape[0] // 3
    _need(taps, "conv weight", torch.float32, (None, D))
    n_taps = taps.shape[0]
    _need(state, "conv state", torch.float32, (None, n_taps - 1, D))
    _need(seq_slot, "seq_slot", torch.int32, (M,))
    if in_bias is not None:
        _need(in_bias, "in_proj bias", torch.float32, (3 * D,))
    if conv_bias is not None:
        _need(conv_bias, "conv bias", torch.float32, (D,))
    y = torch.empty((M, D), dtype=torch.bfloat16, device=w_in.device)
    _check(_fn("gemm_skinny", "zk_gemm_skinny_conv")(X, Xf, nw, eps, _ptr(w_in), _ptr(in_bias), _ptr(state), _ptr(taps),
                                                     _ptr(conv_bias), _ptr(seq_slot), _ptr(y), M, D, K, n_taps, ldx,
                                                     w_in.stride(0), y.stride(0), state.stride(0), ssq, ssq_parts,
                                                     _stream()),
           "gemm_skinny_conv")
    return y


# ------------------------------------------------------------------------------- short convolution

def conv_forward(bcx, state, w, bias, tok_seq, cu_q, seq_slot, interleave: int = 0) -> torch.Tensor:
    """y of the gated short convolution for a packed batch; reads `state`, does not change it.
    bcx [n, 3D] = [B | C | X] (or groups of `interleave` channels as [B | C | X]); state
    [slots, K-1, D] float32; w [K, D] float32; bias [D] float32 or None."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    n, three_d = bcx.shape
    D = three_d // 3
    _need(w, "conv weight", torch.float32, (None, D))
    K = w.shape[0]
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    if bias is not None:
        _need(bias, "conv bias", torch.float32, (D,))
    for t, nm in ((tok_seq, "tok_seq"), (cu_q, "cu_q"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32)
    y = torch.empty((n, D), dtype=bcx.dtype, device=bcx.device)
    _check(_fn("shortconv", "zk_conv_forward")(_ptr(bcx), _ptr(state), _ptr(w), _ptr(bias), _ptr(tok_seq), _ptr(cu_q),
                                               _ptr(seq_slot), _ptr(y), n, D, K, state.stride(0), interleave,
                                               dtype_code(bcx.dtype), _stream()), "conv_forward")
    return y


def conv_state_update(bcx, state, cu_q, seq_slot, n_seqs: int, K: int, interleave: int = 0) -> None:
    """state[slot] <- the last K-1 values of B*X of each sequence (older rows kept if fewer came)."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    D = bcx.shape[1] // 3
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    _check(_fn("shortconv", "zk_conv_state_update")(_ptr(bcx), _ptr(state), _ptr(cu_q), _ptr(seq_slot), n_seqs, D, K,
                                                    state.stride(0), interleave, dtype_code(bcx.dtype), _stream()),
           "conv_state_update")


def conv_decode(bcx, state, w, bias, seq_slot, interleave: int = 0) -> torch.Tensor:
    """Single-token step: y and the shifted state in one kernel; row b of bcx is sequence b."""
    _need(bcx, "bcx", (torch.float32, torch.bfloat16), (None, None))
    n, three_d = bcx.shape
    D = three_d // 3
    _need(w, "conv weight", torch.float32, (None, D))
    K = w.shape[0]
    _need(state, "conv state", torch.float32, (None, K - 1, D))
    if bias is not None:
        _need(bias, "conv bias", torch.float32, (D,))
    _need(seq_slot, "seq_slot", torch.int32)
    y = torch.empty((n, D), dtype=bcx.dtype, device=bcx.device)
    _check(_fn("shortconv", "zk_conv_decode")(_ptr(bcx), _ptr(state), _ptr(w), _ptr(bias), _ptr(seq_slot), _ptr(y), n,
                                              D, K, state.stride(0), interleave, dtype_code(bcx.dtype), _stream()),
           "conv_decode")
    return y


# ------------------------------------------------------------------------------- attention

def attn_rows_per_block() -> int:
    return _constant("attention", "zk_attn_rows_per_block")


def attn_max_head_dim() -> int:
    return _constant("attention", "zk_attn_max_head_dim")


def qk_prepare(qkv, k_cache, v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot, page_table, n_heads: int,
               n_kv: int, head_dim: int, n_rot: int, interleaved: bool, eps: float, status, write_kv: bool = True):
    """Per-head RMSNorm of q and k (if weights are given), rotary encoding (if `inv_freq` is
    given), q out as [n, H*hd], and k, v written to their pages.  k_cache / v_cache are one
    layer's [pages, Hkv, page_size, hd]."""
    _need(qkv, "qkv", (torch.float32, torch.bfloat16), (None, (n_heads + 2 * n_kv) * head_dim))
    n = qkv.shape[0]
    for c, nm in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        _need(c, nm, qkv.dtype, (None, n_kv, None, head_dim))
    page_size = k_cache.shape[2]
    if head_dim % 2 or head_dim > attn_max_head_dim():
        raise KernelError(f"qk_prepare: head_dim {head_dim} must be even and <= {attn_max_head_dim()}")
    for wt, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if wt is not None:
            _need(wt, nm, torch.float32, (head_dim,))
    if inv_freq is not None:
        _need(inv_freq, "inv_freq", torch.float32, (n_rot // 2,))
    _need(page_table, "page_table", torch.int32, (None, None))
    q = torch.empty((n, n_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    _check(_fn("attention", "zk_qk_prepare")(
        _ptr(qkv), _ptr(q), None, _ptr(k_cache), _ptr(v_cache), _ptr(q_w), _ptr(k_w), _ptr(inv_freq), _ptr(tok_seq),
        _ptr(tok_pos), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, n_rot,
        1 if interleaved else 0, eps, page_size, 1 if write_kv else 0, dtype_code(qkv.dtype), _ptr(status), _stream()),
        "qk_prepare")
    return q


def qk_normed(qkv, q_w, k_w, n_heads: int, n_kv: int, head_dim: int, eps: float, tok_pos, status) -> torch.Tensor:
    """Per-head RMSNorm of the q and k heads of qkv [n, (H + 2 Hkv) * hd] into a new tensor of
    the same shape (v copied); no rotation, no cache write."""
    _need(qkv, "qkv", (torch.float32, torch.bfloat16), (None, (n_heads + 2 * n_kv) * head_dim))
    if head_dim % 2 or head_dim > attn_max_head_dim():
        raise KernelError(f"qk_normed: head_dim {head_dim} must be even and <= {attn_max_head_dim()}")
    for wt, nm in ((q_w, "q norm weight"), (k_w, "k norm weight")):
        if wt is not None:
            _need(wt, nm, torch.float32, (head_dim,))
    dense = torch.empty_like(qkv)
    _check(_fn("attention", "zk_qk_prepare")(
        _ptr(qkv), None, _ptr(dense), None, None, _ptr(q_w), _ptr(k_w), None, None, _ptr(tok_pos), None, None, 0,
        qkv.shape[0], n_heads, n_kv, head_dim, 0, 0, eps, 1, 0, dtype_code(qkv.dtype), _ptr(status), _stream()),
        "qk_normed")
    return dense


def attn_tile_shape(n_heads: int, n_kv: int) -> tuple[int, int]:
    """(tokens per query tile, heads of a KV group per block) for these head counts."""
    rows = attn_rows_per_block()
    gc = min(n_heads // n_kv, rows)
    return max(1, rows // gc), gc


def _may_take(lib: str, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    """The sizes a specialised attention library can take at all, known here so that a model it
    cannot serve never has it compiled; the library's own `*_takes` has the last word."""
    group = n_heads // n_kv
    if lib == "attention_decode":
        return head_dim in (32, 64, 96, 128) and group <= 8 and page_size % 32 == 0
    if lib == "attention_decode_tc":
        return head_dim in (64, 128) and group <= 16 and page_size % 64 == 0
    if lib == "attention_prefill":
        return head_dim in (64, 128) and page_size % 64 == 0
    if lib == "attention_prefill_tc5":
        return head_dim == 64 and page_size % 64 == 0
    raise KeyError(lib)


def _takes(lib: str, fn: str, n_heads: int, n_kv: int, head_dim: int, page_size: int) -> bool:
    return _may_take(lib, n_heads, n_kv, head_dim, page_size) and bool(_fn(lib, fn)(n_heads, n_kv, head_dim, page_size))


@functools.lru_cache(maxsize=None)      # a pure function of sizes, asked for by every attention layer of every step
def attention_plan(dtype: torch.dtype, n_heads: int, n_kv: int, head_dim: int, page_size: int,
                   single_token: bool, window: int = 0) -> tuple[str, int]:
    """Which attention kernel runs for these sizes and how many tokens its query tiles hold:
    ("single_token_tc" | "single_token" | "prompt_tc5" | "prompt_tc" | "general", tokens per tile)."""
    if dtype == torch.bfloat16 and n_heads % n_kv == 0:
        if (not single_token and window <= 0 and _may_take("attention_prefill_tc5", n_heads, n_kv, head_dim, page_size)
                and _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_takes")(n_heads, n_kv, head_dim, page_size, window)):
            return "prompt_tc5", _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_tile_tokens")(n_heads, n_kv)
        if single_token and _takes("attention_decode_tc", "zk_attn_decode_tc_takes", n_heads, n_kv, head_dim, page_size):
            return "single_token_tc", 1
        if single_token and _takes("attention_decode", "zk_attn_decode_takes", n_heads, n_kv, head_dim, page_size):
            return "single_token", 1
        if not single_token and _takes("attention_prefill", "zk_attn_prefill_takes", n_heads, n_kv, head_dim, page_size):
            return "prompt_tc", _fn("attention_prefill", "zk_attn_prefill_tile_tokens")(n_heads, n_kv)
    return "general", attn_tile_shape(n_heads, n_kv)[0]


def attention(q, k_cache, v_cache, tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table, n_heads: int, n_kv: int,
              head_dim: int, scale: float, window: int = 0, num_splits: int = 1, split_keys: int = 0,
              single_token: bool = False, kind: Optional[str] = None) -> torch.Tensor:
    """Causal grouped-query attention of a packed batch against the paged cache.  With
    num_splits > 1 the keys are cut at multiples of `split_keys` and merged afterwards.
    `single_token` says that every sequence brings exactly one query (row b = sequence b); the
    bfloat16 kernels for that case are used when they take the sizes.  `kind` names the kernel as
    `attention_plan` chose it (the tile table must then have that plan's tokens per tile);
    without it the general kernel or the single-token kernel runs."""
    _need(q, "q", (torch.float32, torch.bfloat16), (None, n_heads * head_dim))
    n = q.shape[0]
    for c, nm in ((k_cache, "k_cache"), (v_cache, "v_cache")):
        _need(c, nm, q.dtype, (None, n_kv, None, head_dim))
    page_size = k_cache.shape[2]
    if n_heads % n_kv:
        raise KernelError(f"attention: {n_heads} heads are not a multiple of {n_kv} KV heads")
    if head_dim > attn_max_head_dim():
        raise KernelError(f"attention: head_dim {head_dim} exceeds {attn_max_head_dim()}")
    bq, gc = attn_tile_shape(n_heads, n_kv)
    n_tiles = tile_seq.numel()
    out = torch.empty_like(q)
    part_o = part_ml = None
    if num_splits > 1:
        part_o = torch.empty((num_splits, n * n_heads, head_dim), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((num_splits, n * n_heads, 2), dtype=torch.float32, device=q.device)
    if kind == "prompt_tc5":
        if (q.dtype != torch.bfloat16 or window > 0 or not k_cache.is_contiguous() or not v_cache.is_contiguous()
                or not q.is_contiguous()
                or not _fn("attention_prefill_tc5", "zk_attn_prefill_tc5_takes")(n_heads, n_kv, head_dim, page_size, window)):
            raise KernelError("attention: the tcgen05 prompt kernel does not take these sizes")
        _check(_fn("attention_prefill_tc5", "zk_attn_prefill_tc5")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq), _ptr(tile_q0), _ptr(cu_q),
            _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n, k_cache.shape[0],
            n_heads, n_kv, head_dim, page_size, scale, _ptr(status_word(q.device)), _stream()),
            "attention (prompt, tcgen05)")
        return out
    if kind == "prompt_tc":
        if q.dtype != torch.bfloat16 or not _takes("attention_prefill", "zk_attn_prefill_takes", n_heads, n_kv, head_dim,
                                                   page_size):
            raise KernelError("attention: the tensor-core prompt kernel does not take these sizes")
        _check(_fn("attention_prefill", "zk_attn_prefill")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(tile_seq), _ptr(tile_q0), _ptr(cu_q),
            _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n_heads, n_kv, head_dim,
            page_size, window, scale, _stream()), "attention (prompt, tensor cores)")
        return out
    if (single_token and kind in (None, "single_token_tc") and q.dtype == torch.bfloat16
            and _takes("attention_decode_tc", "zk_attn_decode_tc_takes", n_heads, n_kv, head_dim, page_size)):
        _check(_fn("attention_decode_tc", "zk_attn_decode_tc")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(seq_start),
            _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, page_size, window,
            scale, num_splits, split_keys, _stream()), "attention (single token, tensor cores)")
        if num_splits > 1:
            _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, head_dim,
                                                     num_splits, dtype_code(q.dtype), _stream()), "attention merge")
        return out
    if kind == "single_token_tc":
        raise KernelError("attention: the tensor-core single-token kernel does not take these sizes")
    if (single_token and kind in (None, "single_token") and q.dtype == torch.bfloat16
            and _takes("attention_decode", "zk_attn_decode_takes", n_heads, n_kv, head_dim, page_size)):
        _check(_fn("attention_decode", "zk_attn_decode")(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(seq_start),
            _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n, n_heads, n_kv, head_dim, page_size, window,
            scale, num_splits, split_keys, _stream()), "attention (single token)")
        if num_splits > 1:
            _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, head_dim,
                                                     num_splits, dtype_code(q.dtype), _stream()), "attention merge")
        return out
    _check(_fn("attention", "zk_attn_fwd")(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(tile_seq), _ptr(tile_q0),
        _ptr(cu_q), _ptr(seq_start), _ptr(seq_slot), _ptr(page_table), page_table.stride(0), n_tiles, n, n_heads, n_kv,
        head_dim, page_size, window, scale, bq, gc, num_splits, split_keys, dtype_code(q.dtype), _stream()),
        "attention")
    if num_splits > 1:
        _check(_fn("attention", "zk_attn_merge")(_ptr(part_o), _ptr(part_ml), _ptr(out), n * n_heads, head_dim,
                                                 num_splits, dtype_code(q.dtype), _stream()), "attention merge")
    return out


# ------------------------------------------------------------------------------- sampling

def apply_penalties(logits, rep_tokens, rep_penalty: float, dry_tokens, dry_pen) -> None:
    """In place: repetition penalty on the listed tokens of each row ([n, R] int32, -1 = none),
    then logits[row, tok] -= pen for the DRY pairs ([n, P] int32 / float32)."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    R = P = 0
    if rep_tokens is not None:
        _need(rep_tokens, "rep_tokens", torch.int32, (n, None))
        R = rep_tokens.shape[1]
    if dry_tokens is not None:
        _need(dry_tokens, "dry_tokens", torch.int32, (n, None))
        P = dry_tokens.shape[1]
        _need(dry_pen, "dry_pen", torch.float32, (n, P))
    _check(_fn("sampling", "zk_apply_penalties")(_ptr(logits), n, V, _ptr(rep_tokens), R, rep_penalty,
                                                 _ptr(dry_tokens), _ptr(dry_pen), P, _stream()), "apply_penalties")


def recent_window() -> int:
    """How many of a request's last tokens the device's window for the repetition penalty holds."""
    return _constant("sampling", "zk_recent_window")


def penalize_recent(logits, recent, seen, req_ids, penalty: float) -> None:
    """In place: the repetition penalty (l > 0 ? l / F : l * F) on every distinct token among the last
    tokens of each row's request.  recent int32 [requests, recent_window()] is a ring per request,
    seen int32 [requests] how many tokens each has had, req_ids int32 [n] the request of each row."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    _need(recent, "recent", torch.int32, (None, recent_window()))
    _need(seen, "seen", torch.int32, (recent.shape[0],))
    _need(req_ids, "req_ids", torch.int32, (n,))
    _check(_fn("sampling", "zk_penalize_recent")(_ptr(logits), n, V, _ptr(recent), _ptr(seen), _ptr(req_ids),
                                                 float(penalty), _stream()), "penalize_recent")


def recent_append(tokens, recent, seen, req_ids) -> None:
    """tokens int32 [n], one per row, enter their requests' rings (see penalize_recent)."""
    n = tokens.shape[0]
    _need(tokens, "tokens", torch.int32, (n,))
    _need(recent, "recent", torch.int32, (None, recent_window()))
    _need(seen, "seen", torch.int32, (recent.shape[0],))
    _need(req_ids, "req_ids", torch.int32, (n,))
    _check(_fn("sampling", "zk_recent_append")(_ptr(tokens), n, _ptr(recent), _ptr(seen), _ptr(req_ids), _stream()),
           "recent_append")


def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None, feed: Optional[torch.Tensor] = None,
           status: Optional[torch.Tensor] = None, ring: Optional[torch.Tensor] = None,
           ring_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Lowest index among the largest logits of each row; int32 [n].  `out` may be given (with
    `status` it has n + 1 words and the last receives the status word's value); `feed` [n] receives
    the same indices (the next step's token slots).  `ring` int32 [slots, n + 1]: the kernel also
    writes the tokens and the status word into slot (ring_pos % slots) and adds one to `ring_pos`
    (one int32 word on the device), so that a step's result stays where it is while later steps run."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    ring_slots = 0
    if ring is not None:
        _need(ring, "ring", torch.int32, (None, n + 1))
        _need(ring_pos, "ring_pos", torch.int32, (1,))
        ring_slots = ring.shape[0]
    if out is None:
        out = torch.empty(n + (1 if status is not None else 0), dtype=torch.int32, device=logits.device)
    _need(out, "out", torch.int32, (n + (1 if status is not None else 0),))
    if feed is not None:
        _need(feed, "feed", torch.int32, (n,))
    if status is not None:
        _need(status, "status", torch.int32)
    scratch = _argmax_scratch(logits.device, n)
    _check(_fn("sampling", "zk_argmax")(_ptr(logits), n, V, _ptr(out), _ptr(feed), _ptr(status), _ptr(scratch),
                                        _ptr(ring), ring_slots, _ptr(ring_pos), _stream()), "argmax")
    return out


def _argmax_scratch(device, n: int) -> torch.Tensor:
    """Zeroed words in which the blocks of an arg-max meet (n 64-bit keys and a counter) and which the
    kernel leaves zero again; one buffer per device, shared by launches that follow one another."""
    dev = torch.device(device)
    key = ("argmax scratch", dev.index if dev.index is not None else torch.cuda.current_device())
    t = _device_state.get(key)
    if t is None or t.numel() < n + 1:
        t = _device_state[key] = torch.zeros(max(n + 1, 4097), dtype=torch.int64, device=dev)
    return t


def sample(logits, uniforms, temp: float, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
           xtc_probability: float = 0.0, xtc_threshold: float = 0.1, xtc_min_keep: int = 1, seed: int = 0,
           req_ids: Optional[torch.Tensor] = None, draws: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One draw per row after top-k, top-p, min-p, temperature and XTC.  The row's two uniforms in
    [0, 1) are uniforms[row] (float32 [n, 2]), or, with uniforms None, computed on the device as
    sampling.sampler.uniform(seed, req_ids[row], draws[req_ids[row]], 0 and 1): req_ids int32 [n]
    names each row's request (distinct), draws int32 [requests] counts each request's draws so far
    and is advanced by one for the rows' requests."""
    _need(logits, "logits", torch.float32, (None, None))
    n, V = logits.shape
    if uniforms is not None:
        _need(uniforms, "uniforms", torch.float32, (n, 2))
    else:
        _need(req_ids, "req_ids", torch.int32, (n,))
        _need(draws, "draws", torch.int32, (None,))
    if not temp > 0:
        raise KernelError("sample: temperature must be positive (use argmax for greedy)")
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF          # the 64 bits as a signed value for the C side
    if seed >= 1 << 63:
        seed -= 1 << 64
    _check(_fn("sampling", "zk_sample")(_ptr(logits), n, V, temp, top_k, top_p, min_p, xtc_probability, xtc_threshold,
                                        xtc_min_keep, _ptr(uniforms), seed, _ptr(req_ids),
                                        _ptr(draws), _ptr(out), _stream()), "sample")
    return out


__all__ = [n for n in dir() if not n.startswith("_")] + ["KernelBuildError"]
