// Gated short convolution over a packed batch of sequences with per-slot state.
//
// bcx[t] = [B_t, C_t, X_t] (3*D values), u_t = B_t * X_t,
// c_t[ch] = sum_{k=0}^{K-1} w[k][ch] * u_{t-(K-1)+k}[ch]  (+ bias[ch]),   y_t = C_t * c_t,
// with u before the first token of this step taken from the slot's state (the last K-1
// values of u of the sequence, oldest first) -- src/model.zig:1994-2028.  The taps are
// accumulated tap 0 first with float32 FMA, as the reference does.  The convolution has
// finite memory, so every (token, channel) is independent: `conv_forward` is parallel over
// tokens and only reads the state; `conv_state_update` then writes the new state.  For a
// step of single tokens `conv_decode` does both at once.
#include "common.cuh"
#include <stdint.h>

// Column of part p (0 = B, 1 = C, 2 = X) of channel ch in a bcx row: three blocks of D columns
// (il = 0), or groups of il channels laid out as [B (il) | C (il) | X (il)] (il > 0, the layout
// the fused in_proj kernel wants).
__device__ __forceinline__ size_t bcx_col(int p, int ch, int D, int il) {
  return il ? (size_t)(ch / il) * 3 * il + (size_t)p * il + ch % il : (size_t)p * D + ch;
}

// One thread per (token, channel).
template <typename T>
__global__ void conv_forward_kernel(const T* __restrict__ bcx, const float* __restrict__ state,
                                    const float* __restrict__ w, const float* __restrict__ bias,
                                    const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                                    const int* __restrict__ seq_slot, T* __restrict__ y, int n_tokens, int D, int K,
                                    long long state_slot_stride, int il) {
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  const int t = blockIdx.x;
  if (ch >= D || t >= n_tokens) return;
  const int b = tok_seq[t];
  const int i = t - cu_q[b];  // index of the token inside this step's part of the sequence
  const float* st = state + (size_t)seq_slot[b] * state_slot_stride;
  float acc = 0.f;
  for (int k = 0; k < K; ++k) {
    const int j = i - (K - 1) + k;  // source index inside this step; negative = from the state
    float u;
    if (j >= 0) {
      const T* row = bcx + (size_t)(t - (i - j)) * 3 * D;
      u = to_f32(row[bcx_col(0, ch, D, il)]) * to_f32(row[bcx_col(2, ch, D, il)]);
    } else {
      u = st[(size_t)(K - 1 + j) * D + ch];
    }
    acc = fmaf(w[(size_t)k * D + ch], u, acc);
  }
  if (bias) acc += bias[ch];
  y[(size_t)t * D + ch] = from_f32<T>(to_f32(bcx[(size_t)t * 3 * D + bcx_col(1, ch, D, il)]) * acc);
}

// The same for bfloat16 with one thread per (token, 8 adjacent channels): 16-byte loads and
// stores.  D and il are multiples of 8, so the 8 channels are adjacent in every part of a row.
__device__ __forceinline__ void unpack_bf16x8(const uint4& v, float f[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}

__global__ void conv_forward_vec8_kernel(const bf16* __restrict__ bcx, const float* __restrict__ state,
                                         const float* __restrict__ w, const float* __restrict__ bias,
                                         const int* __restrict__ tok_seq, const int* __restrict__ cu_q,
                                         const int* __restrict__ seq_slot, bf16* __restrict__ y, int n_tokens, int D,
                                         int K, long long state_slot_stride, int il) {
  const int ch = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int t = blockIdx.x;
  zk_let_next_start();
  zk_wait_prior();   // bcx is the kernel before's result, and the state is read or written by it
  if (ch >= D || t >= n_tokens) return;
  const int b = tok_seq[t];
  const int i = t - cu_q[b];
  const float* st = state + (size_t)seq_slot[b] * state_slot_stride;
  const size_t cb = bcx_col(0, ch, D, il), cc = bcx_col(1, ch, D, il), cx = bcx_col(2, ch, D, il);
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  for (int k = 0; k < K; ++k) {
    const int j = i - (K - 1) + k;
    float u[8];
    if (j >= 0) {
      const bf16* row = bcx + (size_t)(t - (i - j)) * 3 * D;
      float bv[8], xv[8];
      unpack_bf16x8(*reinterpret_cast<const uint4*>(row + cb), bv);
      unpack_bf16x8(*reinterpret_cast<const uint4*>(row + cx), xv);
#pragma unroll
      for (int e = 0; e < 8; ++e) u[e] = bv[e] * xv[e];
    } else {
      const float4* sp = reinterpret_cast<const float4*>(st + (size_t)(K - 1 + j) * D + ch);
      const float4 a = sp[0], c = sp[1];
      u[0] = a.x, u[1] = a.y, u[2] = a.z, u[3] = a.w, u[4] = c.x, u[5] = c.y, u[6] = c.z, u[7] = c.w;
    }
    const float4* wp = reinterpret_cast<const float4*>(w + (size_t)k * D + ch);
    const float4 wa = wp[0], wc = wp[1];
    const float wk[8] = {wa.x, wa.y, wa.z, wa.w, wc.x, wc.y, wc.z, wc.w};
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk[e], u[e], acc[e]);
  }
  float cv[8];
  unpack_bf16x8(*reinterpret_cast<const uint4*>(bcx + (size_t)t * 3 * D + cc), cv);
  __nv_bfloat162 o[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float b0 = bias ? bias[ch + 2 * e] : 0.f, b1 = bias ? bias[ch + 2 * e + 1] : 0.f;
    o[e] = __floats2bfloat162_rn(cv[2 * e] * (bias ? acc[2 * e] + b0 : acc[2 * e]),
                                 cv[2 * e + 1] * (bias ? acc[2 * e + 1] + b1 : acc[2 * e + 1]));
  }
  *reinterpret_cast<uint4*>(y + (size_t)t * D + ch) = *reinterpret_cast<const uint4*>(o);
}

// The same bits from one thread per (RUN consecutive tokens, 8 adjacent channels), K a template
// parameter: every B, X and C value is loaded once per thread that needs it (RUN + K - 1 rows of B
// and X for RUN tokens, where the kernel above loads K rows per token), all loads are under way
// before the first is used, and the taps are loaded once.  A run may cross from one sequence of the
// packed prompts into the next: each token looks up its own sequence, and takes what lies before
// the sequence's first token of this step from the state.
template <int K, int RUN>
__global__ void __launch_bounds__(128)
    conv_forward_run_kernel(const bf16* __restrict__ bcx, const float* __restrict__ state, const float* __restrict__ w,
                            const float* __restrict__ bias, const int* __restrict__ tok_seq,
                            const int* __restrict__ cu_q, const int* __restrict__ seq_slot, bf16* __restrict__ y,
                            int n_tokens, int D, long long state_slot_stride, int il) {
  const int ch = (blockIdx.y * blockDim.x + threadIdx.x) * 8;
  const int t0 = blockIdx.x * RUN;
  zk_let_next_start();
  zk_wait_prior();   // bcx is the kernel before's result, and the state is read or written by it
  if (ch >= D || t0 >= n_tokens) return;
  const size_t cb = bcx_col(0, ch, D, il), cc = bcx_col(1, ch, D, il), cx = bcx_col(2, ch, D, il);
  constexpr int ROWS = RUN + K - 1;    // tokens t0 - (K - 1) .. t0 + RUN - 1
  uint4 braw[ROWS], xraw[ROWS], craw[RUN];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) {
    const int tt = t0 - (K - 1) + j;
    const bool in = tt >= 0 && tt < n_tokens;
    const bf16* row = bcx + (size_t)(in ? tt : t0) * 3 * D;
    braw[j] = *reinterpret_cast<const uint4*>(row + cb);
    xraw[j] = *reinterpret_cast<const uint4*>(row + cx);
  }
#pragma unroll
  for (int r = 0; r < RUN; ++r)
    craw[r] = *reinterpret_cast<const uint4*>(bcx + (size_t)min(t0 + r, n_tokens - 1) * 3 * D + cc);
  float wk[K][8];
#pragma unroll
  for (int k = 0; k < K; ++k) {
    const float4* wp = reinterpret_cast<const float4*>(w + (size_t)k * D + ch);
    const float4 wa = wp[0], wc = wp[1];
    wk[k][0] = wa.x, wk[k][1] = wa.y, wk[k][2] = wa.z, wk[k][3] = wa.w;
    wk[k][4] = wc.x, wk[k][5] = wc.y, wk[k][6] = wc.z, wk[k][7] = wc.w;
  }
  float bs[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) bs[e] = bias ? bias[ch + e] : 0.f;
  float u[ROWS][8];
#pragma unroll
  for (int j = 0; j < ROWS; ++j) {
    float bv[8], xv[8];
    unpack_bf16x8(braw[j], bv);
    unpack_bf16x8(xraw[j], xv);
#pragma unroll
    for (int e = 0; e < 8; ++e) u[j][e] = bv[e] * xv[e];
  }
#pragma unroll
  for (int r = 0; r < RUN; ++r) {
    const int t = t0 + r;
    if (t >= n_tokens) break;
    const int b = tok_seq[t];
    const int i = t - cu_q[b];            // the token's place in its sequence's part of this step
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) {
      const int j = i - (K - 1) + k;
      if (j >= 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk[k][e], u[r + k][e], acc[e]);
      } else {
        const float4* sp =
            reinterpret_cast<const float4*>(state + (size_t)seq_slot[b] * state_slot_stride + (size_t)(K - 1 + j) * D + ch);
        const float4 a = sp[0], c = sp[1];
        const float us[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = fmaf(wk[k][e], us[e], acc[e]);
      }
    }
    float cv[8];
    unpack_bf16x8(craw[r], cv);
    __nv_bfloat162 o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      o[e] = __floats2bfloat162_rn(cv[2 * e] * (bias ? acc[2 * e] + bs[2 * e] : acc[2 * e]),
                                   cv[2 * e + 1] * (bias ? acc[2 * e + 1] + bs[2 * e + 1] : acc[2 * e + 1]));
    *reinterpret_cast<uint4*>(y + (size_t)t * D + ch) = *reinterpret_cast<const uint4*>(o);
  }
}

// One thread per (sequence, channel): state <- last K-1 values of u, older state rows survive
// when the step brought fewer than K-1 tokens (src/model.zig:2020).  Row r of the new state
// comes from row r + Tq of the old one, which lies above r, so rows are rewritten in
// ascending order without a copy.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ bcx, float* __restrict__ state,
                                         const int* __restrict__ cu_q, const int* __restrict__ seq_slot, int n_seqs,
                                         int D, int K, long long state_slot_stride, int il) {
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  const int b = blockIdx.x;
  zk_let_next_start();
  zk_wait_prior();   // bcx is the kernel before's result, and the state is read or written by it
  if (ch >= D || b >= n_seqs) return;
  const int t0 = cu_q[b], Tq = cu_q[b + 1] - t0;
  if (Tq <= 0) return;
  float* st = state + (size_t)seq_slot[b] * state_slot_stride;
  for (int r = 0; r < K - 1; ++r) {
    const int j = Tq - (K - 1) + r;
    float u;
    if (j >= 0) {
      const T* row = bcx + (size_t)(t0 + j) * 3 * D;
      u = to_f32(row[bcx_col(0, ch, D, il)]) * to_f32(row[bcx_col(2, ch, D, il)]);
    } else {
      u = st[(size_t)(K - 1 + j) * D + ch];
    }
    st[(size_t)r * D + ch] = u;
  }
}

// Single-token steps: one thread per (sequence, channel) reads the state, produces y and
// shifts the state by one.  Token t belongs to sequence t.
template <typename T>
__global__ void conv_decode_kernel(const T* __restrict__ bcx, float* __restrict__ state, const float* __restrict__ w,
                                   const float* __restrict__ bias, const int* __restrict__ seq_slot,
                                   T* __restrict__ y, int n_seqs, int D, int K, long long state_slot_stride, int il) {
  const int ch = blockIdx.y * blockDim.x + threadIdx.x;
  const int b = blockIdx.x;
  zk_let_next_start();
  zk_wait_prior();   // bcx is the kernel before's result
  if (ch >= D || b >= n_seqs) return;
  float* st = state + (size_t)seq_slot[b] * state_slot_stride;
  const T* row = bcx + (size_t)b * 3 * D;
  const float u_new = to_f32(row[bcx_col(0, ch, D, il)]) * to_f32(row[bcx_col(2, ch, D, il)]);
  float acc = 0.f;
  for (int k = 0; k < K - 1; ++k) {
    const float u = st[(size_t)k * D + ch];
    acc = fmaf(w[(size_t)k * D + ch], u, acc);
    if (k > 0) st[(size_t)(k - 1) * D + ch] = u;
  }
  acc = fmaf(w[(size_t)(K - 1) * D + ch], u_new, acc);
  st[(size_t)(K - 2) * D + ch] = u_new;
  if (bias) acc += bias[ch];
  y[(size_t)b * D + ch] = from_f32<T>(to_f32(row[bcx_col(1, ch, D, il)]) * acc);
}

extern "C" {

// bcx [n_tokens, 3D] and y [n_tokens, D] in the run dtype; state [slots, K-1, D] float32 with
// `state_slot_stride` elements between slots; w [K, D] and bias [D] (or null) float32.
int zk_conv_forward(const void* bcx, const float* state, const float* w, const float* bias, const int* tok_seq,
                    const int* cu_q, const int* seq_slot, void* y, int n_tokens, int D, int K,
                    long long state_slot_stride, int il, int dtype, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (D <= 0 || K < 2 || il < 0 || (il > 0 && D % il)) return ZK_EINVAL;
  const int threads = 128;
  if (dtype == ZK_BF16 && D % 8 == 0 && il % 8 == 0 && state_slot_stride % 4 == 0 &&
      (reinterpret_cast<uintptr_t>(bcx) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(state) |
       reinterpret_cast<uintptr_t>(w)) % 16 == 0) {
    // many tokens and few taps: runs of four tokens per thread
    constexpr int RUN = 4;
    if (n_tokens >= 256 && K <= 4) {
      dim3 grid_run(ceil_div_i(n_tokens, RUN), ceil_div_i(D / 8, threads));
#define ZK_CONV_RUN(KV)                                                                                              \
  return zk_launch_dependent(conv_forward_run_kernel<KV, RUN>, grid_run, dim3(threads), 0, stream, (const bf16*)bcx, \
                             state, w, bias, tok_seq, cu_q, seq_slot, (bf16*)y, n_tokens, D, state_slot_stride, il);
      if (K == 2) { ZK_CONV_RUN(2) }
      if (K == 3) { ZK_CONV_RUN(3) }
      ZK_CONV_RUN(4)
#undef ZK_CONV_RUN
    }
    dim3 grid8(n_tokens, ceil_div_i(D / 8, threads));
    return zk_launch_dependent(conv_forward_vec8_kernel, grid8, dim3(threads), 0, stream, (const bf16*)bcx, state, w, bias,
                               tok_seq, cu_q, seq_slot, (bf16*)y, n_tokens, D, K, state_slot_stride, il);
  }
  dim3 grid(n_tokens, ceil_div_i(D, threads));
  if (dtype == ZK_F32)
    conv_forward_kernel<float><<<grid, threads, 0, stream>>>((const float*)bcx, state, w, bias, tok_seq, cu_q, seq_slot,
                                                             (float*)y, n_tokens, D, K, state_slot_stride, il);
  else if (dtype == ZK_BF16)
    conv_forward_kernel<bf16><<<grid, threads, 0, stream>>>((const bf16*)bcx, state, w, bias, tok_seq, cu_q, seq_slot,
                                                            (bf16*)y, n_tokens, D, K, state_slot_stride, il);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_conv_state_update(const void* bcx, float* state, const int* cu_q, const int* seq_slot, int n_seqs, int D, int K,
                         long long state_slot_stride, int il, int dtype, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (D <= 0 || K < 2 || il < 0 || (il > 0 && D % il)) return ZK_EINVAL;
  const int threads = 128;
  dim3 grid(n_seqs, ceil_div_i(D, threads));
  if (dtype == ZK_F32)
    return zk_launch_dependent(conv_state_update_kernel<float>, grid, dim3(threads), 0, stream, (const float*)bcx, state,
                               cu_q, seq_slot, n_seqs, D, K, state_slot_stride, il);
  else if (dtype == ZK_BF16)
    return zk_launch_dependent(conv_state_update_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)bcx, state,
                               cu_q, seq_slot, n_seqs, D, K, state_slot_stride, il);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_conv_decode(const void* bcx, float* state, const float* w, const float* bias, const int* seq_slot, void* y,
                   int n_seqs, int D, int K, long long state_slot_stride, int il, int dtype, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (D <= 0 || K < 2 || il < 0 || (il > 0 && D % il)) return ZK_EINVAL;
  const int threads = 128;
  dim3 grid(n_seqs, ceil_div_i(D, threads));
  if (dtype == ZK_F32)
    return zk_launch_dependent(conv_decode_kernel<float>, grid, dim3(threads), 0, stream, (const float*)bcx, state, w, bias,
                               seq_slot, (float*)y, n_seqs, D, K, state_slot_stride, il);
  if (dtype == ZK_BF16)
    return zk_launch_dependent(conv_decode_kernel<bf16>, grid, dim3(threads), 0, stream, (const bf16*)bcx, state, w, bias,
                               seq_slot, (bf16*)y, n_seqs, D, K, state_slot_stride, il);
  return ZK_EINVAL;
}

}  // extern "C"
