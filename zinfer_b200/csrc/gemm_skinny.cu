// C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias) for a few rows of X (M <= 64): the contraction of a
// single-token step.  Every weight is read exactly once, straight from global memory into
// tensor-core fragments, so the kernel runs at the speed the weights stream from HBM.
//
// The roles are swapped against the usual layout: 16 weight rows are the M side of
// mma.m16n8k16 and 8 tokens its N side.  A lane loads 16 contiguous bytes (8 bfloat16) of a
// weight row and of a token row and feeds them to two MMAs; both operands use the same
// permutation of k inside a 32-wide slab, which a dot product does not see.  A block owns RG
// groups of 16 weight rows; its 8 warps split K between them and their partial sums are added
// in warp order through shared memory, so a result depends neither on M nor on the token's
// place in the batch.  (Reference: one dot product per weight row and token,
// src/model.zig:923-1026; bfloat16 dot with float32 accumulation, src/quant.zig:444-455.)
//
// What is fused around the contraction, because at these sizes a kernel launch costs as much
// as the kernel:
//  * NORM: X is the float32 residual stream and the block applies RMSNorm itself
//    (src/model.zig:1166-1181) while its first weights are in flight;
//  * NORM_SCALED: the kernel that wrote the residual rows also wrote them as bfloat16(x * w) and
//    their sums of squares per 16 columns (EMIT); this kernel reads those rows like any
//    bfloat16 input and multiplies its float32 sums by the row's 1/rms: the norm costs no launch;
//  * EPI_SWIGLU: the block owns gate rows f and up rows F + f and writes silu(g) * u
//    (src/model.zig:1085-1117: gate, up and the activation in one worker);
//  * EPI_CONV: the block owns rows ch, D + ch, 2D + ch of the short convolution's in_proj and
//    runs the gated convolution with its state update on them (src/model.zig:2002-2020).
#include "common.cuh"
#include <stdlib.h>
#include <type_traits>

namespace {

enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_CONV = 2 };
enum { NORM_NONE = 0, NORM_FUSED = 1, NORM_SCALED = 2 };

struct Args {
  const bf16* X;         // [M, K] bfloat16, or null when Xf is given
  const float* Xf;       // [M, K] float32 residual rows to be normalised (NORM)
  const float* norm_w;   // [K]
  float eps;
  const bf16* W;         // [rows, K]
  void* C;
  const float* bias;     // per weight row, or null
  int M, N, K, ldx, ldw, ldc, accumulate;
  // NORM_SCALED: X holds bfloat16(x * norm weight); ssq_in [M, ssq_parts] are partial sums of x^2
  const float* ssq_in;
  int ssq_parts;
  // EMIT: beside C (float32, the residual rows) the kernel writes emit_x [M, N] = bfloat16(C * emit_w)
  // and emit_ssq [M, ceil(N / 16)] = sums of C^2 over 16 columns, for the norm that reads C next
  const float* emit_w;
  bf16* emit_x;
  float* emit_ssq;
  // EPI_CONV
  float* conv_state;     // [slots, taps-1, N] float32
  const float* conv_taps;  // [taps, N]
  const float* conv_bias;  // [N] or null
  const int* seq_slot;   // [M]
  int taps;
  long long state_stride;
};

__device__ __forceinline__ void mma16816(float c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 ld16_stream(const bf16* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned pack2(float a, float b) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&t);
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// RG: groups of 16 weight rows per block; NT: groups of 8 tokens; UNROLL: 32-wide k slabs whose
// weight loads are in flight together.  N is the number of output columns; for EPI_PLAIN weight
// row = column, for the fused epilogues block b holds weight rows b*16*RG .. (interleaved parts).
// Blocks per SM asked of the compiler for the variants of 9 to 16 rows (two groups of 8 tokens): left to
// itself it gave the 8-warp ones 138 registers (one block per SM where two fit with 128) and held the
// 16-warp ones to 74 (few loads in flight).  Measured at 16 rows on the LFM2-1.2B shapes: w1|w3 21.3 ->
// 16.4 us, w2 14.1 -> 9.0, qkv 8.0 -> 5.9, out_proj 3.9 -> 3.1.  The variants of up to 8 rows lose with
// such a bound (a step of 8 rows 0.668 -> 0.724 ms) and keep the compiler's own choice.
constexpr int skinny_min_blocks(int warps, int nt, int epi) { return nt == 2 ? (warps == 8 && epi == EPI_PLAIN ? 2 : 1) : 0; }

template <int WARPS, int RG, int NT, int UNROLL, int EPI, int NORM_MODE, typename TC, bool EMIT = false>
__global__ void __launch_bounds__(WARPS * 32, skinny_min_blocks(WARPS, NT, EPI)) skinny_kernel(const Args a) {
  constexpr bool NORM = NORM_MODE == NORM_FUSED;   // the prologue that normalises float32 rows
  extern __shared__ float smem[];
  constexpr int RED_LD = NT * 8 + 1;
  float(*red)[RG * 16][RED_LD] = reinterpret_cast<float(*)[RG * 16][RED_LD]>(smem);
  float* row_scale = smem + WARPS * RG * 16 * RED_LD;  // [NT * 8], then [NT * 8][WARPS] partial sums
  bf16* xs = reinterpret_cast<bf16*>(smem + ((WARPS * RG * 16 * RED_LD + NT * 8 + NT * 8 * WARPS + 3) / 4) * 4);  // NORM: [NT * 8][K + 8] bfloat16

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int M = a.M, N = a.N, K = a.K;
  // A block takes the tasks blockIdx.x, blockIdx.x + gridDim.x, ...: a task is 16 * RG output
  // columns (EPI_PLAIN) or 16 (fused epilogues).  With as many blocks as tasks that is one each;
  // fewer blocks are launched where a prologue (the norm) should be paid once for several tasks.
  constexpr int TASK_COLS = EPI == EPI_PLAIN ? 16 * RG : 16;
  const int n_tasks = (N + TASK_COLS - 1) / TASK_COLS;
  int task = blockIdx.x;
  int n0 = task * TASK_COLS;

  const int slabs = (K + 31) / 32;
  const int per = (slabs + WARPS - 1) / WARPS;
  const int s_begin = warp * per, s_end = min(slabs, s_begin + per);

  const bf16* wrow[RG][2];
  bool wok[RG][2];
  auto set_task = [&]() {
    n0 = task * TASK_COLS;
#pragma unroll
    for (int r = 0; r < RG; ++r)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        // EPI_PLAIN: weight row = output column.  Fused epilogues: the weights are stored in groups of
        // 16 rows per part (16 gate rows, their 16 up rows; 16 B, 16 C, 16 X rows), so the RG groups of
        // a task are RG * 16 adjacent rows and stream like any 16 * RG rows.
        const int col = n0 + (EPI == EPI_PLAIN ? r * 16 : 0) + g + 8 * h;
        wok[r][h] = col < N;
        const size_t row = EPI == EPI_PLAIN ? (size_t)(wok[r][h] ? col : 0)
                                            : (size_t)task * (16 * RG) + r * 16 + (wok[r][h] ? g + 8 * h : 0);
        wrow[r][h] = a.W + row * a.ldw;
      }
  };
  set_task();
  const uint4 zero = make_uint4(0, 0, 0, 0);

  uint4 wv[UNROLL][RG][2];
  auto load_w = [&](int s) {
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s + u) * 32 + 8 * c;
      const bool kok = (s + u) < s_end && k < K;  // K % 8 == 0: a 16-byte piece is all in or all out
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wv[u][r][h] = (kok && wok[r][h]) ? ld16_stream(wrow[r][h] + k) : zero;
    }
  };
  // Loads of the next slabs are issued after the MMAs of the current ones when a slab carries
  // much arithmetic (many tokens) or a norm prologue can hide them, else at the top of the loop;
  // measured, not derived.
  constexpr bool PIPE = NT >= 4 || NORM;
  // The short norm prologue below (up to 8 rows, K up to 8 values per thread and row).
  const bool norm_one_pass = NORM && NT == 1 && K <= WARPS * 32 * 8;
  // Weights need nothing of the kernel before: the first are requested, then the next kernel is let
  // in, then this one waits.  Measured on the LFM2-1.2B step at 8 rows: 0.712 ms in this order, 0.754
  // with the loads after zk_let_next_start(), 0.770 with zk_let_next_start() after the main loop, and
  // 0.749 when the kernels whose norm fills the registers asked for their first weights with
  // prefetch.global.L2 instead of nothing.
  load_w(s_begin);
  zk_let_next_start();
  zk_wait_prior();   // the rows (X, Xf, the convolution's state) and C are the kernels' before

  // NORM: the block normalises the M rows once into shared memory as bfloat16 (row stride padded
  // by 16 bytes so that the 8 rows a fragment load touches fall into different banks).
  const int xs_ld = K + 8;
  if constexpr (NORM_MODE == NORM_SCALED) {
    // one warp per row adds the row's partial sums in a fixed order; read after the barrier that
    // follows the main loop
    for (int m = warp; m < M; m += WARPS) {
      float t = 0.f;
      for (int p = lane; p < a.ssq_parts; p += 32) t += a.ssq_in[(size_t)m * a.ssq_parts + p];
      t = warp_sum(t);
      if (lane == 0) row_scale[m] = 1.0f / sqrtf(t / (float)K + a.eps);
    }
  }
  if constexpr (NORM) {
    float* part = row_scale + NT * 8;  // [NT * 8][WARPS] partial sums of squares
    constexpr int TH = WARPS * 32;
    if (norm_one_pass) {
      // Up to 8 rows of up to 2 float4 per thread, four rows at a time.  The rows go to shared memory
      // as bfloat16(x * w) WITHOUT the row's scale: the scale is one factor of the whole dot product
      // and is applied to the float32 sum in the epilogue.  So no value has to be kept in registers
      // until the sum of squares is known, and the first weights can be under way meanwhile.  A
      // row's sum is added per thread over k, over the lanes, over the warps.
      float ss[8];
#pragma unroll
      for (int m = 0; m < 8; ++m) ss[m] = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int k = threadIdx.x * 4 + j * TH * 4;
        if (k < K) {
          const float4 w = *reinterpret_cast<const float4*>(a.norm_w + k);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float4 v[4];
#pragma unroll
            for (int m = 0; m < 4; ++m)
              v[m] = (4 * h + m < M) ? *reinterpret_cast<const float4*>(a.Xf + (size_t)(4 * h + m) * a.ldx + k)
                                     : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
              float t = ss[4 * h + m];
              t = fmaf(v[m].x, v[m].x, t);
              t = fmaf(v[m].y, v[m].y, t);
              t = fmaf(v[m].z, v[m].z, t);
              t = fmaf(v[m].w, v[m].w, t);
              ss[4 * h + m] = t;
              if (4 * h + m < M) {
                uint2 pk;
                pk.x = pack2(v[m].x * w.x, v[m].y * w.y);
                pk.y = pack2(v[m].z * w.z, v[m].w * w.w);
                *reinterpret_cast<uint2*>(xs + (size_t)(4 * h + m) * xs_ld + k) = pk;
              }
            }
          }
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const float t = warp_sum(ss[m]);
        if (lane == 0 && m < M) part[m * WARPS + warp] = t;
      }
      __syncthreads();
      if (threadIdx.x < M) {
        float t = 0.f;
#pragma unroll
        for (int ww = 0; ww < WARPS; ++ww) t += part[threadIdx.x * WARPS + ww];
        row_scale[threadIdx.x] = 1.0f / sqrtf(t / (float)K + a.eps);
      }
      __syncthreads();
    } else {
    for (int m0 = 0; m0 < M; m0 += 4) {
      float ss[4] = {0.f, 0.f, 0.f, 0.f};
      for (int k = threadIdx.x * 4; k < K; k += WARPS * 32 * 4) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[j] = (m0 + j < M) ? *reinterpret_cast<const float4*>(a.Xf + (size_t)(m0 + j) * a.ldx + k)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ss[j] = fmaf(v[j].x, v[j].x, ss[j]);
          ss[j] = fmaf(v[j].y, v[j].y, ss[j]);
          ss[j] = fmaf(v[j].z, v[j].z, ss[j]);
          ss[j] = fmaf(v[j].w, v[j].w, ss[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float t = warp_sum(ss[j]);
        if (lane == 0 && m0 + j < M) part[(m0 + j) * WARPS + warp] = t;
      }
    }
    __syncthreads();
    if (threadIdx.x < M) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) t += part[threadIdx.x * WARPS + w];
      row_scale[threadIdx.x] = 1.0f / sqrtf(t / (float)K + a.eps);
    }
    __syncthreads();
    // second pass: the rows again (from L2), four at a time so that their loads are under way together
    for (int k = threadIdx.x * 4; k < K; k += WARPS * 32 * 4) {
      const float4 w = *reinterpret_cast<const float4*>(a.norm_w + k);
      for (int m0 = 0; m0 < M; m0 += 4) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          v[j] = (m0 + j < M) ? *reinterpret_cast<const float4*>(a.Xf + (size_t)(m0 + j) * a.ldx + k)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (m0 + j < M) {
            const float sc = row_scale[m0 + j];
            uint2 pk;
            pk.x = pack2((v[j].x * sc) * w.x, (v[j].y * sc) * w.y);
            pk.y = pack2((v[j].z * sc) * w.z, (v[j].w * sc) * w.w);
            *reinterpret_cast<uint2*>(xs + (size_t)(m0 + j) * xs_ld + k) = pk;
          }
        }
      }
    }
    __syncthreads();
    }
  }

  bool xok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) xok[t] = t * 8 + g < M;

  for (;;) {   // the block's tasks
  float acc[RG][NT][4];
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][t][i] = 0.f;

  for (int s = s_begin; s < s_end; s += UNROLL) {
    if (!PIPE && s != s_begin) load_w(s);
    uint4 xv[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s + u) * 32 + 8 * c;
      const bool kok = (s + u) < s_end && k < K;
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        if (!(kok && xok[t])) {
          xv[u][t] = zero;
        } else if constexpr (NORM) {
          xv[u][t] = *reinterpret_cast<const uint4*>(xs + (size_t)(t * 8 + g) * xs_ld + k);
        } else {
          xv[u][t] = ld16(a.X + (size_t)(t * 8 + g) * a.ldx + k);
        }
      }
    }
    // A warp barrier between the loads and the MMAs of the smallest variant: without it the
    // assembler sinks every load down to the MMA that uses it to save registers (34 registers, one
    // load in flight); with it all loads of the slabs are issued first and are in flight together
    // (62 registers; 11.3 -> 10.3 us on a [2048, 8192] matrix).  The larger variants are scheduled
    // well without it and lose a little with it (measured), so they do not get it.
    if constexpr (RG == 1 && NT == 1) __syncwarp();
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816(acc[r][t], wv[u][r][0].x, wv[u][r][1].x, wv[u][r][0].y, wv[u][r][1].y, xv[u][t].x, xv[u][t].y);
          mma16816(acc[r][t], wv[u][r][0].z, wv[u][r][1].z, wv[u][r][0].w, wv[u][r][1].w, xv[u][t].z, xv[u][t].w);
        }
    if (PIPE && s + UNROLL < s_end) load_w(s + UNROLL);
  }

  // partial sums of the 8 warps -> shared memory; C fragment: rows g, g+8; columns 2c, 2c+1
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      red[warp][r * 16 + g][t * 8 + 2 * c] = acc[r][t][0];
      red[warp][r * 16 + g][t * 8 + 2 * c + 1] = acc[r][t][1];
      red[warp][r * 16 + g + 8][t * 8 + 2 * c] = acc[r][t][2];
      red[warp][r * 16 + g + 8][t * 8 + 2 * c + 1] = acc[r][t][3];
    }
  __syncthreads();

  auto total = [&](int row, int m) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][row][m];
    if ((NORM && norm_one_pass) || NORM_MODE == NORM_SCALED) v *= row_scale[m];   // the rows came without their scale
    return v;
  };

  if constexpr (EPI == EPI_PLAIN) {
    TC* C = reinterpret_cast<TC*>(a.C);
    for (int idx = threadIdx.x; idx < RG * 16 * NT * 8; idx += WARPS * 32) {
      const int m = idx / (RG * 16), nl = idx % (RG * 16);
      const int n = n0 + nl;
      const bool in = m < M && n < N;
      if (!EMIT && !in) continue;
      float v = 0.f;
      if (in) {
        v = total(nl, m);
        if (a.bias) v += a.bias[n];
        TC* dst = C + (size_t)m * a.ldc + n;
        if (a.accumulate) v += to_f32(*dst);
        *dst = from_f32<TC>(v);
      }
      if constexpr (EMIT) {
        // whole warps run this loop (its bound is a multiple of 32); 16 adjacent lanes hold 16
        // adjacent columns of one row
        if (in) a.emit_x[(size_t)m * N + n] = __float2bfloat16_rn(v * a.emit_w[n]);
        float sq = v * v;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
        if ((nl & 15) == 0 && m < M && n < N) a.emit_ssq[(size_t)m * ((N + 15) / 16) + n / 16] = sq;
      }
    }
  } else if constexpr (EPI == EPI_SWIGLU) {
    bf16* C = reinterpret_cast<bf16*>(a.C);
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += WARPS * 32) {
      const int m = idx / 16, i = idx % 16;
      const int n = n0 + i;
      if (m >= M || n >= N) continue;
      const float gate = total(i, m), up = total(16 + i, m);
      C[(size_t)m * a.ldc + n] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
    }
  } else {  // EPI_CONV: token m is sequence m
    bf16* C = reinterpret_cast<bf16*>(a.C);
    const int taps = a.taps;
    for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += WARPS * 32) {
      const int m = idx / 16, i = idx % 16;
      const int ch = n0 + i;
      if (m >= M || ch >= N) continue;
      float bv = total(i, m), cv = total(16 + i, m), xval = total(32 + i, m);
      if (a.bias) {  // stored in the weights' row order
        const size_t base = (size_t)task * 48 + i;
        bv += a.bias[base];
        cv += a.bias[base + 16];
        xval += a.bias[base + 32];
      }
      // rounded as the unfused path stores them, so both paths keep the same state
      const float u_new = round_bf16(bv) * round_bf16(xval);
      float* st = a.conv_state + (size_t)a.seq_slot[m] * a.state_stride;
      float sum = 0.f;
      for (int k = 0; k < taps - 1; ++k) {
        const float u = st[(size_t)k * N + ch];
        sum = fmaf(a.conv_taps[(size_t)k * N + ch], u, sum);
        if (k > 0) st[(size_t)(k - 1) * N + ch] = u;
      }
      sum = fmaf(a.conv_taps[(size_t)(taps - 1) * N + ch], u_new, sum);
      st[(size_t)(taps - 2) * N + ch] = u_new;
      if (a.conv_bias) sum += a.conv_bias[ch];
      C[(size_t)m * a.ldc + ch] = __float2bfloat16_rn(round_bf16(cv) * sum);
    }
  }
  task += gridDim.x;
  if (task >= n_tasks) break;
  __syncthreads();   // the epilogue has read `red`
  set_task();
  load_w(s_begin);
  }
}

// Most blocks of a kernel with the norm prologue: two per SM.  Measured on the LFM2-1.2B shapes at
// one row (where every contraction takes the norm itself): 0.698 ms a step with 296 blocks, 0.771
// with 148, 0.730 with 444, 0.779 with one block per task.
int norm_grid_cap() { return 148 * 2; }

template <int WARPS, int RG, int NT>
size_t smem_bytes(bool norm, int K) {
  size_t floats = (size_t)WARPS * RG * 16 * (NT * 8 + 1) + NT * 8 + NT * 8 * WARPS;
  floats = (floats + 3) / 4 * 4;  // the bfloat16 rows start 16-byte aligned
  return sizeof(float) * floats + (norm ? sizeof(bf16) * (size_t)NT * 8 * (K + 8) : 0);
}

template <int WARPS, int RG, int NT, int UNROLL, int EPI, int NORM_MODE, typename TC, bool EMIT = false>
int launch(const Args& a, cudaStream_t stream) {
  auto kern = skinny_kernel<WARPS, RG, NT, UNROLL, EPI, NORM_MODE, TC, EMIT>;
  constexpr bool NORM = NORM_MODE == NORM_FUSED;
  const size_t smem = smem_bytes<WARPS, RG, NT>(NORM, a.K);
  if (smem > 200 * 1024) return ZK_EINVAL;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int grid = ceil_div_i(a.N, EPI == EPI_PLAIN ? 16 * RG : 16);
  if (NORM && grid > norm_grid_cap()) grid = norm_grid_cap();   // the norm prologue once for several tasks
  return zk_launch_dependent(kern, dim3(grid), dim3(WARPS * 32), smem, stream, a);
}

// Shapes are chosen so that a block streams enough weights to pay for its start-up and so that an
// SM has some 64 KB of loads in flight: 16 warps where N gives few blocks, 32 rows per block
// where N gives many.
template <int NORM_MODE, typename TC>
int dispatch_plain(const Args& a, cudaStream_t stream) {
  const bool few = a.N <= 16 * 148 * 2;    // at most two 16-row blocks per SM: make each block wider in K
  const bool many = a.N >= 16 * 148 * 6;   // many blocks: 32 rows each
  // A warp of a 16-warp block owns K / 16 columns: from K = 4096 on that is 8 slabs and more, and all 8
  // are requested at once (128 registers a thread, one block per SM).  Measured on whole steps of the
  // LFM2-1.2B shape, whose w2 has K = 8192: 0.5810 -> 0.5728 ms at one row, 0.7015 -> 0.6945 ms at 8.
  const bool long_k = a.K >= 4096;
  // one_wave: more 16-row blocks than SMs but at most two per SM (qkv of the LFM2-1.2B shape: 192).  Blocks
  // of 16 warps take an SM each and run in two rounds; blocks of 8 warps with 8 slabs in flight are all
  // resident at once.  Measured on whole steps: 0.5714 -> 0.5604 ms at one row, 0.681 -> 0.670 ms at 8.
  if (a.M <= 8) {
    if constexpr (NORM_MODE == NORM_NONE && std::is_same<TC, float>::value) {
      if (a.emit_x) {
        if (few && long_k) return launch<16, 1, 1, 8, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
        if (few) return launch<16, 1, 1, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
        if (many) return launch<8, 2, 1, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
        return launch<8, 1, 1, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
      }
    }
    if constexpr (NORM_MODE == NORM_NONE) {
      if (few && long_k) return launch<16, 1, 1, 8, EPI_PLAIN, NORM_NONE, TC>(a, stream);
    }
    if (few && a.N > 16 * 148) return launch<8, 1, 1, 8, EPI_PLAIN, NORM_MODE, TC>(a, stream);   // see one_wave above
    if (few) return launch<16, 1, 1, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
    if (many) return launch<8, 2, 1, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
    return launch<8, 1, 1, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
  }
  if (a.M <= 16) {
    if constexpr (NORM_MODE == NORM_NONE && std::is_same<TC, float>::value) {
      if (a.emit_x) {
        if (few) return launch<16, 1, 2, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
        if (many) return launch<8, 2, 2, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
        return launch<8, 1, 2, 4, EPI_PLAIN, NORM_NONE, TC, true>(a, stream);
      }
    }
    if (few) return launch<16, 1, 2, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
    if (many) return launch<8, 2, 2, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
    return launch<8, 1, 2, 4, EPI_PLAIN, NORM_MODE, TC>(a, stream);
  }
  if constexpr (NORM_MODE != NORM_NONE) {
    return ZK_EINVAL;
  } else {
    // the split of K over the warps must not depend on M, or a row's bits would depend on its batch
    if (a.M <= 32) return few ? launch<16, 1, 4, 2, EPI_PLAIN, NORM_NONE, TC>(a, stream)
                              : launch<8, 2, 4, 2, EPI_PLAIN, NORM_NONE, TC>(a, stream);
    return few ? launch<16, 1, 8, 1, EPI_PLAIN, NORM_NONE, TC>(a, stream) : launch<8, 1, 8, 2, EPI_PLAIN, NORM_NONE, TC>(a, stream);
  }
}

template <typename TC>
int dispatch_plain_any(const Args& a, cudaStream_t stream) {
  if (a.Xf) return dispatch_plain<NORM_FUSED, TC>(a, stream);
  if (a.ssq_in) return dispatch_plain<NORM_SCALED, TC>(a, stream);
  return dispatch_plain<NORM_NONE, TC>(a, stream);
}

template <int RG, int EPI, int NORM_MODE>
int dispatch_fused_mode(const Args& a, cudaStream_t stream) {
  if (a.M <= 8) return launch<8, RG, 1, 4, EPI, NORM_MODE, bf16>(a, stream);
  if (a.M <= 16) return launch<8, RG, 2, 2, EPI, NORM_MODE, bf16>(a, stream);
  return ZK_EINVAL;
}

template <int RG, int EPI>
int dispatch_fused(const Args& a, cudaStream_t stream) {
  if (a.Xf) return dispatch_fused_mode<RG, EPI, NORM_FUSED>(a, stream);
  if (a.ssq_in) return dispatch_fused_mode<RG, EPI, NORM_SCALED>(a, stream);
  return dispatch_fused_mode<RG, EPI, NORM_NONE>(a, stream);
}

int check_common(const Args& a, int max_m) {
  if (a.M > max_m || a.K <= 0 || a.K % 8 || a.ldw % 8 || a.ldw < a.K || a.ldx < a.K) return ZK_EINVAL;
  if ((uintptr_t)a.W % 16) return ZK_EINVAL;
  if (a.Xf) {
    if (a.ldx % 4 || (uintptr_t)a.Xf % 16 || (uintptr_t)a.norm_w % 16 || !a.norm_w) return ZK_EINVAL;
  } else {
    if (!a.X || a.ldx % 8 || (uintptr_t)a.X % 16) return ZK_EINVAL;
    if (a.ssq_in && (a.ssq_parts <= 0 || a.M > 16)) return ZK_EINVAL;
  }
  return 0;
}

}  // namespace

extern "C" {

int zk_gemm_skinny_max_m() { return 64; }
int zk_gemm_skinny_fused_max_m() { return 16; }

// X [M, K] bfloat16 (or Xf [M, K] float32 + norm_w [K], eps: RMSNorm fused, M <= 16), W [N, K]
// bfloat16 with K % 8 == 0 and 16-byte aligned rows; C [M, N] bfloat16 or float32.
// ssq_in [M, ssq_parts] (or null): X is bfloat16(x * norm weight) and the sums are scaled by
// 1 / sqrt(sum(ssq_in[m]) / K + eps) (M <= 16).  emit_x (or null; M <= 16, float32 C, no fused norm):
// also writes emit_x [M, N] = bfloat16(C * emit_w) and emit_ssq [M, ceil(N / 16)] for the next norm.
int zk_gemm_skinny(const void* X, const float* Xf, const float* norm_w, float eps, const void* W, void* C,
                   const float* bias, int M, int N, int K, int ldx, int ldw, int ldc, int out_dtype, int accumulate,
                   const float* ssq_in, int ssq_parts, const float* emit_w, void* emit_x, float* emit_ssq,
                   cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  Args a{};
  a.X = (const bf16*)X; a.Xf = Xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.C = C; a.bias = bias;
  a.M = M; a.N = N; a.K = K; a.ldx = ldx; a.ldw = ldw; a.ldc = ldc; a.accumulate = accumulate;
  a.ssq_in = Xf ? nullptr : ssq_in; a.ssq_parts = ssq_parts;
  a.emit_w = emit_w; a.emit_x = (bf16*)emit_x; a.emit_ssq = emit_ssq;
  if (ldc < N || check_common(a, Xf ? 16 : 64)) return ZK_EINVAL;
  if (emit_x && (!emit_w || !emit_ssq || M > 16 || Xf || out_dtype != ZK_F32)) return ZK_EINVAL;
  if (out_dtype == ZK_F32) return dispatch_plain_any<float>(a, stream);
  if (out_dtype == ZK_BF16) return dispatch_plain_any<bf16>(a, stream);
  return ZK_EINVAL;
}

// h[M, F] = silu(x W_gate^T) * (x W_up^T); W [2F, K] holds groups of 16 gate rows followed by their
// 16 up rows (F a multiple of 16); M <= 16.
int zk_gemm_skinny_swiglu(const void* X, const float* Xf, const float* norm_w, float eps, const void* W, void* H,
                          int M, int F, int K, int ldx, int ldw, int ldh, const float* ssq_in, int ssq_parts,
                          cudaStream_t stream) {
  if (M <= 0 || F <= 0) return 0;
  Args a{};
  a.X = (const bf16*)X; a.Xf = Xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.C = H;
  a.M = M; a.N = F; a.K = K; a.ldx = ldx; a.ldw = ldw; a.ldc = ldh;
  a.ssq_in = Xf ? nullptr : ssq_in; a.ssq_parts = ssq_parts;
  if (ldh < F || F % 16 || check_common(a, 16)) return ZK_EINVAL;
  return dispatch_fused<2, EPI_SWIGLU>(a, stream);
}

// Single-token step of the short convolution: [B, C, X] = x W_in^T (+ bias), u = B*X, the causal
// convolution over the slot's state, y = C * conv, state shifted by one.  Token m is sequence m.
// W [3D, K] and in_bias [3D] hold groups of 16 B rows, 16 C rows, 16 X rows (D a multiple of 16);
// state [slots, taps-1, D] float32; taps [taps, D]; y [M, D] bfloat16; M <= 16.
int zk_gemm_skinny_conv(const void* X, const float* Xf, const float* norm_w, float eps, const void* W,
                        const float* in_bias, float* state, const float* taps_w, const float* conv_bias,
                        const int* seq_slot, void* Y, int M, int D, int K, int taps, int ldx, int ldw, int ldy,
                        long long state_stride, const float* ssq_in, int ssq_parts, cudaStream_t stream) {
  if (M <= 0 || D <= 0) return 0;
  Args a{};
  a.X = (const bf16*)X; a.Xf = Xf; a.norm_w = norm_w; a.eps = eps; a.W = (const bf16*)W; a.C = Y; a.bias = in_bias;
  a.M = M; a.N = D; a.K = K; a.ldx = ldx; a.ldw = ldw; a.ldc = ldy;
  a.conv_state = state; a.conv_taps = taps_w; a.conv_bias = conv_bias; a.seq_slot = seq_slot; a.taps = taps;
  a.state_stride = state_stride;
  a.ssq_in = Xf ? nullptr : ssq_in; a.ssq_parts = ssq_parts;
  if (ldy < D || D % 16 || taps < 2 || !state || !taps_w || !seq_slot || check_common(a, 16)) return ZK_EINVAL;
  return dispatch_fused<3, EPI_CONV>(a, stream);
}

}  // extern "C"
