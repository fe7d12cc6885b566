// C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias) for a few rows of X (M <= 64): the contraction of a
// single-token step.  Every weight is read exactly once, straight from global memory into
// tensor-core fragments, so the kernel runs at the speed the weights stream from HBM.
//
// The roles are swapped against the usual layout: 16 weight rows are the M side of
// mma.m16n8k16 and 8 tokens its N side.  A lane loads 16 contiguous bytes (8 bfloat16) of a
// weight row and of a token row and feeds them to two MMAs; both operands use the same
// permutation of k inside a 32-wide slab, which a dot product does not see.  A block owns
// 16*RG weight rows; its 8 warps split K between them and their partial sums are added in warp
// order through shared memory, so a result depends neither on M nor on the token's place in
// the batch.  (Reference: one dot product per weight row and token, src/model.zig:923-1026;
// bfloat16 dot with float32 accumulation, src/quant.zig:444-455.)
#include "common.cuh"

namespace {

constexpr int WARPS = 8;

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

// RG: groups of 16 weight rows per block; NT: groups of 8 tokens; UNROLL: 32-wide k slabs whose
// loads are all issued before their MMAs (what keeps enough bytes in flight).
template <int RG, int NT, int UNROLL, typename TC>
__global__ void __launch_bounds__(WARPS * 32)
    skinny_kernel(const bf16* __restrict__ X, const bf16* __restrict__ W, TC* __restrict__ C,
                  const float* __restrict__ bias, int M, int N, int K, int ldx, int ldw, int ldc, int accumulate) {
  __shared__ float red[WARPS][RG * 16][NT * 8 + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int n0 = blockIdx.x * (16 * RG);

  // this warp's slice of K, in slabs of 32
  const int slabs = (K + 31) / 32;
  const int per = (slabs + WARPS - 1) / WARPS;
  const int s_begin = warp * per, s_end = min(slabs, s_begin + per);

  float acc[RG][NT][4];
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[r][t][i] = 0.f;

  const bf16* wrow[RG][2];
  bool wok[RG][2];
#pragma unroll
  for (int r = 0; r < RG; ++r)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = n0 + r * 16 + g + 8 * h;
      wok[r][h] = n < N;
      wrow[r][h] = W + (size_t)(wok[r][h] ? n : 0) * ldw;
    }
  const bf16* xrow[NT];
  bool xok[NT];
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int m = t * 8 + g;
    xok[t] = m < M;
    xrow[t] = X + (size_t)(xok[t] ? m : 0) * ldx;
  }
  const uint4 zero = make_uint4(0, 0, 0, 0);

  for (int s = s_begin; s < s_end; s += UNROLL) {
    uint4 wv[UNROLL][RG][2], xv[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (s + u) * 32 + 8 * c;
      const bool kok = (s + u) < s_end && k < K;  // K % 8 == 0, so a 16-byte piece is all in or all out
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int h = 0; h < 2; ++h) wv[u][r][h] = (kok && wok[r][h]) ? ld16_stream(wrow[r][h] + k) : zero;
#pragma unroll
      for (int t = 0; t < NT; ++t) xv[u][t] = (kok && xok[t]) ? ld16(xrow[t] + k) : zero;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
      for (int r = 0; r < RG; ++r)
#pragma unroll
        for (int t = 0; t < NT; ++t) {
          mma16816(acc[r][t], wv[u][r][0].x, wv[u][r][1].x, wv[u][r][0].y, wv[u][r][1].y, xv[u][t].x, xv[u][t].y);
          mma16816(acc[r][t], wv[u][r][0].z, wv[u][r][1].z, wv[u][r][0].w, wv[u][r][1].w, xv[u][t].z, xv[u][t].w);
        }
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
  for (int idx = threadIdx.x; idx < RG * 16 * NT * 8; idx += WARPS * 32) {
    const int m = idx / (RG * 16), nl = idx % (RG * 16);
    const int n = n0 + nl;
    if (m >= M || n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][nl][m];
    if (bias) v += bias[n];
    TC* dst = C + (size_t)m * ldc + n;
    if (accumulate) v += to_f32(*dst);
    *dst = from_f32<TC>(v);
  }
}

template <int RG, int NT, int UNROLL, typename TC>
int launch(const void* X, const void* W, void* C, const float* bias, int M, int N, int K, int ldx, int ldw, int ldc,
           int accumulate, cudaStream_t stream) {
  const int grid = ceil_div_i(N, 16 * RG);
  skinny_kernel<RG, NT, UNROLL, TC><<<grid, WARPS * 32, 0, stream>>>((const bf16*)X, (const bf16*)W, (TC*)C, bias, M, N, K, ldx,
                                                             ldw, ldc, accumulate);
  return ZK_LAUNCH_STATUS();
}

template <typename TC>
int dispatch(const void* X, const void* W, void* C, const float* bias, int M, int N, int K, int ldx, int ldw, int ldc,
             int accumulate, cudaStream_t stream) {
  // rows per block: 16 while that still gives every SM a few blocks, else 32
  const bool wide = N >= 16 * 148 * 8;
  if (M <= 8) return wide ? launch<2, 1, 4, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream)
                          : launch<1, 1, 4, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
  if (M <= 16) return wide ? launch<2, 2, 4, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream)
                           : launch<1, 2, 4, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
  if (M <= 32) return launch<2, 4, 2, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
  return launch<1, 8, 2, TC>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
}

}  // namespace

extern "C" {

int zk_gemm_skinny_max_m() { return 64; }

// X [M, K], W [N, K] bfloat16 with K % 8 == 0, rows 16-byte aligned; C [M, N] bfloat16 or float32.
int zk_gemm_skinny(const void* X, const void* W, void* C, const float* bias, int M, int N, int K, int ldx, int ldw,
                   int ldc, int out_dtype, int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldc < N) return ZK_EINVAL;
  if (((uintptr_t)X | (uintptr_t)W) % 16) return ZK_EINVAL;
  if (out_dtype == ZK_F32) return dispatch<float>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
  if (out_dtype == ZK_BF16) return dispatch<bf16>(X, W, C, bias, M, N, K, ldx, ldw, ldc, accumulate, stream);
  return ZK_EINVAL;
}

}  // extern "C"
