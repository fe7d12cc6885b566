// C[M, N] (+)= A[M, K] . W[N, K]^T (+ bias[N]) on the CUDA cores with float32 FMA.
//
// This is the contraction of the true 32-bit path and the fallback of the bfloat16 path for
// shapes the tensor-core kernels refuse.  Each output element is one float32 accumulator that
// walks k = 0 .. K-1 in order, so a row's result does not depend on M, on the row's place in
// the batch or on the tile it falls in (reference: one dot product per output row,
// src/model.zig:923-1026; float32 dot src/quant.zig:424-431; `accumulate` = residual add,
// src/model.zig:918-920).
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename T>
__device__ __forceinline__ void load4(const T* __restrict__ p, bool vec_ok, int k0, int K, bool row_ok, float out[4]) {
  if (!row_ok) {
    out[0] = out[1] = out[2] = out[3] = 0.f;
    return;
  }
  if (vec_ok && k0 + 3 < K) {
    if constexpr (sizeof(T) == 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + k0);
      out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    } else {
      const uint2 v = *reinterpret_cast<const uint2*>(p + k0);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
      out[0] = __low2float(lo); out[1] = __high2float(lo); out[2] = __low2float(hi); out[3] = __high2float(hi);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) out[j] = (k0 + j < K) ? to_f32(p[k0 + j]) : 0.f;
}

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        TC* __restrict__ C, const float* __restrict__ bias, int M, int N,
                                                        int K, int lda, int ldw, int ldc, int accumulate, int vecA,
                                                        int vecW) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const bool a_ok = (m0 + lrow) < M, w_ok = (n0 + lrow) < N;
  const TA* a_row = A + (size_t)(a_ok ? m0 + lrow : 0) * lda;
  const TW* w_row = W + (size_t)(w_ok ? n0 + lrow : 0) * ldw;

  for (int kb = 0; kb < K; kb += BK) {
    float av[4], wv[4];
    load4<TA>(a_row, vecA, kb + lk, K, a_ok, av);
    load4<TW>(w_row, vecW, kb + lk, K, w_ok, wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      As[lk + j][lrow] = av[j];
      Ws[lk + j][lrow] = wv[j];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float ar[4] = {a.x, a.y, a.z, a.w};
      const float br[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias) v += bias[n];
      TC* c = C + (size_t)m * ldc + n;
      if (accumulate) v += to_f32(*c);
      *c = from_f32<TC>(v);
    }
  }
}

template <typename TA, typename TW, typename TC>
int launch(const void* A, const void* W, void* C, const float* bias, int M, int N, int K, int lda, int ldw, int ldc,
           int accumulate, cudaStream_t stream) {
  const int vecA = (lda % 4 == 0) && ((uintptr_t)A % 16 == 0);
  const int vecW = (ldw % 4 == 0) && ((uintptr_t)W % 16 == 0);
  dim3 grid(ceil_div_i(N, BN), ceil_div_i(M, BM));
  gemm_simt_kernel<TA, TW, TC><<<grid, 256, 0, stream>>>((const TA*)A, (const TW*)W, (TC*)C, bias, M, N, K, lda, ldw,
                                                          ldc, accumulate, vecA, vecW);
  return ZK_LAUNCH_STATUS();
}

}  // namespace

extern "C" int zk_gemm_simt(const void* A, const void* W, void* C, const float* bias, int M, int N, int K, int lda,
                            int ldw, int ldc, int in_dtype, int out_dtype, int accumulate, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || lda < K || ldw < K || ldc < N) return ZK_EINVAL;
  if (in_dtype == ZK_F32 && out_dtype == ZK_F32)
    return launch<float, float, float>(A, W, C, bias, M, N, K, lda, ldw, ldc, accumulate, stream);
  if (in_dtype == ZK_BF16 && out_dtype == ZK_F32)
    return launch<bf16, bf16, float>(A, W, C, bias, M, N, K, lda, ldw, ldc, accumulate, stream);
  if (in_dtype == ZK_BF16 && out_dtype == ZK_BF16)
    return launch<bf16, bf16, bf16>(A, W, C, bias, M, N, K, lda, ldw, ldc, accumulate, stream);
  return ZK_EINVAL;
}
