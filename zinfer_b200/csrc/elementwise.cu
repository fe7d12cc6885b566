// Row-wise kernels: embedding gather, RMSNorm (with optional row gather), SiLU-gate product.
// All arithmetic is float32; only loads and stores use the run dtype.
#include "common.cuh"
#include <stdint.h>

// x[t, :] = float(table[tokens[t], :]).  A token id outside [0, vocab) sets *status = 1 and
// yields a zero row (reference: row lookup of token_embd, src/model.zig:2352-2358).
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ x,
                             int dim, int vocab, float scale, int* status) {
  zk_let_next_start();
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int t = blockIdx.x;
  const int tok = tokens[t];
  const bool ok = tok >= 0 && tok < vocab;
  if (!ok && threadIdx.x == 0) atomicExch(status, 1);
  const T* row = table + (size_t)(ok ? tok : 0) * dim;
  float* out = x + (size_t)t * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) out[d] = ok ? to_f32(row[d]) * scale : 0.f;
}

// y[r, :] = (x[src(r), :] * rsqrt(mean(x^2) + eps)) * w   (src/model.zig:1166-1181: scale
// first, weight second).  src(r) = rows ? rows[r] : r.  One block per output row.
template <typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ w,
                               TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
  float ss = 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    const float v = xr[d];
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* yr = y + (size_t)r * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) yr[d] = from_f32<TO>((xr[d] * scale) * w[d]);
}

// The same with 16-byte loads and the row kept in registers between the sum and the scaling
// (dim a multiple of 4, at most 16 values per thread).  The sum of squares is added per thread
// over its float4s in order, then over the block as above.
template <typename TO>
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                    const float* __restrict__ w, TO* __restrict__ y, int dim, float eps) {
  __shared__ float scratch[32];
  const int r = blockIdx.x;
  zk_let_next_start();
  zk_wait_prior();   // x is the kernel before's result
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * dim);
  const int n4 = dim >> 2;
  float4 v[4];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    v[i] = d < n4 ? xr[d] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    ss = fmaf(v[i].x, v[i].x, ss);
    ss = fmaf(v[i].y, v[i].y, ss);
    ss = fmaf(v[i].z, v[i].z, ss);
    ss = fmaf(v[i].w, v[i].w, ss);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
  TO* yr = y + (size_t)r * dim;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int d = threadIdx.x + i * blockDim.x;
    if (d >= n4) continue;
    const float4 wv = reinterpret_cast<const float4*>(w)[d];
    const float o0 = (v[i].x * scale) * wv.x, o1 = (v[i].y * scale) * wv.y, o2 = (v[i].z * scale) * wv.z,
                o3 = (v[i].w * scale) * wv.w;
    if constexpr (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(yr)[d] = make_float4(o0, o1, o2, o3);
    } else {
      __nv_bfloat162 p[2] = {__floats2bfloat162_rn(o0, o1), __floats2bfloat162_rn(o2, o3)};
      reinterpret_cast<uint2*>(yr)[d] = *reinterpret_cast<const uint2*>(p);
    }
  }
}

// h[t, f] = silu(gate_f) * up_f, silu(g) = g / (1 + exp(-g)) (src/ffn.zig:31-33, 49-57).
// A row of gu holds [gate (F) | up (F)] (il = 0), or groups of il gates followed by their il ups
// (il > 0, the layout the fused contraction kernels want).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ h, int n, int F, int il) {
  const size_t total = (size_t)n * F;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t t = i / F, f = i - t * F;
    const size_t gi = il ? (f / il) * 2 * il + f % il : f;
    const size_t ui = il ? gi + il : F + f;
    const float g = to_f32(gu[t * 2 * F + gi]);
    const float u = to_f32(gu[t * 2 * F + ui]);
    h[i] = from_f32<T>(g / (1.0f + expf(-g)) * u);
  }
}

// out[i] = mean + std * n_i with n_i standard normal, a function of (seed, i) only: two hashed
// uniforms through Box-Muller.  Fills large random models on the device in milliseconds.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

template <typename T>
__global__ void fill_normal_kernel(T* __restrict__ out, size_t n, unsigned long long seed, float mean, float std) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const unsigned long long h = splitmix64(seed ^ splitmix64(i));
    const float u1 = ((float)(unsigned)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
    const float u2 = (float)(unsigned)((h >> 8) & 0xFFFFFF) * (1.0f / 16777216.0f);  // [0, 1)
    out[i] = from_f32<T>(mean + std * sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2));
  }
}

extern "C" {

int zk_fill_normal(void* out, long long n, long long seed, float mean, float std, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  const long long want = (n + threads - 1) / threads;
  const int blocks = (int)(want < 148 * 32 ? want : 148 * 32);
  if (dtype == ZK_F32)
    fill_normal_kernel<float><<<blocks, threads, 0, stream>>>((float*)out, (size_t)n, (unsigned long long)seed, mean, std);
  else if (dtype == ZK_BF16)
    fill_normal_kernel<bf16><<<blocks, threads, 0, stream>>>((bf16*)out, (size_t)n, (unsigned long long)seed, mean, std);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

// Name of a status returned by any zk_* launcher (a cudaError_t value, or ZK_EINVAL).
const char* zk_error_name(int code) {
  if (code == ZK_EINVAL) return "ZK_EINVAL (a size or dtype the kernel does not take)";
  return cudaGetErrorName((cudaError_t)code);
}

int zk_embed(const int* tokens, const void* table, float* x, int n, int dim, int vocab, float scale, int dtype,
             int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dim <= 0 || vocab <= 0) return ZK_EINVAL;
  const int threads = dim >= 1024 ? 256 : 128;
  if (dtype == ZK_F32)
    embed_kernel<float><<<n, threads, 0, stream>>>(tokens, (const float*)table, x, dim, vocab, scale, status);
  else if (dtype == ZK_BF16)
    embed_kernel<bf16><<<n, threads, 0, stream>>>(tokens, (const bf16*)table, x, dim, vocab, scale, status);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_rmsnorm(const float* x, const int* rows, const float* w, void* y, int n_out, int dim, float eps, int out_dtype,
               cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (dim <= 0) return ZK_EINVAL;
  int threads = 32;
  while (threads < 256 && threads * 4 < dim) threads <<= 1;
  const bool aligned = (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y)) % 16 == 0;
  if (dim % 4 == 0 && dim <= 16 * threads && aligned && (out_dtype == ZK_F32 || out_dtype == ZK_BF16)) {
    while (threads > 32 && threads * 4 >= 2 * dim) threads >>= 1;   // no idle warps for short rows
    if (out_dtype == ZK_F32)
      return zk_launch_dependent(rmsnorm_vec4_kernel<float>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, (float*)y, dim, eps);
    return zk_launch_dependent(rmsnorm_vec4_kernel<bf16>, dim3(n_out), dim3(threads), 0, stream, x, rows, w, (bf16*)y, dim, eps);
  }
  if (out_dtype == ZK_F32)
    rmsnorm_kernel<float><<<n_out, threads, 0, stream>>>(x, rows, w, (float*)y, dim, eps);
  else if (out_dtype == ZK_BF16)
    rmsnorm_kernel<bf16><<<n_out, threads, 0, stream>>>(x, rows, w, (bf16*)y, dim, eps);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

int zk_silu_mul(const void* gu, void* h, int n, int F, int il, int dtype, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (F <= 0 || il < 0 || (il > 0 && F % il)) return ZK_EINVAL;
  const size_t total = (size_t)n * F;
  const int threads = 256;
  const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
  if (dtype == ZK_F32)
    silu_mul_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)h, n, F, il);
  else if (dtype == ZK_BF16)
    silu_mul_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)h, n, F, il);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

}  // extern "C"
