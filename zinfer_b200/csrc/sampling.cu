// Sampling on the device, one thread block per row of float32 logits [n, V].
//
// The reference's chain (src/sampler.zig:36-37, 190-276): repetition penalty, DRY penalty,
// greedy if temp <= 0, else top-k, top-p and min-p on untempered probabilities relative to the
// best logit, temperature on the survivors, XTC, then one draw.  The reference sorts the
// candidates; here nothing is sorted.  Every filter keeps a prefix of the descending order
// (ties in index order, as a stable sort leaves them), and such a prefix is described by a
// threshold value and, for ties, an index cut.  The thresholds are found by radix selection
// over the order-preserving bit pattern of the floats: 4 passes of 8 bits, counting elements
// for top-k and summing probability mass for top-p.  The draw walks the survivors in index
// order (the reference walks them in descending order; the distribution is the same).
//
// The penalties are sparse: the host computes which tokens are penalised (distinct recent
// tokens; DRY continuation tokens with their penalty) and `zk_apply_penalties` edits those
// logits in place (src/sampler.zig:91-100, 171-181).
#include "common.cuh"
#include <math.h>

#define SAMP_THREADS 1024
#define NO_CUT 0x7fffffff

namespace {

__device__ __forceinline__ unsigned key_of(float f) {
  if (f != f) f = -INFINITY;  // NaN never wins
  const unsigned u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float float_of_key(unsigned k) {
  const unsigned u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// A logit with NaN read as -inf, so that it never wins and carries no mass.
__device__ __forceinline__ float ld(const float* row, int i) {
  const float v = row[i];
  return v == v ? v : -INFINITY;
}

// A prefix of the descending order: key > T, or key == T and index <= cut.
struct Prefix {
  unsigned T;
  int cut;
  __device__ __forceinline__ bool has(unsigned key, int idx) const { return key > T || (key == T && idx <= cut); }
};

// Bin masses are summed as integers (units of 2^-40 of the largest probability), so that a sum
// does not depend on the order in which the threads' atomic adds arrive: the same row and seed
// give the same cut in every run.  A mass is at most 1, so 2^24 of them fit.
constexpr float MASS_UNIT = 1099511627776.0f;    // 2^40

struct Shared {
  unsigned long long mbins[256];
  int ibins[256];
  float fred[32];
  int ired[32];
  float fval;
  int ival, ival2;
  unsigned uval;
};

__device__ float block_reduce_sum(float v, Shared& sh) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.fred[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh.fred[threadIdx.x & 31] : 0.f;
  return warp_sum(t);
}

__device__ float block_reduce_max(float v, Shared& sh) {
  v = warp_max(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.fred[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh.fred[threadIdx.x & 31] : -INFINITY;
  return warp_max(t);
}

__device__ int block_reduce_isum(int v, Shared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.ired[threadIdx.x >> 5] = v;
  __syncthreads();
  int t = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh.ired[threadIdx.x & 31] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ int block_reduce_imin(int v, Shared& sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = min(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh.ired[threadIdx.x >> 5] = v;
  __syncthreads();
  int t = (threadIdx.x & 31) < (blockDim.x >> 5) ? sh.ired[threadIdx.x & 31] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

__device__ int block_reduce_imax(int v, Shared& sh) { return -block_reduce_imin(-v, sh); }

// Inclusive scan of one float per thread over the block, in thread order; also the block total.
__device__ float block_scan_incl(float v, Shared& sh, float* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  __syncthreads();
  if (lane == 31) sh.fred[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < (blockDim.x >> 5) ? sh.fred[lane] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += n;
    }
    sh.fred[lane] = w;
  }
  __syncthreads();
  *total = sh.fred[(blockDim.x >> 5) - 1];
  return v + (warp > 0 ? sh.fred[warp - 1] : 0.f);
}

// Index of the m-th (1-based) element, in index order, with key == T and index <= limit_cut.
__device__ int nth_equal(const float* row, int V, unsigned T, int limit_cut, int m, Shared& sh) {
  int seen = 0;
  for (int base = 0; base < V; base += blockDim.x) {
    const int i = base + threadIdx.x;
    const bool eq = i < V && i <= limit_cut && key_of(ld(row, i)) == T;
    float tot;
    const float incl = block_scan_incl(eq ? 1.f : 0.f, sh, &tot);
    const int hit = (eq && seen + (int)incl == m) ? i : 0x7fffffff;
    const int first = block_reduce_imin(hit, sh);
    if (first != 0x7fffffff) return first;
    seen += (int)tot;
  }
  return limit_cut;
}

// Top-k prefix by counting radix selection.
__device__ Prefix select_top_k(const float* row, int V, int k, Shared& sh) {
  unsigned prefix = 0, mask = 0;
  int k_rem = k, count_eq = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.ibins[b] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const unsigned key = key_of(ld(row, i));
      if ((key & mask) == prefix) atomicAdd(&sh.ibins[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int acc = 0, b = 255;
      for (; b > 0; --b) {
        if (acc + sh.ibins[b] >= k_rem) break;
        acc += sh.ibins[b];
      }
      sh.ival = b;
      sh.ival2 = k_rem - acc;
    }
    __syncthreads();
    const int b = sh.ival;
    k_rem = sh.ival2;
    count_eq = sh.ibins[b];
    prefix |= (unsigned)b << shift;
    mask |= 255u << shift;
    __syncthreads();
  }
  Prefix p{prefix, NO_CUT};
  if (k_rem < count_eq) p.cut = nth_equal(row, V, prefix, NO_CUT, k_rem, sh);
  return p;
}

// Top-p prefix inside `in`: the shortest prefix whose mass exp(l - mx) reaches top_p * total.
__device__ Prefix select_top_p(const float* row, int V, const Prefix& in, float mx, float top_p, Shared& sh) {
  float total = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float l = ld(row, i);
    if (in.has(key_of(l), i)) total += expf(l - mx);
  }
  total = block_reduce_sum(total, sh);
  float target = top_p * total;
  unsigned prefix = 0, mask = 0;
  int count_eq = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) {
      sh.ibins[b] = 0;
      sh.mbins[b] = 0ull;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = ld(row, i);
      const unsigned key = key_of(l);
      if ((key & mask) == prefix && in.has(key, i)) {
        atomicAdd(&sh.ibins[(key >> shift) & 255], 1);
        atomicAdd(&sh.mbins[(key >> shift) & 255], (unsigned long long)(expf(l - mx) * MASS_UNIT));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      float acc = 0.f;
      int b = 255, lowest = 255;
      for (int j = 255; j >= 0; --j)
        if (sh.ibins[j] > 0) lowest = j;
      for (; b > lowest; --b) {
        const float mass = (float)sh.mbins[b] * (1.0f / MASS_UNIT);
        if (sh.ibins[b] > 0 && acc + mass >= target) break;
        acc += mass;
      }
      sh.ival = b;
      sh.fval = target - acc;
    }
    __syncthreads();
    const int b = sh.ival;
    target = sh.fval;
    count_eq = sh.ibins[b];
    prefix |= (unsigned)b << shift;
    mask |= 255u << shift;
    __syncthreads();
  }
  // `count_eq` elements of `in` equal the threshold, each of mass e; take as many as the target needs
  const float e = expf(float_of_key(prefix) - mx);
  int m = e > 0.f ? (int)ceilf(target / e) : count_eq;
  m = max(1, min(m, count_eq));
  Prefix p{prefix, prefix == in.T ? in.cut : NO_CUT};
  if (m < count_eq) p.cut = nth_equal(row, V, prefix, p.cut, m, sh);
  return p;
}

}  // namespace

// logits[row][tok] edited in place: repetition penalty l > 0 ? l / F : l * F for the listed
// tokens (distinct, -1 = none), then logits[row][tok] -= pen for the DRY pairs.
__global__ void penalties_kernel(float* __restrict__ logits, int V, const int* __restrict__ rep_tokens, int R,
                                 float rep_penalty, const int* __restrict__ dry_tokens,
                                 const float* __restrict__ dry_pen, int P) {
  float* row = logits + (size_t)blockIdx.x * V;
  if (rep_tokens && rep_penalty != 1.0f)
    for (int j = threadIdx.x; j < R; j += blockDim.x) {
      const int t = rep_tokens[(size_t)blockIdx.x * R + j];
      if (t >= 0 && t < V) row[t] = row[t] > 0.f ? row[t] / rep_penalty : row[t] * rep_penalty;
    }
  __syncthreads();
  if (dry_tokens)
    for (int j = threadIdx.x; j < P; j += blockDim.x) {
      const int t = dry_tokens[(size_t)blockIdx.x * P + j];
      if (t >= 0 && t < V) row[t] -= dry_pen[(size_t)blockIdx.x * P + j];
    }
}

// Lowest index among the largest logits of each row (src/sampler.zig:532-610).  `feed`, if given, gets
// the same indices (the token slots of the next step's batch description); `status`, if given, is
// copied behind the n indices of `out`, so that one device-to-host copy brings tokens and status.
// A row is cut into gridDim.y pieces, a block each: a block folds its best (value, index) into a
// 64-bit key, larger value first and lower index second, and takes the maximum into the row's word of
// `keys`; the block that finds itself the last of all writes the tokens and leaves the keys and the
// counter zero for the next launch.  The result does not depend on the order of the blocks.
__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
  unsigned u = __float_as_uint(v);
  u = (v != v) ? 0u : ((u & 0x80000000u) ? ~u : (u | 0x80000000u));   // ordered as the values; NaN lowest
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)idx);
}

__global__ void argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, int* __restrict__ feed,
                              const int* __restrict__ status, unsigned long long* __restrict__ keys,
                              unsigned* __restrict__ counter) {
  __shared__ Shared sh;
  __shared__ int sm_last;
  zk_let_next_start();
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int n = gridDim.x, pieces = gridDim.y;
  const float* row = logits + (size_t)blockIdx.x * V;
  const int per = (V + pieces - 1) / pieces, lo = blockIdx.y * per, hi = min(V, lo + per);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    float v = row[i];
    if (v != v) v = -INFINITY;
    if (v > best || (v == best && i < best_i)) {
      best = v;
      best_i = i;
    }
  }
  const float mx = block_reduce_max(best, sh);
  const int idx = block_reduce_imin(best == mx ? best_i : 0x7fffffff, sh);
  if (threadIdx.x == 0) {
    if (idx != 0x7fffffff) atomicMax(keys + blockIdx.x, argmax_key(mx, idx));
    __threadfence();
    sm_last = atomicAdd(counter, 1u) == (unsigned)(n * pieces - 1);
  }
  __syncthreads();
  if (sm_last) {
    __threadfence();
    for (int r = threadIdx.x; r < n; r += blockDim.x) {
      const unsigned long long k = __ldcg(keys + r);
      const int tok = k ? (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull)) : 0;
      out[r] = tok;
      if (feed) feed[r] = tok;
      keys[r] = 0ull;
    }
    if (threadIdx.x == 0) {
      if (status) out[n] = *status;
      *counter = 0u;
    }
  }
}

// One draw per row.  uniforms[row] = {u for the draw, u for the XTC chance}, both in [0, 1).
__global__ void __launch_bounds__(SAMP_THREADS)
    sample_kernel(const float* __restrict__ logits, int V, float temp, int top_k, float top_p, float min_p,
                  float xtc_probability, float xtc_threshold, int xtc_min_keep, const float* __restrict__ uniforms,
                  int* __restrict__ out) {
  __shared__ Shared sh;
  const float* row = logits + (size_t)blockIdx.x * V;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v == v) mx = fmaxf(mx, v);
  }
  mx = block_reduce_max(mx, sh);

  Prefix keep{0u, NO_CUT};  // everything
  if (top_k > 0 && top_k < V) keep = select_top_k(row, V, top_k, sh);
  if (top_p < 1.0f) keep = select_top_p(row, V, keep, mx, top_p, sh);

  // min-p is a predicate on the value; the best logit always passes (keep >= 1)
  const float inv_t = 1.0f / temp;
  float total = 0.f;
  int n_keep = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float l = ld(row, i);
    if (keep.has(key_of(l), i) && (min_p <= 0.f || l == mx || expf(l - mx) >= min_p)) {
      total += expf((l - mx) * inv_t);
      ++n_keep;
    }
  }
  total = block_reduce_sum(total, sh);
  n_keep = block_reduce_isum(n_keep, sh);

  // XTC: with the given chance drop every survivor whose probability reaches the threshold,
  // except the least probable of them (src/sampler.zig:244-268).
  unsigned xtc_key = 0xffffffffu;  // survivors with key > xtc_key, or == and index < xtc_idx, are dropped
  int xtc_idx = -1;
  if (xtc_probability > 0.f && xtc_threshold <= 0.5f && n_keep >= 2 && total > 0.f &&
      uniforms[(size_t)blockIdx.x * 2 + 1] <= xtc_probability) {
    const float inv_tot = 1.0f / total;
    int n_top = 0;
    float min_l = INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = ld(row, i);
      if (keep.has(key_of(l), i) && (min_p <= 0.f || l == mx || expf(l - mx) >= min_p) &&
          expf((l - mx) * inv_t) * inv_tot >= xtc_threshold) {
        ++n_top;
        min_l = fminf(min_l, l);
      }
    }
    n_top = block_reduce_isum(n_top, sh);
    min_l = -block_reduce_max(-min_l, sh);
    const int pos_last = n_top > 0 ? n_top - 1 : 0;
    if (pos_last > 0 && n_keep - pos_last >= max(1, xtc_min_keep)) {
      int last_idx = -1;
      for (int i = threadIdx.x; i < V; i += blockDim.x)
        if (ld(row, i) == min_l && keep.has(key_of(min_l), i)) last_idx = max(last_idx, i);
      xtc_idx = block_reduce_imax(last_idx, sh);
      xtc_key = key_of(min_l);
      total = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = ld(row, i);
        const unsigned key = key_of(l);
        const bool dropped = key > xtc_key || (key == xtc_key && i < xtc_idx);
        if (!dropped && keep.has(key, i) && (min_p <= 0.f || l == mx || expf(l - mx) >= min_p))
          total += expf((l - mx) * inv_t);
      }
      total = block_reduce_sum(total, sh);
    }
  }

  // draw: first survivor, in index order, at which the running sum reaches u * total
  const float r = uniforms[(size_t)blockIdx.x * 2] * total;
  float offset = 0.f;
  int last_member = -1, picked = 0x7fffffff;
  for (int base = 0; base < V; base += blockDim.x) {
    const int i = base + threadIdx.x;
    float w = 0.f;
    bool member = false;
    if (i < V) {
      const float l = ld(row, i);
      const unsigned key = key_of(l);
      const bool dropped = key > xtc_key || (key == xtc_key && i < xtc_idx);
      member = !dropped && keep.has(key, i) && (min_p <= 0.f || l == mx || expf(l - mx) >= min_p);
      if (member) w = expf((l - mx) * inv_t);
    }
    float chunk_total;
    const float incl = block_scan_incl(w, sh, &chunk_total);
    const int hit = (member && offset + incl >= r) ? i : 0x7fffffff;
    picked = block_reduce_imin(hit, sh);
    last_member = max(last_member, block_reduce_imax(member ? i : -1, sh));
    if (picked != 0x7fffffff) break;
    offset += chunk_total;
  }
  if (threadIdx.x == 0) out[blockIdx.x] = picked != 0x7fffffff ? picked : max(last_member, 0);
}

extern "C" {

int zk_apply_penalties(float* logits, int n, int V, const int* rep_tokens, int R, float rep_penalty,
                       const int* dry_tokens, const float* dry_pen, int P, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || R < 0 || P < 0) return ZK_EINVAL;
  penalties_kernel<<<n, 128, 0, stream>>>(logits, V, rep_tokens, R, rep_penalty, dry_tokens, dry_pen, P);
  return ZK_LAUNCH_STATUS();
}

// out [n] (or [n + 1] with `status`: out[n] = *status); feed [n] or null.  `scratch` holds n 64-bit keys
// and, behind them, one 32-bit counter, all zero before the launch and again after it.
int zk_argmax(const float* logits, int n, int V, int* out, int* feed, const int* status, void* scratch,
              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || !scratch) return ZK_EINVAL;
  // a few SMs' worth of blocks per step: a row of 65,536 logits is cut into 16 pieces
  const int pieces = V >= 16384 ? 16 : (V >= 4096 ? 4 : 1);
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(scratch);
  return zk_launch_dependent(argmax_kernel, dim3(n, pieces), dim3(256), 0, stream, logits, V, out, feed, status, keys,
                             reinterpret_cast<unsigned*>(keys + n));
}

int zk_sample(const float* logits, int n, int V, float temp, int top_k, float top_p, float min_p,
              float xtc_probability, float xtc_threshold, int xtc_min_keep, const float* uniforms, int* out,
              cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || !(temp > 0.f) || top_k < 0 || !uniforms) return ZK_EINVAL;
  sample_kernel<<<n, SAMP_THREADS, 0, stream>>>(logits, V, temp, top_k, top_p, min_p, xtc_probability, xtc_threshold,
                                                xtc_min_keep, uniforms, out);
  return ZK_LAUNCH_STATUS();
}

}  // extern "C"
