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

// One pass of a radix selection over the whole row.  Four loads are under way per thread (one at a
// time, a pass is the memory's latency V / threads times), and the lanes of a warp that hit the same
// bin add to it as one: in the first pass nearly every element falls into two or three bins (the
// upper bits of a float are its sign and exponent), and 65,536 atomic adds to three shared-memory
// words, the 64-bit ones by compare-and-swap, took a millisecond.
// f(i, l, &bin, &mass) says whether element i takes part, in which bin, with what mass.
template <typename F>
__device__ __forceinline__ void radix_pass(const float* row, int V, Shared& sh, bool with_mass, F f) {
  constexpr int UN = 4;
  const int lane = threadIdx.x & 31;
  for (int base = 0; base < V; base += blockDim.x * UN) {
    float v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      v[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + u * blockDim.x + threadIdx.x;
      unsigned bin = 0xffffffffu;
      unsigned long long mass = 0ull;
      const bool act = i < V && f(i, v[u] == v[u] ? v[u] : -INFINITY, &bin, &mass);
      if (!__any_sync(0xffffffffu, act)) continue;
      const unsigned peers = __match_any_sync(0xffffffffu, act ? bin : 0xffffffffu);
      if (act) {
        unsigned lo = 0, hi = 0;
        if (with_mass) {     // a mass has at most 41 bits: two sums of 32 lanes' halves fit 32 bits each
          lo = __reduce_add_sync(peers, (unsigned)(mass & 0xFFFFFull));
          hi = __reduce_add_sync(peers, (unsigned)(mass >> 20));
        }
        if (lane == __ffs(peers) - 1) {
          atomicAdd(&sh.ibins[bin], __popc(peers));
          if (with_mass) atomicAdd(&sh.mbins[bin], ((unsigned long long)hi << 20) + lo);
        }
      }
    }
  }
}

// Top-k prefix by counting radix selection.
__device__ Prefix select_top_k(const float* row, int V, int k, Shared& sh) {
  unsigned prefix = 0, mask = 0;
  int k_rem = k, count_eq = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = threadIdx.x; b < 256; b += blockDim.x) sh.ibins[b] = 0;
    __syncthreads();
    radix_pass(row, V, sh, false, [&](int, float l, unsigned* bin, unsigned long long*) {
      const unsigned key = key_of(l);
      *bin = (key >> shift) & 255;
      return (key & mask) == prefix;
    });
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
    radix_pass(row, V, sh, true, [&](int i, float l, unsigned* bin, unsigned long long* mass) {
      const unsigned key = key_of(l);
      if ((key & mask) != prefix || !in.has(key, i)) return false;
      *bin = (key >> shift) & 255;
      *mass = (unsigned long long)(expf(l - mx) * MASS_UNIT);
      return true;
    });
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

// `ring`, if given, holds [ring_slots][n + 1] words: the finalising block also writes the tokens and the
// status word into slot (*ring_pos % ring_slots) and adds one to *ring_pos.  The host, which counts the
// launches too, can then fetch a step's result from its slot on another stream while later steps
// (recorded with the same pointers) run on and fill other slots: no copy has to be queued between two
// steps.  (Pinned host memory as the ring works too, but a kernel that ends on writes to the host held
// up the step behind it by some 25 us.)
__global__ void argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out, int* __restrict__ feed,
                              const int* __restrict__ status, unsigned long long* __restrict__ keys,
                              unsigned* __restrict__ counter, int* __restrict__ ring, int ring_slots,
                              unsigned* __restrict__ ring_pos) {
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
    int* slot = ring ? ring + (size_t)(*ring_pos % (unsigned)ring_slots) * (n + 1) : nullptr;
    for (int r = threadIdx.x; r < n; r += blockDim.x) {
      const unsigned long long k = __ldcg(keys + r);
      const int tok = k ? (int)(0xFFFFFFFFu - (unsigned)(k & 0xFFFFFFFFull)) : 0;
      out[r] = tok;
      if (feed) feed[r] = tok;
      if (slot) slot[r] = tok;
      keys[r] = 0ull;
    }
    __syncthreads();     // every thread has read *ring_pos
    if (threadIdx.x == 0) {
      const int st = status ? *status : 0;
      if (status) out[n] = st;
      if (slot) {
        slot[n] = st;
        *ring_pos = *ring_pos + 1u;
      }
      *counter = 0u;
    }
  }
}

// The host's sampling.sampler.uniform(seed, request, draw, stream): a float32 in [0, 1) that is a
// function of its four arguments only.
__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}
__device__ __forceinline__ float counter_uniform(unsigned long long seed, int request, int draw, int stream) {
  unsigned long long h = mix64(seed);
  h = mix64(h ^ (unsigned long long)(unsigned)request);
  h = mix64(h ^ (unsigned long long)(unsigned)draw);
  h = mix64(h ^ (unsigned long long)stream);
  return (float)(h >> 40) * (1.0f / 16777216.0f);
}

// ---------------------------------------------------------------------------------------
// The chain on a short list.  When the filters can only keep tokens among the CAND_MAX best
// (top-k of at most CAND_MAX; or top-p / min-p whose survivors are seen to lie among them),
// the row is read twice (a histogram of the keys' upper 11 bits, then a gather of everything
// at or above the bin in which the k-th best lies) and the rest of the chain runs on that list
// in shared memory: the same prefixes, ties, predicates and index-order draw as the passes over
// the whole row further down, at a tenth of their time.
constexpr int CAND_MAX = 1024;
constexpr int HIST_BITS = 11, HIST_BINS = 1 << HIST_BITS;

struct Small {
  float l[CAND_MAX];       // candidates in index order
  int idx[CAND_MAX];
  float l2[CAND_MAX];      // as gathered
  int idx2[CAND_MAX];
  float w[CAND_MAX];       // masses exp(l - mx), then weights exp((l - mx) / temp)
  unsigned char in[CAND_MAX];
  int hist[HIST_BINS];
  int count, bin, above;
};

// Returns false, with nothing decided, if the list does not suffice; the caller then takes the
// passes over the whole row.  k_eff: how many of the best the top-k stage keeps (V if it is off).
__device__ bool sample_small(const float* row, int V, int k_eff, float temp, float top_p, float min_p,
                             float xtc_probability, float xtc_threshold, int xtc_min_keep, float u_draw, float u_xtc,
                             Shared& sh, Small& sm, int* picked_out) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int k_list = min(k_eff, CAND_MAX);           // the list holds the k_list best
  // 1. histogram of the upper bits; equal bins of a warp are added as one
  for (int b = tid; b < HIST_BINS; b += blockDim.x) sm.hist[b] = 0;
  if (tid == 0) sm.count = 0;
  __syncthreads();
  // (sixteen loads under way per thread: one at a time, a pass over the row is its latency 64 times)
  constexpr int UN = 16;
  for (int base = 0; base < V; base += blockDim.x * UN) {
    float v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + u * blockDim.x + tid;
      v[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u)
      if (base + u * blockDim.x + tid < V) atomicAdd(&sm.hist[key_of(v[u]) >> (32 - HIST_BITS)], 1);
  }
  __syncthreads();
  // 2. the bin of the k_list-th best: warp 0, lane j owns bins [HIST_BINS - 64 (j + 1), HIST_BINS - 64 j)
  if (tid < 32) {
    constexpr int PER = HIST_BINS / 32;
    const int top = HIST_BINS - PER * lane;           // one past this lane's highest bin
    int mine = 0;
    for (int b = top - 1; b >= top - PER; --b) mine += sm.hist[b];
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    const int before = incl - mine;                    // elements in bins above this lane's
    if (before < k_list && incl >= k_list) {           // exactly one lane (V >= k_list elements exist)
      int acc = before, b = top - 1;
      for (; b > top - PER; --b) {
        if (acc + sm.hist[b] >= k_list) break;
        acc += sm.hist[b];
      }
      sm.bin = b;
      sm.above = acc;
    }
  }
  __syncthreads();
  const int bin0 = sm.bin;
  const int n_c = sm.above + sm.hist[bin0];
  if (n_c > CAND_MAX) return false;                    // too many values share the deciding bin
  // 3. gather everything at or above that bin
  for (int base = 0; base < V; base += blockDim.x * UN) {
    float v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + u * blockDim.x + tid;
      v[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + u * blockDim.x + tid;
      if (i < V && (int)(key_of(v[u]) >> (32 - HIST_BITS)) >= bin0) {
        const int pos = atomicAdd(&sm.count, 1);
        sm.l2[pos] = v[u] == v[u] ? v[u] : -INFINITY;     // NaN read as -inf, as ld() does
        sm.idx2[pos] = i;
      }
    }
  }
  __syncthreads();
  // 4. into index order (the gather's order is whatever the atomics made it)
  if (tid < n_c) {
    const int my = sm.idx2[tid];
    int rank = 0;
    for (int j = 0; j < n_c; ++j) rank += sm.idx2[j] < my;
    sm.l[rank] = sm.l2[tid];
    sm.idx[rank] = my;
  }
  __syncthreads();
  // 5. the k_list best of them: descending value, ties in index order
  const bool have = tid < n_c;
  const float my_l = have ? sm.l[tid] : -INFINITY;
  const unsigned my_key = key_of(my_l);
  int rank_desc = 0;
  if (have)
    for (int j = 0; j < n_c; ++j) {
      const unsigned kj = key_of(sm.l[j]);
      rank_desc += kj > my_key || (kj == my_key && j < tid);
    }
  bool member = have && rank_desc < k_list;
  const float mx = block_reduce_max(member ? my_l : -INFINITY, sh);
  const float e = member ? expf(my_l - mx) : 0.f;
  auto minp_ok = [&](float l, float mass) { return min_p <= 0.f || l == mx || mass >= min_p; };
  // 6. top-p: the shortest prefix of the descending order whose mass reaches top_p * total
  sm.w[tid < CAND_MAX ? tid : 0] = 0.f;                 // (blockDim.x == CAND_MAX)
  __syncthreads();
  if (have) sm.w[tid] = e;
  sm.in[tid] = member;
  __syncthreads();
  float total_e = block_reduce_sum(e, sh);               // a fixed order of additions: the same in every run
  if (k_eff > k_list) {
    // The list is a cut of a longer candidate set: the mass is the whole row's, and the list must be
    // seen to hold every survivor (the prefix ends inside it, or its last member already fails min-p).
    float all = 0.f;
    for (int i = tid; i < V; i += blockDim.x) all += expf(ld(row, i) - mx);
    all = block_reduce_sum(all, sh);
    const bool prefix_inside = top_p < 1.0f && total_e >= top_p * all;
    const float lowest = -block_reduce_max(member ? -my_l : -INFINITY, sh);
    const bool minp_cuts = min_p > 0.f && !minp_ok(lowest, expf(lowest - mx));
    if (!prefix_inside && !minp_cuts) return false;
    total_e = all;
  }
  if (top_p < 1.0f) {
    const float target = top_p * total_e;
    float before = 0.f;
    if (member)
      for (int j = 0; j < n_c; ++j) {
        const unsigned kj = key_of(sm.l[j]);
        if (sm.in[j] && (kj > my_key || (kj == my_key && j < tid))) before += sm.w[j];
      }
    member = member && before < target;
  }
  const bool in_prefix = member;          // after top-k and top-p, before min-p
  // 7. min-p on the value, temperature on the survivors
  member = member && minp_ok(my_l, e);
  const float inv_t = 1.0f / temp;
  float wgt = member ? expf((my_l - mx) * inv_t) : 0.f;
  __syncthreads();
  sm.w[tid] = wgt;
  sm.in[tid] = member;
  __syncthreads();
  float total = block_reduce_sum(wgt, sh);
  const int n_keep = block_reduce_isum(member ? 1 : 0, sh);
  // 8. XTC (src/sampler.zig:244-268): drop every survivor whose probability reaches the threshold
  //    except the least probable of them
  if (xtc_probability > 0.f && xtc_threshold <= 0.5f && n_keep >= 2 && total > 0.f && u_xtc <= xtc_probability) {
    const float inv_tot = 1.0f / total;
    const bool is_top = member && wgt * inv_tot >= xtc_threshold;
    const int n_top = block_reduce_isum(is_top ? 1 : 0, sh);
    const float min_l = -block_reduce_max(is_top ? -my_l : -INFINITY, sh);
    const int pos_last = n_top > 0 ? n_top - 1 : 0;
    if (pos_last > 0 && n_keep - pos_last >= max(1, xtc_min_keep)) {
      // the last of the tops in the descending order: the lowest value, the highest index among its ties
      const int last_idx = block_reduce_imax((in_prefix && my_l == min_l) ? sm.idx[tid] : -1, sh);
      const unsigned xk = key_of(min_l);
      const bool dropped = my_key > xk || (my_key == xk && have && sm.idx[tid] < last_idx);
      if (dropped) {
        member = false;
        wgt = 0.f;
      }
      __syncthreads();
      sm.w[tid] = wgt;
      sm.in[tid] = member;
      __syncthreads();
      total = block_reduce_sum(wgt, sh);
    }
  }
  // 9. the draw: first survivor, in index order, at which the running sum reaches u * total
  const float r = u_draw * total;
  float incl = 0.f;
  if (have)
    for (int j = 0; j <= tid; ++j) incl += sm.w[j];
  const int picked = block_reduce_imin((member && incl >= r) ? sm.idx[tid] : 0x7fffffff, sh);
  const int last_member = block_reduce_imax(member ? sm.idx[tid] : -1, sh);
  *picked_out = picked != 0x7fffffff ? picked : max(last_member, 0);
  return true;
}

// One draw per row.  Its two uniforms in [0, 1) (one for the draw, one for the XTC chance) are
// uniforms[row] if given; else they are computed here from (seed, req_ids[row], draws[req_ids[row]]),
// and that request's count of draws goes up by one: the host then has nothing to send per step.
__global__ void __launch_bounds__(SAMP_THREADS)
    sample_kernel(const float* __restrict__ logits, int V, float temp, int top_k, float top_p, float min_p,
                  float xtc_probability, float xtc_threshold, int xtc_min_keep, const float* __restrict__ uniforms,
                  unsigned long long seed, const int* __restrict__ req_ids, int* __restrict__ draws,
                  int* __restrict__ out) {
  __shared__ Shared sh;
  __shared__ float s_u[2];
  if (threadIdx.x == 0) {
    if (uniforms) {
      s_u[0] = uniforms[(size_t)blockIdx.x * 2];
      s_u[1] = uniforms[(size_t)blockIdx.x * 2 + 1];
    } else {
      const int req = req_ids[blockIdx.x];
      const int d = draws[req];
      s_u[0] = counter_uniform(seed, req, d, 0);
      s_u[1] = counter_uniform(seed, req, d, 1);
      draws[req] = d + 1;
    }
  }
  __syncthreads();
  const float* row = logits + (size_t)blockIdx.x * V;
  {
    __shared__ Small sm;
    const int k_eff = (top_k > 0 && top_k < V) ? top_k : V;
    int picked_small = 0;
    if ((k_eff <= CAND_MAX || top_p < 1.0f || min_p > 0.f) &&
        sample_small(row, V, k_eff, temp, top_p, min_p, xtc_probability, xtc_threshold, xtc_min_keep, s_u[0], s_u[1], sh,
                     sm, &picked_small)) {
      if (threadIdx.x == 0) out[blockIdx.x] = picked_small;
      return;
    }
    __syncthreads();
  }
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
      s_u[1] <= xtc_probability) {
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

  // draw: first survivor, in index order, at which the running sum reaches u * total.  Every warp owns
  // a stretch of the row: the warps' sums say in which stretch the sum reaches the target, and only
  // that warp walks its stretch a second time, scanning 32 weights at a step.
  const float r = s_u[0] * total;
  auto weight_of = [&](int i, float v, bool* member) {
    const float l = v == v ? v : -INFINITY;
    const unsigned key = key_of(l);
    const bool dropped = key > xtc_key || (key == xtc_key && i < xtc_idx);
    *member = !dropped && keep.has(key, i) && (min_p <= 0.f || l == mx || expf(l - mx) >= min_p);
    return *member ? expf((l - mx) * inv_t) : 0.f;
  };
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int stretch = ((V + n_warps - 1) / n_warps + 31) / 32 * 32;
  const int lo = min(V, warp * stretch), hi = min(V, lo + stretch);
  constexpr int UN = 8;
  float wsum = 0.f;
  int wlast = -1;
  for (int base = lo; base < hi; base += 32 * UN) {
    float v[UN];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + 32 * u + lane;
      v[u] = i < hi ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int i = base + 32 * u + lane;
      bool member = false;
      if (i < hi) wsum += weight_of(i, v[u], &member);
      if (member) wlast = i;
    }
  }
  wsum = warp_sum(wsum);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wlast = max(wlast, __shfl_xor_sync(0xffffffffu, wlast, o));
  __syncthreads();
  if (lane == 0) {
    sh.fred[warp] = wsum;
    sh.ired[warp] = wlast;
  }
  __syncthreads();
  float offset = 0.f;          // weight before this warp's stretch, added in warp order by every thread alike
  int target_warp = -1, last_member = -1;
  for (int w = 0; w < n_warps; ++w) {
    if (target_warp < 0 && sh.ired[w] >= 0 && offset + sh.fred[w] >= r) target_warp = w;
    if (target_warp < 0) offset += sh.fred[w];
    last_member = max(last_member, sh.ired[w]);
  }
  if (target_warp < 0) {        // rounding left the target a hair above the whole sum
    if (threadIdx.x == 0) out[blockIdx.x] = max(last_member, 0);
    return;
  }
  if (warp == target_warp) {
    int picked = -1;
    for (int base = lo; base < hi && picked < 0; base += 32) {
      const int i = base + lane;
      bool member = false;
      float w = i < hi ? weight_of(i, row[i], &member) : 0.f;
      float incl = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float nb = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += nb;
      }
      const unsigned hits = __ballot_sync(0xffffffffu, member && offset + incl >= r);
      if (hits) picked = base + __ffs(hits) - 1;
      offset += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) out[blockIdx.x] = picked >= 0 ? picked : wlast;   // wlast: the stretch's last survivor
  }
}

// The repetition penalty from a window kept on the device: recent [requests, RECENT_N] holds each
// request's last tokens as a ring, seen [requests] how many it has had in all.  One warp per row
// penalises every distinct token among the last min(seen, RECENT_N) once (src/sampler.zig:91-100).
constexpr int RECENT_N = 64;

__global__ void penalize_recent_kernel(float* __restrict__ logits, int V, const int* __restrict__ recent,
                                       const int* __restrict__ seen, const int* __restrict__ req_ids, float penalty) {
  __shared__ int win[RECENT_N];
  const int req = req_ids[blockIdx.x];
  const int n = min(seen[req], RECENT_N);
  for (int j = threadIdx.x; j < RECENT_N; j += blockDim.x) win[j] = j < n ? recent[(size_t)req * RECENT_N + j] : -1;
  __syncthreads();
  float* row = logits + (size_t)blockIdx.x * V;
  for (int j = threadIdx.x; j < n; j += blockDim.x) {
    const int tok = win[j];
    bool first = tok >= 0 && tok < V;
    for (int i = 0; i < j && first; ++i) first = win[i] != tok;
    if (first) {
      const float l = row[tok];
      row[tok] = l > 0.f ? l / penalty : l * penalty;
    }
  }
}

// tokens [n] (what the rows just sampled) go into their requests' rings.
__global__ void recent_append_kernel(const int* __restrict__ tokens, int n, int* __restrict__ recent,
                                     int* __restrict__ seen, const int* __restrict__ req_ids) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n) return;
  const int req = req_ids[r];
  const int s = seen[req];
  recent[(size_t)req * RECENT_N + s % RECENT_N] = tokens[r];
  seen[req] = s + 1;
}

extern "C" {

int zk_apply_penalties(float* logits, int n, int V, const int* rep_tokens, int R, float rep_penalty,
                       const int* dry_tokens, const float* dry_pen, int P, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || R < 0 || P < 0) return ZK_EINVAL;
  penalties_kernel<<<n, 128, 0, stream>>>(logits, V, rep_tokens, R, rep_penalty, dry_tokens, dry_pen, P);
  return ZK_LAUNCH_STATUS();
}

int zk_recent_window() { return RECENT_N; }

// logits [n, V] edited in place from the device's windows; req_ids [n] names each row's request.
int zk_penalize_recent(float* logits, int n, int V, const int* recent, const int* seen, const int* req_ids,
                       float penalty, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || !recent || !seen || !req_ids || !(penalty > 0.f)) return ZK_EINVAL;
  penalize_recent_kernel<<<n, 64, 0, stream>>>(logits, V, recent, seen, req_ids, penalty);
  return ZK_LAUNCH_STATUS();
}

int zk_recent_append(const int* tokens, int n, int* recent, int* seen, const int* req_ids, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (!tokens || !recent || !seen || !req_ids) return ZK_EINVAL;
  recent_append_kernel<<<(n + 127) / 128, 128, 0, stream>>>(tokens, n, recent, seen, req_ids);
  return ZK_LAUNCH_STATUS();
}

// out [n] (or [n + 1] with `status`: out[n] = *status); feed [n] or null.  `scratch` holds n 64-bit keys
// and, behind them, one 32-bit counter, all zero before the launch and again after it.
// ring (or null): [ring_slots][n + 1] words, see the kernel; ring_pos: one device word, the number of
// launches with a ring so far.
int zk_argmax(const float* logits, int n, int V, int* out, int* feed, const int* status, void* scratch,
              int* ring, int ring_slots, int* ring_pos, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || !scratch || (ring && (ring_slots <= 0 || !ring_pos))) return ZK_EINVAL;
  // a few SMs' worth of blocks per step: a row of 65,536 logits is cut into 16 pieces
  const int pieces = V >= 16384 ? 16 : (V >= 4096 ? 4 : 1);
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(scratch);
  return zk_launch_dependent(argmax_kernel, dim3(n, pieces), dim3(256), 0, stream, logits, V, out, feed, status, keys,
                             reinterpret_cast<unsigned*>(keys + n), ring, ring_slots,
                             reinterpret_cast<unsigned*>(ring_pos));
}

// uniforms [n, 2], or null and then seed, req_ids [n] (the request of each row; distinct) and
// draws [requests] (how many draws each request has had; the kernel adds one for its rows).
int zk_sample(const float* logits, int n, int V, float temp, int top_k, float top_p, float min_p,
              float xtc_probability, float xtc_threshold, int xtc_min_keep, const float* uniforms,
              long long seed, const int* req_ids, int* draws, int* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V <= 0 || !(temp > 0.f) || top_k < 0 || (!uniforms && (!req_ids || !draws))) return ZK_EINVAL;
  sample_kernel<<<n, SAMP_THREADS, 0, stream>>>(logits, V, temp, top_k, top_p, min_p, xtc_probability, xtc_threshold,
                                                xtc_min_keep, uniforms, (unsigned long long)seed, req_ids, draws, out);
  return ZK_LAUNCH_STATUS();
}

}  // extern "C"
