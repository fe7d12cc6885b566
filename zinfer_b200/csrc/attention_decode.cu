// Attention of single-token steps over the paged bfloat16 cache: one query token per sequence,
// G query heads sharing each KV head.  The step is bound by reading K and V once, so the kernel
// is laid out for that: a block owns (sequence, KV head, chunk of keys); its 4 warps take tiles
// of 32 keys in turn.  For the scores one lane owns one key and reads its whole K row; for P.V
// one lane owns head_dim/32 output columns and the tile's V rows are read coalesced.  Scores,
// softmax and accumulation are float32.  The warps' (m, l, o) are merged in shared memory and
// written either as the result (one chunk) or as a partial for `zk_attn_merge`.
//
// Reference: split of single-token attention into chunks with partial (m, l, o),
// src/model.zig:1941-1955 and src/attention.zig:749-814; the G heads of a KV head are processed
// together, src/model.zig:1352-1366.
#include "common.cuh"
#include <math.h>

#define DEC_WARPS 4
#define DEC_TK 32

namespace {

__device__ __forceinline__ void unpack8(const uint4& v, float f[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}

template <int VPL>
__device__ __forceinline__ void load_v(const bf16* p, float v[VPL]) {
  if constexpr (VPL % 2 == 0) {
#pragma unroll
    for (int i = 0; i < VPL / 2; ++i) {
      const __nv_bfloat162 t = reinterpret_cast<const __nv_bfloat162*>(p)[i];
      v[2 * i] = __low2float(t);
      v[2 * i + 1] = __high2float(t);
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i] = __bfloat162float(p[i]);
  }
}

// VPL = head_dim / 32, G = query heads per KV head.
template <int VPL, int G>
__global__ void __launch_bounds__(DEC_WARPS * 32)
    attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                       bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                       const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                       const int* __restrict__ page_table, int pt_stride, int n_seqs, int Hkv, int page_size,
                       int window, float scale, int num_splits, int split_keys) {
  constexpr int HD = 32 * VPL;
  __shared__ __align__(16) float qs[G][HD];
  __shared__ float sm_m[DEC_WARPS][G], sm_l[DEC_WARPS][G];
  __shared__ float sm_o[DEC_WARPS][G][HD];

  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int H = Hkv * G;
  const int L = seq_start[b] + 1;  // keys 0 .. L-1; the new token's own key is the last
  const int lo = (window > 0 && L > window) ? L - window : 0;
  int c0 = 0, c1 = L;
  if (num_splits > 1) {
    c0 = split * split_keys;
    c1 = min(L, c0 + split_keys);
  }
  const int* pt = page_table + (size_t)seq_slot[b] * pt_stride;

  for (int i = tid; i < G * HD; i += DEC_WARPS * 32)
    qs[i / HD][i % HD] = __bfloat162float(q[(size_t)b * H * HD + (size_t)(kvh * G) * HD + i]) * scale;
  __syncthreads();

  float m[G], l[G], o[G][VPL];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) o[h][i] = 0.f;
  }

  const int first_tile = max(c0, lo) / DEC_TK;
  for (int tile = first_tile + warp; tile * DEC_TK < c1; tile += DEC_WARPS) {
    const int base = tile * DEC_TK;
    const int j_lo = max(max(c0, lo) - base, 0), j_hi = min(c1 - base, DEC_TK);  // valid lanes [j_lo, j_hi)
    const int page = pt[base / page_size];
    if (page < 0 || j_hi <= j_lo) continue;
    const size_t row0 = (((size_t)page * Hkv + kvh) * page_size + base % page_size) * HD;
    const bool valid = lane >= j_lo && lane < j_hi;

    // The tile's K row of this lane and, for head sizes up to 64, all of its V rows are requested
    // before any arithmetic: a warp has few tiles, so what it waits for must be in flight at once.
    constexpr bool PREFETCH_V = VPL <= 2;
    uint4 kv[HD / 8];
    if (valid) {
      const uint4* kr = reinterpret_cast<const uint4*>(k_cache + row0 + (size_t)lane * HD);
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) kv[c] = kr[c];
    }
    const bf16* vr = v_cache + row0 + (size_t)lane * VPL;
    float vpre[PREFETCH_V ? DEC_TK : 1][VPL];
    if constexpr (PREFETCH_V) {
#pragma unroll
      for (int j = 0; j < DEC_TK; ++j) {
        if (j >= j_lo && j < j_hi) {
          load_v<VPL>(vr + (size_t)j * HD, vpre[j]);
        } else {
#pragma unroll
          for (int i = 0; i < VPL; ++i) vpre[j][i] = 0.f;
        }
      }
    }

    // scores: this lane's key against the G query heads
    float s[G];
#pragma unroll
    for (int h = 0; h < G; ++h) s[h] = 0.f;
    if (valid) {
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        float kf[8];
        unpack8(kv[c], kf);
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float4 q0 = *reinterpret_cast<const float4*>(&qs[h][c * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&qs[h][c * 8 + 4]);
          s[h] = fmaf(q0.x, kf[0], s[h]);
          s[h] = fmaf(q0.y, kf[1], s[h]);
          s[h] = fmaf(q0.z, kf[2], s[h]);
          s[h] = fmaf(q0.w, kf[3], s[h]);
          s[h] = fmaf(q1.x, kf[4], s[h]);
          s[h] = fmaf(q1.y, kf[5], s[h]);
          s[h] = fmaf(q1.z, kf[6], s[h]);
          s[h] = fmaf(q1.w, kf[7], s[h]);
        }
      }
    }
    float p[G];
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float sc = valid ? s[h] : -INFINITY;
      const float m_new = fmaxf(m[h], warp_max(sc));
      const float alpha = expf(m[h] - m_new);
      p[h] = valid ? expf(sc - m_new) : 0.f;
      l[h] = l[h] * alpha + warp_sum(p[h]);
      m[h] = m_new;
#pragma unroll
      for (int i = 0; i < VPL; ++i) o[h][i] *= alpha;
    }
    // P.V: V rows of the tile, read coalesced; this lane owns columns lane*VPL .. lane*VPL+VPL-1
#pragma unroll
    for (int j = 0; j < DEC_TK; ++j) {
      float v[VPL];
      if constexpr (PREFETCH_V) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) v[i] = vpre[j][i];
      } else if (j >= j_lo && j < j_hi) {
        load_v<VPL>(vr + (size_t)j * HD, v);
      } else {
#pragma unroll
        for (int i = 0; i < VPL; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float pj = __shfl_sync(0xffffffffu, p[h], j);
#pragma unroll
        for (int i = 0; i < VPL; ++i) o[h][i] = fmaf(pj, v[i], o[h][i]);
      }
    }
  }

  // merge the 4 warps
#pragma unroll
  for (int h = 0; h < G; ++h) {
    if (lane == 0) {
      sm_m[warp][h] = m[h];
      sm_l[warp][h] = l[h];
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) sm_o[warp][h][lane * VPL + i] = o[h][i];
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += DEC_WARPS * 32) {
    const int h = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm_m[w][h]);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
      const float e = sm_m[w][h] == -INFINITY ? 0.f : expf(sm_m[w][h] - M);
      Lsum = fmaf(e, sm_l[w][h], Lsum);
      O = fmaf(e, sm_o[w][h][d], O);
    }
    const int head = kvh * G + h;
    if (num_splits == 1) {
      out[(size_t)b * H * HD + (size_t)head * HD + d] = __float2bfloat16_rn(Lsum > 0.f ? O / Lsum : 0.f);
    } else {
      const size_t row = ((size_t)split * n_seqs + b) * H + head;
      part_o[row * HD + d] = O;
      if (d == 0) {
        part_ml[row * 2] = M;
        part_ml[row * 2 + 1] = Lsum;
      }
    }
  }
}

template <int VPL, int G>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
           const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int Hkv,
           int page_size, int window, float scale, int num_splits, int split_keys, cudaStream_t stream) {
  dim3 grid(n_seqs, Hkv, num_splits);
  return zk_launch_dependent(attn_decode_kernel<VPL, G>, grid, dim3(DEC_WARPS * 32), 0, stream,
      (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out, part_o, part_ml, seq_start, seq_slot,
      page_table, pt_stride, n_seqs, Hkv, page_size, window, scale, num_splits, split_keys);
  return ZK_LAUNCH_STATUS();
}

template <int VPL>
int dispatch_g(int G, const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
               const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int Hkv,
               int page_size, int window, float scale, int num_splits, int split_keys, cudaStream_t stream) {
#define ZK_DEC_CASE(GG)                                                                                              \
  case GG:                                                                                                           \
    return launch<VPL, GG>(q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride,    \
                           n_seqs, Hkv, page_size, window, scale, num_splits, split_keys, stream);
  switch (G) {
    ZK_DEC_CASE(1) ZK_DEC_CASE(2) ZK_DEC_CASE(3) ZK_DEC_CASE(4) ZK_DEC_CASE(5) ZK_DEC_CASE(6) ZK_DEC_CASE(7) ZK_DEC_CASE(8)
  }
#undef ZK_DEC_CASE
  return ZK_EINVAL;
}

}  // namespace

extern "C" {

// Whether the single-token kernel takes these sizes; other sizes go to the general kernel.
int zk_attn_decode_takes(int H, int Hkv, int hd, int page_size) {
  if (Hkv <= 0 || H % Hkv) return 0;
  const int G = H / Hkv;
  return (hd == 32 || hd == 64 || hd == 96 || hd == 128) && G >= 1 && G <= 8 && page_size % DEC_TK == 0;
}

// q, out [n_seqs, H*hd] bfloat16; partials as for zk_attn_fwd when num_splits > 1.
int zk_attn_decode(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                   const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H,
                   int Hkv, int hd, int page_size, int window, float scale, int num_splits, int split_keys,
                   cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (!zk_attn_decode_takes(H, Hkv, hd, page_size) || num_splits < 1) return ZK_EINVAL;
  if (num_splits > 1 && (split_keys <= 0 || split_keys % DEC_TK || !part_o || !part_ml)) return ZK_EINVAL;
  const int G = H / Hkv;
#define ZK_DEC_HD(V)                                                                                                  \
  case V:                                                                                                             \
    return dispatch_g<V>(G, q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride,    \
                         n_seqs, Hkv, page_size, window, scale, num_splits, split_keys, stream);
  switch (hd / 32) { ZK_DEC_HD(1) ZK_DEC_HD(2) ZK_DEC_HD(3) ZK_DEC_HD(4) }
#undef ZK_DEC_HD
  return ZK_EINVAL;
}

}  // extern "C"
