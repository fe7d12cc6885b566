// Attention over the paged cache: (1) per-head q/k RMSNorm + rotary encoding + cache write,
// (2) causal grouped-query attention of a packed batch against the pages, with an optional
// window and an optional split of the keys into chunks, (3) the merge of the chunks.
//
// Softmax, norms and rotation angles are float32; the cache holds the run dtype.
// Cache layout of one layer: K and V are each [num_pages, kv_heads, page_size, head_dim];
// position p of a sequence lives in page page_table[slot][p / page_size] at row p % page_size.
//
// Reference: per-head norms and RoPE before the cache write, src/model.zig:1736-1773;
// NeoX pairing, src/rope.zig:50-64; angle = float(pos) * f_i, src/rope.zig:34-45; queries of one
// KV head ordered (token, head in group), src/model.zig:1352-1366; online softmax
// m, l, o with result o / l, src/attention.zig:478-517, 737-745; merge of split chunks,
// src/attention.zig:749-814.  No tile is skipped here (the reference drops tiles whose
// maximum is 13 below the running maximum, src/attention.zig:493).
#include "common.cuh"
#include <math.h>

#define ATT_MAX_HD 256
#define ATT_ROWS 16      // query rows (token, head-in-group) per block
#define ATT_TK 32        // keys per tile: one lane per key
#define ATT_WARPS 4

// ---------------------------------------------------------------------------------------
// (1) q/k norm + rope + cache write.  One warp per (token, head slot); head slots are the H
// query heads, then the Hkv key heads, then the Hkv value heads, as they lie in a qkv row.
// With `dense_out` the results of all three kinds go to a dense [n, (H + 2 Hkv) * hd] tensor
// instead (no cache write): the first half of a two-step path for position encodings that
// are not a rotation table.
template <typename T>
__global__ void qk_prepare_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ dense_out,
                                  T* __restrict__ k_cache,
                                  T* __restrict__ v_cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                                  const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
                                  const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                                  const int* __restrict__ page_table, int pt_stride, int n_tokens, int H, int Hkv,
                                  int hd, int n_rot, int interleaved, float eps, int page_size, int write_kv,
                                  int* status) {
  __shared__ float sm_all[ATT_WARPS][ATT_MAX_HD];
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slots = H + 2 * Hkv;
  const long long item = (long long)blockIdx.x * ATT_WARPS + warp;
  if (item >= (long long)n_tokens * slots) return;
  const int t = (int)(item / slots), s = (int)(item % slots);
  const int kind = s < H ? 0 : (s < H + Hkv ? 1 : 2);  // 0 q, 1 k, 2 v
  if (kind != 0 && !write_kv && !dense_out) return;
  float* sm = sm_all[warp];
  const T* src = qkv + (size_t)t * slots * hd + (size_t)s * hd;
  const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);

  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) {
    const float v = to_f32(src[d]);
    sm[d] = v;
    ss = fmaf(v, v, ss);
  }
  if (w) {
    ss = warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)hd + eps);
    for (int d = lane; d < hd; d += 32) sm[d] = (sm[d] * scale) * w[d];
  }
  __syncwarp();
  const int pos = tok_pos[t];
  if (kind != 2 && inv_freq) {
    const int half = n_rot >> 1;
    for (int i = lane; i < half; i += 32) {
      const int ia = interleaved ? 2 * i : i;
      const int ib = interleaved ? 2 * i + 1 : i + half;
      const float ang = (float)pos * inv_freq[i];
      const float c = cosf(ang), sn = sinf(ang);
      const float a = sm[ia], b = sm[ib];
      sm[ia] = a * c - b * sn;
      sm[ib] = a * sn + b * c;
    }
    __syncwarp();
  }
  T* dst;
  if (dense_out) {
    dst = dense_out + (size_t)t * slots * hd + (size_t)s * hd;
  } else if (kind == 0) {
    dst = q_out + (size_t)t * H * hd + (size_t)s * hd;
  } else {
    const int slot = seq_slot[tok_seq[t]];
    const int page = page_table[(size_t)slot * pt_stride + pos / page_size];
    if (page < 0) {
      if (lane == 0) atomicExch(status, 2);
      return;
    }
    const int kh = kind == 1 ? s - H : s - H - Hkv;
    T* base = kind == 1 ? k_cache : v_cache;
    dst = base + (((size_t)page * Hkv + kh) * page_size + pos % page_size) * hd;
  }
  for (int d = lane; d < hd; d += 32) dst[d] = from_f32<T>(sm[d]);
}

// The same for prompt steps with head sizes 64 and 128 and a rotation over the whole head in
// half-split pairing (or none): one block per token, its warps take the head slots in turn, the
// angles' cosines and sines are computed once per warp instead of once per head, and a lane keeps
// its pairs (d, d + hd/2) in registers.  The arithmetic and its order are those of
// qk_prepare_kernel, so both give the same bits.
template <typename T, int HD>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    qk_prepare_token_kernel(const T* __restrict__ qkv, T* __restrict__ q_out, T* __restrict__ k_cache,
                            T* __restrict__ v_cache, const float* __restrict__ q_w, const float* __restrict__ k_w,
                            const float* __restrict__ inv_freq, const int* __restrict__ tok_seq,
                            const int* __restrict__ tok_pos, const int* __restrict__ seq_slot,
                            const int* __restrict__ page_table, int pt_stride, int H, int Hkv, float eps, int page_size,
                            int write_kv, int* status) {
  constexpr int E = HD / 64, HALF = HD / 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int slots = H + 2 * Hkv;
  zk_let_next_start();
  zk_wait_prior();   // qkv is the kernel before's result
  const int pos = tok_pos[t];
  float cs[E], sn[E];
#pragma unroll
  for (int e = 0; e < E; ++e) {
    const float ang = inv_freq ? (float)pos * inv_freq[lane + 32 * e] : 0.f;
    cs[e] = cosf(ang);
    sn[e] = sinf(ang);
  }
  int page = -2;   // not looked up yet
  const int n_slots = write_kv ? slots : H;
  // A warp's head slots four at a time: their loads are all under way before the first is used.
  // One after the other, a warp waited for memory once per slot, and the kernel's time was that
  // chain (18 us for 2,048 tokens of 48 slots, whose 25 MB would take 5).
  constexpr int UN = 4;
  for (int s0 = warp; s0 < n_slots; s0 += ATT_WARPS * UN) {
    float av[UN][E], bv[UN][E];
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int s = s0 + u * ATT_WARPS;
      const T* src = qkv + (size_t)t * slots * HD + (size_t)min(s, n_slots - 1) * HD;
#pragma unroll
      for (int e = 0; e < E; ++e) {
        av[u][e] = to_f32(src[lane + 32 * e]);
        bv[u][e] = to_f32(src[lane + 32 * e + HALF]);
      }
    }
#pragma unroll
    for (int u = 0; u < UN; ++u) {
      const int s = s0 + u * ATT_WARPS;
      if (s >= n_slots) break;
      const int kind = s < H ? 0 : (s < H + Hkv ? 1 : 2);
      const float* w = kind == 0 ? q_w : (kind == 1 ? k_w : nullptr);
      float a[E], b[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        a[e] = av[u][e];
        b[e] = bv[u][e];
      }
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(a[e], a[e], ss);
#pragma unroll
        for (int e = 0; e < E; ++e) ss = fmaf(b[e], b[e], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          a[e] = (a[e] * scale) * w[lane + 32 * e];
          b[e] = (b[e] * scale) * w[lane + 32 * e + HALF];
        }
      }
      if (kind != 2 && inv_freq) {
#pragma unroll
        for (int e = 0; e < E; ++e) {
          const float x = a[e], y = b[e];
          a[e] = x * cs[e] - y * sn[e];
          b[e] = x * sn[e] + y * cs[e];
        }
      }
      T* dst;
      if (kind == 0) {
        dst = q_out + (size_t)t * H * HD + (size_t)s * HD;
      } else {
        if (page == -2) page = page_table[(size_t)seq_slot[tok_seq[t]] * pt_stride + pos / page_size];
        if (page < 0) {
          if (lane == 0) atomicExch(status, 2);
          continue;
        }
        const int kh = kind == 1 ? s - H : s - H - Hkv;
        dst = (kind == 1 ? k_cache : v_cache) + (((size_t)page * Hkv + kh) * page_size + pos % page_size) * HD;
      }
#pragma unroll
      for (int e = 0; e < E; ++e) {
        dst[lane + 32 * e] = from_f32<T>(a[e]);
        dst[lane + 32 * e + HALF] = from_f32<T>(b[e]);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// (2) attention.  Block = (query tile, kv head x head chunk, key split).  A query tile is
// `bq` consecutive tokens of one sequence; its rows are (token, head in group) pairs, at
// most ATT_ROWS of them; row r belongs to warp r % 4.  Keys are walked in tiles of 32 that
// start at multiples of 32, one lane per key.
template <typename T, int NPL>
__global__ void __launch_bounds__(ATT_WARPS * 32)
    attn_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                    T* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                    const int* __restrict__ tile_seq, const int* __restrict__ tile_q0, const int* __restrict__ cu_q,
                    const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                    const int* __restrict__ page_table, int pt_stride, int n_tokens, int H, int Hkv, int hd,
                    int page_size, int window, float scale, int bq, int gc, int num_splits, int split_keys) {
  extern __shared__ float smem[];
  float* qs = smem;                               // [ATT_ROWS][hd]
  float* Ks = qs + ATT_ROWS * hd;                 // [ATT_TK][hd + 1]
  float* Vs = Ks + ATT_TK * (hd + 1);             // [ATT_TK][hd]
  long long* rowoff = reinterpret_cast<long long*>(Vs + ATT_TK * hd);  // [ATT_TK]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = H / Hkv;
  const int chunks = (g + gc - 1) / gc;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int b = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
  const int split = blockIdx.z;
  const int t_base = cu_q[b], Tq = cu_q[b + 1] - t_base;
  const int start = seq_start[b];
  const int slot = seq_slot[b];
  const int* pt = page_table + (size_t)slot * pt_stride;

  // rows of this warp: r = warp + 4*i
  int row_t[4], row_h[4], row_lo[4], row_hi[4];
  bool row_ok[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp + ATT_WARPS * i;
    const int tq = r / gc, hl = r % gc;
    row_ok[i] = (tq < bq) && (q0 + tq < Tq) && (chunk * gc + hl < g);
    row_t[i] = t_base + q0 + tq;
    row_h[i] = kvh * g + chunk * gc + hl;
    row_hi[i] = start + q0 + tq + 1;
    row_lo[i] = (window > 0 && row_hi[i] > window) ? row_hi[i] - window : 0;
  }

  // stage the query rows as float32
  for (int idx = tid; idx < ATT_ROWS * hd; idx += ATT_WARPS * 32) {
    const int r = idx / hd, d = idx - r * hd;
    const int tq = r / gc, hl = r % gc;
    const bool ok = (tq < bq) && (q0 + tq < Tq) && (chunk * gc + hl < g);
    qs[idx] = ok ? to_f32(q[(size_t)(t_base + q0 + tq) * H * hd + (size_t)(kvh * g + chunk * gc + hl) * hd + d]) : 0.f;
  }

  // key range of the block
  const int last_tq = min(q0 + bq, Tq) - 1;
  int k_end = start + last_tq + 1;
  int k_begin = 0;
  if (window > 0) {
    const int first_hi = start + q0 + 1;
    k_begin = first_hi > window ? first_hi - window : 0;
  }
  if (num_splits > 1) {
    k_begin = max(k_begin, split * split_keys);
    k_end = min(k_end, (split + 1) * split_keys);
  }
  k_begin = (k_begin / ATT_TK) * ATT_TK;

  float m[4], l[4], o[4][NPL];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int c = 0; c < NPL; ++c) o[i][c] = 0.f;
  }
  const int split_lo = num_splits > 1 ? split * split_keys : 0;

  for (int kb = k_begin; kb < k_end; kb += ATT_TK) {
    __syncthreads();  // previous tile fully consumed (and qs staged, first time)
    if (tid < ATT_TK) {
      const int kp = kb + tid;
      long long off = -1;
      if (kp < k_end) {
        const int page = pt[kp / page_size];
        if (page >= 0) off = (((long long)page * Hkv + kvh) * page_size + kp % page_size) * hd;
      }
      rowoff[tid] = off;
    }
    __syncthreads();
    for (int idx = tid; idx < ATT_TK * hd; idx += ATT_WARPS * 32) {
      const int j = idx / hd, d = idx - j * hd;
      const long long off = rowoff[j];
      float kv = 0.f, vv = 0.f;
      if (off >= 0) {
        kv = to_f32(k_cache[off + d]);
        vv = to_f32(v_cache[off + d]);
      }
      Ks[j * (hd + 1) + d] = kv;
      Vs[j * hd + d] = vv;
    }
    __syncthreads();

    float s[4] = {0.f, 0.f, 0.f, 0.f};
    const float* kr = Ks + lane * (hd + 1);
    for (int d = 0; d < hd; ++d) {
      const float kd = kr[d];
#pragma unroll
      for (int i = 0; i < 4; ++i) s[i] = fmaf(qs[(warp + ATT_WARPS * i) * hd + d], kd, s[i]);
    }
    const int kp = kb + lane;
    const bool key_ok = kp < k_end && kp >= split_lo && rowoff[lane] >= 0;
    float p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const bool ok = row_ok[i] && key_ok && kp >= row_lo[i] && kp < row_hi[i];
      const float sc = ok ? s[i] * scale : -INFINITY;
      const float mt = warp_max(sc);
      if (mt == -INFINITY) {  // no key of this tile is visible to this row
        p[i] = 0.f;
        continue;
      }
      const float m_new = fmaxf(m[i], mt);
      const float alpha = expf(m[i] - m_new);
      p[i] = ok ? expf(sc - m_new) : 0.f;
      l[i] = l[i] * alpha + warp_sum(p[i]);
      m[i] = m_new;
#pragma unroll
      for (int c = 0; c < NPL; ++c) o[i][c] *= alpha;
    }
    for (int j = 0; j < ATT_TK; ++j) {
      float vj[NPL];
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        vj[c] = d < hd ? Vs[j * hd + d] : 0.f;
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pj = __shfl_sync(0xffffffffu, p[i], j);
#pragma unroll
        for (int c = 0; c < NPL; ++c) o[i][c] = fmaf(pj, vj[c], o[i][c]);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (!row_ok[i]) continue;
    if (num_splits == 1) {
      const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
      T* dst = out + (size_t)row_t[i] * H * hd + (size_t)row_h[i] * hd;
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) dst[d] = from_f32<T>(o[i][c] * inv);
      }
    } else {
      const size_t row = ((size_t)split * n_tokens + row_t[i]) * H + row_h[i];
      float* dst = part_o + row * hd;
#pragma unroll
      for (int c = 0; c < NPL; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) dst[d] = o[i][c];
      }
      if (lane == 0) {
        part_ml[row * 2] = m[i];
        part_ml[row * 2 + 1] = l[i];
      }
    }
  }
}

// (3) merge: out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s.  One warp per (token, head).
// A lane holds the (m, l) of one chunk (32 chunks at a time), so that the loads of all chunks are
// under way together; the sums run over the chunks in ascending order whatever the timing.
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                  T* __restrict__ out, int n_rows, int hd, int num_splits) {
  zk_let_next_start();
  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float M = -INFINITY;
  for (int s0 = 0; s0 < num_splits; s0 += 32) {
    const int s = s0 + lane;
    const float ms = s < num_splits ? part_ml[((size_t)s * n_rows + row) * 2] : -INFINITY;
    M = fmaxf(M, warp_max(ms));
  }
  float L = 0.f;
  float acc[8];   // head sizes up to 256: 8 values per lane
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int s0 = 0; s0 < num_splits; s0 += 32) {
    const int s = s0 + lane;
    float ms = -INFINITY, ls = 0.f;
    if (s < num_splits) {
      const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)s * n_rows + row) * 2);
      ms = ml.x;
      ls = ml.y;
    }
    const float e = ms == -INFINITY ? 0.f : expf(ms - M);
    const int n_here = min(32, num_splits - s0);
    for (int j = 0; j < n_here; ++j) L = fmaf(__shfl_sync(0xffffffffu, e, j), __shfl_sync(0xffffffffu, ls, j), L);
    for (int j0 = 0; j0 < n_here; j0 += 8) {
      float v[8][8], w[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = j0 + u;
        w[u] = j < n_here ? __shfl_sync(0xffffffffu, e, j & 31) : 0.f;
        const float* po = part_o + ((size_t)(s0 + j) * n_rows + row) * hd;
#pragma unroll
        for (int i = 0; i < 8; ++i) v[u][i] = (w[u] != 0.f && lane + 32 * i < hd) ? po[lane + 32 * i] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w[u], v[u][i], acc[i]);
    }
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i)
    if (lane + 32 * i < hd) out[(size_t)row * hd + lane + 32 * i] = from_f32<T>(acc[i] * inv);
}

namespace {

size_t attn_smem_bytes(int hd) {
  return sizeof(float) * ((size_t)ATT_ROWS * hd + (size_t)ATT_TK * (hd + 1) + (size_t)ATT_TK * hd) + sizeof(long long) * ATT_TK + 16;
}

template <typename T, int NPL>
int launch_attn(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv, int hd, int page_size,
                int window, float scale, int bq, int gc, int num_splits, int split_keys, cudaStream_t stream) {
  const size_t smem = attn_smem_bytes(hd);
  auto kern = attn_fwd_kernel<T, NPL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int g = H / Hkv;
  const int chunks = (g + gc - 1) / gc;
  dim3 grid(n_tiles, Hkv * chunks, num_splits);
  kern<<<grid, ATT_WARPS * 32, smem, stream>>>((const T*)q, (const T*)k_cache, (const T*)v_cache, (T*)out, part_o,
                                               part_ml, tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table,
                                               pt_stride, n_tokens, H, Hkv, hd, page_size, window, scale, bq, gc,
                                               num_splits, split_keys);
  return ZK_LAUNCH_STATUS();
}

template <typename T>
int dispatch_attn(int hd, const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o,
                  float* part_ml, const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start,
                  const int* seq_slot, const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv,
                  int page_size, int window, float scale, int bq, int gc, int num_splits, int split_keys,
                  cudaStream_t stream) {
#define ZK_ATT_CASE(N)                                                                                               \
  case N:                                                                                                            \
    return launch_attn<T, N>(q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start, seq_slot, \
                             page_table, pt_stride, n_tiles, n_tokens, H, Hkv, hd, page_size, window, scale, bq, gc,  \
                             num_splits, split_keys, stream);
  switch ((hd + 31) / 32) {
    ZK_ATT_CASE(1) ZK_ATT_CASE(2) ZK_ATT_CASE(3) ZK_ATT_CASE(4) ZK_ATT_CASE(5) ZK_ATT_CASE(6) ZK_ATT_CASE(7)
    ZK_ATT_CASE(8)
  }
#undef ZK_ATT_CASE
  return ZK_EINVAL;
}

}  // namespace

extern "C" {

// Rows per block and the split of a KV group's heads, for the host to build its tile table:
// gc heads of a group per block, bq = ATT_ROWS / gc tokens per tile.
int zk_attn_rows_per_block() { return ATT_ROWS; }
int zk_attn_max_head_dim() { return ATT_MAX_HD; }

int zk_qk_prepare(const void* qkv, void* q_out, void* dense_out, void* k_cache, void* v_cache, const float* q_w, const float* k_w,
                  const float* inv_freq, const int* tok_seq, const int* tok_pos, const int* seq_slot,
                  const int* page_table, int pt_stride, int n_tokens, int H, int Hkv, int hd, int n_rot,
                  int interleaved, float eps, int page_size, int write_kv, int dtype, int* status,
                  cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (hd <= 0 || hd > ATT_MAX_HD || H <= 0 || Hkv <= 0 || n_rot > hd || (n_rot & 1) || page_size <= 0) return ZK_EINVAL;
  // many tokens, whole-head half-split rotation (or none): one block per token
  if (n_tokens >= 256 && !dense_out && (hd == 64 || hd == 128) && (!inv_freq || (n_rot == hd && !interleaved)) &&
      (dtype == ZK_F32 || dtype == ZK_BF16)) {
#define ZK_QKP(T, HDV)                                                                                               \
  zk_launch_dependent(qk_prepare_token_kernel<T, HDV>, dim3(n_tokens), dim3(ATT_WARPS * 32), 0, stream,             \
      (const T*)qkv, (T*)q_out, (T*)k_cache, (T*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot, page_table, \
      pt_stride, H, Hkv, eps, page_size, write_kv, status)
    if (dtype == ZK_F32 && hd == 64) ZK_QKP(float, 64);
    else if (dtype == ZK_F32) ZK_QKP(float, 128);
    else if (hd == 64) ZK_QKP(bf16, 64);
    else ZK_QKP(bf16, 128);
#undef ZK_QKP
    return ZK_LAUNCH_STATUS();
  }
  const long long items = (long long)n_tokens * (H + 2 * Hkv);
  const int blocks = (int)((items + ATT_WARPS - 1) / ATT_WARPS);
  if (dtype == ZK_F32)
    return zk_launch_dependent(qk_prepare_kernel<float>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream,
        (const float*)qkv, (float*)q_out, (float*)dense_out, (float*)k_cache, (float*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos,
        seq_slot, page_table, pt_stride, n_tokens, H, Hkv, hd, n_rot, interleaved, eps, page_size, write_kv, status);
  else if (dtype == ZK_BF16)
    return zk_launch_dependent(qk_prepare_kernel<bf16>, dim3(blocks), dim3(ATT_WARPS * 32), 0, stream,
        (const bf16*)qkv, (bf16*)q_out, (bf16*)dense_out, (bf16*)k_cache, (bf16*)v_cache, q_w, k_w, inv_freq, tok_seq, tok_pos, seq_slot,
        page_table, pt_stride, n_tokens, H, Hkv, hd, n_rot, interleaved, eps, page_size, write_kv, status);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

// q, out [n_tokens, H*hd]; part_o [num_splits, n_tokens*H, hd] and part_ml [num_splits,
// n_tokens*H, 2] float32 scratch, used when num_splits > 1 (then call zk_attn_merge).
int zk_attn_fwd(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                const int* tile_seq, const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                const int* page_table, int pt_stride, int n_tiles, int n_tokens, int H, int Hkv, int hd, int page_size,
                int window, float scale, int bq, int gc, int num_splits, int split_keys, int dtype,
                cudaStream_t stream) {
  if (n_tiles <= 0 || n_tokens <= 0) return 0;
  if (hd <= 0 || hd > ATT_MAX_HD || H <= 0 || Hkv <= 0 || H % Hkv || page_size <= 0) return ZK_EINVAL;
  if (gc <= 0 || gc > ATT_ROWS || bq <= 0 || bq * gc > ATT_ROWS || num_splits < 1) return ZK_EINVAL;
  if (num_splits > 1 && (split_keys <= 0 || split_keys % ATT_TK || !part_o || !part_ml)) return ZK_EINVAL;
  if (dtype == ZK_F32)
    return dispatch_attn<float>(hd, q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start,
                                seq_slot, page_table, pt_stride, n_tiles, n_tokens, H, Hkv, page_size, window, scale,
                                bq, gc, num_splits, split_keys, stream);
  if (dtype == ZK_BF16)
    return dispatch_attn<bf16>(hd, q, k_cache, v_cache, out, part_o, part_ml, tile_seq, tile_q0, cu_q, seq_start,
                               seq_slot, page_table, pt_stride, n_tiles, n_tokens, H, Hkv, page_size, window, scale, bq,
                               gc, num_splits, split_keys, stream);
  return ZK_EINVAL;
}

int zk_attn_merge(const float* part_o, const float* part_ml, void* out, int n_rows, int hd, int num_splits, int dtype,
                  cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  const int warps = 4;
  const int blocks = (n_rows + warps - 1) / warps;
  if (dtype == ZK_F32)
    return zk_launch_dependent(attn_merge_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, (float*)out, n_rows, hd, num_splits);
  else if (dtype == ZK_BF16)
    return zk_launch_dependent(attn_merge_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, part_o, part_ml, (bf16*)out, n_rows, hd, num_splits);
  else
    return ZK_EINVAL;
  return ZK_LAUNCH_STATUS();
}

}  // extern "C"
