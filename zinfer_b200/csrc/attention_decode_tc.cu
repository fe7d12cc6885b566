// Attention of single-token steps over the paged bfloat16 cache on the tensor cores
// (mma.sync.m16n8k16, float32 accumulation and softmax).
//
// One query token per sequence; the G query heads of a KV head are the rows of one 16-row MMA
// tile (rows G..15 are zero), so one pass over the K and V of a KV head serves all of them (the
// reference orders the queries of a KV head the same way, src/model.zig:1352-1366).  A block owns
// (sequence, KV head, chunk of keys).  Its keys are walked in tiles of 64 that lie inside one cache
// page; the four warps bring a tile in together with cp.async into XOR-swizzled shared memory
// (a ring of two to four tile buffers), and then each warp takes 16 of the tile's keys: S = Q K^T from ldmatrix
// fragments, online softmax (src/attention.zig:478-517, no tile skipped), O += P V.  The warps'
// (m, l, o) are merged in shared memory and written either as the result (one chunk) or as a
// partial for `zk_attn_merge` (src/model.zig:1941-1955, src/attention.zig:749-814).
//
// Against the kernel of attention_decode.cu (one lane per key, float32 FMAs) this one issues about
// a fifth of the instructions per byte of cache, which is what bounds long contexts and large
// batches.  Rows of a tile beyond the last visible key are zero-filled on load, so stale cache
// contents never reach the arithmetic.
#include "common.cuh"
#include <math.h>

#define DT_TK 64
#define DT_WARPS 4

namespace {

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int n = valid ? 16 : 0;  // src-size 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(unsigned r[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned r[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma16816(float c[4], const unsigned a[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (x <= 0 here; -inf gives 0)
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&t);
}

// Byte offset of 16-byte chunk `ch` of row `r` in a tile whose rows are HD bfloat16 long.
template <int HD>
__device__ __forceinline__ int swz(int r, int ch) {
  return r * (HD * 2) + ((ch & ~7) | ((ch ^ r) & 7)) * 16;
}

// HD: head_dim, 64 or 128 (rows of a tile are whole 128-byte lines, which the swizzle assumes).
template <int HD, int NST>
__global__ void __launch_bounds__(DT_WARPS * 32)
    attn_decode_tc_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                          bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                          const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                          const int* __restrict__ page_table, int pt_stride, int n_seqs, int H, int Hkv, int page_size,
                          int window, float scale, int num_splits, int split_keys) {
  constexpr int KS = HD / 16;               // k steps of Q K^T
  constexpr int CH = HD / 8;                // 16-byte chunks per row
  constexpr int TILE_BYTES = DT_TK * HD * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  auto Ksm = [&](int buf) { return smem + (size_t)(2 * buf) * TILE_BYTES; };
  auto Vsm = [&](int buf) { return smem + (size_t)(2 * buf + 1) * TILE_BYTES; };

  zk_wait_prior();   // nothing of the kernels before is read, and nothing written, above this line
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int G = H / Hkv;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int L = seq_start[b] + 1;  // keys 0 .. L-1; the new token's own key is the last
  const int lo = (window > 0 && L > window) ? L - window : 0;
  int c0 = lo, c1 = L;             // this block's keys [c0, c1)
  if (num_splits > 1) {
    c0 = max(lo, split * split_keys);
    c1 = min(L, (split + 1) * split_keys);
  }
  const int* pt = page_table + (size_t)seq_slot[b] * pt_stride;

  // Q fragments straight from global memory: row g = head g of the group, row g + 8 = head g + 8
  unsigned qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int hl = g + 8 * h;
      const bf16* src = q + (size_t)b * H * HD + (size_t)(kvh * G + min(hl, G - 1)) * HD + ks * 16 + 2 * c;
      qf[ks][h] = hl < G ? *reinterpret_cast<const unsigned*>(src) : 0u;
      qf[ks][h + 2] = hl < G ? *reinterpret_cast<const unsigned*>(src + 8) : 0u;
    }

  const int k_begin = (c0 / DT_TK) * DT_TK;
  const int n_tiles = c1 > c0 ? (c1 - k_begin + DT_TK - 1) / DT_TK : 0;

  // A thread's 16-byte pieces of a tile: piece n is row r0 + n * ROWS_STEP, chunk ch0.  The swizzle
  // depends on the row only through its low three bits, which ROWS_STEP (a multiple of 8) leaves
  // alone, so piece n lies a fixed distance behind piece 0 both in the cache and in shared memory.
  constexpr int PIECES = DT_TK * CH / (DT_WARPS * 32), ROWS_STEP = DT_WARPS * 32 / CH;
  static_assert(ROWS_STEP % 8 == 0 && PIECES * ROWS_STEP == DT_TK, "pieces of a tile");
  const int r0 = tid / CH, ch0 = tid % CH;
  const int sm_off0 = swz<HD>(r0, ch0), g_off0 = r0 * HD + ch0 * 8;

  // Tiles are loaded in order, so where the next one lies (entry of the page table, place in the page)
  // is carried along: no division per tile.
  int ld_kb = k_begin, ld_entry = k_begin / page_size, ld_in_page = k_begin % page_size;
  auto load_tile = [&](int buf) {
    const int kb = ld_kb;
    const int page = pt[ld_entry];
    const size_t base = (((size_t)(page < 0 ? 0 : page) * Hkv + kvh) * page_size + ld_in_page) * HD;
    ld_kb += DT_TK;
    ld_in_page += DT_TK;
    if (ld_in_page == page_size) {
      ld_in_page = 0;
      ++ld_entry;
    }
    if (page >= 0 && kb + DT_TK <= c1) {     // a whole tile: nothing to test per piece
      const bf16* kg = k_cache + base + g_off0;
      const bf16* vg = v_cache + base + g_off0;
      unsigned char* ks = Ksm(buf) + sm_off0;
      unsigned char* vs = Vsm(buf) + sm_off0;
#pragma unroll
      for (int n = 0; n < PIECES; ++n) {
        cp_async16(ks + n * ROWS_STEP * HD * 2, kg + n * ROWS_STEP * HD, true);
        cp_async16(vs + n * ROWS_STEP * HD * 2, vg + n * ROWS_STEP * HD, true);
      }
    } else {
      for (int i = tid; i < DT_TK * CH; i += DT_WARPS * 32) {
        const int r = i / CH, ch = i % CH;
        const bool valid = page >= 0 && kb + r < c1;
        const size_t off = base + (size_t)(valid ? r : 0) * HD + ch * 8;
        cp_async16(Ksm(buf) + swz<HD>(r, ch), k_cache + off, valid);
        cp_async16(Vsm(buf) + swz<HD>(r, ch), v_cache + off, valid);
      }
    }
    cp_async_commit();
  };

  // The softmax runs on base 2: scores are scaled by scale * log2(e) and the exponentials are ex2.approx
  // (one instruction where expf is eight); the maxima go back to base e when they leave the loop.
  const float scale2 = scale * 1.4426950408889634f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

  // NST buffers: tiles t + 1 .. t + NST - 1 are under way while tile t is worked on.  Every
  // iteration commits one group (an empty one when no tile is left), so "all but the newest
  // NST - 1 groups" is always "tile t has landed".
  for (int t = 0; t < NST - 1; ++t) {
    if (t < n_tiles) load_tile(t);
    else cp_async_commit();
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t % NST;
    if (t + NST - 1 < n_tiles) load_tile((t + NST - 1) % NST);
    else cp_async_commit();
    cp_async_wait<NST - 1>();
    __syncthreads();
    const int kb = k_begin + t * DT_TK + 16 * warp;   // this warp's 16 keys of the tile

    // S = Q K^T: 2 key groups of 8, KS k steps
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ks += 2) {
        unsigned bfr[4];
        const int r = 16 * warp + 8 * j + (lane & 7), ch = 2 * ks + (lane >> 3);
        ldmatrix_x4(bfr, Ksm(buf) + swz<HD>(r, ch));
        mma16816(s[j], qf[ks], bfr[0], bfr[1]);
        mma16816(s[j], qf[ks + 1], bfr[2], bfr[3]);
      }
    }

    // scale, mask, online softmax; a row's 16 scores of this warp sit in the 4 lanes of a quad.
    // Only a chunk's first and last tile can hold keys outside [c0, c1).
    const bool edge_tile = kb - 16 * warp < c0 || kb - 16 * warp + DT_TK > c1;   // the same for the whole block
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (edge_tile) {
          const int kp = kb + 8 * j + 2 * c + (i & 1);
          const bool vis = kp >= c0 && kp < c1;
          s[j][i] = vis ? s[j][i] * scale2 : -INFINITY;
        } else {
          s[j][i] *= scale2;
        }
        m_new[i >> 1] = fmaxf(m_new[i >> 1], s[j][i]);
      }
    float alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      alpha[h] = m_new[h] == -INFINITY ? 1.f : ex2(m_run[h] - m_new[h]);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int h = i >> 1;
        // a masked score is -inf, and so is m_new while a row has seen masked keys only: only edge tiles
        const float p = (edge_tile && s[j][i] == -INFINITY) ? 0.f : ex2(s[j][i] - m_new[h]);
        s[j][i] = p;
        row_sum[h] += p;
      }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
      l_run[h] = l_run[h] * alpha[h] + row_sum[h];
      m_run[h] = m_new[h];
    }
    // o * 1.0f is o: where no row of the warp found a new maximum the multiplications are left out
    if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
      for (int j = 0; j < HD / 8; ++j) {
        o[j][0] *= alpha[0];
        o[j][1] *= alpha[0];
        o[j][2] *= alpha[1];
        o[j][3] *= alpha[1];
      }
    }

    // O += P V: one key step of 16, HD/8 column groups (two per ldmatrix)
    unsigned pa[4];
    pa[0] = pack_bf16(s[0][0], s[0][1]);
    pa[1] = pack_bf16(s[0][2], s[0][3]);
    pa[2] = pack_bf16(s[1][0], s[1][1]);
    pa[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
    for (int jn = 0; jn < HD / 8; jn += 2) {
      unsigned bfr[4];
      const int r = 16 * warp + (lane & 7) + ((lane >> 3) & 1) * 8, ch = jn + (lane >> 4);
      ldmatrix_x4_trans(bfr, Vsm(buf) + swz<HD>(r, ch));
      mma16816(o[jn], pa, bfr[0], bfr[1]);
      mma16816(o[jn + 1], pa, bfr[2], bfr[3]);
    }
    __syncthreads();  // the tile is consumed before the next load overwrites its buffer
  }

  cp_async_wait<0>();   // only empty groups are left
  // merge the four warps' partial results in shared memory (the tile buffers are free now)
  float* sm_m = reinterpret_cast<float*>(smem);              // [warps][16]
  float* sm_l = sm_m + DT_WARPS * 16;                        // [warps][16]
  float* sm_o = sm_l + DT_WARPS * 16;                        // [warps][16][HD]
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = g + 8 * h;
    if (c == 0) {
      sm_m[warp * 16 + row] = m_run[h] * 0.6931471805599453f;
      sm_l[warp * 16 + row] = l_run[h];
    }
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      sm_o[(warp * 16 + row) * HD + 8 * j + 2 * c] = o[j][2 * h];
      sm_o[(warp * 16 + row) * HD + 8 * j + 2 * c + 1] = o[j][2 * h + 1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < G * HD; idx += DT_WARPS * 32) {
    const int h = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) M = fmaxf(M, sm_m[w * 16 + h]);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < DT_WARPS; ++w) {
      const float e = sm_m[w * 16 + h] == -INFINITY ? 0.f : expf(sm_m[w * 16 + h] - M);
      Lsum = fmaf(e, sm_l[w * 16 + h], Lsum);
      O = fmaf(e, sm_o[(w * 16 + h) * HD + d], O);
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

template <int HD, int NST>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
           const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H, int Hkv,
           int page_size, int window, float scale, int num_splits, int split_keys, cudaStream_t stream) {
  auto kern = attn_decode_tc_kernel<HD, NST>;
  const size_t smem = 2 * NST * (size_t)DT_TK * HD * 2;
  static_assert(2 * NST * DT_TK * HD * 2 >= (2 * DT_WARPS * 16 + DT_WARPS * 16 * HD) * 4, "the merge fits in the tile buffers");
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_seqs, Hkv, num_splits);
  return zk_launch_dependent(kern, grid, dim3(DT_WARPS * 32), smem, stream, (const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out,
                                              part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H, Hkv,
                                              page_size, window, scale, num_splits, split_keys);
  return ZK_LAUNCH_STATUS();
}

}  // namespace

extern "C" {

// Whether the tensor-core single-token kernel takes these sizes (head_dim 64 or 128, up to 16
// heads per KV head, pages of a multiple of 64 tokens); other sizes go to zk_attn_decode or to
// the general kernel.
int zk_attn_decode_tc_takes(int H, int Hkv, int hd, int page_size) {
  if (Hkv <= 0 || H % Hkv) return 0;
  const int G = H / Hkv;
  return (hd == 64 || hd == 128) && G >= 1 && G <= 16 && page_size % DT_TK == 0;
}

// q, out [n_seqs, H*hd] bfloat16; partials as for zk_attn_fwd when num_splits > 1.
int zk_attn_decode_tc(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_o, float* part_ml,
                      const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H,
                      int Hkv, int hd, int page_size, int window, float scale, int num_splits, int split_keys,
                      cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (!zk_attn_decode_tc_takes(H, Hkv, hd, page_size) || num_splits < 1) return ZK_EINVAL;
  if (num_splits > 1 && (split_keys <= 0 || split_keys % DT_TK || !part_o || !part_ml)) return ZK_EINVAL;
  // Tile buffers (head_dim 64): a block whose chunk is at most four tiles asks for all of them at once;
  // longer chunks are double-buffered, because more blocks on an SM hide more latency than a deeper
  // ring in fewer blocks.  Measured on whole steps, two / three / four buffers: LFM2-1.2B shape with 8
  // sequences (chunks of three tiles) 0.707 / 0.720 / 0.695 ms; with 64 sequences (chunks of some ten
  // tiles) 1.55 / 1.53 / 1.57 ms; LFM2-350M shape with 64 sequences of up to 32,768 tokens (chunks of
  // 4,096 keys) 3.41 / 3.72 / 4.16 ms.
  const bool short_chunks = num_splits > 1 && split_keys <= 4 * DT_TK;
  if (hd == 64 && short_chunks)
    return launch<64, 4>(q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H,
                         Hkv, page_size, window, scale, num_splits, split_keys, stream);
  if (hd == 64)
    return launch<64, 2>(q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H,
                         Hkv, page_size, window, scale, num_splits, split_keys, stream);
  return launch<128, 2>(q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs, H,
                     Hkv, page_size, window, scale, num_splits, split_keys, stream);
}

}  // extern "C"
