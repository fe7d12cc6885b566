// Causal grouped-query attention of prompt steps over the paged bfloat16 cache, on the tensor
// cores (mma.sync.m16n8k16, float32 accumulation and softmax).
//
// A block owns 64 query rows of one (sequence, KV head): rows are (token, head-in-group) pairs,
// GP heads of the group packed beside each other so that one K/V tile serves all of them (the
// reference orders the queries of a KV head the same way, src/model.zig:1352-1366).  Four warps
// take 16 rows each.  Keys are walked in tiles of 64 that lie inside one cache page; tiles are
// brought in with cp.async into XOR-swizzled shared memory, double-buffered; S = Q K^T and
// O += P V run from ldmatrix fragments; the running maximum, sum and output follow the online
// softmax of src/attention.zig:478-517 (no tile is skipped).  Rows of a tile beyond the last
// visible key are zero-filled on load, so stale cache contents never reach the arithmetic.
#include "common.cuh"
#include <math.h>

#define PF_ROWS 64
#define PF_TK 64
#define PF_WARPS 4

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
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&t);
}

// Byte offset of 16-byte chunk `ch` of row `r` in a tile whose rows are HD bfloat16 long.
template <int HD>
__device__ __forceinline__ int swz(int r, int ch) {
  return r * (HD * 2) + ((ch & ~7) | ((ch ^ r) & 7)) * 16;
}

// HD: head_dim, 64 or 128 (rows of a tile are whole 128-byte lines, which the swizzle assumes).  GP: heads of a KV group packed into one block.
template <int HD, int GP>
__global__ void __launch_bounds__(PF_WARPS * 32)
    attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        bf16* __restrict__ out, const int* __restrict__ tile_seq, const int* __restrict__ tile_q0,
                        const int* __restrict__ cu_q, const int* __restrict__ seq_start,
                        const int* __restrict__ seq_slot, const int* __restrict__ page_table, int pt_stride, int H,
                        int Hkv, int page_size, int window, float scale) {
  constexpr int BQ = PF_ROWS / GP;          // tokens per block
  constexpr int KS = HD / 16;               // k steps of Q K^T
  constexpr int CH = HD / 8;                // 16-byte chunks per row
  constexpr int TILE_BYTES = PF_TK * HD * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* Ksm[2] = {smem, smem + 2 * TILE_BYTES};
  unsigned char* Vsm[2] = {smem + TILE_BYTES, smem + 3 * TILE_BYTES};

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int G = H / Hkv, chunks = G / GP;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  // tiles are taken from the last (a sequence's late tokens see the most keys) to the first, so
  // that the long blocks start first and the short ones fill the tail
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int b = tile_seq[tile], q0 = tile_q0[tile];
  const int t_base = cu_q[b], Tq = cu_q[b + 1] - t_base;
  const int start = seq_start[b];
  const int* pt = page_table + (size_t)seq_slot[b] * pt_stride;

  // this thread's two rows: r0 = warp*16 + g and r0 + 8
  int row_tok[2], row_head[2], row_hi[2], row_lo[2];
  bool row_ok[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + g + 8 * h;
    const int tq = r / GP, hl = r % GP;
    row_ok[h] = q0 + tq < Tq;
    row_tok[h] = t_base + min(q0 + tq, Tq - 1);
    row_head[h] = kvh * G + chunk * GP + hl;
    row_hi[h] = start + q0 + tq + 1;
    row_lo[h] = (window > 0 && row_hi[h] > window) ? row_hi[h] - window : 0;
  }

  // Q fragments straight from global memory: a0a1 = Q[row g][2c, 2c+1], a2a3 = row g+8, a4a5 / a6a7 = +8 in k
  unsigned qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const bf16* src = q + (size_t)row_tok[h] * H * HD + (size_t)row_head[h] * HD + ks * 16 + 2 * c;
      qf[ks][h] = *reinterpret_cast<const unsigned*>(src);
      qf[ks][h + 2] = *reinterpret_cast<const unsigned*>(src + 8);
    }

  const int last_tq = min(q0 + BQ, Tq) - 1;
  const int k_end = start + last_tq + 1;  // keys [k_begin, k_end)
  int k_begin = 0;
  if (window > 0) {
    const int first_hi = start + q0 + 1;
    k_begin = first_hi > window ? first_hi - window : 0;
  }
  k_begin = (k_begin / PF_TK) * PF_TK;
  const int n_tiles = (k_end - k_begin + PF_TK - 1) / PF_TK;

  auto load_tile = [&](int t, int buf) {
    const int kb = k_begin + t * PF_TK;
    const int page = pt[kb / page_size];
    const size_t base = (((size_t)(page < 0 ? 0 : page) * Hkv + kvh) * page_size + kb % page_size) * HD;
    for (int i = tid; i < PF_TK * CH; i += PF_WARPS * 32) {
      const int r = i / CH, ch = i % CH;
      const bool valid = page >= 0 && kb + r < k_end;
      const size_t off = base + (size_t)(valid ? r : 0) * HD + ch * 8;
      cp_async16(Ksm[buf] + swz<HD>(r, ch), k_cache + off, valid);
      cp_async16(Vsm[buf] + swz<HD>(r, ch), v_cache + off, valid);
    }
    cp_async_commit();
  };

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

  if (n_tiles > 0) load_tile(0, 0);
  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      load_tile(t + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int kb = k_begin + t * PF_TK;

    // S = Q K^T: 8 key groups of 8, KS k steps
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) s[j][i] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int ks = 0; ks < KS; ks += 2) {
        // four 8x8 matrices: keys 8j..8j+7, chunks 2ks .. 2ks+3 (k steps ks and ks+1)
        unsigned bfr[4];
        const int r = 8 * j + (lane & 7), ch = 2 * ks + (lane >> 3);
        ldmatrix_x4(bfr, Ksm[buf] + swz<HD>(r, ch < CH ? ch : 0));
        mma16816(s[j], qf[ks], bfr[0], bfr[1]);
        if (ks + 1 < KS) mma16816(s[j], qf[ks + 1], bfr[2], bfr[3]);
      }
    }

    // scale, mask, online softmax; each row's 64 scores sit in the 4 lanes of a quad
    float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int h = i >> 1;
        const int kp = kb + 8 * j + 2 * c + (i & 1);
        const bool vis = row_ok[h] && kp >= row_lo[h] && kp < row_hi[h];
        s[j][i] = vis ? s[j][i] * scale : -INFINITY;
        m_new[h] = fmaxf(m_new[h], s[j][i]);
      }
    float alpha[2], row_sum[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 1));
      m_new[h] = fmaxf(m_new[h], __shfl_xor_sync(0xffffffffu, m_new[h], 2));
      alpha[h] = m_new[h] == -INFINITY ? 1.f : expf(m_run[h] - m_new[h]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int h = i >> 1;
        const float p = s[j][i] == -INFINITY ? 0.f : expf(s[j][i] - m_new[h]);
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
#pragma unroll
    for (int j = 0; j < HD / 8; ++j) {
      o[j][0] *= alpha[0];
      o[j][1] *= alpha[0];
      o[j][2] *= alpha[1];
      o[j][3] *= alpha[1];
    }

    // O += P V: 4 key steps of 16, HD/8 column groups (two per ldmatrix)
#pragma unroll
    for (int kk = 0; kk < PF_TK / 16; ++kk) {
      unsigned pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int jn = 0; jn < HD / 8; jn += 2) {
        unsigned bfr[4];
        const int r = 16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8, ch = jn + (lane >> 4);
        ldmatrix_x4_trans(bfr, Vsm[buf] + swz<HD>(r, ch));
        mma16816(o[jn], pa, bfr[0], bfr[1]);
        mma16816(o[jn + 1], pa, bfr[2], bfr[3]);
      }
    }
    __syncthreads();  // the tile is consumed before the next load overwrites its buffer
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (!row_ok[h]) continue;
    const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
    bf16* dst = out + (size_t)row_tok[h] * H * HD + (size_t)row_head[h] * HD;
#pragma unroll
    for (int j = 0; j < HD / 8; ++j)
      *reinterpret_cast<unsigned*>(dst + 8 * j + 2 * c) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
  }
}

template <int HD, int GP>
int launch(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq, const int* tile_q0,
           const int* cu_q, const int* seq_start, const int* seq_slot, const int* page_table, int pt_stride, int n_tiles,
           int H, int Hkv, int page_size, int window, float scale, cudaStream_t stream) {
  auto kern = attn_prefill_kernel<HD, GP>;
  const size_t smem = 4 * (size_t)PF_TK * HD * 2;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(n_tiles, Hkv * ((H / Hkv) / GP));
  kern<<<grid, PF_WARPS * 32, smem, stream>>>((const bf16*)q, (const bf16*)k_cache, (const bf16*)v_cache, (bf16*)out,
                                              tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table, pt_stride, H,
                                              Hkv, page_size, window, scale);
  return ZK_LAUNCH_STATUS();
}

int packed_heads(int G) {
  for (int gp = 8; gp >= 1; gp >>= 1)
    if (G % gp == 0) return gp;
  return 1;
}

}  // namespace

extern "C" {

// Whether the kernel takes these sizes, and how many tokens one of its query tiles holds
// (the host builds the tile table with that many tokens per tile).
int zk_attn_prefill_takes(int H, int Hkv, int hd, int page_size) {
  if (Hkv <= 0 || H % Hkv) return 0;
  return (hd == 64 || hd == 128) && page_size % PF_TK == 0;
}
int zk_attn_prefill_tile_tokens(int H, int Hkv) { return PF_ROWS / packed_heads(H / Hkv); }

// q, out [n_tokens, H*hd] bfloat16; tiles of zk_attn_prefill_tile_tokens tokens.
int zk_attn_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                    const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                    const int* page_table, int pt_stride, int n_tiles, int H, int Hkv, int hd, int page_size,
                    int window, float scale, cudaStream_t stream) {
  if (n_tiles <= 0) return 0;
  if (!zk_attn_prefill_takes(H, Hkv, hd, page_size)) return ZK_EINVAL;
  const int gp = packed_heads(H / Hkv);
#define ZK_PF(HDV, GPV)                                                                                          \
  if (hd == HDV && gp == GPV)                                                                                    \
    return launch<HDV, GPV>(q, k_cache, v_cache, out, tile_seq, tile_q0, cu_q, seq_start, seq_slot, page_table,  \
                            pt_stride, n_tiles, H, Hkv, page_size, window, scale, stream);
  ZK_PF(64, 1) ZK_PF(64, 2) ZK_PF(64, 4) ZK_PF(64, 8)
  ZK_PF(128, 1) ZK_PF(128, 2) ZK_PF(128, 4) ZK_PF(128, 8)
#undef ZK_PF
  return ZK_EINVAL;
}

}  // extern "C"
