// Causal grouped-query attention of prompt steps over the paged bfloat16 cache on the
// fifth-generation tensor cores: head size 64, full (unwindowed) attention.
//
// A block owns 128 query rows of one (sequence, KV head): rows are (token, head-in-group) pairs,
// GP heads of the group packed beside each other (the reference orders the queries of a KV head the
// same way, src/model.zig:1352-1366), and walks the keys in tiles of 64 that lie inside one cache
// page.  Roles:
//   * warp 4 (one lane) is the producer: one 3-D TMA load brings the 128 x 64 query tile, then per
//     key tile two 2-D TMA loads bring K and V ([64 keys, 64] each, 128-byte swizzle) into a ring of
//     two stages;
//   * warp 5 (one lane) issues tcgen05.mma: S = Q K^T (M 128, N 64 keys, four k steps; K is the
//     K-major B operand) into one of two score buffers in tensor memory, and O += P V (N 64 columns,
//     four k steps over the 64 keys; V as it lies in the cache is the MN-major B operand);
//   * warps 0..3 are the softmax: thread r owns row r of the tile, reads its 64 scores with
//     tcgen05.ld, applies scale and the causal mask, keeps the running maximum and sum of the online
//     softmax (src/attention.zig:478-517, no tile skipped), rescales its row of O in tensor memory,
//     and writes its row of P as bfloat16 into the shared-memory tile that is the A operand of P V.
// One block needs 128 columns of tensor memory and 65 KB of shared memory, so three blocks share an
// SM and their softmax phases overlap one another's MMAs.  Scores stay unscaled in registers; the
// scale is folded into the exponent (2^((s - m) * scale * log2 e), ex2.approx), tiles below the
// diagonal skip the mask, and a warp whose rows keep their maximum skips the rescaling of O.
//
// Rows of V beyond the last visible key are set to zero in shared memory before P V (their
// probabilities are zero, but zero times a stale NaN would not be); scores of masked keys are
// replaced, never used.  Every wait on an mbarrier is bounded: after about two seconds the block
// records a code in *status, stops issuing work, frees its tensor memory and returns.
#include "tcgen05.cuh"
#include <math.h>
#include <stdint.h>

namespace {

using namespace tc5;

constexpr int HD = 64;            // head size
constexpr int ROWS = 128;         // query rows per block = accumulator lanes
constexpr int TK = 64;            // keys per tile
constexpr int THREADS = 192;      // four softmax warps, producer warp, MMA warp
constexpr int Q_BYTES = ROWS * HD * 2, KV_BYTES = TK * HD * 2, P_BYTES = ROWS * TK * 2;
constexpr size_t SMEM_BYTES = Q_BYTES + 4 * KV_BYTES + P_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr unsigned TMEM_COLS = 128;   // S at column 0, O at column 64: three blocks fit an SM (by shared memory)

struct Params {
  bf16* out;
  const int* tile_seq;
  const int* tile_q0;
  const int* cu_q;
  const int* seq_start;
  const int* seq_slot;
  const int* page_table;
  int* status;
  int pt_stride, H, Hkv, page_size, gp;   // gp: heads of a KV group packed into one block
  float scale;
};

// 2^x on the special-function unit (relative error about 2^-22; 2^-inf = 0).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const unsigned*>(&t);
}

__global__ void __launch_bounds__(THREADS, 3)
    attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_sm = base;
  unsigned char* k_sm[2] = {base + Q_BYTES, base + Q_BYTES + 2 * KV_BYTES};
  unsigned char* v_sm[2] = {base + Q_BYTES + KV_BYTES, base + Q_BYTES + 3 * KV_BYTES};
  unsigned char* p_sm = base + Q_BYTES + 4 * KV_BYTES;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(p_sm + P_BYTES);
  unsigned long long* q_full = bars;            // 1
  unsigned long long* kv_full = bars + 1;       // [2]
  unsigned long long* kv_empty = bars + 3;      // [2]
  unsigned long long* s_full = bars + 5;        // 1 (bars + 6 unused)
  unsigned long long* p_ready = bars + 7;       // 1, 128 arrivals
  unsigned long long* pv_done = bars + 8;       // 1
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 9);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int GP = p.gp, G = p.H / p.Hkv, chunks = G / GP;
  const int BQ = ROWS / GP;                   // tokens per block
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  // tiles are taken from the last (a sequence's late tokens see the most keys) to the first
  const int tile = gridDim.x - 1 - blockIdx.x;
  const int b = p.tile_seq[tile], q0 = p.tile_q0[tile];
  const int t_base = p.cu_q[b], Tq = p.cu_q[b + 1] - t_base;
  const int start = p.seq_start[b];
  const int last_tq = min(q0 + BQ, Tq) - 1;
  const int k_end = start + last_tq + 1;      // keys [0, k_end)
  const int n_tiles = (k_end + TK - 1) / TK;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(pv_done, 1);
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 5) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_o = tmem_base + 64;
  // Barriers and tensor memory are set up while the kernel before this one ends; q and the cache
  // are its results.  (The batch's index arrays read above were uploaded before the step began.)
  zk_let_next_start();
  zk_wait_prior();

  if (warp == 4 && lane == 0) {
    // ---------------------------------------------------------------- producer
    const int* pt = p.page_table + (size_t)p.seq_slot[b] * p.pt_stride;
    mbar_expect_tx(q_full, Q_BYTES);
    tma_load_3d(q_sm, &map_q, 0, kvh * G + chunk * GP, t_base + q0, q_full);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t & 1;
      if (!mbar_wait(&kv_empty[s], ((t >> 1) & 1) ^ 1)) {
        atomicExch(p.status, 14);
        *aborted = 1;
        break;
      }
      if (*aborted) break;
      const int kb = t * TK;
      const int page = pt[kb / p.page_size];
      if (page < 0) {               // a visible position without a page: the step's inputs are wrong
        atomicExch(p.status, 2);
        *aborted = 1;
        break;
      }
      const int row = (page * p.Hkv + kvh) * p.page_size + kb % p.page_size;
      mbar_expect_tx(&kv_full[s], 2 * KV_BYTES);
      tma_load_2d(k_sm[s], &map_k, 0, row, &kv_full[s]);
      tma_load_2d(v_sm[s], &map_v, 0, row, &kv_full[s]);
    }
  } else if (warp == 5 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const unsigned idesc_s = instr_desc(ROWS, TK);                    // Q [128 x 64] . K^T: both K-major
    const unsigned idesc_o = instr_desc(ROWS, HD) | (1u << 16);       // P [128 x 64 keys] . V: V is MN-major
    bool ok = mbar_wait(q_full, 0);
    if (!ok) atomicExch(p.status, 15);
    auto issue_s = [&](int t) {
      const int s = t & 1;
      if (!mbar_wait(&kv_full[s], (t >> 1) & 1)) {
        atomicExch(p.status, 15);
        return false;
      }
      tc_fence_after();
      const unsigned long long dq = smem_desc(q_sm), dk = smem_desc(k_sm[s]);
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)   // 32 bytes further along the swizzled rows per k step
        umma_bf16(tmem_base, dq + (unsigned long long)(2 * k), dk + (unsigned long long)(2 * k), idesc_s,
                  k > 0 ? 1u : 0u);
      umma_commit(s_full);
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_s(0);
    for (int t = 0; t < n_tiles && ok && !*aborted; ++t) {
      if (!mbar_wait(p_ready, t & 1)) {               // the scores are read, P of tile t is in shared memory, O is rescaled
        atomicExch(p.status, 16);
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned long long dp = smem_desc(p_sm), dv = smem_desc(v_sm[t & 1]);
#pragma unroll
      for (int k = 0; k < TK / 16; ++k)   // P: 32 bytes along its rows; V: 16 key rows of 128 bytes further
        umma_bf16(tmem_o, dp + (unsigned long long)(2 * k), dv + (unsigned long long)(128 * k), idesc_o,
                  (t > 0 || k > 0) ? 1u : 0u);
      umma_commit(&kv_empty[t & 1]);
      umma_commit(pv_done);
      if (t + 1 < n_tiles) ok = issue_s(t + 1);
    }
    if (!ok) *aborted = 1;
  } else if (warp < 4) {
    // ---------------------------------------------------------------- softmax and epilogue
    const int r = threadIdx.x;                       // row of the tile = accumulator lane
    const int tq = r / GP, hl = r % GP;
    const bool row_ok = q0 + tq < Tq;
    const int row_hi = start + q0 + tq + 1;          // this row sees keys [0, row_hi)
    const unsigned lane_sel = (unsigned)(warp * 32) << 16;
    // scores are kept raw; the scale goes into the exponent: p = 2^((s - m) * scale * log2(e))
    const float c2 = p.scale * 1.4426950408889634f;
    const int all_visible = start + q0 + 1;          // keys below this are visible to every row of the tile
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t & 1, kb = t * TK;
      // (a warp decides as one: the tensor-memory loads and stores below are warp-collective)
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, t & 1));
      if (!ok || *aborted) {
        if (!ok) atomicExch(p.status, 17);
        *aborted = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      float sc[TK];
#pragma unroll
      for (int c0 = 0; c0 < TK; c0 += 16) tmem_ld16(tmem_base + lane_sel + (unsigned)c0, sc + c0);
      if (kb + TK > all_visible || !row_ok) {          // a tile on the diagonal (or a row that does not exist): mask
#pragma unroll
        for (int j = 0; j < TK; ++j) sc[j] = (row_ok && kb + j < row_hi) ? sc[j] : -INFINITY;
      }
      float m_new = m_run;
#pragma unroll
      for (int j = 0; j < TK; ++j) m_new = fmaxf(m_new, sc[j]);
      const float mc = m_new == -INFINITY ? 0.f : m_new * c2;
      const float alpha = ex2((m_run == -INFINITY ? -INFINITY : m_run * c2) - mc);
      float row_sum = 0.f;
      unsigned pk[TK / 2];
#pragma unroll
      for (int j = 0; j < TK; j += 2) {
        const float p0 = ex2(fmaf(sc[j], c2, -mc)), p1 = ex2(fmaf(sc[j + 1], c2, -mc));
        row_sum += p0 + p1;
        pk[j / 2] = pack_bf16(p0, p1);
      }
      l_run = l_run * alpha + row_sum;
      const bool rescale = m_new != m_run;
      m_run = m_new;
      if (t > 0) {
        // P V of the previous tile has finished: its P tile may be overwritten and O may be rescaled
        ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (t - 1) & 1));
        if (!ok) {
          atomicExch(p.status, 18);
          *aborted = 1;
          break;
        }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {        // no row of the warp has a new maximum: O stays
#pragma unroll
          for (int c0 = 0; c0 < HD; c0 += 16) {
            float o[16];
            tmem_ld16(tmem_o + lane_sel + (unsigned)c0, o);
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] *= alpha;
            tmem_st16(tmem_o + lane_sel + (unsigned)c0, o);
          }
        }
      }
      // this row of P: 8 chunks of 8 keys, chunk c at the swizzled place (c ^ (r & 7))
#pragma unroll
      for (int c = 0; c < TK / 8; ++c)
        *reinterpret_cast<uint4*>(p_sm + r * 128 + ((c ^ (r & 7)) * 16)) =
            make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      // rows of V beyond the last key of the sequence's step hold stale cache contents
      if (kb + TK > k_end) {
        const int first = k_end - kb;   // 1 .. 63
        for (int i = threadIdx.x; i < (TK - first) * 8; i += 128)
          *reinterpret_cast<uint4*>(v_sm[s] + (first + i / 8) * 128 + (i % 8) * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (n_tiles - 1) & 1));
    if (!ok) {
      atomicExch(p.status, 18);
      *aborted = 1;
    }
    tc_fence_after();
    if (ok) {   // uniform in the warp: every lane reads its row of O, the rows that exist store it
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      bf16* dst = p.out + (size_t)(t_base + min(q0 + tq, Tq - 1)) * p.H * HD + (size_t)(kvh * G + chunk * GP + hl) * HD;
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 16) {
        float o[16];
        tmem_ld16(tmem_o + lane_sel + (unsigned)c0, o);
        uint4 w0, w1;
        w0.x = pack_bf16(o[0] * inv, o[1] * inv);   w0.y = pack_bf16(o[2] * inv, o[3] * inv);
        w0.z = pack_bf16(o[4] * inv, o[5] * inv);   w0.w = pack_bf16(o[6] * inv, o[7] * inv);
        w1.x = pack_bf16(o[8] * inv, o[9] * inv);   w1.y = pack_bf16(o[10] * inv, o[11] * inv);
        w1.z = pack_bf16(o[12] * inv, o[13] * inv); w1.w = pack_bf16(o[14] * inv, o[15] * inv);
        if (row_ok) {
          *reinterpret_cast<uint4*>(dst + c0) = w0;
          *reinterpret_cast<uint4*>(dst + c0 + 8) = w1;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int packed_heads(int G) {
  for (int gp = 8; gp >= 1; gp >>= 1)
    if (G % gp == 0) return gp;
  return 1;
}

}  // namespace

extern "C" {

// Whether the kernel takes these sizes, and how many tokens one of its query tiles holds (the host
// builds the tile table with that many tokens per tile).
int zk_attn_prefill_tc5_takes(int H, int Hkv, int hd, int page_size, int window) {
  if (Hkv <= 0 || H % Hkv) return 0;
  return hd == HD && page_size % TK == 0 && window <= 0;
}
int zk_attn_prefill_tc5_tile_tokens(int H, int Hkv) { return ROWS / packed_heads(H / Hkv); }

// q, out [n_tokens, H*64] bfloat16; k_cache, v_cache [num_pages, Hkv, page_size, 64] bfloat16;
// tiles of zk_attn_prefill_tc5_tile_tokens tokens.
int zk_attn_prefill_tc5(const void* q, const void* k_cache, const void* v_cache, void* out, const int* tile_seq,
                        const int* tile_q0, const int* cu_q, const int* seq_start, const int* seq_slot,
                        const int* page_table, int pt_stride, int n_tiles, int n_tokens, long long num_pages, int H,
                        int Hkv, int hd, int page_size, float scale, int* status, cudaStream_t stream) {
  if (n_tiles <= 0 || n_tokens <= 0) return 0;
  if (!zk_attn_prefill_tc5_takes(H, Hkv, hd, page_size, 0) || !status || num_pages <= 0) return ZK_EINVAL;
  if (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) % 16) return ZK_EINVAL;
  EncodeTiledFn fn = encode_fn();
  if (!fn) return ZK_EINVAL;
  const int G = H / Hkv, gp = packed_heads(G);
  CUtensorMap mq, mk, mv;
  {
    const cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)n_tokens};
    const cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)H * HD * 2};
    const cuuint32_t box[3] = {(cuuint32_t)HD, (cuuint32_t)gp, (cuuint32_t)(ROWS / gp)};
    const cuuint32_t estr[3] = {1, 1, 1};
    if (fn(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ZK_EINVAL;
  }
  for (int which = 0; which < 2; ++which) {
    const cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)num_pages * Hkv * page_size};
    const cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
    const cuuint32_t box[2] = {(cuuint32_t)HD, (cuuint32_t)TK};
    const cuuint32_t estr[2] = {1, 1};
    if (fn(which ? &mv : &mk, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(which ? v_cache : k_cache), dims,
           strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
           CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return ZK_EINVAL;
  }
  Params p{};
  p.out = (bf16*)out; p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.cu_q = cu_q; p.seq_start = seq_start;
  p.seq_slot = seq_slot; p.page_table = page_table; p.status = status;
  p.pt_stride = pt_stride; p.H = H; p.Hkv = Hkv; p.page_size = page_size; p.gp = gp; p.scale = scale;
  cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(n_tiles, Hkv * (G / gp));
  return zk_launch_dependent(attn_prefill_tc5_kernel, grid, dim3(THREADS), SMEM_BYTES, stream, mq, mk, mv, p);
}

}  // extern "C"
