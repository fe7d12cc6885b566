// Causal grouped-query attention of prompt steps over the paged bfloat16 cache on the
// fifth-generation tensor cores: head size 64, full (unwindowed) attention.
//
// A block owns 128 query rows of one (sequence, KV head): rows are (token, head-in-group) pairs,
// GP heads of the group packed beside each other (the reference orders the queries of a KV head the
// same way, src/model.zig:1352-1366), and walks the keys in tiles of 64 that lie inside one cache
// page.  Roles:
//   * warp 8 (one lane) is the producer: one 3-D TMA load brings the 128 x 64 query tile, then per
//     key tile two 2-D TMA loads bring K and V ([64 keys, 64] each, 128-byte swizzle) into a ring of
//     four stages, so that the loads run three tiles ahead of the MMAs;
//   * warp 9 (one lane) issues tcgen05.mma: S = Q K^T (M 128, N 64 keys, four k steps; K is the
//     K-major B operand) into one of two score buffers in tensor memory, and O += P V (N 64 columns,
//     four k steps over the 64 keys; V as it lies in the cache is the MN-major B operand);
//   * warps 0..7 are the softmax, two threads per row: threads r and r + 128 own row r of the tile
//     (a warp reaches the 32 accumulator lanes 32 (w mod 4) .., so warps w and w + 4 share rows),
//     the first the scores of keys 0..31 of the tile and columns 0..31 of O, the second the other
//     halves.  Each reads its 32 scores with tcgen05.ld, applies the causal mask, the two exchange
//     their maxima through shared memory (a named barrier per pair of warps), keep the running
//     maximum and their halves of the sum of the online softmax (src/attention.zig:478-517, no tile
//     skipped), rescale their halves of the row of O in tensor memory and write their halves of the
//     row of P as bfloat16 into the shared-memory tile that is the A operand of P V.  A row's chain
//     of dependent operations per key tile is half as long as with one thread, which is what bounds
//     a block (its tiles form one chain softmax -> P V -> Q K^T -> softmax).
// The scores have two buffers in tensor memory: Q K^T of tile t + 1 is issued before the MMA warp waits
// for P of tile t, so it runs while the softmax warps work on tile t, and P V of tile t runs while they
// work on tile t + 1.  One block needs 256 columns of tensor memory (two score buffers and O) and 99 KB
// of shared memory, so two blocks share an SM.  Measured on a B200 for 32 heads on 8 KV heads: a
// prompt of 8,192 tokens 832 -> 577 us a layer (476 TFLOP/s), of 2,048 tokens 90 -> 72 us, against the
// version with one thread per row, one score buffer and two K/V stages.  (Computing a part of the
// exponentials by polynomial on the FMA pipe, beside ex2.approx, made it slower: the softmax warps are
// bound by instruction issue, not by the special-function unit.)  Scores stay unscaled in registers; the
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
constexpr int SM_THREADS = 256;   // eight softmax warps: two threads per row
constexpr int THREADS = SM_THREADS + 64;   // then the producer warp and the MMA warp
constexpr int Q_BYTES = ROWS * HD * 2, KV_BYTES = TK * HD * 2, P_BYTES = ROWS * TK * 2;
constexpr int XCH_BYTES = 2 * 2 * ROWS * 4;   // the halves' maxima, double-buffered (the sums reuse it at the end)
constexpr int NSTG = 4;           // K/V tiles in shared memory: the loads run three tiles ahead of the MMAs
constexpr size_t SMEM_BYTES = Q_BYTES + 2 * NSTG * KV_BYTES + P_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + XCH_BYTES;
constexpr unsigned TMEM_COLS = 256;   // two score buffers at columns 0 and 64, O at column 128: two blocks fit an SM

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

__global__ void __launch_bounds__(THREADS, 2)
    attn_prefill_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* q_sm = base;
  unsigned char* kv_sm = base + Q_BYTES;          // stage s: K at kv_sm + 2 s KV_BYTES, V behind it
  auto k_sm = [&](int s) { return kv_sm + 2 * s * KV_BYTES; };
  auto v_sm = [&](int s) { return kv_sm + (2 * s + 1) * KV_BYTES; };
  unsigned char* p_sm = base + Q_BYTES + 2 * NSTG * KV_BYTES;
  unsigned long long* bars = reinterpret_cast<unsigned long long*>(p_sm + P_BYTES);
  unsigned long long* q_full = bars;            // 1
  unsigned long long* kv_full = bars + 1;               // [NSTG]
  unsigned long long* kv_empty = bars + 1 + NSTG;       // [NSTG]
  unsigned long long* s_full = bars + 1 + 2 * NSTG;     // [2]: one per score buffer
  unsigned long long* p_ready = bars + 3 + 2 * NSTG;    // 1, an arrival per softmax thread
  unsigned long long* pv_done = bars + 4 + 2 * NSTG;    // 1
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 5 + 2 * NSTG);
  static_assert((5 + 2 * NSTG) * 8 + 16 <= 256, "the barriers fit their 256 bytes");
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile float* xch = reinterpret_cast<volatile float*>(p_sm + P_BYTES + 256);   // [2 buffers][2 halves][ROWS]

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
    for (int s = 0; s < NSTG; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(&s_full[0], 1);
    mbar_init(&s_full[1], 1);
    mbar_init(p_ready, SM_THREADS);
    mbar_init(pv_done, 1);
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_async_smem();
  }
  if (warp == 9) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;
  const unsigned tmem_o = tmem_base + 128;
  // Barriers and tensor memory are set up while the kernel before this one ends; q and the cache
  // are its results.  (The batch's index arrays read above were uploaded before the step began.)
  zk_let_next_start();
  zk_wait_prior();

  if (warp == 8 && lane == 0) {
    // ---------------------------------------------------------------- producer
    const int* pt = p.page_table + (size_t)p.seq_slot[b] * p.pt_stride;
    mbar_expect_tx(q_full, Q_BYTES);
    tma_load_3d(q_sm, &map_q, 0, kvh * G + chunk * GP, t_base + q0, q_full);
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % NSTG;
      if (!mbar_wait(&kv_empty[s], ((t / NSTG) & 1) ^ 1)) {
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
      tma_load_2d(k_sm(s), &map_k, 0, row, &kv_full[s]);
      tma_load_2d(v_sm(s), &map_v, 0, row, &kv_full[s]);
    }
  } else if (warp == 9 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const unsigned idesc_s = instr_desc(ROWS, TK);                    // Q [128 x 64] . K^T: both K-major
    const unsigned idesc_o = instr_desc(ROWS, HD) | (1u << 16);       // P [128 x 64 keys] . V: V is MN-major
    bool ok = mbar_wait(q_full, 0);
    if (!ok) atomicExch(p.status, 15);
    auto issue_s = [&](int t) {
      const int s = t % NSTG, sb = t & 1;   // the K/V stage; the score buffer
      if (!mbar_wait(&kv_full[s], (t / NSTG) & 1)) {
        atomicExch(p.status, 15);
        return false;
      }
      tc_fence_after();
      const unsigned long long dq = smem_desc(q_sm), dk = smem_desc(k_sm(s));
#pragma unroll
      for (int k = 0; k < HD / 16; ++k)   // 32 bytes further along the swizzled rows per k step
        umma_bf16(tmem_base + 64u * (unsigned)sb, dq + (unsigned long long)(2 * k), dk + (unsigned long long)(2 * k),
                  idesc_s, k > 0 ? 1u : 0u);
      umma_commit(&s_full[sb]);
      return true;
    };
    if (ok && n_tiles > 0) ok = issue_s(0);
    for (int t = 0; t < n_tiles && ok && !*aborted; ++t) {
      // The scores of the next tile are computed while the softmax warps work on this one: they go to the
      // other score buffer, whose last scores (tile t - 1) were read before P of that tile was announced.
      if (t + 1 < n_tiles) {
        ok = issue_s(t + 1);
        if (!ok) break;
      }
      if (!mbar_wait(p_ready, t & 1)) {               // the scores are read, P of tile t is in shared memory, O is rescaled
        atomicExch(p.status, 16);
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned long long dp = smem_desc(p_sm), dv = smem_desc(v_sm(t % NSTG));
#pragma unroll
      for (int k = 0; k < TK / 16; ++k)   // P: 32 bytes along its rows; V: 16 key rows of 128 bytes further
        umma_bf16(tmem_o, dp + (unsigned long long)(2 * k), dv + (unsigned long long)(128 * k), idesc_o,
                  (t > 0 || k > 0) ? 1u : 0u);
      umma_commit(&kv_empty[t % NSTG]);
      umma_commit(pv_done);
    }
    if (!ok) *aborted = 1;
  } else if (warp < 8) {
    // ---------------------------------------------------------------- softmax and epilogue
    constexpr int HK = TK / 2, HO = HD / 2;         // a thread's keys of a tile, its columns of O
    const int half = warp >> 2;                     // 0: keys 0..31 of a tile, columns 0..31 of O; 1: the others
    const int r = threadIdx.x & (ROWS - 1);         // row of the tile = accumulator lane
    const int tq = r / GP, hl = r % GP;
    const bool row_ok = q0 + tq < Tq;
    const int row_hi = start + q0 + tq + 1;          // this row sees keys [0, row_hi)
    const unsigned lane_sel = (unsigned)((warp & 3) * 32) << 16;
    const int pair_bar = 1 + (warp & 3);             // named barrier of the two warps that share these rows
    // scores are kept raw; the scale goes into the exponent: p = 2^((s - m) * scale * log2(e))
    const float c2 = p.scale * 1.4426950408889634f;
    const int all_visible = start + q0 + 1;          // keys below this are visible to every row of the tile
    float m_run = -INFINITY, l_run = 0.f;            // l_run: the sum over this thread's keys only
    bool ok = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int s = t & 1, kb = t * TK + half * HK;
      // (a warp decides as one: the tensor-memory loads and stores below are warp-collective)
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[s], (t >> 1) & 1));
      if (!ok) {
        atomicExch(p.status, 17);
        *aborted = 1;
        break;
      }
      tc_fence_after();
      float sc[HK];
#pragma unroll
      for (int c0 = 0; c0 < HK; c0 += 16) tmem_ld16(tmem_base + 64u * (unsigned)s + lane_sel + (unsigned)(half * HK + c0), sc + c0);
      if (kb + HK > all_visible || !row_ok) {          // a tile on the diagonal (or a row that does not exist): mask
#pragma unroll
        for (int j = 0; j < HK; ++j) sc[j] = (row_ok && kb + j < row_hi) ? sc[j] : -INFINITY;
      }
      float m_mine = -INFINITY;
#pragma unroll
      for (int j = 0; j < HK; ++j) m_mine = fmaxf(m_mine, sc[j]);
      // the row's maximum over both halves
      // (the two warps of a row leave this loop only where a bounded wait on a barrier they both wait for
      // ran out, so neither can be left alone at the named barrier below)
      volatile float* xm = xch + (t & 1) * 2 * ROWS;   // the buffers alternate: a value is read before it is replaced
      xm[half * ROWS + r] = m_mine;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float m_other = xm[(half ^ 1) * ROWS + r];
      const float m_new = fmaxf(m_run, fmaxf(m_mine, m_other));
      const float mc = m_new == -INFINITY ? 0.f : m_new * c2;
      const float alpha = ex2((m_run == -INFINITY ? -INFINITY : m_run * c2) - mc);
      float row_sum = 0.f;
      unsigned pk[HK / 2];
#pragma unroll
      for (int j = 0; j < HK; j += 2) {
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
          for (int c0 = 0; c0 < HO; c0 += 16) {
            float o[16];
            tmem_ld16(tmem_o + lane_sel + (unsigned)(half * HO + c0), o);
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] *= alpha;
            tmem_st16(tmem_o + lane_sel + (unsigned)(half * HO + c0), o);
          }
        }
      }
      // this thread's half of the row of P: 4 chunks of 8 keys, chunk c at the swizzled place (c ^ (r & 7))
#pragma unroll
      for (int c = 0; c < HK / 8; ++c)
        *reinterpret_cast<uint4*>(p_sm + r * 128 + (((half * (HK / 8) + c) ^ (r & 7)) * 16)) =
            make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      // rows of V beyond the last key of the sequence's step hold stale cache contents
      if (t * TK + TK > k_end) {
        const int first = k_end - t * TK;   // 1 .. 63
        for (int i = threadIdx.x; i < (TK - first) * 8; i += SM_THREADS)
          *reinterpret_cast<uint4*>(v_sm(t % NSTG) + (first + i / 8) * 128 + (i % 8) * 16) = make_uint4(0, 0, 0, 0);
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
    if (ok) {   // uniform in the warp: every lane reads its half of its row of O, the rows that exist store it
      // the row's sum is the two halves' sums (both ran with the same maxima)
      volatile float* xs = xch + (n_tiles & 1) * 2 * ROWS;
      xs[half * ROWS + r] = l_run;
      asm volatile("bar.sync %0, 64;" ::"r"(pair_bar) : "memory");
      const float l_other = xs[(half ^ 1) * ROWS + r];
      const float l_row = half == 0 ? l_run + l_other : l_other + l_run;   // first half + second half, in both threads
      const float inv = l_row > 0.f ? 1.0f / l_row : 0.f;
      bf16* dst = p.out + (size_t)(t_base + min(q0 + tq, Tq - 1)) * p.H * HD + (size_t)(kvh * G + chunk * GP + hl) * HD +
                  half * HO;
#pragma unroll
      for (int c0 = 0; c0 < HO; c0 += 16) {
        float o[16];
        tmem_ld16(tmem_o + lane_sel + (unsigned)(half * HO + c0), o);
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
  if (warp == 9) tmem_dealloc(tmem_base, TMEM_COLS);
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
