// C[M, N] (+)= X[M, K] . W[N, K]^T (+ bias) on the fifth-generation tensor cores of sm_100a.
//
// One block computes one 128 x BN tile of the product of two K-major bfloat16 operands:
//   * warp 0 (one lane) is the producer: per 64-wide k block it issues two TMA tile loads
//     (cp.async.bulk.tensor.2d, 128-byte swizzle) into a ring of shared-memory stages and arms
//     the stage's mbarrier with the byte count;
//   * warp 1 allocates the tile's accumulator in tensor memory and (one lane) issues
//     tcgen05.mma.kind::f16 -- four k=16 steps per stage -- then tcgen05.commit, which frees the
//     stage when the MMAs have read it, and finally signals the accumulator as complete;
//   * warps 2..5 are the epilogue: each reads its quarter of the accumulator's 128 lanes with
//     tcgen05.ld and stores the tile with bias / residual add / conversion.
// Two roles of the operands:
//   normal : rows of the tile are tokens (X), columns are weight rows (W): prompt steps;
//   swapped: rows of the tile are weight rows, columns are the few tokens of a single-token
//            step (16..64): every weight is read once, and K may be split over the 2, 4 or 8
//            blocks of a thread-block cluster so that more SMs stream; each block leaves its
//            partial tile in its own shared memory, and after a cluster barrier every block adds
//            the partials of its share of the tokens in split order, reading the other blocks'
//            shared memory directly (no workspace, no atomics, the same bits each run).
//            Its epilogues also take part in the RMSNorm around them: a product whose input rows
//            came as bfloat16(x * norm weight) with partial sums of x^2 scales token t's sums by
//            1 / sqrt(sum / K + eps), and a product that sums into the float32 residual rows can
//            write those two things for the norm that reads the rows next.
// Products of more than 64 rows with N a multiple of 256 take the persistent form further down
// (one block, or a pair of blocks with tcgen05.mma.cta_group::2, per SM walking 256-wide tiles, a
// TMA-store epilogue).  Every kernel here is launched as a dependent launch: the producer requests
// the weight tiles of its first stages before it waits for the kernel before this one.
// Accumulation is float32 in tensor memory.  (Reference: the matmul driver with its accumulate
// flag, src/model.zig:903-1026, 918-920.)
//
// Every wait on an mbarrier is bounded: after about two seconds the block records a code in
// *status, stops issuing work, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace {

using namespace tc5;   // mbarrier, TMA, tensor-memory and tcgen05.mma wrappers; descriptors

constexpr int BM = 128;          // tile rows = accumulator lanes
constexpr int BK = 64;           // k block: 64 bfloat16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;     // producer warp, MMA warp, four epilogue warps

struct Params {
  void* C;
  const float* bias;
  int* status;
  int M, N, K;         // M tokens, N weight rows
  int ldc, accumulate, splits;
  int swiglu;          // normal mode: W rows are groups of 16 gate rows + their 16 up rows; C [M, N/2] = silu(g)*u
  // Up to 64 tokens only.  ssq_in: X holds bfloat16(x * norm weight) of rows whose RMSNorm is still to be
  // applied, ssq_in [M, ssq_parts] partial sums of x^2: token t's sums are scaled by
  // 1 / sqrt(sum(ssq_in[t]) / K + eps).  emit_x: beside C (the float32 residual rows) the kernel writes
  // emit_x [M, N] = bfloat16(C * emit_w) and emit_ssq [M, ceil(N / 32)] = sums of C^2 over 32 columns,
  // for the norm that reads C next.
  const float* ssq_in;
  int ssq_parts;
  float eps;
  const float* emit_w;
  bf16* emit_x;
  float* emit_ssq;
};

// q[j] of every lane, j < T (T = 4, 8 or 16): the sums over the warp's 32 lanes, T - 1 + log2(32 / T)
// shuffles in place of 5 T.  Every lane returns the sum of q[token_of_lane<T>(lane)].
template <int T>
__device__ __forceinline__ int token_of_lane(int lane) {
  int j = 0;
#pragma unroll
  for (int w = T / 2, mask = 16; w >= 1; w >>= 1, mask >>= 1)
    if (lane & mask) j += w;
  return j;
}
template <int T>
__device__ __forceinline__ float warp_sums(float (&q)[T], int lane) {
  int mask = 16;
#pragma unroll
  for (int w = T / 2; w >= 1; w >>= 1, mask >>= 1) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < w; ++i) {
      const float keep = upper ? q[i + w] : q[i], send = upper ? q[i] : q[i + w];
      q[i] = keep + __shfl_xor_sync(0xffffffffu, send, mask);
    }
  }
  float v = q[0];
  for (; mask >= 1; mask >>= 1) v += __shfl_xor_sync(0xffffffffu, v, mask);
  return v;
}
// the lanes that write a warp_sums result: one per token
template <int T>
__device__ __forceinline__ bool writes_sum(int lane) { return (lane & (32 / T - 1)) == 0; }

// Thread-block cluster: barrier over all threads of all blocks, rank, and loads from another
// block's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float ld_remote_f32(unsigned local_smem_addr, unsigned rank) {
  unsigned remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

template <int BN, int STAGES>
struct Smem {
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr size_t BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 512 /*barriers, row scales*/;
};

// SWAP = false: A tiles are 128 tokens of X, B tiles are BN weight rows; C[token][weight row].
// SWAP = true : A tiles are 128 weight rows, B tile is the BN-padded token block.
template <int BN, int STAGES, bool SWAP, typename TC>
__global__ void __launch_bounds__(THREADS)
    gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  using S = Smem<BN, STAGES>;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned long long* full = reinterpret_cast<unsigned long long*>(tiles + (size_t)STAGES * S::STAGE_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_done = empty + STAGES;
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_done + 1);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* row_scale = reinterpret_cast<float*>(full) + 32;   // [64], 128 bytes behind the first barrier

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int a_tile = blockIdx.x, b_tile = blockIdx.y, split = blockIdx.z;
  constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;

  const int nkb = (p.K + BK - 1) / BK;
  const int per = (nkb + p.splits - 1) / p.splits;
  const int kb0 = split * per, kb1 = min(nkb, kb0 + per);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_done, 1);
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer
    // The operand that holds weights needs nothing of the kernel before this one: its tiles of the
    // first stages are requested, the next kernel is let in, and only then does the producer wait
    // for the kernel before and request the rows.
    const CUtensorMap* map_w = SWAP ? &map_a : &map_b;
    const CUtensorMap* map_x = SWAP ? &map_b : &map_a;
    const int w_row = SWAP ? a_tile * BM : b_tile * BN, x_row = SWAP ? b_tile * BN : a_tile * BM;
    constexpr int W_OFF = SWAP ? 0 : S::A_BYTES, X_OFF = SWAP ? S::A_BYTES : 0;
    const int pre = min(STAGES, kb1 - kb0);
    for (int it = 0; it < pre; ++it) {
      mbar_expect_tx(&full[it], S::STAGE_BYTES);
      tma_load_2d(tiles + (size_t)it * S::STAGE_BYTES + W_OFF, map_w, (kb0 + it) * BK, w_row, &full[it]);
    }
    zk_let_next_start();
    zk_wait_prior();
    for (int it = 0; it < pre; ++it)
      tma_load_2d(tiles + (size_t)it * S::STAGE_BYTES + X_OFF, map_x, (kb0 + it) * BK, x_row, &full[it]);
    for (int kb = kb0 + pre, it = pre; kb < kb1; ++kb, ++it) {
      const int s = it % STAGES;
      if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) {
        atomicExch(p.status, 11);
        *aborted = 1;
        break;
      }
      if (*aborted) break;
      unsigned char* a_dst = tiles + (size_t)s * S::STAGE_BYTES;
      mbar_expect_tx(&full[s], S::STAGE_BYTES);
      tma_load_2d(a_dst, &map_a, kb * BK, a_tile * BM, &full[s]);
      tma_load_2d(a_dst + S::A_BYTES, &map_b, kb * BK, b_tile * BN, &full[s]);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const unsigned idesc = instr_desc(BM, BN);
    bool ok = true;
    for (int kb = kb0, it = 0; kb < kb1 && ok; ++kb, ++it) {
      const int s = it % STAGES;
      if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
        atomicExch(p.status, 12);
        *aborted = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const unsigned char* a_src = tiles + (size_t)s * S::STAGE_BYTES;
      const unsigned long long da = smem_desc(a_src), db = smem_desc(a_src + S::A_BYTES);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes further along the swizzled row per step
        umma_bf16(tmem_base, da + (unsigned long long)(2 * k), db + (unsigned long long)(2 * k), idesc,
                  (it > 0 || k > 0) ? 1u : 0u);
      umma_commit(&empty[s]);
    }
    umma_commit(acc_done);  // arrives when every MMA above has finished (at once if none was issued)
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- epilogue
    const int quarter = warp & 3;            // the 32 accumulator lanes this warp may read
    const int row = quarter * 32 + lane;     // row of the tile
    zk_wait_prior();                         // C, which this warp reads and writes, is the kernels' before
    if constexpr (SWAP) {
      if (p.ssq_in) {
        // two lanes per token add its partial sums in a fixed order; every block of a cluster does so
        static_assert(STAGES <= 6, "the row scales lie 128 bytes behind the barriers");
        const int e = (warp - 2) * 32 + lane, t = e >> 1;
        float sum = 0.f;
        if (t < p.M) {
          const float* mine = p.ssq_in + (size_t)t * p.ssq_parts;
          for (int q0 = e & 1; q0 < p.ssq_parts; q0 += 32) {   // 16 loads under way at a time
            float v[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) v[u] = q0 + 2 * u < p.ssq_parts ? mine[q0 + 2 * u] : 0.f;
#pragma unroll
            for (int u = 0; u < 16; ++u) sum += v[u];
          }
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        if ((e & 1) == 0) row_scale[t] = t < p.M ? 1.0f / sqrtf(sum / (float)p.K + p.eps) : 0.f;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
      }
    }
    bool ok = mbar_wait(acc_done, 0);
    if (!ok) {
      if (lane == 0) atomicExch(p.status, 13);
      *aborted = 1;
    }
    ok = ok && !*aborted && kb1 > kb0;
    tc_fence_after();
    const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16);

    if constexpr (!SWAP) {
      // The accumulator goes through shared memory (the pipeline's stages are free by now: every
      // MMA has read them) so that global rows are read and written as whole 128-byte lines.
      constexpr int LD = BN + 1;  // odd row stride: a warp's 32 rows fall into 32 banks
      float* stage = reinterpret_cast<float*>(tiles);
      static_assert((size_t)BM * LD * 4 <= (size_t)STAGES * S::STAGE_BYTES, "tile does not fit the stages");
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (ok) {
          tmem_ld16(lane_addr + c0, v);   // warp-collective
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) stage[row * LD + c0 + j] = v[j];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
      if (ok && p.swiglu) {
        // columns of the tile: 16 gates, their 16 ups, 16 gates, ...: BN/2 outputs per row
        const int h_base = b_tile * (BN / 2), F = p.N / 2;
        for (int r = quarter * 32; r < quarter * 32 + 32; ++r) {
          const int m = a_tile * BM + r;
          if (m >= p.M) break;
          TC* hrow = reinterpret_cast<TC*>(p.C) + (size_t)m * p.ldc + h_base;
          const float* srow = stage + r * LD;
#pragma unroll
          for (int i = 0; i < BN / 64; ++i) {
            const int oc = lane + 32 * i;                    // output column inside the tile
            const int gc = (oc / 16) * 32 + (oc % 16);      // its gate's column; the up is 16 further
            if (h_base + oc < F) {
              const float gate = srow[gc], up = srow[gc + 16];
              hrow[oc] = from_f32<TC>(gate / (1.0f + expf(-gate)) * up);
            }
          }
        }
      } else if (ok) {
        const int n_base = b_tile * BN;
#pragma unroll 4
        for (int r = quarter * 32; r < quarter * 32 + 32; ++r) {
          const int m = a_tile * BM + r;
          if (m >= p.M) break;
          TC* crow = reinterpret_cast<TC*>(p.C) + (size_t)m * p.ldc + n_base;
          const float* srow = stage + r * LD;
          if constexpr (sizeof(TC) == 4) {
            float o[BN / 32];
#pragma unroll
            for (int i = 0; i < BN / 32; ++i) {
              const int col = lane + 32 * i;
              o[i] = (p.accumulate && n_base + col < p.N) ? crow[col] : 0.f;   // all loads of the row first
            }
#pragma unroll
            for (int i = 0; i < BN / 32; ++i) {
              const int col = lane + 32 * i;
              if (n_base + col < p.N) crow[col] = o[i] + srow[col] + (p.bias ? p.bias[n_base + col] : 0.f);
            }
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) {
              const int col = 2 * lane + 64 * i;
              if (n_base + col + 1 < p.N && (p.ldc & 1) == 0) {
                float o0 = srow[col] + (p.bias ? p.bias[n_base + col] : 0.f);
                float o1 = srow[col + 1] + (p.bias ? p.bias[n_base + col + 1] : 0.f);
                __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(crow + col);
                if (p.accumulate) {
                  const __nv_bfloat162 old = *dst;
                  o0 += __low2float(old);
                  o1 += __high2float(old);
                }
                *dst = __floats2bfloat162_rn(o0, o1);
              } else {
                for (int e = 0; e < 2; ++e)
                  if (n_base + col + e < p.N) {
                    float o = srow[col + e] + (p.bias ? p.bias[n_base + col + e] : 0.f);
                    if (p.accumulate) o += to_f32(crow[col + e]);
                    crow[col + e] = from_f32<TC>(o);
                  }
              }
            }
          }
        }
      }
    } else {
      // rows are weight rows n, columns are tokens; a warp's lanes are 32 consecutive n
      const int n = a_tile * BM + row;
      TC* C = reinterpret_cast<TC*>(p.C);
      float* part = reinterpret_cast<float*>(tiles);   // [BN][128] partial tile (the stages are free by now)
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        float v[16];
        if (ok) {
          tmem_ld16(lane_addr + c0, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (p.splits > 1) {
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(c0 + j) * BM + row] = v[j];
          continue;
        }
        if (p.ssq_in) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] *= row_scale[c0 + j];   // BN <= 64 tokens
        }
        if (p.swiglu) {
          // a warp's 32 rows are 16 gate rows and their 16 up rows (N is a multiple of 32, so the
          // whole warp is on one side of N): lane l < 16 takes the up value of lane l + 16
          const int f = (n >> 5) * 16 + (n & 15);   // output column of this gate row
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float up = __shfl_down_sync(0xffffffffu, v[j], 16);
            if ((lane & 16) == 0 && n < p.N && c0 + j < p.M)
              C[(size_t)(c0 + j) * p.ldc + f] = from_f32<TC>(v[j] / (1.0f + expf(-v[j])) * up);
          }
        } else {
          const bool n_in = n < p.N;
          const float b = (p.bias && n_in) ? p.bias[n] : 0.f;
          float old[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)   // all loads first: they do not depend on one another
            old[j] = (p.accumulate && n_in && c0 + j < p.M) ? to_f32(C[(size_t)(c0 + j) * p.ldc + n]) : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            v[j] = (n_in && c0 + j < p.M) ? v[j] + b + old[j] : 0.f;
            if (n_in && c0 + j < p.M) C[(size_t)(c0 + j) * p.ldc + n] = from_f32<TC>(v[j]);
          }
          if (p.emit_x) {   // float32 C: v is what was stored
            const float nw = n_in ? p.emit_w[n] : 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (n_in && c0 + j < p.M) p.emit_x[(size_t)(c0 + j) * p.N + n] = __float2bfloat16_rn(v[j] * nw);
              v[j] *= v[j];
            }
            const float sq = warp_sums<16>(v, lane);
            const int t = c0 + token_of_lane<16>(lane);
            if (writes_sum<16>(lane) && t < p.M && a_tile * BM + quarter * 32 < p.N)
              p.emit_ssq[(size_t)t * ((p.N + 31) / 32) + a_tile * (BM / 32) + quarter] = sq;
          }
        }
      }
    }
  }

  if constexpr (SWAP) {
    if (p.splits > 1) {
      // Every block of the cluster has its partial tile in shared memory; block r adds, in split
      // order, the partials of the tokens r, r + splits, ... and writes them.
      __syncwarp();
      cluster_sync_all();
      if (warp >= 2) {
        const int row = (warp & 3) * 32 + lane;
        const int n = a_tile * BM + row;
        TC* C = reinterpret_cast<TC*>(p.C);
        const unsigned base = smem_u32(tiles);
        const unsigned rank = cluster_rank();
        const bool n_in = n < p.N;
        const float b = (p.bias && n_in) ? p.bias[n] : 0.f;
        const float nw = (p.emit_x && n_in) ? p.emit_w[n] : 0.f;
        // The remote partials and old values of 32 / splits tokens (32 loads from the cluster's
        // shared memory and up to 16 from global memory) are all requested before the first sum,
        // so a thread waits for them once, not once per token: with four tokens at a time the
        // loop took longer than the contraction when K was split in two.
        auto reduce = [&](auto splits_c) {
          constexpr int SP = decltype(splits_c)::value, TOK = 32 / SP;
          for (int t0 = (int)rank; t0 < p.M; t0 += TOK * SP) {
            float pv[TOK][SP], old[TOK];
#pragma unroll
            for (int i = 0; i < TOK; ++i) {
              const int t = t0 + i * SP;
#pragma unroll
              for (int z = 0; z < SP; ++z)
                pv[i][z] = t < p.M ? ld_remote_f32(base + (unsigned)(t * BM + row) * 4u, (unsigned)z) : 0.f;
              old[i] = (t < p.M && n_in && p.accumulate) ? to_f32(C[(size_t)t * p.ldc + n]) : 0.f;
            }
            float sq[TOK];
#pragma unroll
            for (int i = 0; i < TOK; ++i) {
              const int t = t0 + i * SP;
              sq[i] = 0.f;
              if (t >= p.M) continue;        // the same for every lane
              float acc = 0.f;
#pragma unroll
              for (int z = 0; z < SP; ++z) acc += pv[i][z];
              if (p.ssq_in) acc *= row_scale[t];
              acc += b;
              if (p.swiglu) {
                // as in the unsplit epilogue: a warp's rows are 16 gate rows and their 16 up rows
                const float up = __shfl_down_sync(0xffffffffu, acc, 16);
                if ((lane & 16) == 0 && n_in)
                  C[(size_t)t * p.ldc + (n >> 5) * 16 + (n & 15)] = from_f32<TC>(acc / (1.0f + expf(-acc)) * up);
              } else if (n_in) {
                acc += old[i];
                C[(size_t)t * p.ldc + n] = from_f32<TC>(acc);
                if (p.emit_x) {
                  p.emit_x[(size_t)t * p.N + n] = __float2bfloat16_rn(acc * nw);
                  sq[i] = acc * acc;
                }
              }
            }
            if (p.emit_x) {
              const float total = warp_sums<TOK>(sq, lane);
              const int t = t0 + token_of_lane<TOK>(lane) * SP;
              if (writes_sum<TOK>(lane) && t < p.M && a_tile * BM + (warp & 3) * 32 < p.N)
                p.emit_ssq[(size_t)t * ((p.N + 31) / 32) + a_tile * (BM / 32) + (warp & 3)] = total;
            }
          }
        };
        if (p.splits == 2) reduce(std::integral_constant<int, 2>());
        else if (p.splits == 4) reduce(std::integral_constant<int, 4>());
        else reduce(std::integral_constant<int, 8>());
      }
      __syncwarp();
      cluster_sync_all();   // nobody leaves while its shared memory may still be read
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ------------------------------------------------------------------------------ persistent form
// Products of more than 64 rows with N a multiple of 256: one block per SM walks the tiles (token
// tiles fastest, so that the blocks running together share weight tiles in L2).  The stage ring
// runs on across tiles, the accumulator is double-buffered in tensor memory (2 x BN columns), and
// the epilogue warps store tile i while the MMA warp works on tile i + 1.  With PAIR two blocks of
// a cluster share 256 x BN tiles through tcgen05.mma.cta_group::2.  The epilogue goes from tensor
// memory through registers and a swizzled staging tile to a TMA store (or a TMA reduce-add for the
// float32 residual sum): a per-row loop of ordinary loads and stores in its place held these
// kernels at 0.8-0.9 PFLOP/s; without any stores they ran at 1.4.
// NV outputs of this thread's row into its 128-byte row of a staging tile with 128-byte swizzle: the
// 16-byte chunk c of row r lies at chunk c ^ (r & 7).  `chunk0` is the first chunk they fill.
template <typename TC, int NV>
__device__ __forceinline__ void stage_row(unsigned char* row, int r, int chunk0, const float* v) {
  constexpr int PER = 16 / (int)sizeof(TC);   // outputs in a chunk
#pragma unroll
  for (int i = 0; i < NV / PER; ++i) {
    uint4 q;
    if constexpr (sizeof(TC) == 4) {
      q = make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]), __float_as_uint(v[4 * i + 2]),
                     __float_as_uint(v[4 * i + 3]));
    } else {
      __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * i], v[8 * i + 1]), h1 = __floats2bfloat162_rn(v[8 * i + 2], v[8 * i + 3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * i + 4], v[8 * i + 5]), h3 = __floats2bfloat162_rn(v[8 * i + 6], v[8 * i + 7]);
      q = make_uint4(*reinterpret_cast<unsigned*>(&h0), *reinterpret_cast<unsigned*>(&h1), *reinterpret_cast<unsigned*>(&h2),
                     *reinterpret_cast<unsigned*>(&h3));
    }
    *reinterpret_cast<uint4*>(row + (((chunk0 + i) ^ (r & 7)) << 4)) = q;
  }
}

template <int BN, int STAGES, bool PAIR>
struct SmemP {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;            // weight rows this block loads per stage
  static constexpr int A_BYTES = BM * BK * 2, B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int PIECE_BYTES = 32 * 128;               // 32 rows x 128 bytes of output: one TMA store
  static constexpr int EPI_BYTES = 4 * 2 * PIECE_BYTES;      // two staging tiles for each epilogue warp
  static constexpr size_t BYTES = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
};

template <int BN, int STAGES, bool PAIR, typename TC>
__global__ void __launch_bounds__(THREADS, PAIR ? 1 : 0)
    gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              const __grid_constant__ CUtensorMap map_c, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  using S = SmemP<BN, STAGES, PAIR>;
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* stage_base = tiles + (size_t)STAGES * S::STAGE_BYTES;   // 1024-byte aligned, as the swizzle needs
  unsigned long long* full = reinterpret_cast<unsigned long long*>(stage_base + S::EPI_BYTES);
  unsigned long long* empty = full + STAGES;
  unsigned long long* acc_full = empty + STAGES;     // [2]
  unsigned long long* acc_empty = acc_full + 2;      // [2]
  unsigned* tmem_slot = reinterpret_cast<unsigned*>(acc_empty + 2);
  volatile int* aborted = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr unsigned TMEM_COLS = 2 * BN;
  static_assert(TMEM_COLS <= 512 && (TMEM_COLS & (TMEM_COLS - 1)) == 0, "tensor memory holds two accumulators");
  // A unit is a block, or a pair of blocks (ranks 0 and 1 of a cluster) that shares 256 x BN tiles:
  // each block of a pair loads its 128 token rows and its half of the BN weight rows, the block of
  // rank 0 issues the pair's MMAs, and each block stores the 128 x BN accumulator of its own rows.
  const unsigned rank = PAIR ? cluster_rank() : 0u;
  const int unit = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_units = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TM = PAIR ? 2 * BM : BM;     // token rows of a unit's tile
  const int tiles_m = (p.M + TM - 1) / TM, tiles_n = (p.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n;
  const int nkb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], PAIR ? 8 : 4);   // one arrival per epilogue warp (of both blocks of a pair)
    }
    *aborted = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    else tmem_alloc(tmem_slot, TMEM_COLS);
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();   // the other block's barriers are initialised before anything arrives on them
  else __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = *tmem_slot;

  if (warp == 0 && lane == 0) {
    // ---------------------------------------------------------------- producer
    // The weights need nothing of the kernel before this one: the weight tiles of the first tile's
    // first stages are requested, the next kernel is let in, and only then does the producer wait
    // for the kernel before and request the rows.
    const int pre = unit < n_tiles ? min(STAGES, nkb) : 0;
    const unsigned bar0 = PAIR ? cluster_addr(&full[0], 0) : 0u;   // stage s: bar0 + 8 s
    for (int s = 0; s < pre; ++s) {
      unsigned char* b_dst = tiles + (size_t)s * S::STAGE_BYTES + S::A_BYTES;
      const int b_tile = unit / tiles_m;
      if constexpr (PAIR) {
        if (rank == 0) mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);
        tma_load_2d_pair(b_dst, &map_b, s * BK, b_tile * BN + (int)rank * S::B_ROWS, bar0 + 8u * s);
      } else {
        mbar_expect_tx(&full[s], S::STAGE_BYTES);
        tma_load_2d(b_dst, &map_b, s * BK, b_tile * BN, &full[s]);
      }
    }
    zk_let_next_start();
    zk_wait_prior();
    for (int s = 0; s < pre; ++s) {
      unsigned char* a_dst = tiles + (size_t)s * S::STAGE_BYTES;
      const int a_tile = unit % tiles_m;
      if constexpr (PAIR) tma_load_2d_pair(a_dst, &map_a, s * BK, a_tile * TM + (int)rank * BM, bar0 + 8u * s);
      else tma_load_2d(a_dst, &map_a, s * BK, a_tile * BM, &full[s]);
    }
    int it = pre;
    for (int t = unit; t < n_tiles && !*aborted; t += n_units) {
      const int a_tile = t % tiles_m, b_tile = t / tiles_m;
      for (int kb = (t == unit ? pre : 0); kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1)) {
          atomicExch(p.status, 11);
          *aborted = 1;
          break;
        }
        if (*aborted) break;
        unsigned char* a_dst = tiles + (size_t)s * S::STAGE_BYTES;
        if constexpr (PAIR) {
          // both blocks' bytes are counted on the barrier of rank 0, where the MMAs are issued
          if (rank == 0) mbar_expect_tx(&full[s], 2 * S::STAGE_BYTES);
          const unsigned bar = cluster_addr(&full[s], 0);
          tma_load_2d_pair(a_dst, &map_a, kb * BK, a_tile * TM + (int)rank * BM, bar);
          tma_load_2d_pair(a_dst + S::A_BYTES, &map_b, kb * BK, b_tile * BN + (int)rank * S::B_ROWS, bar);
        } else {
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, kb * BK, a_tile * BM, &full[s]);
          tma_load_2d(a_dst + S::A_BYTES, &map_b, kb * BK, b_tile * BN, &full[s]);
        }
      }
    }
  } else if (warp == 1 && lane == 0 && rank == 0) {
    // ---------------------------------------------------------------- MMA issuer
    const unsigned idesc = instr_desc(TM, BN);
    int it = 0, local = 0;
    for (int t = unit; t < n_tiles && !*aborted; t += n_units, ++local) {
      const int buf = local & 1;
      if (!mbar_wait(&acc_empty[buf], ((local >> 1) & 1) ^ 1)) {   // the epilogue has read this accumulator
        atomicExch(p.status, 13);
        *aborted = 1;
        break;
      }
      tc_fence_after();
      const unsigned d_tmem = tmem_base + (unsigned)(buf * BN);
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb, ++it) {
        const int s = it % STAGES;
        if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
          atomicExch(p.status, 12);
          *aborted = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const unsigned char* a_src = tiles + (size_t)s * S::STAGE_BYTES;
        const unsigned long long da = smem_desc(a_src), db = smem_desc(a_src + S::A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          if constexpr (PAIR)
            umma_bf16_pair(d_tmem, da + (unsigned long long)(2 * k), db + (unsigned long long)(2 * k), idesc,
                           (kb > 0 || k > 0) ? 1u : 0u);
          else
            umma_bf16(d_tmem, da + (unsigned long long)(2 * k), db + (unsigned long long)(2 * k), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
        }
        if constexpr (PAIR) umma_commit_pair(&empty[s]);   // frees the stage in both blocks
        else umma_commit(&empty[s]);
      }
      if (!ok) break;
      if constexpr (PAIR) umma_commit_pair(&acc_full[buf]);
      else umma_commit(&acc_full[buf]);
    }
  } else if (warp >= 2) {
    // ---------------------------------------------------------------- epilogue
    // Each warp stores the 32 accumulator rows that it may read, on its own: 32 columns at a time
    // from tensor memory into registers (one thread per row), the outputs as pieces of 128 bytes
    // per row into one of its two staging tiles (128-byte swizzle, as the map of C expects), and
    // lane 0 hands the tile to the TMA: a store, or an add to what C holds (the residual sum).
    // The TMA leaves out rows past M.
    const int quarter = warp & 3;            // the 32 accumulator lanes this warp may read
    zk_wait_prior();                         // C, which this warp stores to or adds to, is the kernels' before
    unsigned char* my_stage = stage_base + quarter * (2 * S::PIECE_BYTES);
    constexpr int OUTC = 128 / (int)sizeof(TC);                   // output columns of a piece
    const int groups_per_piece = OUTC / (p.swiglu ? 16 : 32);     // 32 accumulator columns give 32 outputs, or 16
    int local = 0, sb = 0;
    for (int t = unit; t < n_tiles; t += n_units, ++local) {
      const int a_tile = t % tiles_m, b_tile = t / tiles_m;
      const int m0 = a_tile * TM + (int)rank * BM + quarter * 32;   // first token row of this warp
      const int buf = local & 1;
      const bool ok = mbar_wait(&acc_full[buf], (local >> 1) & 1);
      if (!__all_sync(0xffffffffu, ok) || *aborted) {
        if (!ok && lane == 0) atomicExch(p.status, 13);
        *aborted = 1;
        break;
      }
      tc_fence_after();
      const unsigned lane_addr = tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(buf * BN);
      const int x_tile = b_tile * (p.swiglu ? BN / 2 : BN);
#pragma unroll 1
      for (int g = 0; g < BN / 32; ++g) {
        float v[32];
        tmem_ld32(lane_addr + (unsigned)(g * 32), v);   // warp-collective
        if (g == BN / 32 - 1) {   // the whole accumulator has been read: the MMA warp may overwrite it
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (PAIR) mbar_arrive_cluster(cluster_addr(&acc_empty[buf], 0));
            else mbar_arrive(&acc_empty[buf]);
          }
        }
        const int part = g % groups_per_piece;
        if (part == 0) {   // a new piece: the store before last has read this staging tile
          if (lane == 0) bulk_wait_read<1>();
          __syncwarp();
        }
        unsigned char* row = my_stage + sb * S::PIECE_BYTES + lane * 128;
        if (p.swiglu) {    // columns: 16 gates, then their 16 ups
          float o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = v[j] / (1.0f + expf(-v[j])) * v[j + 16];
          stage_row<TC, 16>(row, lane, part * (16 * (int)sizeof(TC) / 16), o);
        } else {
          if (p.bias) {
            const float* b = p.bias + b_tile * BN + g * 32;
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += b[j];
          }
          stage_row<TC, 32>(row, lane, part * (32 * (int)sizeof(TC) / 16), v);
        }
        if (part == groups_per_piece - 1) {
          fence_async_smem();   // the staged rows are visible to the TMA
          __syncwarp();
          if (lane == 0) {
            if (m0 < p.M) {
              const int x = x_tile + (g / groups_per_piece) * OUTC;
              if (p.accumulate) tma_reduce_add_2d(&map_c, my_stage + sb * S::PIECE_BYTES, x, m0);
              else tma_store_2d(&map_c, my_stage + sb * S::PIECE_BYTES, x, m0);
            }
            // a group for every piece, an empty one for rows past M: "all but the newest group" above
            // then always means the store that read the other staging tile
            bulk_commit();
          }
          sb ^= 1;
        }
      }
    }
    if (lane == 0) bulk_wait_all();   // the stores are complete before the block ends
  }

  tc_fence_before();
  if constexpr (PAIR) {
    cluster_sync_all();   // neither block leaves, or frees tensor memory, while the pair's MMAs may still use it
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
  } else {
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------ host side
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

// Map of a row-major [rows, K] bfloat16 matrix (row stride ld elements), tiles of box_rows x 64.
bool make_map(CUtensorMap* map, const void* base, int rows, int K, int ld, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Map of the output C [rows, cols] (row stride ld elements) for stores of 32 rows x 128 bytes.
bool make_out_map(CUtensorMap* map, void* base, int rows, int cols, int ld, bool f32) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const int elt = f32 ? 4 : 2;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * elt};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / elt), 32};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, bool SWAP, typename TC>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& p, dim3 grid, cudaStream_t stream) {
  auto kern = gemm_tc_kernel<BN, STAGES, SWAP, TC>;
  const size_t smem = Smem<BN, STAGES>::BYTES;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits for the one before by itself
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;   // the blocks that split K form one cluster
  attr[1].val.clusterDim.x = 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = p.splits;
  cfg.attrs = attr;
  cfg.numAttrs = p.splits > 1 ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, p);
}

// `n_tiles` tiles of the unit's size (128 x BN, or 256 x BN for pairs); one block per SM at most.
template <int BN, int STAGES, bool PAIR, typename TC>
int launch_persistent(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mc, const Params& p, int n_tiles,
                      cudaStream_t stream) {
  auto kern = gemm_tc_persistent_kernel<BN, STAGES, PAIR, TC>;
  const size_t smem = SmemP<BN, STAGES, PAIR>::BYTES;
  static_assert(SmemP<BN, STAGES, PAIR>::BYTES <= 227 * 1024, "shared memory of one block");
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return ZK_EINVAL;
  if constexpr (!PAIR) {
    return zk_launch_dependent(kern, dim3(n_tiles < sms ? n_tiles : sms), dim3(THREADS), smem, stream, ma, mb, mc, p);
  } else {
    const int units = n_tiles < sms / 2 ? n_tiles : sms / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * units);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;   // blocks 2u and 2u + 1 are the pair u
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the kernel waits for the one before by itself
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return (int)cudaLaunchKernelEx(&cfg, kern, ma, mb, mc, p);
  }
}

// Which form a product of more than 64 rows takes: 0 = one 128 x 128 tile per block; 256 = persistent
// blocks with 128 x 256 tiles; 512 = persistent pairs of blocks with 256 x 256 tiles
// (tcgen05.mma.cta_group::2: each block loads half of the weight tile, so a multiply-add needs half
// the bytes from L2 and from shared memory that a 128 x 128 tile needs).  The persistent forms
// overlap a tile's stores with the next tile's MMAs and store through the TMA; they take N a
// multiple of 256.  Measured on the LFM2-1.2B shapes with 2,048 rows (TFLOP/s, forms 0 / 256 / 512):
// w1|w3 786 / 1291 / 1321, w2 848 / 1181 / 1272, in_proj 787 / 1177 / 1275, qkv 605 / 819 / 865,
// out_proj 536 / 825 / 820; with 256 rows the pairs still lead, with 128 rows a pair's second block
// has no rows and single blocks are chosen.
int forced_form = -1;   // set by zk_gemm_tc_force_form for measurements and tests; -1 = choose
int normal_form(int M, int N) {
  if (N % 256) return 0;
  if (forced_form >= 0) return forced_form;
  return M > 128 ? 512 : 256;
}

}  // namespace

extern "C" {

// X [M, K], W [N, K] bfloat16, K % 8 == 0, rows 16-byte aligned; C [M, N] bfloat16 or float32.
// M <= 64 runs swapped (weights on the 128-row side) with K cut into `splits` parts (rounded down
// to 1, 2, 4 or 8: a cluster's size); larger M runs normal and ignores splits.  With `swiglu`
// W's rows are groups of 16 gate rows and their 16 up rows and C [M, N/2] receives
// silu(gate) * up (src/model.zig:1085-1117).  M <= 64 only: ssq_in [M, ssq_parts] (or null) says
// that X is bfloat16(x * norm weight) and scales token t's sums by 1 / sqrt(sum(ssq_in[t]) / K +
// eps); emit_x (or null; float32 C, no SwiGLU) is written as bfloat16(C * emit_w), [M, N], and
// emit_ssq [M, ceil(N / 32)] as the sums of C^2 over 32 columns.
int zk_gemm_tc(const void* X, const void* W, void* C, const float* bias, int M, int N, int K, int ldx, int ldw, int ldc,
               int out_dtype, int accumulate, int splits, int swiglu, const float* ssq_in, int ssq_parts, float eps,
               const float* emit_w, void* emit_x, float* emit_ssq, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((ssq_in || emit_x) && M > 64) return ZK_EINVAL;
  if (ssq_in && ssq_parts <= 0) return ZK_EINVAL;
  if (emit_x && (!emit_w || !emit_ssq || swiglu || out_dtype != ZK_F32)) return ZK_EINVAL;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || ldx < K || ldw < K || ldc < (swiglu ? N / 2 : N) || !status) return ZK_EINVAL;
  if (swiglu && (N % 32 || bias || accumulate)) return ZK_EINVAL;
  if (((uintptr_t)X | (uintptr_t)W | (uintptr_t)C) % 16) return ZK_EINVAL;
  if (out_dtype != ZK_F32 && out_dtype != ZK_BF16) return ZK_EINVAL;
  Params p{};
  p.C = C; p.bias = bias; p.status = status;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.accumulate = accumulate; p.splits = 1; p.swiglu = swiglu;
  p.ssq_in = ssq_in; p.ssq_parts = ssq_parts; p.eps = eps;
  p.emit_w = emit_w; p.emit_x = (bf16*)emit_x; p.emit_ssq = emit_ssq;
  CUtensorMap ma, mb, mc;
  const bool f32 = out_dtype == ZK_F32;
  if (M > 64) {
    // the persistent forms store through the TMA: rows of C 16-byte aligned, and an add only in float32
    const bool tma_out = (ldc * (f32 ? 4 : 2)) % 16 == 0 && (f32 || !accumulate);
    const int form = tma_out ? normal_form(M, N) : 0;
    if (form == 512 || form == 256) {
      constexpr int BW = 256;
      const bool pair = form == 512;
      if (!make_map(&ma, X, M, K, ldx, BM) || !make_map(&mb, W, N, K, ldw, pair ? BW / 2 : BW) ||
          !make_out_map(&mc, C, M, swiglu ? N / 2 : N, ldc, f32))
        return ZK_EINVAL;
      const int n_tiles = ceil_div_i(M, pair ? 2 * BM : BM) * ceil_div_i(N, BW);
      if (pair)
        return f32 ? launch_persistent<BW, 6, true, float>(ma, mb, mc, p, n_tiles, stream)
                   : launch_persistent<BW, 6, true, bf16>(ma, mb, mc, p, n_tiles, stream);
      return f32 ? launch_persistent<BW, 4, false, float>(ma, mb, mc, p, n_tiles, stream)
                 : launch_persistent<BW, 4, false, bf16>(ma, mb, mc, p, n_tiles, stream);
    }
    constexpr int BN = 128;
    if (!make_map(&ma, X, M, K, ldx, BM) || !make_map(&mb, W, N, K, ldw, BN)) return ZK_EINVAL;
    dim3 grid(ceil_div_i(M, BM), ceil_div_i(N, BN), 1);
    // three stages of 32 KB: two blocks fit an SM, so one block's epilogue overlaps the other's MMAs
    return f32 ? launch<BN, 3, false, float>(ma, mb, p, grid, stream) : launch<BN, 3, false, bf16>(ma, mb, p, grid, stream);
  }
  const int nkb = ceil_div_i(K, BK);
  int s2 = 1;
  while (s2 * 2 <= splits && s2 * 2 <= 8 && s2 * 2 <= nkb) s2 *= 2;
  while (s2 > 1 && ceil_div_i(nkb, s2) * (s2 - 1) >= nkb) s2 /= 2;  // no empty split
  p.splits = s2;
  splits = s2;
  const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  if (!make_map(&ma, W, N, K, ldw, BM) || !make_map(&mb, X, M, K, ldx, bn)) return ZK_EINVAL;
  dim3 grid(ceil_div_i(N, BM), 1, splits);
  // four stages: measured on whole steps of 16 / 64 sequences 1.09 / 1.40 ms, with three stages 1.12 / 1.48,
  // with eight 1.18 / 1.72
#define ZK_TC_SWAP(BNV)                                                                     \
  return f32 ? launch<BNV, 4, true, float>(ma, mb, p, grid, stream) : launch<BNV, 4, true, bf16>(ma, mb, p, grid, stream);
  if (bn == 16) { ZK_TC_SWAP(16) }
  if (bn == 32) { ZK_TC_SWAP(32) }
  ZK_TC_SWAP(64)
#undef ZK_TC_SWAP
}

// Forces the form of products with more than 64 rows and N a multiple of 256: 0 one 128 x 128 tile
// per block, 256 persistent blocks, 512 persistent pairs of blocks; -1 gives the choice back.
int zk_gemm_tc_force_form(int form) {
  if (form != -1 && form != 0 && form != 256 && form != 512) return ZK_EINVAL;
  forced_form = form;
  return 0;
}

}  // extern "C"
