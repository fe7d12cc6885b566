// One kernel for a whole single-token step (up to 16 sequences, bfloat16).
//
// A single-token step of a 16-layer model is some hundred small contractions and row kernels that
// each depend on the one before.  Here the step is a *program*: an array of operations (embedding,
// contractions with their fused prologues and epilogues, attention) that ONE persistent grid of
// one block per SM runs in order, with a grid-wide barrier where an operation needs the previous
// one's result.  Within an operation the tasks (groups of 16 weight rows; (sequence, KV head)
// pairs) are dealt round-robin to the blocks.  Weights reach shared memory through a per-thread
// cp.async ring that runs ahead of the barriers (see "weight stream" below).
//
// The arithmetic is that of the separate kernels: gemm_skinny.cu (mma.sync.m16n8k16 with the
// weights on the 16-row side, K split over the block's 16 warps, partial sums added in warp
// order), the RMSNorm prologue, the SwiGLU and short-convolution epilogues, and the single-token
// attention of attention_decode.cu with the q/k norm, rotation and cache write of attention.cu in
// front of it.  References: the layer loop src/model.zig:2395-2422; shortConv
// src/model.zig:1994-2028; attention src/model.zig:1715-1991; final norm and head
// src/model.zig:2484-2490.
//
// Memory: activations written by one block and read by another go through L2 (loads with
// ld.global.cg); a block never reads through L1 what another block wrote during the launch.
// The barrier is a counter in global memory that only grows; its spin is bounded (about two
// seconds), after which the block sets *status = 21 and marks the counter so that every block
// leaves at once.  The host zeroes the counter before each launch.  *status = 22: an operation asks
// for a K that is no multiple of 32 or a normalised input too long to stage; nothing runs.
//
// Measured on a B200 (LFM2-1.2B shape, 8 sequences, 72 operations): 1.40 ms a step against 1.04 ms
// for the CUDA graph of the separate kernels, so the engine uses this kernel only on request.  Per
// operation block 0 spends about 2 us at the barrier and 2 to 3.5 us staging its input (chains of
// L2 round trips of 0.7 to 1 us); the contraction loops run at some 35 GB/s per SM whether the
// weights come from DRAM or from L2 (they are bound by instruction issue, not by memory); and the
// attention operation gives a sequence's keys to one block, which at one to eight sequences
// leaves most SMs idle.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int WARPS = 16;
constexpr int THREADS = WARPS * 32;
constexpr int MAX_M = 16;
constexpr int SMEM_BYTES = 227 * 1024;
constexpr int SCRATCH_FLOATS = MAX_M + MAX_M * WARPS + 4;  // row scales, their partial sums, the barrier's flag

// Shared memory of a launch for up to 8 (NT = 1) or 16 (NT = 2) sequences: the partial sums of
// the warps, the scratch, the weight ring and the staged input rows.
template <int NT>
struct Layout {
  static constexpr int RED_FLOATS = WARPS * 48 * (NT * 8 + 1);   // [warps][3 x 16 rows][tokens + 1]
  static constexpr int CAP = NT == 1 ? 8 : 4;                    // ring units of 32 bytes per thread (a power of two)
  static constexpr int RING_BYTES = CAP * 2 * THREADS * 16;
  static constexpr int XS_BYTES = SMEM_BYTES - 4 * (RED_FLOATS + SCRATCH_FLOATS) - RING_BYTES;
  // columns of X staged at once: whole slab rounds of the 16 warps
  static constexpr int KC = (XS_BYTES / (NT * 8 * 2) - 8) / (32 * WARPS) * (32 * WARPS);
  static_assert(KC >= 2048, "the staged rows must hold a model width");
};
constexpr long long WAIT_CYCLES = 4000000000LL;

enum { OP_EMBED = 0, OP_GEMM = 1, OP_ATTN = 2 };
enum { XIN_BF16 = 0, XIN_NORM = 1 };
enum { EPI_BF16 = 0, EPI_ACC_F32 = 1, EPI_F32 = 2, EPI_SWIGLU = 3, EPI_CONV = 4 };

struct Op {
  int kind, xin, epi, rg;
  int N, K, ldw, ldx, ldc, taps;
  int H, Hkv, hd, n_rot, rope_interleaved, page_size, window, pt_stride, vocab, pad0;
  float eps, scale;
  long long state_stride;
  const bf16* W;
  const void* X;
  const float* norm_w;
  void* C;
  const float* bias;
  float* conv_state;
  const float* conv_taps;
  const float* conv_bias;
  bf16* k_cache;
  bf16* v_cache;
  const float* q_norm;
  const float* k_norm;
  const float* inv_freq;
  const int* page_table;
  const bf16* table;
};

struct Step {
  const Op* ops;
  int n_ops, M;
  const int* tokens;     // [M]
  const int* seq_start;  // [M] tokens already cached = position of this step's token
  const int* seq_slot;   // [M]
  unsigned* barrier;     // arrivals of all barriers so far (zero at launch)
  int* status;
  long long* trace;      // optional [n_ops][4] nanosecond stamps of block 0: operation entered, input staged (first
                         // task), work done, barrier passed
};

// ------------------------------------------------------------------------------ small helpers
__device__ __forceinline__ void mma16816(float c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                         unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ld_act16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float4 ld_act_f4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void stamp(const Step& st, int op_index, int phase) {
  if (st.trace && blockIdx.x == 0 && threadIdx.x == 0) {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    st.trace[op_index * 4 + phase] = t;
  }
}
__device__ __forceinline__ unsigned pack2(float a, float b) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const unsigned*>(&t);
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ void unpack8(const uint4& v, float f[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(p[i]);
    f[2 * i + 1] = __high2float(p[i]);
  }
}

// Grid-wide barrier number `index` (0, 1, ...) of the launch; false = gave up.  One counter that
// only grows: thread 0 of each block adds one (release) and spins (acquire) until all blocks of
// this and every earlier barrier have arrived.  A block that gives up sets the counter's top bit,
// which ends every other block's wait at once.
__device__ bool grid_barrier(unsigned* bar, int index, int* status, int* sm_flag) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned target = (unsigned)(index + 1) * gridDim.x;
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(bar) : "memory");
    const long long t0 = clock64();
    unsigned now;
    for (;;) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(bar) : "memory");
      if (now >= target) break;
      if (clock64() - t0 > WAIT_CYCLES) {
        atomicExch(status, 21);
        now = atomicOr(bar, 0x80000000u) | 0x80000000u;
        break;
      }
    }
    *sm_flag = (now & 0x80000000u) ? 0 : 1;
  }
  __syncthreads();
  return *sm_flag != 0;
}

// ------------------------------------------------------------------------------ embedding
__device__ void embed_op(const Op& op, const Step& st) {
  for (int m = blockIdx.x; m < st.M; m += gridDim.x) {
    const int tok = st.tokens[m];
    const bool ok = tok >= 0 && tok < op.vocab;
    if (!ok && threadIdx.x == 0) atomicExch(st.status, 1);
    const bf16* row = op.table + (size_t)(ok ? tok : 0) * op.K;
    float* out = reinterpret_cast<float*>(op.C) + (size_t)m * op.K;
    for (int d = threadIdx.x; d < op.K; d += THREADS) out[d] = ok ? __bfloat162float(row[d]) * op.scale : 0.f;
  }
}

// ------------------------------------------------------------------------------ weight stream
// Weights do not depend on the step, so their way from DRAM need not wait for the operation that
// uses them.  Every thread knows, from the program alone, the sequence of 16-byte weight pieces
// it will feed to its MMAs during the whole launch: for each contraction, for each of its block's
// tasks, for each group of 16 rows of the task, for each 32-wide k slab of its warp (slab s
// belongs to warp s mod 16), the pieces (row g, k 8c..8c+7) and (row g+8, same k).  It copies them
// with cp.async into a ring of its own in shared memory (unit u, half h at
// ((2u+h)*512 + tid)*16: no two threads share a bank group), always CAP-1 units ahead of the unit
// it consumes: one unit is issued for every unit consumed, so `cp.async.wait_group CAP-1` is the
// oldest unit's arrival.  The copies in flight (CAP-1 units of 16 KB per SM) outlive barriers,
// prologues and epilogues, which is what a chain of separate kernels cannot do.
constexpr unsigned UNIT_BYTES = 2 * THREADS * 16;   // one unit of all threads of the block

struct Producer {
  const bf16* ptr0;      // piece of row g at this warp's next slab
  const bf16* ptr1;      // piece of row g + 8
  int rem;               // slabs left in the current group of rows (0: the stream has ended)
  int bytes0, bytes1;    // 16, or 0 where the row lies beyond the matrix (the copy then writes zeros)
  unsigned dst;          // offset in the ring of the next unit to issue
  int op, task, r;       // the group being produced
  int n_tasks, rg;       // of ops[op]
};

__device__ __forceinline__ int task_groups(const Op& op) {   // groups of 16 weight rows per task
  return op.epi <= EPI_F32 ? op.rg : (op.epi == EPI_SWIGLU ? 2 : 3);
}
__device__ __forceinline__ int task_columns(const Op& op) { return op.epi <= EPI_F32 ? 16 * op.rg : 16; }
__device__ __forceinline__ int weight_rows(const Op& op) {
  return op.epi <= EPI_F32 ? op.N : (op.epi == EPI_SWIGLU ? 2 * op.N : 3 * op.N);
}

// Moves to the next group of 16 rows in which this warp has a slab: the next group of the task,
// the block's next task, the next contraction of the program.
__device__ __forceinline__ void producer_next_group(Producer& p, const Step& st, bool first) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
  if (!first) {
    if (++p.r == p.rg) {
      p.r = 0;
      p.task += gridDim.x;
    }
  }
  for (;;) {
    if (p.task < p.n_tasks) {
      const Op& op = st.ops[p.op];
      const int slabs = op.K / 32;
      if (warp < slabs) {
        const int row = (p.task * p.rg + p.r) * 16 + g, rows = weight_rows(op);
        p.bytes0 = row < rows ? 16 : 0;
        p.bytes1 = row + 8 < rows ? 16 : 0;
        p.ptr0 = op.W + (size_t)(p.bytes0 ? row : 0) * op.ldw + warp * 32 + 8 * c;
        p.ptr1 = op.W + (size_t)(p.bytes1 ? row + 8 : 0) * op.ldw + warp * 32 + 8 * c;
        p.rem = (slabs - warp + WARPS - 1) / WARPS;
        return;
      }
      p.task = p.n_tasks;   // fewer slabs than warps: this warp has no part in the operation
    }
    if (++p.op >= st.n_ops) {
      p.rem = 0;
      return;
    }
    const Op& op = st.ops[p.op];
    p.n_tasks = op.kind == OP_GEMM ? (op.N + task_columns(op) - 1) / task_columns(op) : 0;
    p.rg = task_groups(op);
    p.task = blockIdx.x;
    p.r = 0;
  }
}

// `ring_mine`: shared-memory address of this thread's 16 bytes in unit 0, half 0.
template <int CAP>
__device__ __forceinline__ void produce_unit(Producer& p, const Step& st, unsigned ring_mine) {
  if (p.rem > 0) {
    const unsigned dst = ring_mine + p.dst;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(p.ptr0), "r"(p.bytes0) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + THREADS * 16), "l"(p.ptr1), "r"(p.bytes1)
                 : "memory");
    p.ptr0 += WARPS * 32;
    p.ptr1 += WARPS * 32;
    if (--p.rem == 0) producer_next_group(p, st, false);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  p.dst = (p.dst + UNIT_BYTES) & (CAP * UNIT_BYTES - 1);
}

__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// ------------------------------------------------------------------------------ contraction
// One task: RG groups of 16 adjacent weight rows (interleaved parts for the fused epilogues)
// against the M tokens, group after group; K is split over the block's 16 warps slab by slab and
// the partial sums are added in warp order.  X is staged in shared memory (`xs`), normalised on
// the way if asked, in pieces of KC columns when a whole row does not fit; rows M.. of the staged
// tile are zero.
template <int NT>
__device__ __forceinline__ void stage_rows(const Op& op, const Step& st, int k0, int k1, bf16* xs, int xs_ld,
                                           float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int M = st.M, K = op.K;
  float* row_scale = scratch;          // [16]
  float* part = scratch + MAX_M;       // [16][WARPS]
  if (op.xin == XIN_NORM) {
    // RMSNorm of the M residual rows (src/model.zig:1166-1181); always a whole row.  A thread owns
    // the columns 4*tid + 2048*r of every row; a row's sum of squares is added per thread over r,
    // then over the lanes, then over the warps, whatever M is.
    const float* X = reinterpret_cast<const float*>(op.X);
    const float* xcol = X + threadIdx.x * 4;
    if (K == THREADS * 4) {
      // the thread's values stay in registers: the rows are read once, all loads under way at once
      float4 v[NT * 8];
#pragma unroll
      for (int m = 0; m < NT * 8; ++m)
        v[m] = m < M ? ld_act_f4(xcol + (size_t)m * op.ldx) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float4 w = *reinterpret_cast<const float4*>(op.norm_w + threadIdx.x * 4);
#pragma unroll
      for (int m = 0; m < NT * 8; ++m) {
        float ss = v[m].x * v[m].x;
        ss = fmaf(v[m].y, v[m].y, ss);
        ss = fmaf(v[m].z, v[m].z, ss);
        ss = fmaf(v[m].w, v[m].w, ss);
        const float t = warp_sum(ss);
        if (lane == 0) part[m * WARPS + warp] = t;
      }
      __syncthreads();
      if (threadIdx.x < NT * 8) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < WARPS; ++i) t += part[threadIdx.x * WARPS + i];
        row_scale[threadIdx.x] = 1.0f / sqrtf(t / (float)K + op.eps);
      }
      __syncthreads();
#pragma unroll
      for (int m = 0; m < NT * 8; ++m) {
        const float sc = row_scale[m];
        uint2 pk;
        pk.x = pack2((v[m].x * sc) * w.x, (v[m].y * sc) * w.y);
        pk.y = pack2((v[m].z * sc) * w.z, (v[m].w * sc) * w.w);
        *reinterpret_cast<uint2*>(xs + (size_t)m * xs_ld + threadIdx.x * 4) = pk;
      }
    } else {
      for (int m0 = 0; m0 < NT * 8; m0 += 4) {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        bool any = false;
        for (int k = threadIdx.x * 4; k < K; k += THREADS * 4) {
          float4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = (m0 + j < M) ? ld_act_f4(X + (size_t)(m0 + j) * op.ldx + k) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            ss[j] = any ? fmaf(v[j].x, v[j].x, ss[j]) : v[j].x * v[j].x;
            ss[j] = fmaf(v[j].y, v[j].y, ss[j]);
            ss[j] = fmaf(v[j].z, v[j].z, ss[j]);
            ss[j] = fmaf(v[j].w, v[j].w, ss[j]);
          }
          any = true;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float t = warp_sum(ss[j]);
          if (lane == 0) part[(m0 + j) * WARPS + warp] = t;
        }
      }
      __syncthreads();
      if (threadIdx.x < NT * 8) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < WARPS; ++i) t += part[threadIdx.x * WARPS + i];
        row_scale[threadIdx.x] = 1.0f / sqrtf(t / (float)K + op.eps);
      }
      __syncthreads();
      for (int m0 = 0; m0 < NT * 8; m0 += 4)
        for (int k = threadIdx.x * 4; k < K; k += THREADS * 4) {
          float4 v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            v[j] = (m0 + j < M) ? ld_act_f4(X + (size_t)(m0 + j) * op.ldx + k) : make_float4(0.f, 0.f, 0.f, 0.f);
          const float4 w = *reinterpret_cast<const float4*>(op.norm_w + k);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float sc = row_scale[m0 + j];
            uint2 pk;
            pk.x = pack2((v[j].x * sc) * w.x, (v[j].y * sc) * w.y);
            pk.y = pack2((v[j].z * sc) * w.z, (v[j].w * sc) * w.w);
            *reinterpret_cast<uint2*>(xs + (size_t)(m0 + j) * xs_ld + k) = pk;
          }
        }
    }
  } else {
    // pieces of 8 columns: a thread takes a column of pieces through all rows, its loads in one batch
    const bf16* X = reinterpret_cast<const bf16*>(op.X);
    for (int k = k0 + threadIdx.x * 8; k < k1; k += THREADS * 8) {
      uint4 v[NT * 8];
#pragma unroll
      for (int m = 0; m < NT * 8; ++m) v[m] = m < M ? ld_act16(X + (size_t)m * op.ldx + k) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int m = 0; m < NT * 8; ++m) *reinterpret_cast<uint4*>(xs + (size_t)m * xs_ld + (k - k0)) = v[m];
    }
  }
}

template <int NT, int CAP, int KC>
__device__ __forceinline__ void gemm_op(const Op& op, const Step& st, int op_index, Producer& p, unsigned& c_off,
                                        unsigned ring_mine, float* red_raw, float* scratch, bf16* xs) {
  float(*red)[48][NT * 8 + 1] = reinterpret_cast<float(*)[48][NT * 8 + 1]>(red_raw);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int M = st.M, N = op.N, K = op.K, epi = op.epi;
  const bool plain = epi <= EPI_F32;
  const int RG = task_groups(op);
  const int cols = plain ? 16 * RG : 16;
  const int n_tasks = (N + cols - 1) / cols;
  if ((int)blockIdx.x >= n_tasks) return;
  const int slabs = K / 32;
  const int n_chunks = (K + KC - 1) / KC;
  const int xs_ld = min(K, KC) + 8;
  // shared-memory address of this lane's piece of token g in the slab `warp` of the staged tile
  const unsigned xp = (unsigned)__cvta_generic_to_shared(xs) + (unsigned)((g * xs_ld + 8 * c + warp * 32) * 2);
  bool staged = false;

  for (int task = blockIdx.x; task < n_tasks; task += gridDim.x) {
    const int n0 = task * cols;                        // first output column of the task
    const size_t row0 = (size_t)task * (16 * RG);      // first weight row of the task
    // the residual value a thread will add to is fetched now, not after the contraction
    float old = 0.f;
    if (epi == EPI_ACC_F32 && threadIdx.x < cols * NT * 8) {
      const int m = threadIdx.x / cols, n = n0 + threadIdx.x % cols;
      if (m < M && n < N) old = __ldcg(reinterpret_cast<const float*>(op.C) + (size_t)m * op.ldc + n);
    }
    __syncthreads();   // the previous task's epilogue has read `red`; its MMAs have read `xs`

    for (int r = 0; r < RG; ++r) {
      float acc[NT][4];
#pragma unroll
      for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][i] = 0.f;
      for (int chunk = 0; chunk < n_chunks; ++chunk) {
        const int k0 = chunk * KC;
        if (n_chunks > 1 || !staged) {
          if (staged) __syncthreads();   // xs is still being read
          stage_rows<NT>(op, st, k0, min(K, k0 + KC), xs, xs_ld, scratch);
          __syncthreads();
          if (!staged) stamp(st, op_index, 1);
          staged = true;
        }
        const int s_end = min(slabs, (k0 + KC) / 32);
        int n = (s_end - k0 / 32 - warp + WARPS - 1) / WARPS;   // this warp's slabs in the piece
        unsigned xa = xp;
#pragma unroll 1
        for (; n > 0; --n) {
          produce_unit<CAP>(p, st, ring_mine);
          asm volatile("cp.async.wait_group %0;" ::"n"(CAP - 1) : "memory");
          const uint4 w0 = lds128(ring_mine + c_off);
          const uint4 w1 = lds128(ring_mine + c_off + THREADS * 16);
          c_off = (c_off + UNIT_BYTES) & (CAP * UNIT_BYTES - 1);
#pragma unroll
          for (int t = 0; t < NT; ++t) {
            const uint4 xv = lds128(xa + (unsigned)(t * 8 * xs_ld * 2));
            mma16816(acc[t], w0.x, w1.x, w0.y, w1.y, xv.x, xv.y);
            mma16816(acc[t], w0.z, w1.z, w0.w, w1.w, xv.z, xv.w);
          }
          xa += WARPS * 32 * 2;
        }
      }
#pragma unroll
      for (int t = 0; t < NT; ++t) {
        red[warp][r * 16 + g][t * 8 + 2 * c] = acc[t][0];
        red[warp][r * 16 + g][t * 8 + 2 * c + 1] = acc[t][1];
        red[warp][r * 16 + g + 8][t * 8 + 2 * c] = acc[t][2];
        red[warp][r * 16 + g + 8][t * 8 + 2 * c + 1] = acc[t][3];
      }
    }
    __syncthreads();
    auto total = [&](int row, int m) {
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[w][row][m];
      return v;
    };

    if (plain) {
      for (int idx = threadIdx.x; idx < cols * NT * 8; idx += THREADS) {
        const int m = idx / cols, nl = idx % cols;
        const int n = n0 + nl;
        if (m >= M || n >= N) continue;
        float v = total(nl, m);
        if (op.bias) v += op.bias[n];
        if (epi == EPI_BF16) {
          reinterpret_cast<bf16*>(op.C)[(size_t)m * op.ldc + n] = __float2bfloat16_rn(v);
        } else {
          float* dst = reinterpret_cast<float*>(op.C) + (size_t)m * op.ldc + n;
          if (epi == EPI_ACC_F32) v += idx == (int)threadIdx.x ? old : __ldcg(dst);
          *dst = v;
        }
      }
    } else if (epi == EPI_SWIGLU) {
      bf16* C = reinterpret_cast<bf16*>(op.C);
      for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += THREADS) {
        const int m = idx / 16, i = idx % 16;
        const int n = n0 + i;
        if (m >= M || n >= N) continue;
        const float gate = total(i, m), up = total(16 + i, m);
        C[(size_t)m * op.ldc + n] = __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
      }
    } else {   // EPI_CONV: token m is sequence m
      bf16* C = reinterpret_cast<bf16*>(op.C);
      const int taps = op.taps;
      for (int idx = threadIdx.x; idx < 16 * NT * 8; idx += THREADS) {
        const int m = idx / 16, i = idx % 16;
        const int ch = n0 + i;
        if (m >= M || ch >= N) continue;
        float bv = total(i, m), cv = total(16 + i, m), xval = total(32 + i, m);
        if (op.bias) {
          const size_t base = row0 + i;
          bv += op.bias[base];
          cv += op.bias[base + 16];
          xval += op.bias[base + 32];
        }
        const float u_new = round_bf16(bv) * round_bf16(xval);
        float* state = op.conv_state + (size_t)st.seq_slot[m] * op.state_stride;
        float sum = 0.f;
        for (int kk = 0; kk < taps - 1; ++kk) {
          const float u = state[(size_t)kk * N + ch];
          sum = fmaf(op.conv_taps[(size_t)kk * N + ch], u, sum);
          if (kk > 0) state[(size_t)(kk - 1) * N + ch] = u;
        }
        sum = fmaf(op.conv_taps[(size_t)(taps - 1) * N + ch], u_new, sum);
        state[(size_t)(taps - 2) * N + ch] = u_new;
        if (op.conv_bias) sum += op.conv_bias[ch];
        C[(size_t)m * op.ldc + ch] = __float2bfloat16_rn(round_bf16(cv) * sum);
      }
    }
  }
}

// ------------------------------------------------------------------------------ attention
// One task = (sequence b, KV head): per-head RMSNorm and rotation of the G query heads and of the
// new key, cache write of the new key and value, then attention of the G heads over the cache.
// The new token's own key and value are taken from shared memory, not read back.
template <int VPL, int G>
__device__ __noinline__ void attn_task(const Op& op, const Step& st, int task, float* smem_f) {
  constexpr int HD = 32 * VPL;
  float* qs = smem_f;                          // [G][HD] scaled queries
  float* knew = qs + G * HD;                   // [HD]
  float* vnew = knew + HD;                     // [HD]
  float* sm_m = vnew + HD;                     // [WARPS][G]
  float* sm_l = sm_m + WARPS * G;              // [WARPS][G]
  float* sm_o = sm_l + WARPS * G;              // [WARPS][G][HD]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int H = op.H, Hkv = op.Hkv;
  const int b = task / Hkv, kvh = task % Hkv;
  const int pos = st.seq_start[b], L = pos + 1;
  const int* pt = op.page_table + (size_t)st.seq_slot[b] * op.pt_stride;
  const int lo = (op.window > 0 && L > op.window) ? L - op.window : 0;
  const bf16* qkv = reinterpret_cast<const bf16*>(op.X) + (size_t)b * (H + 2 * Hkv) * HD;

  __syncthreads();   // the shared memory of the previous task is free
  if (warp < G + 2) {
    const int kind = warp < G ? 0 : (warp == G ? 1 : 2);
    const bf16* src = qkv + (size_t)(kind == 0 ? kvh * G + warp : (kind == 1 ? H + kvh : H + Hkv + kvh)) * HD;
    const float* w = kind == 0 ? op.q_norm : (kind == 1 ? op.k_norm : nullptr);
    float* dst = kind == 0 ? qs + warp * HD : (kind == 1 ? knew : vnew);
    float ss = 0.f;
    for (int d = lane; d < HD; d += 32) {
      const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(src) + d);
      const float v = __bfloat162float(__ushort_as_bfloat16(raw));
      dst[d] = v;
      ss = fmaf(v, v, ss);
    }
    if (w) {
      ss = warp_sum(ss);
      const float sc = 1.0f / sqrtf(ss / (float)HD + op.eps);
      for (int d = lane; d < HD; d += 32) dst[d] = (dst[d] * sc) * w[d];
    }
    __syncwarp();
    if (kind != 2 && op.inv_freq) {
      const int half = op.n_rot >> 1;
      for (int i = lane; i < half; i += 32) {
        const int ia = op.rope_interleaved ? 2 * i : i, ib = op.rope_interleaved ? 2 * i + 1 : i + half;
        const float ang = (float)pos * op.inv_freq[i];
        const float cs = cosf(ang), sn = sinf(ang);
        const float a = dst[ia], bb = dst[ib];
        dst[ia] = a * cs - bb * sn;
        dst[ib] = a * sn + bb * cs;
      }
      __syncwarp();
    }
    if (kind == 0) {
      for (int d = lane; d < HD; d += 32) dst[d] = round_bf16(dst[d]) * op.scale;
    } else {
      const int page = pt[pos / op.page_size];
      if (page < 0) {
        if (lane == 0) atomicExch(st.status, 2);
      } else {
        bf16* cache = kind == 1 ? op.k_cache : op.v_cache;
        bf16* out = cache + (((size_t)page * Hkv + kvh) * op.page_size + pos % op.page_size) * HD;
        for (int d = lane; d < HD; d += 32) {
          const bf16 r = __float2bfloat16_rn(dst[d]);
          out[d] = r;
          dst[d] = __bfloat162float(r);
        }
      }
    }
  }
  __syncthreads();

  float m[G], l[G], o[G][VPL];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    m[h] = -INFINITY;
    l[h] = 0.f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) o[h][i] = 0.f;
  }
  for (int tile = lo / 32 + warp; tile * 32 < L; tile += WARPS) {
    const int base = tile * 32;
    const int j_lo = max(lo - base, 0), j_hi = min(L - base, 32);
    const int page = pt[base / op.page_size];
    if (page < 0 || j_hi <= j_lo) continue;
    const size_t row0 = (((size_t)page * Hkv + kvh) * op.page_size + base % op.page_size) * HD;
    const bool valid = lane >= j_lo && lane < j_hi;
    const int j_new = pos - base;   // lane of the new token in this tile, if 0 <= j_new < 32

    // the tile's 32 value rows (two values per lane each) are requested before the scores need
    // the keys, all at once: loads inside the j loop's branches would wait for one another
    static_assert(VPL == 2, "one 32-bit load per value row and lane");
    unsigned vraw[32];
    {
      const bf16* vr = op.v_cache + row0 + (size_t)lane * VPL;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const bool in = j >= j_lo && j < j_hi && j != j_new;
        vraw[j] = in ? __ldcg(reinterpret_cast<const unsigned*>(vr + (size_t)j * HD)) : 0u;
      }
    }
    float s[G];
#pragma unroll
    for (int h = 0; h < G; ++h) s[h] = 0.f;
    if (valid) {
      uint4 kv[HD / 8];
      if (lane != j_new) {
        const uint4* kr = reinterpret_cast<const uint4*>(op.k_cache + row0 + (size_t)lane * HD);
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) kv[c] = __ldcg(kr + c);
      }
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        float kf[8];
        if (lane != j_new) {
          unpack8(kv[c], kf);
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) kf[i] = knew[c * 8 + i];
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
          const float4 q0 = *reinterpret_cast<const float4*>(&qs[h * HD + c * 8]);
          const float4 q1 = *reinterpret_cast<const float4*>(&qs[h * HD + c * 8 + 4]);
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
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      float v[VPL];
      if (j == j_new) {
#pragma unroll
        for (int i = 0; i < VPL; ++i) v[i] = vnew[lane * VPL + i];
      } else {
        const __nv_bfloat162 t2 = *reinterpret_cast<const __nv_bfloat162*>(&vraw[j]);
        v[0] = __low2float(t2);
        v[1] = __high2float(t2);
      }
#pragma unroll
      for (int h = 0; h < G; ++h) {
        const float pj = __shfl_sync(0xffffffffu, p[h], j);
#pragma unroll
        for (int i = 0; i < VPL; ++i) o[h][i] = fmaf(pj, v[i], o[h][i]);
      }
    }
  }
#pragma unroll
  for (int h = 0; h < G; ++h) {
    if (lane == 0) {
      sm_m[warp * G + h] = m[h];
      sm_l[warp * G + h] = l[h];
    }
#pragma unroll
    for (int i = 0; i < VPL; ++i) sm_o[(warp * G + h) * HD + lane * VPL + i] = o[h][i];
  }
  __syncthreads();
  bf16* out = reinterpret_cast<bf16*>(op.C);
  for (int idx = tid; idx < G * HD; idx += THREADS) {
    const int h = idx / HD, d = idx % HD;
    float Mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) Mx = fmaxf(Mx, sm_m[w * G + h]);
    float Ls = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float e = sm_m[w * G + h] == -INFINITY ? 0.f : expf(sm_m[w * G + h] - Mx);
      Ls = fmaf(e, sm_l[w * G + h], Ls);
      O = fmaf(e, sm_o[(w * G + h) * HD + d], O);
    }
    out[(size_t)b * H * HD + (size_t)(kvh * G + h) * HD + d] = __float2bfloat16_rn(Ls > 0.f ? O / Ls : 0.f);
  }
}

__device__ __forceinline__ void attn_op(const Op& op, const Step& st, float* smem_f) {
  const int n_tasks = st.M * op.Hkv;
  const int G = op.H / op.Hkv, vpl = op.hd / 32;
  for (int task = blockIdx.x; task < n_tasks; task += gridDim.x) {
#define ZK_ATT_CASE(V, GG)                                  \
  if (vpl == V && G == GG) {                                \
    attn_task<V, GG>(op, st, task, smem_f);                 \
    continue;                                               \
  }
    ZK_ATT_CASE(2, 1) ZK_ATT_CASE(2, 2) ZK_ATT_CASE(2, 4)
#undef ZK_ATT_CASE
  }
}
// attention's shared memory (for 4 heads of 64 per KV head) lies in the partial sums' region
static_assert((4 * 64 + 2 * 64 + 2 * WARPS * 4 + WARPS * 4 * 64) <= Layout<1>::RED_FLOATS, "attention scratch");

template <int NT>
__global__ void __launch_bounds__(THREADS, 1) fused_decode_kernel(const Step st) {
  using L = Layout<NT>;
  extern __shared__ __align__(16) float smem[];
  float* red = smem;
  float* scratch = red + L::RED_FLOATS;
  int* sm_flag = reinterpret_cast<int*>(scratch + MAX_M + MAX_M * WARPS);
  char* ring = reinterpret_cast<char*>(scratch + SCRATCH_FLOATS);
  bf16* xs = reinterpret_cast<bf16*>(ring + L::RING_BYTES);
  const unsigned ring_mine = (unsigned)__cvta_generic_to_shared(ring) + threadIdx.x * 16;

  // The host builds no program the kernel cannot run; if one arrives all blocks refuse it alike.
  for (int i = 0; i < st.n_ops; ++i) {
    const Op& op = st.ops[i];
    if (op.kind == OP_GEMM && (op.K % 32 != 0 || (op.xin == XIN_NORM && op.K > L::KC) || task_groups(op) < 1 ||
                               task_groups(op) > 3)) {
      if (threadIdx.x == 0) atomicExch(st.status, 22);
      return;
    }
  }

  Producer p;
  p.ptr0 = p.ptr1 = nullptr;
  p.rem = p.bytes0 = p.bytes1 = 0;
  p.dst = 0;
  p.op = -1;
  p.task = p.n_tasks = p.r = 0;
  p.rg = 1;
  producer_next_group(p, st, true);
#pragma unroll 1
  for (int i = 0; i < L::CAP - 1; ++i) produce_unit<L::CAP>(p, st, ring_mine);
  unsigned c_off = 0;

#pragma unroll 1
  for (int i = 0; i < st.n_ops; ++i) {
    const Op& op = st.ops[i];
    stamp(st, i, 0);
    if (op.kind == OP_EMBED) embed_op(op, st);
    else if (op.kind == OP_GEMM) gemm_op<NT, L::CAP, L::KC>(op, st, i, p, c_off, ring_mine, red, scratch, xs);
    else attn_op(op, st, smem);
    stamp(st, i, 2);
    if (i + 1 < st.n_ops && !grid_barrier(st.barrier, i, st.status, sm_flag)) break;
    stamp(st, i, 3);
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
}

}  // namespace

extern "C" {

int zk_fused_decode_op_bytes() { return (int)sizeof(Op); }
int zk_fused_decode_max_rows() { return MAX_M; }
// Longest row a normalised input may have with `M` sequences (other inputs are staged in pieces).
int zk_fused_decode_max_staged_k(int M) { return M <= 8 ? Layout<1>::KC : Layout<2>::KC; }

// Whether the attention operation takes these sizes (head_dim 64; 1, 2 or 4 heads per KV head).
int zk_fused_decode_attn_takes(int H, int Hkv, int hd, int page_size) {
  if (Hkv <= 0 || H % Hkv) return 0;
  const int G = H / Hkv;
  return hd == 64 && (G == 1 || G == 2 || G == 4) && page_size % 32 == 0;
}

// Runs the program `ops` (device array of n_ops records laid out as `Op`) for M sequences.
// `barrier` is a zeroed 32-bit word.  One block per SM (`n_blocks` <= the number of SMs).
// `trace`, if not null, receives [n_ops][4] nanosecond stamps of block 0 (see Step).
int zk_fused_decode(const void* ops, int n_ops, int M, const int* tokens, const int* seq_start, const int* seq_slot,
                    unsigned* barrier, int* status, int n_blocks, long long* trace, cudaStream_t stream) {
  if (n_ops <= 0 || M <= 0) return 0;
  if (M > MAX_M || n_blocks <= 0 || !barrier || !status) return ZK_EINVAL;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(fused_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fused_decode_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  Step st{};
  st.ops = reinterpret_cast<const Op*>(ops);
  st.n_ops = n_ops;
  st.M = M;
  st.tokens = tokens;
  st.seq_start = seq_start;
  st.seq_slot = seq_slot;
  st.barrier = barrier;
  st.status = status;
  st.trace = trace;
  void* args[] = {&st};
  // a cooperative launch: the runtime refuses it unless all blocks can be resident at once, which
  // the grid barrier needs
  const void* kern = M <= 8 ? (const void*)fused_decode_kernel<1> : (const void*)fused_decode_kernel<2>;
  return (int)cudaLaunchCooperativeKernel(kern, dim3(n_blocks), dim3(THREADS), args, SMEM_BYTES, stream);
}

}  // extern "C"
