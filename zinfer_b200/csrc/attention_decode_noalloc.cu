// Implementation of attention_decode_noalloc.h: the single-token attention kernel of
// attention_decode.cu with its chunk scratch in a file-scope device array.
#include "attention_decode_noalloc.h"

#include <mutex>
#include <stdio.h>

#include "attention_decode.cu"  // the kernel template and its launcher (zk_attn_decode)

// The scratch: partial outputs [num_splits, n_seqs*H, hd] float32, then (m, l) pairs
// [num_splits, n_seqs*H, 2] float32.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char zk_noalloc_scratch[ZK_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int MAX_DEVICES = 64;
float* g_scratch[MAX_DEVICES];   // device address of the array, per device; null until looked up
std::mutex g_mutex;
thread_local char g_error[256];

// out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s over the chunks; one warp per (token, head).
__global__ void noalloc_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     bf16* __restrict__ out, int n_rows, int hd, int num_splits) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, part_ml[((size_t)s * n_rows + row) * 2]);
  float L = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = part_ml[((size_t)s * n_rows + row) * 2];
    if (ms != -INFINITY) L += expf(ms - M) * part_ml[((size_t)s * n_rows + row) * 2 + 1];
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  for (int d = lane; d < hd; d += 32) {
    float acc = 0.f;
    for (int s = 0; s < num_splits; ++s) {
      const float ms = part_ml[((size_t)s * n_rows + row) * 2];
      if (ms != -INFINITY) acc = fmaf(expf(ms - M), part_o[((size_t)s * n_rows + row) * hd + d], acc);
    }
    out[(size_t)row * hd + d] = __float2bfloat16_rn(acc * inv);
  }
}

// Device address of the scratch on the current device; looked up once per device.
int scratch_address(float** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return ZK_EINVAL;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (!g_scratch[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, zk_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch[dev] = static_cast<float*>(p);
  }
  *ptr = g_scratch[dev];
  return 0;
}

}  // namespace

extern "C" {

long long zk_attn_decode_noalloc_bytes(int n_seqs, int H, int hd, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long long)num_splits * n_seqs * H * (hd + 2) * (long long)sizeof(float);
}

const char* zk_attn_decode_noalloc_error(void) { return g_error; }

int zk_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* seq_start,
                           const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H, int Hkv,
                           int hd, int page_size, int window, float scale, int num_splits, int split_keys,
                           cudaStream_t stream) {
  g_error[0] = 0;
  if (n_seqs <= 0) return 0;
  if (!zk_attn_decode_takes(H, Hkv, hd, page_size) || num_splits < 1 ||
      (num_splits > 1 && (split_keys <= 0 || split_keys % DEC_TK))) {
    snprintf(g_error, sizeof g_error,
             "zk_attn_decode_noalloc: sizes not taken (H %d, Hkv %d, head_dim %d, page_size %d, num_splits %d, "
             "split_keys %d): head_dim in {32, 64, 96, 128}, at most 8 heads per KV head, page_size and split_keys "
             "multiples of 32", H, Hkv, hd, page_size, num_splits, split_keys);
    return ZK_EINVAL;
  }
  const long long need = zk_attn_decode_noalloc_bytes(n_seqs, H, hd, num_splits);
  if (need > (long long)ZK_NOALLOC_SCRATCH_BYTES) {
    snprintf(g_error, sizeof g_error,
             "zk_attn_decode_noalloc: %d chunks x %d sequences x %d heads of %d need %lld bytes of scratch, the "
             "built-in array holds %u: use fewer chunks or the allocating entry point",
             num_splits, n_seqs, H, hd, need, ZK_NOALLOC_SCRATCH_BYTES);
    return ZK_NOALLOC_TOO_LARGE;
  }
  float* part_o = nullptr;
  float* part_ml = nullptr;
  if (num_splits > 1) {
    float* base = nullptr;
    const int rc = scratch_address(&base);
    if (rc != 0) {
      snprintf(g_error, sizeof g_error, "zk_attn_decode_noalloc: cudaGetSymbolAddress failed with status %d", rc);
      return rc;
    }
    part_o = base;
    part_ml = base + (size_t)num_splits * n_seqs * H * hd;
  }
  int rc = zk_attn_decode(q, k_cache, v_cache, out, part_o, part_ml, seq_start, seq_slot, page_table, pt_stride, n_seqs,
                          H, Hkv, hd, page_size, window, scale, num_splits, split_keys, stream);
  if (rc == 0 && num_splits > 1) {
    const int n_rows = n_seqs * H, warps = 4;
    noalloc_merge_kernel<<<(n_rows + warps - 1) / warps, warps * 32, 0, stream>>>(part_o, part_ml, (bf16*)out, n_rows,
                                                                                 hd, num_splits);
    rc = (int)cudaGetLastError();
  }
  if (rc != 0) snprintf(g_error, sizeof g_error, "zk_attn_decode_noalloc: launch failed with status %d", rc);
  return rc;
}

}  // extern "C"
