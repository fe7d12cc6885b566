// Single-token attention over the paged cache for callers that must not allocate.
//
// This entry point has no counterpart in pylypenko99/zinfer (a CPU program that owns all of
// its buffers); it exists for hosts of this library that cannot call cudaMalloc at the moment
// they need attention: code that runs while a CUDA graph is being captured, a real-time loop
// that may not take the allocator's lock, a process whose memory budget was handed out at
// start-up and is closed afterwards.  The regular entry point (`zk_attn_decode`) cuts long
// key ranges into chunks and needs scratch memory for the chunks' partial results, which its
// caller allocates.  Here that scratch is a fixed array inside the library.
//
// Cost and limit: every GPU that loads this library holds ZK_NOALLOC_SCRATCH_BYTES (8 MiB) of
// device memory until the process exits.  A call needs
//     num_splits * n_seqs * H * (head_dim + 2) * 4 bytes
// of it (nothing when num_splits == 1) and is refused with ZK_NOALLOC_TOO_LARGE if that is more.
//
// Rules for callers:
//  * The chunks must cover the longest sequence: num_splits * split_keys >= seq_start[b] + 1 for
//    every b (with num_splits == 1 all keys are one chunk, whatever their number).  The lengths
//    live on the device, so the call cannot check this; keys beyond the last chunk would be
//    left out of the result without an error.  A caller whose sequences grow keeps
//    num_splits * split_keys ahead of them.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress).  Make that first call outside any stream capture.
//  * All calls on a device share the one array, and it keeps what the last call left in it.
//    Nothing in it has to be zero: every value a call reads it has written before in the same
//    call.  But two calls that overlap on the GPU (different streams, or graphs replayed
//    concurrently) would overwrite each other's partial results: run them one after another.
//  * The call makes no cudaMalloc, cudaFree or other allocating call; inputs and outputs are
//    the caller's.
#pragma once

#include <cuda_runtime.h>

#define ZK_NOALLOC_SCRATCH_BYTES (8u << 20)
#define ZK_NOALLOC_TOO_LARGE (-7)

#ifdef __cplusplus
extern "C" {
#endif

// q, out [n_seqs, H*hd] bfloat16; k_cache, v_cache one layer's [pages, Hkv, page_size, hd]
// bfloat16; seq_start[b] = number of tokens of sequence b already in the cache before this
// step's token (whose key and value must already be written at that position); seq_slot[b] =
// row of page_table ([slots, pt_stride] int32, -1 = no page); keys are cut at multiples of
// split_keys (a multiple of 32) into num_splits chunks.  Returns 0, a cudaError_t value,
// ZK_EINVAL (-22) for sizes the kernel does not take, or ZK_NOALLOC_TOO_LARGE.
int zk_attn_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out, const int* seq_start,
                           const int* seq_slot, const int* page_table, int pt_stride, int n_seqs, int H, int Hkv,
                           int hd, int page_size, int window, float scale, int num_splits, int split_keys,
                           cudaStream_t stream);

// Bytes of the built-in scratch a call with these sizes needs.
long long zk_attn_decode_noalloc_bytes(int n_seqs, int H, int hd, int num_splits);

// Text for the last non-zero status this thread got from zk_attn_decode_noalloc.
const char* zk_attn_decode_noalloc_error(void);

#ifdef __cplusplus
}
#endif
