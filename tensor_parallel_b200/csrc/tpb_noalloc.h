// Allocation-free decode attention.
//
// This entry point has no counterpart in the reference library (which never touches device memory itself);
// it exists for callers of this library that are not in a position to allocate GPU memory at all:
//   * serving processes that hand the whole GPU to their KV cache at start-up, so that any later
//     cudaMalloc simply fails;
//   * hosts that embed this library behind a plain C interface and own every buffer themselves (another
//     framework's allocator, a memory pool of fixed size), where a hidden allocation would escape
//     their accounting;
//   * latency-critical loops that cannot afford the implicit device-wide synchronisation of cudaMalloc /
//     cudaFree between two kernels.
// The regular entry point tpb_attn_decode needs a caller-provided workspace for its split-KV partial results.
// The variant below keeps that workspace inside the library instead, in one statically allocated device array,
// so the caller passes nothing but inputs and outputs and the library calls no allocation routine of any
// kind (no cudaMalloc / cudaFree, no stream-ordered allocator, no framework allocator).
#pragma once
#include "tpb_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Size of the built-in workspace in floats (8 MiB).  Every GPU that loads the library carries this array
// from load until the process exits, whether or not the entry point is ever called.
#define TPB_NOALLOC_SCRATCH_FLOATS (2 * 1024 * 1024)

// Same operation and argument meaning as tpb_attn_decode, minus the two workspace pointers:
//   q [batch, q_heads, head_dim] bf16, kcache / vcache [batch, kv_heads, max_seq, head_dim] bf16,
//   out [batch, q_heads, head_dim] bf16; the number of valid keys is len_ptr[0] + len_add (len_ptr may be
//   null); head_dim is 64 or 128; the key range is cut into `splits` pieces that run in parallel.
//
// Limit: batch * q_heads * splits * (head_dim + 2) must not exceed TPB_NOALLOC_SCRATCH_FLOATS, otherwise
// nothing is launched and TPB_ERR_SIZE is returned (use fewer splits, or the regular entry point with a
// workspace of your own).
//
// First call on each device: the library looks up the device address of its workspace with
// cudaGetSymbolAddress while that device is current, and opts the attention kernels in to their dynamic shared
// memory (cudaFuncSetAttribute, once per kernel and device).  Neither one-time step is a stream operation, so make
// the first call on every device you use BEFORE starting any stream capture; later calls only launch kernels.
//
// Sharing: all calls on one device use the same workspace.  Nothing in it has to be zero at entry - every word
// that is read has been written earlier in the same call - so leftovers of the previous call are harmless,
// but two calls that overlap on the GPU (different streams, or a captured graph replayed concurrently) would
// overwrite each other's partial results.  Serialise calls per device (one stream, or events between streams).
int tpb_attn_decode_noalloc(const void* q, const void* kcache, const void* vcache, void* out, const int* len_ptr,
                            int len_add, int batch, int q_heads, int kv_heads, int head_dim, int max_seq, int splits,
                            float scale, void* stream);

#ifdef __cplusplus
}
#endif
