// C ABI of libtpb200: every entry point is extern "C", takes raw device pointers plus a CUDA stream
// handle, launches asynchronously on that stream and returns one of the TPB_* codes below.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TPB_OK = 0,
  TPB_ERR_ARG = 1,        // null pointer / non-positive size / unsupported value
  TPB_ERR_ALIGN = 2,      // pointer or leading dimension violates an alignment rule (TMA needs 16 bytes)
  TPB_ERR_CUDA = 3,       // a CUDA runtime call failed (see cudaGetLastError)
  TPB_ERR_DRIVER = 4,     // a driver entry point is unavailable
  TPB_ERR_TMAP = 5,       // cuTensorMapEncodeTiled rejected the descriptor
  TPB_ERR_WORKSPACE = 6,  // reduction workspace too small for this shape
  TPB_ERR_SIZE = 7,       // size beyond a compiled-in maximum
};

#define TPB_MAX_WORLD 8

typedef struct {
  int swapped;  // 1: weight rows fill the 128 tensor-core rows (few tokens), 0: tokens do
  int bn;       // accumulator columns per tile
  int kbox;     // 64-column k-blocks fetched per pipeline stage (k_blocks / kb_per_split count stages)
  int m_tiles, n_tiles, k_blocks, k_splits, kb_per_split;
  int reduce;   // partial tiles go through the slot workspace (split-K and / or several ranks)
  int grid;
  int tokens_pad;
  int tiles;
  size_t slot_elems;  // fp32 elements one slot must hold
  int stream_k;       // 1: the (tile, k-block) units are dealt out as one contiguous range per CTA; k_splits then is an
                      // upper bound of the CTAs that contribute to one tile
} tpb_gemm_plan_t;

// Workspace of the fused split-K / all-reduce epilogue.  All pointers are device pointers valid on the
// launching GPU; slots[d] / arrivals[d] point into rank d's memory (peer-mapped for d != rank).
typedef struct {
  int world, rank;
  void* slots[TPB_MAX_WORLD];     // fp32 [max_slots][slot_stride]; needs world + k_splits slots
  void* arrivals[TPB_MAX_WORLD];  // uint32 [max_tiles]
  void* expected;                 // local uint32 [max_tiles]
  void* split_counters;           // local uint32 [max_tiles], zero-initialised
  void* status;                   // local uint32 status word
  size_t slot_stride;             // elements per slot
  int max_slots, max_tiles;
  void* ll_epochs;                // local uint32 [max_tiles], zero-initialised: epochs of the flagged-word exchange that small
                                  // cross-rank sums use (needs max_slots >= 32 + 2 * world); null selects arrival counters
} tpb_reduce_ctx_t;

// Operands of the fused all-gather + GEMM (see tpb_gemm_allgather_bf16).
typedef struct {
  int world, rank;
  const void* local;                  // this rank's column slice [tokens, cols_local] bf16
  int local_ld, cols_local;
  void* gathered[TPB_MAX_WORLD];      // every rank's gathered buffer [tokens, world * cols_local] (peer-mapped)
  void* flags[TPB_MAX_WORLD];         // every rank's arrival words, uint32 [world], indexed by source rank
  void* push_counter;                 // local uint32, zero-initialised
  unsigned epoch;                     // number of fused all-gather calls issued on these flags, this one included
} tpb_allgather_ctx_t;

int tpb_gemm_plan(int tokens, int features, int k, int world, int force_splits, int force_kbox,
                  tpb_gemm_plan_t* plan);

// out[tokens, features] = act(x[tokens, k] @ w[features, k]^T + bias_scale * bias) + residual
// (bf16 operands, fp32 accumulation).  With rc->world > 1 the product is additionally summed over all ranks
// inside the same kernel (every rank must launch it with the same shapes).
int tpb_gemm_bf16(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                  int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                  const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, void* stream);

int tpb_gemm_allgather_bf16(const void* w, void* out, const void* bias, int tokens, int features, int k, int ld_gathered,
                            int ldw, int ld_out, int act, const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc,
                            const tpb_allgather_ctx_t* ag, void* stream);

// Measurement aids.  tpb_gemm_debug caps the smem ring depth / skips the MMAs (0, 0 restores the defaults).
// tpb_gemm_trace makes CTA `block` of every following GEMM launch record %globaltimer stamps of its phases
// (block < 0: off); tpb_gemm_trace_read copies the 32 stamps of the current device to the host.
int tpb_gemm_debug(int stages, int skip_mma);
int tpb_gemm_trace(int block);
int tpb_gemm_disable_flagged_exchange(int disable);
int tpb_gemm_enable_stream_k(int enable);
int tpb_gemm_trace_read(unsigned long long* out32);

#ifdef __cplusplus
}
#endif
