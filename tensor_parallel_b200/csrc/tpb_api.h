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
#define TPB_COMM_MAX_BLOCKS 160  // largest grid of a stand-alone collective = rows of its signal arrays (one CTA per SM and more)
#define TPB_COMM_LL_MAX_WORDS 32768  // 16-byte words (8 payload bytes each) per rank and parity in the flagged-word area

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
  void* mc_slots;                 // NVLink multicast alias of slots[*] (the same offsets reach every rank's workspace): the flagged
                                  // words are then pushed with one multimem.st instead of one store per rank; null: peer stores
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
  void* mc_gathered;                  // multicast (NVLS) view of the gathered buffers, or null: the slice is then pushed with
                                      // one plain store per peer instead of one multimem.st
} tpb_allgather_ctx_t;

// Options of tpb_gemm_bf16_ex.
typedef struct {
  int x_mn, w_mn;            // the operand lies transposed in memory: x as [k, tokens] (row pitch ldx), w as [k, features]
                             // (row pitch ldw).  Needs a plan made with flag bit 0 (tokens on the tensor-core rows).
  int norm_mode;             // 0 none, 1 RMSNorm, 2 LayerNorm of the rows of x, folded into the kernel (<= 64 tokens):
                             // x must be the UNNORMALISED rows, w must already carry the norm weight (w'[f, k] = w[f, k] g[k])
                             // and the result is rstd (x w'^T - mean rowsum) + bias_scale * bias
  float norm_eps;
  const void* norm_x;        // rows the statistics are taken over: x itself, or (norm_k > k) the full rows x is a column
                             // slice of (a row-parallel projection of a normalised state)
  long long norm_ld;
  int norm_k;                // columns of norm_x; <= 0: k
  const float* norm_rowsum;  // LayerNorm: fp32 [features], sum over k of w'[f, k]; the caller folds W beta into the bias
  double wait_seconds;       // bound of the waits for peer GPUs; <= 0: the library default (tpb_set_wait_limit)
  size_t out_elems;          // extent of `out` in elements, for the index checks of a -DTPB_BOUNDS build; 0: derived from the shape
} tpb_gemm_opts_t;

// 1 if this library was built with -DTPB_BOUNDS (kernels check their store indices and report STATUS_BAD_ARG = 3 in the
// status word instead of touching memory outside the extents they were given).
int tpb_bounds_checked(void);

int tpb_gemm_plan(int tokens, int features, int k, int world, int force_splits, int force_kbox,
                  tpb_gemm_plan_t* plan);
int tpb_gemm_plan_ex(int tokens, int features, int k, int world, int force_splits, int force_kbox, int flags,
                     tpb_gemm_plan_t* plan);
int tpb_gemm_tune_split(int min_tile_kb, int target_kb);
int tpb_set_wait_limit(double seconds);

// out[tokens, features] = act(x[tokens, k] @ w[features, k]^T + bias_scale * bias) + residual
// (bf16 operands, fp32 accumulation).  With rc->world > 1 the product is additionally summed over all ranks
// inside the same kernel (every rank must launch it with the same shapes).
int tpb_gemm_bf16(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                  int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                  const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, void* stream);

int tpb_gemm_bf16_ex(const void* x, const void* w, void* out, const void* bias, const void* residual, int tokens,
                     int features, int k, int ldx, int ldw, int ld_out, int act, float bias_scale,
                     const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc, const tpb_gemm_opts_t* opts, void* stream);

int tpb_gemm_allgather_bf16(const void* w, void* out, const void* bias, int tokens, int features, int k, int ld_gathered,
                            int ldw, int ld_out, int act, const tpb_gemm_plan_t* plan, const tpb_reduce_ctx_t* rc,
                            const tpb_allgather_ctx_t* ag, void* stream);

// Measurement aids.  tpb_gemm_debug caps the smem ring depth (0 restores the default).  Skipping the MMAs and the
// kernel-internal %globaltimer trace (tpb_gemm_trace / tpb_gemm_trace_read) exist only in a library built with
// -DTPB_GEMM_TRACE; in the product build they return TPB_ERR_ARG and the kernels carry no trace code.
int tpb_gemm_debug(int stages, int skip_mma);
int tpb_gemm_trace(int block);
int tpb_gemm_disable_flagged_exchange(int disable);
int tpb_gemm_enable_stream_k(int enable);
int tpb_gemm_trace_read(unsigned long long* out32);

#ifdef __cplusplus
}
#endif
