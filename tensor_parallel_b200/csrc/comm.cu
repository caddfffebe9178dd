// Symmetric-memory runtime and stand-alone device-side collectives over NVLink peer memory.
//
// Memory model: every rank owns one cudaMalloc'ed "symmetric" region of identical layout; all ranks map
// all regions (cudaDeviceEnablePeerAccess inside one process, CUDA IPC handles across processes), so a
// kernel can load from and store to any peer's region with ordinary global accesses.
//
// Synchronisation: per-(block, rank) 32-bit signal words inside the regions, written by peers with
// st.release.sys and polled with ld.acquire.sys under a wall-clock bound.  Signal values are epochs that
// only grow; each block keeps its own epoch in local device memory, so nothing is reset between calls
// and a captured CUDA graph can be replayed.  Each collective is bracketed by a start barrier ("every
// peer's block b has entered this call", so inputs written by earlier kernels are complete and last
// call's outputs have been consumed) and an end barrier ("every peer's block b has finished its
// pushes / reads"), matched by block index across ranks.
//
// Collectives (bf16 or fp32 payload, fp32 accumulation, fixed summation order -> identical bits on all ranks):
//   all-reduce   flagged   : up to 256 KB; data and flag travel in the same 16-byte word, no barrier and no fence
//                one-shot : every rank reads all peers' inputs and reduces everything locally
//                two-shot : rank r reduces slice r from all peers and pushes it to every rank's output
//   all-gather            : rank r pushes its slice to offset r of every rank's output
//   reduce-scatter        : rank r reduces slice r from all peers into its local output
// With an NVLink multicast (NVLS) view of the heap (symm.cu) the large-message variants let the NVSwitch do the work:
//   all-reduce   two-shot : rank r fetches the switch-reduced slice r (multimem.ld_reduce, fp32 accumulation) and writes it
//                           to every rank's output with one multimem.st: about S bytes per direction per GPU instead of
//                           2 S (N - 1) / N through peer loads and stores
//   all-gather            : one multimem.st per packet instead of N peer stores
//   reduce-scatter        : multimem.ld_reduce of the own slice
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "ptx_sm100.cuh"
#include "tpb_api.h"

namespace tpb {

constexpr int COMM_MAX_BLOCKS = TPB_COMM_MAX_BLOCKS;
constexpr int COMM_THREADS = 512;
constexpr int LL_BLOCKS = 64;                                  // block b always owns words i with (i / COMM_THREADS) % LL_BLOCKS == b
constexpr long long LL_MAX_WORDS = TPB_COMM_LL_MAX_WORDS;      // 8 payload bytes per word

struct CommParams {
  int world, rank;
  const void* in[TPB_MAX_WORLD];   // every rank's input buffer
  void* out[TPB_MAX_WORLD];        // every rank's output buffer
  uint32_t* sig[TPB_MAX_WORLD];    // every rank's signal array: [2][COMM_MAX_BLOCKS][TPB_MAX_WORLD]
  uint32_t* epochs;                // local: [2][COMM_MAX_BLOCKS] (barrier epochs | epochs of the flagged-word all-reduce)
  uint32_t* status;                // local status word
  long long n;                     // elements (all-reduce: total; all-gather / reduce-scatter: per-rank slice)
  uint64_t wait_ns;
  const void* mc_in;               // multicast view of the input buffers (null: no NVLS)
  void* mc_out;                    // multicast view of the output buffers
  uint4* ll[TPB_MAX_WORLD];        // every rank's flagged-word area: [2 parities][world][LL_MAX_WORDS] 16-byte words
};

__device__ __forceinline__ bool block_barrier(const CommParams& p, int phase, uint32_t epoch) {
  // thread r < world: tell peer r that block blockIdx.x of this rank reached `phase`, then wait for peer r
  __shared__ uint32_t ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const int peer = threadIdx.x;
    uint32_t* theirs = p.sig[peer] + (size_t(phase) * COMM_MAX_BLOCKS + blockIdx.x) * TPB_MAX_WORLD + p.rank;
    st_release_sys(theirs, epoch);
    const uint32_t* mine = p.sig[p.rank] + (size_t(phase) * COMM_MAX_BLOCKS + blockIdx.x) * TPB_MAX_WORLD + peer;
    if (!wait_flag_ge(mine, epoch, p.wait_ns)) {
      atomicMax(p.status, STATUS_TIMEOUT_FLAG);
      ok_s = 0;
    }
  }
  __syncthreads();
  return ok_s != 0;
}

template <typename T> struct Pack {};  // 16-byte packets
template <> struct Pack<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { f[2 * i] = __uint_as_float(w[i] << 16); f[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u); }
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]); u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
    return u;
  }
};
template <> struct Pack<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& u, float (&f)[8]) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float (&f)[8]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

__device__ __forceinline__ uint4 ld_peer(const void* base, long long packet) {
  // volatile-style load that must not be served from a stale L1 line
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(static_cast<const uint4*>(base) + packet)
               : "memory");
  return v;
}

// NVLS: one instruction returns the element-wise sum of the 16-byte packet over every rank's copy, reduced inside the
// NVSwitch (bf16 pairs are accumulated in fp32); the store writes the packet to every rank's copy.
template <typename T> __device__ __forceinline__ uint4 multimem_ld_reduce(const void* mc_addr);
template <> __device__ __forceinline__ uint4 multimem_ld_reduce<__nv_bfloat16>(const void* mc_addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 multimem_ld_reduce<float>(const void* mc_addr) {
  float4 f;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w) : "l"(mc_addr) : "memory");
  return make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
}

template <typename T>
__device__ __forceinline__ uint4 reduce_packet(const CommParams& p, long long packet) {
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int r = 0; r < TPB_MAX_WORLD; ++r) {
    if (r < p.world) {
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      Pack<T>::unpack(ld_peer(p.in[r], packet), f);
#pragma unroll
      for (int i = 0; i < Pack<T>::N; ++i) acc[i] += f[i];
    }
  }
  return Pack<T>::pack(acc);
}

// mode: 0 all-reduce one-shot, 1 all-reduce two-shot, 2 all-gather, 3 reduce-scatter; 4, 5, 6 = 1, 2, 3 through the multicast view
template <typename T, int MODE>
__global__ void __launch_bounds__(COMM_THREADS, 3) collective_kernel(const CommParams p) {
  const uint32_t epoch = p.epochs[blockIdx.x] + 1;
  __syncthreads();
  if (threadIdx.x == 0) p.epochs[blockIdx.x] = epoch;
  bool ok = block_barrier(p, 0, epoch);
  constexpr int N = Pack<T>::N;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (ok) {
    if (MODE == 0) {
      const long long packets = p.n / N;
      for (long long i = tid; i < packets; i += stride) static_cast<uint4*>(p.out[p.rank])[i] = reduce_packet<T>(p, i);
    } else if (MODE == 1) {
      const long long packets = p.n / N;
      const long long per = (packets + p.world - 1) / p.world;
      const long long lo = per * p.rank, hi = min(packets, lo + per);
      for (long long i = lo + tid; i < hi; i += stride) {
        const uint4 v = reduce_packet<T>(p, i);
#pragma unroll
        for (int r = 0; r < TPB_MAX_WORLD; ++r)
          if (r < p.world) static_cast<uint4*>(p.out[r])[i] = v;
      }
    } else if (MODE == 2) {
      const long long packets = p.n / N;
      for (long long i = tid; i < packets; i += stride) {
        const uint4 v = static_cast<const uint4*>(p.in[p.rank])[i];
#pragma unroll
        for (int r = 0; r < TPB_MAX_WORLD; ++r)
          if (r < p.world) static_cast<uint4*>(p.out[r])[p.rank * packets + i] = v;
      }
    } else if (MODE == 3) {
      const long long packets = p.n / N;
      for (long long i = tid; i < packets; i += stride)
        static_cast<uint4*>(p.out[p.rank])[i] = reduce_packet<T>(p, p.rank * packets + i);
    } else if (MODE == 4) {
      const long long packets = p.n / N;
      const long long per = (packets + p.world - 1) / p.world;
      const long long lo = per * p.rank, hi = min(packets, lo + per);
      const uint4* src = static_cast<const uint4*>(p.mc_in);
      uint4* dst = static_cast<uint4*>(p.mc_out);
      long long i = lo + tid;
      for (; i + 3 * stride < hi; i += 4 * stride) {  // four reductions in flight per thread
        const uint4 a = multimem_ld_reduce<T>(src + i), b = multimem_ld_reduce<T>(src + i + stride);
        const uint4 c = multimem_ld_reduce<T>(src + i + 2 * stride), d = multimem_ld_reduce<T>(src + i + 3 * stride);
        multimem_st(dst + i, a);
        multimem_st(dst + i + stride, b);
        multimem_st(dst + i + 2 * stride, c);
        multimem_st(dst + i + 3 * stride, d);
      }
      for (; i < hi; i += stride) multimem_st(dst + i, multimem_ld_reduce<T>(src + i));
    } else if (MODE == 5) {
      const long long packets = p.n / N;
      uint4* dst = static_cast<uint4*>(p.mc_out);
      for (long long i = tid; i < packets; i += stride)
        multimem_st(dst + p.rank * packets + i, static_cast<const uint4*>(p.in[p.rank])[i]);
    } else {
      const long long packets = p.n / N;
      const uint4* src = static_cast<const uint4*>(p.mc_in);
      for (long long i = tid; i < packets; i += stride)
        static_cast<uint4*>(p.out[p.rank])[i] = multimem_ld_reduce<T>(src + p.rank * packets + i);
    }
    __threadfence_system();
  }
  block_barrier(p, 1, epoch);
}

// Small all-reduce without barriers or fences: every 8 payload bytes travel as one 16-byte word {lo, epoch, hi, epoch}
// stored to every rank's flagged-word area (st.relaxed.sys.v4: the four fields of a word arrive together), and every rank
// sums the words of all ranks as they turn up, in rank order (identical bits everywhere).  Two parities alternate: a rank
// that writes epoch e + 2 has finished epoch e + 1, for which it needed every peer's words of e + 1, which a peer sends only
// after it has finished reading epoch e.  The input is read locally, so it may lie anywhere.  A word is always owned by
// the same block index, whatever the size of the call, and a block keeps its own epoch (in device memory, so that a
// captured graph can be replayed): a word left behind by an earlier call can never carry the epoch a later one waits for.
// GATHER: the same exchange without the sum - rank r's words land at out[r * words + i] (a small all-gather).
template <typename T, bool GATHER = false>
__global__ void __launch_bounds__(COMM_THREADS) ll_allreduce_kernel(const CommParams p, const uint2* __restrict__ in, uint2* __restrict__ out,
                                                                     long long words) {
  const uint32_t epoch = p.epochs[COMM_MAX_BLOCKS + blockIdx.x] + 1;
  __syncthreads();
  if (threadIdx.x == 0) p.epochs[COMM_MAX_BLOCKS + blockIdx.x] = epoch;
  const long long parity_off = (long long)(epoch & 1) * p.world * LL_MAX_WORDS;
  const long long stride = (long long)LL_BLOCKS * COMM_THREADS;
  for (long long i = blockIdx.x * (long long)COMM_THREADS + threadIdx.x; i < words; i += stride) {
    const uint2 d = in[i];
#pragma unroll
    for (int r = 0; r < TPB_MAX_WORLD; ++r)
      if (r < p.world) st_relaxed_sys_v4(p.ll[r] + parity_off + p.rank * LL_MAX_WORDS + i, d.x, epoch, d.y, epoch);
  }
  const uint4* mine = p.ll[p.rank] + parity_off;
  const uint64_t t0 = globaltimer_ns();
  bool ok = true;
  for (long long i = blockIdx.x * (long long)COMM_THREADS + threadIdx.x; ok && i < words; i += stride) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < TPB_MAX_WORLD; ++r) {
      if (r < p.world && ok) {
        uint4 w = ld_relaxed_sys_v4(mine + r * LL_MAX_WORDS + i);
        uint32_t spins = 0;
        while (w.y != epoch || w.w != epoch) {
          if ((++spins & 63u) == 0 && globaltimer_ns() - t0 > p.wait_ns) {
            atomicMax(p.status, STATUS_TIMEOUT_FLAG);
            ok = false;
            break;
          }
          w = ld_relaxed_sys_v4(mine + r * LL_MAX_WORDS + i);
        }
        if (GATHER) {
          if (ok) out[r * words + i] = make_uint2(w.x, w.z);
        } else if (sizeof(T) == 2) {
          acc[0] += __uint_as_float(w.x << 16); acc[1] += __uint_as_float(w.x & 0xFFFF0000u);
          acc[2] += __uint_as_float(w.z << 16); acc[3] += __uint_as_float(w.z & 0xFFFF0000u);
        } else {
          acc[0] += __uint_as_float(w.x); acc[1] += __uint_as_float(w.z);
        }
      }
    }
    if (ok && !GATHER) out[i] = sizeof(T) == 2 ? make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]))
                                    : make_uint2(__float_as_uint(acc[0]), __float_as_uint(acc[1]));
  }
}

__global__ void wait_flag_test_kernel(const uint32_t* flag, uint32_t target, uint32_t* status, uint64_t wait_ns) {
  if (!wait_flag_ge(flag, target, wait_ns)) atomicMax(status, STATUS_TIMEOUT_FLAG);
}

}  // namespace tpb

using namespace tpb;

extern "C" int tpb_device_count(int* n) { return cudaGetDeviceCount(n) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA; }

extern "C" int tpb_malloc(void** ptr, size_t bytes) {
  if (!ptr) return TPB_ERR_ARG;
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return TPB_ERR_CUDA;
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}
extern "C" int tpb_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA; }

extern "C" int tpb_enable_peer_access(int peer_device) {
  int dev = 0, can = 0;
  cudaGetDevice(&dev);
  if (dev == peer_device) return TPB_OK;
  if (cudaDeviceCanAccessPeer(&can, dev, peer_device) != cudaSuccess || !can) return TPB_ERR_CUDA;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return TPB_OK; }
  return e == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

extern "C" int tpb_ipc_get_handle(void* dev_ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, dev_ptr) != cudaSuccess) return TPB_ERR_CUDA;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return TPB_OK;
}
extern "C" int tpb_ipc_open_handle(const void* handle64, void** out_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}
extern "C" int tpb_ipc_close_handle(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? TPB_OK : TPB_ERR_CUDA; }

extern "C" int tpb_last_cuda_error(char* buf, int len) {
  const char* s = cudaGetErrorString(cudaGetLastError());
  strncpy(buf, s, len - 1);
  buf[len - 1] = 0;
  return TPB_OK;
}

// A CTA can only join an SM whose shared-memory / L1 split suits its kernel, and an SM changes the split only when it is
// idle.  The GEMM and attention kernels run with the largest shared-memory carve-out; the collectives (which bypass L1
// anyway: system-scope and multimem accesses) ask for the same one, so that their CTAs can be resident BESIDE a GEMM's
// instead of waiting for the SMs to drain - which is what lets the prefill pipeline hide an all-reduce under a GEMM.
static int comm_configure() {
  static std::atomic<bool> configured[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TPB_ERR_CUDA;
  if (configured[dev].load(std::memory_order_acquire)) return TPB_OK;
  cudaError_t e = cudaSuccess;
#define CARVE(K) if (e == cudaSuccess) e = cudaFuncSetAttribute(K, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared)
#define CARVE_ALL(T) CARVE((collective_kernel<T, 0>)); CARVE((collective_kernel<T, 1>)); CARVE((collective_kernel<T, 2>)); \
                     CARVE((collective_kernel<T, 3>)); CARVE((collective_kernel<T, 4>)); CARVE((collective_kernel<T, 5>)); \
                     CARVE((collective_kernel<T, 6>)); CARVE((ll_allreduce_kernel<T, false>)); CARVE((ll_allreduce_kernel<T, true>))
  CARVE_ALL(__nv_bfloat16);
  CARVE_ALL(float);
#undef CARVE_ALL
#undef CARVE
  if (e != cudaSuccess) return TPB_ERR_CUDA;
  configured[dev].store(true, std::memory_order_release);
  return TPB_OK;
}

// kind: 0 all-reduce (algorithm chosen by size), 2 all-gather, 3 reduce-scatter.  dtype: 0 bf16, 1 fp32.
// `n` = total elements for all-reduce, per-rank slice elements otherwise.  Buffers must be 16-byte aligned
// and n * sizeof(T) a multiple of 16.
// mc_in / mc_out: multicast views of the input / output buffers (null: plain peer loads and stores).  With them, all-reduces
// above 512 KiB, all-gathers and reduce-scatters go through the NVSwitch (force_algo 4 / 1 picks the two-shot variant by hand).
// block_threads: 0 (512) or 128 / 256: a collective that should run BESIDE another kernel (a GEMM that holds 48 K registers of
// every SM) must fit into what that kernel leaves free; 256 threads of at most 64 registers do.
// ll: every rank's flagged-word area (null: none).  With it, all-reduces of up to 8 * TPB_COMM_LL_MAX_WORDS bytes (force_algo 7:
// by hand) take the barrier-free path; `local_in` (optional) is then read instead of in[rank] and may lie outside the heap.
extern "C" int tpb_collective(int kind, int dtype, int world, int rank, void* const* in, void* const* out,
                              void* const* sig, void* epochs, void* status, long long n, int force_algo,
                              double wait_seconds, const void* mc_in, void* mc_out, void* const* ll, const void* local_in,
                              int block_threads, void* stream_) {
  if (world < 1 || world > TPB_MAX_WORLD || rank < 0 || rank >= world || !in || !out || !sig || !epochs || !status || n <= 0)
    return TPB_ERR_ARG;
  const int per_packet = dtype == 0 ? 8 : 4;
  if (n % per_packet) return TPB_ERR_ALIGN;
  if (comm_configure() != TPB_OK) return TPB_ERR_CUDA;
  CommParams p;
  memset(&p, 0, sizeof(p));
  p.world = world;
  p.rank = rank;
  for (int r = 0; r < world; ++r) { p.in[r] = in[r]; p.out[r] = out[r]; p.sig[r] = static_cast<uint32_t*>(sig[r]); }
  p.epochs = static_cast<uint32_t*>(epochs);
  p.status = static_cast<uint32_t*>(status);
  p.n = n;
  p.wait_ns = wait_seconds > 0 ? uint64_t(wait_seconds * 1e9) : TPB_WAIT_LIMIT_NS;
  const bool nvls = mc_in && mc_out && world > 1;
  p.mc_in = nvls ? mc_in : nullptr;
  p.mc_out = nvls ? mc_out : nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream_);
  const long long bytes = n * (dtype == 0 ? 2 : 4);
  int mode = kind;
  // through the switch from 4 ranks on: at 2 ranks the peer two-shot moves the same bytes with less latency
  // (128 MiB: 234 us against 377 us with multimem, NCCL 280 us; measured on B200)
  const bool nvls_auto = nvls && world >= 4;
  const bool ll_ok = ll && world > 1 && bytes <= 8 * LL_MAX_WORDS;
  if (kind == 0) mode = force_algo >= 0 ? force_algo : (ll_ok ? 7 : (bytes <= 512 * 1024 ? 0 : (nvls_auto ? 4 : 1)));
  if (kind == 2 && ll_ok && (force_algo < 0 || force_algo == 8)) mode = 8;  // small all-gather: the same words, not summed
  if (mode == 8) {
    if (kind != 2 || !ll_ok) return TPB_ERR_ARG;
    for (int r = 0; r < world; ++r) p.ll[r] = static_cast<uint4*>(ll[r]);
    const long long words = bytes / 8;
    const int ll_blocks = int(words + COMM_THREADS - 1) / COMM_THREADS > LL_BLOCKS ? LL_BLOCKS : int((words + COMM_THREADS - 1) / COMM_THREADS);
    const uint2* src = static_cast<const uint2*>(local_in ? local_in : in[rank]);
    if (reinterpret_cast<uintptr_t>(src) & 7) return TPB_ERR_ALIGN;
    ll_allreduce_kernel<float, true><<<ll_blocks, COMM_THREADS, 0, s>>>(p, src, static_cast<uint2*>(out[rank]), words);  // (bytes are bytes)
    return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
  }
  if (mode == 7) {
    if (kind != 0 || !ll_ok) return TPB_ERR_ARG;
    for (int r = 0; r < world; ++r) p.ll[r] = static_cast<uint4*>(ll[r]);
    const long long words = bytes / 8;
    const int ll_blocks = int(words + COMM_THREADS - 1) / COMM_THREADS > LL_BLOCKS ? LL_BLOCKS : int((words + COMM_THREADS - 1) / COMM_THREADS);
    const uint2* src = static_cast<const uint2*>(local_in ? local_in : in[rank]);
    if (reinterpret_cast<uintptr_t>(src) & 7) return TPB_ERR_ALIGN;
    if (dtype == 0)
      ll_allreduce_kernel<__nv_bfloat16><<<ll_blocks, COMM_THREADS, 0, s>>>(p, src, static_cast<uint2*>(out[rank]), words);
    else
      ll_allreduce_kernel<float><<<ll_blocks, COMM_THREADS, 0, s>>>(p, src, static_cast<uint2*>(out[rank]), words);
    return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
  }
  if (kind == 2 && nvls_auto && force_algo != 2) mode = 5;  // (a small one takes the flagged-word path below instead)
  if (kind == 3 && nvls_auto && force_algo != 3) mode = 6;
  if (mode >= 4 && !nvls) return TPB_ERR_ARG;
  const long long packets = n / per_packet;
  long long work = (mode == 1 || mode == 4) ? (packets + world - 1) / world : packets;
  const int threads = (block_threads == 128 || block_threads == 256) ? block_threads : COMM_THREADS;
  int blocks = int((work + threads - 1) / threads);
  if (blocks < 1) blocks = 1;
  if (blocks > COMM_MAX_BLOCKS) blocks = COMM_MAX_BLOCKS;
#define RUN(T, M) collective_kernel<T, M><<<blocks, threads, 0, s>>>(p)
  if (dtype == 0) {
    switch (mode) { case 0: RUN(__nv_bfloat16, 0); break; case 1: RUN(__nv_bfloat16, 1); break;
                    case 2: RUN(__nv_bfloat16, 2); break; case 3: RUN(__nv_bfloat16, 3); break;
                    case 4: RUN(__nv_bfloat16, 4); break; case 5: RUN(__nv_bfloat16, 5); break;
                    case 6: RUN(__nv_bfloat16, 6); break; default: return TPB_ERR_ARG; }
  } else {
    switch (mode) { case 0: RUN(float, 0); break; case 1: RUN(float, 1); break;
                    case 2: RUN(float, 2); break; case 3: RUN(float, 3); break;
                    case 4: RUN(float, 4); break; case 5: RUN(float, 5); break;
                    case 6: RUN(float, 6); break; default: return TPB_ERR_ARG; }
  }
#undef RUN
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Loads every collective kernel on the current device.  With lazy module loading the first launch of a kernel may
// have to synchronise the device; a host thread that drives several GPUs must not meet that behind a kernel that is
// waiting for a peer the same thread has yet to launch.
extern "C" int tpb_comm_preload(void) {
  cudaFuncAttributes attr;
  cudaError_t e = cudaSuccess;
#define LOAD(T, M) if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, collective_kernel<T, M>)
  LOAD(__nv_bfloat16, 0); LOAD(__nv_bfloat16, 1); LOAD(__nv_bfloat16, 2); LOAD(__nv_bfloat16, 3);
  LOAD(__nv_bfloat16, 4); LOAD(__nv_bfloat16, 5); LOAD(__nv_bfloat16, 6);
  LOAD(float, 0); LOAD(float, 1); LOAD(float, 2); LOAD(float, 3); LOAD(float, 4); LOAD(float, 5); LOAD(float, 6);
#undef LOAD
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, ll_allreduce_kernel<__nv_bfloat16>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, ll_allreduce_kernel<float>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&attr, ll_allreduce_kernel<float, true>);
  return e == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}

// Launches a one-thread kernel that waits (bounded by wait_seconds) for *flag >= target and records a
// timeout in *status.  Used to exercise the give-up path: the kernel always terminates.
extern "C" int tpb_wait_flag_test(const void* flag, unsigned target, void* status, double wait_seconds, void* stream_) {
  if (!flag || !status) return TPB_ERR_ARG;
  wait_flag_test_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream_)>>>(static_cast<const uint32_t*>(flag), target,
                                                                        static_cast<uint32_t*>(status), uint64_t(wait_seconds * 1e9));
  return cudaGetLastError() == cudaSuccess ? TPB_OK : TPB_ERR_CUDA;
}
