"""Symmetric heap and device-side collectives (Python side of ``csrc/comm.cu`` and ``csrc/symm.cu``).

Every rank owns one region of identical layout that all ranks map.  Preferred form: a physical allocation
from the virtual-memory-management API, shared between rank processes as a POSIX file descriptor (passed over a
Unix-domain socket) or simply by handle inside one process, mapped by every rank for plain peer loads / stores
AND bound into one NVLink multicast object, so that kernels can also issue ``multimem`` instructions that the
NVSwitch executes on all ranks' copies at once (``RankComm.mc_base``).  Fallback when the driver offers
neither: ``cudaMalloc`` + ``cudaDeviceEnablePeerAccess`` (one process) or CUDA IPC handles (one process per
GPU).  ``TPB_VMM=0`` forces the fallback, ``TPB_NVLS=0`` keeps the VMM heap but creates no multicast view.
Kernels address peers' regions directly over NVLink; no NCCL call is on these paths.

Layout of a region (offsets identical on all ranks)::

    signals   : uint32 [2][160][8]           start / end barrier words of the collectives
    arrivals  : uint32 [2 regions][MAX_TILES] per-tile arrival counters of the fused GEMM epilogue
    slots     : fp32   [2 regions][max_slots][slot_stride]  partial tiles pushed by peers
    staging   : two payload buffers for the stand-alone collectives (input side / output side)

The two "regions" alternate between consecutive fused GEMM calls: a rank that runs ahead writes
into the other half than the one a slower peer may still be reducing from.
"""
from __future__ import annotations

import atexit
import ctypes
import math
import logging
import os
import socket
import threading
import uuid
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from tensor_parallel_b200.ops import native
from tensor_parallel_b200.utils.tracing import traced
from tensor_parallel_b200.ops.native import LIB, ReduceCtx, c_int, c_ll, c_void_p, check

logger = logging.getLogger(__name__)

MAX_WORLD = 8
COMM_MAX_BLOCKS = 160  # = TPB_COMM_MAX_BLOCKS of csrc/tpb_api.h
SIGNAL_BYTES = 2 * COMM_MAX_BLOCKS * MAX_WORLD * 4
MAX_TILES = native.MAX_TILES
LL_MAX_WORDS = 32768  # = TPB_COMM_LL_MAX_WORDS of csrc/tpb_api.h: 16-byte words per rank and parity of the barrier-free all-reduce
LL_AREA_BYTES = 2 * MAX_WORLD * LL_MAX_WORDS * 16

LIB.tpb_malloc.argtypes = [ctypes.POINTER(c_void_p), ctypes.c_size_t]
LIB.tpb_free.argtypes = [c_void_p]
LIB.tpb_enable_peer_access.argtypes = [c_int]
LIB.tpb_ipc_get_handle.argtypes = [c_void_p, c_void_p]
LIB.tpb_ipc_open_handle.argtypes = [c_void_p, ctypes.POINTER(c_void_p)]
LIB.tpb_ipc_close_handle.argtypes = [c_void_p]
LIB.tpb_collective.argtypes = [c_int, c_int, c_int, c_int, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                               ctypes.POINTER(c_void_p), c_void_p, c_void_p, c_ll, c_int, ctypes.c_double, c_void_p, c_void_p,
                               ctypes.POINTER(c_void_p), c_void_p, c_int, c_void_p]
_ull, _size_t = ctypes.c_ulonglong, ctypes.c_size_t
LIB.tpb_symm_support.argtypes = [c_int, ctypes.POINTER(c_int), ctypes.POINTER(c_int)]
LIB.tpb_symm_round_size.argtypes = [c_int, c_int, _size_t, ctypes.POINTER(_size_t)]
LIB.tpb_symm_create.argtypes = [c_int, _size_t, ctypes.POINTER(_ull), ctypes.POINTER(c_int)]
LIB.tpb_symm_import.argtypes = [c_int, ctypes.POINTER(_ull)]
LIB.tpb_symm_map.argtypes = [_ull, _size_t, ctypes.POINTER(c_int), c_int, ctypes.POINTER(c_void_p)]
LIB.tpb_symm_unmap.argtypes = [c_void_p, _size_t]
LIB.tpb_symm_release.argtypes = [_ull]
LIB.tpb_mc_create.argtypes = [c_int, _size_t, ctypes.POINTER(_ull), ctypes.POINTER(c_int)]
LIB.tpb_mc_add_device.argtypes = [_ull, c_int]
LIB.tpb_mc_bind.argtypes = [_ull, _ull, _size_t]
LIB.tpb_mc_unbind.argtypes = [_ull, c_int, _size_t]


class AllGatherCtx(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("local", c_void_p), ("local_ld", c_int), ("cols_local", c_int),
                ("gathered", c_void_p * 8), ("flags", c_void_p * 8), ("push_counter", c_void_p), ("epoch", ctypes.c_uint),
                ("mc_gathered", c_void_p)]


LIB.tpb_gemm_allgather_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                        ctypes.POINTER(native.GemmPlan), ctypes.POINTER(ReduceCtx), ctypes.POINTER(AllGatherCtx), c_void_p]
LIB.tpb_wait_flag_test.argtypes = [c_void_p, ctypes.c_uint, c_void_p, ctypes.c_double, c_void_p]


class _DeviceBlob:
    """Exposes raw device memory to ``torch.as_tensor`` (zero-copy) via the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    with torch.cuda.device(device):
        return torch.as_tensor(_DeviceBlob(ptr, nbytes), device=device)


def _align(n: int, a: int = 1024) -> int:
    return (n + a - 1) // a * a


GUARD_BYTES = 4096   # (a multiple of the 1024-byte area alignment)
GUARD_PATTERN = 0xA5


class HeapLayout:
    def __init__(self, slot_stride: int, max_slots: int, staging_bytes: int, gather_bytes: int = 96 << 20):
        self.slot_stride, self.max_slots, self.staging_bytes = slot_stride, max_slots, staging_bytes
        self.gather_bytes = gather_bytes
        self.off_signals = 0
        self.off_ag_flags = SIGNAL_BYTES  # uint32 [2 regions][MAX_WORLD] arrival words of the fused all-gather
        self.off_arrivals = _align(SIGNAL_BYTES + 2 * MAX_WORLD * 4)
        # every area below is followed by a guard band holding a fixed byte pattern; a kernel that writes past the end
        # of its area (on this GPU or through a peer mapping) shows up in RankComm.check_guards()
        g = GUARD_BYTES
        self.off_slots = self.off_arrivals + _align(2 * MAX_TILES * 4) + g
        self.region_slot_bytes = _align(max_slots * slot_stride * 4)
        self.off_staging_in = self.off_slots + 2 * self.region_slot_bytes + g
        self.off_staging_out = self.off_staging_in + _align(staging_bytes) + g
        self.off_gather = self.off_staging_out + _align(staging_bytes) + g  # two gathered-operand buffers
        self.off_ll = self.off_gather + 2 * _align(gather_bytes) + g        # flagged words of the small all-reduce
        self.total = self.off_ll + LL_AREA_BYTES + g
        self.guards = [self.off_slots - g, self.off_staging_in - g, self.off_staging_out - g, self.off_gather - g, self.off_ll - g, self.total - g]


class RankComm:
    """One rank's view of the symmetric heap: its own region plus peer-mapped pointers."""

    def __init__(self, world: int, rank: int, device: torch.device, layout: HeapLayout, base_ptrs: Sequence[int],
                 mc_base: int = 0, heap=None):
        self.world, self.rank, self.device, self.layout = world, rank, device, layout
        self.base = list(base_ptrs)
        self.mc_base = mc_base  # multicast (NVLS) view of all ranks' regions, same offsets; 0: none
        self.heap = heap        # owner of the mappings (None: cudaMalloc'ed region, freed with the process)
        with torch.cuda.device(device):
            self.epochs = torch.zeros(2 * COMM_MAX_BLOCKS, dtype=torch.int32, device=device)  # barrier epochs | flagged-word epochs
            self.expected = torch.zeros(2 * MAX_TILES, dtype=torch.int32, device=device)
            self.split_counters = torch.zeros(2 * MAX_TILES, dtype=torch.int32, device=device)
            self.ll_epochs = torch.zeros(2 * MAX_TILES, dtype=torch.int32, device=device)
            self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.local = tensor_from_ptr(self.base[rank], layout.total, device)
        self.staging_in = self.local[layout.off_staging_in : layout.off_staging_in + layout.staging_bytes]
        self.staging_out = self.local[layout.off_staging_out : layout.off_staging_out + layout.staging_bytes]
        for off in layout.guards:
            self.local[off : off + GUARD_BYTES].fill_(GUARD_PATTERN)
        self._call = 0
        self._ctxs = [self._make_ctx(0), self._make_ctx(1)]
        self._ptr_arrays: Dict = {}
        self._views: Dict = {}
        self._c_epochs, self._c_status = c_void_p(self.epochs.data_ptr()), c_void_p(self.status.data_ptr())
        for name, off in (("in", layout.off_staging_in), ("out", layout.off_staging_out), ("sig", layout.off_signals), ("ll", layout.off_ll)):
            arr = (c_void_p * MAX_WORLD)()
            for r in range(world):
                arr[r] = self.base[r] + off
            self._ptr_arrays[name] = arr
        self.wait_seconds = native.device_wait_seconds()
        self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._status_event: Optional[torch.cuda.Event] = None
        with torch.cuda.device(device):
            self.ag_push_counter = torch.zeros(4, dtype=torch.int32, device=device)
        self._ag_calls = [0, 0]

    def _make_ctx(self, region: int) -> ReduceCtx:
        ctx = ReduceCtx()
        ctx.world, ctx.rank = self.world, self.rank
        for r in range(self.world):
            ctx.slots[r] = self.base[r] + self.layout.off_slots + region * self.layout.region_slot_bytes
            ctx.arrivals[r] = self.base[r] + self.layout.off_arrivals + region * MAX_TILES * 4
        ctx.expected = self.expected.data_ptr() + region * MAX_TILES * 4
        ctx.split_counters = self.split_counters.data_ptr() + region * MAX_TILES * 4
        ctx.status = self.status.data_ptr()
        ctx.ll_epochs = self.ll_epochs.data_ptr() + region * MAX_TILES * 4
        # TPB_FUSED_MULTICAST=1: the flagged words of the fused GEMM + all-reduce go out through the multicast mapping (one
        # multimem.st instead of one store per rank).  Off by default: at 4 ranks it measured slower than the peer stores
        # (o_proj 13.8 vs 13.0 us, down_proj 18.3 vs 17.6 us, replayed from a CUDA graph); not measured at 8 ranks.
        if self.mc_base and self.world >= 4 and os.environ.get("TPB_FUSED_MULTICAST", "0") == "1":
            ctx.mc_slots = self.mc_base + self.layout.off_slots + region * self.layout.region_slot_bytes
        ctx.slot_stride = self.layout.slot_stride
        ctx.max_slots, ctx.max_tiles = self.layout.max_slots, MAX_TILES
        return ctx

    # -- fused GEMM + all-reduce ------------------------------------------------------------------

    def next_reduce_ctx(self) -> ReduceCtx:
        """Context for the next fused call; consecutive calls alternate workspace halves.  Every rank
        must issue the same sequence of fused calls."""
        ctx = self._ctxs[self._call & 1]
        self._call += 1
        return ctx

    @traced("tpb.gemm_allreduce")
    def gemm_allreduce(self, x2d, weight, bias=None, residual=None, out=None, bias_scale: float = 1.0):
        """``sum over ranks of (x2d @ weight.T) + bias_scale * bias + residual`` in ONE kernel: partial tiles are
        pushed to every peer from the GEMM epilogue and reduced as they arrive."""
        tokens, features = x2d.shape[0], weight.shape[0]
        if tokens * features > self.layout.slot_stride:
            raise ValueError(f"fused GEMM+all-reduce workspace holds {self.layout.slot_stride} elements per slot, need {tokens * features}")
        return native.gemm_nt(x2d, weight, bias=bias, residual=residual, out=out, reduce_ctx=self.next_reduce_ctx(),
                              world=self.world, bias_scale=bias_scale)

    def fits_fused(self, tokens: int, features: int, k: int) -> bool:
        if tokens * features > self.layout.slot_stride:
            return False
        plan = native.gemm_plan(tokens, features, k, self.world)
        return self.world + plan.k_splits <= self.layout.max_slots and plan.tiles <= MAX_TILES

    # -- fused all-gather + GEMM ------------------------------------------------------------------

    @traced("tpb.allgather_gemm")
    def allgather_gemm(self, x_local: torch.Tensor, weight: torch.Tensor, bias=None, act=None, out=None, force_peer_stores: bool = False):
        """``concat_over_ranks(x_local, dim=1) @ weight.T`` in ONE kernel: every rank pushes its column slice
        ``x_local [tokens, k / world]`` into all peers' gathered buffers from the kernel's prologue, and the GEMM
        main loop consumes the k-blocks of a slice as soon as that slice has arrived (own slice first), so the
        transfer overlaps the tensor-core work.  All ranks must call with the same shapes, in the same order."""
        tokens, cols = x_local.shape
        features, k = weight.shape
        if k != cols * self.world or x_local.dtype != torch.bfloat16:
            raise ValueError("weight.shape[1] must equal world * x_local.shape[1] (bf16 operands)")
        if tokens * k * 2 > self.layout.gather_bytes:
            raise ValueError(f"gathered operand of {tokens * k * 2} bytes exceeds the heap's gather buffers")
        x_local = native._tma_ready(x_local)
        weight = native._tma_ready(weight)
        kbox = 4 if (tokens <= 32 and cols % 256 == 0) else (2 if (tokens <= 32 and cols % 128 == 0) else 1)
        if cols % (64 * kbox):
            raise ValueError("the per-rank column count must be a multiple of 64")
        plan = native.gemm_plan(tokens, features, k, 1, 1, kbox)
        region = (self._ag_calls[0] + self._ag_calls[1]) & 1
        self._ag_calls[region] += 1
        ctx = AllGatherCtx()
        ctx.world, ctx.rank = self.world, self.rank
        ctx.local, ctx.local_ld, ctx.cols_local = x_local.data_ptr(), x_local.stride(0), cols
        for r in range(self.world):
            ctx.gathered[r] = self.base[r] + self.layout.off_gather + region * _align(self.layout.gather_bytes)
            ctx.flags[r] = self.base[r] + self.layout.off_ag_flags + region * MAX_WORLD * 4
        ctx.push_counter = self.ag_push_counter.data_ptr()
        ctx.epoch = self._ag_calls[region]
        if self.mc_base and self.world >= 4 and not force_peer_stores:  # (2 ranks: a peer store moves the same bytes)
            ctx.mc_gathered = self.mc_base + self.layout.off_gather + region * _align(self.layout.gather_bytes)
        if out is None:
            out = torch.empty(tokens, features, dtype=torch.bfloat16, device=x_local.device)
        rctx = self._ctxs[0]
        check(LIB.tpb_gemm_allgather_bf16(c_void_p(weight.data_ptr()), c_void_p(out.data_ptr()),
                                          c_void_p(bias.data_ptr() if bias is not None else 0), tokens, features, k, k,
                                          weight.stride(0), out.stride(0), native.ACT_CODES[act], ctypes.byref(plan),
                                          ctypes.byref(rctx), ctypes.byref(ctx), native._stream()), "tpb_gemm_allgather_bf16")
        native.launch_count += 1
        return out

    # -- stand-alone collectives on the staging buffers -------------------------------------------

    def _collective(self, kind: int, dtype: torch.dtype, n: int, force_algo: int = -1, offset: int = 0, local_in: int = 0,
                    block_threads: int = 0):
        """``offset`` (bytes, the same on every rank) moves the operation to a later part of the staging buffers;
        ``local_in``: address the barrier-free small all-reduce reads its input from instead of the staging buffer."""
        code = 0 if dtype == torch.bfloat16 else 1
        mc_in = self.mc_base + self.layout.off_staging_in + offset if self.mc_base else 0
        mc_out = self.mc_base + self.layout.off_staging_out + offset if self.mc_base else 0
        ins, outs = self._ptr_arrays["in"], self._ptr_arrays["out"]
        if offset:
            key = ("off", offset)
            if key not in self._ptr_arrays:
                pair = ((c_void_p * MAX_WORLD)(), (c_void_p * MAX_WORLD)())
                for r in range(self.world):
                    pair[0][r] = self.base[r] + self.layout.off_staging_in + offset
                    pair[1][r] = self.base[r] + self.layout.off_staging_out + offset
                self._ptr_arrays[key] = pair
            ins, outs = self._ptr_arrays[key]
        check(LIB.tpb_collective(kind, code, self.world, self.rank, ins, outs,
                                 self._ptr_arrays["sig"], self._c_epochs, self._c_status, n,
                                 force_algo, self.wait_seconds, mc_in, mc_out, self._ptr_arrays["ll"], local_in,
                                 block_threads, native._stream()), "tpb_collective")
        native.launch_count += 1

    def all_reduce_staged(self, offset: int, shape, dtype=torch.bfloat16, block_threads: int = 0) -> torch.Tensor:
        """Sum over ranks of the tensor that already lies in the staging-in buffer at byte ``offset`` (a multiple of
        1024, the same on every rank); returns the view of the staging-out buffer that holds the result.  Launches on
        the current stream: callers that overlap the reduction with other work (``engine.py``: prefill) call it under a
        side stream, one collective at a time and in the same order on every rank; ``block_threads=256`` keeps the
        kernel's CTAs small enough to be resident beside the CTAs of a GEMM."""
        n = int(torch.Size(shape).numel())
        size = 2 if dtype == torch.bfloat16 else 4
        if offset % 1024 or (n * size) % 16 or offset + n * size > self.staging_in.numel():
            raise ValueError("staged all-reduce: misaligned or outside the staging buffers")
        self._collective(0, dtype, n, offset=offset, block_threads=block_threads)
        return self.staging_out[offset : offset + n * size].view(dtype).view(shape)

    def _capacity(self, dtype: torch.dtype, in_copies: int, out_copies: int) -> int:
        """Largest element count (a multiple of 16 bytes) whose ``in_copies`` / ``out_copies`` fit the staging buffers."""
        size = 2 if dtype == torch.bfloat16 else 4
        per = 16 // size
        return min(self.staging_in.numel() // (size * in_copies), self.staging_out.numel() // (size * out_copies)) // per * per

    def staging_view(self, which: str, shape, dtype) -> torch.Tensor:
        buf = self.staging_in if which == "in" else self.staging_out
        key = (which, buf.data_ptr(), buf.numel(), tuple(shape), dtype)
        view = self._views.get(key)  # (a collective of a few microseconds should not spend more than that on view objects)
        if view is None:
            nbytes = math.prod(shape) * (2 if dtype == torch.bfloat16 else torch.empty((), dtype=dtype).element_size())
            if nbytes > buf.numel():
                raise ValueError(f"collective payload of {nbytes} bytes exceeds the staging buffer ({buf.numel()} bytes)")
            if len(self._views) > 256:
                self._views.clear()
            view = self._views[key] = buf[:nbytes].view(dtype).view(tuple(shape))
        return view

    @traced("tpb.all_reduce")
    def all_reduce(self, x: torch.Tensor, force_algo: int = -1) -> torch.Tensor:
        """Sum over ranks.  ``x`` is copied into symmetric memory unless it already is the staging-in view."""
        dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.float32
        n = x.numel()
        per = 8 if dtype == torch.bfloat16 else 4
        n_pad = (n + per - 1) // per * per
        cap = self._capacity(dtype, 1, 1)
        if n_pad > cap:  # larger than the staging buffers: one collective per staging-sized piece
            flat, out = x.reshape(-1), torch.empty(n, dtype=dtype, device=x.device)
            for s in range(0, n, cap):
                out[s : s + cap].copy_(self.all_reduce(flat[s : s + cap], force_algo))
            return out.view(x.shape)
        size = 2 if dtype == torch.bfloat16 else 4
        if (force_algo in (-1, 7) and self.world > 1 and n_pad * size <= 8 * LL_MAX_WORDS and n_pad == n and x.dtype == dtype
                and x.is_contiguous() and x.data_ptr() % 8 == 0):
            # small: the barrier-free kernel reads its input where it lies (no copy into the heap)
            self._collective(0, dtype, n_pad, force_algo, local_in=x.data_ptr())
            return self.staging_view("out", x.shape, dtype)
        src = self.staging_view("in", (n_pad,), dtype)
        if x.data_ptr() != src.data_ptr():
            src[:n].copy_(x.reshape(-1))
            if n_pad != n:
                src[n:].zero_()
        self._collective(0, dtype, n_pad, force_algo)
        return self.staging_view("out", (n_pad,), dtype)[:n].view(x.shape)

    @traced("tpb.all_gather")
    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """Returns ``[world, *x.shape]`` (every rank's ``x``); all ranks must pass the same shape."""
        dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.float32
        n = x.numel()
        per = 8 if dtype == torch.bfloat16 else 4
        n_pad = (n + per - 1) // per * per
        cap = self._capacity(dtype, 1, self.world)
        if n_pad > cap:
            flat, out = x.reshape(-1), torch.empty(self.world, n, dtype=dtype, device=x.device)
            for s in range(0, n, cap):
                out[:, s : s + cap].copy_(self.all_gather(flat[s : s + cap]))
            return out.view(self.world, *x.shape)
        size = 2 if dtype == torch.bfloat16 else 4
        if (self.world > 1 and n_pad * size <= 8 * LL_MAX_WORDS and n_pad == n and x.dtype == dtype and x.is_contiguous()
                and x.data_ptr() % 8 == 0):
            # small: the barrier-free kernel reads the slice where it lies and every rank stores it beside the others'
            self._collective(2, dtype, n_pad, local_in=x.data_ptr())
            return self.staging_view("out", (self.world, *x.shape), dtype)
        src = self.staging_view("in", (n_pad,), dtype)
        if x.data_ptr() != src.data_ptr():
            src[:n].copy_(x.reshape(-1))
        self._collective(2, dtype, n_pad)
        return self.staging_view("out", (self.world, n_pad), dtype)[:, :n].reshape(self.world, *x.shape)

    @traced("tpb.reduce_scatter")
    def reduce_scatter(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` is ``[world, ...]``; returns the sum over ranks of ``x[rank]``."""
        dtype = x.dtype if x.dtype in (torch.bfloat16, torch.float32) else torch.float32
        per = 8 if dtype == torch.bfloat16 else 4
        n = x[0].numel()
        if n % per:
            raise ValueError("reduce_scatter slices must be a multiple of 16 bytes")
        cap = self._capacity(dtype, self.world, 1)
        if n > cap:
            flat, out = x.reshape(self.world, n), torch.empty(n, dtype=dtype, device=x.device)
            for s in range(0, n, cap):
                out[s : s + cap].copy_(self.reduce_scatter(flat[:, s : s + cap].contiguous()))
            return out.view(x.shape[1:])
        src = self.staging_view("in", (self.world * n,), dtype)
        if x.data_ptr() != src.data_ptr():
            src.copy_(x.reshape(-1))
        self._collective(3, dtype, n)
        return self.staging_view("out", (n,), dtype).view(x.shape[1:])

    def check_guards(self):
        """Raises if any guard band of this rank's heap region has been written to (synchronises the device)."""
        for i, off in enumerate(self.layout.guards):
            band = self.local[off : off + GUARD_BYTES]
            if not bool((band == GUARD_PATTERN).all().item()):
                raise RuntimeError(f"guard band {i} of rank {self.rank}'s symmetric heap was overwritten")

    def _raise(self, code: int):
        self.status.zero_()
        from tensor_parallel_b200.parallel.collectives import TPCollectiveError

        what = {1: "an mbarrier wait", 2: "a wait for a peer GPU"}.get(code, f"status {code}")
        raise TPCollectiveError(f"{what} timed out inside a kernel on rank {self.rank}: the collective did not complete and "
                                "its result must not be used (a peer is late by more than the device wait limit, or gone)")

    def check_status(self):
        """Raises if a kernel of this rank gave up on a wait.  Synchronises the device."""
        code = int(self.status[0].item())
        if code:
            self._raise(code)

    def poll_status(self):
        """Non-blocking form for hot loops: reads the host copy of the status word that the previous call queued behind
        the kernels then in flight, raises if it is set, and queues the next copy.  A timeout therefore surfaces one call
        late at the latest, without the host ever waiting for the GPU."""
        if self._status_event is not None and self._status_event.query():
            code = int(self._status_host[0])
            self._status_event = None
            if code:
                self._raise(code)
        if self._status_event is None:
            with torch.cuda.device(self.device):
                self._status_host.copy_(self.status, non_blocking=True)
                self._status_event = torch.cuda.Event()
                self._status_event.record()

    def close(self):
        """Unmaps this rank's views of the heap (multicast first).  Every rank calls it before any rank exits."""
        if self.heap is not None:
            self.heap.close()
            self.heap = None
            self.mc_base = 0


def _alloc_region(device: torch.device, nbytes: int) -> int:
    ptr = c_void_p()
    with torch.cuda.device(device):
        check(LIB.tpb_malloc(ctypes.byref(ptr), nbytes), "tpb_malloc")
    return ptr.value


DEFAULT_SLOT_STRIDE = 64 * 16384       # fp32 elements per partial slot: 64 tokens x 16384 features
DEFAULT_STAGING = 288 * 1024 * 1024    # bytes per staging buffer (16384 x 8192 bf16 fits)


class VmmHeap:
    """One rank's (or, inside one process, all ranks') mappings of a VMM symmetric heap; see ``csrc/symm.cu``."""

    _open: List["VmmHeap"] = []

    def __init__(self, size: int):
        VmmHeap._open.append(self)
        self.size = size
        self.handles: List[int] = []      # allocation handles held by this process (own and imported)
        self.mappings: List[int] = []     # unicast virtual addresses
        self.mc_handle = 0
        self.mc_ptr = 0
        self.bound: List[int] = []        # device indices whose memory this process bound to the multicast object
        self._closed = False
        atexit.register(self.close)

    def close(self):
        if self._closed:
            return
        self._closed = True
        try:
            torch.cuda.synchronize()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass
        if self.mc_ptr:
            LIB.tpb_symm_unmap(c_void_p(self.mc_ptr), self.size)
        for dev in self.bound:
            LIB.tpb_mc_unbind(self.mc_handle, dev, self.size)
        if self.mc_handle:
            LIB.tpb_symm_release(self.mc_handle)
        for ptr in self.mappings:
            LIB.tpb_symm_unmap(c_void_p(ptr), self.size)
        for handle in self.handles:
            LIB.tpb_symm_release(handle)
        self.mc_ptr = self.mc_handle = 0
        self.mappings, self.handles, self.bound = [], [], []


def close_all_heaps():
    """Tears down every VMM heap of this process (multicast views first).  For an orderly exit of a multi-rank job:
    every rank stops launching, the ranks meet at a barrier, every rank calls this, and only then do they exit."""
    for heap in list(VmmHeap._open):
        heap.close()
    VmmHeap._open.clear()
    _process_backends.clear()
    _thread_backends.clear()


def _vmm_wanted() -> bool:
    return os.environ.get("TPB_VMM", "1") != "0"


def _nvls_wanted() -> bool:
    return os.environ.get("TPB_NVLS", "1") != "0"


def _symm_support(device: torch.device):
    vmm, mc = c_int(0), c_int(0)
    with torch.cuda.device(device):
        if LIB.tpb_symm_support(device.index, ctypes.byref(vmm), ctypes.byref(mc)) != 0:
            return False, False
    return bool(vmm.value), bool(mc.value)


def _map(handle: int, size: int, devices: Sequence[int]) -> int:
    arr = (c_int * len(devices))(*devices)
    ptr = c_void_p()
    check(LIB.tpb_symm_map(handle, size, arr, len(devices), ctypes.byref(ptr)), "tpb_symm_map")
    return ptr.value


def _exchange_fds(fd: Optional[int], rank: int, world: int, process_group, only_from: Optional[int] = None) -> List[Optional[int]]:
    """Every rank hands its descriptor ``fd`` to every other rank (``only_from``: just that rank sends) over Unix-domain
    sockets in the abstract namespace; returns the received descriptors by source rank (own slot: ``fd``)."""
    name = f"\0tpb-{uuid.uuid4().hex}-{rank}"
    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(name)
    server.listen(world)
    names: List[Optional[str]] = [None] * world
    dist.all_gather_object(names, name, group=process_group)  # also orders "everyone listens" before the first connect
    senders = range(world) if only_from is None else [only_from]
    if rank in senders:
        for peer in range(world):
            if peer == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as conn:
                conn.connect(names[peer])
                socket.send_fds(conn, [rank.to_bytes(4, "little")], [fd])
    received: List[Optional[int]] = [None] * world
    received[rank] = fd
    expect = sum(1 for r in senders if r != rank)
    server.settimeout(60.0)
    for _ in range(expect):
        conn, _addr = server.accept()
        with conn:
            msg, fds, _flags, _a = socket.recv_fds(conn, 4, 1)
            received[int.from_bytes(msg, "little")] = fds[0]
    server.close()
    dist.barrier(group=process_group)
    return received


def _all_ok(ok: bool, process_group) -> bool:
    flags: List[Optional[bool]] = [None] * dist.get_world_size(process_group)
    dist.all_gather_object(flags, bool(ok), group=process_group)
    return all(flags)


def _vmm_process_heap(device: torch.device, layout: HeapLayout, process_group):
    """``(base pointers, multicast pointer or 0, VmmHeap)`` or ``None`` when any rank cannot take part."""
    world, rank = dist.get_world_size(process_group), dist.get_rank(process_group)
    vmm, mc = _symm_support(device)
    if not _all_ok(vmm and _vmm_wanted(), process_group):
        return None
    use_mc = _all_ok(mc and _nvls_wanted(), process_group)
    size = _size_t(0)
    with torch.cuda.device(device):
        ok = LIB.tpb_symm_round_size(device.index, world if use_mc else 1, layout.total, ctypes.byref(size)) == 0
        handle, fd = _ull(0), c_int(-1)
        ok = ok and LIB.tpb_symm_create(device.index, size.value, ctypes.byref(handle), ctypes.byref(fd)) == 0
    if not _all_ok(ok, process_group):
        if ok:
            os.close(fd.value)
            LIB.tpb_symm_release(handle.value)
        return None
    heap = VmmHeap(size.value)
    heap.handles.append(handle.value)
    fds = _exchange_fds(fd.value, rank, world, process_group)
    ptrs = []
    with torch.cuda.device(device):
        for r in range(world):
            h = handle.value
            if r != rank:
                imported = _ull(0)
                check(LIB.tpb_symm_import(fds[r], ctypes.byref(imported)), "tpb_symm_import")
                os.close(fds[r])
                h = imported.value
                heap.handles.append(h)
            ptrs.append(_map(h, size.value, [device.index]))
        os.close(fd.value)
        heap.mappings = list(ptrs)
        torch.cuda.synchronize(device)
        tensor_from_ptr(ptrs[rank], size.value, device).zero_()
        torch.cuda.synchronize(device)
    mc_ptr = 0
    if use_mc:
        mc_handle, mc_fd = _ull(0), c_int(-1)
        ok = True
        with torch.cuda.device(device):
            if rank == 0:
                ok = LIB.tpb_mc_create(world, size.value, ctypes.byref(mc_handle), ctypes.byref(mc_fd)) == 0
        if _all_ok(ok, process_group):
            mc_fds = _exchange_fds(mc_fd.value if rank == 0 else None, rank, world, process_group, only_from=0)
            with torch.cuda.device(device):
                if rank != 0:
                    ok = LIB.tpb_symm_import(mc_fds[0], ctypes.byref(mc_handle)) == 0
                    os.close(mc_fds[0])
                else:
                    os.close(mc_fd.value)
                ok = ok and LIB.tpb_mc_add_device(mc_handle.value, device.index) == 0
            if _all_ok(ok, process_group):  # every device is added before anyone binds
                with torch.cuda.device(device):
                    ok = LIB.tpb_mc_bind(mc_handle.value, handle.value, size.value) == 0
                    if ok:
                        heap.mc_handle = mc_handle.value
                        heap.bound.append(device.index)
                if _all_ok(ok, process_group):
                    with torch.cuda.device(device):
                        mc_ptr = _map(mc_handle.value, size.value, [device.index])
                    heap.mc_ptr = mc_ptr
        if not mc_ptr:
            logger.warning("NVLink multicast set-up failed; collectives use plain peer loads and stores")
    dist.barrier(group=process_group)
    return ptrs, mc_ptr, heap


def make_process_comm(device: torch.device, process_group=None, slot_stride: int = DEFAULT_SLOT_STRIDE,
                      max_slots: int = 64, staging_bytes: int = DEFAULT_STAGING) -> RankComm:
    """One process per GPU: allocate the local region, share it with the peers, map theirs."""
    world, rank = dist.get_world_size(process_group), dist.get_rank(process_group)
    if world > MAX_WORLD:
        raise ValueError(f"at most {MAX_WORLD} ranks are supported by the device collectives")
    layout = HeapLayout(slot_stride, max(max_slots, world), staging_bytes)
    vmm = _vmm_process_heap(device, layout, process_group)
    if vmm is not None:
        ptrs, mc_ptr, heap = vmm
        comm = RankComm(world, rank, device, layout, ptrs, mc_base=mc_ptr, heap=heap)
        dist.barrier(group=process_group)
        return comm
    base = _alloc_region(device, layout.total)
    handle = ctypes.create_string_buffer(64)
    with torch.cuda.device(device):
        check(LIB.tpb_ipc_get_handle(c_void_p(base), handle), "tpb_ipc_get_handle")
    handles: List[Optional[bytes]] = [None] * world
    dist.all_gather_object(handles, handle.raw, group=process_group)
    ptrs = []
    for r in range(world):
        if r == rank:
            ptrs.append(base)
            continue
        peer = c_void_p()
        with torch.cuda.device(device):
            check(LIB.tpb_ipc_open_handle(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)), "tpb_ipc_open_handle")
        ptrs.append(peer.value)
    comm = RankComm(world, rank, device, layout, ptrs)
    dist.barrier(group=process_group)  # nobody launches before every mapping exists
    return comm


def _vmm_thread_heap(devices: Sequence[torch.device], layout: HeapLayout):
    """All ranks in one process: every region is mapped once with access for every device; one multicast view."""
    if not _vmm_wanted():
        return None
    support = [_symm_support(d) for d in devices]
    if not all(v for v, _ in support):
        return None
    use_mc = all(m for _, m in support) and _nvls_wanted() and len(devices) > 1
    indices = [d.index for d in devices]
    size = _size_t(0)
    with torch.cuda.device(devices[0]):
        if LIB.tpb_symm_round_size(indices[0], len(devices) if use_mc else 1, layout.total, ctypes.byref(size)) != 0:
            return None
    heap = VmmHeap(size.value)
    try:
        for d in devices:
            handle = _ull(0)
            with torch.cuda.device(d):
                check(LIB.tpb_symm_create(d.index, size.value, ctypes.byref(handle), None), "tpb_symm_create")
                heap.handles.append(handle.value)
                heap.mappings.append(_map(handle.value, size.value, indices))
                tensor_from_ptr(heap.mappings[-1], size.value, d).zero_()
                torch.cuda.synchronize(d)
    except RuntimeError as exc:
        logger.warning("VMM symmetric heap unavailable (%s); using cudaMalloc + peer access", exc)
        heap.close()
        return None
    mc_ptr = 0
    if use_mc:
        mc_handle = _ull(0)
        with torch.cuda.device(devices[0]):
            ok = LIB.tpb_mc_create(len(devices), size.value, ctypes.byref(mc_handle), None) == 0
        ok = ok and all(LIB.tpb_mc_add_device(mc_handle.value, i) == 0 for i in indices)
        if ok:
            heap.mc_handle = mc_handle.value
            for d, handle in zip(devices, heap.handles):
                with torch.cuda.device(d):
                    if LIB.tpb_mc_bind(mc_handle.value, handle, size.value) == 0:
                        heap.bound.append(d.index)
                    else:
                        ok = False
        if ok:
            with torch.cuda.device(devices[0]):
                mc_ptr = heap.mc_ptr = _map(mc_handle.value, size.value, indices)
        else:
            logger.warning("NVLink multicast set-up failed; collectives use plain peer loads and stores")
    return list(heap.mappings), mc_ptr, heap


def make_thread_comms(devices: Sequence[torch.device], slot_stride: int = DEFAULT_SLOT_STRIDE, max_slots: int = 64,
                      staging_bytes: int = DEFAULT_STAGING) -> Optional[List[RankComm]]:
    """All ranks in one process: share plain pointers (VMM mappings, or cudaMalloc + pairwise peer access)."""
    world = len(devices)
    if world > MAX_WORLD or len({d.index for d in devices}) != world:
        return None
    for d in devices:
        with torch.cuda.device(d):
            for peer in devices:
                if peer != d and LIB.tpb_enable_peer_access(peer.index) != 0:
                    logger.warning("no peer access between %s and %s; device collectives disabled", d, peer)
                    return None
    layout = HeapLayout(slot_stride, max(max_slots, world), staging_bytes)
    vmm = _vmm_thread_heap(devices, layout)
    if vmm is not None:
        bases, mc_ptr, heap = vmm
        return [RankComm(world, r, devices[r], layout, bases, mc_base=mc_ptr, heap=heap) for r in range(world)]
    bases = [_alloc_region(d, layout.total) for d in devices]
    return [RankComm(world, r, devices[r], layout, bases) for r in range(world)]


# ------------------------------------------------------------------------------------------------
# rule-action adaptors ("sum" / "gather d") and autograd
# ------------------------------------------------------------------------------------------------


class _AllReduceFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm: RankComm):
        ctx.comm = comm
        return comm.all_reduce(x.contiguous()).clone()

    @staticmethod
    def backward(ctx, grad):
        return ctx.comm.all_reduce(grad.contiguous()).clone(), None


class _AllGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, comm: RankComm):
        ctx.comm, ctx.dim, ctx.shape = comm, dim, x.shape
        stacked = comm.all_gather(x.contiguous())  # [world, ...]
        return torch.cat(list(stacked.unbind(0)), dim=dim)

    @staticmethod
    def backward(ctx, grad):
        comm, dim = ctx.comm, ctx.dim
        parts = torch.stack(grad.chunk(comm.world, dim=dim))  # [world, *x.shape]
        return comm.reduce_scatter(parts.contiguous()).clone(), None, None


class DeviceAllReduce:
    """``"sum"`` on the symmetric heap (one process per rank).  The kernels sum bf16 and fp32; any other dtype (fp16,
    integers ...) goes to ``fallback`` - the process-group all-reduce - so that the result keeps the input's dtype."""

    def __init__(self, comm: RankComm, fallback=None):
        self.comm, self.fallback = comm, fallback

    def __call__(self, x: torch.Tensor, rank: int = 0):
        if x.dtype not in (torch.bfloat16, torch.float32) or not x.is_cuda:
            if self.fallback is None:
                raise TypeError(f"the device all-reduce sums bf16 and fp32 tensors, got {x.dtype} and no fallback collective")
            return self.fallback(x, rank)
        self.comm.poll_status()
        return _AllReduceFn.apply(x, self.comm)


class DeviceAllGather:
    """``"gather d"`` on the symmetric heap; falls back to the process group for uneven slices."""

    def __init__(self, comm: RankComm, dim: int, fallback, process_group=None):
        self.comm, self.dim, self.fallback, self.pg = comm, dim, fallback, process_group
        self._even: Dict[tuple, bool] = {}
        self._warned = False

    def __call__(self, x: torch.Tensor, rank: int = 0):
        dim = self.dim % x.ndim
        key = (tuple(x.shape), dim)
        even = self._even.get(key)
        if even is None:
            sizes = torch.tensor([x.shape[dim]], device=x.device)
            gathered = [torch.zeros_like(sizes) for _ in range(self.comm.world)]
            dist.all_gather(gathered, sizes, group=self.pg)
            even = self._even[key] = len({int(t.item()) for t in gathered}) == 1
        per = 8 if x.dtype == torch.bfloat16 else 4
        if not even or x.numel() % per or x.dtype not in (torch.bfloat16, torch.float32):
            if not self._warned:
                self._warned = True
                logger.info("gather of %s %s along dim %d goes through the process group: the device all-gather takes equal "
                            "bf16 / fp32 slices whose size is a multiple of 16 bytes", tuple(x.shape), x.dtype, dim)
            return self.fallback(x, rank)
        self.comm.poll_status()
        return _AllGatherFn.apply(x, dim, self.comm)


class _FlatGatherFn(torch.autograd.Function):
    """ZeRO-3 flat-shard gather: ``[L] -> [world, L]``; backward = summing reduce-scatter."""

    @staticmethod
    def forward(ctx, flat, comm: RankComm):
        ctx.comm = comm
        return comm.all_gather(flat.detach()).clone()

    @staticmethod
    def backward(ctx, grad):
        return ctx.comm.reduce_scatter(grad.contiguous()).clone(), None


class DeviceFlatGather:
    def __init__(self, comm: RankComm, fallback):
        self.comm, self.fallback = comm, fallback

    def all_gather_flat(self, flats):
        flat = flats[0]
        per = 8 if flat.dtype == torch.bfloat16 else 4
        if flat.dtype not in (torch.bfloat16, torch.float32) or flat.numel() % per:
            return self.fallback.all_gather_flat(flats)
        return [_FlatGatherFn.apply(flat, self.comm)]


class ProcessBackend:
    """Collective factory used by ``Config.create_collective_ops`` in the one-process-per-GPU mode."""

    def __init__(self, comm: RankComm, process_group=None):
        self.comm, self.pg = comm, process_group

    def all_reduce_op(self, group):
        from tensor_parallel_b200.parallel.collectives import DistributedAllReduce

        return DeviceAllReduce(self.comm, DistributedAllReduce(self.comm.world, self.pg))

    def all_gather_op(self, group, dim):
        from tensor_parallel_b200.parallel.collectives import DistributedAllGather

        return DeviceAllGather(self.comm, dim, DistributedAllGather(self.comm.world, dim, self.pg), self.pg)

    def flat_gather(self):
        from tensor_parallel_b200.parallel.distributed import ProcessGroupFlatGather

        return DeviceFlatGather(self.comm, ProcessGroupFlatGather(self.pg))


_process_backends: Dict[int, ProcessBackend] = {}
_lock = threading.Lock()


def process_backend(device: torch.device, process_group=None) -> Optional[ProcessBackend]:
    key = id(process_group)
    with _lock:
        backend = _process_backends.get(key)
        if backend is None:
            backend = _process_backends[key] = ProcessBackend(make_process_comm(device, process_group), process_group)
        return backend


# ------------------------------------------------------------------------------------------------
# single-process multi-GPU mode: one host thread per rank, kernels launched for all ranks by one thread
# ------------------------------------------------------------------------------------------------


class _MultiRankAllReduce(torch.autograd.Function):
    """All ranks' tensors in, all ranks' sums out: one autograd node spanning every device, so the backward
    pass (driven by a single thread) launches the mirrored collective on all devices as well."""

    @staticmethod
    def forward(ctx, comms, *xs):
        ctx.comms = comms
        outs = []
        for comm, x in zip(comms, xs):
            with torch.cuda.device(comm.device):
                outs.append(comm.all_reduce(x.contiguous()).clone())
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        outs = []
        shapes = [g for g in grads if g is not None]
        for comm, g in zip(ctx.comms, grads):
            with torch.cuda.device(comm.device):
                if g is None:
                    g = torch.zeros(shapes[0].shape, dtype=shapes[0].dtype, device=comm.device)
                outs.append(comm.all_reduce(g.contiguous()).clone())
        return (None, *outs)


class _MultiRankAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, comms, dim, *xs):
        ctx.comms, ctx.dim = comms, dim
        outs = []
        for comm, x in zip(comms, xs):
            with torch.cuda.device(comm.device):
                stacked = comm.all_gather(x.contiguous())
                outs.append(torch.cat(list(stacked.unbind(0)), dim=dim))
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        outs = []
        shapes = [g for g in grads if g is not None]
        world = len(ctx.comms)
        for comm, g in zip(ctx.comms, grads):
            with torch.cuda.device(comm.device):
                if g is None:
                    g = torch.zeros(shapes[0].shape, dtype=shapes[0].dtype, device=comm.device)
                parts = torch.stack(g.chunk(world, dim=ctx.dim)).contiguous()
                outs.append(comm.reduce_scatter(parts).clone())
        return (None, None, *outs)


class ThreadDeviceAllReduce:
    """``"sum"`` for the threaded mode on CUDA.

    Without gradients (inference) every rank thread launches its own all-reduce kernel on its own GPU and moves on:
    the kernels meet on the GPUs through flags in the shared symmetric heaps (bounded waits), the host threads never
    wait for each other - the reference puts two host barriers around every collective
    (``src/tensor_parallel/communications.py:34-52``).  With gradients the ranks still meet once on the host, because
    the backward pass is driven by ONE autograd graph that spans all devices: the authoritative thread then launches the
    kernel of every rank from one autograd node (no NCCL, no host-side reduction)."""

    def __init__(self, group, comms, fallback):
        from tensor_parallel_b200.parallel.collectives import CollectiveOperation

        self.comms, self.fallback = comms, fallback
        self._op = CollectiveOperation(len(comms), lambda *xs: _MultiRankAllReduce.apply(comms, *xs), group=group)

    def __call__(self, x: torch.Tensor, rank: int):
        if not x.is_cuda or x.dtype not in (torch.bfloat16, torch.float32) or x.numel() * x.element_size() > self.comms[0].layout.staging_bytes:
            return self.fallback(x, rank)
        if not (torch.is_grad_enabled() and x.requires_grad):
            comm = self.comms[rank]
            comm.poll_status()
            with torch.cuda.device(comm.device):
                return comm.all_reduce(x.contiguous()).clone()
        return self._op(x, rank)


class ThreadDeviceAllGather:
    def __init__(self, group, comms, dim, fallback):
        from tensor_parallel_b200.parallel.collectives import CollectiveOperation, Rendezvous

        self.comms, self.dim, self.fallback = comms, dim, fallback
        self._shapes = Rendezvous(group)
        self._even: List[Dict[tuple, bool]] = [dict() for _ in comms]  # per rank: (shape, dtype, device kind) -> all ranks alike
        self._op = CollectiveOperation(len(comms), lambda *xs: _MultiRankAllGather.apply(comms, self.dim % xs[0].ndim, *xs), group=group)

    def __call__(self, x: torch.Tensor, rank: int):
        key = (tuple(x.shape), x.dtype, x.is_cuda)
        even = self._even[rank].get(key)
        if even is None:  # the ranks compare shapes on the host once per shape; later calls go straight to the GPU
            shapes = self._shapes.exchange(rank, key)
            even = self._even[rank][key] = len(set(shapes)) == 1
        per = 8 if x.dtype == torch.bfloat16 else 4
        world = len(self.comms)
        ok = (even and x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and x.numel() % per == 0
              and world * x.numel() * x.element_size() <= self.comms[0].layout.staging_bytes)
        if not ok:
            return self.fallback(x, rank)
        if not (torch.is_grad_enabled() and x.requires_grad):
            comm = self.comms[rank]
            comm.poll_status()
            with torch.cuda.device(comm.device):
                stacked = comm.all_gather(x.contiguous())
                return torch.cat(list(stacked.unbind(0)), dim=self.dim % x.ndim)
        return self._op(x, rank)


class ThreadBackend:
    """Collective factory for ``Config.create_collective_ops`` when all ranks are CUDA devices of one process."""

    def __init__(self, comms):
        self.comms = comms

    def all_reduce_op(self, group):
        from tensor_parallel_b200.parallel.collectives import ThreadAllReduce

        return ThreadDeviceAllReduce(group, self.comms, ThreadAllReduce(group))

    def all_gather_op(self, group, dim):
        from tensor_parallel_b200.parallel.collectives import ThreadAllGather

        return ThreadDeviceAllGather(group, self.comms, dim, ThreadAllGather(group, dim))


_thread_backends: Dict[tuple, Optional[ThreadBackend]] = {}


def thread_backend(devices: Sequence[torch.device], staging_bytes: int = 64 << 20) -> Optional[ThreadBackend]:
    """Symmetric heaps for all ``devices`` of this process (peer access must be available), or ``None``."""
    key = tuple(d.index for d in devices)
    with _lock:
        if key not in _thread_backends:
            comms = make_thread_comms(devices, staging_bytes=staging_bytes)
            _thread_backends[key] = ThreadBackend(comms) if comms is not None else None
        return _thread_backends[key]
