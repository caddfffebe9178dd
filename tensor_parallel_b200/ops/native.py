"""ctypes binding of ``libtpb200.so`` plus autograd wrappers around its kernels.

Importing this module loads the library (building it first if the sources are newer and nvcc is
present) and raises if that is impossible: on a machine with CUDA tensors there is no silent
fallback to stock PyTorch operators.
"""
from __future__ import annotations

import ctypes
import math
import os
import threading
from typing import Dict, Optional, Tuple

import torch

from tensor_parallel_b200 import build as _build

_ERRORS = {1: "bad argument", 2: "alignment rule violated", 3: "CUDA runtime error", 4: "driver entry point missing",
           5: "tensor map rejected", 6: "reduction workspace too small", 7: "size beyond compiled-in maximum"}


def _load() -> ctypes.CDLL:
    variant = os.environ.get("TPB_LIB_PATH")  # a variant built with build(lib_path=..., extra_flags=...)
    if variant:
        return ctypes.CDLL(variant)
    path = _build.LIB_PATH
    if not path.exists() or os.environ.get("TPB_REBUILD"):
        _build.build()  # explicit rebuilds otherwise: python -m tensor_parallel_b200.build
    return ctypes.CDLL(str(path))


LIB = _load()
launch_count = 0  # kernels launched through this binding since import (bench.py reports the delta)

c_void_p, c_int, c_float, c_ll, c_size_t = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_size_t


class GemmPlan(ctypes.Structure):
    _fields_ = [("swapped", c_int), ("bn", c_int), ("kbox", c_int), ("m_tiles", c_int), ("n_tiles", c_int), ("k_blocks", c_int),
                ("k_splits", c_int), ("kb_per_split", c_int), ("reduce", c_int), ("grid", c_int), ("tokens_pad", c_int),
                ("tiles", c_int), ("slot_elems", c_size_t), ("stream_k", c_int)]


class ReduceCtx(ctypes.Structure):
    _fields_ = [("world", c_int), ("rank", c_int), ("slots", c_void_p * 8), ("arrivals", c_void_p * 8),
                ("expected", c_void_p), ("split_counters", c_void_p), ("status", c_void_p), ("slot_stride", c_size_t), ("max_slots", c_int),
                ("max_tiles", c_int), ("ll_epochs", c_void_p), ("mc_slots", c_void_p)]


class GemmOpts(ctypes.Structure):
    _fields_ = [("x_mn", c_int), ("w_mn", c_int), ("norm_mode", c_int), ("norm_eps", c_float), ("norm_x", c_void_p),
                ("norm_ld", c_ll), ("norm_k", c_int), ("norm_rowsum", c_void_p), ("wait_seconds", ctypes.c_double),
                ("out_elems", c_size_t)]


def device_wait_seconds() -> float:
    """Bound of every wait for a peer GPU inside a kernel.  ``TPB_DEVICE_WAIT_S`` if set, else the host-side
    collective timeout ``TENSOR_PARALLEL_TIMEOUT`` capped at 30 s: ranks may legitimately drift apart by seconds
    (a checkpoint written by one rank, a slow data loader), but a kernel should not spin for minutes on a dead peer."""
    explicit = os.environ.get("TPB_DEVICE_WAIT_S")
    if explicit:
        return float(explicit)
    return min(float(os.environ.get("TENSOR_PARALLEL_TIMEOUT", "600")), 30.0)


def check(code: int, what: str):
    if code != 0:
        detail = ""
        if code == 3:
            buf = ctypes.create_string_buffer(256)
            LIB.tpb_last_cuda_error(buf, 256)
            detail = f": {buf.value.decode()}"
        raise RuntimeError(f"{what} failed: {_ERRORS.get(code, code)}{detail}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 0
    if t.dtype == torch.float32:
        return 1
    raise TypeError(f"native kernels take bf16 or fp32 tensors, got {t.dtype}")


# ------------------------------------------------------------------------------------------------
# per-device scratch: status word + split-K workspace
# ------------------------------------------------------------------------------------------------

MAX_TILES = 4096
MAX_SLOTS = 17  # 1 cross-rank slot (world = 1) + up to 16 split-K partials


class DeviceState:
    """Status word and the local split-K reduction workspace of one GPU."""

    def __init__(self, device: torch.device):
        self.device = device
        self.status = torch.zeros(4, dtype=torch.int32, device=device)
        self.arrivals = torch.zeros(MAX_TILES, dtype=torch.int32, device=device)
        self.expected = torch.zeros(MAX_TILES, dtype=torch.int32, device=device)
        self.split_counters = torch.zeros(MAX_TILES, dtype=torch.int32, device=device)
        self.slots: Optional[torch.Tensor] = None
        self.slot_stride = 0
        self.ctx = ReduceCtx()
        self._refresh()

    def _refresh(self):
        ctx = self.ctx
        ctx.world, ctx.rank = 1, 0
        ctx.slots[0] = self.slots.data_ptr() if self.slots is not None else 0
        ctx.arrivals[0] = self.arrivals.data_ptr()
        ctx.expected = self.expected.data_ptr()
        ctx.split_counters = self.split_counters.data_ptr()
        ctx.status = self.status.data_ptr()
        ctx.slot_stride = self.slot_stride
        ctx.max_slots, ctx.max_tiles = MAX_SLOTS, MAX_TILES

    def ensure_slots(self, elems: int):
        """Grow-only; growing replaces the buffer, so warm shapes up before capturing a CUDA graph."""
        if elems > self.slot_stride:
            self.slot_stride = max(elems, 1 << 20)
            self.slots = torch.empty(MAX_SLOTS * self.slot_stride, dtype=torch.float32, device=self.device)
            self._refresh()

    def check_status(self):
        code = int(self.status[0].item())
        if code:
            self.status.zero_()
            raise RuntimeError({1: "an mbarrier wait", 2: "a peer flag wait"}.get(code, f"status {code}") + " timed out inside a kernel")


_states: Dict[int, DeviceState] = {}
_states_lock = threading.Lock()


def device_state(device: torch.device) -> DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    with _states_lock:
        st = _states.get(idx)
        if st is None:
            st = _states[idx] = DeviceState(torch.device("cuda", idx))
        return st


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------

LIB.tpb_gemm_plan.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(GemmPlan)]
LIB.tpb_gemm_plan_ex.argtypes = [c_int, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(GemmPlan)]
LIB.tpb_gemm_bf16_ex.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_int, c_float, ctypes.POINTER(GemmPlan), ctypes.POINTER(ReduceCtx), ctypes.POINTER(GemmOpts), c_void_p]
LIB.tpb_gemm_tune_split.argtypes = [c_int, c_int]
LIB.tpb_set_wait_limit.argtypes = [ctypes.c_double]
LIB.tpb_set_wait_limit(device_wait_seconds())
LIB.tpb_gemm_disable_flagged_exchange.argtypes = [c_int]
# TPB_FLAGGED_EXCHANGE = always | never: fixes the cross-rank protocol of the fused few-token GEMM + all-reduce
# (default: chosen by rank count, see csrc/gemm_sm100.cu)
_exchange = os.environ.get("TPB_FLAGGED_EXCHANGE", "")
if _exchange in ("always", "never"):
    LIB.tpb_gemm_disable_flagged_exchange(-1 if _exchange == "always" else 1)
LIB.tpb_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                              c_int, c_float, ctypes.POINTER(GemmPlan), ctypes.POINTER(ReduceCtx), c_void_p]
ACT_CODES = {None: 0, "none": 0, "relu": 1, "gelu": 2, "gelu_tanh": 3, "silu": 4, "swiglu16": 5}
_plan_cache: Dict[Tuple, GemmPlan] = {}


def gemm_plan(tokens: int, features: int, k: int, world: int = 1, force_splits: int = 0, force_kbox: int = 0,
              no_swap: bool = False) -> GemmPlan:
    key = (tokens, features, k, world, force_splits, force_kbox, no_swap, torch.cuda.current_device())
    plan = _plan_cache.get(key)
    if plan is None:
        plan = GemmPlan()
        check(LIB.tpb_gemm_plan_ex(tokens, features, k, world, force_splits, force_kbox, int(no_swap), ctypes.byref(plan)), "gemm_plan")
        _plan_cache[key] = plan
    return plan


def tune_split(min_tile_kb: int = 0, target_kb: int = 0):
    """Thresholds of the automatic split-K of few-tile decode GEMMs; cached plans are dropped."""
    LIB.tpb_gemm_tune_split(min_tile_kb, target_kb)
    _plan_cache.clear()


def gemm_supported(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (
        x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.ndim == 2 and x.shape[-1] == weight.shape[1]
        and x.numel() > 0 and weight.shape[0] > 0
    )


def gemm_nt(x2d: torch.Tensor, w: torch.Tensor, bias=None, residual=None, act=None, out=None, force_splits: int = 0,
            reduce_ctx: Optional[ReduceCtx] = None, world: int = 1, bias_scale: float = 1.0, force_kbox: int = 0,
            x_t: bool = False, w_t: bool = False, norm: Optional[Tuple] = None, norm_rows: Optional[torch.Tensor] = None,
            out_elems: int = 0) -> torch.Tensor:
    """``out[tokens, features] = act(x2d @ w.T + bias) + residual`` on the tcgen05 kernel.

    ``x_t`` / ``w_t``: the operand is passed transposed, ``x2d`` as ``[k, tokens]`` / ``w`` as ``[k, features]`` (row
    major), and is read as it lies in memory (MN-major tensor-core operand) - what the backward GEMMs of a linear
    layer need.  ``norm = (mode, eps, rowsum)`` folds an RMSNorm (``mode`` 1) or LayerNorm (2) of the rows of ``x2d``
    into the kernel (at most 64 tokens): ``w`` must already be multiplied by the norm weight along k.  ``norm_rows``
    ``[tokens, n]`` are the rows the statistics are taken over when ``x2d`` is only a column slice of them.
    ``out_elems`` (a library built with ``-DTPB_BOUNDS`` only): extent of ``out`` that the kernel checks its store
    indices against; 0 derives it from the shape."""
    global launch_count
    if x_t:
        k, tokens = x2d.shape
    else:
        tokens, k = x2d.shape
    features = w.shape[1] if w_t else w.shape[0]
    x2d, w = _tma_ready(x2d), _tma_ready(w)
    if out is None:
        out = torch.empty(tokens, features // 2 if act == "swiglu16" else features, dtype=torch.bfloat16, device=x2d.device)
    plan = gemm_plan(tokens, features, k, world, force_splits, force_kbox, no_swap=x_t or w_t)
    state = device_state(x2d.device)
    ctx = reduce_ctx
    if ctx is None:
        if plan.reduce:
            state.ensure_slots(tokens * (features if act == "swiglu16" else out.stride(0)))
        ctx = state.ctx
    opts = None
    if x_t or w_t or norm is not None or out_elems:
        opts = GemmOpts()
        opts.x_mn, opts.w_mn, opts.out_elems = int(x_t), int(w_t), int(out_elems)
        if norm is not None:
            mode, eps, rowsum = norm
            opts.norm_mode, opts.norm_eps = int(mode), float(eps)
            rows = x2d if norm_rows is None else norm_rows
            opts.norm_x, opts.norm_ld, opts.norm_k = rows.data_ptr(), rows.stride(0), rows.shape[1]
            opts.norm_rowsum = rowsum.data_ptr() if rowsum is not None else 0
    check(LIB.tpb_gemm_bf16_ex(_ptr(x2d), _ptr(w), _ptr(out), _ptr(bias), _ptr(residual), tokens, features, k, x2d.stride(0),
                               w.stride(0), out.stride(0), ACT_CODES[act], bias_scale, ctypes.byref(plan), ctypes.byref(ctx),
                               ctypes.byref(opts) if opts is not None else None, _stream()), "tpb_gemm_bf16")
    launch_count += 1
    return out


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """TMA needs a unit inner stride, a 16-byte aligned base and a row pitch that is a multiple of 16 bytes.
    Tensors that break a rule are copied into a buffer with a padded row pitch (the pad is never read: columns
    past the logical width are out of bounds for the tensor map and come back as zeros)."""
    if t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    rows, cols = t.shape
    pitch = (cols + 7) // 8 * 8
    buf = torch.empty(rows, pitch, dtype=t.dtype, device=t.device)
    view = buf[:, :cols]
    view.copy_(t)
    return view


def interleave_gate_up(gate_w: torch.Tensor, up_w: torch.Tensor) -> torch.Tensor:
    """Weight of a fused gate|up projection for ``gemm_nt(..., act="swiglu16")``: rows alternate in groups of
    16 gate rows followed by their 16 up rows, so the GEMM epilogue can form ``silu(gate) * up`` in registers."""
    f, h = gate_w.shape
    if f % 16:
        raise ValueError("the gated width must be a multiple of 16")
    return torch.stack((gate_w.reshape(f // 16, 16, h), up_w.reshape(f // 16, 16, h)), dim=1).reshape(2 * f, h).contiguous()


LIB.tpb_transpose_bf16.argtypes = [c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_void_p]


def transpose(x2d: torch.Tensor) -> torch.Tensor:
    global launch_count
    rows, cols = x2d.shape
    if x2d.stride(1) != 1:
        x2d = x2d.contiguous()
    pitch = (rows + 7) // 8 * 8  # keeps the result usable as a TMA operand
    out = torch.empty(cols, pitch, dtype=x2d.dtype, device=x2d.device)[:, :rows]
    check(LIB.tpb_transpose_bf16(_ptr(x2d), _ptr(out), rows, cols, x2d.stride(0), pitch, _stream()), "tpb_transpose_bf16")
    launch_count += 1
    return out


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias):
        x2d = x.reshape(-1, x.shape[-1])
        out = gemm_nt(x2d, weight, bias)
        ctx.save_for_backward(x2d, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return out.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad):
        x2d, weight = ctx.saved_tensors
        g2d = grad.reshape(-1, grad.shape[-1])
        if g2d.dtype != torch.bfloat16:
            g2d = g2d.to(torch.bfloat16)
        if not g2d.is_contiguous():
            g2d = g2d.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = linear_dgrad(g2d, weight).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = linear_wgrad(g2d, x2d)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g2d.float().sum(0).to(grad.dtype)
        return gx, gw, gb


def linear_dgrad(g2d: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``dX[m, k] = sum_n dY[m, n] W[n, k]``: the contraction runs over W's rows, so W ``[n, k]`` is read as it lies in
    memory as an MN-major operand (no transposed copy of the weight)."""
    return gemm_nt(g2d, weight, w_t=True)


def linear_wgrad(g2d: torch.Tensor, x2d: torch.Tensor) -> torch.Tensor:
    """``dW[n, k] = sum_m dY[m, n] X[m, k]``: both operands are contracted over their rows and are read in place as
    MN-major operands (no transposed copies of the gradient and the activation)."""
    return gemm_nt(g2d, x2d, x_t=True, w_t=True)


def linear(x, weight, bias=None):
    if torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad or (bias is not None and bias.requires_grad)):
        return _LinearFn.apply(x, weight, bias)
    x2d = x.reshape(-1, x.shape[-1])
    return gemm_nt(x2d, weight, bias).view(*x.shape[:-1], weight.shape[0])


# ------------------------------------------------------------------------------------------------
# norms
# ------------------------------------------------------------------------------------------------

LIB.tpb_norm_fwd.argtypes = [c_void_p] * 8 + [c_int, c_int, c_float, c_int, c_int, c_void_p]
LIB.tpb_norm_bwd.argtypes = [c_void_p] * 8 + [c_int, c_int, c_int, c_int, c_void_p]


def norm_supported(x: torch.Tensor) -> bool:
    return x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192 and x.numel() > 0


def norm_forward(x2d, weight, bias, eps, mode, residual=None, sum_out=None, want_stats=False, out=None):
    global launch_count
    rows, cols = x2d.shape
    out = torch.empty_like(x2d) if out is None else out
    rstd = torch.empty(rows, dtype=torch.float32, device=x2d.device) if want_stats else None
    mean = torch.empty(rows, dtype=torch.float32, device=x2d.device) if (want_stats and mode == 1) else None
    check(LIB.tpb_norm_fwd(_ptr(x2d), _ptr(residual), _ptr(weight), _ptr(bias), _ptr(out), _ptr(sum_out), _ptr(rstd), _ptr(mean),
                           rows, cols, eps, mode, _dtype_code(x2d), _stream()), "tpb_norm_fwd")
    launch_count += 1
    return out, rstd, mean


class _NormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, mode):
        x2d = x.reshape(-1, x.shape[-1]).contiguous()
        w = None if weight is None else weight.to(x.dtype).contiguous()
        b = None if bias is None else bias.to(x.dtype).contiguous()
        out, rstd, mean = norm_forward(x2d, w, b, eps, mode, want_stats=True)
        ctx.save_for_backward(x2d, w, rstd, mean if mean is not None else rstd)
        ctx.mode, ctx.shape = mode, x.shape
        ctx.wdtype = None if weight is None else weight.dtype
        ctx.bdtype = None if bias is None else bias.dtype
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, grad):
        global launch_count
        x2d, w, rstd, mean = ctx.saved_tensors
        g2d = grad.reshape(x2d.shape).to(x2d.dtype).contiguous()
        rows, cols = x2d.shape
        dx = torch.empty_like(x2d)
        dw = torch.zeros(cols, dtype=torch.float32, device=x2d.device) if w is not None else None
        db = torch.zeros(cols, dtype=torch.float32, device=x2d.device) if ctx.bdtype is not None else None
        check(LIB.tpb_norm_bwd(_ptr(g2d), _ptr(x2d), _ptr(w), _ptr(rstd), _ptr(mean), _ptr(dx), _ptr(dw), _ptr(db), rows, cols,
                               ctx.mode, _dtype_code(x2d), _stream()), "tpb_norm_bwd")
        launch_count += 1
        return (dx.view(ctx.shape), None if dw is None else dw.to(ctx.wdtype), None if db is None else db.to(ctx.bdtype), None, None)


def rms_norm(x, weight, eps):
    return _NormFn.apply(x, weight, None, eps, 0)


def layer_norm(x, weight, bias, eps):
    return _NormFn.apply(x, weight, bias, eps, 1)


# ------------------------------------------------------------------------------------------------
# rotary embedding
# ------------------------------------------------------------------------------------------------

LIB.tpb_rope.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_ll,
                         c_ll, c_int, c_void_p]


def rope_supported(x: torch.Tensor) -> bool:
    return x.dtype in (torch.bfloat16, torch.float32) and x.ndim == 4 and x.numel() > 0


def _rope_launch(x, positions, theta, rotary_dim, interleaved, inverse):
    global launch_count
    b, s, h, d = x.shape
    xc = x.contiguous()
    out = torch.empty_like(xc)
    pos = positions.to(device=x.device, dtype=torch.int64).expand(b, s).contiguous()
    check(LIB.tpb_rope(_ptr(xc), _ptr(out), _ptr(pos), c_void_p(0), s, b * s, h, d, rotary_dim, theta, int(interleaved), int(inverse),
                       h * d, h * d, _dtype_code(xc), _stream()), "tpb_rope")
    launch_count += 1
    return out


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, theta, rotary_dim, interleaved):
        ctx.args = (positions, theta, rotary_dim, interleaved)
        return _rope_launch(x, positions, theta, rotary_dim, interleaved, False)

    @staticmethod
    def backward(ctx, grad):
        positions, theta, rotary_dim, interleaved = ctx.args
        return _rope_launch(grad, positions, theta, rotary_dim, interleaved, True), None, None, None, None


def rope(x, positions, theta, rotary_dim, interleaved):
    rotary_dim = x.shape[-1] if rotary_dim is None else rotary_dim
    return _RopeFn.apply(x, positions, float(theta), int(rotary_dim), bool(interleaved))


# ------------------------------------------------------------------------------------------------
# activations
# ------------------------------------------------------------------------------------------------

LIB.tpb_act_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_int, c_int, c_void_p]
LIB.tpb_act_bwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p]


def elementwise_supported(x: torch.Tensor) -> bool:
    return x.dtype in (torch.bfloat16, torch.float32) and x.shape[-1] % 8 == 0 and x.numel() > 0


def act_forward(gate, up, kind: int, out=None):
    """``act(gate) * up`` (``up`` may be None); ``gate`` / ``up`` may be column slices of one wider tensor."""
    global launch_count
    cols = gate.shape[-1]
    g2 = gate.reshape(-1, cols) if gate.stride(-1) == 1 else gate.contiguous().view(-1, cols)
    u2 = None if up is None else (up.reshape(-1, cols) if up.stride(-1) == 1 else up.contiguous().view(-1, cols))
    rows = g2.shape[0]
    if out is None:
        out = torch.empty(*gate.shape, dtype=gate.dtype, device=gate.device)
    check(LIB.tpb_act_fwd(_ptr(g2), _ptr(u2), _ptr(out), rows, cols, g2.stride(0), 0 if u2 is None else u2.stride(0), kind,
                          _dtype_code(gate), _stream()), "tpb_act_fwd")
    launch_count += 1
    return out


class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up, kind):
        gate_c = gate.contiguous()
        up_c = None if up is None else up.contiguous()
        ctx.save_for_backward(gate_c, up_c if up_c is not None else gate_c)
        ctx.kind, ctx.has_up = kind, up is not None
        return act_forward(gate_c, up_c, kind)

    @staticmethod
    def backward(ctx, grad):
        global launch_count
        gate, up = ctx.saved_tensors
        up = up if ctx.has_up else None
        g = grad.to(gate.dtype).contiguous()
        dgate = torch.empty_like(gate)
        dup = torch.empty_like(gate) if up is not None else None
        check(LIB.tpb_act_bwd(_ptr(g), _ptr(gate), _ptr(up), _ptr(dgate), _ptr(dup), gate.numel(), ctx.kind, _dtype_code(gate), _stream()),
              "tpb_act_bwd")
        launch_count += 1
        return dgate, dup, None


def gelu(x, approximate="none"):
    return _ActFn.apply(x, None, 3 if approximate == "tanh" else 2)


def relu(x):
    return _ActFn.apply(x, None, 1)


def swiglu(gate, up):
    return _ActFn.apply(gate, up, 4)


def geglu(gate, up, approximate="tanh"):
    return _ActFn.apply(gate, up, 3 if approximate == "tanh" else 2)


# ------------------------------------------------------------------------------------------------
# attention
# ------------------------------------------------------------------------------------------------

LIB.tpb_attn_prefill.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_ll] * 12 + [c_int, c_float, c_void_p]
LIB.tpb_attn_prefill_bias.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_ll] * 12 + [c_int, c_float, c_void_p, c_int] + [c_ll] * 4 + [c_void_p]
LIB.tpb_attn_prefill_sm100.argtypes = [c_void_p] * 5 + [c_int] * 6 + [c_ll] * 12 + [c_int, c_float, c_void_p, c_int] + [c_ll] * 4 + [c_void_p, c_void_p]
LIB.tpb_attn_decode.argtypes = [c_void_p] * 7 + [c_int] * 7 + [c_float, c_void_p]
_LEGACY_ATTENTION = bool(os.environ.get("TPB_ATTN_LEGACY"))  # the mma.sync forward kernel instead of the tcgen05 one
LIB.tpb_qkv_rope_append.argtypes = [c_void_p] * 7 + [c_int] * 6 + [c_float, c_int, c_int, c_ll, c_ll, c_ll, c_void_p]


def attention_supported(q, k, v, bias) -> bool:
    if not (q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and q.shape[2] % k.shape[2] == 0 and q.numel() > 0 and k.numel() > 0):
        return False
    if bias is None:
        return True
    # additive score bias (relative positions, ALiBi, padding masks): forward and backward, bias gradient included
    return (bias.is_cuda and bias.dtype in (torch.bfloat16, torch.float32) and bias.ndim <= 4
            and _broadcastable(bias.shape, (q.shape[0], q.shape[2], q.shape[1], k.shape[1])))


def _broadcastable(shape, target) -> bool:
    shape = (1,) * (len(target) - len(shape)) + tuple(shape)
    return all(s == t or s == 1 for s, t in zip(shape, target))


def _strided_ok(t: torch.Tensor) -> bool:
    return t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0


def attention_forward(q, k, v, causal, scale, want_lse=False, bias=None, out=None):
    """q ``[B,Sq,Hq,D]``, k / v ``[B,Sk,Hkv,D]`` (any strides with contiguous head_dim) -> ``[B,Sq,Hq,D]``.
    ``bias`` (bf16 / fp32, broadcastable to ``[B,Hq,Sq,Sk]``) is added to the scaled scores; ``-inf`` masks a key."""
    global launch_count
    q = q if _strided_ok(q) else q.contiguous()
    k = k if _strided_ok(k) else k.contiguous()
    v = v if _strided_ok(v) else v.contiguous()
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    if out is None:  # (a caller's `out` may be a strided [b, sq, hq, d] view with contiguous head_dim)
        out = torch.empty(b, sq, hq, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device) if want_lse else None
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if not _LEGACY_ATTENTION:
        # tcgen05 / TMEM kernel: Q, K, V tiles by TMA straight from the strided views, scores and P V on the tensor cores
        bias4 = None if bias is None else bias.reshape((1,) * (4 - bias.ndim) + tuple(bias.shape))
        strides = [0, 0, 0, 0] if bias4 is None else [0 if bias4.shape[i] == 1 else bias4.stride(i) for i in range(4)]
        status = device_state(q.device).status
        check(LIB.tpb_attn_prefill_sm100(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), b, sq, sk, hq, hkv, d,
                                         q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                         v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
                                         int(causal), scale, _ptr(bias4), 1 if (bias4 is not None and bias4.dtype == torch.float32) else 0,
                                         strides[0], strides[1], strides[2], strides[3], _ptr(status), _stream()), "tpb_attn_prefill_sm100")
    elif bias is None:
        check(LIB.tpb_attn_prefill(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), b, sq, sk, hq, hkv, d,
                                   q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                   v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
                                   int(causal), scale, _stream()), "tpb_attn_prefill")
    else:
        bias4 = bias.reshape((1,) * (4 - bias.ndim) + tuple(bias.shape))
        strides = [0 if bias4.shape[i] == 1 else bias4.stride(i) for i in range(4)]  # size-1 dimensions broadcast
        check(LIB.tpb_attn_prefill_bias(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(lse), b, sq, sk, hq, hkv, d,
                                        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                        v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
                                        int(causal), scale, _ptr(bias4), 1 if bias4.dtype == torch.float32 else 0,
                                        strides[0], strides[1], strides[2], strides[3], _stream()), "tpb_attn_prefill_bias")
    launch_count += 1
    return out, lse


LIB.tpb_attn_backward.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_ll] * 21 + [c_int, c_float, c_void_p]
LIB.tpb_attn_backward_bias.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_ll] * 21 + [c_int, c_float, c_void_p, c_int] + [c_ll] * 4 + [c_void_p, c_void_p]
LIB.tpb_attn_backward_sm100.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_ll] * 21 + [c_int, c_float, c_void_p, c_int] + [c_ll] * 4 + [c_void_p, c_void_p, c_void_p]


def _bias_view(bias):
    """``bias`` as a 4-D tensor over (batch, head, query, key) and its element strides with broadcast dimensions at 0."""
    bias4 = bias.reshape((1,) * (4 - bias.ndim) + tuple(bias.shape))
    return bias4, [0 if bias4.shape[i] == 1 else bias4.stride(i) for i in range(4)]


def attention_backward(q, k, v, out, dout, lse, causal, scale, bias=None, want_dbias=False):
    """Gradients of :func:`attention_forward` (scores are recomputed tile by tile).  With ``bias`` the scores are
    re-biased; ``want_dbias`` also returns the gradient of the bias (fp32, in the bias' own shape)."""
    global launch_count
    q, k, v, dout = (t if _strided_ok(t) else t.contiguous() for t in (q, k, v, dout))
    b, sq, hq, d = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    dq = torch.empty(b, sq, hq, d, dtype=q.dtype, device=q.device)
    dk = torch.empty(b, sk, hkv, d, dtype=q.dtype, device=q.device)
    dv = torch.empty(b, sk, hkv, d, dtype=q.dtype, device=q.device)
    delta = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device)
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    bias4, bstr, dbias = None, [0, 0, 0, 0], None
    if bias is not None:
        bias4, bstr = _bias_view(bias)
        if want_dbias:  # dense fp32 buffer in the bias' shape: the kernel addresses it with the bias' broadcast pattern
            dbias = torch.zeros(bias4.shape, dtype=torch.float32, device=q.device)
            dstr = [0 if dbias.shape[i] == 1 else dbias.stride(i) for i in range(4)]
            if dstr != bstr:  # a non-contiguous bias view: keep one addressing for both
                bias4 = bias4.contiguous()
                bstr = dstr
    bias_is_fp32 = 1 if (bias4 is not None and bias4.dtype == torch.float32) else 0
    if not _LEGACY_ATTENTION:  # tcgen05 kernels (two launches of one template) + the delta kernel
        status = device_state(q.device).status
        check(LIB.tpb_attn_backward_sm100(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse), _ptr(delta), _ptr(dq), _ptr(dk), _ptr(dv),
                                          b, sq, sk, hq, hkv, d,
                                          q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                          v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
                                          dout.stride(0), dout.stride(1), dout.stride(2), dq.stride(0), dq.stride(1), dq.stride(2),
                                          dk.stride(0), dk.stride(1), dk.stride(2), int(causal), scale, _ptr(bias4), bias_is_fp32,
                                          bstr[0], bstr[1], bstr[2], bstr[3], _ptr(dbias), _ptr(status), _stream()),
              "tpb_attn_backward_sm100")
        launch_count += 3
        if want_dbias:
            return dq, dk, dv, dbias.reshape(bias.shape)
        return dq, dk, dv
    check(LIB.tpb_attn_backward_bias(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse), _ptr(delta), _ptr(dq), _ptr(dk), _ptr(dv),
                                     b, sq, sk, hq, hkv, d,
                                     q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
                                     v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
                                     dout.stride(0), dout.stride(1), dout.stride(2), dq.stride(0), dq.stride(1), dq.stride(2),
                                     dk.stride(0), dk.stride(1), dk.stride(2), int(causal), scale, _ptr(bias4),
                                     bias_is_fp32, bstr[0], bstr[1], bstr[2], bstr[3],
                                     _ptr(dbias), _stream()), "tpb_attn_backward")
    launch_count += 3
    if want_dbias:
        return dq, dk, dv, dbias.reshape(bias.shape)
    return dq, dk, dv


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, bias):
        out, lse = attention_forward(q, k, v, causal, scale, want_lse=True, bias=bias)
        ctx.save_for_backward(q, k, v, out, lse, *([bias] if bias is not None else []))
        ctx.causal, ctx.scale, ctx.has_bias = causal, scale, bias is not None
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, out, lse = ctx.saved_tensors[:5]
        bias = ctx.saved_tensors[5] if ctx.has_bias else None
        want_dbias = ctx.has_bias and ctx.needs_input_grad[5]
        grads = attention_backward(q, k, v, out, grad.to(q.dtype), lse, ctx.causal, ctx.scale, bias=bias, want_dbias=want_dbias)
        dbias = grads[3].to(bias.dtype) if want_dbias else None
        return grads[0], grads[1], grads[2], None, None, dbias


def attention(q, k, v, causal, bias=None, scale=None):
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad or (bias is not None and bias.requires_grad))
    if needs_grad:
        return _AttentionFn.apply(q, k, v, bool(causal), scale, bias)
    return attention_forward(q, k, v, causal, scale, bias=bias)[0]


def attn_decode(q, kcache, vcache, len_ptr, len_add, scale=None, splits=1, workspace=None, out=None):
    """q ``[B,Hq,D]`` against cache ``[B,Hkv,Smax,D]``; the number of valid keys is ``len_ptr[0] + len_add``."""
    global launch_count
    b, hq, d = q.shape
    hkv, smax = kcache.shape[1], kcache.shape[2]
    out = torch.empty_like(q) if out is None else out
    part_o = part_ml = None
    if splits > 1:
        if workspace is None:
            workspace = (torch.empty(b * hq * splits * d, dtype=torch.float32, device=q.device),
                         torch.empty(b * hq * splits * 2, dtype=torch.float32, device=q.device))
        part_o, part_ml = workspace
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    check(LIB.tpb_attn_decode(_ptr(q), _ptr(kcache), _ptr(vcache), _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(len_ptr), len_add,
                              b, hq, hkv, d, smax, splits, scale, _stream()), "tpb_attn_decode")
    launch_count += LIB.tpb_last_launches()
    return out


LIB.tpb_attn_decode_fused.argtypes = [c_void_p] * 10 + [c_int] * 6 + [c_float, c_int, c_float, c_int, c_ll, c_ll, c_ll, c_void_p, c_ll, c_int, c_void_p]
LIB.tpb_rope_table.argtypes = [c_void_p, c_int, c_int, c_float, c_void_p]


def rope_table(positions: int, rotary_dim: int, theta: float, device) -> torch.Tensor:
    """fp32 ``[positions, rotary_dim // 2, 2]`` table of (cos, sin) rotary angles for :func:`attn_decode_fused`."""
    global launch_count
    table = torch.empty(positions, rotary_dim // 2, 2, dtype=torch.float32, device=device)
    with torch.cuda.device(device):
        check(LIB.tpb_rope_table(_ptr(table), positions, rotary_dim, theta, _stream()), "tpb_rope_table")
    launch_count += 1
    return table


def attn_decode_fused(q, k, v, kcache, vcache, pos_ptr, rotary_dim, theta, interleaved=False, scale=None, splits=1,
                      workspace=None, out=None, rope_angles=None):
    """One decode step of attention in a single launch: rotate q / k of the new token (``q/k/v``: 2-D row views of the
    projection output), append k, v to the cache at ``pos_ptr[0]``, attend over ``[0, pos]`` and merge the key splits.
    ``workspace = (part_o, part_ml, counters)`` with ``counters`` an int32 tensor of at least ``batch * kv_heads`` elements
    zeroed once (``batch * q_heads``: all query-head groups of a KV head share one launch)."""
    global launch_count
    d = kcache.shape[3]
    b, hq, hkv, smax = q.shape[0], q.shape[1] // d, kcache.shape[1], kcache.shape[2]
    out = torch.empty(b, hq, d, dtype=q.dtype, device=q.device) if out is None else out  # (rows may be column slices of a wider buffer)
    part_o = part_ml = counters = None
    if splits > 1:
        if workspace is None:
            workspace = (torch.empty(b * hq * splits * d, dtype=torch.float32, device=q.device),
                         torch.empty(b * hq * splits * 2, dtype=torch.float32, device=q.device),
                         torch.zeros(b * hq, dtype=torch.int32, device=q.device))
        part_o, part_ml, counters = workspace
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    check(LIB.tpb_attn_decode_fused(_ptr(q), _ptr(k), _ptr(v), _ptr(kcache), _ptr(vcache), _ptr(out), _ptr(part_o), _ptr(part_ml),
                                    _ptr(counters), _ptr(pos_ptr), b, hq, hkv, d, smax, splits, scale, rotary_dim, theta,
                                    int(interleaved), q.stride(0), k.stride(0), v.stride(0), _ptr(rope_angles),
                                    out.stride(0) if out.stride(0) != hq * d else 0, 0 if counters is None else counters.numel(), _stream()),
          "tpb_attn_decode_fused")
    launch_count += LIB.tpb_last_launches()
    return out


def qkv_rope_append(q, k, v, q_out, kcache, vcache, base_pos, batch, seq, rotary_dim, theta, interleaved=False):
    """Rotary-embed q / k of ``batch*seq`` new tokens and append k, v to the cache at ``base_pos[0] + s``.
    q / k / v are 2-D views ``[tokens, heads*head_dim]`` (column slices of one fused projection are fine)."""
    global launch_count
    d = kcache.shape[3]
    hq, hkv, smax = q.shape[1] // d, kcache.shape[1], kcache.shape[2]
    check(LIB.tpb_qkv_rope_append(_ptr(q), _ptr(k), _ptr(v), _ptr(q_out), _ptr(kcache), _ptr(vcache), _ptr(base_pos), batch, seq,
                                  hq, hkv, d, rotary_dim, theta, int(interleaved), smax, q.stride(0), k.stride(0), v.stride(0),
                                  _stream()), "tpb_qkv_rope_append")
    launch_count += 1
    return q_out


# ------------------------------------------------------------------------------------------------
# embedding / optimizer / casts
# ------------------------------------------------------------------------------------------------

LIB.tpb_embedding.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_ll, c_ll, c_int, c_void_p]
LIB.tpb_adamw.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_ll] + [c_float] * 5 + [c_int, c_float, c_int, c_int, c_void_p]
LIB.tpb_cast.argtypes = [c_void_p, c_void_p, c_ll, c_float, c_int, c_void_p]


def embedding(ids: torch.Tensor, table: torch.Tensor, out=None):
    global launch_count
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    cols = table.shape[1]
    if out is None:
        out = torch.empty(flat.numel(), cols, dtype=table.dtype, device=table.device)
    check(LIB.tpb_embedding(_ptr(flat), _ptr(table), _ptr(out), flat.numel(), cols, table.stride(0), out.stride(0), _dtype_code(table),
                            _stream()), "tpb_embedding")
    launch_count += 1
    return out.view(*ids.shape, cols) if out.shape[0] == flat.numel() and out.is_contiguous() else out


def adamw_step(param, grad, exp_avg, exp_avg_sq, step, lr, beta1, beta2, eps, weight_decay, master=None, grad_scale=1.0):
    global launch_count
    check(LIB.tpb_adamw(_ptr(param), _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq), _ptr(master), param.numel(), lr, beta1, beta2, eps,
                        weight_decay, step, grad_scale, _dtype_code(param), int(grad.dtype == torch.float32), _stream()), "tpb_adamw")
    launch_count += 1


LIB.tpb_last_cuda_error.argtypes = [ctypes.c_char_p, c_int]
