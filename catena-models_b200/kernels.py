"""Python face of the CUDA library: one function per entry point, taking torch tensors.

Every call launches on torch's current stream, checks the entry point's return code and
raises `KernelError` with the library's message.  There is no fallback: if the library
cannot be built or loaded, importing a kernel raises.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .csrc import build as _build
from .csrc import limits as _limits
from .csrc.limits import ATTN_DECODE_CHUNK, PAGE_TOKENS  # noqa: F401  (re-exported)

DT_F32, DT_BF16 = 0, 1

_vp, _i, _ll, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_SIGNATURES = {
    "cm_embed_gather": [_i, _i, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _vp, _vp],
    "cm_scale_softcap": [_vp, _ll, _f, _f, _vp],
    "cm_rmsnorm": [_i, _vp, _vp, _vp, _i, _i, _f, _ll, _ll, _vp],
    "cm_add_norm": [_i, _vp, _vp, _vp, _vp, _i, _ll, _vp, _vp, _vp, _i, _i, _f, _f, _vp],
    "cm_gemm_tc_few_rows_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _vp, _vp],
    "cm_gemm_skinny_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _ll, _i, _vp],
    "cm_swiglu": [_i, _vp, _vp, _i, _i, _i, _f, _vp],
    "cm_gather_rows": [_i, _vp, _vp, _vp, _i, _i, _vp],
    "cm_gemm_simt": [_i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _vp],
    "cm_gemm_skinny": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _f, _vp],
    "cm_gemm_tc": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _f, _vp],
    "cm_gemm_tc_few_rows": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _f, _vp],
    "cm_qk_prepare": [_i, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _i,
                      _i, _f, _i, _f, _i, _vp],
    "cm_attn_prefill_simt": [_i, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "cm_attn_prefill_mma": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _vp],
    "cm_attn_prefill_tc": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _i, _i, _ll, _i, _i, _i, _i, _f, _f, _vp, _vp, _vp],
    "cm_attn_decode": [_i, _vp, _ll, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _i, _i, _i, _i, _i, _i, _i,
                       _i, _f, _f, _vp, _vp, _vp, _vp],
    "cm_gemm_skinny_shortconv": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _ll, _ll, _ll, _vp],
    "cm_shortconv": [_i, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "cm_attn_append_simt": [_i, _vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i,
                            _i, _i, _i, _f, _f, _vp, _vp],
    "cm_attn_append_mma": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _i,
                           _i, _i, _f, _f, _vp, _vp],
    "cm_attn_append_tc": [_vp, _ll, _vp, _vp, _vp, _ll, _vp, _ll, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _ll, _i,
                          _i, _i, _i, _f, _f, _vp, _vp, _vp],
    "cm_gemm_tc_parts": [_vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _i, _vp, _vp],
    "cm_kv_store": [_i, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _ll, _vp, _ll, _i, _i, _i, _i, _vp],
    "cm_sample": [_vp, _vp, _ll, _i, _i, _vp, _vp, _vp, _vp, _vp],
    "cm_scatter_i32": [_vp, _vp, _vp, _vp, _i, _vp],
    "cm_zero_slots": [_vp, _i, _ll, _ll, ctypes.POINTER(ctypes.c_int), _i, _vp],
    "cm_copy_pages": [_vp, _vp, _vp, _i, _i, _ll, _ll, _vp],
    "cm_norm_f32in": [_i, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _vp, _vp],
    "cm_residual_add_norm": [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _vp, _vp],
    "cm_postnorm_residual": [_i, _vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _f, _vp, _i, _i, _f, _vp, _ll, _i, _vp, _vp],
    "cm_relu2_inplace": [_i, _vp, _ll, _vp],
    "cm_tap_rotate_store": [_i, _vp, _vp],
    "cm_diff_attn": [_i, _vp, _i, _i, _vp, _i, _vp],
    "cm_diff_attn_mma": [_vp, _i, _vp],
    "cm_concat_cast": [_i, _vp, _vp, _vp, _ll, _i, _vp],
    "cm_shift_mix": [_i, _vp, _vp, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _i, _ll, _i, _vp],
    "cm_lowrank_decay": [_i, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _f, _vp],
    "cm_capped_gates": [_i, _vp, _vp, _vp, _vp, _f, _ll, _i, _i, _vp],
    "cm_tanh_inplace": [_i, _vp, _ll, _vp],
    "cm_decay_from_logits": [_vp, _vp, _vp, _ll, _i, _i, _f, _vp],
    "cm_matrix_scan": [_i, _i, _vp, _i, _vp],
    "cm_lightning_chunked": [_i, _vp, _i, _i, _vp, _vp],
    "cm_moe_route": [_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _i, _i, _i, _f, _f, _i, _vp],
    "cm_moe_identity": [_i, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp],
    "cm_latent_prepare": [_i, _vp, _vp],
    "cm_latent_query_turn": [_i, _vp, _vp],
    "cm_latent_expand": [_i, _vp, _vp],
    "cm_latent_attn": [_i, _vp, _vp],
    "cm_latent_attn_mma": [_vp, _vp],
    "cm_head_linear": [_i, _vp, _vp, _vp, _ll, _i, _i, _i, _ll, _ll, _i, _i, _i, _i, _vp],
    "cm_moe_gather": [_i, _vp, _vp, _vp, _vp, _ll, _i, _i, _i, _vp],
    "cm_gemm_tc_grouped": [_i, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _vp, _i, _vp, _f, _vp],
    "cm_moe_grouped": [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _f, _vp],
}


class KernelError(RuntimeError):
    pass


_lib = None


class Timeline:
    """Times every launch of the library between `with kernels.Timeline() as t:` and its end, with a
    pair of CUDA events around each entry-point call, and keeps what the binding knows about the
    call: its name, the operands' shape and the bytes and floating-point operations that the
    operation needs by its definition (each operand once).  `rows()` adds the calls up by name
    and shape.  catena-models prints its own phase timers on request (CATENA_COMPILE_TIMINGS,
    src/catena.rs:82-87; per-phase rates, src/main.rs:364-371); this is that habit for kernels.
    Off unless entered: an ordinary run records no events.

    `in_graph=True` makes the events of a kind that may be recorded while a CUDA graph is captured and
    read after the graph has been replayed: the calls of a decode step are then timed inside the
    recorded step (`keep_last(n)` drops what was collected before the capture), where a kernel follows
    its predecessor as it does in production, instead of after the host's pause between two launches."""

    def __init__(self, in_graph=False):
        self.calls = []            # [name, shape, bytes, flops, start event, end event, launches]
        self._start = None
        self._event = ((lambda: torch.cuda.Event(enable_timing=True, external=True)) if in_graph
                       else (lambda: torch.cuda.Event(enable_timing=True)))

    def keep_last(self, n):
        self.calls = self.calls[-n:]

    def __enter__(self):
        global _timeline
        self._before, _timeline = _timeline, self
        return self

    def __exit__(self, *exc):
        global _timeline
        _timeline = self._before

    def begin(self):
        self._start = self._event()
        self._start.record()

    def end(self, name, n, cost):
        if self._start is None:
            return
        stop = self._event()
        stop.record()
        shape, nbytes, flops = cost() if cost is not None else ("", 0, 0)
        self.calls.append([name, shape, nbytes, flops, self._start, stop, n])
        self._start = None

    def rows(self):
        """[{name, shape, calls, launches, us, bytes, flops}] by name and shape, in order of first use
        (synchronises)."""
        torch.cuda.synchronize()
        out = {}
        for name, shape, nbytes, flops, a, b, n in self.calls:
            row = out.setdefault((name, shape), dict(name=name, shape=shape, calls=0, launches=0, us=0.0, bytes=0, flops=0))
            row["calls"] += 1
            row["launches"] += n
            row["us"] += a.elapsed_time(b) * 1e3
            row["bytes"] += nbytes
            row["flops"] += flops
        return list(out.values())


_timeline = None


def _nbytes(*tensors):
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


# ------------------------------------------------------------------ fused decode segments
FD_GEMV, FD_ADD_NORM, FD_CONV = 0, 1, 2
FD_PLAIN, FD_SWIGLU, FD_PARTS, FD_F32 = 0, 1, 2, 3
FD_MAX_ROWS = 16


class _FdOp(ctypes.Structure):
    """csrc/decode_fused.h: FdOp."""
    _fields_ = ([(n, ctypes.c_int) for n in ("kind", "mode", "M", "N", "K", "ksplit", "n_parts", "taps")]
                + [(n, ctypes.c_longlong) for n in ("ldx", "ldw", "ldy", "part_stride")]
                + [(n, ctypes.c_void_p) for n in ("x", "w", "y", "aux0", "aux1", "aux2", "aux3", "idx")]
                + [("eps0", ctypes.c_float), ("eps1", ctypes.c_float), ("pad0", ctypes.c_int), ("pad1", ctypes.c_int)])


class FusedDecode:
    """While entered, the calls of a decode step that the fused kernel knows (`gemm_skinny` and its
    forms, `add_norm`, the short convolution's decode form; bfloat16, at most 16 rows) are not
    launched but collected, in program order, and run as ONE cooperative launch (`cm_fused_decode`)
    as soon as a call comes that the kernel does not know, when the kernel's table is full, or at
    the end.  Memory that the collected calls use stays referenced until they have been launched.
    `bar`: the kernel's barrier word (uint32 zero on the device); `err`: the device flag that a
    block raises when its wait at the barrier runs out."""

    def __init__(self, bar, err):
        self.bar, self.err = bar, err
        self.ops, self.keep = [], []
        self.max_ops = lib().cm_fused_decode_max_ops()
        self.max_width = lib().cm_fused_decode_max_width()
        self._flushing = False

    def __enter__(self):
        global _fuser
        self._before, _fuser = _fuser, self
        return self

    def __exit__(self, exc_type, *exc):
        global _fuser
        try:
            if exc_type is None:
                self.flush()
        finally:
            _fuser = self._before
            self.ops, self.keep = [], []

    def add(self, keep, **fields):
        op = _FdOp()
        for k, v in fields.items():
            setattr(op, k, v)
        self.ops.append(op)
        self.keep.extend(keep)
        if len(self.ops) >= self.max_ops:
            self.flush()

    def flush(self):
        if not self.ops or self._flushing:
            return
        self._flushing = True
        try:
            n = len(self.ops)
            seg = (ctypes.c_int * 4)(n, 0, 0, 0)
            blob = bytes(seg) + b"".join(bytes(op) for op in self.ops)
            blob += b"\0" * (16 + self.max_ops * ctypes.sizeof(_FdOp) - len(blob))
            ops, self.ops, self.keep = self.ops, [], []
            _check(lib().cm_fused_decode(blob, _ptr(self.bar), _ptr(self.err), _stream()), "fused_decode",
                   cost=lambda: (f"{n} operations", 0, 0))
        finally:
            self._flushing = False


_fuser = None


def _fusable_rows(x, w):
    """x @ w^T can join a fused segment: bfloat16, at most 16 rows, 16-byte aligned rows."""
    return (_fuser is not None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= FD_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1
            and w.stride(1) == 1 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def lib():
    """The loaded CUDA library, with argument types set."""
    global _lib
    if _fuser is not None and _fuser.ops and not _fuser._flushing:
        _fuser.flush()             # a call that is launched on its own: what was collected runs before it
    if _timeline is not None and _lib is not None:
        _timeline.begin()          # every binding asks for the library right before its launch
    if _lib is None:
        handle = _build.load()
        handle.cm_last_error.restype = ctypes.c_char_p
        _limits.check_library(handle)
        for name, args in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = _i
        handle.cm_set_pdl.argtypes = [_i]
        handle.cm_set_pdl.restype = None
        handle.cm_fused_decode.argtypes = [ctypes.c_char_p, _vp, _vp, _vp]
        handle.cm_fused_decode.restype = _i
        if os.environ.get("CATENA_B200_PDL", "1") == "0":
            handle.cm_set_pdl(0)
        _lib = handle
    return _lib


def set_pdl(on):
    """Programmatic dependent launch for every kernel of the library (on by default; the
    environment variable CATENA_B200_PDL=0 turns it off at load)."""
    lib().cm_set_pdl(1 if on else 0)


def library_path():
    return lib()._name


def dtype_code(dtype):
    if dtype == torch.float32:
        return DT_F32
    if dtype == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"no kernels for dtype {dtype}")


def _ptr(t):
    return None if t is None else t.data_ptr()


_pinned_stream = None


def _stream():
    if _pinned_stream is not None:
        return _pinned_stream
    return torch.cuda.current_stream().cuda_stream


class pinned_stream:
    """Within this context every kernel of the library is launched on the stream that was current
    when it was entered, looked up once instead of once per launch (the lookup costs several
    microseconds, as much as a launch).  The caller must not change the current stream inside."""

    def __enter__(self):
        global _pinned_stream
        self._before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self._before


launches = 0          # kernels launched (or recorded into a graph) by this process, counted per call


def _check(code, name, n=1, cost=None):
    """`cost`: a callable that gives (shape text, bytes, floating-point operations) of the call; it is
    evaluated only while a Timeline records."""
    global launches
    launches += n
    if _timeline is not None:
        _timeline.end(name, n, cost)
    if code != 0:
        raise KernelError(f"{name} returned {code}: {_lib.cm_last_error().decode(errors='replace')}")


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels take CUDA tensors only; there is no CPU path")


# ---------------------------------------------------------------------------- row-wise
def embed_gather(out, table, tokens, err=None, sampled=None, scale=1.0):
    """out[t] = table[tokens[t]] * scale; with `sampled` (int32 device tensor) an entry -(1 + i) of
    tokens stands for sampled[i]."""
    _need_cuda(out, table, tokens)
    T, H = out.shape
    _check(lib().cm_embed_gather(dtype_code(out.dtype), dtype_code(table.dtype), _ptr(out), _ptr(table), _ptr(tokens),
                                 _ptr(sampled), T, H, table.shape[0], scale, _ptr(err), _stream()), "embed_gather",
           cost=lambda: (f"{T}x{H}", T * H * table.element_size() + _nbytes(out, tokens), 0))


def rmsnorm(out, x, w, eps):
    _need_cuda(out, x, w)
    rows, H = x.shape
    _check(lib().cm_rmsnorm(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(w), rows, H, eps, x.stride(0),
                            out.stride(0), _stream()), "rmsnorm",
           cost=lambda: (f"{rows}x{H}", _nbytes(x, out, w), 4 * rows * H))


class PartialSums:
    """A product x @ w^T left as float partial sums over slices of its inner dimension:
    `parts` [slices, rows, width].  Whoever consumes it adds the slices in index order and rounds
    the total to the activation dtype (`add_norm` does both while it reads them)."""

    def __init__(self, parts, dtype):
        self.parts, self.dtype = parts, dtype

    @property
    def shape(self):
        return self.parts.shape[1:]


class Terms(list):
    """What a sublayer adds to a float32 residual stream: (tensor, factor, pieces per row[, index[, weights]])
    entries; the tensor holds a row's pieces one below the other (rows * pieces rows), or anywhere, with `index`
    (int32 [rows * pieces], negative: no piece) saying where; `weights` (float32 [rows * pieces]): a factor on
    each piece; float32 or the activation dtype (`residual_add_norm`, `postnorm_residual`)."""


def add_norm(h_out, n_out, m, h_in, w_post, w_next, eps_post, eps_next):
    """h_out = h_in + (norm(m; w_post) or m); n_out = norm(h_out; w_next) when w_next is given.
    m: a tensor, or the PartialSums a product left."""
    if (_fuser is not None and h_in.dtype == torch.bfloat16 and h_in.shape[0] <= FD_MAX_ROWS and h_in.shape[1] % 8 == 0
            and h_in.shape[1] <= _fuser.max_width and h_in.is_contiguous() and h_out.is_contiguous()
            and (n_out is None or n_out.is_contiguous())):
        rows, H = h_in.shape
        if isinstance(m, PartialSums):
            src, n_parts, stride = m.parts, m.parts.shape[0], rows * H
            ok = src.dtype == torch.float32 and src.is_contiguous() and n_parts <= 8
        else:
            src, n_parts, stride = m, 0, 0
            ok = m.dtype == torch.bfloat16 and m.is_contiguous()
        if ok:
            _fuser.add((h_out, n_out, src, h_in, w_post, w_next), kind=FD_ADD_NORM, M=rows, N=H, n_parts=n_parts,
                       part_stride=stride, x=_ptr(h_in), y=_ptr(h_out), aux0=_ptr(src), aux1=_ptr(w_post),
                       aux2=_ptr(w_next), aux3=_ptr(n_out), eps0=eps_post, eps1=eps_next)
            return
    if isinstance(m, PartialSums):
        parts = m.parts
        _need_cuda(h_out, parts, h_in)
        n_parts, rows, H = parts.shape
        if parts.dtype != torch.float32 or not parts.is_contiguous():
            raise KernelError("add_norm: partial sums must be contiguous float32")
        _check(lib().cm_add_norm(dtype_code(h_in.dtype), _ptr(h_out), _ptr(n_out), None, _ptr(parts), n_parts, rows * H,
                                 _ptr(h_in), _ptr(w_post), _ptr(w_next), rows, H, eps_post, eps_next, _stream()),
               "add_norm", cost=lambda: (f"{rows}x{H} over {n_parts} partial sums",
                                         _nbytes(parts, h_in, h_out, n_out, w_post, w_next), (n_parts + 8) * rows * H))
        return
    _need_cuda(h_out, m, h_in)
    rows, H = m.shape
    _check(lib().cm_add_norm(dtype_code(m.dtype), _ptr(h_out), _ptr(n_out), _ptr(m), None, 0, 0, _ptr(h_in), _ptr(w_post),
                             _ptr(w_next), rows, H, eps_post, eps_next, _stream()), "add_norm",
           cost=lambda: (f"{rows}x{H}", _nbytes(m, h_in, h_out, n_out, w_post, w_next), 8 * rows * H))


def scale_softcap(logits, scale=1.0, cap=0.0):
    """logits <- cap * tanh(logits * scale / cap) (cap > 0) or logits * scale, in place; float32."""
    if logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelError("scale_softcap takes contiguous float32 logits")
    _check(lib().cm_scale_softcap(_ptr(logits), logits.numel(), scale, cap, _stream()), "scale_softcap")


ACT_SILU, ACT_GELU_TANH, ACT_CLAMPED_SWISH = 0, 1, 2       # csrc/common.cuh: gated_act
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH, "clamped_swish": ACT_CLAMPED_SWISH}


def swiglu(out, gate_up, gelu=False, act=None, limit=0.0):
    """out = act(gate, up) for the packed contiguous rows [gate | up].  act: ACT_SILU silu(g) u (the default), ACT_GELU_TANH
    (or `gelu`) the tanh form of gelu on g, times u; ACT_CLAMPED_SWISH: with g' = min(g, limit) and u' = clamp(u, -limit,
    limit), g' sigmoid(1.702 g') (u' + 1)."""
    rows, F = out.shape
    act = (ACT_GELU_TANH if gelu else ACT_SILU) if act is None else int(act)
    if not gate_up.is_contiguous() or gate_up.shape != (rows, 2 * F) or not out.is_contiguous():
        raise KernelError("swiglu: contiguous rows [gate | up]")
    _check(lib().cm_swiglu(dtype_code(out.dtype), _ptr(out), _ptr(gate_up), rows, F, act, float(limit), _stream()), "swiglu",
           cost=lambda: (f"{rows}x{F}", _nbytes(out, gate_up), 8 * rows * F))


def gather_rows(out, x, rows):
    n, H = out.shape
    _check(lib().cm_gather_rows(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(rows), n, H, _stream()),
           "gather_rows")


# ------------------------------------------------------------------------------- gemm
def gemm_simt(y, x, w):
    """y[M,N] = x[M,K] @ w[N,K]^T on the CUDA cores (float accumulation)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or tuple(y.shape) != (M, N):
        raise KernelError(f"gemm shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    _check(lib().cm_gemm_simt(dtype_code(x.dtype), dtype_code(w.dtype), dtype_code(y.dtype), _ptr(y), _ptr(x),
                              _ptr(w), M, N, K, x.stride(0), w.stride(0), y.stride(0), _stream()), "gemm_simt",
           cost=lambda: (f"{M}x{N}x{K}", _nbytes(x, w, y), 2 * M * N * K))


_GATE_SUFFIX = ("", "_swiglu", "_geglu", "_clamped")     # a product's name by its gate flag


def gemm_skinny(y, x, w, swiglu=False, limit=0.0):
    """y = x @ w^T for at most 64 bfloat16 rows, weights streamed once (mma.sync, float sums).
    swiglu: w is [gate; up] with 2F rows and y[M, F] = silu(x Wgate^T) * (x Wup^T); swiglu=2 (all products that
    take the flag): the tanh form of gelu in silu's place; swiglu=3 with `limit` L: the clamped gate, g' sigmoid(1.702 g')
    (u' + 1) with g' = min(g, L), u' = clamp(u, -L, L)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_skinny shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny takes bfloat16 operands")
    if (_fusable_rows(x, w) and y.stride(1) == 1 and int(swiglu) < 2
            and (y.dtype == torch.bfloat16 or (y.dtype == torch.float32 and not swiglu))):
        mode = FD_SWIGLU if swiglu else (FD_PLAIN if y.dtype == torch.bfloat16 else FD_F32)
        _fuser.add((y, x, w), kind=FD_GEMV, mode=mode, M=M, N=N, K=K, ksplit=1, ldx=x.stride(0), ldw=w.stride(0),
                   ldy=y.stride(0), x=_ptr(x), w=_ptr(w), y=_ptr(y))
        return
    _check(lib().cm_gemm_skinny(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                                y.stride(0), int(swiglu), float(limit), _stream()), "gemm_skinny" + _GATE_SUFFIX[int(swiglu)],
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


def gemm_skinny_parts(parts, x, w):
    """parts[s] = x[:, slice s of K] @ w[:, slice s of K]^T in float, for at most 16 bfloat16 rows:
    the weight-streaming product with K cut over parts.shape[0] independent groups of blocks."""
    _need_cuda(parts, x, w)
    M, K = x.shape
    S, _, N = parts.shape
    if w.shape != (N, K) or parts.shape[1] != M or parts.dtype != torch.float32 or not parts.is_contiguous():
        raise KernelError(f"gemm_skinny_parts shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, parts {tuple(parts.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_skinny_parts takes bfloat16 operands")
    if _fusable_rows(x, w) and S <= 8:
        _fuser.add((parts, x, w), kind=FD_GEMV, mode=FD_PARTS, M=M, N=N, K=K, ksplit=S, ldx=x.stride(0), ldw=w.stride(0),
                   ldy=N, part_stride=M * N, x=_ptr(x), w=_ptr(w), y=_ptr(parts))
        return
    _check(lib().cm_gemm_skinny_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), N, M * N, S,
                                      _stream()), "gemm_skinny_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} slices", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc_few_rows_parts(parts, x, w, err=None):
    """The same from the tcgen05 few-rows product (at most 128 bfloat16 rows): parts[s] holds the
    float sums over the s-th slice of K; no exchange between the blocks of a column tile."""
    _need_cuda(parts, x, w)
    M, K = x.shape
    S, _, N = parts.shape
    if w.shape != (N, K) or parts.shape[1] != M or parts.dtype != torch.float32 or not parts.is_contiguous():
        raise KernelError(f"gemm_tc_few_rows_parts shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, parts {tuple(parts.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_tc_few_rows_parts takes row-major bfloat16 operands")
    _check(lib().cm_gemm_tc_few_rows_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), M * N, S,
                                           _ptr(err), _stream()), "gemm_tc_few_rows_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} slices", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc_parts(parts, x, w, err=None, block_n=256):
    """parts[r] = x @ w^T over the r-th of parts.shape[0] runs of the inner dimension, float32
    [runs, rows, width] contiguous: the tiled tcgen05 product for a few hundred rows times a narrow
    output, cut over K so that its (run, tile) items occupy the device; no exchange between blocks,
    the consumer adds the runs in order (`add_norm` takes them as `PartialSums`)."""
    _need_cuda(parts, x, w)
    S, M, N = parts.shape
    if parts.dtype != torch.float32 or not parts.is_contiguous() or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_parts: contiguous float32 partial sums of a bfloat16 product")
    if x.shape[0] != M or w.shape[0] != N or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tc_parts: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(parts.shape)}")
    K = x.shape[1]
    _check(lib().cm_gemm_tc_parts(_ptr(parts), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0), S, block_n, _ptr(err),
                                  _stream()), "gemm_tc_parts",
           cost=lambda: (f"{M}x{N}x{K} in {S} runs", _nbytes(x, w, parts), 2 * M * N * K))


def gemm_tc(y, x, w, swiglu=False, err=None, block_n=256, limit=0.0):
    """y = x @ w^T on the tcgen05 tensor cores (TMA-fed, accumulator in tensor memory), any
    number of bfloat16 rows.  swiglu: w is [gate; up] with 2F rows and y[M, F] = silu(g) * u.
    err: device int32 that a block raises if one of its bounded pipeline waits runs out.
    block_n: 256 (128 x 256 tiles), 128 (twice as many 128 x 128 tiles, for few rows) or 192 (plain
    bfloat16 products only)."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_tc shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc takes bfloat16 operands")
    if x.stride(1) != 1 or w.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gemm_tc takes row-major operands")
    _check(lib().cm_gemm_tc(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(0),
                            y.stride(0), int(swiglu), block_n, _ptr(err), float(limit), _stream()), "gemm_tc" + _GATE_SUFFIX[int(swiglu)],
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


def gemm_tc_few_rows(y, x, w, swiglu=False, err=None, splits=0, limit=0.0):
    """gemm_tc for at most 128 rows.  When the product has too few 128-column tiles for the
    device, K is split over a thread-block cluster of up to 8 blocks that add their partial
    sums through distributed shared memory.  splits: 0 chooses, 1..8 forces."""
    _need_cuda(y, x, w)
    M, K = x.shape
    N = y.shape[1]
    if w.shape[1] != K or w.shape[0] != (2 * N if swiglu else N) or y.shape[0] != M:
        raise KernelError(f"gemm_tc_few_rows shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tc_few_rows takes bfloat16 operands")
    if x.stride(1) != 1 or w.stride(1) != 1 or y.stride(1) != 1:
        raise KernelError("gemm_tc_few_rows takes row-major operands")
    _check(lib().cm_gemm_tc_few_rows(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0),
                                     w.stride(0), y.stride(0), int(swiglu), splits, _ptr(err), float(limit), _stream()),
           "gemm_tc_few_rows" + _GATE_SUFFIX[int(swiglu)],
           cost=lambda: (f"{M}x{w.shape[0]}x{K}", _nbytes(x, w, y), 2 * M * w.shape[0] * K))


# -------------------------------------------------------------------------- attention
def qk_prepare(qkv, wq, wk, rate, tok_pos, tok_seq, seq_slot, seq_end, pool, pages, ptab, ring,
               QH, KVH, HD, eps, interleaved=False, q_temp=None):
    """Head norm + rotation in place on the q and k columns of qkv; k and v go to the cache
    (pool: this layer's [2, pages, KVH, 64, HD] storage, or None to write no cache).  The rotation
    pairs element i with i + HD/2, or, with `interleaved`, 2i with 2i + 1.  `q_temp` = (coef, every):
    the queries at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)."""
    qt_coef, qt_every = (float(q_temp[0]), int(q_temp[1])) if q_temp else (0.0, 0)
    T = qkv.shape[0]
    _check(lib().cm_qk_prepare(dtype_code(qkv.dtype), _ptr(qkv), qkv.stride(0), _ptr(wq), _ptr(wk), _ptr(rate),
                               _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot), _ptr(seq_end), _ptr(pool), pages,
                               _ptr(ptab), 0 if ptab is None else ptab.stride(0), ring, T, QH, KVH, HD, eps,
                               int(interleaved), qt_coef, qt_every, _stream()), "qk_prepare",
           cost=lambda: (f"{T} tokens, {QH}+{KVH} heads of {HD}",
                         T * HD * qkv.element_size() * (2 * QH + (2 * KVH if pool is None else 4 * KVH)), 0))


def attn_prefill_simt(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale, sink=None, softcap=0.0):
    """q, k, v, gate are column views of one packed row-major buffer (same row stride).  `sink` (all
    attention kernels): float32 [QH], a learned logit per query head that joins the softmax's denominator
    and nothing else (it has no key and no value), or None.  `softcap` (all attention kernels) = c > 0: every
    score is bounded before the mask and the softmax, s <- c * tanh(s / c) with s = (q . k) * scale."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("attn_prefill: q, k and v must share a row stride")
    _check(lib().cm_attn_prefill_simt(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v),
                                      q.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0),
                                      _ptr(seq_start), B, max_len, QH, KVH, HD, window, scale, softcap, _ptr(sink), _stream()),
           "attn_prefill_simt",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def attn_prefill_mma(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale, sink=None, softcap=0.0):
    """The same on the tensor cores: bfloat16, head sizes that are multiples of 16 up to 128."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_mma: bfloat16 q, k and v that share a row stride")
    _check(lib().cm_attn_prefill_mma(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                     0 if gate is None else gate.stride(0), _ptr(seq_start), B, max_len, QH, KVH,
                                     HD, window, scale, softcap, _ptr(sink), _stream()), "attn_prefill_mma",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def attn_append(ctx, q, k, v, gate, seq_start, seq_pos0, seq_slot, pool, pages, ptab, ring, B, max_len, QH, KVH, HD,
                window, scale, tensor_cores=True, sink=None, softcap=0.0):
    """Attention of a step whose sequences may stand at seq_pos0[b] > 0: keys and values below that
    position come from the paged cache `pool`, the rest from the step's own rows (q, k, v as for the
    prefill kernels), which the caller writes to the cache afterwards (`kv_store`).  bfloat16 with a
    head size that is a multiple of 16 up to 128 runs on the tensor cores unless `tensor_cores` is off."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)):
        raise KernelError("attn_append: q, k and v must share a row stride")
    mma = (tensor_cores and q.dtype == torch.bfloat16 and HD % 16 == 0 and HD <= 128 and q.stride(0) % 8 == 0
           and (q.data_ptr() | k.data_ptr() | v.data_ptr() | pool.data_ptr()) % 16 == 0)
    common = (_ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0), _ptr(seq_start),
              _ptr(seq_pos0), _ptr(seq_slot), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, B, max_len, QH, KVH,
              HD, window, scale, softcap, _ptr(sink), _stream())
    if mma:
        _check(lib().cm_attn_append_mma(_ptr(ctx), ctx.stride(0), *common), "attn_append_mma")
    else:
        _check(lib().cm_attn_append_simt(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), *common), "attn_append_simt")


def attn_append_tc(ctx, q, k, v, gate, seq_start, seq_pos0, seq_slot, pool, pages, ptab, ring, B, max_len, QH, KVH, HD,
                   window, scale, err=None, sink=None, softcap=0.0):
    """`attn_append` on the tcgen05 tensor cores: bfloat16, head size 64 or 128, the cache read page by
    page with TMA.  err: device int32 that a block raises if a bounded pipeline wait runs out."""
    if (not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16
            or q.shape[0] != k.shape[0]):
        raise KernelError("attn_append_tc: bfloat16 q, k, v and cache; q, k and v share rows and a row stride")
    if not pool.is_contiguous() or tuple(pool.shape[2:]) != (KVH, PAGE_TOKENS, HD):
        raise KernelError(f"attn_append_tc: the cache must be contiguous [2, pages, {KVH}, {PAGE_TOKENS}, {HD}]")
    _check(lib().cm_attn_append_tc(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                   0 if gate is None else gate.stride(0), _ptr(seq_start), _ptr(seq_pos0),
                                   _ptr(seq_slot), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, B, max_len,
                                   q.shape[0], QH, KVH, HD, window, scale, softcap, _ptr(sink), _ptr(err), _stream()), "attn_append_tc",
           cost=lambda: (f"{B} sequences of up to {max_len} rows, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def kv_store(kv, tok_pos, tok_seq, seq_slot, seq_end, pool, pages, ptab, ring, KVH, HD):
    """kv: the k | v columns [T, 2 * KVH * HD] of the step's packed rows (k normed and rotated);
    writes them to the cache entries of their positions (a ring keeps the last `ring` of a sequence)."""
    T = kv.shape[0]
    _check(lib().cm_kv_store(dtype_code(kv.dtype), _ptr(kv), kv.stride(0), _ptr(tok_pos), _ptr(tok_seq), _ptr(seq_slot),
                             _ptr(seq_end), _ptr(pool), pages, _ptr(ptab), ptab.stride(0), ring, T, KVH, HD, _stream()),
           "kv_store")


def attn_prefill_tc(ctx, q, k, v, gate, seq_start, B, max_len, QH, KVH, HD, window, scale, err=None, sink=None, softcap=0.0):
    """The same on the tcgen05 tensor cores (TMA-fed, scores and outputs in tensor memory): bfloat16,
    head size 64 or 128.  q, k and v are column blocks of one row-major buffer.  err: device int32
    that a block raises if one of its bounded pipeline waits runs out."""
    if not (q.stride(0) == k.stride(0) == v.stride(0)) or q.dtype != torch.bfloat16 or q.shape[0] != k.shape[0]:
        raise KernelError("attn_prefill_tc: bfloat16 q, k and v that share rows and a row stride")
    _check(lib().cm_attn_prefill_tc(_ptr(ctx), ctx.stride(0), _ptr(q), _ptr(k), _ptr(v), q.stride(0), _ptr(gate),
                                    0 if gate is None else gate.stride(0), _ptr(seq_start), B, max_len, q.shape[0],
                                    QH, KVH, HD, window, scale, softcap, _ptr(sink), _ptr(err), _stream()), "attn_prefill_tc",
           cost=lambda: (f"{B} sequences up to {max_len}, {QH}/{KVH} heads of {HD}, window {window}", 0, 0))


def set_decode_attention_target_blocks(blocks):
    """Blocks the tensor-core decode attention aims at (0: chosen from the amount of work, the
    default).  With fewer, each block walks several 256-entry chunks of a sequence."""
    lib().cm_attn_decode_set_target_blocks(int(blocks))


def set_decode_attention_tensor_cores(on):
    """bfloat16 decode attention normally runs its first stage on the tensor cores when the head
    size allows it; off forces the CUDA-core stage (tests compare the two)."""
    lib().cm_attn_decode_set_mma.argtypes = [_i]
    lib().cm_attn_decode_set_mma.restype = None
    lib().cm_attn_decode_set_mma(1 if on else 0)


def attn_decode_scratch(B, QH, HD, n_chunks, device):
    return (torch.empty(B * QH * n_chunks * HD, dtype=torch.float32, device=device),
            torch.empty(B * QH * n_chunks * 2, dtype=torch.float32, device=device))


def attn_decode(ctx, q, gate, seq_pos, seq_slot, pool, pages, ptab, ring, window, QH, KVH, HD, n_chunks,
                scale, part_o, part_ml, sink=None, softcap=0.0):
    B = q.shape[0]
    _check(lib().cm_attn_decode(dtype_code(q.dtype), _ptr(ctx), ctx.stride(0), _ptr(q), q.stride(0), _ptr(gate),
                                0 if gate is None else gate.stride(0), _ptr(seq_pos), _ptr(seq_slot), _ptr(pool),
                                pages, _ptr(ptab), ptab.stride(0), ring, window, B, QH, KVH, HD, n_chunks, scale, softcap,
                                _ptr(part_o), _ptr(part_ml), _ptr(sink), _stream()), "attn_decode", 2,
           cost=lambda: (f"{B} sequences, {QH}/{KVH} heads of {HD}, window {window}, {n_chunks} chunks", 0, 0))


# -------------------------------------------------------------------------- short conv
def shortconv(y, bcx, w, state, tok_seq, seq_start, seq_slot, K, from_zero, one_token_each, w_t=None, seq_pos0=None):
    """w: taps [H, K]; w_t: the same stored [K, H] (optional, for 16-byte reads of the taps).
    from_zero: every sequence starts from an empty state; one_token_each: a decode step.  Neither:
    several tokens on top of the stored state (two launches: outputs, then the state); seq_pos0
    (first position per sequence) then lets a sequence that stands at 0 start from an empty state."""
    T, H = y.shape
    two = not from_zero and not one_token_each
    _check(lib().cm_shortconv(dtype_code(y.dtype), _ptr(y), _ptr(bcx), bcx.stride(0), _ptr(w), _ptr(w_t), _ptr(state),
                              _ptr(tok_seq), _ptr(seq_start), _ptr(seq_slot), _ptr(seq_pos0), T, H, K, int(from_zero),
                              int(one_token_each), _stream()), "shortconv", 2 if two else 1,
           cost=lambda: (f"{T}x{H}, {K} taps", _nbytes(bcx, y), 2 * (K + 1) * T * H))


def gemm_skinny_shortconv(y, x, w_in, taps, state, seq_slot):
    """A decode step's in_proj and short convolution in one kernel: x [M <= 16, K] and w_in [3H, K]
    bfloat16 (rows B | C | X), taps [H, KT] float, state [slots, KT - 1, H] float (shifted in
    place), seq_slot [M]; y [M, H] bfloat16."""
    _need_cuda(y, x, w_in)
    M, K = x.shape
    H, KT = taps.shape
    if w_in.shape != (3 * H, K) or y.shape != (M, H) or state.shape[1:] != (KT - 1, H):
        raise KernelError(f"gemm_skinny_shortconv shapes: x {tuple(x.shape)}, w {tuple(w_in.shape)}, "
                          f"y {tuple(y.shape)}, taps {tuple(taps.shape)}, state {tuple(state.shape)}")
    if not (x.dtype == w_in.dtype == y.dtype == torch.bfloat16 and taps.dtype == state.dtype == torch.float32):
        raise KernelError("gemm_skinny_shortconv takes bfloat16 operands, float taps and state")
    if not (taps.is_contiguous() and state.is_contiguous()):
        raise KernelError("gemm_skinny_shortconv: taps and state must be contiguous")
    if _fusable_rows(x, w_in) and H % 8 == 0 and y.stride(0) % 8 == 0 and y.data_ptr() % 16 == 0:
        # in the fused kernel: in_proj as a product of its own, then the convolution over its output
        bcx = torch.empty((M, 3 * H), dtype=torch.bfloat16, device=x.device)
        _fuser.add((bcx, x, w_in), kind=FD_GEMV, mode=FD_PLAIN, M=M, N=3 * H, K=K, ksplit=1, ldx=x.stride(0),
                   ldw=w_in.stride(0), ldy=3 * H, x=_ptr(x), w=_ptr(w_in), y=_ptr(bcx))
        _fuser.add((y, taps, state, seq_slot), kind=FD_CONV, M=M, N=H, taps=KT, ldx=3 * H, ldy=y.stride(0), x=_ptr(bcx),
                   y=_ptr(y), aux0=_ptr(taps), aux3=_ptr(state), idx=_ptr(seq_slot))
        return
    _check(lib().cm_gemm_skinny_shortconv(_ptr(y), _ptr(x), _ptr(w_in), _ptr(taps), _ptr(state), _ptr(seq_slot), M, H,
                                          K, KT, x.stride(0), w_in.stride(0), y.stride(0), _stream()),
           "gemm_skinny_shortconv",
           cost=lambda: (f"{M}x{3 * H}x{K}", _nbytes(x, w_in, y, taps) + 2 * M * (KT - 1) * H * 4, 2 * M * 3 * H * K))


# ---------------------------------------------------------------------------- sampling
def sample(out, logits, temperature, sequence, step, seed_words):
    n, V = logits.shape
    _check(lib().cm_sample(_ptr(out), _ptr(logits), logits.stride(0), n, V, _ptr(temperature), _ptr(sequence),
                           _ptr(step), _ptr(seed_words), _stream()), "sample",
           cost=lambda: (f"{n}x{V}", n * V * 4, 0))


# ------------------------------------------------------------------------------- cache
def scatter_i32(table, index, value, count, max_count):
    _check(lib().cm_scatter_i32(_ptr(table), _ptr(index), _ptr(value), _ptr(count), max_count, _stream()),
           "scatter_i32")


def copy_pages(pool, src, dst):
    """pool: [layers, planes, pages, ...] paged storage of one group; page src[i] is copied to page dst[i]
    in every layer and plane (int32 device tensors of equal length)."""
    n = src.numel()
    outer, pages = pool.shape[0] * pool.shape[1], pool.shape[2]
    page_bytes = pool[0, 0, 0].numel() * pool.element_size()
    _check(lib().cm_copy_pages(_ptr(pool), _ptr(src), _ptr(dst), n, outer, pages, page_bytes, _stream()), "copy_pages")


def zero_slots(store, slots):
    """store: [layers, slots, ...] fixed-size states (32-bit words or pairs of 16-bit); clears the rows
    of the given slots (Python ints) in every layer."""
    if not slots:
        return
    layers, total = store.shape[0], store.shape[1]
    row_bytes = store[0, 0].numel() * store.element_size()
    ids = (ctypes.c_int * len(slots))(*slots)
    n_launches = -(-len(slots) // 64)
    _check(lib().cm_zero_slots(_ptr(store), layers, total, row_bytes, ids, len(slots), _stream()), "zero_slots", n_launches)


# ------------------------------------------------------------------ float residual stream
NORM_RMS, NORM_DYT = 0, 1          # csrc/residual32.cu


def norm_f32in(out, x, w, eps, dyt=None):
    """out = norm(x) * w for float32 rows x; out in the activation dtype.  `dyt` = (alpha, shift): a dynamic
    tanh instead, out = tanh(alpha x) * w + shift (alpha a float32 tensor of one element, shift float32 [H])."""
    _need_cuda(out, x, w)
    rows, H = x.shape
    if x.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("norm_f32in takes contiguous float32 rows")
    kind, alpha, shift = (NORM_DYT, dyt[0], dyt[1]) if dyt is not None else (NORM_RMS, None, None)
    _check(lib().cm_norm_f32in(dtype_code(out.dtype), _ptr(out), _ptr(x), _ptr(w), rows, H, eps, kind, _ptr(alpha),
                               _ptr(shift), _stream()), "norm_f32in",
           cost=lambda: (f"{rows}x{H}", _nbytes(x, out, w), 4 * rows * H))


def relu2_inplace(x):
    """x <- max(x, 0)^2, in x's dtype (contiguous)."""
    if not x.is_contiguous():
        raise KernelError("relu2_inplace takes a contiguous tensor")
    _check(lib().cm_relu2_inplace(dtype_code(x.dtype), _ptr(x), x.numel(), _stream()), "relu2_inplace",
           cost=lambda: (f"{tuple(x.shape)}", 2 * _nbytes(x), 0))


def _term_arrays(terms, rows, H, act, name):
    """The parallel arrays that the residual kernels take for up to four terms."""
    if len(terms) > 4:
        raise KernelError(f"{name}: at most four terms")
    terms = [tuple(t) + (None,) * (5 - len(t)) for t in terms]
    for t, _, per_row, index, weights in terms:
        fits = t.numel() == rows * per_row * H if index is None else (index.numel() == rows * per_row and t.shape[-1] == H)
        if not t.is_contiguous() or not fits or t.dtype not in (torch.float32, act):
            raise KernelError(f"{name}: a term's shape or dtype does not fit")
        if weights is not None and (weights.dtype != torch.float32 or weights.numel() != rows * per_row):
            raise KernelError(f"{name}: a term's weights are float32, one per piece")
    n = len(terms)
    ptrs = (ctypes.c_void_p * 4)(*[t[0].data_ptr() for t in terms], *([None] * (4 - n)))
    scales = (ctypes.c_float * 4)(*[float(t[1]) for t in terms], *([0.0] * (4 - n)))
    per = (ctypes.c_int * 4)(*[int(t[2]) for t in terms], *([0] * (4 - n)))
    f32 = (ctypes.c_int * 4)(*[int(t[0].dtype == torch.float32) for t in terms], *([0] * (4 - n)))
    index = (ctypes.c_void_p * 4)(*[_ptr(t[3]) for t in terms], *([None] * (4 - n)))
    weights = (ctypes.c_void_p * 4)(*[_ptr(t[4]) for t in terms], *([None] * (4 - n)))
    return terms, n, ptrs, scales, per, f32, index, weights


def residual_add_norm(h, terms, n_out=None, w_next=None, eps=0.0, bias=None, dyt=None):
    """h (float32, in place) += sum over `terms` of scale * (the sum of a row's pieces) (+ bias, a float32
    row); n_out = norm(h) * w_next in the activation dtype when given (`dyt` = (alpha, shift): a dynamic tanh,
    as for `norm_f32in`).  A term is (tensor, scale, pieces per row[, index[, weights]]): see `Terms`."""
    rows, H = h.shape
    if h.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("residual_add_norm: a contiguous float32 stream")
    act = n_out.dtype if n_out is not None else next((t[0].dtype for t in terms if t[0].dtype != torch.float32), torch.float32)
    terms, n, ptrs, scales, per, f32, index, weights = _term_arrays(terms, rows, H, act, "residual_add_norm")
    kind, alpha, shift = (NORM_DYT, dyt[0], dyt[1]) if dyt is not None else (NORM_RMS, None, None)
    _check(lib().cm_residual_add_norm(dtype_code(act), _ptr(h), _ptr(n_out), n, ptrs, scales, per, f32, index, weights, _ptr(bias),
                                      _ptr(w_next), rows, H, eps, kind, _ptr(alpha), _ptr(shift), _stream()), "residual_add_norm",
           cost=lambda: (f"{rows}x{H}, {n} terms", 2 * _nbytes(h) + _nbytes(n_out) + sum(rows * t[2] * H * t[0].element_size() for t in terms),
                         (n + 5) * rows * H))


def postnorm_residual(h, terms, h_scale, w, eps, n_out=None, history=None, coef=None):
    """The norm behind the sum: x = norm(h_scale * h + terms) * w (w float32 [H]; a norm with one number has it
    repeated), float32.  Without `history`, h <- x.  With `history` (float32 [n, rows, H], contiguous: what the stack
    held before each layer so far, entry n - 1 free) and `coef` (float32 [n] on the device): entry n - 1 <- x and
    h <- sum_j coef[j] * entry j.  n_out (activation dtype, optional) <- h, for the next reader's products."""
    rows, H = h.shape
    if h.dtype != torch.float32 or not h.is_contiguous():
        raise KernelError("postnorm_residual: a contiguous float32 stream")
    act = n_out.dtype if n_out is not None else next((t[0].dtype for t in terms if t[0].dtype != torch.float32), torch.float32)
    terms, n, ptrs, scales, per, f32, index, weights = _term_arrays(terms, rows, H, act, "postnorm_residual")
    n_hist, stride = 0, 0
    if history is not None:
        n_hist, stride = history.shape[0], history.stride(0)
        if (history.dtype != torch.float32 or tuple(history.shape[1:]) != (rows, H) or not history[0].is_contiguous()
                or coef is None or coef.dtype != torch.float32 or coef.numel() != n_hist):
            raise KernelError("postnorm_residual: history float32 [n, rows, H] with n float32 coefficients")
    _check(lib().cm_postnorm_residual(dtype_code(act), _ptr(h), _ptr(n_out), n, ptrs, scales, per, f32, index, weights,
                                      float(h_scale), _ptr(w), rows, H, eps, _ptr(history), stride, n_hist, _ptr(coef), _stream()),
           "postnorm_residual",
           cost=lambda: (f"{rows}x{H}, {n} terms, depth {n_hist}", 2 * _nbytes(h) + _nbytes(n_out) + (n_hist + 1) * rows * H * 4
                         + sum(rows * t[2] * H * t[0].element_size() for t in terms), (n + 5 + 2 * n_hist) * rows * H))


def concat_cast(out, a, b):
    """out[r] = [a[r]; b[r]] in out's dtype, for float32 rows a and b."""
    rows, H = a.shape
    _check(lib().cm_concat_cast(dtype_code(out.dtype), _ptr(out), _ptr(a), _ptr(b), rows, H, _stream()), "concat_cast",
           cost=lambda: (f"{rows}x{2 * H}", _nbytes(a, b, out), 0))


# ------------------------------------------------------------------ mixers with a matrix state
def shift_mix(out, h, mu, state, tok_seq, tok_pos, seq_pos0, seq_slot):
    """out[s][t] = h[t] + (previous input - h[t]) * mu[s]; the previous input of a sequence's first row of
    the step is the head of its state row (state: float32 [slots, n], n >= width)."""
    S, rows, W = out.shape
    _check(lib().cm_shift_mix(dtype_code(h.dtype), _ptr(out), _ptr(h), _ptr(mu), _ptr(state), state.stride(0),
                              _ptr(tok_seq), _ptr(tok_pos), _ptr(seq_pos0), _ptr(seq_slot), S, rows, W, _stream()),
           "shift_mix", cost=lambda: (f"{S}x{rows}x{W}", _nbytes(h, out, mu), 2 * S * rows * W))


def lowrank_decay(out, x, w1, w2, w0, tau=None):
    """out = exp(-exp(W2 tanh(W1 x) + w0)) in float32: x [rows, W], W1 [R, W], w2 = W2 transposed [R, C], w0 [C].
    With `tau`: out = sigmoid(W2 (W1 x) + w0)^(1/tau) instead (no activation between the two products)."""
    rows, W = x.shape
    R, C = w1.shape[0], w2.shape[1]
    if w1.dtype != x.dtype or w2.dtype != x.dtype or not (x.is_contiguous() and w1.is_contiguous() and w2.is_contiguous()):
        raise KernelError("lowrank_decay: contiguous operands of one dtype")
    _check(lib().cm_lowrank_decay(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(w1), _ptr(w2), _ptr(w0), rows, W, R, C,
                                  int(tau is not None), float(tau or 0.0), _stream()), "lowrank_decay",
           cost=lambda: (f"{rows}x{W} rank {R} -> {C}", _nbytes(x, out, w1, w2), 2 * rows * R * (W + C)))


def tanh_inplace(x):
    """x <- tanh(x), in x's dtype (contiguous)."""
    _check(lib().cm_tanh_inplace(dtype_code(x.dtype), _ptr(x), x.numel(), _stream()), "tanh_inplace",
           cost=lambda: (f"{tuple(x.shape)}", 2 * _nbytes(x), 0))


def decay_from_logits(out, z, w0, tau=None):
    """out = exp(-exp(z + w0)), or sigmoid(z + w0)^(1/tau) with `tau`: z, out float32 [rows, C] contiguous, w0 float32 [C]."""
    rows, C = z.shape
    _check(lib().cm_decay_from_logits(_ptr(out), _ptr(z), _ptr(w0), rows, C, int(tau is not None), float(tau or 0.0), _stream()),
           "decay_from_logits",
           cost=lambda: (f"{rows}x{C}", _nbytes(z, out), 0))


def capped_gates(out, x, w, bias, cap):
    """out[t] = [cap tanh(z / cap) for the first H rows of w; log sigmoid of the same for the other H],
    z = w x + bias; out float32 [rows, 2 H]."""
    rows, W = x.shape
    H = w.shape[0] // 2
    if w.dtype != x.dtype or not (x.is_contiguous() and w.is_contiguous()):
        raise KernelError("capped_gates: contiguous operands of one dtype")
    _check(lib().cm_capped_gates(dtype_code(x.dtype), _ptr(out), _ptr(x), _ptr(w), _ptr(bias), cap, rows, W, H, _stream()),
           "capped_gates", cost=lambda: (f"{rows}x{W} -> {2 * H}", _nbytes(x, out, w), 4 * rows * H * W))


class _ScanArgs(ctypes.Structure):
    """csrc/recurrent.cu: ScanArgs."""
    _fields_ = [("q", _vp), ("k", _vp), ("v", _vp), ("g", _vp), ("ldq", _ll), ("ldk", _ll), ("ldv", _ll), ("ldg", _ll),
                ("decay", _vp), ("bonus", _vp), ("norm_w", _vp), ("out", _vp), ("ldo", _ll), ("state", _vp),
                ("state_stride", _ll), ("state_offset", _ll), ("shift_src", _vp), ("W", _i), ("seq_start", _vp),
                ("seq_slot", _vp), ("H", _i), ("D", _i), ("DV", _i), ("KS", _i), ("q_scale", _f), ("eps", _f), ("raw", _vp),
                ("rows", _ll), ("qkv_act", _i), ("norm_all_heads", _i)]


def matrix_scan(mode, out, q, k, v, g, decay, bonus, norm_w, state, state_offset, seq_start, seq_slot, B, H, D, DV,
                q_scale, eps, shift_src=None, qkv_silu=False, norm_all_heads=False, chunk_scratch=None, max_len=0):
    """The recurrence of a mixer with a matrix state per head over the step's rows of B sequences, with the
    heads' unit norm, channel weights and output gate.  mode "decay": o = (S + diag(bonus) k v^T)^T q, then
    S <- diag(decay_t) S + k v^T (decay float32 [rows, H D]; gate silu(g)).  mode "memory": log-domain
    gates with a running maximum and a normaliser (decay float32 [rows, 2 H]: i, then f; gate sigmoid(g)).
    mode "constant": S <- w S + k v^T, o = S^T q with one decay per head (decay float32 [H]; gate sigmoid(g));
    mode "gated": S <- diag(decay_t) S + k v^T, o = S^T q (decay float32 [rows, H D]; gate silu(g)).
    `qkv_silu`: q, k and v pass through silu as they are read.  `norm_all_heads`: the unit norm runs over all
    heads of a row together.  `chunk_scratch` (mode "constant"; float32, at least `lightning_scratch_floats` elements for
    sequences of up to `max_len` rows): the prompt form, which regroups the sums into chunks of 64 rows so that only the
    state's step from chunk to chunk is serial (csrc/lightning.cu); the numbers agree with the scan's beyond rounding.
    q, k [rows, H D], v, g, out [rows, H DV]: activation dtype, any row pitch.  state: float32 [slots, n];
    this mixer's part of a row starts at `state_offset`.  `shift_src` [rows, W] (mode "decay"): its last
    row of each sequence is kept at the head of the state row."""
    for t in (q, k, v, g, out):
        if t.stride(1) != 1 or t.dtype != out.dtype:
            raise KernelError("matrix_scan: row-major operands of one dtype")
    rows = q.shape[0]
    raw = torch.empty((rows, H * DV), dtype=torch.float32, device=q.device)      # the heads' outputs before norm and gate
    a = _ScanArgs(raw=_ptr(raw), rows=rows, q=_ptr(q), k=_ptr(k), v=_ptr(v), g=_ptr(g), ldq=q.stride(0), ldk=k.stride(0), ldv=v.stride(0),
                  ldg=g.stride(0), decay=_ptr(decay), bonus=_ptr(bonus), norm_w=_ptr(norm_w), out=_ptr(out),
                  ldo=out.stride(0), state=_ptr(state), state_stride=state.stride(0), state_offset=state_offset,
                  shift_src=_ptr(shift_src), W=0 if shift_src is None else shift_src.shape[1], seq_start=_ptr(seq_start),
                  seq_slot=_ptr(seq_slot), H=H, D=D, DV=DV, KS=0, q_scale=q_scale, eps=eps, qkv_act=int(qkv_silu),
                  norm_all_heads=int(norm_all_heads))
    if mode == "constant" and (decay.dtype != torch.float32 or decay.numel() != H):
        raise KernelError("matrix_scan: mode 'constant' takes one float32 decay per head")
    if chunk_scratch is not None:
        if mode != "constant" or chunk_scratch.dtype != torch.float32 or chunk_scratch.numel() < lightning_scratch_floats(B, max_len, H, D, DV):
            raise KernelError("matrix_scan: the chunked form is for mode 'constant' and needs its float32 scratch")
        _check(lib().cm_lightning_chunked(dtype_code(out.dtype), ctypes.byref(a), B, max_len, _ptr(chunk_scratch), _stream()),
               "lightning_chunked", 4,
               cost=lambda: (f"{B} sequences, {rows} rows, {H} heads of {D}x{DV}", _nbytes(q, k, v, g, out) + 2 * B * H * D * DV * 4,
                             6 * rows * H * D * DV))
        return
    _check(lib().cm_matrix_scan(dtype_code(out.dtype), {"decay": 0, "memory": 1, "constant": 2, "gated": 3}[mode], ctypes.byref(a), B, _stream()),
           "matrix_scan_" + mode, 2,
           cost=lambda: (f"{B} sequences, {rows} rows, {H} heads of {D}x{DV}",
                         _nbytes(q, k, v, g, out) + (0 if decay is None or decay.dim() < 2 else rows * decay.shape[1] * 4) + 2 * B * H * D * DV * 4,
                         6 * rows * H * D * DV))


LIGHTNING_CHUNK = 64               # csrc/lightning.cu: rows of a chunk of the prompt form


def lightning_scratch_floats(B, max_len, H, D, DV):
    """Floats of scratch that the chunked prompt form needs: a state per chunk, head and sequence."""
    return B * -(-max_len // LIGHTNING_CHUNK) * H * D * DV


def lightning_chunked_fits(D, DV):
    """True if heads of D x DV fit the chunked form's shared memory."""
    fn = lib().cm_lightning_chunked_smem
    fn.argtypes, fn.restype = [_i, _i], _ll
    return fn(D, DV) <= 200 * 1024


# ------------------------------------------------------------------ attention as a difference of two maps
class _TapRotArgs(ctypes.Structure):
    """csrc/diffattn.cu: TapRotArgs."""
    _fields_ = [("proj", _vp), ("ldp", _ll), ("bias", _vp), ("taps", _vp), ("state", _vp), ("state_stride", _ll),
                ("q_out", _vp), ("ldq", _ll), ("pool", _vp), ("pages", _ll), ("ptab", _vp), ("ptab_stride", _ll),
                ("rate", _vp), ("mag", _f), ("tok_seq", _vp), ("tok_pos", _vp), ("seq_start", _vp), ("seq_pos0", _vp),
                ("seq_slot", _vp)] + [(n, _i) for n in ("T", "B", "QC", "KC", "VC", "K", "sub", "rot", "G", "KW", "DV", "HDC",
                                                        "one_token_each", "interleaved", "value_from_key", "ring",
                                                        "no_store", "rows_out", "from_zero")]


def tap_rotate_store(proj, bias, taps, state, q_out, batch, q_channels, sub, rate, mag, kv=None, one_token_each=False,
                     interleaved=False, value_from_key=False, ring=0, store=True, rows_out=False, from_zero=False):
    """Short causal taps over the leading channels of the projected rows `proj` (q, then k and v when this layer
    has them), the partial rotation of q and k, and the cache write.  bias float32 [C] or None; taps float32
    [C, K]; state float32 [slots, >= K C] (a ring of the last K projected rows of every sequence, moved on by
    this call); q_out [T, q_channels] receives the queries.  `sub`: channels of one rotated vector; rate float32
    [rot / 2] or None; mag: the factor on sine and cosine.  kv = (pool, pages, ptab, G, key row width, value row
    width): this layer's pages [2, pages, G, PAGE_TOKENS, HDC]; keys and values follow q in `proj`.
    `interleaved`: the rotation pairs channel 2i with 2i + 1.  `value_from_key`: there are no value channels (value
    row width 0 in `kv`); a position's value is its key before the rotation.  `ring`: the pages are a ring of that many
    entries.  `store` False leaves the cache alone.  `rows_out`: q_out rows are [q | turned k | v].  `from_zero`: every
    sequence of the step starts at position 0 (a whole-prompt step), so nothing reads the state and the form for long
    interleaved steps writes it in its one launch."""
    T = proj.shape[0]
    C, K = taps.shape
    G = KW = DV = HDC = 0
    pool = ptab = None
    pages = 0
    if kv is not None:
        pool, pages, ptab, G, KW, DV = kv
        HDC = pool.shape[-1]
    if C != q_channels + G * (KW + DV) or proj.shape[1] < C or proj.stride(1) != 1 or q_out.dtype != proj.dtype:
        raise KernelError("tap_rotate_store: the projected rows do not hold the channels that the taps name")
    if not (taps.is_contiguous() and taps.dtype == torch.float32) or (K > 1 and state is None):
        raise KernelError("tap_rotate_store: float32 taps, and a state for more than one tap")
    if state is not None and (state.dtype != torch.float32 or state.stride(-1) != 1):
        raise KernelError("tap_rotate_store: float32 taps and state")
    if q_out.shape[1] < (C + (G * KW if value_from_key else 0) if rows_out else q_channels):
        raise KernelError("tap_rotate_store: the output rows are too short")
    a = _TapRotArgs(proj=_ptr(proj), ldp=proj.stride(0), bias=_ptr(bias), taps=_ptr(taps), state=_ptr(state),
                    state_stride=0 if state is None else state.stride(0), q_out=_ptr(q_out), ldq=q_out.stride(0), pool=_ptr(pool), pages=pages,
                    ptab=_ptr(ptab), ptab_stride=0 if ptab is None else ptab.stride(0), rate=_ptr(rate), mag=mag,
                    tok_seq=_ptr(batch.tok_seq), tok_pos=_ptr(batch.tok_pos), seq_start=_ptr(batch.seq_start),
                    seq_pos0=_ptr(batch.seq_pos0), seq_slot=_ptr(batch.seq_slot), T=T, B=batch.B, QC=q_channels,
                    KC=G * KW, VC=G * DV, K=K, sub=sub, rot=0 if rate is None else 2 * rate.numel(), G=G, KW=KW, DV=DV,
                    HDC=HDC, one_token_each=int(one_token_each), interleaved=int(interleaved),
                    value_from_key=int(value_from_key), ring=int(ring), no_store=int(not store), rows_out=int(rows_out), from_zero=int(from_zero))
    _check(lib().cm_tap_rotate_store(dtype_code(proj.dtype), ctypes.byref(a), _stream()), "tap_rotate_store",
           1 if one_token_each or K < 2 or (from_zero and interleaved and T >= 64 and K <= 4) else 2,
           cost=lambda: (f"{T}x{C}, {K} taps", 2 * T * C * proj.element_size(), 2 * K * T * C))


class _DiffAttnArgs(ctypes.Structure):
    """csrc/diffattn.cu: DiffAttnArgs."""
    _fields_ = [("ctx", _vp), ("ldc", _ll), ("q", _vp), ("ldq", _ll), ("gate", _vp), ("ldg", _ll), ("pool", _vp),
                ("pages", _ll), ("ptab", _vp), ("ptab_stride", _ll), ("tok_seq", _vp), ("tok_pos", _vp), ("seq_start", _vp),
                ("seq_pos0", _vp), ("seq_slot", _vp)] + [(n, _i) for n in ("T", "B", "H", "G", "D", "DV", "HDC", "window", "keep")] \
               + [(n, _f) for n in ("scale", "lam", "out_scale", "eps")]


DIFF_ATTN_ROW_WARPS, DIFF_ATTN_MAX_SPLITS = 4, 16      # csrc/diffattn.cu: warps of a block of the rows form; most shares


def diff_attn_splits(rows, H, G, keys, sm_count=148):
    """Into how many shares the rows form cuts a row's visible keys (at most `keys` of them): enough blocks for two per
    SM, while every warp still has a tile of 32 keys.  A block takes four query heads of a key/value head together
    where their number is a multiple of four."""
    tiles = -(-max(1, keys) // 32)
    blocks = rows * (H // 4 if (H // G) % 4 == 0 else H)
    want = -(-2 * sm_count // max(1, blocks))
    return max(1, min(DIFF_ATTN_MAX_SPLITS, want, -(-tiles // DIFF_ATTN_ROW_WARPS)))


def diff_attn(ctx, q, gate, pool, pages, ptab, batch, H, G, D, DV, window, keep, scale, lam, out_scale, eps, rows_form,
              parts=None, splits=1, tensor_cores=False):
    """Attention whose output is the difference of two softmax maps over the same values, read from the paged
    cache: q [T, H * 2 * D] (per head map 1, then map 2), ctx [T, H * DV]; a key at j is visible from i when
    j <= i and (i - j < window or j < keep) (window <= 0: all j <= i); o = a1 - lam * a2, brought to unit root mean
    square per head, times out_scale and sigmoid(gate[t, head]) (gate may be None).  `rows_form`: a block per row
    and head (steps of one token a sequence), whose visible keys may be cut into `splits` shares with float32 scratch
    `parts` of at least T * H * splits * (4 + 2 DV) elements between two launches; else tiles of queries, launched for
    batch.max_len rows a sequence, on the tensor cores with `tensor_cores` (bfloat16, head sizes that are multiples of 16
    up to 128: `diff_attn_mma_fits`)."""
    if splits > 1 and (parts is None or parts.dtype != torch.float32 or parts.numel() < _diff_attn_parts_floats(q, H, splits, DV)):
        raise KernelError("diff_attn: the shares' scratch is missing or too small")
    T = q.shape[0]
    if q.stride(1) != 1 or ctx.stride(1) != 1 or q.dtype != ctx.dtype or pool.dtype != q.dtype:
        raise KernelError("diff_attn: row-major operands and a cache of one dtype")
    a = _DiffAttnArgs(ctx=_ptr(ctx), ldc=ctx.stride(0), q=_ptr(q), ldq=q.stride(0), gate=_ptr(gate),
                      ldg=0 if gate is None else gate.stride(0), pool=_ptr(pool), pages=pages, ptab=_ptr(ptab),
                      ptab_stride=ptab.stride(0), tok_seq=_ptr(batch.tok_seq), tok_pos=_ptr(batch.tok_pos),
                      seq_start=_ptr(batch.seq_start), seq_pos0=_ptr(batch.seq_pos0), seq_slot=_ptr(batch.seq_slot), T=T,
                      B=batch.B, H=H, G=G, D=D, DV=DV, HDC=pool.shape[-1], window=window, keep=keep, scale=scale, lam=lam,
                      out_scale=out_scale, eps=eps)
    if tensor_cores and not rows_form:
        if q.dtype != torch.bfloat16:
            raise KernelError("diff_attn: the tensor-core form takes bfloat16")
        _check(lib().cm_diff_attn_mma(ctypes.byref(a), batch.max_len, _stream()), "diff_attn_mma",
               cost=lambda: _diff_attn_cost(batch, T, H, G, D, DV, window, keep, q.element_size(), rows_form))
        return
    _check(lib().cm_diff_attn(dtype_code(q.dtype), ctypes.byref(a), int(rows_form), batch.max_len, _ptr(parts), splits,
                              _stream()), "diff_attn", 2 if rows_form and splits > 1 else 1,
           cost=lambda: _diff_attn_cost(batch, T, H, G, D, DV, window, keep, q.element_size(), rows_form))


def diff_attn_mma_fits(D, DV, H, q_row, cache_entry):
    """True if the tensor-core tiles form takes these sizes (key and value heads, heads, elements of a query row and of a
    cache entry)."""
    return D % 16 == 0 and DV % 16 == 0 and 0 < D <= 128 and 0 < DV <= 128 and q_row % 8 == 0 and cache_entry % 8 == 0


def _diff_attn_parts_floats(q, H, splits, DV):
    """Floats of scratch between the two launches of the rows form: maxima, sums and value sums per row, head and share."""
    return q.shape[0] * H * splits * (4 + 2 * DV)


def _diff_attn_cost(batch, T, H, G, D, DV, window, keep, esz, rows_form):
    """(shape text, bytes, floating-point operations) by definition: the keys a row sees are those of its window and the
    kept ones, half of its sequence for a prompt from position 0; every key and value row is read once per sequence."""
    reach = batch.max_end if rows_form else max(1, batch.max_end // 2)
    seen = min(reach, window + keep) if window > 0 else reach
    held = min(batch.max_end, window + keep + (0 if rows_form else batch.max_len)) if window > 0 else batch.max_end
    nbytes = batch.B * held * G * (2 * D + DV) * esz + T * H * (2 * D + DV) * esz
    return (f"{batch.B} sequences, {T} rows, {H}/{G} heads of 2x{D}, {DV}, window {window}+{keep}", nbytes,
            2 * 2 * T * seen * H * (D + DV))


# ------------------------------------------------------------------ latent attention
class _LatentArgs(ctypes.Structure):
    """csrc/latent.h: LatentArgs."""
    _fields_ = [("proj", _vp), ("ld_proj", _ll), ("q_off", _i), ("kv_off", _i), ("cq", _vp), ("wq_norm", _vp), ("wkv_norm", _vp),
                ("rate", _vp), ("q", _vp), ("ldq", _ll), ("qa", _vp), ("ldqa", _ll), ("gate", _vp), ("ld_gate", _ll),
                ("out", _vp), ("ldo", _ll), ("H", _i), ("D", _i), ("R", _i), ("KR", _i), ("QR", _i), ("E", _i), ("EC", _i),
                ("eps", _f), ("scale", _f), ("rows", _ll), ("tok_pos", _vp), ("tok_seq", _vp), ("seq_start", _vp),
                ("seq_pos0", _vp), ("seq_end", _vp), ("seq_slot", _vp), ("pool", _vp), ("ptab", _vp), ("ptab_stride", _ll),
                ("B", _i), ("max_len", _i), ("splits", _i), ("chunk", _i), ("parts", _vp), ("ckv", _vp), ("kvu", _vp),
                ("ld_kvu", _ll), ("qkv", _vp), ("ld_qkv", _ll), ("HD", _i), ("DV", _i), ("mag", _f), ("no_entry", _i)]


latent_decode_tensor_cores = True   # off: single-token steps of the latent attention stay on the CUDA cores (tests compare)


def set_latent_decode_tensor_cores(on):
    global latent_decode_tensor_cores
    latent_decode_tensor_cores = bool(on)


LATENT_KEY_TILE = 32               # csrc/latent.cu: cache entries of a key tile; a split's keys are a multiple of it


def latent_entry_size(kv_rank, rot_dim):
    """Channels of a cache entry of the latent attention: the latent, the turned key part, zeros up to a multiple of 8."""
    return -(-(kv_rank + rot_dim) // 8) * 8


def _latent_args(batch, pool, ptab, H, D, R, KR, QR, eps=0.0, scale=1.0, mag=1.0, **fields):
    return _LatentArgs(mag=mag, H=H, D=D, R=R, KR=KR, QR=QR, E=KR + R, EC=pool.shape[-1], eps=eps, scale=scale, rows=batch.T,
                       tok_pos=_ptr(batch.tok_pos), tok_seq=_ptr(batch.tok_seq), seq_start=_ptr(batch.seq_start),
                       seq_pos0=_ptr(batch.seq_pos0), seq_end=_ptr(batch.seq_end), seq_slot=_ptr(batch.seq_slot),
                       pool=_ptr(pool), ptab=_ptr(ptab), ptab_stride=ptab.stride(0), B=batch.B, max_len=batch.max_len,
                       splits=1, chunk=0, **fields)


def latent_prepare(cq, proj, q_off, kv_off, wq_norm, wkv_norm, rate, pool, ptab, batch, H, D, R, KR, QR, eps, entries=None,
                   mag=1.0, make_entry=True):
    """Per row of the step: cq = norm(proj[q_off : q_off + QR]) * wq_norm (activation dtype, for the product that
    makes the heads' queries), and the row's cache entry [norm(proj[kv_off : kv_off + KR]) * wkv_norm | the next R
    channels turned by the position (pairs 2i, 2i + 1 by position * rate[i]) | zeros] into pool [pages, PAGE_TOKENS, EC]
    through the page table.  Norms and angles are float32.  `entries` [rows, EC] (contiguous): the same entries once
    more in the order of the step's rows (zeros for rows of padding), for a product over them.  `mag`: the factor on
    sine and cosine (all rotations of the latent attention take it).  `make_entry` False: only cq is made (a layer that
    reads another layer's entries; kv_off and wkv_norm are then not used)."""
    a = _latent_args(batch, pool, ptab, H, D, R, KR, QR, eps=eps, mag=mag, no_entry=int(not make_entry), proj=_ptr(proj), ld_proj=proj.stride(0), q_off=q_off,
                     kv_off=kv_off, cq=_ptr(cq), wq_norm=_ptr(wq_norm), wkv_norm=_ptr(wkv_norm), rate=_ptr(rate),
                     ckv=_ptr(entries))
    if proj.stride(1) != 1 or not cq.is_contiguous() or cq.dtype != proj.dtype or pool.dtype != proj.dtype:
        raise KernelError("latent_prepare: row-major operands of one dtype")
    if entries is not None and (entries.shape != (batch.T, pool.shape[-1]) or not entries.is_contiguous() or entries.dtype != pool.dtype):
        raise KernelError("latent_prepare: the entries' copy is [rows, entry size] in the cache's dtype")
    _check(lib().cm_latent_prepare(dtype_code(proj.dtype), ctypes.byref(a), _stream()), "latent_prepare",
           cost=lambda: (f"{batch.T} rows, {QR} + {KR} + {R}", batch.T * (2 * QR + 2 * (KR + R)) * proj.element_size(), 6 * batch.T * (QR + KR)))


def latent_query_turn(qa, q, rate, pool, ptab, batch, H, D, R, KR, mag=1.0):
    """qa[t, h, KR:KR + R] (float32) = the last R channels of head h's query q[t, h, :D + R], turned by the position."""
    a = _latent_args(batch, pool, ptab, H, D, R, KR, 0, mag=mag, q=_ptr(q), ldq=q.stride(0), qa=_ptr(qa), ldqa=qa.stride(0),
                     rate=_ptr(rate))
    if qa.dtype != torch.float32 or qa.stride(1) != 1 or q.stride(1) != 1:
        raise KernelError("latent_query_turn: float32 rows for the turned queries")
    _check(lib().cm_latent_query_turn(dtype_code(q.dtype), ctypes.byref(a), _stream()), "latent_query_turn",
           cost=lambda: (f"{batch.T} rows, {H} heads of {R}", batch.T * H * R * (4 + q.element_size()), 6 * batch.T * H * R))


def latent_expand(qkv, q, kvu, entries, rate, pool, ptab, batch, H, D, R, DV, KR, HD, mag=1.0):
    """The operands of an attention over keys and values per head, for a prompt step: qkv [rows, 3 * H * HD] =
    per head [q_plain | q_turn turned by the position | 0], then per head [kvu's unturned key | the row's turned key
    part from `entries` | 0], then per head [kvu's value | 0].  q [rows, H * (D + R)] as the product left it; kvu
    [rows, H * D + H * DV] = [W_uk; W_uv] times the row's latent; entries [rows, EC] from `latent_prepare`.  Rows of
    padding become zeros."""
    a = _latent_args(batch, pool, ptab, H, D, R, KR, 0, mag=mag, q=_ptr(q), ldq=q.stride(0), rate=_ptr(rate), ckv=_ptr(entries),
                     kvu=_ptr(kvu), ld_kvu=kvu.stride(0), qkv=_ptr(qkv), ld_qkv=qkv.stride(0), HD=HD, DV=DV)
    if (qkv.shape[1] != 3 * H * HD or kvu.shape[1] != H * (D + DV) or q.shape[1] != H * (D + R) or not entries.is_contiguous()
            or any(t.stride(1) != 1 or t.dtype != qkv.dtype for t in (qkv, q, kvu, entries))):
        raise KernelError("latent_expand: row-major operands of one dtype, heads of HD channels")
    _check(lib().cm_latent_expand(dtype_code(qkv.dtype), ctypes.byref(a), _stream()), "latent_expand",
           cost=lambda: (f"{batch.T} rows, {H} heads of {D}+{R} and {DV} in {HD}",
                         batch.T * (3 * H * HD + H * (2 * D + R + DV) + R) * qkv.element_size(), 6 * batch.T * H * R))


def latent_attn_splits(rows, H, keys, sm_count=148, heads_per_block=32, kv_rank=256):
    """(splits, keys per split) for a step of `rows` single-token rows over up to `keys` cache entries.  A split of a
    sequence is one block per 32 heads (16 in the tensor-core form).  The blocks should be about as many as are resident
    together (four a multiprocessor; two for the tensor-core form's tiles of latents wider than 256), rounded up: a
    block walks its key tiles one behind the other, and the others hide its waits.  A split is at least two key tiles
    long (four in the tensor-core form, where a block's queries weigh as much as a tile of entries).  Measured on B200,
    tensor-core form, both launches: 128 sequences at 2,048 tokens, 16 heads over 256 + 32: 5 splits (640 blocks, a few
    more than are resident) 120 us, 4 splits (512 blocks) 135 us; 8 sequences, 32 heads over 512 + 32 inside a decode
    step: 18 splits 1.22 ms a step, 32 splits 1.28 ms."""
    per_split = rows * -(-H // heads_per_block)
    tiles = -(-keys // LATENT_KEY_TILE)
    resident = sm_count * (2 if heads_per_block == 16 and kv_rank > 256 else 4)
    splits = max(1, min(tiles // (4 if heads_per_block == 16 else 2), -(-resident // per_split)))
    chunk = -(-tiles // splits) * LATENT_KEY_TILE
    return -(-keys // chunk) if splits > 1 else 1, chunk


def latent_attn(out, qa, gate, pool, ptab, batch, H, R, KR, scale, splits=1, chunk=0, parts=None, tensor_cores=False):
    """Causal softmax attention of every head's query row qa [rows, H, KR + R] (float32) over the cache entries of
    its sequence (positions <= the row's own); out [rows, H, KR] (float32) = the weights' sum over the latents,
    times sigmoid(gate[t, h]) when `gate` ([rows, >= H] logits, activation dtype) is given.  `splits` > 1: the keys
    are cut into runs of `chunk` entries, each run a block of its own, merged afterwards (`parts`: float32 scratch of
    rows * H * splits * (2 + KR)).  `tensor_cores`: a step of one token per sequence over a bfloat16 cache takes the
    mma.sync form (the queries rounded to bfloat16, sums in float32)."""
    a = _latent_args(batch, pool, ptab, H, 0, R, KR, 0, scale=scale, qa=_ptr(qa), ldqa=qa.stride(0), gate=_ptr(gate),
                     ld_gate=0 if gate is None else gate.stride(0), out=_ptr(out), ldo=out.stride(0))
    a.splits, a.chunk, a.parts = splits, chunk, _ptr(parts)
    if qa.dtype != torch.float32 or out.dtype != torch.float32 or (gate is not None and gate.dtype != pool.dtype):
        raise KernelError("latent_attn: float32 queries and sums")
    if splits > 1 and (parts is None or parts.numel() < batch.T * H * splits * (2 + KR)):
        raise KernelError("latent_attn: the splits' scratch is missing or short")
    cost = lambda: (f"{batch.B} sequences, {batch.T} rows, {H} heads over {KR}+{R}",
                    _nbytes(qa, out) + sum((p + n) * pool.shape[-1] * pool.element_size() for p, n in zip(batch.positions, batch.lengths)),
                    sum(2 * n * H * (p + (n + 1) // 2) * (2 * KR + R) for p, n in zip(batch.positions, batch.lengths)))
    if tensor_cores:
        if batch.kind != "decode" or batch.T != batch.B or pool.dtype != torch.bfloat16:
            raise KernelError("latent_attn: the tensor-core form takes one token per sequence over a bfloat16 cache")
        _check(lib().cm_latent_attn_mma(ctypes.byref(a), _stream()), "latent_attn_mma", 2 if splits > 1 else 1, cost=cost)
        return
    _check(lib().cm_latent_attn(dtype_code(pool.dtype), ctypes.byref(a), _stream()), "latent_attn", 2 if splits > 1 else 1, cost=cost)


def head_linear(y, x, w, H, x_size, y_size):
    """A matrix per head: y[t, h * y_size + n] = sum_k x[t, h * x_size + k] * w[h, n, k] for w [H, N, K].  x and y are
    in w's dtype or float32 (a sum that stays unrounded between two steps)."""
    rows = x.shape[0]
    N, K = w.shape[1], w.shape[2]
    if x.stride(1) != 1 or y.stride(1) != 1 or not w.is_contiguous() or w.shape[0] != H:
        raise KernelError("head_linear: row-major operands, one matrix per head")
    for t in (x, y):
        if t.dtype not in (w.dtype, torch.float32):
            raise KernelError("head_linear: rows in the matrices' dtype or float32")
    _check(lib().cm_head_linear(dtype_code(w.dtype), _ptr(y), _ptr(x), _ptr(w), rows, H, N, K, x.stride(0), y.stride(0), x_size,
                                y_size, int(x.dtype == torch.float32 and w.dtype != torch.float32),
                                int(y.dtype == torch.float32 and w.dtype != torch.float32), _stream()), "head_linear",
           cost=lambda: (f"{rows} rows, {H} heads of {N}x{K}", rows * H * (N * y.element_size() + K * x.element_size()) + _nbytes(w),
                         2 * rows * H * N * K))


# ------------------------------------------------------------------ routed feed-forward
MOE_TILE_SIMT, MOE_TILE_TC = 32, 128     # rows of a row tile: the CUDA-core grouped products, the tcgen05 grouped product


def moe_max_tiles(pairs, experts, tile_rows=MOE_TILE_SIMT):
    fn = lib().cm_moe_max_tiles
    fn.argtypes, fn.restype = [_ll, _i, _i], _i
    return fn(pairs, experts, tile_rows)


def moe_work_size(pairs, experts, tile_rows=MOE_TILE_SIMT):
    """int32 entries of `moe_route`'s scratch: counts, cursors, the list of row tiles, each row tile's expert."""
    return 2 * experts + 1 + 4 * moe_max_tiles(pairs, experts, tile_rows)


def moe_tile_group(work, pairs, experts, tile_rows):
    """The part of `work` that holds each row tile's expert (what the grouped tcgen05 product reads)."""
    tiles = moe_max_tiles(pairs, experts, tile_rows)
    return work[2 * experts + 1 + 3 * tiles:2 * experts + 1 + 4 * tiles]


def moe_route(ids, wts, perm, dest, work, h, w_router, tok_seq, top, softmax_gate=False, renormalize=False,
              tile_rows=MOE_TILE_SIMT, xs=None, apply_weight=False, correction=None, groups=0, keep=0, identity=0, scale=1.0,
              renorm_eps=0.0, group_best=1):
    """Scores of every token's experts in float32 (sigmoid, or softmax over the experts), the `top` best
    (ids, wts: [rows * top]; -1 for rows of padding), and the pairs in the order of their experts, every expert's
    rows beginning a row tile of `tile_rows` rows: perm[sorted row] = pair (moe_max_tiles * tile_rows entries),
    dest[pair] = sorted row (-1: none), the list of row tiles in `work` (int32, moe_work_size entries).  With `xs`
    ([moe_max_tiles * tile_rows, W]) the experts' inputs are gathered into it in the same call (`moe_gather`).  A step of
    up to 64 rows runs all of this in one launch of one block.
    `correction` (float32 [E]): added to the scores for the choice only.  `groups`, `keep`: the experts form `groups` equal
    groups of neighbours, and only experts of the `keep` groups with the largest score can be chosen; a group's score is
    the sum of its `group_best` largest choice scores (1: its largest).
    `identity`: the last `identity` router outputs are experts without matrices whose output is their input: their pairs get
    a weight and dest -1 (`moe_identity` adds them).  `scale`: a factor on the weights; `renorm_eps`: added to the sum that
    `renormalize` divides by."""
    rows, W = h.shape
    E = w_router.shape[0]
    if correction is not None and (correction.dtype != torch.float32 or correction.numel() != E):
        raise KernelError("moe_route: one float32 correction per router output")
    if w_router.dtype != h.dtype or not (h.is_contiguous() and w_router.is_contiguous()):
        raise KernelError("moe_route: contiguous operands of one dtype")
    _check(lib().cm_moe_route(dtype_code(h.dtype), _ptr(ids), _ptr(wts), _ptr(perm), _ptr(dest), _ptr(work), _ptr(h),
                              _ptr(w_router), _ptr(tok_seq), rows, W, E, top, int(softmax_gate), int(renormalize), tile_rows,
                              _ptr(xs), int(apply_weight), _ptr(correction), int(groups), int(keep), int(identity), float(scale),
                              float(renorm_eps), int(group_best), _stream()), "moe_route",
           1 if rows <= 64 and rows * E * (2 if correction is not None or groups else 1) <= 8192 else (4 if xs is not None else 3),
           cost=lambda: (f"{rows}x{W} over {E}, top {top}", _nbytes(h, w_router), 2 * rows * E * W))


def moe_identity(y, h, ids, wts, top, real):
    """y[t] (float32) = h[t] times the sum of the weights of token t's pairs whose expert is an identity expert
    (id >= real)."""
    rows, K = h.shape
    _check(lib().cm_moe_identity(dtype_code(h.dtype), _ptr(y), _ptr(h), _ptr(ids), _ptr(wts), rows, top, real, K, _stream()),
           "moe_identity", cost=lambda: (f"{rows}x{K}", _nbytes(h, y), rows * K))


def moe_gather(xs, h, dest, wts, top, apply_weight):
    """xs[dest[p]] = h[p // top] (times wts[p] if apply_weight): the experts' inputs in the order of the experts."""
    pairs, K = dest.numel(), h.shape[1]
    _check(lib().cm_moe_gather(dtype_code(h.dtype), _ptr(xs), _ptr(h), _ptr(dest), _ptr(wts), pairs, top, K, int(apply_weight),
                               _stream()), "moe_gather", cost=lambda: (f"{pairs}x{K}", 2 * pairs * K * h.element_size(), pairs * K))


def moe_grouped(out, x, w, work, perm, wts, top, max_tiles, up, apply_weight, gelu=False, act=None, limit=0.0):
    """The experts' products over the rows that `moe_route` gave them (row tiles of 32), on the CUDA cores.
    up: out[sorted row] = act(Wg x) * (Wu x) with x = h[token] (times the pair's weight if apply_weight), w [E, 2 F, K];
    else out[sorted row] (float32) = Wd a (times the weight if apply_weight), w [E, N, K].  `act`, `limit`: as `swiglu`."""
    act = (ACT_GELU_TANH if gelu else ACT_SILU) if act is None else int(act)
    E = w.shape[0]
    N = w.shape[1] // 2 if up else w.shape[1]
    K = w.shape[2]
    if w.dtype != x.dtype or not (x.is_contiguous() and w.is_contiguous() and out.is_contiguous()) or x.shape[1] != K:
        raise KernelError("moe_grouped: contiguous operands of one dtype")
    _check(lib().cm_moe_grouped(dtype_code(x.dtype), int(up), _ptr(out), _ptr(x), _ptr(w), _ptr(work), _ptr(perm), _ptr(wts),
                                E, top, max_tiles, N, K, int(apply_weight), act, float(limit), _stream()),
           "moe_grouped_" + ("up" if up else "down"),
           cost=lambda: (f"{out.shape[0]} rows, {w.shape[1]}x{K} per expert", _nbytes(x, out) + min(E, out.shape[0]) * w[0].numel() * w.element_size(),
                         2 * out.shape[0] * w.shape[1] * K))


def gemm_tc_grouped(y, x, w, tile_group, swiglu=False, err=None, block_n=256, limit=0.0):
    """`gemm_tc` with a matrix per row tile: w [groups, N (2 N when swiglu), K] bfloat16, tile_group (device int32)
    names the matrix that multiplies each tile of 128 rows of x.  y bfloat16, or float32 for the plain product.
    swiglu: True (silu) or 3 with `limit` (the clamped gate), as `gemm_tc`."""
    M, K = x.shape
    G, N = w.shape[0], y.shape[1]
    if w.shape[2] != K or w.shape[1] != (2 * N if swiglu else N) or y.shape[0] != M or tile_group.numel() * 128 < M:
        raise KernelError(f"gemm_tc_grouped shapes: x {tuple(x.shape)}, w {tuple(w.shape)}, y {tuple(y.shape)}")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not (x.is_contiguous() and w.is_contiguous() and y.is_contiguous()):
        raise KernelError("gemm_tc_grouped takes contiguous bfloat16 operands")
    _check(lib().cm_gemm_tc_grouped(dtype_code(y.dtype), _ptr(y), _ptr(x), _ptr(w), M, N, K, x.stride(0), w.stride(1), y.stride(0),
                                    int(swiglu), block_n, _ptr(tile_group), G, _ptr(err), float(limit), _stream()),
           "gemm_tc_grouped" + _GATE_SUFFIX[int(swiglu)],
           cost=lambda: (f"{M}x{w.shape[1]}x{K} over {G} matrices", _nbytes(x, y) + min(G, -(-M // 128)) * w[0].numel() * 2,
                         2 * M * w.shape[1] * K))
