"""Python bindings of the CUDA kernels in `llm_b200/csrc`.

Every function takes torch tensors that live on the GPU, checks what the
kernel cannot check itself, picks the kernel variant for the shape
(`tactics`) and launches on torch's current stream. There is no CPU path
and no library fallback: a missing or failing library raises KernelError.

The parts call these functions as attributes of this module
(`ops.rmsnorm(...)`).
"""
from __future__ import annotations

import atexit
import ctypes
import functools
import os
import sys

import torch

from .. import native
from ..errors import KernelError
from . import tactics
from .build import all_sources, ensure_built, load_library

PAGE = native.plan_constant("page")              # positions per cache page (csrc/plan.h)
BFLOAT16_ONLY = ("gemm_tc", "gemm_skinny", "attention_decode", "attention_decode_window", "attention_prefill",
                 "attention_prefill_tc")     # (diff_attention holds the 32-bit kernel too)

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}
_c_int, _c_float, _c_void = ctypes.c_int, ctypes.c_float, ctypes.c_void_p


def _code(dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} has no kernel (float32 and bfloat16 are built)") from None


def _ptr(t):
    if t is None:
        return None
    if _recording is not None:
        _recording.keep.append(t)          # a recorded pass points at this tensor: it must outlive the record
    return ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream():
    """The current stream's handle (the short way where this torch has it: a launch costs the host
    a few microseconds, the stream object's construction as much again)."""
    if _raw_stream is not None and _current_device is not None:
        return ctypes.c_void_p(_raw_stream(_current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("llm_b200 kernels need tensors on a CUDA device; there is no CPU path")


def _check_out(out, shape, dtype, what: str):
    """Refuse a caller's `out` that the kernel would not fill as the caller thinks: the kernels
    write rows of the result's own width one after the other, so a buffer of another shape,
    dtype or layout would be overrun or garbled without a word."""
    if out is None:
        return
    _require_cuda(out)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or not out.is_contiguous():
        raise KernelError(f"{what}: out is {tuple(out.shape)} {out.dtype}"
                          f"{'' if out.is_contiguous() else ' (not contiguous)'}, the result is "
                          f"{tuple(shape)} {dtype}")


_launches = 0


def launch_count() -> int:
    """Kernels of this library launched so far by this process. A step that is
    replayed from a CUDA graph adds the kernels the graph holds."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


# LLMB_PROFILE=1: every launch between two CUDA events, a table of milliseconds and calls per
# kernel entry at exit (the per-launch timing of MythEclipse/llm's LLM_PROFILE=1,
# apps/engine/src/cuda/mod.rs:1857-1866,1917-1972). Profiling switches graph replay off.
PROFILING = os.environ.get("LLMB_PROFILE", "0") not in ("", "0")
_profile: dict = {}


def _report_profile() -> None:
    if not _profile:
        return
    torch.cuda.synchronize()
    rows = []
    for name, events in _profile.items():
        ms = sum(a.elapsed_time(b) for a, b in events)
        rows.append((ms, len(events), name))
    total = sum(r[0] for r in rows) or 1.0
    print(f"[llm_b200] kernel time by entry point ({total:.2f} ms in all)", file=sys.stderr)
    for ms, calls, name in sorted(rows, reverse=True):
        print(f"  {name:28s}{ms:10.3f} ms{calls:8d} calls{ms / calls * 1e3:10.1f} us/call"
              f"{100 * ms / total:7.1f} %", file=sys.stderr)


if PROFILING:
    atexit.register(_report_profile)


# ----------------------------------------------------------------------------- recorded passes

_recording = None           # the Recording that launches are being entered into, or None
_scratch_generation = 0     # grows when a scratch buffer that recorded passes point at is replaced


class Recording:
    """The launches of one pass as they were made: (library, entry point, ctypes arguments)."""

    def __init__(self):
        self.calls, self.keep, self.kernels = [], [], 0


def begin_recording() -> Recording:
    """From here on every launch of this module is also entered into the returned Recording
    (it still runs), until end_recording()."""
    global _recording
    _recording = Recording()
    return _recording


def end_recording() -> None:
    global _recording
    _recording = None


class RecordedPass:
    """A Recording turned into a native plan (csrc/host/plan_run.cpp): `run()` makes the same
    launches with the same arguments on the current stream through the entry points' packed
    doors, in one call of the native host library. The tensors the launches point at are kept
    alive here. Valid while no scratch buffer of this module was replaced
    (`scratch_generation`)."""

    def __init__(self, recording: Recording):
        doors, counts, stream_slots, slots = [], [], [], []
        self._keep = [recording.keep]
        for lib_name, fn_name, args in recording.calls:
            lib = load_library(lib_name)
            door = ctypes.cast(getattr(lib, fn_name + "_packed"), ctypes.c_void_p).value
            doors.append(door)
            counts.append(len(args))
            stream_slots.append(len(args) - 1)            # every launching entry point ends with its stream
            for a in args:
                slots.append(self._slot(a))
        n = len(doors)
        block = (ctypes.c_ulonglong * max(len(slots), 1))(*slots)
        handle = ctypes.c_void_p()
        native.check(native.lib().llmh_plan_create(
            n, (ctypes.c_void_p * max(n, 1))(*doors), native.ints(counts), native.ints(stream_slots),
            ctypes.cast(block, ctypes.c_void_p), ctypes.byref(handle)))
        self._handle = handle
        self.kernels = recording.kernels
        self.launches = n
        self.scratch_generation = _scratch_generation
        self._libraries = [c[0] for c in recording.calls]
        self._failed = ctypes.c_int(-1)

    def _slot(self, a) -> int:
        """The 8-byte slot of a ctypes argument: an address, a widened integer, or a double's bits."""
        if a is None:
            return 0
        if isinstance(a, ctypes.c_void_p):
            return a.value or 0
        if isinstance(a, (ctypes.c_int, ctypes.c_longlong, ctypes.c_ulonglong)):
            return a.value & 0xFFFFFFFFFFFFFFFF
        if isinstance(a, ctypes.c_float):
            return ctypes.c_ulonglong.from_buffer_copy(ctypes.c_double(a.value)).value
        target = getattr(a, "_obj", None)                 # byref(structure): the structure lives on here
        if target is not None:
            self._keep.append(target)
            return ctypes.addressof(target)
        raise KernelError(f"a launch argument of type {type(a).__name__} cannot be recorded")

    def __del__(self):
        handle = getattr(self, "_handle", None)
        if handle and native is not None:                 # (modules are gone when the interpreter ends)
            native.lib().llmh_plan_destroy(handle)
            self._handle = None

    def run(self) -> None:
        global _launches
        code = native.lib().llmh_plan_run(self._handle, _stream(), ctypes.byref(self._failed))
        _launches += self.kernels
        if code != 0:
            lib_name = self._libraries[self._failed.value]
            reader = getattr(load_library(lib_name), f"llmb_{lib_name}_last_error")
            reader.restype = ctypes.c_char_p
            raise KernelError(f"recorded launch {self._failed.value} ({lib_name}): "
                              f"{reader().decode('utf-8', 'replace')}")


def scratch_generation() -> int:
    return _scratch_generation


def _call(lib_name: str, fn_name: str, *args, kernels: int = 1):
    global _launches
    lib = load_library(lib_name)
    _launches += kernels
    if _recording is not None:
        _recording.calls.append((lib_name, fn_name, args))
        _recording.kernels += kernels
    if PROFILING and not torch.cuda.is_current_stream_capturing():
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        code = getattr(lib, fn_name)(*args)
        end.record()
        _profile.setdefault(fn_name, []).append((begin, end))
    else:
        code = getattr(lib, fn_name)(*args)
    if code != 0:
        reader = getattr(lib, f"llmb_{lib_name}_last_error")
        reader.restype = ctypes.c_char_p
        raise KernelError(f"{fn_name}: {reader().decode('utf-8', 'replace')}")


# ----------------------------------------------------------------------------- row-wise

def embed(tokens, table, out=None, scale: float = 1.0, emit=None):
    """x[t, :] = table[tokens[t], :] * scale as float32 [T, hidden]. With `emit` (an Emit) the
    rows are also written as bfloat16 with the sum of their squares: the first norm's input."""
    _require_cuda(tokens, table)
    n, (vocab, hidden) = tokens.numel(), table.shape
    _check_out(out, (n, hidden), torch.float32, "embed")
    if out is None:
        out = torch.empty((n, hidden), dtype=torch.float32, device=table.device)
    if emit is not None:
        emit.check(n, hidden)
        emit.parts = 1
    _call("elementwise", "llmb_embed", _ptr(tokens), _ptr(table), _c_int(_code(table.dtype)),
          _ptr(out), _c_int(n), _c_int(hidden), _c_int(vocab), _c_float(scale),
          _ptr(emit.rows) if emit is not None else None, _ptr(emit.sumsq) if emit is not None else None,
          _stream())
    return out


SUMSQ_LD = 64          # floats per row of a sum-of-squares array (LLMB_SUMSQ_LD of csrc/fusion.h)


class Emit:
    """Where a product that adds into the residual stream (or the embedding) leaves the next
    norm's input: `rows` bfloat16 [T, hidden], the updated residual rows, and `sumsq` float32
    [T, 64], partial sums of their squares; `parts` says how many of the 64 are in use (set by
    the op that wrote them)."""
    __slots__ = ("rows", "sumsq", "parts")

    def __init__(self, rows, sumsq):
        self.rows, self.sumsq, self.parts = rows, sumsq, 0

    def check(self, n: int, width: int) -> None:
        _require_cuda(self.rows, self.sumsq)
        if (tuple(self.rows.shape) != (n, width) or self.rows.dtype != torch.bfloat16 or not self.rows.is_contiguous()
                or tuple(self.sumsq.shape) != (n, SUMSQ_LD) or self.sumsq.dtype != torch.float32
                or not self.sumsq.is_contiguous()):
            raise KernelError(f"emit: rows must be contiguous bfloat16 [{n}, {width}] and sumsq float32 "
                              f"[{n}, {SUMSQ_LD}]")


class FoldedNorm:
    """The input of a product whose norm is folded into it: `rows` are the un-normalised rows as
    bfloat16, the norm's gain is already multiplied into the weight's columns, and the product
    scales result row t by 1 / sqrt(sum(sumsq[t, :parts]) / width + eps)."""
    __slots__ = ("rows", "sumsq", "parts", "eps", "width")

    def __init__(self, rows, sumsq, parts: int, eps: float, width: int):
        self.rows, self.sumsq, self.parts, self.eps, self.width = rows, sumsq, parts, eps, width


class RopeWrite:
    """The rotation and cache write behind the q/k/v product (the arguments of rope_cache_write)."""
    __slots__ = ("table", "tok_pos", "tok_seq", "block_table", "ring_pages", "k_cache", "v_cache",
                 "n_heads", "n_kv_heads", "head_dim", "interleaved", "write_cache")

    def __init__(self, table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache, n_heads,
                 n_kv_heads, head_dim, interleaved=False, write_cache=True):
        self.table, self.tok_pos, self.tok_seq, self.block_table = table, tok_pos, tok_seq, block_table
        self.ring_pages, self.k_cache, self.v_cache = ring_pages, k_cache, v_cache
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.interleaved, self.write_cache = interleaved, write_cache


class _Fusion(ctypes.Structure):
    """llmb_gemm_fusion of csrc/fusion.h."""
    _fields_ = [("norm_sumsq", ctypes.c_void_p), ("norm_parts", ctypes.c_int), ("norm_eps", ctypes.c_float),
                ("norm_width", ctypes.c_float), ("emit_rows", ctypes.c_void_p), ("emit_sumsq", ctypes.c_void_p),
                ("rope", ctypes.c_int), ("interleaved", ctypes.c_int), ("write_cache", ctypes.c_int),
                ("n_heads", ctypes.c_int), ("n_kv_heads", ctypes.c_int), ("head_dim", ctypes.c_int),
                ("rope_table", ctypes.c_void_p), ("tok_pos", ctypes.c_void_p), ("tok_seq", ctypes.c_void_p),
                ("block_table", ctypes.c_void_p), ("table_stride", ctypes.c_int), ("ring_pages", ctypes.c_int),
                ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p)]


FUSED_NORM, FUSED_EMIT, FUSED_ROPE = 1, 2, 4


def cast_sumsq(x, emit: Emit):
    """emit.rows = bfloat16(x), emit.sumsq[:, 0] = the rows' sums of squares (x float32 [T, hidden])."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("cast_sumsq: x must be contiguous float32")
    emit.check(x.shape[0], x.shape[1])
    _call("elementwise", "llmb_cast_sumsq", _ptr(x), _ptr(emit.rows), _ptr(emit.sumsq), _c_int(x.shape[0]),
          _c_int(x.shape[1]), _stream())
    emit.parts = 1
    return emit


def random_normal_(out, key: int, mean: float, deviation: float):
    """out[i] = mean + deviation * N(0, 1) drawn from (key, i); float32 or bfloat16, contiguous."""
    _require_cuda(out)
    if not out.is_contiguous():
        raise KernelError("random_normal_: the tensor must be contiguous")
    _call("elementwise", "llmb_random_normal", _ptr(out), _c_int(_code(out.dtype)),
          ctypes.c_longlong(out.numel()), ctypes.c_ulonglong(key), _c_float(mean), _c_float(deviation),
          _stream())
    return out


def scale_(x, scale: float):
    """x *= scale in place (float32, contiguous)."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_: the tensor must be contiguous float32")
    _call("elementwise", "llmb_scale", _ptr(x), ctypes.c_longlong(x.numel()), _c_float(scale), _stream())
    return x


def softcap_(x, cap: float):
    """x = cap * tanh(x / cap) in place (float32, contiguous)."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("softcap_: the tensor must be contiguous float32")
    _call("elementwise", "llmb_softcap", _ptr(x), ctypes.c_longlong(x.numel()), _c_float(cap), _stream())
    return x


def add_rows_(x, y, emit=None):
    """x += y in place (both contiguous float32 [T, hidden]). With `emit` (an Emit) the sums are also
    left as bfloat16 rows with the sums of their squares: the next norm's input."""
    _require_cuda(x, y)
    if (x.dtype != torch.float32 or y.dtype != torch.float32 or x.shape != y.shape or not x.is_contiguous()
            or not y.is_contiguous()):
        raise KernelError("add_rows_: both tensors must be contiguous float32 of one shape")
    if emit is not None:
        emit.check(x.shape[0], x.shape[1])
        emit.parts = 1
    _call("elementwise", "llmb_add_rows", _ptr(x), _ptr(y), _c_int(x.shape[0]), _c_int(x.shape[1]),
          _ptr(emit.rows) if emit is not None else None, _ptr(emit.sumsq) if emit is not None else None, _stream())
    return x


def rmsnorm(x, gain, eps, out_dtype, rows=None, out=None):
    """out[r, :] = x[rows[r] or r, :] / sqrt(mean(x^2) + eps) * gain; x and gain float32."""
    _require_cuda(x, gain, rows)
    hidden = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if x.dtype != torch.float32 or gain.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("rmsnorm: x and gain must be float32, x contiguous")
    _check_out(out, (n, hidden), out_dtype, "rmsnorm")
    if out is None:
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    _call("elementwise", "llmb_rmsnorm", _ptr(x), _ptr(gain), _ptr(rows), _ptr(out),
          _c_int(_code(out_dtype)), _c_int(n), _c_int(hidden), _c_float(eps), _stream())
    return out


def tanh_norm(x, alpha: float, gain, bias, out_dtype, rows=None, out=None, second=None):
    """out[r, :] = tanh(alpha * x[rows[r] or r, :]) * gain + bias; x, gain and bias float32. `second`
    (alpha, gain, bias, out): a second norm of the same rows, written by the same launch."""
    _require_cuda(x, gain, bias, rows)
    hidden = x.shape[-1]
    n = rows.numel() if rows is not None else x.shape[0]
    if (x.dtype != torch.float32 or gain.dtype != torch.float32 or bias.dtype != torch.float32
            or not x.is_contiguous() or gain.numel() != hidden or bias.numel() != hidden):
        raise KernelError("tanh_norm: x, gain and bias must be float32, x contiguous, gain and bias of x's width")
    _check_out(out, (n, hidden), out_dtype, "tanh_norm")
    if out is None:
        out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    alpha2, gain2, bias2, out2 = second if second is not None else (0.0, None, None, None)
    if second is not None:
        _require_cuda(gain2, bias2, out2)
        _check_out(out2, (n, hidden), out_dtype, "tanh_norm")
        if gain2.dtype != torch.float32 or bias2.dtype != torch.float32 or gain2.numel() != hidden or bias2.numel() != hidden:
            raise KernelError("tanh_norm: the second gain and bias must be float32 of x's width")
    _call("elementwise", "llmb_tanh_norm", _ptr(x), _ptr(gain), _ptr(bias), _c_float(alpha), _ptr(rows), _ptr(out),
          _c_float(alpha2), _ptr(gain2), _ptr(bias2), _ptr(out2), _c_int(_code(out_dtype)), _c_int(n), _c_int(hidden),
          _stream())
    return out


def _check_rows(t, n: int, width: int, dtype, what: str):
    """A [n, width] tensor of `dtype` whose rows are contiguous (it may be a range of columns of a wider one)."""
    _require_cuda(t)
    if t.dim() != 2 or tuple(t.shape) != (n, width) or t.dtype != dtype or (width > 1 and t.stride(1) != 1):
        raise KernelError(f"{what}: {tuple(t.shape)} {t.dtype} is not [{n}, {width}] {dtype} with contiguous rows")


def norm_rope_cache_write(u, q_width, k_width, v_width, q_gain, k_gain, eps, rope_table, rot_unit, interleaved,
                          tok_pos, tok_seq, q_out, block_table, ring_pages, k_cache, v_cache, write_cache=True,
                          value_source=None, norm_unit: int = 0, mix_cache=None, mix_table=None, mix_ring: int = 0,
                          mix: float = 0.0):
    """What lies between a projection and the attention of a mixer that norms whole projections:
    the first q_width columns of `u` are the queries, the next k_width the keys, the next v_width
    the values (u may have more columns). With `q_gain` (float32 [q_width]) the queries of a token
    are divided by the root of (the mean of all their squares + eps) and multiplied by the gain;
    `k_gain` does the same for the keys. Then every unit of `rot_unit` columns of both is rotated
    by `rope_table` [positions, n_rot] (None: no rotation). Queries go to `q_out` [T, q_width],
    keys into k_cache [pages, Hk, 64, Dk] (Hk * Dk = k_width), values (v_width > 0) into v_cache
    [pages, Hv, 64, Dv]. Sums, the norm's factor and angles are 32-bit. `value_source` (a column of u;
    default q_width + k_width): where a token's values start; q_width makes the values the keys as
    projected, before norm and rotation (a mixer without a value projection).

    `norm_unit` > 0: the norms run over units of that many columns (a head each) with gains of norm_unit
    elements that all units share. `mix_cache` (a value cache of another layer, same shape as `v_cache`, with
    its page table `mix_table` and ring `mix_ring`): the values are blended before they are cached,
    v <- (1 - mix) v + mix * (the row that cache holds for the same token), in 32-bit, rounded once."""
    _require_cuda(u, q_gain, k_gain, rope_table, tok_pos, tok_seq, q_out, block_table, k_cache, v_cache, mix_cache, mix_table)
    n = q_out.shape[0]
    if value_source is None:
        value_source = q_width + k_width
    if (u.dim() != 2 or u.shape[0] != n or u.shape[1] < max(q_width + k_width, value_source + v_width) or u.stride(1) != 1
            or value_source < 0):
        raise KernelError(f"norm_rope_cache_write: u {tuple(u.shape)} does not hold [{n}, {q_width} + {k_width} + {v_width}]")
    _check_rows(q_out, n, q_width, u.dtype, "norm_rope_cache_write: q_out")
    if norm_unit < 0 or (norm_unit and (q_width % norm_unit or k_width % norm_unit)):
        raise KernelError(f"norm_rope_cache_write: units of {norm_unit} columns do not divide {q_width} and {k_width}")
    for gain, width in ((q_gain, norm_unit or q_width), (k_gain, norm_unit or k_width)):
        if gain is not None and (gain.dtype != torch.float32 or gain.numel() != width or not gain.is_contiguous()):
            raise KernelError(f"norm_rope_cache_write: a gain must be contiguous float32 [{width}]")
    if mix_cache is not None and (mix_table is None or mix_ring < 1 or not v_width or v_cache is None
                                  or mix_cache.dtype != v_cache.dtype or tuple(mix_cache.shape[1:]) != tuple(v_cache.shape[1:])
                                  or not mix_cache.is_contiguous() or mix_table.shape[0] != block_table.shape[0]):
        raise KernelError("norm_rope_cache_write: the cache whose values are blended in must have the value cache's "
                          "head count and width, and come with its page table")
    n_rot = 0
    if rope_table is not None:
        n_rot = rope_table.shape[1]
        if (rope_table.dtype != torch.float32 or not rope_table.is_contiguous() or n_rot % 2 or n_rot > rot_unit
                or q_width % rot_unit or k_width % rot_unit):
            raise KernelError("norm_rope_cache_write: the table of angles must be contiguous float32 [positions, n_rot] "
                              f"with an even n_rot <= {rot_unit}, and the units must divide both widths")
    if (k_cache.dtype != u.dtype or not k_cache.is_contiguous() or k_cache.shape[1] * k_cache.shape[3] != k_width
            or k_cache.shape[2] != PAGE):
        raise KernelError(f"norm_rope_cache_write: the key cache {tuple(k_cache.shape)} does not fit keys of {k_width}")
    if v_width and (v_cache is None or v_cache.dtype != u.dtype or not v_cache.is_contiguous()
                    or v_cache.shape[1] * v_cache.shape[3] != v_width or v_cache.shape[2] != PAGE):
        raise KernelError(f"norm_rope_cache_write: the value cache does not fit values of {v_width}")
    _call("projection_norm", "llmb_norm_rope_cache_write", _ptr(u), _c_int(u.stride(0)), _c_int(_code(u.dtype)),
          _c_int(q_width), _c_int(k_width), _c_int(v_width), _ptr(q_gain), _ptr(k_gain), _c_float(eps),
          _ptr(rope_table), _c_int(n_rot), _c_int(rot_unit), _c_int(1 if interleaved else 0), _ptr(tok_pos),
          _ptr(tok_seq), _ptr(q_out), _c_int(q_out.stride(0)), _ptr(block_table), _c_int(block_table.shape[1]),
          _c_int(ring_pages), _ptr(k_cache), _c_int(k_cache.shape[1]), _ptr(v_cache if v_width else None),
          _c_int(v_cache.shape[1] if v_width else 0), _c_int(1 if write_cache else 0), _c_int(value_source),
          _c_int(norm_unit), _ptr(mix_cache), _ptr(mix_table), _c_int(mix_table.shape[1] if mix_table is not None else 0),
          _c_int(mix_ring), _c_float(mix), _c_int(n), _stream())
    return q_out


# ----------------------------------------------------------------------------- norms on both sides of a part

def norm_add_(x, y, gain_post, eps_post, terms: int = 1, gain_next=None, eps_next: float = 0.0, out=None,
              out_dtype=None):
    """x[t] += s / sqrt(mean(s^2) + eps_post) * gain_post with s = sum_k y[t * terms + k] (y float32
    [T * terms, hidden]): the norm behind a part and the residual sum. With `gain_next` also
    out[t] = x[t] / sqrt(mean(x[t]^2) + eps_next) * gain_next in `out_dtype`: the norm in front of the
    next part, of the updated rows. Returns `out` (or None)."""
    _require_cuda(x, y, gain_post, gain_next, out)
    n, hidden = x.shape
    if (x.dtype != torch.float32 or y.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous()
            or tuple(y.shape) != (n * terms, hidden) or gain_post.dtype != torch.float32 or gain_post.numel() != hidden):
        raise KernelError(f"norm_add_: x {tuple(x.shape)} and y {tuple(y.shape)} must be contiguous float32 "
                          f"[T, hidden] and [T * {terms}, hidden], the gain float32 [hidden]")
    if gain_next is not None:
        if gain_next.dtype != torch.float32 or gain_next.numel() != hidden:
            raise KernelError("norm_add_: the next norm's gain must be float32 [hidden]")
        out_dtype = out_dtype or (out.dtype if out is not None else torch.float32)
        _check_out(out, (n, hidden), out_dtype, "norm_add_")
        if out is None:
            out = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
    else:
        out = None
    _call("post_norm", "llmb_norm_add", _ptr(y), _c_int(terms), _ptr(gain_post), _c_float(eps_post), _ptr(x),
          _ptr(gain_next), _c_float(eps_next), _ptr(out), _c_int(_code(out.dtype) if out is not None else 0),
          _c_int(n), _c_int(hidden), _stream())
    return out


def gelu_(a):
    """a = 0.5 a (1 + tanh(sqrt(2 / pi) (a + 0.044715 a^3))) in place (contiguous; 32-bit arithmetic)."""
    _require_cuda(a)
    if not a.is_contiguous():
        raise KernelError("gelu_: the tensor must be contiguous")
    _call("post_norm", "llmb_gelu", _ptr(a), _c_int(_code(a.dtype)), ctypes.c_longlong(a.numel()), _stream())
    return a


def sigmoid_gate_(out, gate):
    """out[t, c] *= sigmoid(gate[t, c]); both [T, width] of one dtype with contiguous rows (either may be a
    range of columns of a wider buffer)."""
    _require_cuda(out, gate)
    n, width = out.shape
    _check_rows(gate, n, width, out.dtype, "sigmoid_gate_: gate")
    _check_rows(out, n, width, out.dtype, "sigmoid_gate_: out")
    _call("post_norm", "llmb_sigmoid_gate", _ptr(out), _c_int(out.stride(0)), _ptr(gate), _c_int(gate.stride(0)),
          _c_int(_code(out.dtype)), _c_int(n), _c_int(width), _stream())
    return out


def add_terms_(x, y, terms: int):
    """x[t] += sum_k y[t * terms + k], the terms in index order (both contiguous float32)."""
    _require_cuda(x, y)
    n, hidden = x.shape
    if (x.dtype != torch.float32 or y.dtype != torch.float32 or not x.is_contiguous() or not y.is_contiguous()
            or y.numel() < n * terms * hidden):
        raise KernelError("add_terms_: x [T, hidden] and y [T * terms, hidden] must be contiguous float32")
    _call("post_norm", "llmb_add_terms", _ptr(x), _ptr(y), _c_int(terms), _c_int(n), _c_int(hidden), _stream())
    return x


def fill_(x, value: float):
    """x[:] = value (float32, contiguous)."""
    _require_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("fill_: the tensor must be contiguous float32")
    _call("post_norm", "llmb_fill", _ptr(x), ctypes.c_longlong(x.numel()), _c_float(value), _stream())
    return x


# ----------------------------------------------------------------------------- gated delta rule

def delta_rule_work_width(n_heads: int, n_kv_heads: int, dim: int, vdim: int) -> int:
    """Floats of a token's 32-bit work row: unit q and k, v, beta and decay per head, k.q per key head; rounded up to
    16 bytes so that a row starts where a 16-byte copy may start."""
    return (2 * n_kv_heads * dim + n_heads * vdim + 2 * n_heads + n_kv_heads + 3) // 4 * 4


def delta_rule(proj, taps, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, unit_eps, norm_weight, eps, work, o,
               mixed, n_heads, n_kv_heads, dim, vdim):
    """The gated delta rule behind its projection. `proj` [T, >= C + H V + 2 H] (run dtype, rows
    contiguous) holds per token [q (G D) | k (G D) | v (H V) | gate (H V) | b (H) | a (H)], C = 2 G D + H V.
    q, k, v pass a causal convolution per channel (`taps` float32 [C, K], the last column the current
    token's) and silu; q and k become unit vectors per head (q also times D^-1/2); beta = sigmoid(b);
    decay = exp(rate * softplus(a + dt_bias)) (`rate` float32 [H], negative). Per head, token by token:
    M_t = a_t M_{t-1} + k_t w_t^T with w_t = b_t (v_t - a_t M_{t-1}^T k_t) (a_t the decay, b_t = beta); o_t = M_t^T q_t. Then o / sqrt(mean(o^2) + eps) *
    norm_weight * silu(gate) into `mixed` [T, H V] (run dtype). `state` float32 [slots, (K - 1) C + H D V]:
    the convolution's last inputs, then S; read and updated for the slots of the step. `work` float32
    [T, delta_rule_work_width], `o` float32 [T, H V]: scratch."""
    _require_cuda(proj, taps, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, norm_weight, work, o, mixed)
    n = proj.shape[0]
    H, G, D, V = n_heads, n_kv_heads, dim, vdim
    C = 2 * G * D + H * V
    n_taps = taps.shape[1]
    if proj.dim() != 2 or proj.shape[1] < C + H * V + 2 * H or proj.stride(1) != 1:
        raise KernelError(f"delta_rule: the projection {tuple(proj.shape)} does not hold {C + H * V + 2 * H} columns")
    _check_rows(mixed, n, H * V, proj.dtype, "delta_rule: mixed")
    for t, shape, what in ((taps, (C, n_taps), "taps"), (rate, (H,), "rate"), (dt_bias, (H,), "dt_bias"),
                           (norm_weight, (V,), "norm weight"), (o, (n, H * V), "o")):
        if t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous():
            raise KernelError(f"delta_rule: {what} must be contiguous float32 {shape}")
    width = delta_rule_work_width(H, G, D, V)
    if work.dtype != torch.float32 or work.dim() != 2 or work.shape[0] < n or work.shape[1] < width or not work.is_contiguous():
        raise KernelError(f"delta_rule: work must be contiguous float32 [T, >= {width}]")
    need = (n_taps - 1) * C + H * D * V
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < need or state.stride(1) != 1:
        raise KernelError(f"delta_rule: the state must be float32 [slots, >= {need}]")
    _call("delta_rule", "llmb_delta_rule", _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(taps),
          _c_int(n_taps), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(tok_seq), _ptr(cu_seqlens),
          _ptr(slot_ids), _ptr(rate), _ptr(dt_bias), _c_float(unit_eps), _ptr(norm_weight), _c_float(eps), _ptr(work),
          _c_int(work.shape[1]), _ptr(o), _ptr(mixed), _c_int(mixed.stride(0)), _c_int(n), _c_int(cu_seqlens.numel() - 1),
          _c_int(H), _c_int(G), _c_int(D), _c_int(V), _stream(), kernels=4 if n_taps > 1 else 3)
    return mixed


# ----------------------------------------------------------------------------- state-space recurrence

def state_space_work_width(n_heads: int, groups: int, state: int, vdim: int) -> int:
    """Floats of a token's 32-bit work row: x, B, C behind the convolution, the step size and the decay per head."""
    return (n_heads * vdim + 2 * groups * state + 2 * n_heads + 3) // 4 * 4


def state_space(proj, taps, conv_bias, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, skip, norm_weight, eps,
                norm_groups, out_scale, work, y, mixed, n_heads, groups, n_state, vdim):
    """A state-space recurrence with a scalar decay per head, behind its projection. `proj` [T, >= 2 H V + 2 G N + H]
    (run dtype, rows contiguous) holds per token [z (H V) | x (H V) | B (G N) | C (G N) | dt (H)]. x, B and C pass a
    causal convolution per channel (`taps` float32 [C, K], the last column the current token's; `conv_bias` float32
    [C] or None) and silu; dt <- softplus(dt + dt_bias); per head (a group of B and C serves H / G heads)
    S_t = exp(rate dt) S_(t-1) + dt B_t x_t^T and y_t = S_t^T C_t + skip x_t (`rate` float32 [H], negative; `skip`
    float32 [H] or None). Then y silu(z), divided by its root mean square in `norm_groups` equal parts (eps), times
    `norm_weight` float32 [H V] and `out_scale`, into `mixed` [T, H V] (run dtype). `state` float32 [slots,
    (K - 1) C + H V N]: the convolution's last inputs, then S as [H, V, N]; read and updated for the slots of the step.
    `work` float32 [T, state_space_work_width], `y` float32 [T, H V]: scratch."""
    _require_cuda(proj, taps, conv_bias, state, tok_seq, cu_seqlens, slot_ids, rate, dt_bias, skip, norm_weight, work, y, mixed)
    n = proj.shape[0]
    H, G, N, V = n_heads, groups, n_state, vdim
    inner = H * V
    C = inner + 2 * G * N
    n_taps = taps.shape[1]
    if proj.dim() != 2 or proj.shape[1] < inner + C + H or proj.stride(1) != 1:
        raise KernelError(f"state_space: the projection {tuple(proj.shape)} does not hold {inner + C + H} columns")
    _check_rows(mixed, n, inner, proj.dtype, "state_space: mixed")
    for t, shape, what in ((taps, (C, n_taps), "taps"), (conv_bias, (C,), "the convolution's bias"), (rate, (H,), "rate"),
                           (dt_bias, (H,), "dt_bias"), (skip, (H,), "skip"), (norm_weight, (inner,), "norm weight"),
                           (y, (n, inner), "y")):
        if t is not None and (t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous()):
            raise KernelError(f"state_space: {what} must be contiguous float32 {shape}")
    width = state_space_work_width(H, G, N, V)
    if work.dtype != torch.float32 or work.dim() != 2 or work.shape[0] < n or work.shape[1] < width or not work.is_contiguous():
        raise KernelError(f"state_space: work must be contiguous float32 [T, >= {width}]")
    need = (n_taps - 1) * C + H * N * V
    if state.dtype != torch.float32 or state.dim() != 2 or state.shape[1] < need or state.stride(1) != 1:
        raise KernelError(f"state_space: the state must be float32 [slots, >= {need}]")
    if norm_groups < 1 or inner % norm_groups:
        raise KernelError(f"state_space: {inner} channels cannot be normed in {norm_groups} equal parts")
    _call("state_space", "llmb_state_space", _ptr(proj), _c_int(proj.stride(0)), _c_int(_code(proj.dtype)), _ptr(taps),
          _ptr(conv_bias), _c_int(n_taps), _ptr(state), ctypes.c_longlong(state.stride(0)), _ptr(tok_seq), _ptr(cu_seqlens),
          _ptr(slot_ids), _ptr(rate), _ptr(dt_bias), _ptr(skip), _ptr(norm_weight), _c_float(eps), _c_int(norm_groups),
          _c_float(out_scale), _ptr(work), _c_int(work.shape[1]), _ptr(y), _ptr(mixed), _c_int(mixed.stride(0)), _c_int(n),
          _c_int(cu_seqlens.numel() - 1), _c_int(H), _c_int(G), _c_int(N), _c_int(V), _stream(),
          kernels=4 if n_taps > 1 else 3)
    return mixed


# ----------------------------------------------------------------------------- routed experts

def routed_experts_plan_ints(n_tokens: int, top: int, n_experts: int) -> int:
    sizer = load_library("routed_experts").llmb_routed_experts_plan_ints
    sizer.restype = ctypes.c_longlong
    return int(sizer(_c_int(n_tokens), _c_int(top), _c_int(n_experts)))


#: the tcgen05 tiles of 128 rows are taken from this many rows an expert (on average) on; below, a step streams the
#: experts' matrices once whatever the tile, and the 32-row tiles waste less of a block
WIDE_EXPERT_ROWS = 32


def routed_experts_wide(n_tokens: int, top: int, n_experts: int, hidden: int, intermediate: int, dtype) -> bool:
    """True if a step of n_tokens takes the tcgen05 form of the experts' products (and so needs the scratch for
    the gathered rows)."""
    return (dtype == torch.bfloat16 and hidden % 8 == 0 and intermediate % 8 == 0
            and n_tokens * top >= WIDE_EXPERT_ROWS * n_experts and not tactics.is_disabled("routed_experts_tc")
            and not tactics.is_disabled("routed_experts_wide"))


def routed_experts(h, router, router_bias, w_up, w_down, top: int, ids, weights, order, plan, act, y, gathered=None,
                   scoring: int = 0, correction=None, pass_through: int = 0, weight_scale: float = 1.0):
    """A feed-forward of routed experts on the rows of h [T, hidden] (run dtype). Router logits
    z = router h + router_bias in 32-bit (`router` float32 [E, hidden]); the `top` largest are chosen and
    weighted by the softmax over them. Expert e: W_down,e (silu(W_gate,e h) * (W_up,e h)) with `w_up`
    [E, 2 F, hidden] (gate rows, then up rows) and `w_down` [E, hidden, F] in h's dtype. Leaves
    y[t * top + k] = weight[t, k] * expert_(chosen k)(h[t]) as float32 [T * top, hidden]; the caller adds the
    `top` rows of a token. Scratch: `ids` int32 [T * top], `weights` float32 [T * top], `order` int32 [T * top],
    `plan` int32 [routed_experts_plan_ints], `act` [T * top, F] in h's dtype, and, for the steps that
    routed_experts_wide names, `gathered` [T * top, hidden] in h's dtype (the rows of h in the plan's order).

    `scoring` 1: scores s = softmax(z) over all router outputs, the `top` largest of s + `correction` (float32, one
    per output; it takes part in the choice only) are chosen, weights s / (sum of the chosen s + 1e-20).
    `pass_through` > 0: the router has E + pass_through outputs, and the last ones are experts without matrices
    whose result is h itself. `weight_scale` multiplies every weight."""
    _require_cuda(h, router, router_bias, w_up, w_down, ids, weights, order, plan, act, y, gathered, correction)
    n, hidden = h.shape
    E, two_f, _ = w_up.shape
    F = two_f // 2
    if (h.stride(1) != 1 or w_up.dtype != h.dtype or w_down.dtype != h.dtype or not w_up.is_contiguous()
            or not w_down.is_contiguous() or tuple(w_up.shape) != (E, 2 * F, hidden) or tuple(w_down.shape) != (E, hidden, F)):
        raise KernelError("routed_experts: the expert matrices must be contiguous [E, 2 F, hidden] and [E, hidden, F] in h's dtype")
    outputs = E + pass_through
    if router.dtype != torch.float32 or tuple(router.shape) != (outputs, hidden) or not router.is_contiguous():
        raise KernelError(f"routed_experts: the router must be contiguous float32 [{outputs}, {hidden}]")
    for vector, what in ((router_bias, "bias"), (correction, "correction")):
        if vector is not None and (vector.dtype != torch.float32 or vector.numel() != outputs or not vector.is_contiguous()):
            raise KernelError(f"routed_experts: the router's {what} must be contiguous float32 [{outputs}]")
    a = n * top
    for t, dtype, count, what in ((ids, torch.int32, a, "ids"), (weights, torch.float32, a, "weights"),
                                  (order, torch.int32, a, "order"), (plan, torch.int32, routed_experts_plan_ints(n, top, E), "plan"),
                                  (act, h.dtype, a * F, "act"), (y, torch.float32, a * hidden, "y")):
        if t.dtype != dtype or t.numel() < count or not t.is_contiguous():
            raise KernelError(f"routed_experts: {what} must be contiguous {dtype} with at least {count} elements")
    wide = gathered is not None and routed_experts_wide(n, top, E, hidden, F, h.dtype)
    if wide and (gathered.dtype != h.dtype or gathered.numel() < a * hidden or not gathered.is_contiguous()):
        raise KernelError(f"routed_experts: gathered must be contiguous {h.dtype} with at least {a * hidden} elements")
    level = 0 if tactics.is_disabled("routed_experts_tc") else (
        (2 if tactics.is_disabled("routed_experts_wide256") else 3) if wide else 1)
    _call("routed_experts", "llmb_routed_experts", _ptr(h), _c_int(h.stride(0)), _c_int(_code(h.dtype)), _ptr(router),
          _ptr(router_bias), _ptr(w_up), _ptr(w_down), _ptr(ids), _ptr(weights), _ptr(order), _ptr(plan), _ptr(act),
          _ptr(y), _ptr(gathered if wide else None), _c_int(n), _c_int(hidden), _c_int(F), _c_int(E), _c_int(top),
          _c_int(level), _c_int(scoring), _ptr(correction), _c_int(pass_through), _c_float(weight_scale), _stream(),
          kernels=(5 if wide else 4) + (1 if pass_through else 0))
    return y


def swiglu(gate_up, out=None):
    """act[t, f] = silu(gate_up[t, f]) * gate_up[t, F + f]."""
    _require_cuda(gate_up)
    n, two_f = gate_up.shape
    width = two_f // 2
    if not gate_up.is_contiguous():
        raise KernelError("swiglu: the input must be contiguous")
    _check_out(out, (n, width), gate_up.dtype, "swiglu")
    if out is None:
        out = torch.empty((n, width), dtype=gate_up.dtype, device=gate_up.device)
    _call("elementwise", "llmb_swiglu", _ptr(gate_up), _ptr(out), _c_int(_code(gate_up.dtype)),
          _c_int(n), _c_int(width), _stream())
    return out


def rope_cache_write(qkv, rope_table, tok_pos, tok_seq, block_table, ring_pages, k_cache, v_cache,
                     n_heads, n_kv_heads, head_dim, interleaved=False, write_cache=True):
    """Rotate q (in place) and k of the fused [T, (Hq + 2 Hkv) D] projection by the
    angles of `rope_table` [positions, n_rot] (None: no rotation; n_rot <= D: only the
    first n_rot elements of a head are rotated) and store k and v of every token into the
    paged cache [pages, Hkv, 64, D]."""
    _require_cuda(qkv, rope_table, tok_pos, tok_seq, block_table, k_cache, v_cache)
    n = qkv.shape[0]
    if qkv.dim() != 2 or qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim or not qkv.is_contiguous():
        raise KernelError(f"rope_cache_write: qkv {tuple(qkv.shape)} is not contiguous "
                          f"[T, ({n_heads} + 2 * {n_kv_heads}) * {head_dim}]")
    n_rot = head_dim if rope_table is None else rope_table.shape[1]
    if rope_table is not None and (rope_table.dtype != torch.float32 or not rope_table.is_contiguous()
                                   or n_rot > head_dim or n_rot % 2):
        raise KernelError(f"rope_cache_write: the table of angles must be contiguous float32 "
                          f"[positions, n_rot] with an even n_rot <= {head_dim}")
    _call("elementwise", "llmb_rope_cache_write", _ptr(qkv), _c_int(_code(qkv.dtype)),
          _ptr(rope_table), _ptr(tok_pos), _ptr(tok_seq), _ptr(block_table),
          _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(k_cache), _ptr(v_cache),
          _c_int(n), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_int(n_rot),
          _c_int(1 if interleaved else 0), _c_int(1 if write_cache else 0), _stream())


def conv_rope_cache_write(u, conv_w, state, tok_pos, tok_seq, cu_seqlens, seq_lens, slot_ids, rope_table,
                          rot_unit, interleaved, q_out, k_width, v_width, block_table, ring_pages, k_cache,
                          v_cache, write_cache=True, single_tokens=False, conv_w_rows=None):
    """What lies between the q/k/v projection and the attention of a mixer with a short convolution:
    a causal convolution over time on every channel of `u` [T, Cq + Ck + Cv] (weights `conv_w`
    float32 [C, taps], or None for no convolution; `state` [slots, taps - 1, C] in u's dtype holds the
    rows before the step's first token and is brought up to date), then the rotation of every unit of
    `rot_unit` channels of the query and key parts by `rope_table` [positions, n_rot] (None: no
    rotation), queries to `q_out` [T, Cq], keys and values into the paged cache
    (k_cache [pages, Hk, 64, Dk], v_cache [pages, Hv, 64, Dv] with Hk * Dk = Ck, Hv * Dv = Cv).
    `single_tokens`: every sequence brings exactly one token (the kernel then shifts the state
    itself; otherwise a second kernel does). `conv_w_rows` (optional): the taps once more as
    bfloat16 [taps, C], exact copies, for the 16-byte kernel of bfloat16 runs."""
    _require_cuda(u, conv_w, conv_w_rows, state, tok_pos, tok_seq, cu_seqlens, seq_lens, slot_ids, rope_table, q_out,
                  block_table, k_cache, v_cache)
    n, q_width = q_out.shape
    channels = q_width + k_width + v_width
    if u.dim() != 2 or u.shape != (n, channels) or u.stride(1) != 1 or not q_out.is_contiguous() or q_out.dtype != u.dtype:
        raise KernelError(f"conv_rope_cache_write: u {tuple(u.shape)} does not fit [{n}, {q_width} + {k_width} + {v_width}]")
    taps = 0
    if conv_w is not None:
        taps = conv_w.shape[1]
        if conv_w.dtype != torch.float32 or conv_w.shape[0] != channels or not conv_w.is_contiguous():
            raise KernelError(f"conv_rope_cache_write: the taps must be contiguous float32 [{channels}, taps]")
        if taps > 1 and (state is None or state.dtype != u.dtype or tuple(state.shape[1:]) != (taps - 1, channels)
                         or not state.is_contiguous()):
            raise KernelError(f"conv_rope_cache_write: the state must be contiguous {u.dtype} [slots, {taps - 1}, {channels}]")
    n_rot = 0
    if rope_table is not None:
        n_rot = rope_table.shape[1]
        if rope_table.dtype != torch.float32 or not rope_table.is_contiguous():
            raise KernelError("conv_rope_cache_write: the table of angles must be contiguous float32")
    if k_cache.dtype != u.dtype or v_cache.dtype != u.dtype or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise KernelError("conv_rope_cache_write: the cache must be contiguous and of the projection's dtype")
    if conv_w_rows is not None and (conv_w is None or conv_w_rows.dtype != torch.bfloat16
                                    or tuple(conv_w_rows.shape) != (taps, channels) or not conv_w_rows.is_contiguous()):
        raise KernelError(f"conv_rope_cache_write: the taps' copy must be contiguous bfloat16 [{taps}, {channels}]")
    kernels = 2 if (conv_w is not None and taps > 1 and not single_tokens) else 1
    _call("short_conv", "llmb_conv_rope_cache_write", _ptr(u), _c_int(u.stride(0)), _c_int(_code(u.dtype)),
          _ptr(conv_w), _ptr(conv_w_rows), _c_int(taps), _ptr(state), _ptr(tok_pos), _ptr(tok_seq), _ptr(cu_seqlens), _ptr(seq_lens),
          _ptr(slot_ids), _ptr(rope_table), _c_int(n_rot), _c_int(rot_unit), _c_int(1 if interleaved else 0),
          _ptr(q_out), _c_int(q_width), _c_int(k_width), _c_int(v_width), _ptr(block_table),
          _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(k_cache), _c_int(k_cache.shape[1]),
          _c_int(k_cache.shape[3]), _ptr(v_cache), _c_int(v_cache.shape[1]), _c_int(v_cache.shape[3]),
          _c_int(1 if write_cache else 0), _c_int(n), _c_int(cu_seqlens.numel() - 1),
          _c_int(1 if single_tokens else 0), _stream(), kernels=kernels)
    return q_out


# ----------------------------------------------------------------------------- matrix product

_scratch: dict = {}
_retired: list = []      # outgrown scratch buffers, kept alive for CUDA graphs that hold their address


def _split_scratch(device, floats: int, counters: int):
    """Partial sums and tile counters of the split-K products, one pair per
    device, shared by every call on the stream (calls run one after the other).
    It grows when a call needs more; an outgrown pair is kept alive because a
    captured step may still hold its address."""
    held = _scratch.get(device)
    if held is None or held[0].numel() < floats or held[1].numel() < counters:
        n_floats = max(floats, held[0].numel() if held else 0, 1 << 23)
        n_counters = max(counters, held[1].numel() if held else 0, 1 << 14)
        global _scratch_generation
        if held is not None:
            _retired.append(held)
            _scratch_generation += 1
        held = (torch.empty(n_floats, dtype=torch.float32, device=device),
                torch.zeros(n_counters, dtype=torch.int32, device=device))
        _scratch[device] = held
    return held


def _skinny_scratch(device, m, n, k):
    lib = load_library("gemm_skinny")
    lib.llmb_gemm_skinny_scratch_bytes.restype = ctypes.c_longlong
    need = lib.llmb_gemm_skinny_scratch_bytes(_c_int(m), _c_int(n), _c_int(k))
    return _split_scratch(device, need // 4, (n + 15) // 16)


@functools.lru_cache(maxsize=4096)
def _tc_needs(m: int, n: int, k: int) -> tuple:
    """(floats of partial sums, tile counters, kernels launched) of a tcgen05 product of this shape."""
    lib = load_library("gemm_tc")
    lib.llmb_gemm_tc_scratch_floats.restype = ctypes.c_longlong
    return (lib.llmb_gemm_tc_scratch_floats(_c_int(m), _c_int(n), _c_int(k)),
            lib.llmb_gemm_tc_counters(_c_int(m), _c_int(n), _c_int(k)),
            lib.llmb_gemm_tc_kernels(_c_int(m), _c_int(n), _c_int(k)))


def _tc_scratch(device, m, n, k):
    floats, counters, _ = _tc_needs(m, n, k)
    return _split_scratch(device, floats, counters)


def tensor_core_status() -> int:
    """0, or the code of a bounded wait that ran out in a tcgen05 kernel since the
    last call (1 producer, 2 mma issuer, 3 epilogue). Call after a synchronisation."""
    return load_library("gemm_tc").llmb_gemm_tc_status()


def check_device_status() -> None:
    """Raise if a kernel of a loaded library reported a wait that ran out. Cheap (it
    reads a word of host memory); meaningful after the stream was synchronised."""
    from .build import _loaded
    for name in ("gemm_tc", "attention_prefill_tc", "routed_experts"):
        if name in _loaded:
            code = getattr(_loaded[name], f"llmb_{name}_status")()
            if code != 0:
                raise KernelError(f"{name}: a bounded wait ran out (code {code}); the results of the "
                                  "last steps are not valid")


GLU_BLOCK = native.plan_constant("glu_block")    # gate and up rows alternate in blocks of this many rows (csrc/plan.h)


def glu_fusable(n_rows: int, k: int, dtype) -> bool:
    """Whether `linear(..., glu=True)` serves a gate/up matrix of n_rows = 2 F rows."""
    return dtype == torch.bfloat16 and n_rows % (2 * GLU_BLOCK) == 0 and k % 8 == 0


def _tc_kernels(m: int, n: int, k: int) -> int:
    """Kernels one call of the tcgen05 product launches (2 where the split-K sum is its own kernel)."""
    return _tc_needs(m, n, k)[2]


def _fusion_struct(norm, emit, rope):
    f = _Fusion()
    if norm is not None:
        f.norm_sumsq, f.norm_parts = norm.sumsq.data_ptr(), norm.parts
        f.norm_eps, f.norm_width = norm.eps, float(norm.width)
    if emit is not None:
        f.emit_rows, f.emit_sumsq = emit.rows.data_ptr(), emit.sumsq.data_ptr()
    if rope is not None:
        f.rope, f.interleaved, f.write_cache = 1, int(bool(rope.interleaved)), int(bool(rope.write_cache))
        f.n_heads, f.n_kv_heads, f.head_dim = rope.n_heads, rope.n_kv_heads, rope.head_dim
        f.rope_table = rope.table.data_ptr() if rope.table is not None else None
        f.tok_pos, f.tok_seq = rope.tok_pos.data_ptr(), rope.tok_seq.data_ptr()
        f.block_table, f.table_stride = rope.block_table.data_ptr(), rope.block_table.shape[1]
        f.ring_pages, f.k_cache, f.v_cache = rope.ring_pages, rope.k_cache.data_ptr(), rope.v_cache.data_ptr()
    return f


@functools.lru_cache(maxsize=4096)
def _tc_emit_parts(m: int, n: int, k: int) -> int:
    return load_library("gemm_tc").llmb_gemm_tc_emit_parts(_c_int(m), _c_int(n), _c_int(k))


def _check_norm(norm, m, k):
    if (norm.sumsq.dtype != torch.float32 or tuple(norm.sumsq.shape) != (m, SUMSQ_LD)
            or not norm.sumsq.is_contiguous() or not 1 <= norm.parts <= SUMSQ_LD):
        raise KernelError(f"linear: a folded norm needs sums of squares as contiguous float32 [{m}, {SUMSQ_LD}] "
                          f"with 1 to {SUMSQ_LD} parts in use")


def linear(a, w, bias=None, out_dtype=None, residual=None, out=None, glu=False, norm=None, emit=None,
           rope=None):
    """a [M, K] . w [N, K]^T (+ bias [N], float32). With `residual` (float32
    [M, N]) the product is added to it in place and it is returned; otherwise a
    new [M, N] tensor of `out_dtype` (default: a's dtype). With `glu`, w holds
    gate and up rows alternating in blocks of 16 and the result is
    silu(gate) * up as [M, N / 2] in a's dtype, computed in the product's epilogue.

    What can ride along (bfloat16; where the shape's kernel does not have it, a kernel of its
    own runs behind the product, with the same result):
    `norm` (FoldedNorm): a holds un-normalised rows, w has the norm's gain folded in, and the
    rows of the result are scaled by the norm's 1 / sqrt(mean square + eps) before the bias.
    `emit` (Emit, with `residual`): the updated residual rows as bfloat16 and the partial sums
    of their squares, for the next norm. `rope` (RopeWrite): the result is the q/k/v projection;
    queries and keys are rotated, queries stay in the result, keys and values go to the cache."""
    _require_cuda(a, w, bias, residual)
    (m, k), (n, k2) = a.shape, w.shape
    if norm is not None:
        _check_norm(norm, m, k)
    if emit is not None:
        if residual is None:
            raise KernelError("linear: emit needs a residual")
        emit.check(m, n)
    fused = norm is not None or emit is not None or rope is not None
    if glu:
        if not glu_fusable(n, k, a.dtype) or bias is not None or residual is not None or a.stride(0) % 8:
            raise KernelError("linear: the gated epilogue needs bfloat16, 2 F rows with F % 16 == 0, "
                              "K % 8 == 0, no bias and no residual")
        _check_out(out, (m, n // 2), a.dtype, "linear")
        result = out if out is not None else torch.empty((m, n // 2), dtype=a.dtype, device=a.device)
        partials, counters = _tc_scratch(a.device, m, n, k)
        if emit is not None or rope is not None:
            raise KernelError("linear: the gated epilogue takes a folded norm only")
        _call("gemm_tc", "llmb_gemm_tc_ex", _ptr(a), _c_int(a.stride(0)), _ptr(w), None, _ptr(result),
              _c_int(_code(a.dtype)), None, _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k),
              _c_int(n // 2), _c_int(1), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1),
              ctypes.byref(_fusion_struct(norm, None, None)) if norm is not None else None, None,
              _stream(), kernels=_tc_kernels(m, n, k))
        return result
    if k != k2 or a.dtype != w.dtype:
        raise KernelError(f"linear: a {tuple(a.shape)} {a.dtype} does not fit w {tuple(w.shape)} {w.dtype}")
    if a.stride(1) != 1 or not w.is_contiguous():
        raise KernelError("linear: operands must be row-major")
    if residual is not None:
        target_dtype, result = torch.float32, residual
        if residual.shape != (m, n) or residual.dtype != torch.float32 or not residual.is_contiguous():
            raise KernelError("linear: residual must be contiguous float32 [M, N]")
    else:
        target_dtype = out_dtype or a.dtype
        _check_out(out, (m, n), target_dtype, "linear")
        result = out if out is not None else torch.empty((m, n), dtype=target_dtype, device=a.device)
    variant = tactics.choose_linear(m, n, k, a.dtype, target_dtype, a.stride(0),
                                    a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)
    if fused and a.dtype != torch.bfloat16:
        raise KernelError("linear: norm, emit and rope ride only with bfloat16 products")
    if variant == "gemm_tc" and fused:
        partials, counters = _tc_scratch(a.device, m, n, k)
        applied = _c_int(0)
        _call("gemm_tc", "llmb_gemm_tc_ex", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _c_int(0), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1),
              ctypes.byref(_fusion_struct(norm, emit, rope)), ctypes.byref(applied), _stream(),
              kernels=_tc_kernels(m, n, k))
        if emit is not None:
            if applied.value & FUSED_EMIT:
                emit.parts = _tc_emit_parts(m, n, k)
            else:
                cast_sumsq(residual, emit)
        if rope is not None and not applied.value & FUSED_ROPE:
            rope_cache_write(result, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                             rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                             rope.interleaved, rope.write_cache)
        return result
    if fused:
        # a variant without the fused epilogues: the plain product, then each part as its own kernel
        if norm is not None and residual is not None:
            raise KernelError("linear: a folded norm with a residual has no kernel")
        result = linear(a, w, None if norm is not None else bias, out_dtype, residual, out)
        if norm is not None:
            _call("elementwise", "llmb_scale_rows", _ptr(result), _c_int(_code(result.dtype)), _c_int(m), _c_int(n),
                  _ptr(norm.sumsq), _c_int(norm.parts), _c_float(norm.eps), _c_float(float(norm.width)),
                  _ptr(bias), _stream())
        if emit is not None:
            cast_sumsq(residual, emit)
        if rope is not None:
            rope_cache_write(result, rope.table, rope.tok_pos, rope.tok_seq, rope.block_table, rope.ring_pages,
                             rope.k_cache, rope.v_cache, rope.n_heads, rope.n_kv_heads, rope.head_dim,
                             rope.interleaved, rope.write_cache)
        return result
    if variant == "gemm_tc":
        partials, counters = _tc_scratch(a.device, m, n, k)
        _call("gemm_tc", "llmb_gemm_tc", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel()),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _c_int(0), _c_int(0 if tactics.is_disabled("gemm_tc_pair") else 1), _stream(),
              kernels=_tc_kernels(m, n, k))
    elif variant == "gemm_skinny":
        partials, counters = _skinny_scratch(a.device, m, n, k)
        _call("gemm_skinny", "llmb_gemm_skinny", _ptr(a), _c_int(a.stride(0)), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _c_int(_code(target_dtype)),
              _ptr(residual), _ptr(partials), ctypes.c_longlong(partials.numel() * 4),
              _ptr(counters), _c_int(counters.numel()), _c_int(m), _c_int(n), _c_int(k), _c_int(n),
              _stream())
    elif variant == "gemm_simt":
        _call("gemm_simt", "llmb_gemm_simt", _ptr(a), _ptr(w), _ptr(bias),
              _ptr(result if residual is None else None), _ptr(residual),
              _c_int(_code(a.dtype)), _c_int(_code(target_dtype)), _c_int(m), _c_int(n), _c_int(k),
              _c_int(a.stride(0)), _c_int(n), _stream())
    else:
        raise KernelError(f"linear: no kernel named {variant}")
    return result


# ----------------------------------------------------------------------------- attention

_attention_scratch: dict = {}      # outgrown buffers join `_retired` above


def decode_splits(n_seqs: int, n_kv_heads: int, max_len: int, wave: int = 296) -> int:
    """Into how many slices the keys of every sequence are cut for decode
    attention. Blocks are (slice, kv head, sequence) and two fit on an SM: the
    count is the largest power of two that keeps all blocks in one wave of
    2 x 148 (measured on a B200 at 8,192 positions: batch 8 is fastest with 4
    slices = 256 blocks, batch 1 with 16 to 32), and never less than two pages
    a slice. When the batch alone exceeds a wave, slices still shorten the
    longest block of work (sequences of a batch differ in length, and the step
    ends with its longest slice): one slice per 16 pages of the longest
    sequence, at most four (batch 64 at equal lengths: 28 us with one slice
    against 39 us with four at 512 positions, 334 against 352 us with four at
    8,192; 16 sequences of 64 to 2,176 positions with 32 kv heads decode
    fastest with two). One slice writes the result itself and skips the
    combining kernel. The count depends on the
    length only through the power-of-two bucket of its page count, so that all
    steps replayed from one captured graph agree on it."""
    if os.environ.get("LLMB_DECODE_SPLITS"):             # for measurements: force a slice count
        return int(os.environ["LLMB_DECODE_SPLITS"])
    pages = max(1, (max_len + PAGE - 1) // PAGE)
    floor_pages = max(1, 1 << max(0, (pages - 1).bit_length() - 1))      # the bucket is (floor, 2 floor] pages
    pairs = max(1, n_seqs * n_kv_heads)
    want = wave // pairs if pairs < wave else min(4, max(1, floor_pages // 16))     # (wave: the blocks all SMs hold at once)
    splits = 1
    while splits * 2 <= want and splits * 2 <= 32:
        splits *= 2
    while splits > 1 and splits > floor_pages // 2:
        splits //= 2
    return splits


def attention_decode_splits(n_seqs: int, n_heads: int, n_kv_heads: int, max_len: int, window: int = 0) -> int:
    """Slices of the decode attention kernel: `decode_splits` for its blocks a sequence (a group of more
    than 8 query heads is several blocks over one key/value head) and the keys a query sees at most."""
    chunks = (n_heads // max(n_kv_heads, 1) + 7) // 8
    seen = min(max_len, window + PAGE) if window > 0 else max_len
    return decode_splits(n_seqs, n_kv_heads * chunks, seen)


def attention(qkv, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads,
              n_kv_heads, head_dim, scale, window=0, out=None, decode=False, seq_lens=None,
              max_len=0, cu_seqlens=None, max_new=0, seq_order=None, sinks=None, gate=None, out_scale=1.0,
              softcap=0.0, value_dim=None):
    """Causal grouped-query attention of the new tokens' queries (the first
    Hq * D columns of `qkv`) over the paged cache, which already holds the new
    tokens' keys and values. Returns [T, Hq * D] in qkv's dtype. `seq_order`
    (optional, int32 [B]): the sequences by falling length; the kernels that
    take one block of work per sequence then start the longest first.

    `sinks` (float32 [Hq]): e^sinks[a] is one more term of head a's softmax denominator; it has
    no key and no value and is not scaled. `gate` ([T, Hq] in qkv's dtype, rows contiguous): the
    result of head a for token t is multiplied by sigmoid(gate[t, a]). `out_scale` multiplies the
    result. With any of the three, `out` may be a range of columns of a wider buffer. The value
    cache may be the key cache itself (a mixer whose values are its keys). `softcap` > 0 bounds the scaled
    scores before the softmax: s <- softcap * tanh(s / softcap). `value_dim` (default head_dim): the size of a
    value where it differs from a key's; the result is then [T, Hq * value_dim] (the kernel for any sizes)."""
    _require_cuda(qkv, k_cache, v_cache, block_table, tok_pos, tok_seq, sinks, gate)
    n = qkv.shape[0]
    value_dim = value_dim or head_dim
    extras = (sinks is not None or gate is not None or out_scale != 1.0 or softcap > 0.0 or value_dim != head_dim
              or (out is not None and not out.is_contiguous()))
    if extras:
        if out is not None:
            _check_rows(out, n, n_heads * value_dim, qkv.dtype, "attention: out")
        if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != n_heads or not sinks.is_contiguous()):
            raise KernelError(f"attention: sinks must be contiguous float32 [{n_heads}]")
        if gate is not None:
            _check_rows(gate, n, n_heads, qkv.dtype, "attention: gate")
    else:
        _check_out(out, (n, n_heads * head_dim), qkv.dtype, "attention")
    if out is None:
        out = torch.empty((n, n_heads * value_dim), dtype=qkv.dtype, device=qkv.device)
    variant = tactics.choose_attention(decode, qkv.dtype, n_heads, n_kv_heads, head_dim, window,
                                       cu_seqlens is not None and seq_lens is not None,
                                       qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0)
    if extras and variant not in _ATTENTION_WITH_EXTRAS:
        # the next choice that takes a sink, a gate, a scale and rows inside a wider buffer
        variant = "attention_generic"
        if not tactics.is_disabled("attention_prefill") and qkv.dtype == torch.bfloat16 and head_dim in (32, 64, 96, 128) \
                and cu_seqlens is not None and seq_lens is not None and qkv.stride(0) % 2 == 0 and out.stride(0) % 2 == 0 \
                and qkv.data_ptr() % 4 == 0 and out.data_ptr() % 4 == 0:
            variant = "attention_prefill"
    if value_dim != head_dim:
        variant = "attention_generic"                 # the tile kernels take values of the keys' size
    if variant == "attention_decode" and (qkv.stride(0) % 2 or qkv.data_ptr() % 4):
        variant = "attention_generic"
    if variant == "attention_prefill_tc":
        _call("attention_prefill_tc", "llmb_attention_prefill_tc", _ptr(qkv), _c_int(qkv.stride(0)),
              _c_int(n), _ptr(k_cache), _ptr(v_cache), _c_int(k_cache.shape[0]), _ptr(block_table),
              _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(cu_seqlens), _ptr(seq_lens),
              _ptr(seq_order), _ptr(out), _c_int(out.stride(0)), _c_int(cu_seqlens.numel() - 1),
              _c_int(max_new), _c_int(n_heads), _c_int(n_kv_heads), _c_int(head_dim), _c_float(scale),
              _c_int(window), _stream())
    elif variant == "attention_prefill":
        _call("attention_prefill", "llmb_attention_prefill", _ptr(qkv), _c_int(qkv.stride(0)),
              _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]),
              _c_int(ring_pages), _ptr(cu_seqlens), _ptr(seq_lens), _ptr(out), _c_int(out.stride(0)),
              _c_int(cu_seqlens.numel() - 1), _c_int(max_new), _c_int(n_heads), _c_int(n_kv_heads),
              _c_int(head_dim), _c_float(scale), _c_int(window), _ptr(sinks), _ptr(gate),
              _c_int(gate.stride(0) if gate is not None else 0), _c_float(out_scale), _c_float(softcap), _stream())
    elif variant == "attention_decode":
        # the plain grouped-query case keeps the kernel file it was tuned in; a window, a sink, a gate, a scale, a
        # value cache that is the key cache and groups above 8 run the same kernel with those additions
        plain = (window == 0 and sinks is None and gate is None and out_scale == 1.0 and n_heads // n_kv_heads <= 8
                 and softcap <= 0.0 and k_cache.data_ptr() != v_cache.data_ptr())
        name = "attention_decode" if plain else "attention_decode_window"
        splits = attention_decode_splits(n, n_heads, n_kv_heads, max_len, window)
        lib = load_library(name)
        sizer = getattr(lib, f"llmb_{name}_scratch_floats")
        sizer.restype = ctypes.c_longlong
        need = sizer(_c_int(n), _c_int(n_heads), _c_int(head_dim), _c_int(splits))
        scratch = _attention_scratch.get(qkv.device)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                global _scratch_generation
                _retired.append(scratch)
                _scratch_generation += 1
            scratch = torch.empty(max(need, 1 << 23), dtype=torch.float32, device=qkv.device)
            _attention_scratch[qkv.device] = scratch
        head = (_ptr(qkv), _c_int(qkv.stride(0)), _ptr(k_cache), _ptr(v_cache), _ptr(block_table),
                _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(seq_lens), _ptr(seq_order), _ptr(out),
                _c_int(out.stride(0)), _ptr(scratch), ctypes.c_longlong(scratch.numel()), _c_int(n), _c_int(n_heads),
                _c_int(n_kv_heads), _c_int(head_dim), _c_float(scale), _c_int(window))
        if plain:
            _call(name, "llmb_attention_decode", *head, _c_int(splits), _stream(), kernels=2 if splits > 1 else 1)
        else:
            _call(name, "llmb_attention_decode_window", *head, _ptr(sinks), _ptr(gate),
                  _c_int(gate.stride(0) if gate is not None else 0), _c_float(out_scale), _c_float(softcap),
                  _c_int(splits), _stream(), kernels=2 if splits > 1 else 1)
    elif variant == "attention_generic":
        _call("attention_generic", "llmb_attention_generic", _ptr(qkv), _c_int(qkv.stride(0)),
              _ptr(k_cache), _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]),
              _c_int(ring_pages), _ptr(tok_pos), _ptr(tok_seq), _ptr(out), _c_int(out.stride(0)),
              _c_int(_code(qkv.dtype)), _c_int(n), _c_int(n_heads), _c_int(n_kv_heads),
              _c_int(head_dim), _c_float(scale), _c_int(window), _ptr(sinks), _ptr(gate),
              _c_int(gate.stride(0) if gate is not None else 0), _c_float(out_scale), _c_float(softcap),
              _c_int(value_dim), _stream())
    else:
        raise KernelError(f"attention: no kernel named {variant}")
    return out


# the attention kernels that take a sink, a gate and a scale of the result
_ATTENTION_WITH_EXTRAS = ("attention_generic", "attention_prefill", "attention_decode")


def attention_replay_key(step, n_heads: int, n_kv_heads: int, window: int = 0):
    """What the launches of `attention` depend on beyond the token and sequence counts
    (Part.replay_key): the most new tokens of a sequence (prefill grids), the slices (decode)."""
    if step.decode:
        return (True, attention_decode_splits(step.n_seqs, n_heads, n_kv_heads, step.max_len, window))
    return (False, max(step.new_counts))


def sigmoid_decode_splits(n_seqs: int, max_len: int, window: int, mixed_width: int = 1024) -> int:
    """Slices of the decode kernel of the sigmoid attention (a block serves all heads of a sequence):
    `decode_splits` for the keys a query sees at most. Two blocks share an SM where the mixed queries are
    wide (`mixed_width` = kv heads x head size above 512), four where they are narrow."""
    seen = min(max_len, window + PAGE) if window > 0 else max_len
    return decode_splits(n_seqs, 1, seen, wave=296 if mixed_width > 512 else 592)


def sigmoid_attention_replay_key(step, spec):
    if step.decode:
        return (True, sigmoid_decode_splits(step.n_seqs, step.max_len, spec.window, spec.n_kv_heads * spec.head_dim))
    return (False, max(step.new_counts))


def sigmoid_attention(q, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads, n_kv_heads, dim, vdim,
                      scale, window, talk, head_bias, out_scale, out, decode=False, seq_lens=None, max_len=0,
                      cu_seqlens=None, max_new=0, seq_order=None):
    """Causal grouped-query attention without a softmax, of the new tokens' queries q [T, H * dim]
    over the paged cache (keys [pages, G, 64, dim], values [pages, G, 64, vdim]), which already
    holds the new tokens. For query t at position p and every key j with j <= p (and p - j <
    window, where window > 0): s_a = scale q_a . k_g(a),j; with `talk` (float32 [H, H])
    s_a <- sum_b talk[a, b] s_b; with `head_bias` (float32 [H]) s_a += head_bias[a]; then
    out[t, a] = out_scale * sum_j sigmoid(s_a) v_g(a),j. Scores, weights and sums are 32-bit.
    `out` [T, H * vdim] in q's dtype may be a range of columns of a wider buffer."""
    _require_cuda(q, k_cache, v_cache, block_table, tok_pos, tok_seq, talk, head_bias, out)
    n = q.shape[0]
    _check_rows(q, n, n_heads * dim, q.dtype, "sigmoid_attention: q")
    _check_rows(out, n, n_heads * vdim, q.dtype, "sigmoid_attention: out")
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, dim) or tuple(v_cache.shape[1:]) != (n_kv_heads, PAGE, vdim):
        raise KernelError(f"sigmoid_attention: the cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} does not fit "
                          f"{n_kv_heads} heads of {dim} and {vdim}")
    if talk is not None and (talk.dtype != torch.float32 or tuple(talk.shape) != (n_heads, n_heads) or not talk.is_contiguous()):
        raise KernelError(f"sigmoid_attention: talk must be contiguous float32 [{n_heads}, {n_heads}]")
    if head_bias is not None and (head_bias.dtype != torch.float32 or head_bias.numel() != n_heads):
        raise KernelError(f"sigmoid_attention: head_bias must be float32 [{n_heads}]")
    variant = tactics.choose_sigmoid_attention(
        decode, q.dtype, n_heads, n_kv_heads, dim, vdim, window, cu_seqlens is not None and seq_lens is not None,
        q.stride(0) % 2 == 0 and out.stride(0) % 2 == 0 and q.data_ptr() % 4 == 0 and out.data_ptr() % 4 == 0)
    if variant == "sigmoid_attention_decode":
        splits = sigmoid_decode_splits(n, max_len, window, n_kv_heads * dim)
        need = (n * (16 if n_heads <= 16 else 32) * n_kv_heads * dim + 1) // 2 + (n * splits * n_heads * vdim if splits > 1 else 0)
        scratch = _attention_scratch.get(q.device)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                global _scratch_generation
                _retired.append(scratch)
                _scratch_generation += 1
            scratch = torch.empty(max(need, 1 << 23), dtype=torch.float32, device=q.device)
            _attention_scratch[q.device] = scratch
        _call("sigmoid_attention", "llmb_sigmoid_attention_decode", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(seq_lens),
              _ptr(out), _c_int(out.stride(0)), _ptr(scratch), ctypes.c_longlong(scratch.numel()), _c_int(n),
              _c_int(n_heads), _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale), _c_int(window),
              _ptr(talk), _ptr(head_bias), _c_float(out_scale), _c_int(splits), _stream(), kernels=3 if splits > 1 else 2)
        return out
    if variant == "sigmoid_attention_tiles":
        _call("sigmoid_attention", "llmb_sigmoid_attention_tiles", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(cu_seqlens),
              _ptr(seq_lens), _ptr(out), _c_int(out.stride(0)), _c_int(cu_seqlens.numel() - 1), _c_int(max_new),
              _c_int(n_heads), _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale), _c_int(window),
              _ptr(talk), _ptr(head_bias), _c_float(out_scale), _stream())
        return out
    _call("sigmoid_attention", "llmb_sigmoid_attention_generic", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
          _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(tok_pos),
          _ptr(tok_seq), _ptr(out), _c_int(out.stride(0)), _c_int(_code(q.dtype)), _c_int(n), _c_int(n_heads),
          _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale), _c_int(window), _ptr(talk), _ptr(head_bias),
          _c_float(out_scale), _stream())
    return out


def gated_recurrence(y, x, conv_w, conv_b, gate_a, gate_a_bias, gate_i, gate_i_bias, rate, state, tok_seq,
                     cu_seqlens, slot_ids, out, out_scale, work, single_tokens=False):
    """A real-gated linear recurrence behind a short causal convolution, on C channels. `y`, `x`
    [T, C] (the run's dtype; rows contiguous, may be column ranges): the two branches' projections
    with their biases. u = conv_b + sum_j conv_w[:, j] * x[t - (taps - 1) + j] over the tokens of
    a sequence (conv_w float32 [C, taps]; the inputs before the step's first token come from the
    state). The channels are cut into gate_a.shape[0] equal parts; in part b,
    r = sigmoid(gate_a[b] u_b + gate_a_bias), i = sigmoid(gate_i[b] u_b + gate_i_bias) (float32
    [blocks, C / blocks, C / blocks], rows = outputs). a = exp(rate * r) (rate float32 [C], negative),
    S <- a S + sqrt(1 - a^2) i u, out[t] = out_scale * S * gelu(y[t]) (tanh form). `state` float32
    [slots, taps, C]: rows 0 .. taps - 2 the convolution's last inputs (oldest first), the last row
    S; it is read at the slot of each sequence and brought up to date. `work` float32 [3, T, C]:
    u, a and the driving term of every token, between the three kernels. Everything but the rounding of
    `out` is 32-bit. `single_tokens`: every sequence brings exactly one token (token b is sequence b's)."""
    _require_cuda(y, x, conv_w, conv_b, gate_a, gate_a_bias, gate_i, gate_i_bias, rate, state, tok_seq, cu_seqlens,
                  slot_ids, out, work)
    n, channels = y.shape
    taps, blocks = conv_w.shape[1], gate_a.shape[0]
    _check_rows(y, n, channels, y.dtype, "gated_recurrence: y")
    _check_rows(x, n, channels, y.dtype, "gated_recurrence: x")
    _check_rows(out, n, channels, y.dtype, "gated_recurrence: out")
    part = channels // max(blocks, 1)
    for t, shape in ((conv_w, (channels, taps)), (conv_b, (channels,)), (gate_a, (blocks, part, part)),
                     (gate_i, (blocks, part, part)), (gate_a_bias, (channels,)), (gate_i_bias, (channels,)),
                     (rate, (channels,))):
        if t.dtype != torch.float32 or tuple(t.shape) != shape or not t.is_contiguous():
            raise KernelError(f"gated_recurrence: a parameter is {tuple(t.shape)} {t.dtype}, not contiguous float32 {shape}")
    if state.dtype != torch.float32 or tuple(state.shape[1:]) != (taps, channels) or not state.is_contiguous():
        raise KernelError(f"gated_recurrence: the state must be contiguous float32 [slots, {taps}, {channels}]")
    if work.dtype != torch.float32 or tuple(work.shape) != (3, n, channels) or not work.is_contiguous():
        raise KernelError(f"gated_recurrence: work must be contiguous float32 [3, {n}, {channels}]")
    _call("gated_recurrence", "llmb_gated_recurrence", _ptr(y), _c_int(y.stride(0)), _ptr(x), _c_int(x.stride(0)),
          _c_int(_code(y.dtype)), _ptr(conv_w), _ptr(conv_b), _c_int(taps), _ptr(gate_a), _ptr(gate_a_bias),
          _ptr(gate_i), _ptr(gate_i_bias), _c_int(blocks), _ptr(rate), _ptr(state), _ptr(tok_seq), _ptr(cu_seqlens),
          _ptr(slot_ids), _ptr(out), _c_int(out.stride(0)), _c_float(out_scale), _ptr(work), _c_int(n),
          _c_int(channels), _c_int(cu_seqlens.numel() - 1), _c_int(1 if single_tokens else 0), _stream(),
          kernels=3 if n <= 256 else 5)
    return out


def diff_decode_splits(n_seqs: int, n_kv_heads: int, max_len: int, window: int, keep_first: int) -> int:
    """Slices of the decode kernel of the differential attention: `decode_splits` for the keys a query
    sees at most (with a window: the window, a page of slack, and the pages of the kept first
    tokens)."""
    seen = max_len
    if window > 0:
        seen = min(max_len, window + PAGE + (((keep_first + PAGE - 1) // PAGE) * PAGE if keep_first else 0))
    return decode_splits(n_seqs, n_kv_heads, seen)


def diff_attention_replay_key(step, spec):
    """What the launches of a differential attention depend on beyond the token and sequence counts
    (Part.replay_key): the most new tokens of a sequence (prefill grids), the slices (decode)."""
    if step.decode:
        return (True, diff_decode_splits(step.n_seqs, spec.n_kv_heads, step.max_len, spec.window, spec.keep_first))
    return (False, max(step.new_counts))


def diff_attention(q, k_cache, v_cache, block_table, ring_pages, tok_pos, tok_seq, n_heads, n_kv_heads, dim,
                   vdim, scale, window, keep_first, lam, eps, out_scale, head_norm=True, out=None, decode=False,
                   seq_lens=None, max_len=0, cu_seqlens=None, max_new=0, seq_order=None):
    """Differential attention of the new tokens' queries q [T, H * 2 * dim] (per head: map 1, map 2)
    over the paged cache (keys [pages, G, 64, 2 * dim], values [pages, G, 64, vdim]), which already
    holds the new tokens. Per head: o = a1 - lam * a2 with a1, a2 the two maps' softmax attentions
    over the same values; then (with `head_norm`) o / sqrt(mean(o^2) + eps); times out_scale. A
    query at position p sees key j <= p if window == 0, p - j < window or j < keep_first.
    Returns [T, H * vdim] in q's dtype."""
    _require_cuda(q, k_cache, v_cache, block_table, tok_pos, tok_seq)
    n = q.shape[0]
    if q.shape[1] != n_heads * 2 * dim or q.stride(1) != 1:
        raise KernelError(f"diff_attention: q {tuple(q.shape)} is not [T, {n_heads} * 2 * {dim}]")
    if tuple(k_cache.shape[1:]) != (n_kv_heads, PAGE, 2 * dim) or tuple(v_cache.shape[1:]) != (n_kv_heads, PAGE, vdim):
        raise KernelError(f"diff_attention: the cache {tuple(k_cache.shape)} / {tuple(v_cache.shape)} does not fit "
                          f"{n_kv_heads} heads of 2 * {dim} and {vdim}")
    _check_out(out, (n, n_heads * vdim), q.dtype, "diff_attention")
    if out is None:
        out = torch.empty((n, n_heads * vdim), dtype=q.dtype, device=q.device)
    variant = tactics.choose_diff_attention(decode, q.dtype, n_heads, n_kv_heads, dim, vdim, window, keep_first,
                                            cu_seqlens is not None and seq_lens is not None,
                                            q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)
    if variant == "diff_attention_prefill":
        _call("diff_attention", "llmb_diff_attention_prefill", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(cu_seqlens),
              _ptr(seq_lens), _ptr(out), _c_int(out.stride(0)), _c_int(cu_seqlens.numel() - 1), _c_int(max_new),
              _c_int(n_heads), _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale), _c_int(window),
              _c_int(keep_first), _c_float(lam), _c_float(eps), _c_float(out_scale), _c_int(1 if head_norm else 0),
              _stream())
    elif variant == "diff_attention_decode":
        splits = diff_decode_splits(n, n_kv_heads, max_len, window, keep_first)
        need = n * n_heads * 2 * splits * (vdim + 2)
        scratch = _attention_scratch.get(q.device)
        if scratch is None or scratch.numel() < need:
            if scratch is not None:
                global _scratch_generation
                _retired.append(scratch)
                _scratch_generation += 1
            scratch = torch.empty(max(need, 1 << 23), dtype=torch.float32, device=q.device)
            _attention_scratch[q.device] = scratch
        _call("diff_attention", "llmb_diff_attention_decode", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(seq_lens),
              _ptr(seq_order), _ptr(out), _c_int(out.stride(0)), _ptr(scratch), ctypes.c_longlong(scratch.numel()),
              _c_int(n), _c_int(n_heads), _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale),
              _c_int(window), _c_int(keep_first), _c_float(lam), _c_float(eps), _c_float(out_scale),
              _c_int(1 if head_norm else 0), _c_int(splits), _stream(), kernels=2 if splits > 1 else 1)
    elif variant == "diff_attention_generic":
        _call("diff_attention", "llmb_diff_attention_generic", _ptr(q), _c_int(q.stride(0)), _ptr(k_cache),
              _ptr(v_cache), _ptr(block_table), _c_int(block_table.shape[1]), _c_int(ring_pages), _ptr(tok_pos),
              _ptr(tok_seq), _ptr(out), _c_int(out.stride(0)), _c_int(_code(q.dtype)), _c_int(n), _c_int(n_heads),
              _c_int(n_kv_heads), _c_int(dim), _c_int(vdim), _c_float(scale), _c_int(window), _c_int(keep_first),
              _c_float(lam), _c_float(eps), _c_float(out_scale), _c_int(1 if head_norm else 0), _stream())
    else:
        raise KernelError(f"diff_attention: no kernel named {variant}")
    return out


# ----------------------------------------------------------------------------- sampling

def argmax_rows(logits, out=None):
    """First maximum of every row of float32 logits [B, V] as int32 [B]."""
    _require_cuda(logits)
    n, vocab = logits.shape
    if out is None:
        out = torch.empty((n,), dtype=torch.int32, device=logits.device)
    _call("sampling", "llmb_argmax_rows", _ptr(logits), _c_int(logits.stride(0)), _c_int(n),
          _c_int(vocab), _ptr(out), _stream())
    return out


def sample_rows(logits, params, iparams, recent, recent_len, rng_state, out, status, record=False,
                state_rows=None):
    """The whole sampling chain for every row; see csrc/sampling.cu. `logits`
    (float32 [B, V]) is changed where the repeat penalty applies. params float32 [B, 4],
    iparams int32 [B, 2], recent int32 [B, cap] or None, recent_len int32 [B], rng_state
    int64 [B], out int32 [B], status int32 [B]. With `record` the kernel also enters every
    drawn token into its row's window (recent, recent_len). `state_rows` (int32 [B], optional):
    row i of the logits belongs to the sequence whose parameters, window, generator and status
    are in row state_rows[i] of those arrays (which may then have more rows than the logits)."""
    _require_cuda(logits, params, iparams, recent, rng_state, out, status)
    n, vocab = logits.shape
    _call("sampling", "llmb_sample_rows", _ptr(logits), _c_int(logits.stride(0)), _c_int(n),
          _c_int(vocab), _ptr(params), _ptr(iparams), _ptr(recent), _ptr(recent_len),
          _c_int(recent.shape[1] if recent is not None else 0), _ptr(rng_state), _ptr(out),
          _ptr(status), _c_int(1 if record else 0), _ptr(state_rows), _stream())
    return out


def required_libraries() -> list:
    """Names of the kernel files the decoder parts of this package use."""
    return ["elementwise", "gemm_simt", "gemm_skinny", "gemm_tc", "attention_generic",
            "attention_decode", "attention_prefill", "attention_prefill_tc", "sampling"]


__all__ = ["PAGE", "GLU_BLOCK", "glu_fusable", "embed", "scale_", "random_normal_", "begin_recording", "end_recording", "RecordedPass", "scratch_generation", "Emit", "FoldedNorm", "RopeWrite", "cast_sumsq", "SUMSQ_LD", "rmsnorm", "swiglu", "rope_cache_write", "linear", "attention",
           "softcap_", "add_rows_", "conv_rope_cache_write", "diff_attention", "tanh_norm", "norm_rope_cache_write",
           "sigmoid_attention", "gated_recurrence", "state_space", "attention_replay_key", "attention_decode_splits", "sigmoid_attention_replay_key", "sigmoid_decode_splits",
           "argmax_rows", "sample_rows", "launch_count", "count_launches", "tensor_core_status", "check_device_status", "ensure_built", "load_library", "all_sources",
           "required_libraries", "tactics"]
