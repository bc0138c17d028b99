"""Python faces of the CUDA kernels: check sizes, pass pointers, launch on torch's current stream.

Every function refuses what its kernel cannot take with `Unsupported` (never a wrong result) and
raises `EngineError` when a launch fails. Tensors must live on the CUDA device; there is no CPU path.
"""

from __future__ import annotations

import contextlib
import os
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..errors import EngineError, InvalidArgument, Unsupported
from . import lib as _lib

DL_ERR_UNSUPPORTED = 10001

_P, _I, _F, _L = c_void_p, c_int, c_float, c_longlong

# library -> function -> argument types
_SIGNATURES = {
    "embedding": {"dl_embed": [_I, _P, _P, _P, _I, _I, _I, _F, _P]},
    "norm": {
        "dl_rmsnorm": [_I, _I, _P, _P, _F, _P, _F, _P, _P, _I, _I, _I, _I, _L, _P, _L, _P],
        "dl_residual_add": [_I, _P, _P, _F, _L, _I, _L, _P],
    },
    "activation": {"dl_silu_mul": [_I, _P, _P, _I, _I, _P]},
    "rope_cache": {
        "dl_rope_cache_write": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _F, _I, _I, _I, _I, _I, _I, _P],
        "dl_rope_angles": [_P, _P, _I, _F, _I, _P, _P]},
    "attention_generic": {
        "dl_paged_attention_generic": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P]},
    "attention_decode": {
        "dl_paged_attention_decode": [_I, _P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
        "dl_paged_attention_decode_planned": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P,
                                              _I, _I, _P, _L, _P],
        "dl_paged_attention_decode_tc": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P, _L, _P]},
    "attention_prefill": {
        "dl_paged_attention_prefill": [_P, _I, _P, _P, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P]},
    "attention_prefill_tcgen05": {
        "dl_paged_attention_prefill_tcgen05": [_P, _I, _I, _P, _P, _L, _P, _I, _P, _I, _P, _I, _I, _I, _I, _I, _F, _I, _P, _P,
                                               _P, _P, _I, _P]},
    "gemm_skinny": {
        "dl_gemm_skinny": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _L, _P, _L, _P],
        "dl_gemm_skinny_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _F, _I, _I, _I, _I, _P]},
    "gemm_tcgen05": {
        "dl_gemm_tcgen05": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
        "dl_gemm_tcgen05_tile_coords": [_I, _I, _I, _I, _P, _P],
        "dl_gemm_tcgen05_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P, _P]},
    "gemm_tcgen05_cluster": {
        "dl_gemm_tcgen05_cluster": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _P, _P],
        "dl_gemm_tcgen05_cluster_qkv_rope": [_P, _I, _P, _P, _I, _I, _I, _P, _P, _P, _I, _P, _P, _P, _P, _F, _I, _I, _I, _I, _P, _P]},
    "gemm_stream_tcgen05": {
        "dl_gemm_stream": [_P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _L, _P, _P]},
    "gemm_simt": {"dl_gemm_simt": [_I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _F, _P]},
    "sampling": {
        "dl_argmax": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
        "dl_sample_temperature": [_P, _I, _I, _I, _P, _P, _P, _P, _P],
        "dl_apply_penalties": [_P, _I, _I, _P, _P, _I, _P, _P, _I, _P, _P, _P],
        "dl_sample_filtered": [_P, _I, _I, _P, _I, _P, _P, _P, _P],
        "dl_argmax_of_parts": [_P, _P, _I, _I, _P, _P, _P, _P],
        "dl_feedback_tokens": [_P, _P, _P, _I, _P],
    },
    "streams": {"dl_stream_fork": [_P, _P], "dl_stream_join": [_P, _P]},
    "table_update": {"dl_table_updates": [_P, _P, _I, _I, _I, _I, _P],
                     "dl_zero_pages": [_P, _L, _I, _I, _P, _I, _I, _P]},
}

_funcs = {}


_recording: Optional[list] = None

# The checked build of the kernels (DYNALM_CHECK=1, csrc/check.cuh): every index a kernel takes from device memory
# is compared with its range before use; after every launch the host reads the library's record of the first
# violation and raises EngineError. Steps then run launch by launch (no CUDA graphs), each launch followed by a
# wait for its stream: a build for finding faults, not for speed.
CHECKED = bool(_lib.extra_flags())

CHECK_CODES = {
    1: "a token id outside the vocabulary",
    2: "a gathered row outside the rows of the step",
    3: "a request index outside the block table",
    4: "a position whose block lies outside the request's row of the block table",
    5: "a page id outside the pool",
    6: "a place outside the array of chosen ids",
    7: "a query tile whose rows lie outside the step",
    8: "a part of a query tile outside its parts, or its records outside the scratch",
}


def decode_check_record(record) -> str:
    """The sentence for a record of csrc/check.cuh: (code, value, lowest allowed, one past the highest allowed,
    blockIdx.x, blockIdx.y, blockIdx.z, threadIdx.x); '' when the code is 0."""
    code, value, lo, hi, bx, by, bz, tx = (int(v) for v in record)
    if code == 0:
        return ""
    what = CHECK_CODES.get(code, f"check code {code}")
    return f"{what}: {value} is not in [{lo}, {hi}) (block {bx},{by},{bz}, thread {tx})"


def _checked(library: str, name: str, f):
    take = getattr(_lib.load(library), "dl_check_take")
    take.argtypes = [c_void_p, c_void_p]
    take.restype = c_int
    record = (c_longlong * 8)()

    def call(*args):
        code = f(*args)
        if code != 0:
            return code
        rc = take(record, _stream())
        if rc != 0:
            raise EngineError(f"{name}: CUDA error {rc} after the launch")
        if record[0] != 0:
            raise EngineError(f"{name} (checked build): {decode_check_record(record)}; the access was not made")
        return 0
    return call


def check_limits(library: str, pages: int = 0, requests: int = 0, rows: int = 0, vocab: int = 0) -> None:
    """In a checked build: the ranges that the kernels of `library` compare their indices with from now on (in
    stream order); 0 = not known, not checked. Nothing otherwise."""
    if not CHECKED:
        return
    f = _funcs.get(("limits", library))
    if f is None:
        f = getattr(_lib.load(library), "dl_check_limits")
        f.argtypes = [_I, _I, _I, _I, _P]
        f.restype = c_int
        _funcs[("limits", library)] = f
    code = f(int(pages), int(requests), int(rows), int(vocab), _stream())
    if code != 0:
        raise EngineError(f"dl_check_limits of {library}: CUDA error {code}")


def _fn(library: str, name: str):
    f = _funcs.get(name)
    if f is None:
        f = getattr(_lib.load(library), name)
        f.argtypes = _SIGNATURES[library][name]
        f.restype = c_int
        if CHECKED and library != "streams":
            f = _checked(library, name, f)
        _funcs[name] = f
    if _timing is not None:
        return _timing.timed(name, f)
    if _recording is None:
        return f
    calls = _recording

    def recorded(*args):
        calls.append((f, args))
        return f(*args)
    return recorded


@contextlib.contextmanager
def on_stream(handle: int):
    """Inside the block every launch of this module goes to the stream with this handle."""
    global _pinned_stream
    previous = _pinned_stream
    _pinned_stream = int(handle)
    try:
        yield
    finally:
        _pinned_stream = previous


def counts_as_kernel(f) -> bool:
    """Whether a recorded function launches a kernel of this package (a library product and the ordering of two
    streams do not)."""
    return f is not library_mm_again and f is not _funcs.get("dl_stream_fork") and f is not _funcs.get("dl_stream_join")


def stream_fork(side: int) -> None:
    """What the stream `side` is given from now on runs after everything the current stream has been given so far
    (csrc/streams.cu)."""
    code = _fn("streams", "dl_stream_fork")(_stream(), int(side))
    if code != 0:
        raise EngineError(f"stream_fork: CUDA error {code}")


def stream_join(side: int) -> None:
    """What the current stream is given from now on runs after everything `side` has been given so far."""
    code = _fn("streams", "dl_stream_join")(_stream(), int(side))
    if code != 0:
        raise EngineError(f"stream_join: CUDA error {code}")


def library_mm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out = x w^T by the library (cuBLAS through torch), written down like a launch of this module's when a
    recording is on."""
    if _timing is not None:
        _timing.timed("library product (torch.mm)", library_mm_again)(x, w, out)
        return
    torch.mm(x, w.t(), out=out)
    if _recording is not None:
        _recording.append((library_mm_again, (x, w, out)))


def note_unrecorded_work() -> None:
    """For device work that is not written down while a recording is on: marks the recording as incomplete, so
    that nobody repeats it."""
    if _recording is not None:
        _recording.append((None, ()))


def library_mm_again(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> int:
    torch.mm(x, w.t(), out=out)
    return 0


_timing: Optional["KernelTimes"] = None

# What the next weight-streaming kernel but one will read (see `stream_ahead`): (address, bytes) or None.
_ahead: Optional[tuple] = None
AHEAD = os.environ.get("DYNALM_AHEAD", "1") != "0"
# At most this many bytes of a hint are requested. Measured on B200 (1B shapes, decode step at batch 8 / batch 1):
# without 0.945 / 0.778 ms; 4 MB 0.934 / 0.776; 12 MB 0.912 / 0.756; 16 MB 0.920; 24 MB 0.921 / 0.759; 34 MB 0.929 / 0.780;
# everything (the 67 MB of gate | up included) 0.984 / 0.810: what is requested too early is pushed out of L2 again by
# the kernels in between and is read twice.
AHEAD_MAX = int(os.environ.get("DYNALM_AHEAD_MAX", str(12 << 20)))


def stream_ahead(weights: Optional[torch.Tensor]) -> None:
    """Says that `weights` will be streamed from memory by a kernel soon. The next kernel launched through this
    module that can do so (the norm, the decode attention, the weight-streaming products for few rows) asks for them
    to be brought into L2 before it waits for the kernel in front of it: while that kernel is still running, the
    weights of the kernel after the next already cross the memory bus, which otherwise idles at every seam between
    two short kernels of a decode step. One hint is taken by one launch; a hint nobody takes is dropped by the next
    launch that cannot. DYNALM_AHEAD=0 turns it off."""
    global _ahead
    _ahead = None if (weights is None or not AHEAD) else (weights.data_ptr(), min(AHEAD_MAX, weights.numel() * weights.element_size()))


def _take_ahead():
    global _ahead
    got, _ahead = _ahead, None
    return got if got is not None else (None, 0)


class KernelTimes:
    """Inside the block every kernel launch of this module stands between two CUDA events on its stream;
    `totals()` then gives {C entry point: (launches, milliseconds)}. A kernel launched to start beside the end of
    the one in front of it (programmatic dependent launch, on by default for the products and the attention) lets the
    event behind it pass early: run with DYNALM_PDL=0 for times that are each kernel's own. The counterpart of the reference's per-op marks
    in its forward pass (`ForwardProfile`, dynalm/src/model/transformer.h:34-49): off unless asked for, and meant
    for steps that run launch by launch (engine/profile.py sees to that)."""

    def __enter__(self):
        global _timing
        self.marks: list = []
        self._outer = _timing
        _timing = self
        return self

    def __exit__(self, *exc):
        global _timing
        _timing = self._outer
        return False

    def timed(self, name: str, f):
        def call(*args):
            # the stream the launch goes to, as a torch stream: torch's own current stream where that is it (an external
            # handle of the default stream is not the same stream to torch, and events recorded there wait for nothing)
            current = torch.cuda.current_stream()
            stream = current if current.cuda_stream == _stream() else torch.cuda.ExternalStream(_stream())
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record(stream)
            code = f(*args)
            end.record(stream)
            self.marks.append((name, begin, end))
            return code
        return call

    def totals(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, begin, end in self.marks:
            n, ms = out.get(name, (0, 0.0))
            out[name] = (n + 1, ms + begin.elapsed_time(end))
        return out


class Recording:
    """Inside the block every kernel launch of this module is also written down as (function, arguments), in
    order: `calls`; a function returns 0 when its launch went well. Issuing the list again repeats the launches
    (engine/launch_memo.py does, for the next layer)."""

    def __enter__(self):
        global _recording
        self._outer = _recording
        self.calls: list = []
        _recording = self.calls
        return self

    def __exit__(self, *exc):
        global _recording
        _recording = self._outer
        return False


_pinned_stream: Optional[int] = None


def _stream() -> int:
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


@contextlib.contextmanager
def pinned_stream():
    """Inside the block every launch goes to the stream that is current on entry: one lookup for a whole forward
    pass instead of one per launch (the lookup costs more than the launch)."""
    global _pinned_stream
    previous = _pinned_stream
    _pinned_stream = torch.cuda.current_stream().cuda_stream
    try:
        yield
    finally:
        _pinned_stream = previous


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


LAUNCHES = 0     # kernels of this package launched so far (bench.py reports the count of its timed region)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code == 0:
        LAUNCHES += 1
        return
    if code == DL_ERR_UNSUPPORTED:
        raise Unsupported(f"{what}: the kernel refuses these sizes")
    raise EngineError(f"{what}: CUDA error {code}")


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise Unsupported(f"dtype {dtype} has no kernels (float32 and bfloat16 do)")


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise InvalidArgument("kernels take CUDA tensors only; there is no CPU path")


def _rows_contiguous(t: torch.Tensor, what: str) -> None:
    if t.dim() != 2 or t.stride(1) != 1:
        raise InvalidArgument(f"{what} must be 2-D with unit stride along its rows")


# ---------------------------------------------------------------------------------------------

def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> None:
    """out[i, :] = table[ids[i], :] * scale; out is the float32 residual stream [rows, width]."""
    _cuda(table, ids, out)
    rows, width = out.shape
    if out.dtype != torch.float32 or not out.is_contiguous() or ids.dtype != torch.int32 or not table.is_contiguous():
        raise InvalidArgument("embed: out float32 contiguous, ids int32, table contiguous")
    if table.shape[1] != width or ids.numel() < rows:
        raise InvalidArgument("embed: shapes disagree")
    _check(_fn("embedding", "dl_embed")(dtype_code(table.dtype), _p(table), _p(ids), _p(out), rows, width,
                                         table.shape[0], scale, _stream()), "embed")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, delta: Optional[torch.Tensor] = None,
            delta_scale: float = 1.0, rows: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """out[r] = rmsnorm(x[src] + delta_scale * delta[src]) * weight, src = rows[r] or r.

    x: float32 [n, width] residual stream, updated in place with the sum when `delta` is given and
    `write_residual`; delta: [n, width] of either dtype, or [parts, n, width] partial sums that are
    added in order; weight: float32 [width]; out: [n_out, width]."""
    _cuda(x, weight, out, delta, rows)
    width = x.shape[1]
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or not x.is_contiguous() or not out.is_contiguous():
        raise InvalidArgument("rmsnorm: x and weight float32, x and out contiguous")
    if out.shape[1] != width or weight.numel() != width:
        raise InvalidArgument("rmsnorm: widths disagree")
    n_rows = out.shape[0]
    if rows is not None:
        if rows.dtype != torch.int32 or rows.numel() < n_rows:
            raise InvalidArgument("rmsnorm: rows must be int32 with one entry per output row")
        write_residual = False
    elif x.shape[0] < n_rows:
        raise InvalidArgument("rmsnorm: fewer input rows than output rows")
    parts, part_stride = _delta_parts(delta, width, "rmsnorm")
    dd = dtype_code(delta.dtype) if delta is not None else dtype_code(out.dtype)
    check_limits("norm", rows=x.shape[0])
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("norm", "dl_rmsnorm")(dtype_code(out.dtype), dd, _p(x), _p(delta), delta_scale, _p(weight), eps,
                                      _p(out), _p(rows), n_rows, width, 1 if write_residual else 0, parts, part_stride,
                                      ahead, ahead_bytes, _stream()), "rmsnorm")


def _delta_parts(delta: Optional[torch.Tensor], width: int, what: str):
    """(number of partial sums, elements between them) of a delta that is [n, width] or [parts, n, width]."""
    if delta is None:
        return 1, 0
    if not delta.is_contiguous() or delta.shape[-1] != width or delta.dim() not in (2, 3):
        raise InvalidArgument(f"{what}: delta must be contiguous [n, width] or [parts, n, width]")
    if delta.dim() == 3:
        return delta.shape[0], delta.stride(0)
    return 1, 0


def residual_add(x: torch.Tensor, delta: torch.Tensor, scale: float = 1.0) -> None:
    """x += scale * delta over delta's rows (x float32); delta may be [parts, n, width] partial sums."""
    _cuda(x, delta)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise InvalidArgument("residual_add: x float32 and contiguous")
    parts, part_stride = _delta_parts(delta, x.shape[1], "residual_add")
    _check(_fn("norm", "dl_residual_add")(dtype_code(delta.dtype), _p(x), _p(delta), scale, delta.numel() // parts,
                                           parts, part_stride, _stream()), "residual_add")


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, inner + j]."""
    _cuda(gate_up, out)
    rows, inner = out.shape
    if gate_up.shape != (rows, 2 * inner) or not gate_up.is_contiguous() or not out.is_contiguous() \
            or gate_up.dtype != out.dtype:
        raise InvalidArgument("silu_mul: gate_up [rows, 2*inner] and out [rows, inner], contiguous, one dtype")
    _check(_fn("activation", "dl_silu_mul")(dtype_code(out.dtype), _p(gate_up), _p(out), rows, inner, _stream()),
           "silu_mul")


def rope_cache_write(qkv: torch.Tensor, positions: torch.Tensor, row_request: torch.Tensor,
                     block_table: Optional[torch.Tensor], k_cache: Optional[torch.Tensor],
                     v_cache: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rotary_dim: int,
                     pos_scale: float, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                     write_cache: bool = True) -> None:
    """Rotate the q heads of `qkv` in place; rotate the k heads and copy the v heads into the paged
    cache at each row's position. qkv: [rows, >= (n_heads + 2 n_kv_heads) head_dim]."""
    _cuda(qkv, positions, row_request, block_table, k_cache, v_cache, inv_freq)
    _rows_contiguous(qkv, "qkv")
    rows = qkv.shape[0]
    need = (n_heads + (2 * n_kv_heads if write_cache else 0)) * head_dim
    if qkv.shape[1] < need:
        raise InvalidArgument("rope_cache_write: qkv is narrower than its heads")
    if write_cache:
        if k_cache is None or v_cache is None or block_table is None:
            raise InvalidArgument("rope_cache_write: a cache write needs k_cache, v_cache and a block table")
        if k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype or not k_cache.is_contiguous() or not v_cache.is_contiguous():
            raise InvalidArgument("rope_cache_write: cache arrays must be contiguous and of qkv's dtype")
        if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim):
            raise InvalidArgument("rope_cache_write: cache shape is not [pages, page_size, kv_heads, head_dim]")
        if block_table.dtype != torch.int32 or block_table.stride(-1) != 1:
            raise InvalidArgument("rope_cache_write: block_table must be int32 rows")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != rotary_dim):
        raise InvalidArgument("rope_cache_write: inv_freq must be float32 [rotary_dim / 2]")
    if rotary_dim > head_dim or rotary_dim % 2:
        raise Unsupported(f"rotary_dim {rotary_dim} does not fit head_dim {head_dim}")
    max_blocks = block_table.stride(0) if block_table is not None else 0
    if write_cache:
        check_limits("rope_cache", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    _check(_fn("rope_cache", "dl_rope_cache_write")(
        dtype_code(qkv.dtype), _p(qkv), qkv.stride(0), _p(positions), _p(row_request), _p(block_table), max_blocks,
        _p(k_cache), _p(v_cache), _p(inv_freq), rotary_dim if inv_freq is not None else 0, pos_scale, rows, n_heads,
        n_kv_heads, head_dim, page_size, 1 if write_cache else 0, _stream()), "rope_cache_write")


def paged_attention_generic(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor, n_heads: int,
                            n_kv_heads: int, head_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """Causal attention of every row over its request's cached keys; see csrc/attention_generic.cu.
    q, out: [rows, >= n_heads * head_dim] views with unit column stride."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if head_dim % 16 or head_dim > 256:
        raise Unsupported(f"attention: head_dim {head_dim} must be a multiple of 16, at most 256")
    if n_heads % n_kv_heads:
        raise Unsupported(f"attention: {n_heads} heads do not divide into {n_kv_heads} KV heads")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    check_limits("attention_generic", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_generic", "dl_paged_attention_generic")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0),
        _p(positions), _p(row_request), _p(out), out.stride(0), q.shape[0], n_heads, n_kv_heads, head_dim, page_size,
        scale, window, _stream()), "paged_attention_generic")


def decode_scratch_floats(rows: int, n_heads: int, head_dim: int, n_split: int) -> int:
    """Floats of scratch `paged_attention_decode` needs."""
    return 0 if n_split <= 1 else rows * n_heads * n_split * (head_dim + 2)


def paged_attention_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                           positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor,
                           scratch: Optional[torch.Tensor], n_heads: int, n_kv_heads: int, head_dim: int,
                           page_size: int, scale: float, window: int, n_split: int, tensor_cores: bool = False) -> None:
    """Split-KV attention for rows that bring few tokens; see csrc/attention_decode.cu. `scratch`:
    float32 with at least decode_scratch_floats(...) elements when n_split > 1. `tensor_cores`
    picks the mma variant (bfloat16, head_dim up to 128)."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out, scratch)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    rows = q.shape[0]
    if page_size & (page_size - 1):
        raise Unsupported(f"decode attention: page size {page_size} is not a power of two")
    if head_dim % 16 or head_dim > 256 or n_heads % n_kv_heads:
        raise Unsupported(f"decode attention: head_dim {head_dim} / heads {n_heads}:{n_kv_heads} not supported")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("decode attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("decode attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    need = decode_scratch_floats(rows, n_heads, head_dim, n_split)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise InvalidArgument(f"decode attention: scratch must be float32 with at least {need} elements")
    check_limits("attention_decode", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    if tensor_cores:
        if q.dtype != torch.bfloat16 or head_dim > 128 or q.stride(0) % 8 or q.data_ptr() % 16:
            raise Unsupported("decode attention (tensor cores): bfloat16, head_dim up to 128, 16-byte aligned q rows")
        ahead, ahead_bytes = _take_ahead()
        _check(_fn("attention_decode", "dl_paged_attention_decode_tc")(
            _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(positions),
            _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim, page_size, scale,
            window, n_split, ahead, ahead_bytes, _stream()), "paged_attention_decode_tc")
        return
    _check(_fn("attention_decode", "dl_paged_attention_decode")(
        dtype_code(q.dtype), _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0),
        _p(positions), _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim,
        page_size, scale, window, n_split, _stream()), "paged_attention_decode")


def decode_tile_keys(head_dim: int) -> int:
    """Keys per tile of the tensor-core decode attention (what its plans count keys in); the table of
    csrc/attention_decode.cu (dl_paged_attention_decode_tile), kept here so that a plan can be made without the
    library."""
    return 16 if head_dim >= 96 or head_dim == 64 else 32


def paged_attention_decode_planned(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                                   positions: torch.Tensor, row_request: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
                                   counters: torch.Tensor, plan: torch.Tensor, unit_cap: int, part_stride: int, n_heads: int,
                                   n_kv_heads: int, head_dim: int, page_size: int, scale: float, window: int) -> None:
    """The tensor-core split-KV attention with the keys of all rows dealt into units by the host (`plan`, see
    kernels/attention.DecodeUnits): one block per unit, `unit_cap` blocks launched; the last block of a row's group of
    heads to finish merges the row's parts. bfloat16, head_dim up to 128. scratch: float32, rows * n_heads * part_stride *
    (head_dim + 2) elements; counters: int32, rows * KV-head chunks, zero (the kernel leaves them zero)."""
    _cuda(q, k_cache, v_cache, block_table, positions, row_request, out, scratch, counters, plan)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    rows = q.shape[0]
    chunks = n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    if q.dtype != torch.bfloat16 or head_dim % 16 or head_dim > 128 or n_heads % n_kv_heads or page_size & (page_size - 1) \
            or q.stride(0) % 8 or q.data_ptr() % 16:
        raise Unsupported("decode attention (planned): bfloat16, head_dim up to 128, 16-byte aligned q rows")
    if q.dtype != out.dtype or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise InvalidArgument("decode attention: q, out and the cache must share one dtype")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("decode attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if scratch.dtype != torch.float32 or scratch.numel() < rows * n_heads * part_stride * (head_dim + 2) \
            or counters.dtype != torch.int32 or counters.numel() < rows * chunks or plan.dtype != torch.int32 \
            or plan.numel() < 4 + 4 * unit_cap or plan.data_ptr() % 16:
        raise InvalidArgument("decode attention (planned): scratch, counters or plan too small or of the wrong type")
    check_limits("attention_decode", pages=k_cache.shape[0], requests=block_table.shape[0], rows=rows)
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("attention_decode", "dl_paged_attention_decode_planned")(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(positions),
        _p(row_request), _p(out), out.stride(0), _p(scratch), rows, n_heads, n_kv_heads, head_dim, page_size, scale,
        window, _p(plan), _p(counters), unit_cap, part_stride, ahead, ahead_bytes, _stream()),
        "paged_attention_decode_planned")


QKV_ROPE_TCGEN05_HEAD_DIMS = (64, 128)
# From how many rounds of 256-wide tiles over the SMs the tcgen05 product with the rotating epilogue is ahead of the
# product followed by the rotation kernel. The rotating epilogue of a tile takes about 10 us more than the plain one
# and only hides behind the next tile of the same block. Measured in CUDA graphs (us: fused / own product + rotation /
# library product + rotation), head size 128, width 3072 with 24+8+8 heads: 544 rows 27.7 / 21.1 / 20.4, 1,024 rows
# 43.8 / 35.5 / 29.8, 2,048 rows (2.2 rounds) 63.1 / 58.1 / 55.0, 4,096 rows 103 / 112 / 102; width 4096 with 32+8+8
# heads: 1,024 rows 58.4 / 51.2 / 44.0, 2,048 rows (2.6 rounds) 90.1 / 94.7 / 85.4, 4,096 rows 169 / 191 / 188. At
# head size 64 (width 2048, 32+8+8 heads) the two are level from 544 rows on (15.6 / 15.4, 27.5 / 28.8 at 2,048 rows),
# and one launch less is worth more to a step that waits for the host.
QKV_ROPE_TCGEN05_MIN_ROUNDS = {64: 0.0, 128: 2.4}


def rope_angles(positions: torch.Tensor, inv_freq: torch.Tensor, pos_scale: float, rows: int, out: torch.Tensor) -> None:
    """out[r, i] = (cos, sin)(float(positions[r]) * pos_scale * inv_freq[i]): float32 [rows, len(inv_freq), 2]."""
    _cuda(positions, inv_freq, out)
    half = inv_freq.numel()
    if positions.dtype != torch.int32 or inv_freq.dtype != torch.float32 or out.dtype != torch.float32 \
            or out.numel() < rows * half * 2 or not out.is_contiguous() or out.data_ptr() % 16:
        raise InvalidArgument("rope_angles: int32 positions, float32 inv_freq, contiguous float32 out [rows, half, 2]")
    _check(_fn("rope_cache", "dl_rope_angles")(_p(positions), _p(inv_freq), half, pos_scale, rows, _p(out), _stream()),
           "rope_angles")


def gemm_qkv_rope(x: torch.Tensor, w_qkv: torch.Tensor, q_out: torch.Tensor, positions: torch.Tensor,
                  row_request: torch.Tensor, block_table: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  inv_freq: torch.Tensor, pos_scale: float, n_heads: int, n_kv_heads: int, head_dim: int,
                  page_size: int, angles: Optional[torch.Tensor] = None) -> None:
    """The q | k | v projection with rotary encoding and cache write in its epilogue: rotated q into
    q_out [rows, >= n_heads * head_dim], rotated k and plain v into the paged cache. The whole head is rotated
    (inv_freq has head_dim / 2 entries). bfloat16. Up to 16 rows: the weight-streaming kernel
    (csrc/gemm_skinny.cu, head_dim a multiple of 16); more rows: the tcgen05 kernel (csrc/gemm_tcgen05.cu,
    head_dim 64 or 128), which reads the step's (cos, sin) pairs from `angles` (see rope_angles) when given."""
    _cuda(x, w_qkv, q_out, positions, row_request, block_table, k_cache, v_cache, inv_freq)
    _rows_contiguous(x, "x")
    _rows_contiguous(q_out, "q_out")
    M, K = x.shape
    if any(t.dtype != torch.bfloat16 for t in (x, w_qkv, q_out, k_cache, v_cache)):
        raise Unsupported("gemm_qkv_rope: bfloat16 only")
    few = M <= SKINNY_FAST_ROWS
    if K % 8 or x.stride(0) % 8 or (head_dim % 16 if few else head_dim not in QKV_ROPE_TCGEN05_HEAD_DIMS):
        raise Unsupported(f"gemm_qkv_rope: {M} rows, K {K} and head_dim {head_dim}")
    if angles is not None and (angles.dtype != torch.float32 or angles.numel() < M * head_dim or not angles.is_contiguous()):
        raise InvalidArgument("gemm_qkv_rope: angles must be contiguous float32 [rows, head_dim / 2, 2]")
    if not few and (x.data_ptr() % 16 or w_qkv.data_ptr() % 16 or q_out.data_ptr() % 16 or q_out.stride(0) % 8):
        raise Unsupported("gemm_qkv_rope: x, w and q_out rows must be 16-byte aligned")
    if tuple(w_qkv.shape) != ((n_heads + 2 * n_kv_heads) * head_dim, K) or not w_qkv.is_contiguous():
        raise InvalidArgument("gemm_qkv_rope: w must be contiguous [(heads + 2 kv_heads) * head_dim, K]")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() * 2 != head_dim:
        raise Unsupported("gemm_qkv_rope: the rotary width must be the whole head (inv_freq float32 [head_dim / 2])")
    if q_out.shape[0] < M or q_out.shape[1] < n_heads * head_dim:
        raise InvalidArgument("gemm_qkv_rope: q_out is smaller than [rows, heads * head_dim]")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or k_cache.shape != v_cache.shape \
            or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("gemm_qkv_rope: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if block_table.dtype != torch.int32 or block_table.stride(-1) != 1 or positions.dtype != torch.int32 \
            or row_request.dtype != torch.int32:
        raise InvalidArgument("gemm_qkv_rope: positions, row_request and block_table must be int32")
    if not few:
        library, name = (("gemm_tcgen05_cluster", "dl_gemm_tcgen05_cluster_qkv_rope") if tcgen05_pairs(M, w_qkv.shape[0])
                         else ("gemm_tcgen05", "dl_gemm_tcgen05_qkv_rope"))
        check_limits(library, pages=k_cache.shape[0], requests=block_table.shape[0], rows=M)
        _check(_fn(library, name)(
            _p(x), x.stride(0), _p(w_qkv), _p(q_out), q_out.stride(0), M, K, _p(positions), _p(row_request),
            _p(block_table), block_table.stride(0), _p(k_cache), _p(v_cache), _p(inv_freq), _p(angles), pos_scale, n_heads,
            n_kv_heads, head_dim, page_size, _p(_status_word(x.device)), _stream()), "gemm_tcgen05_qkv_rope")
        return
    check_limits("gemm_skinny", pages=k_cache.shape[0], requests=block_table.shape[0], rows=M)
    _check(_fn("gemm_skinny", "dl_gemm_skinny_qkv_rope")(
        _p(x), x.stride(0), _p(w_qkv), _p(q_out), q_out.stride(0), M, K, _p(positions), _p(row_request), _p(block_table),
        block_table.stride(0), _p(k_cache), _p(v_cache), _p(inv_freq), pos_scale, n_heads, n_kv_heads, head_dim, page_size,
        _stream()), "gemm_skinny_qkv_rope")


_tcgen05_status = {}
_pairs: Optional[bool] = None      # whether the variant with pairs of blocks sharing W tiles can be used


# rounds of 128 x 256 tiles over the SMs from which sharing W tiles between two blocks pays (measured on B200)
PAIRS_MIN_WAVES = float(os.environ.get("DYNALM_GEMM_PAIRS_MIN_WAVES", "4"))


def tcgen05_pairs(rows: int, features: int) -> bool:
    """Large products run the tcgen05 kernel in which two thread blocks share each tile of W
    (csrc/gemm_tcgen05_cluster.cu: 108 us against 119 us for 2048 x 16384 x 2048, 423 against 454 for 8192 rows),
    unless DYNALM_GEMM_PAIRS=0 or that source file is not there; smaller ones, where the pairing only couples the
    blocks' pipelines (54 us against 52 us for 2048 x 2048 x 8192), run csrc/gemm_tcgen05.cu."""
    global _pairs
    if _pairs is None:
        _pairs = os.environ.get("DYNALM_GEMM_PAIRS", "1") != "0" and \
            os.path.isfile(os.path.join(_lib.CSRC, "gemm_tcgen05_cluster.cu"))
    from .device import sm_count
    return _pairs and -(-rows // 128) * -(-features // 256) >= PAIRS_MIN_WAVES * sm_count()


def _status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that the tcgen05 kernels write a code into when a wait inside them times out."""
    status = _tcgen05_status.get(device)
    if status is None:
        status = torch.zeros(1, dtype=torch.int32, device=device)
        _tcgen05_status[device] = status
    return status


def gemm_tcgen05_status(device=None) -> int:
    """The timeout code the tcgen05 kernels (matrix product, prompt attention) left on `device` (0: none).
    Reading it synchronises."""
    if device is None:
        return max((int(t.item()) for t in _tcgen05_status.values()), default=0)
    t = _tcgen05_status.get(torch.device(device))
    return 0 if t is None else int(t.item())


PREFILL_TCGEN05_HEAD_DIMS = (64, 128)


def paged_attention_prefill_tcgen05(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                                    q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                                    head_dim: int, page_size: int, scale: float, window: int = 0,
                                    unit_parts: Optional[torch.Tensor] = None, partial: Optional[torch.Tensor] = None,
                                    counters: Optional[torch.Tensor] = None) -> None:
    """Flash attention of query tiles over the paged cache on tcgen05 tensor cores, bfloat16, head_dim 64 or
    128, pages of at least 16 keys; see csrc/attention_prefill_tcgen05.cu. Arguments as paged_attention_prefill.

    unit_parts: int32 [n_tiles], when the keys of some tiles are dealt over several entries of q_tiles (see
    kernels/attention.QueryTileParts): part | parts << 8 | scratch slot << 16 per entry, 0 = whole. Then partial:
    float32, (slots in use) * n_heads * (head_dim + 2) * 128 elements; counters: int32, (slots in use) * n_heads, zero."""
    _cuda(q, k_cache, v_cache, block_table, q_tiles, out, unit_parts, partial, counters)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise Unsupported("prefill attention (tcgen05): bfloat16 only")
    if head_dim not in PREFILL_TCGEN05_HEAD_DIMS or page_size < 16 or page_size & (page_size - 1) or n_heads % n_kv_heads:
        raise Unsupported(f"prefill attention (tcgen05): head_dim {head_dim} (64 or 128), page size {page_size} "
                          f"(a power of two from 16), heads {n_heads}:{n_kv_heads}")
    if (q.stride(0) % 8 or out.stride(0) % 8 or q.data_ptr() % 16 or out.data_ptr() % 16 or q_tiles.data_ptr() % 16
            or k_cache.data_ptr() % 16 or v_cache.data_ptr() % 16):
        raise Unsupported("prefill attention (tcgen05): q, out and cache rows must be 16-byte aligned")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous() \
            or v_cache.shape != k_cache.shape:
        raise InvalidArgument("prefill attention (tcgen05): cache shape is not [pages, page_size, kv_heads, head_dim]")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("prefill attention (tcgen05): q_tiles must be int32 [n_tiles, 4]")
    records = 0
    if unit_parts is not None:
        if unit_parts.dtype != torch.int32 or unit_parts.numel() < n_tiles or partial is None or counters is None \
                or partial.dtype != torch.float32 or counters.dtype != torch.int32:
            raise InvalidArgument("prefill attention (tcgen05): unit_parts int32 [n_tiles] with float32 partial and int32 counters")
        records = min(partial.numel() // (n_heads * (head_dim + 2) * 128), counters.numel() // n_heads)
        _status_companions.setdefault(q.device, {})[counters.data_ptr()] = counters
    check_limits("attention_prefill_tcgen05", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_prefill_tcgen05", "dl_paged_attention_prefill_tcgen05")(
        _p(q), q.stride(0), q.shape[0], _p(k_cache), _p(v_cache), k_cache.shape[0], _p(block_table), block_table.stride(0),
        _p(q_tiles), n_tiles, _p(out), out.stride(0), n_heads, n_kv_heads, head_dim, page_size, scale, window,
        _p(_status_word(q.device)), _p(unit_parts), _p(partial), _p(counters), records, _stream()),
        "paged_attention_prefill_tcgen05")


def paged_attention_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                            q_tiles: torch.Tensor, n_tiles: int, out: torch.Tensor, n_heads: int, n_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0) -> None:
    """Flash attention of query tiles over the paged cache, bfloat16; see csrc/attention_prefill.cu.
    q_tiles: int32 [n_tiles, 4] = (request, first row, rows <= 128, first position)."""
    _cuda(q, k_cache, v_cache, block_table, q_tiles, out)
    _rows_contiguous(q, "q")
    _rows_contiguous(out, "out")
    if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise Unsupported("prefill attention: bfloat16 only")
    if head_dim % 16 or head_dim > 128 or page_size & (page_size - 1) or n_heads % n_kv_heads:
        raise Unsupported(f"prefill attention: head_dim {head_dim} (multiple of 16 up to 128), page size {page_size} "
                          f"(a power of two), heads {n_heads}:{n_kv_heads}")
    if q.stride(0) % 8 or out.stride(0) % 2 or q.data_ptr() % 16 or out.data_ptr() % 4 or q_tiles.data_ptr() % 16:
        raise Unsupported("prefill attention: q rows must be 16-byte aligned, out rows 4-byte aligned")
    if tuple(k_cache.shape[1:]) != (page_size, n_kv_heads, head_dim) or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise InvalidArgument("prefill attention: cache shape is not [pages, page_size, kv_heads, head_dim]")
    if q_tiles.dtype != torch.int32 or q_tiles.numel() < 4 * n_tiles:
        raise InvalidArgument("prefill attention: q_tiles must be int32 [n_tiles, 4]")
    check_limits("attention_prefill", pages=k_cache.shape[0], requests=block_table.shape[0], rows=q.shape[0])
    _check(_fn("attention_prefill", "dl_paged_attention_prefill")(
        _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0), _p(q_tiles), n_tiles,
        _p(out), out.stride(0), n_heads, n_kv_heads, head_dim, page_size, scale, window, _stream()),
        "paged_attention_prefill")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
              out_scale: float = 1.0) -> None:
    """out = (x @ w.T + bias) * out_scale with fp32 accumulation in a fixed order; see csrc/gemm_simt.cu."""
    _cuda(x, w, out, bias)
    _rows_contiguous(x, "x")
    _rows_contiguous(out, "out")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or out.shape != (M, N) or x.dtype != w.dtype:
        raise InvalidArgument("gemm: x [M, K], w [N, K] contiguous and of x's dtype, out [M, N]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise InvalidArgument("gemm: bias must be float32 [N]")
    _check(_fn("gemm_simt", "dl_gemm_simt")(dtype_code(x.dtype), dtype_code(out.dtype), _p(x), x.stride(0), _p(w),
                                             _p(bias), _p(out), out.stride(0), M, N, K, out_scale, _stream()), "gemm_simt")


SKINNY_MAX_ROWS = 64      # what the kernel takes
SKINNY_FAST_ROWS = int(os.environ.get("DYNALM_SKINNY_ROWS", "16"))     # up to here the dispatchers use it (measured on B200)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """Weight-streaming product for at most 64 rows, bfloat16 operands; see csrc/gemm_skinny.cu.

    mode "store": out [M, N] bfloat16 or float32, or float32 [parts, M, N] to split K over `parts`
    blocks (the consumer adds the parts); mode "swiglu": w = [gate; up], out [M, N/2] bfloat16."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_skinny: x and w bfloat16, w [N, K] contiguous")
    if M > SKINNY_MAX_ROWS or K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        raise Unsupported(f"gemm_skinny: at most {SKINNY_MAX_ROWS} rows, K a multiple of 8, 16-byte aligned rows")
    n_split, split_stride = 1, 0
    if mode == "swiglu":
        if N % 2 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise InvalidArgument("gemm_skinny: swiglu needs out [M, N/2] bfloat16")
        code, ldy = 2, out.stride(0)
    elif out.dim() == 3:
        if out.dtype != torch.float32 or out.shape[1:] != (M, N) or not out.is_contiguous():
            raise InvalidArgument("gemm_skinny: split output must be contiguous float32 [parts, M, N]")
        code, ldy, n_split, split_stride = 1, N, out.shape[0], out.stride(0)
    else:
        if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise InvalidArgument("gemm_skinny: out [M, N] bfloat16 or float32")
        code, ldy = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("gemm_skinny", "dl_gemm_skinny")(_p(x), x.stride(0), _p(w), _p(out), ldy, M, N, K, code, out_scale,
                                                 n_split, split_stride, ahead, ahead_bytes, _stream()), "gemm_skinny")


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """x W^T on tcgen05 tensor cores with TMA-fed operands; see csrc/gemm_tcgen05.cu.

    x [M, K] and w [N, K] bfloat16; out [M, N] bfloat16 or float32, or with mode "swiglu"
    (w = [gate; up]) out [M, N/2] bfloat16."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_tcgen05: x and w bfloat16, w [N, K] contiguous")
    if K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16 or out.data_ptr() % 16 or out.stride(1) != 1:
        raise Unsupported("gemm_tcgen05: K and row pitches must be multiples of 8 elements, bases 16-byte aligned")
    if mode == "swiglu":
        if N % 16 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(0) % 8:
            raise Unsupported("gemm_tcgen05: swiglu needs out [M, N/2] bfloat16 with N/2 a multiple of 8")
        code = 2
    else:
        if out.shape != (M, N):
            raise InvalidArgument("gemm_tcgen05: out [M, N]")
        if out.dtype == torch.bfloat16:
            if N % 8 or out.stride(0) % 8:
                raise Unsupported("gemm_tcgen05: bfloat16 output needs N and its row pitch to be multiples of 8")
            code = 0
        elif out.dtype == torch.float32:
            if N % 4 or out.stride(0) % 4:
                raise Unsupported("gemm_tcgen05: float32 output needs N and its row pitch to be multiples of 4")
            code = 1
        else:
            raise InvalidArgument("gemm_tcgen05: out bfloat16 or float32")
    status = _status_word(x.device)
    library, name = (("gemm_tcgen05_cluster", "dl_gemm_tcgen05_cluster") if tcgen05_pairs(M, N)
                     else ("gemm_tcgen05", "dl_gemm_tcgen05"))
    _check(_fn(library, name)(_p(x), x.stride(0), _p(w), _p(out), out.stride(0), M, N, K, code, out_scale, _p(status),
                              _stream()), "gemm_tcgen05")


def gemm_tcgen05_tile_coords(tile: int, tiles_n: int, num_tiles: int, group_m: int):
    """(row block, column block) of tile number `tile` in the tcgen05 product's numbering of num_tiles output tiles in
    tiles_n columns, groups of group_m row blocks (csrc/gemm_tcgen05_impl.cuh, t5_tile_coords). Runs on the host: it
    is there so that the numbering can be tested without a GPU."""
    from ctypes import byref, c_int
    m, n = c_int(-1), c_int(-1)
    _check(_fn("gemm_tcgen05", "dl_gemm_tcgen05_tile_coords")(tile, tiles_n, num_tiles, group_m, byref(m), byref(n)),
           "gemm_tcgen05_tile_coords")
    return m.value, n.value


STREAM_MAX_ROWS = 64       # what the tcgen05 weight-streaming product takes


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str = "store", out_scale: float = 1.0) -> None:
    """x W^T for up to 64 bfloat16 rows on tcgen05, built around the stream of W (csrc/gemm_stream_tcgen05.cu).

    out [M, N] bfloat16 or float32; float32 [parts, M, N] (contiguous): K is split over `parts` blocks and each
    leaves its partial sums; mode "swiglu" (w = [gate; up]): out [M, N/2] bfloat16."""
    _cuda(x, w, out)
    _rows_contiguous(x, "x")
    M, K = x.shape
    N = w.shape[0]
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or w.shape[1] != K:
        raise InvalidArgument("gemm_stream: x and w bfloat16, w [N, K] contiguous")
    if M > STREAM_MAX_ROWS or K % 8 or x.stride(0) % 8 or x.data_ptr() % 16 or w.data_ptr() % 16:
        raise Unsupported(f"gemm_stream: at most {STREAM_MAX_ROWS} rows, K a multiple of 8, 16-byte aligned rows")
    n_split, split_stride = 1, 0
    if mode == "swiglu":
        if N % 2 or out.shape != (M, N // 2) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
            raise InvalidArgument("gemm_stream: swiglu needs out [M, N/2] bfloat16")
        code, ldy = 2, out.stride(0)
    elif out.dim() == 3:
        if out.dtype != torch.float32 or out.shape[1:] != (M, N) or not out.is_contiguous():
            raise InvalidArgument("gemm_stream: split output must be contiguous float32 [parts, M, N]")
        code, ldy, n_split, split_stride = 1, N, out.shape[0], out.stride(0)
    else:
        if out.shape != (M, N) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
            raise InvalidArgument("gemm_stream: out [M, N] bfloat16 or float32")
        code, ldy = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
    _check(_fn("gemm_stream_tcgen05", "dl_gemm_stream")(
        _p(x), x.stride(0), _p(w), _p(out), ldy, M, N, K, code, out_scale, n_split, split_stride,
        _p(_status_word(x.device)), _stream()), "gemm_stream")


_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, status_to: Optional[torch.Tensor] = None) -> None:
    """out[r] = lowest index of the largest value of logits[r, :] (float32 rows, int32 out). `status_to` (int32, one
    element): also receives the device's status word (see gemm_tcgen05_status), so that it can travel to the host
    in the copy that carries the chosen ids."""
    _cuda(logits, out)
    _rows_contiguous(logits, "logits")
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < rows:
        raise InvalidArgument("argmax: logits float32, out int32 with one entry per row")
    # partial (value, index) pairs of the two-stage kernel; grown in powers of two, kept per device
    key = logits.device
    scratch = _argmax_scratch.get(key)
    if scratch is None or scratch.numel() < rows * 64:
        scratch = torch.empty(max(64, 1 << (rows * 64 - 1).bit_length()), dtype=torch.float32, device=logits.device)
        _argmax_scratch[key] = scratch
    status = _status_word(logits.device) if status_to is not None else None
    _check(_fn("sampling", "dl_argmax")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(out), _p(scratch),
                                         _p(status), _p(status_to), _stream()), "argmax")


_status_companions: dict = {}      # device -> {address: counters that a kernel leaves nonzero only when a wait timed out}


def clear_status(device) -> None:
    """Zero the device's status word after its code has been reported, and the counters that a kernel which gave up
    may have left half counted (the prompt attention's parts)."""
    t = _tcgen05_status.get(torch.device(device))
    if t is not None:
        t.zero_()
    for counters in _status_companions.get(torch.device(device), {}).values():
        counters.zero_()


def zero_pages(storage: torch.Tensor, fresh: torch.Tensor, n: int, group: int) -> None:
    """Clear the pages listed for `group` in the first n pairs (group id, page) of `fresh` (int32) in every array of a
    cache group's storage [entries, tensors, pages, page_size, ...] (csrc/table_update.cu)."""
    _cuda(storage, fresh)
    if not storage.is_contiguous() or storage.dim() < 4 or fresh.dtype != torch.int32 or fresh.numel() < 2 * n:
        raise InvalidArgument("zero_pages: contiguous storage [entries, tensors, pages, ...] and int32 pairs")
    pages = storage.shape[2]
    page_bytes = storage[0, 0, 0].numel() * storage.element_size()
    _check(_fn("table_update", "dl_zero_pages")(_p(storage), page_bytes, pages, storage.shape[0] * storage.shape[1], _p(fresh),
                                                 n, group, _stream()), "zero_pages")


def table_updates(tables: torch.Tensor, updates: torch.Tensor, n: int) -> None:
    """tables[g, s, b] = p for the first n quadruples (g, s, b, p) of `updates` (csrc/table_update.cu): the
    device's block tables [groups, slots, max_blocks], int32, brought up to date with what a step changed."""
    _cuda(tables, updates)
    if tables.dtype != torch.int32 or updates.dtype != torch.int32 or tables.dim() != 3 or not tables.is_contiguous() \
            or updates.numel() < 4 * n or updates.data_ptr() % 16:
        raise InvalidArgument("table_updates: int32 tables [groups, slots, blocks] and int32 updates [n, 4], 16-byte aligned")
    check_limits("table_update", requests=tables.shape[1])
    _check(_fn("table_update", "dl_table_updates")(_p(tables), _p(updates), n, tables.shape[0], tables.shape[1],
                                                    tables.shape[2], _stream()), "table_updates")


def gemm_argmax_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether `gemm_argmax` takes this product: the weight-streaming kernel's shapes, up to 8 rows."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 8 and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0)


def gemm_argmax(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, out_scale: float = 1.0,
                status_to: Optional[torch.Tensor] = None) -> None:
    """out[r] = the index of the largest element of (x W^T)[r] * out_scale, the lowest among equals, without the
    product ever being written: the weight-streaming kernel leaves one candidate per block (csrc/gemm_skinny.cu,
    mode 3) and a small kernel picks among them. `scratch`: float32, at least 2 * rows * ceil(N / 16) elements.
    out_scale must be positive. `status_to` as in `argmax`."""
    _cuda(x, w, out, scratch)
    if not gemm_argmax_applies(x, w) or w.shape[1] != x.shape[1] or out_scale <= 0:
        raise Unsupported("gemm_argmax: up to 8 bfloat16 rows, K a multiple of 8, 16-byte aligned rows, a positive scale")
    M, K = x.shape
    N = w.shape[0]
    blocks = -(-N // 16)
    if scratch.dtype != torch.float32 or scratch.numel() < 2 * M * blocks or out.dtype != torch.int32 or out.numel() < M:
        raise InvalidArgument("gemm_argmax: float32 scratch of 2 * rows * ceil(N / 16) elements, int32 out of one per row")
    ahead, ahead_bytes = _take_ahead()
    _check(_fn("gemm_skinny", "dl_gemm_skinny")(_p(x), x.stride(0), _p(w), _p(scratch), blocks, M, N, K, 3, out_scale,
                                                 1, 0, ahead, ahead_bytes, _stream()), "gemm_skinny (argmax)")
    status = _status_word(x.device) if status_to is not None else None
    _check(_fn("sampling", "dl_argmax_of_parts")(_p(scratch), scratch.data_ptr() + 4 * M * blocks, M, blocks, _p(out),
                                                  _p(status), _p(status_to), _stream()), "argmax_of_parts")


def feedback_tokens(token_ids: torch.Tensor, chosen: torch.Tensor, src: torch.Tensor, n: int) -> None:
    """token_ids[r] = chosen[src[r]] for r < n where src[r] >= 0 (all int32, on the device)."""
    _cuda(token_ids, chosen, src)
    if token_ids.dtype != torch.int32 or chosen.dtype != torch.int32 or src.dtype != torch.int32 or min(token_ids.numel(), src.numel()) < n:
        raise InvalidArgument("feedback_tokens: int32 tensors with at least n entries")
    check_limits("sampling", rows=chosen.numel())
    _check(_fn("sampling", "dl_feedback_tokens")(_p(token_ids), _p(chosen), _p(src), n, _stream()), "feedback_tokens")


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor,
                       cut_offset: Optional[torch.Tensor] = None) -> None:
    """Draw out[r] from softmax(logits[r] / temperature[r]) by walking the ids in order with uniform[r]. With
    cut_offset (float64 [rows]: temperature * log(min_p), -inf where off) the ids whose logit lies below the row's
    largest plus the offset have no mass (min-p)."""
    _cuda(logits, temperature, uniform, out, cut_offset)
    _rows_contiguous(logits, "logits")
    rows = logits.shape[0]
    if (logits.dtype != torch.float32 or temperature.dtype != torch.float32 or uniform.dtype != torch.float64
            or out.dtype != torch.int32 or min(temperature.numel(), uniform.numel(), out.numel()) < rows):
        raise InvalidArgument("sample_temperature: logits/temperature float32, uniform float64, out int32, one per row")
    if cut_offset is not None and (cut_offset.dtype != torch.float64 or cut_offset.numel() < rows):
        raise InvalidArgument("sample_temperature: cut_offset float64, one per row")
    _check(_fn("sampling", "dl_sample_temperature")(_p(logits), logits.stride(0), rows, logits.shape[1], _p(temperature),
                                                     _p(uniform), _p(cut_offset), _p(out), _stream()), "sample_temperature")


def apply_penalties(logits: torch.Tensor, rows: torch.Tensor, triples: torch.Tensor, n_triples: int,
                    params: torch.Tensor, first: torch.Tensor, chosen: Optional[torch.Tensor] = None,
                    pending: Optional[torch.Tensor] = None) -> None:
    """Repetition, frequency and presence penalties, in place: triple j = (selection, token id, count) changes
    logits[rows[selection], id] with params[selection] = (repetition, frequency, presence). The ids of one selection
    are distinct and its triples lie next to one another, from first[selection] to first[selection + 1]. rows int32
    [selections], triples int32 [>= n_triples, 3], params float32 [selections, 3], first int32 [selections + 1].
    chosen and pending (int32, both or neither): pending[selection] >= 0 is the place in `chosen` of one more token
    of that selection's context, which only the device knows yet; it counts as seen once more."""
    _cuda(logits, rows, triples, params, first, chosen, pending)
    _rows_contiguous(logits, "logits")
    n_sel = rows.numel()
    if (logits.dtype != torch.float32 or rows.dtype != torch.int32 or triples.dtype != torch.int32
            or params.dtype != torch.float32 or first.dtype != torch.int32 or triples.numel() < 3 * n_triples
            or not triples.is_contiguous() or not params.is_contiguous() or params.numel() < 3 * n_sel
            or first.numel() < n_sel + 1):
        raise InvalidArgument("apply_penalties: logits/params float32, rows/triples/first int32, triples [n, 3]")
    if (chosen is None) != (pending is None) or (pending is not None and (
            pending.dtype != torch.int32 or chosen.dtype != torch.int32 or pending.numel() < n_sel)):
        raise InvalidArgument("apply_penalties: chosen and pending int32, together, pending one per selection")
    if CHECKED:
        check_limits("sampling", rows=logits.shape[0])
    _check(_fn("sampling", "dl_apply_penalties")(_p(logits), logits.stride(0), logits.shape[1], _p(rows), _p(triples),
                                                  int(n_triples), _p(params), _p(first), n_sel, _p(chosen), _p(pending),
                                                  _stream()), "apply_penalties")


SAMPLE_FILTERED_HOST = -1      # what sample_filtered leaves for a row that the host has to finish


def sample_filtered(logits: torch.Tensor, rows: torch.Tensor, n_sel: int, dparams: torch.Tensor, top_k: torch.Tensor,
                    out: torch.Tensor) -> None:
    """One draw per selection through top-k, min-p and top-p in the reference's order. rows int32 [n_sel]: the
    logits row of each selection; dparams float64 [n_sel, 4] = (temperature, temperature * log(min_p) or -inf, top_p,
    uniform in [0, 1)); top_k int32 [n_sel] (0 = off); out int32 with a place for every row named: out[rows[sel]] gets the id,
    or SAMPLE_FILTERED_HOST where the row does not fit the kernel (top-k above 1,024, say)."""
    _cuda(logits, rows, dparams, top_k, out)
    _rows_contiguous(logits, "logits")
    if (logits.dtype != torch.float32 or rows.dtype != torch.int32 or dparams.dtype != torch.float64
            or top_k.dtype != torch.int32 or out.dtype != torch.int32 or not dparams.is_contiguous()
            or min(rows.numel(), top_k.numel(), out.numel()) < n_sel or dparams.numel() < 4 * n_sel):
        raise InvalidArgument("sample_filtered: logits float32, rows/top_k/out int32, dparams float64 [n, 4]")
    if CHECKED:
        check_limits("sampling", rows=min(logits.shape[0], out.numel()))      # a row is also a place in `out`
    _check(_fn("sampling", "dl_sample_filtered")(_p(logits), logits.stride(0), logits.shape[1], _p(rows), int(n_sel),
                                                  _p(dparams), _p(top_k), _p(out), _stream()), "sample_filtered")
