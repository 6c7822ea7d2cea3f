"""Python entry points of the CUDA kernels.

Each function checks its operands (device, dtype, contiguity, sizes the kernel can take),
launches on torch's current stream and raises on any error.  Nothing here computes: a
missing CUDA library or a tensor on the CPU is an error, never a fallback.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import build

_I, _F, _P, _LL = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

F32, BF16 = 0, 1
_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16}

_ERRORS = {-1: "bad argument", -2: "size not supported by this kernel",
           -3: "a wait inside the kernel ran out (device timeout)"}

# module -> {function: argtypes}
_SIGNATURES = {
    "elementwise": {
        "ni_embedding": [_P, _P, _I, _P, _I, _I, _I, _P],
        "ni_add_rmsnorm": [_P, _P, _I, _P, _F, _P, _I, _P, _I, _I, _P],
        "ni_residual_add": [_P, _P, _I, _LL, _P],
        "ni_swiglu": [_P, _P, _I, _I, _I, _P],
        "ni_swiglu_blocked": [_P, _P, _I, _I, _I, _P],
    },
    "rope_kv": {
        "ni_rope_kv_write": [_P, _I, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    },
    "attention_generic": {
        "ni_attention_generic": [_P, _I, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _P],
    },
    "gemm_f32": {
        "ni_gemm_f32": [_P, _P, _P, _I, _I, _I, _P],
    },
    "gemv_bf16": {
        "ni_gemv_bf16": [_P, _P, _P, _I, _I, _I, _I, _P, _LL, _P, _P, _P, _I, _P, _I, _F, _P],
        "ni_gemv_bf16_out_tiles": [_I, _I],
        "ni_gemv_bf16_writes_handoff": [_I, _I, _I],
        "ni_gemv_bf16_reads_handoff": [_I, _I],
        "ni_gemv_norm_bf16": [_P, _P, _F, _P, _P, _P, _I, _I, _I, _I, _P, _LL, _P],
        "ni_gemv_qkv_rope": [_P, _P, _F, _P, _P, _P, _P, _P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _LL, _P, _I, _F, _P],
    },
    "gemv_ksplit": {
        "ni_gemv_ksplit": [_P, _P, _P, _I, _I, _I, _I, _P, _LL, _P, _P, _P, _I, _P],
        "ni_gemv_ksplit_out_tiles": [_I, _I],
        "ni_gemv_ksplit_supports": [_I, _I, _I],
    },
    "attention_decode": {
        "ni_attention_decode": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P, _P, _LL, _P, _LL, _P],
        "ni_attention_decode_balanced": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P, _P, _LL, _P, _LL, _P],
        "ni_attention_decode_fresh_keys": [],
        "ni_attention_decode_set_cluster_merge": [_I],
        # the variant whose scratch lies in the library's own image (attention_decode_noalloc.h)
        "ni_attention_decode_noalloc": [_P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P],
    },
    "attention_prefill": {
        "ni_attention_prefill": [_P, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P],
    },
    "attention_prefill_tc": {
        "ni_attention_prefill_tc": [_P, _P, _P, _P, _I, _I, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P, _P],
        "ni_attention_prefill_tc_supports": [_I, _I, _I, _I],
        "ni_attention_prefill_tc_set_wait": [_LL, _I],
    },
    "gemm_swap_tc": {
        "ni_gemm_swap_tc": [_P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _P, _P],
        "ni_gemm_swap_tc_splits": [_I, _I, _I],
        "ni_gemm_swap_tc_scratch": [_I, _I, _I],
        "ni_gemm_swap_tc_set_wait": [_LL, _I],
    },
    "gemm_tc2": {
        "ni_gemm_tc2": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
        "ni_gemm_tc2_set_wait": [_LL, _I],
    },
    "gemm_tc": {
        "ni_gemm_tc": [_P, _P, _P, _I, _I, _I, _I, _P, _P],
        "ni_gemm_tc_set_wait": [_LL, _I],
    },
    "decode_fused": {
        "ni_decode_fused": [_P, _P],
        "ni_decode_fused_supports": [_I] * 9,
        "ni_decode_fused_max_rows": [],
        "ni_decode_fused_max_groups": [],
        "ni_decode_fused_blocks": [],
    },
    "sampling": {
        "ni_argmax": [_P, _P, _I, _I, _P, _P],
        "ni_repetition_penalty": [_P, _P, _P, _I, _I, _I, _P],
        "ni_sample": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _P],
        "ni_sample_set_cluster": [_I],
    },
}

_libs: Dict[str, ctypes.CDLL] = {}


class KernelError(RuntimeError):
    pass


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise KernelError("nanoinfer_b200 runs on a CUDA device (sm_100a) only; "
                          "torch.cuda.is_available() is False and there is no CPU path")


def load(module: str) -> ctypes.CDLL:
    lib = _libs.get(module)
    if lib is None:
        path = build.ensure_built([module])[module]
        lib = ctypes.CDLL(path)
        for fn, argtypes in _SIGNATURES.get(module, {}).items():
            f = getattr(lib, fn)
            f.argtypes = argtypes
            f.restype = _I
        import os
        if module == "sampling" and os.environ.get("NANOINFER_B200_SAMPLE_ONE_BLOCK"):      # for comparisons
            lib.ni_sample_set_cluster(0)
        if module == "attention_decode" and os.environ.get("NANOINFER_B200_SCRATCH_MERGE"):
            lib.ni_attention_decode_set_cluster_merge(0)
        if module == "attention_decode" and lib.ni_attention_decode_fresh_keys() != DECODE_FRESH_KEYS:
            raise KernelError("attention_decode: DEC_FRESH_KEYS of the built kernel differs from ops.DECODE_FRESH_KEYS")
        _libs[module] = lib
    return lib


def preload(modules) -> None:
    """Build (in parallel) and load the given modules ahead of their first use."""
    build.ensure_built(list(modules))
    for m in modules:
        load(m)


_sm_counts: Dict[int, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (148 on a B200); every work split asks here."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


_launches = 0


def launch_count() -> int:
    """How many kernels of this package have been launched (or captured) so far."""
    return _launches


def _check(code: int, what: str) -> None:
    global _launches
    if code == 0:
        _launches += 1
        return
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    raise KernelError(f"{what}: CUDA error {code} at launch")


def _check_plain(code: int, what: str) -> None:
    """As _check, for calls that launch nothing."""
    if code < 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")
    if code > 0:
        raise KernelError(f"{what}: CUDA error {code}")


def _stream() -> int:
    """The raw handle of torch's current stream on the current device (the C accessors: the Python
    wrapper costs more than a short kernel's launch)."""
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_stream_objects: Dict[int, "torch.cuda.Stream"] = {}


def current_stream_object() -> "torch.cuda.Stream":
    """torch's current stream as an object (for Event.record), cached by raw handle."""
    raw = _stream()
    obj = _stream_objects.get(raw)
    if obj is None:
        obj = _stream_objects[raw] = torch.cuda.current_stream()
    return obj


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    return t.data_ptr()


def _code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DTYPE_CODE:
        raise KernelError(f"{name}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return _DTYPE_CODE[t.dtype]


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, :] = float32(table[tokens[t], :]);  tokens int32 [T], out float32 [T, d]."""
    n, d = out.shape
    if tokens.numel() != n or table.shape[1] != d:
        raise KernelError("embedding: shapes do not agree")
    _check(load("elementwise").ni_embedding(_dev(tokens, "tokens", torch.int32), _dev(table, "table"),
                                            _code(table, "table"), _dev(out, "out", torch.float32),
                                            n, d, table.shape[0], _stream()), "embedding")


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """Residual add fused with RMSNorm.

    h float32 [T, d]; delta [T, d] or None; gain float32 [d]; out [R, d].
    rows None: R = T, h += delta in place, out = norm(h) * gain.
    rows int32 [R]: out[r] = norm(h[rows[r]] + delta[rows[r]]) * gain, h untouched.
    """
    d = h.shape[1]
    n_out = out.shape[0]
    if out.shape[1] != d or gain.numel() != d:
        raise KernelError("add_rmsnorm: widths do not agree")
    if rows is None and n_out != h.shape[0]:
        raise KernelError("add_rmsnorm: out must have as many rows as h")
    if rows is not None and rows.numel() != n_out:
        raise KernelError("add_rmsnorm: rows and out do not agree")
    if delta is not None and delta.shape != h.shape:
        raise KernelError("add_rmsnorm: delta must have the shape of h")
    _check(load("elementwise").ni_add_rmsnorm(
        _dev(h, "h", torch.float32), _dev(delta, "delta") if delta is not None else None,
        _code(delta, "delta") if delta is not None else F32, _dev(gain, "gain", torch.float32),
        float(eps), _dev(out, "out"), _code(out, "out"),
        _dev(rows, "rows", torch.int32) if rows is not None else None, n_out, d, _stream()),
        "add_rmsnorm")


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> None:
    if delta.shape != h.shape:
        raise KernelError("residual_add: shapes do not agree")
    _check(load("elementwise").ni_residual_add(_dev(h, "h", torch.float32), _dev(delta, "delta"),
                                               _code(delta, "delta"), h.numel(), _stream()),
           "residual_add")


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, blocked: bool = False) -> None:
    """out[t, i] = silu(gate[t, i]) * up[t, i].  Plain layout: gate_up = [gate | up] along the
    columns.  Blocked layout (I a multiple of 8): columns in blocks of 8 gate values followed by
    their 8 up values."""
    n, inter = out.shape
    if gate_up.shape != (n, 2 * inter) or gate_up.dtype != out.dtype:
        raise KernelError("swiglu: gate_up must be [T, 2I] of out's dtype")
    if blocked and inter % 8:
        raise KernelError("swiglu: the blocked layout needs I to be a multiple of 8")
    fn = load("elementwise").ni_swiglu_blocked if blocked else load("elementwise").ni_swiglu
    _check(fn(_dev(gate_up, "gate_up"), _dev(out, "out"), _code(out, "out"), n, inter, _stream()), "swiglu")


def rope_kv_write(qkv: torch.Tensor, q_out: torch.Tensor, k_pages: Optional[torch.Tensor],
                  v_pages: Optional[torch.Tensor], positions: torch.Tensor,
                  seq_of_token: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor,
                  n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                  interleaved: bool, page_size: int) -> None:
    """Rotate q and k of the fused projection qkv [T, (Hq + 2 Hkv) hd]; q -> q_out
    [T, Hq hd]; k (rotated) and v -> pages [P, Hkv, page_size, hd] unless k_pages is None."""
    n = qkv.shape[0]
    write = k_pages is not None
    if qkv.shape[1] != (n_q_heads + 2 * n_kv_heads) * head_dim or q_out.shape != (n, n_q_heads * head_dim):
        raise KernelError("rope_kv_write: widths do not agree with the head counts")
    if q_out.dtype != qkv.dtype or (write and (k_pages.dtype != qkv.dtype or v_pages.dtype != qkv.dtype)):
        raise KernelError("rope_kv_write: all operands must share one dtype")
    if write and tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim):
        raise KernelError("rope_kv_write: pages must be [P, Hkv, page_size, head_dim]")
    if inv_freq.numel() != rotary_dim // 2 and rotary_dim > 0:
        raise KernelError("rope_kv_write: inv_freq must have rotary_dim / 2 entries")
    _check(load("rope_kv").ni_rope_kv_write(
        _dev(qkv, "qkv"), _code(qkv, "qkv"), _dev(q_out, "q_out"),
        _dev(k_pages, "k_pages") if write else None, _dev(v_pages, "v_pages") if write else None,
        _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(inv_freq, "inv_freq", torch.float32), n, n_q_heads, n_kv_heads, head_dim, rotary_dim,
        1 if interleaved else 0, page_size, 1 if write else 0, _stream()), "rope_kv_write")


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      out: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                      block_table: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                      page_size: int, window: Optional[int], scale: float,
                      token_list: Optional[torch.Tensor] = None, head_slopes: Optional[torch.Tensor] = None) -> None:
    """The plain attention kernel (any dtype, any head size up to 256).  ``token_list``
    int32 [n] restricts it to those tokens of the step.  ``head_slopes`` float32 [Hq] adds
    slope[h] * (key position - query position) to the scaled scores of head h."""
    if head_slopes is not None and head_slopes.numel() != n_q_heads:
        raise KernelError("attention: one slope per query head")
    n = q.shape[0]
    if q.shape != (n, n_q_heads * head_dim) or out.shape != q.shape:
        raise KernelError("attention: q and out must be [T, Hq * head_dim]")
    if not (q.dtype == out.dtype == k_pages.dtype == v_pages.dtype):
        raise KernelError("attention: all operands must share one dtype")
    if head_dim > 256:
        raise KernelError(f"attention: head_dim {head_dim} > 256 is not supported")
    _check(load("attention_generic").ni_attention_generic(
        _dev(q, "q"), _code(q, "q"), _dev(k_pages, "k_pages"), _dev(v_pages, "v_pages"),
        _dev(out, "out"), _dev(token_list, "token_list", torch.int32) if token_list is not None else None,
        _dev(positions, "positions", torch.int32),
        _dev(seq_of_token, "seq_of_token", torch.int32), _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], n if token_list is None else token_list.numel(), n_q_heads, n_kv_heads, head_dim, page_size,
        int(window) if window else 0, float(scale),
        _dev(head_slopes, "head_slopes", torch.float32) if head_slopes is not None else None, _stream()), "attention_generic")


def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = x[M, K] . w[N, K]^T, all float32, plain FP32 arithmetic."""
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n):
        raise KernelError("gemm_f32: shapes do not agree")
    _check(load("gemm_f32").ni_gemm_f32(_dev(x, "x", torch.float32), _dev(w, "w", torch.float32),
                                        _dev(out, "out", torch.float32), m, n, k, _stream()), "gemm_f32")


GEMV_MAX_ROWS = 16      # what the skinny kernels take
# Up to this many rows the engine uses them.  With 9 to 16 rows they need two batch tiles, which
# halves the blocks per SM and the loads in flight: measured on a decode step at batch 16,
# 1.40 ms against 1.21 ms for the library product with separate element-wise kernels.
SKINNY_ROWS = 8
STORE_BF16, STORE_F32, ADD_F32, SWIGLU_BF16 = 0, 1, 2, 3


def _gemv_check(m: int, n: int, k: int, w: torch.Tensor, out: torch.Tensor, mode: int, what: str) -> None:
    if w.shape != (n, k):
        raise KernelError(f"{what}: shapes do not agree")
    if m > GEMV_MAX_ROWS or k % 8:
        raise KernelError(f"{what}: takes at most {GEMV_MAX_ROWS} rows and K a multiple of 8 "
                          f"(got M={m}, K={k})")
    if mode == SWIGLU_BF16:
        if n % 16 or out.shape != (m, n // 2) or out.dtype != torch.bfloat16:
            raise KernelError(f"{what}: the SwiGLU epilogue needs N a multiple of 16 and out bf16 [M, N/2]")
    else:
        want = torch.bfloat16 if mode == STORE_BF16 else torch.float32
        if out.shape != (m, n) or out.dtype != want:
            raise KernelError(f"{what}: out must be {want} [M, N]")


def warm_region(warm) -> tuple:
    """(address, bytes) of a hint ``(tensor, first byte, bytes)`` - a stretch of a tensor that a
    kernel asks into L2 on its way - cut to the tensor and to multiples of 16 bytes; (None, 0) for None."""
    if warm is None:
        return None, 0
    t, first, nbytes = warm
    size = t.numel() * t.element_size()
    first = min(max(int(first), 0), size) & ~15
    nbytes = min(int(nbytes), size - first) & ~15
    if nbytes <= 0 or not t.is_cuda or (t.data_ptr() + first) % 16:
        return None, 0
    return t.data_ptr() + first, nbytes


HANDOFF_ROWS = 8      # rows up to which a norm can be handed from the kernel that adds into the stream to its reader


class NormHandoff:
    """A norm prepared by the kernel that last added into the residual stream, for the kernel that
    reads it (up to HANDOFF_ROWS rows): ``x`` = bfloat16(h * gain) [M, d], ``ssq`` float32
    [8, parts] = per row and tile of columns the sum of h^2 (parts: the tiles rounded up to a multiple
    of 4, the rest zero), ``eps``.  The reader multiplies its
    finished products by 1 / sqrt(sum(ssq) / d + eps) per row: together RMSNorm(h) * gain without a
    kernel of its own.  ``norm`` is the part it stands for."""

    def __init__(self, norm, gain: torch.Tensor, eps: float, rows: int, width: int, tiles: int, device) -> None:
        self.norm, self.gain, self.eps, self.tiles = norm, gain, float(eps), int(tiles)
        self.parts = -(-self.tiles // 4) * 4
        self.x = torch.empty(rows, width, dtype=torch.bfloat16, device=device)
        self.ssq = torch.empty(8, self.parts, dtype=torch.float32, device=device)
        if self.parts != self.tiles:
            self.ssq[:, self.tiles:].zero_()        # what no tile writes must add nothing

    def producer_args(self):
        return _dev(self.gain, "gain", torch.float32), self.x.data_ptr(), self.ssq.data_ptr(), self.parts

    def reader_args(self):
        return self.ssq.data_ptr(), self.parts, self.eps


_NO_HANDOFF = (None, None, None, 0)
_NO_PRE = (None, 0, 0.0)


def gemv_out_tiles(m: int, n: int, k: int) -> int:
    """How many tiles of output columns the skinny product that adds [m, n] into the stream works in
    (the partial sums per row of a NormHandoff) - of whichever kernel linear_bf16 picks - or 0 if that
    kernel cannot prepare a norm for these sizes."""
    if m <= KSPLIT_ROWS and KSPLIT_MIN_K <= k <= KSPLIT_MAX_K and gemv_ksplit_supports(m, n, k):
        return int(load("gemv_ksplit").ni_gemv_ksplit_out_tiles(n, k))
    lib = load("gemv_bf16")
    return int(lib.ni_gemv_bf16_out_tiles(n, ADD_F32)) if lib.ni_gemv_bf16_writes_handoff(m, n, k) else 0


def gemv_reads_handoff(m: int, k: int) -> bool:
    """True if the skinny products can take a prepared norm on an input of m rows and width k."""
    return bool(load("gemv_bf16").ni_gemv_bf16_reads_handoff(m, k))


def gemv_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, warm=None,
              handoff: Optional["NormHandoff"] = None, pre: Optional["NormHandoff"] = None) -> None:
    """x[M, K] . w[N, K]^T for M <= 16, K % 8 == 0.  mode STORE_BF16 / STORE_F32: out[M, N] =;
    ADD_F32: out[M, N] +=; SWIGLU_BF16: w's rows in blocks of 8 gate + 8 up rows,
    out[M, N/2] = silu(gate) * up.  ``warm`` (tensor, first byte, bytes): weights of the kernels
    after this one, asked into L2 when this kernel's own loads have been issued.  ``handoff`` (with
    ADD_F32, up to 8 rows): also prepare the norm that follows; ``pre``: x is such a prepared input."""
    if (handoff is not None or pre is not None) and x.shape[0] > HANDOFF_ROWS:
        raise KernelError("gemv_bf16: a norm is handed over for at most 8 rows")
    if handoff is not None and (mode != ADD_F32 or handoff.x.shape != out.shape or handoff.tiles != int(load("gemv_bf16").ni_gemv_bf16_out_tiles(w.shape[0], ADD_F32))):
        raise KernelError("gemv_bf16: the handoff does not fit this product")
    m, k = x.shape
    n = w.shape[0]
    _gemv_check(m, n, k, w, out, mode, "gemv_bf16")
    _check(load("gemv_bf16").ni_gemv_bf16(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16),
                                          _dev(out, "out"), m, n, k, mode, *warm_region(warm),
                                          *(handoff.producer_args() if handoff is not None else _NO_HANDOFF),
                                          *(pre.reader_args() if pre is not None else _NO_PRE), _stream()), "gemv_bf16")


KSPLIT_ROWS = 8          # rows the cluster split-K skinny product takes
# The engine uses it for 2,048 < K <= 8,192 (2 to 4 slices).  Measured at 8 rows, against gemv_bf16:
# N 2,048 x K 8,192: 8.5 us against 10.1;  3,072 x 8,192: 11.1 against 16.7;  4,096 x 4,096: 8.5 against 10.2;
# 3,072 x 3,072: 7.0 against 8.3;  but 4,096 x 14,336 (7 slices: 37 clusters of 7 blocks leave SMs idle): 27.8 against 26.4.
KSPLIT_MIN_K, KSPLIT_MAX_K = 2049, 8192


def gemv_ksplit_supports(m: int, n: int, k: int) -> bool:
    """True if gemv_ksplit takes the product: up to 8 rows, K a multiple of 8 in 2 to 8 slices of at most 2,048."""
    return bool(load("gemv_ksplit").ni_gemv_ksplit_supports(m, n, k))


def gemv_ksplit(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, warm=None,
                handoff: Optional["NormHandoff"] = None, pre=None) -> None:
    """x[M, K] . w[N, K]^T for M <= 8 and a long K, split over the blocks of a cluster (each keeps
    its slice of the activations in registers; the slices' sums are added in slice order).
    mode STORE_BF16 / STORE_F32 / ADD_F32 as gemv_bf16."""
    m, k = x.shape
    n = w.shape[0]
    if mode not in (STORE_BF16, STORE_F32, ADD_F32):
        raise KernelError("gemv_ksplit: mode must be STORE_BF16, STORE_F32 or ADD_F32")
    _gemv_check(m, n, k, w, out, mode, "gemv_ksplit")
    if not gemv_ksplit_supports(m, n, k):
        raise KernelError(f"gemv_ksplit: M={m}, N={n}, K={k} is not supported (up to 8 rows, K in 2 to 8 slices of 2,048)")
    if pre is not None:
        raise KernelError("gemv_ksplit: takes no prepared norm on its input")
    if handoff is not None and (mode != ADD_F32 or handoff.x.shape != out.shape
                                or handoff.tiles != int(load("gemv_ksplit").ni_gemv_ksplit_out_tiles(n, k))):
        raise KernelError("gemv_ksplit: the handoff does not fit this product")
    _check(load("gemv_ksplit").ni_gemv_ksplit(_dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16),
                                              _dev(out, "out"), m, n, k, mode, *warm_region(warm),
                                              *(handoff.producer_args() if handoff is not None else _NO_HANDOFF),
                                              _stream()), "gemv_ksplit")


def gemv_norm_bf16(h: torch.Tensor, gain: torch.Tensor, eps: float, rows: Optional[torch.Tensor],
                   w: torch.Tensor, out: torch.Tensor, mode: int, warm=None) -> None:
    """The same product with RMSNorm fused in front: x = norm(h[rows]) * gain, h float32
    [*, K] (the residual stream), rows int32 [M] or None for rows 0..M-1.  (``warm`` is accepted
    and dropped: the kernels with the norm fused run at their register limit and carry no request code.)"""
    k = h.shape[1]
    m = h.shape[0] if rows is None else rows.numel()
    n = w.shape[0]
    _gemv_check(m, n, k, w, out, mode, "gemv_norm_bf16")
    if gain.numel() != k:
        raise KernelError("gemv_norm_bf16: gain must have K entries")
    _check(load("gemv_bf16").ni_gemv_norm_bf16(
        _dev(h, "h", torch.float32), _dev(gain, "gain", torch.float32), float(eps),
        _dev(rows, "rows", torch.int32) if rows is not None else None, _dev(w, "w", torch.bfloat16),
        _dev(out, "out"), m, n, k, mode, *warm_region(warm), _stream()), "gemv_norm_bf16")


def gemv_qkv_rope(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float, w: torch.Tensor,
                  q_out: torch.Tensor, k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                  positions: torch.Tensor, seq_of_token: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: torch.Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                  page_size: int, warm=None, pre: Optional["NormHandoff"] = None) -> None:
    """Fused QKV projection of at most 16 single tokens: optional RMSNorm in front (x float32
    residual stream and ``gain`` given) or bfloat16 activations (gain None); rotary encoding of
    adjacent pairs and the paged K/V write behind.  q -> q_out bf16 [M, Hq hd]."""
    m, k = x.shape
    n = (n_q_heads + 2 * n_kv_heads) * head_dim
    if w.shape != (n, k) or q_out.shape != (m, n_q_heads * head_dim):
        raise KernelError("gemv_qkv_rope: shapes do not agree")
    if m > GEMV_MAX_ROWS or k % 8 or head_dim % 16:
        raise KernelError("gemv_qkv_rope: at most 16 rows, K a multiple of 8, head_dim a multiple of 16")
    write = k_pages is not None
    if write and tuple(k_pages.shape[1:]) != (n_kv_heads, page_size, head_dim):
        raise KernelError("gemv_qkv_rope: pages must be [P, Hkv, page_size, head_dim]")
    _check(load("gemv_bf16").ni_gemv_qkv_rope(
        _dev(x, "x", torch.float32 if gain is not None else torch.bfloat16),
        _dev(gain, "gain", torch.float32) if gain is not None else None, float(eps),
        _dev(w, "w", torch.bfloat16), _dev(q_out, "q_out", torch.bfloat16),
        _dev(k_pages, "k_pages", torch.bfloat16) if write else None,
        _dev(v_pages, "v_pages", torch.bfloat16) if write else None,
        _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1],
        _dev(inv_freq, "inv_freq", torch.float32), m, k, n_q_heads, n_kv_heads, head_dim, rotary_dim,
        page_size, 1 if write else 0, *warm_region(warm), *(pre.reader_args() if pre is not None else _NO_PRE),
        _stream()), "gemv_qkv_rope")


def linear_bf16(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype,
                residual: Optional[torch.Tensor] = None, warm=None, handoff: Optional["NormHandoff"] = None) -> Optional[torch.Tensor]:
    """y = x . w^T for bfloat16 operands with FP32 accumulation.

    Up to SKINNY_ROWS rows (decode): the package's own bandwidth kernel; with ``residual`` (float32
    [M, N]) the product is added into it and None is returned.  More rows: a library matrix
    product (cuBLASLt through torch), as the reference's projections are cuBLAS calls
    (src/op/kernels/cuda/matmul_kernel.cu:76-86); the caller adds the result to the residual.
    """
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("linear_bf16: operands must be bfloat16")
    if not x.is_cuda or not w.is_cuda:
        raise KernelError("linear_bf16: operands must be CUDA tensors")
    m, k = x.shape
    if m <= SKINNY_ROWS and k % 8 == 0:
        # a long contraction: K split over a cluster, activations in registers (else re-read per row tile)
        product = gemv_ksplit if (m <= KSPLIT_ROWS and KSPLIT_MIN_K <= k <= KSPLIT_MAX_K
                                  and gemv_ksplit_supports(m, w.shape[0], k)) else gemv_bf16
        if residual is not None:
            product(x, w, residual, ADD_F32, warm, handoff=handoff)
            return None
        out = torch.empty(m, w.shape[0], dtype=out_dtype, device=x.device)
        product(x, w, out, STORE_BF16 if out_dtype == torch.bfloat16 else STORE_F32, warm)
        return out
    if handoff is not None:
        raise KernelError("linear_bf16: a norm can only be handed over by the skinny product (up to 8 rows)")
    if out_dtype == torch.bfloat16:
        return torch.matmul(x, w.t())
    return torch.mm(x, w.t(), out_dtype=torch.float32)


_error_words: Dict[torch.device, torch.Tensor] = {}

# What the codes in the error word stand for (each kernel writes its own when a bounded wait runs out).
DEVICE_ERROR_CODES = {
    1: "tensor-core product (gemm_tc / gemm_tc2): the loader gave up waiting for a free stage",
    2: "tensor-core product (gemm_tc / gemm_tc2): the MMA issuer gave up waiting",
    3: "tensor-core product (gemm_tc / gemm_tc2): the epilogue gave up waiting for an accumulator",
    11: "tensor-core prefill attention: the loader gave up waiting",
    12: "tensor-core prefill attention: the MMA issuer gave up waiting",
    13: "tensor-core prefill attention: the softmax warps gave up waiting",
    21: "swapped-operand product (gemm_swap_tc): the loader gave up waiting",
    22: "swapped-operand product (gemm_swap_tc): the MMA issuer gave up waiting",
    23: "swapped-operand product (gemm_swap_tc): the epilogue gave up waiting",
    31: "fused decode step (decode_fused): a grid barrier was not reached by every block in time",
    32: "fused decode step (decode_fused): the weight loader gave up waiting for a free stage",
    33: "fused decode step (decode_fused): a consumer gave up waiting for its weights",
}


def error_word(device) -> torch.Tensor:
    """The device's error word: int32 [1], zero unless a kernel recorded that one of its bounded
    waits ran out.  The engine copies it to the host with every step's sampled ids."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device(device.type, torch.cuda.current_device())
    w = _error_words.get(device)
    if w is None:
        w = _error_words[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return w


_error_word = error_word


def describe_device_error(code: int) -> str:
    return f"code {code}: {DEVICE_ERROR_CODES.get(code, 'unknown kernel')}"


def check_device_errors(device=None) -> None:
    """Raise if a kernel recorded that one of its bounded waits ran out (synchronises), and
    clear the record."""
    for dev, w in _error_words.items():
        if device is not None and dev != torch.device(device):
            continue
        code = int(w.item())
        if code:
            w.zero_()
            raise KernelError(f"a kernel on {dev} gave up waiting ({describe_device_error(code)}); "
                              f"the results of that step are not valid")


_WAIT_SETTERS = {"gemm_tc": "ni_gemm_tc_set_wait", "gemm_tc2": "ni_gemm_tc2_set_wait",
                 "gemm_swap_tc": "ni_gemm_swap_tc_set_wait",
                 "attention_prefill_tc": "ni_attention_prefill_tc_set_wait"}


def set_wait_limit(module: str, ticks: int = 0, extra_wait: bool = False) -> None:
    """How long a wait inside the module's kernels may last, in clock ticks (0: the default of one
    to two seconds).  ``extra_wait`` makes the kernels wait once more at their end for something
    that never comes - the way the tests make a bounded wait run out."""
    if module not in _WAIT_SETTERS:
        raise KernelError(f"module '{module}' has no bounded waits to set")
    _check_plain(getattr(load(module), _WAIT_SETTERS[module])(int(ticks), 1 if extra_wait else 0),
                 f"set_wait_limit({module})")


def gemm_tc(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, mode: int, kernel: Optional[str] = None,
            accumulators: int = 2, tile_n: int = 0) -> None:
    """out = a[M, K] . b[N, K]^T on the tcgen05 tensor cores (bfloat16 in, FP32 accumulate).
    mode STORE_BF16 / STORE_F32 / ADD_F32 as in gemv_bf16; SWIGLU_BF16: b's rows in blocks of 8
    gate + 8 up rows, out bf16 [M, N/2].  ``kernel``: "pair" = two SMs per 256 x 256 tile
    (gemm_tc2.cu; ``tile_n`` 128 / 192 / 256 columns per tile, 0 = chosen by size), "single" = one SM per
    128 x 256 tile (gemm_tc.cu); default: the pair kernel from 256 rows and 256 columns on."""
    m, k = a.shape
    n = b.shape[0]
    if b.shape[1] != k:
        raise KernelError("gemm_tc: inner sizes do not agree")
    if k % 8:
        raise KernelError(f"gemm_tc: K must be a multiple of 8 (got {k})")
    if mode == SWIGLU_BF16:
        if n % 16 or out.shape != (m, n // 2) or out.dtype != torch.bfloat16:
            raise KernelError("gemm_tc: the SwiGLU epilogue needs N a multiple of 16 and out bf16 [M, N/2]")
    else:
        want = torch.bfloat16 if mode == STORE_BF16 else torch.float32
        if out.shape != (m, n) or out.dtype != want:
            raise KernelError(f"gemm_tc: out must be {want} [M, N]")
    if kernel is None:
        kernel = "pair" if (GEMM_PAIR_DEFAULT and m >= 256 and n >= 256) else "single"
    if kernel == "pair":
        _check(load("gemm_tc2").ni_gemm_tc2(_dev(a, "a", torch.bfloat16), _dev(b, "b", torch.bfloat16), _dev(out, "out"),
                                            m, n, k, mode, accumulators, tile_n, _error_word(a.device).data_ptr(), _stream()),
               "gemm_tc2")
        return
    _check(load("gemm_tc").ni_gemm_tc(_dev(a, "a", torch.bfloat16), _dev(b, "b", torch.bfloat16), _dev(out, "out"),
                                      m, n, k, mode, _error_word(a.device).data_ptr(), _stream()), "gemm_tc")


# Two SMs per tile from 256 rows and columns on: 100 us against 113 us on the gate/up projection of
# a 2,048-token prompt (a block takes in a third less per k-block).
GEMM_PAIR_DEFAULT = True


ROPE_KV = 4                 # gemm_swap_tc: rotary encoding + paged K/V write of a fused QKV projection
SWAP_MAX_ROWS = 128         # most activation rows of the swapped-operand tensor-core product


def gemm_swap_scratch(m: int, n: int, k: int) -> int:
    """FP32 words of scratch that gemm_swap_tc needs for this product (0: K is not split)."""
    f = load("gemm_swap_tc").ni_gemm_swap_tc_scratch
    f.restype = ctypes.c_longlong
    return int(f(m, n, k))


def gemm_swap_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, scratch=None, tickets=None,
                 rope=None) -> None:
    """out = x[M, K] . w[N, K]^T for up to SWAP_MAX_ROWS rows on the tcgen05 tensor cores with the
    weights on the tile's 128 lanes (bfloat16 in, FP32 accumulate).  mode: STORE_BF16 / STORE_F32 /
    ADD_F32 / SWIGLU_BF16 as in gemv_bf16, or ROPE_KV with ``rope`` = (positions, seq_of_token,
    block_table, inv_freq, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim, rotary_dim, page_size)
    and out = q [M, Hq * hd].  ``scratch`` (FP32, gemm_swap_scratch words) and ``tickets`` (int32
    zeros, one per 128 weight rows; left zero) are needed when K is split."""
    m, k = x.shape
    n = w.shape[0]
    if m > SWAP_MAX_ROWS or k % 8:
        raise KernelError(f"gemm_swap_tc: takes at most {SWAP_MAX_ROWS} rows and K a multiple of 8 (M={m}, K={k})")
    if w.shape[1] != k:
        raise KernelError("gemm_swap_tc: inner sizes differ")
    need = gemm_swap_scratch(m, n, k)
    if need and (scratch is None or tickets is None or scratch.numel() < need or tickets.numel() < -(-n // 128)):
        raise KernelError("gemm_swap_tc: scratch or tickets missing or too small")
    if mode == ROPE_KV:
        pos, seq, table, inv_freq, kp, vp, nq, nkv, hd, rot, page = rope
        extra = (_dev(pos, "positions", torch.int32), _dev(seq, "seq_of_token", torch.int32),
                 _dev(table, "block_table", torch.int32), table.shape[1], _dev(inv_freq, "inv_freq", torch.float32),
                 _dev(kp, "k_pages", torch.bfloat16) if kp is not None else None,
                 _dev(vp, "v_pages", torch.bfloat16) if vp is not None else None, nq, nkv, hd, rot, page)
        if out.shape != (m, nq * hd) or out.dtype != torch.bfloat16:
            raise KernelError("gemm_swap_tc: with ROPE_KV out is q, bfloat16 [M, Hq * hd]")
    else:
        extra = (None, None, None, 0, None, None, None, 0, 0, 0, 0, 0)
        want = (m, n // 2) if mode == SWIGLU_BF16 else (m, n)
        dt = torch.float32 if mode in (STORE_F32, ADD_F32) else torch.bfloat16
        if tuple(out.shape) != want or out.dtype != dt:
            raise KernelError(f"gemm_swap_tc: out must be {dt} {list(want)}")
    _check(load("gemm_swap_tc").ni_gemm_swap_tc(
        _dev(x, "x", torch.bfloat16), _dev(w, "w", torch.bfloat16), _dev(out, "out"), m, n, k, mode,
        _dev(scratch, "scratch", torch.float32) if need else None,
        _dev(tickets, "tickets", torch.int32) if need else None, *extra,
        _error_word(x.device).data_ptr(), _stream()), "gemm_swap_tc")


DECODE_HEAD_DIMS = (64, 128)
DECODE_SEGMENT_KEYS = {64: 64, 128: 64}      # keys per shared-memory buffer of a decode-attention block
DECODE_BLOCKS_PER_SM = 4
# The decode kernel reads all but a token's last DECODE_FRESH_KEYS keys while the kernel that
# writes this step's keys may still run, so a portion sent to it has at most this many tokens
# (the same constant as in attention_decode.cu; ni_attention_decode_fresh_keys() returns it).
DECODE_FRESH_KEYS = 2


def decode_splits(n_items: int, n_kv_heads: int, head_dim: int, max_kv_len: int, n_sms: Optional[int] = None) -> int:
    """How many blocks share one (token, kv head): as many as fill the GPU once (three blocks of
    the split kernel are resident per SM; a second wave costs more than longer blocks), each with
    at least 384 keys of the longest context - 256 when there are few pairs, whose blocks are
    bound by latency, not by bandwidth - and cut so that no block is left with a short remainder.
    Middle batches of 64-wide heads (more than one pair per SM): two or three lean blocks per pair,
    four of which fit an SM (batch 32 at 3,072 tokens: 48.1 us unsplit, 43.0 us in two).
    More pairs than the GPU holds at once: one lean block per pair with heads of 64 (four of
    those fit an SM); with heads of 128 (three per SM) the count, up to 4, that fills the last
    wave best (512 pairs: 58 % of two waves unsplit, 87 % of four waves in three parts)."""
    if n_sms is None:
        n_sms = sm_count()
    pairs = max(1, n_items * n_kv_heads)
    chunks = -(-max_kv_len // 64)                 # the kernel cuts a context into 64-key chunks
    slots = n_sms * 3
    if head_dim > 64 and pairs > slots:
        best, best_fill = 1, 0.0
        for s in range(1, 5):
            if s > 1 and chunks < 6 * s:
                break
            fill = pairs * s / (-(-pairs * s // slots) * slots)
            if fill > best_fill + 0.03:
                best, best_fill = s, fill
        per_split = -(-chunks // best)
        return max(1, -(-chunks // per_split))
    if (n_sms * DECODE_BLOCKS_PER_SM) // pairs <= 1:
        return 1                                  # large batch: one lean block per pair
    if pairs > n_sms and head_dim <= 64:          # more than one pair per SM: lean blocks, four per SM
        slots = n_sms * DECODE_BLOCKS_PER_SM
    fill = slots // pairs
    keys_per_split = 256 if pairs <= 16 else 384
    target = max(1, min(64, fill, -(-max_kv_len // keys_per_split)))
    per_split = -(-chunks // target)
    return max(1, -(-chunks // per_split))


PREFILL_MAX_HEAD_DIM = 128
PREFILL_TILE_ROWS = 128      # query rows per block of the flash-style kernel


DECODE_BALANCED_MAX_ITEMS = 1024


def attention_decode_balanced_scratch(n_q_heads: int, n_kv_heads: int, head_dim: int) -> int:
    """Scratch floats that attention_decode_balanced needs (two slots per block; independent of the batch)."""
    lib = load("attention_decode")
    lib.ni_attention_decode_balanced_scratch.restype = ctypes.c_longlong
    lib.ni_attention_decode_balanced_scratch.argtypes = [_I, _I, _I]
    return int(lib.ni_attention_decode_balanced_scratch(n_q_heads, n_kv_heads, head_dim))


def attention_decode_balanced(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token, block_table,
                              n_q_heads, n_kv_heads, head_dim, page_size, window, scale, scratch, tickets, warm=()) -> None:
    """Attention of single query tokens (bfloat16) with the keys of all tokens dealt evenly over a fixed
    set of blocks (three per SM): for many tokens, or tokens of very different context lengths.
    scratch: float32, at least attention_decode_balanced_scratch(...); tickets: int32 zeros, at least
    n_items * Hkv (left zero by the kernel).  At most DECODE_BALANCED_MAX_ITEMS tokens.  ``warm`` as in
    attention_decode."""
    regions = [v for w_ in (list(warm) + [None, None])[:2] for v in warm_region(w_)]
    if head_dim not in DECODE_HEAD_DIMS or n_q_heads // n_kv_heads > 16 or n_items > DECODE_BALANCED_MAX_ITEMS:
        raise KernelError(f"attention_decode_balanced: head_dim {head_dim} / group {n_q_heads // n_kv_heads} / "
                          f"{n_items} tokens not supported")
    if scratch.numel() < attention_decode_balanced_scratch(n_q_heads, n_kv_heads, head_dim) or tickets.numel() < n_items * n_kv_heads:
        raise KernelError("attention_decode_balanced: scratch or tickets too small")
    _check(load("attention_decode").ni_attention_decode_balanced(
        _dev(q, "q", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), _dev(out, "out", torch.bfloat16),
        _dev(token_list, "token_list", torch.int32) if token_list is not None else None, n_items,
        _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], n_q_heads, n_kv_heads,
        head_dim, page_size, int(window) if window else 0, float(scale),
        _dev(scratch, "scratch", torch.float32), _dev(tickets, "tickets", torch.int32), *regions, _stream()),
        "attention_decode_balanced")


def attention_decode_cluster_merge(on: bool) -> None:
    """Whether the splits of a (token, kv head) merge inside a thread-block cluster where they can
    (the default) or always through the scratch buffer and the tickets."""
    _check_plain(load("attention_decode").ni_attention_decode_set_cluster_merge(1 if on else 0), "attention_decode")


def attention_decode(q, k_pages, v_pages, out, token_list, n_items, positions, seq_of_token, block_table,
                     n_q_heads, n_kv_heads, head_dim, page_size, window, scale, n_splits, scratch,
                     tickets, warm=()) -> None:
    """Split-K attention of single query tokens (bfloat16).  ``token_list`` int32 [n_items] or
    None for tokens 0..n_items-1.  scratch: float32, at least n_items * Hq * n_splits *
    (head_dim + 2); tickets: int32 zeros, at least n_items * Hkv (left zero by the kernel).
    ``warm``: up to two (tensor, first byte, bytes) (weights that the kernels after it read): the
    kernel asks the first stretch into L2 when it starts, the second when its own stream has ended."""
    regions = [v for w_ in (list(warm) + [None, None])[:2] for v in warm_region(w_)]
    if head_dim not in DECODE_HEAD_DIMS or n_q_heads // n_kv_heads > 16:
        raise KernelError(f"attention_decode: head_dim {head_dim} / group {n_q_heads // n_kv_heads} not supported")
    if scratch.numel() < n_items * n_q_heads * n_splits * (head_dim + 2) or tickets.numel() < n_items * n_kv_heads:
        raise KernelError("attention_decode: scratch or tickets too small")
    _check(load("attention_decode").ni_attention_decode(
        _dev(q, "q", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), _dev(out, "out", torch.bfloat16),
        _dev(token_list, "token_list", torch.int32) if token_list is not None else None, n_items,
        _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], n_q_heads, n_kv_heads,
        head_dim, page_size, int(window) if window else 0, float(scale), n_splits,
        _dev(scratch, "scratch", torch.float32), _dev(tickets, "tickets", torch.int32),
        *regions, _stream()), "attention_decode")


def attention_prefill_tc_supports(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """True if the tcgen05 prefill attention takes the case: head size 64 or 128, at least two
    query heads per kv head (an odd group's last head shares its block with a silent copy of
    itself), a page size from 8 to 128 that divides 128."""
    return (n_kv_heads > 0 and n_q_heads % n_kv_heads == 0 and n_q_heads // n_kv_heads >= 2
            and head_dim in (64, 128) and 8 <= page_size <= 128 and 128 % page_size == 0)


def attention_prefill(q, k_pages, v_pages, out, tile_seq, tile_row0, n_tiles, cu_q, kv_len, block_table,
                      n_q_heads, n_kv_heads, head_dim, page_size, window, scale, kernel: Optional[str] = None) -> None:
    """Flash-style causal attention of prompt portions (bfloat16): one block per tile of
    PREFILL_TILE_ROWS query rows and query head (mma.sync kernel) or pair of query heads
    (tcgen05 kernel, where it takes the case); tile_seq / tile_row0 int32 [n_tiles] name each
    tile's request and first row.  ``kernel``: "tc" or "mma" to insist on one of the two."""
    if head_dim % 16 or head_dim > PREFILL_MAX_HEAD_DIM:
        raise KernelError(f"attention_prefill: head_dim {head_dim} not supported (multiples of 16 up to 128)")
    tc_ok = attention_prefill_tc_supports(n_q_heads, n_kv_heads, head_dim, page_size)
    if kernel == "tc" and not tc_ok:
        raise KernelError("attention_prefill: the tcgen05 kernel does not take this case")
    if tc_ok and kernel != "mma":
        _check(load("attention_prefill_tc").ni_attention_prefill_tc(
            _dev(q, "q", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
            _dev(v_pages, "v_pages", torch.bfloat16), _dev(out, "out", torch.bfloat16), q.shape[0], k_pages.shape[0],
            _dev(tile_seq, "tile_seq", torch.int32), _dev(tile_row0, "tile_row0", torch.int32), n_tiles,
            _dev(cu_q, "cu_q", torch.int32), _dev(kv_len, "kv_len", torch.int32),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1], n_q_heads, n_kv_heads,
            head_dim, page_size, int(window) if window else 0, float(scale), _error_word(q.device).data_ptr(),
            _stream()), "attention_prefill_tc")
        return
    _check(load("attention_prefill").ni_attention_prefill(
        _dev(q, "q", torch.bfloat16), _dev(k_pages, "k_pages", torch.bfloat16),
        _dev(v_pages, "v_pages", torch.bfloat16), _dev(out, "out", torch.bfloat16),
        _dev(tile_seq, "tile_seq", torch.int32), _dev(tile_row0, "tile_row0", torch.int32), n_tiles,
        _dev(cu_q, "cu_q", torch.int32), _dev(kv_len, "kv_len", torch.int32),
        _dev(block_table, "block_table", torch.int32), block_table.shape[1], n_q_heads, n_kv_heads,
        head_dim, page_size, int(window) if window else 0, float(scale), _stream()), "attention_prefill")


_argmax_keys: Dict[torch.device, torch.Tensor] = {}   # per device: merge keys, zero between calls


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = index of the largest logit of row r, ties to the lowest index."""
    n, v = logits.shape
    keys = _argmax_keys.get(logits.device)
    if keys is None and not torch.cuda.is_current_stream_capturing():
        keys = _argmax_keys[logits.device] = torch.zeros(4096, dtype=torch.int64, device=logits.device)
    use_keys = keys is not None and n <= keys.numel()
    _check(load("sampling").ni_argmax(_dev(logits, "logits", torch.float32), _dev(out, "out", torch.int32),
                                      n, v, keys.data_ptr() if use_keys else None, _stream()), "argmax")


def repetition_penalty(logits: torch.Tensor, ids: torch.Tensor, penalties: torch.Tensor) -> None:
    """In place: logits[r, id] = l / p if l > 0 else l * p for the ids listed in row r of
    ``ids`` (int32 [R, W], padded with -1, each id at most once per row)."""
    n, v = logits.shape
    if ids.shape[0] != n or penalties.numel() != n:
        raise KernelError("repetition_penalty: one id list and one penalty per row")
    _check(load("sampling").ni_repetition_penalty(
        _dev(logits, "logits", torch.float32), _dev(ids, "ids", torch.int32),
        _dev(penalties, "penalties", torch.float32), n, v, ids.shape[1], _stream()), "repetition_penalty")


def sample_by_cluster(on: bool) -> None:
    """Whether ``sample`` gives every row a thread-block cluster where the vocabulary allows it (the
    default) or always one block (the two give the same tokens; for comparisons)."""
    _check_plain(load("sampling").ni_sample_set_cluster(1 if on else 0), "sample")


def sample(logits, out, temperatures, top_ks, top_ps, seeds, counters) -> None:
    """One token per row by the row's own parameters; seeds and counters are 64-bit."""
    n, v = logits.shape
    for name, t in (("temperatures", temperatures), ("top_ks", top_ks), ("top_ps", top_ps),
                    ("seeds", seeds), ("counters", counters)):
        if t.numel() != n:
            raise KernelError(f"sample: {name} must have one entry per row")
    _check(load("sampling").ni_sample(
        _dev(logits, "logits", torch.float32), _dev(out, "out", torch.int32),
        _dev(temperatures, "temperatures", torch.float32), _dev(top_ks, "top_ks", torch.int32),
        _dev(top_ps, "top_ps", torch.float32), _dev(seeds, "seeds", torch.int64),
        _dev(counters, "counters", torch.int64), n, v, _stream()), "sample")


# ---- the fused decode step ---------------------------------------------------------------------------
FUSED_MAX_GROUPS = 4


class FusedLayer(ctypes.Structure):
    """One scheduled layer run of the fused decode kernel (mirrors FdLayer of decode_fused.cu)."""
    _fields_ = [("w_qkv", _P), ("w_o", _P), ("w_gate_up", _P), ("w_down", _P), ("gain_mixer", _P), ("gain_ffn", _P),
                ("k_pages", _P), ("v_pages", _P), ("eps_mixer", _F), ("eps_ffn", _F), ("write_cache", _I), ("group", _I)]


class FusedParams(ctypes.Structure):
    """Arguments of the fused decode kernel (mirrors FdParams of decode_fused.cu)."""
    _fields_ = [("layers", _P), ("inv_freq", _P), ("embedding", _P), ("lm_head", _P), ("gain_final", _P),
                ("tokens", _P), ("positions", _P), ("seq_of_token", _P), ("logit_rows", _P),
                ("tables", _P * FUSED_MAX_GROUPS),
                ("h", _P), ("q", _P), ("att", _P), ("act", _P), ("logits", _P), ("partials", _P), ("tickets", _P),
                ("barrier", _P), ("error", _P), ("trace", _P), ("wait_limit", _LL), ("bt_stride", _I * FUSED_MAX_GROUPS),
                ("n_layers", _I), ("M", _I), ("R", _I), ("d", _I), ("n_q_heads", _I), ("n_kv_heads", _I),
                ("head_dim", _I), ("rotary_dim", _I), ("inter", _I), ("vocab", _I), ("page_size", _I), ("window", _I),
                ("scale_log2e", _F), ("eps_final", _F), ("skip_arrive_at", _I)]


def decode_fused_lib() -> ctypes.CDLL:
    lib = load("decode_fused")
    if not getattr(lib, "_ni_checked", False):
        for fn, size in (("ni_decode_fused_params_size", ctypes.sizeof(FusedParams)),
                         ("ni_decode_fused_layer_size", ctypes.sizeof(FusedLayer))):
            f = getattr(lib, fn)
            f.restype = ctypes.c_longlong
            if int(f()) != size:
                raise KernelError(f"decode_fused: the argument records of the built kernel and of ops.py differ ({fn})")
        if lib.ni_decode_fused_max_groups() != FUSED_MAX_GROUPS:
            raise KernelError("decode_fused: FD_MAX_GROUPS of the built kernel differs from ops.FUSED_MAX_GROUPS")
        lib._ni_checked = True
    return lib


def decode_fused_supports(m: int, d: int, n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                          inter: int, vocab: int, page_size: int) -> bool:
    return bool(decode_fused_lib().ni_decode_fused_supports(m, d, n_q_heads, n_kv_heads, head_dim, rotary_dim, inter,
                                                            vocab, page_size))


def decode_fused_partials(m: int, n_kv_heads: int, head_dim: int) -> int:
    f = decode_fused_lib().ni_decode_fused_partials
    f.restype = ctypes.c_longlong
    f.argtypes = [_I, _I, _I]
    return int(f(m, n_kv_heads, head_dim))


def decode_fused(params: FusedParams) -> None:
    """One decode step of up to 8 single tokens as one persistent kernel (see decode_fused.cu).
    The caller fills ``params`` with device pointers and sizes; the launch is on the current stream."""
    _check(decode_fused_lib().ni_decode_fused(ctypes.byref(params), _stream()), "decode_fused")
