"""The engine's operations: thin checked wrappers over the package's CUDA kernels.

Every function takes CUDA tensors and launches on the current stream.  There
is no CPU path and no silent fallback: a CPU tensor, an unsupported dtype or a
refused size raises.  Matrix products of the bfloat16 engine go to cuBLAS
through ``torch.mm`` (the reference uses the same library for them:
src/layers/linear.rs:5-7); everything else is this package's own code.
"""
from __future__ import annotations

import contextlib
import ctypes
import gc
import os
import sys
from typing import Optional

import torch

from .build import load_cuda_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
ERROR_BITS = {1: "a token id outside the embedding table", 2: "a cache slot outside the pool",
              4: "a position beyond the rotary table", 8: "sampling found no valid token",
              16: "a bounded wait inside a kernel ran out"}
_RC = {-1: "unsupported dtype", -2: "a size the kernel refuses", -3: "misaligned pointer"}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    """Checks that the operands are on the device.  Every wrapper that launches calls this first, so it is also
    where products that wait in the chain (see ``chain_linear``) are launched: whatever runs next may read them."""
    flush_chain()
    _cuda_only(*tensors)


def _cuda_only(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


def _contig(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("a kernel was given a non-contiguous tensor")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# Launches of this package's kernels so far (library matrix products are not counted).
_launches = [0]


def launch_count() -> int:
    return _launches[0]


def add_launches(n: int) -> None:
    """Account for kernels that ran without passing through a wrapper (a replayed graph)."""
    _launches[0] += n


def _ok(rc: int, name: str, kernels: int = 1) -> None:
    if rc == 0:
        _launches[0] += kernels
        return
    if rc in _RC:
        raise KernelError(f"{name}: {_RC[rc]}")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


# --------------------------------------------------------------------------- error word
_error_words = {}


def error_word(device: torch.device) -> torch.Tensor:
    """The device word into which kernels OR their error bits."""
    key = torch.device(device).index or 0
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_errors(device: torch.device) -> None:
    """Read the error word (synchronises) and raise if a kernel flagged a fault."""
    flush_chain()
    word = error_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        _reset_chain_state(device)
        what = [text for bit, text in ERROR_BITS.items() if value & bit]
        raise KernelError("a kernel refused an access: " + "; ".join(what))


_staging = {}


class PendingRead:
    """Token ids and the error word on their way to the host: ``begin_read`` enqueues the copies and an event,
    ``finish`` waits for that event only, so kernels enqueued after ``begin_read`` keep the GPU busy meanwhile."""

    def __init__(self, buf, n, event, device):
        self.buf, self.n, self.event, self.device = buf, n, event, device

    def finish(self) -> list:
        self.event.synchronize()
        value = int(self.buf[self.n])
        if value:
            error_word(self.device).zero_()
            _reset_chain_state(self.device)
            what = [text for bit, text in ERROR_BITS.items() if value & bit]
            raise KernelError("a kernel refused an access: " + "; ".join(what))
        return self.buf[:self.n].tolist()


def begin_read(ids: torch.Tensor) -> PendingRead:
    """Start copying ``ids`` (int32, on the device) and the error word into pinned memory (two small copies on
    the current stream, then an event).  Four staging buffers per device take turns: at most three reads may be
    pending when a fourth begins."""
    flush_chain()
    device = ids.device
    key = device.index or 0
    n = ids.numel()
    ring = _staging.get(key)
    if ring is None or ring[0][0].numel() < n + 1:
        size = max(1024, 2 * (n + 1))
        ring = _staging[key] = ([torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(4)], [0])
    bufs, turn = ring
    buf = bufs[turn[0] % len(bufs)]
    turn[0] += 1
    buf[:n].copy_(ids.reshape(-1), non_blocking=True)
    buf[n:n + 1].copy_(error_word(device), non_blocking=True)
    event = torch.cuda.Event()
    event.record(torch.cuda.current_stream(device))
    return PendingRead(buf, n, event, device)


# --------------------------------------------------------------------------- libraries
def _elementwise():
    return load_cuda_library("elementwise.cu")


def padded_head_dim(head_dim: int) -> int:
    """The compile-time head size of the all-sizes attention kernels for a real head size: the next multiple of 16."""
    return -(-head_dim // 16) * 16


def _attention(head_dim: int):
    """The all-sizes attention library for a real head size (any even number up to 512)."""
    if head_dim % 2 != 0 or not 2 <= head_dim <= 512:
        raise KernelError(f"head size {head_dim} is refused: the attention kernels take even head sizes up to 512")
    return load_cuda_library("attention.cu", {"HEAD_DIM": padded_head_dim(head_dim)})


# --------------------------------------------------------------------------- element-wise
def embedding(ids: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    _cuda(ids, table)
    _contig(ids, table)
    if ids.dtype != torch.int32:
        raise KernelError("token ids must be int32")
    out = torch.empty((ids.numel(), table.shape[1]), dtype=out_dtype, device=table.device)
    rc = _elementwise().b200_embedding(_p(out), _p(table), _p(ids), ids.numel(), table.shape[1],
                                       table.shape[0], _code(out), _code(table),
                                       _p(error_word(table.device)), _stream())
    _ok(rc, "embedding")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
             rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rms_norm(x[rows[r]]) * weight (rows None: every row, in place allowed)."""
    return _norm(x, None, weight, eps, out, rows, False)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                 out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                 write_residual: bool = True) -> torch.Tensor:
    """s = x + residual in float; residual <- round(s); out = rms_norm(s) * weight."""
    return _norm(x, residual, weight, eps, out, rows, write_residual)


def _norm(x, residual, weight, eps, out, rows, write_residual):
    _cuda(x, residual, weight, out, rows)
    _contig(x, residual, weight, out, rows)
    width = x.shape[-1]
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} elements, the rows have {width}")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise KernelError("the residual must have the shape and dtype of x")
    n = x.numel() // width if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("row indices must be int32")
    if out is None:
        out = torch.empty((n, width), dtype=x.dtype, device=x.device)
    elif out.dtype != x.dtype or out.numel() != n * width:
        raise KernelError("norm output has the wrong dtype or size")
    rc = _elementwise().b200_rms_norm(_p(out), _p(x), _p(residual), _p(weight), _p(rows), n, width,
                                      ctypes.c_float(eps), int(bool(write_residual)), _code(x),
                                      _code(weight), _stream())
    _ok(rc, "rms_norm")
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _cuda(gate_up, out)
    _contig(gate_up, out)
    tokens, width2 = gate_up.shape
    if width2 % 2:
        raise KernelError("silu_mul needs an even width")
    if out is None:
        out = torch.empty((tokens, width2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    rc = _elementwise().b200_silu_mul(_p(out), _p(gate_up), tokens, width2 // 2, _code(gate_up), _stream())
    _ok(rc, "silu_mul")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _cuda(x)
    _contig(x)
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    rc = _elementwise().b200_cast(_p(out), _p(x), ctypes.c_longlong(x.numel()), _code(out), _code(x), _stream())
    _ok(rc, "cast")
    return out


# --------------------------------------------------------------------------- between QKV and attention
def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
             v_cache: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
             k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
             sin: Optional[torch.Tensor], rot_dim: int, positions: torch.Tensor,
             slots: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Per-head norm, rotary encoding, cache store.  ``slots`` None: nothing is stored."""
    _cuda(qkv, q_out, k_cache, v_cache, q_weight, k_weight, cos, sin, positions, slots)
    _contig(qkv, q_out, k_cache, v_cache, q_weight, k_weight, cos, sin, positions, slots)
    tokens = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("qkv width does not match the head counts")
    if slots is not None and (k_cache is None or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype):
        raise KernelError("the cache must have the activations' dtype")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("q and k norm weights come together")
    if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32):
        raise KernelError("rotary tables must be float32")
    wcode = _code(q_weight) if q_weight is not None else _code(qkv)
    if q_weight is not None and k_weight.dtype != q_weight.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    # cache tensors are [pages + 1, kv_heads, page_size, head_dim]
    page_size = 1 if k_cache is None else k_cache.shape[2]
    cache_slots = 0 if k_cache is None else k_cache.shape[0] * k_cache.shape[2]
    if k_cache is not None and (k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim):
        raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
    max_pos = 0 if cos is None else cos.shape[0]
    lib = load_cuda_library("qkv_post.cu")
    rc = lib.b200_qkv_post(_p(qkv), _p(q_out), _p(k_cache), _p(v_cache), _p(q_weight), _p(k_weight),
                           ctypes.c_float(eps), _p(cos), _p(sin), rot_dim, max_pos, _p(positions), _p(slots),
                           tokens, num_heads, num_kv_heads, head_dim, page_size, ctypes.c_longlong(cache_slots),
                           _code(qkv), wcode, _p(error_word(qkv.device)), _stream())
    _ok(rc, "qkv_post")


# --------------------------------------------------------------------------- attention
def tcgen05_attention_launches() -> tuple:
    """(launches of the one-tile kernel, launches of the two-tile kernel) of the tcgen05 prefill attention so far."""
    lib = load_cuda_library("attention_tcgen05.cu")
    lib.b200_attention_tcgen05_launches.restype = ctypes.c_longlong
    return int(lib.b200_attention_tcgen05_launches(0)), int(lib.b200_attention_tcgen05_launches(1))


def prefill_attention(q, k_cache, v_cache, out, block_table, cu_q, kv_len, prefix_len, rows, n_rows,
                      max_q_len, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                      tiles_per_cta: int = 0) -> None:
    """Causal attention of prompt portions over the paged cache (rows: which batch rows).

    ``tiles_per_cta`` (head size 128 on the tcgen05 kernel only): 1 or 2 tiles of 128 query vectors per
    CTA, 0 lets the kernel's launcher choose by the size of the grid."""
    _cuda(q, k_cache, v_cache, out, block_table, cu_q, kv_len, prefix_len, rows)
    _contig(q, k_cache, v_cache, out, block_table)
    if n_rows == 0:
        return
    if k_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("q, cache and output must share a dtype")
    if decode_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim, page_size):
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[2] != page_size:
            raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
        box_rows = min(page_size, 32)
        group = num_heads // num_kv_heads
        if head_dim == 128 and 128 % group == 0 and max_q_len * group >= 128:
            # head size 128 and at least one full tile of 128 query vectors: the tcgen05 kernel
            rc = load_cuda_library("attention_tcgen05.cu").b200_prefill_attention_tcgen05(
                _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(block_table),
                block_table.shape[-1], _p(cu_q), _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads,
                num_kv_heads, page_size, int(window or 0), ctypes.c_float(scale), int(tiles_per_cta),
                _p(error_word(q.device)), _stream())
            _ok(rc, "prefill_attention_tcgen05")
            return
        rc = _attention_mma(head_dim).b200_prefill_attention_mma(
            _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(block_table),
            block_table.shape[-1], _p(cu_q), _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads,
            num_kv_heads, page_size, int(window or 0), ctypes.c_float(scale), _p(error_word(q.device)), _stream())
        _ok(rc, "prefill_attention_mma")
        return
    rc = _attention(head_dim).b200_prefill_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(block_table), block_table.shape[-1], _p(cu_q),
        _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads, num_kv_heads, page_size,
        int(window or 0), ctypes.c_float(scale), _code(q), head_dim, _stream())
    _ok(rc, "prefill_attention")


MMA_MAX_GROUP = 16
MMA_MAX_HEAD_DIM = 256


def _attention_mma(head_dim: int):
    return load_cuda_library("attention_mma.cu", {"HEAD_DIM": head_dim})


def decode_uses_tensor_cores(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                             page_size: int) -> bool:
    """bfloat16 caches with at most 16 query heads per KV head, heads up to 256 wide and a page size
    that is a power of two take the TMA / tensor-core kernel; everything else the all-sizes kernel."""
    return (dtype == torch.bfloat16 and num_heads // num_kv_heads <= MMA_MAX_GROUP
            and head_dim <= MMA_MAX_HEAD_DIM and head_dim % 16 == 0
            and page_size > 0 and page_size & (page_size - 1) == 0)


_kv_maps = {}


def kv_tensor_map(cache: torch.Tensor, box_rows: int):
    """The 128-byte TMA descriptor of a cache tensor [pages + 1, kv_heads, page_size, head_dim] (made once)."""
    key = (cache.data_ptr(), tuple(cache.shape), box_rows)
    buf = _kv_maps.get(key)
    if buf is None:
        if cache.dtype != torch.bfloat16 or not cache.is_contiguous() or cache.dim() != 4:
            raise KernelError("a TMA descriptor needs a contiguous bfloat16 cache [pages + 1, kv_heads, page_size, head_dim]")
        buf = ctypes.create_string_buffer(128)
        rows = cache.shape[0] * cache.shape[1] * cache.shape[2]
        rc = _attention_mma(cache.shape[3]).b200_kv_tensor_map(buf, _p(cache), ctypes.c_longlong(rows), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a cache tensor could not be made (code {rc})")
        if len(_kv_maps) > 4096:
            _kv_maps.clear()
        _kv_maps[key] = buf
    return buf


def decode_ctas_per_split(dtype: torch.dtype, n_rows: int, num_heads: int, num_kv_heads: int, head_dim: int,
                          page_size: int) -> int:
    """CTAs that the decode kernel launches for each split of the keys."""
    if decode_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim, page_size):
        return n_rows * num_kv_heads
    return n_rows * num_kv_heads * ((num_heads // num_kv_heads + 3) // 4)


def decode_scratch_floats(n_rows: int, num_heads: int, head_dim: int, splits: int) -> int:
    """Floats of scratch that decode attention needs (partial outputs are rows of the padded head size)."""
    return 0 if splits <= 1 else n_rows * num_heads * splits * (padded_head_dim(head_dim) + 2)


def decode_attention(q, k_cache, v_cache, out, scratch, block_table, cu_q, kv_len, rows, n_rows,
                     num_heads, num_kv_heads, head_dim, page_size, window, scale, splits) -> None:
    """Attention of single decoded tokens, the keys split over ``splits`` blocks per row."""
    _cuda(q, k_cache, v_cache, out, scratch, block_table, cu_q, kv_len, rows)
    _contig(q, k_cache, v_cache, out, block_table, scratch)
    if n_rows == 0:
        return
    if k_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("q, cache and output must share a dtype")
    need = decode_scratch_floats(n_rows, num_heads, head_dim, splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"decode attention needs {need} floats of scratch")
    if decode_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim, page_size):
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[2] != page_size:
            raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
        box_rows = min(page_size, 32)
        rc = _attention_mma(head_dim).b200_decode_attention_mma(
            _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(scratch), _p(block_table), block_table.shape[-1],
            _p(cu_q), _p(kv_len), _p(rows), n_rows, num_heads, num_kv_heads, page_size, int(window or 0),
            ctypes.c_float(scale), splits, _p(error_word(q.device)), _stream())
        in_kernel = splits == 1 or (splits in (2, 4, 8) and splits * num_kv_heads * n_rows <= _sm_count(q.device))
        _ok(rc, "decode_attention_mma", 1 if in_kernel else 2)      # (a cluster of 2, 4 or 8 splits combines them itself)
        return
    rc = _attention(head_dim).b200_decode_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scratch), _p(block_table), block_table.shape[-1],
        _p(cu_q), _p(kv_len), _p(rows), n_rows, num_heads, num_kv_heads, page_size, int(window or 0),
        ctypes.c_float(scale), splits, _code(q), head_dim, _stream())
    _ok(rc, "decode_attention", 2 if splits > 1 else 1)


# --------------------------------------------------------------------------- few-row products with fused ends
SKINNY_MAX_ROWS = 16
EPI_PLAIN_BF16, EPI_PLAIN_F32, EPI_SWIGLU, EPI_QKV = 0, 1, 2, 3


class _SkinnyParams(ctypes.Structure):
    """Mirror of ``SkinnyParams`` in csrc/skinny_linear.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("ksplit", ctypes.c_int), ("mode", ctypes.c_int), ("out", ctypes.c_void_p),
                ("nh", ctypes.c_int), ("nkv", ctypes.c_int), ("rot_dim", ctypes.c_int), ("max_pos", ctypes.c_int),
                ("page_size", ctypes.c_int), ("cache_slots", ctypes.c_longlong), ("qk_eps", ctypes.c_float),
                ("q_w", ctypes.c_void_p), ("k_w", ctypes.c_void_p), ("qk_w_f32", ctypes.c_int),
                ("cos_table", ctypes.c_void_p), ("sin_table", ctypes.c_void_p), ("positions", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("err", ctypes.c_void_p), ("post_residual", ctypes.c_void_p), ("post_sum_out", ctypes.c_void_p),
                ("post_stats", ctypes.c_void_p), ("stats_in", ctypes.c_void_p), ("stats_tiles", ctypes.c_int),
                ("trace", ctypes.c_void_p)]


# For tuning: an int64 tensor [4096, 32] on the device; the first thread of every CTA of the next single-product
# launches then leaves the nanosecond clock there at the kernel's phases (0 start, 1 dependency wait over, 2 x staged,
# 3 products done, 4 own sums stored, 5 the cluster's sums have met, 6 a rank other than 0 leaves, 7 epilogue done),
# and in slots 16 to 31 the SM's cycle counter at the same places.
skinny_trace: Optional[torch.Tensor] = None


class PendingNorm:
    """An RMSNorm (with or without a residual add before it) that has not run: the product that consumes it runs
    it as its prologue.

    ``residual`` None: the plain norm of ``x``.  ``residual_out`` is the tensor that will hold the rounded sum
    (None: the sum is not kept).  ``materialize()`` runs the norm as a kernel of its own, for a consumer that
    cannot fuse it.
    """

    def __init__(self, x, residual, weight, eps, rows=None, write_residual=True):
        self.x, self.residual, self.weight, self.eps, self.rows = x, residual, weight, float(eps), rows
        self.residual_out = torch.empty_like(residual) if write_residual and residual is not None else None
        self.dtype, self.device = x.dtype, x.device
        n = x.shape[0] if rows is None else rows.numel()
        self.shape = (n, x.shape[-1])

    def materialize(self) -> torch.Tensor:
        if self.residual is None:
            return rms_norm(self.x, self.weight, self.eps, rows=self.rows)
        if self.residual_out is not None:
            flush_chain()
            self.residual_out.copy_(self.residual)
            return add_rms_norm(self.x, self.residual_out, self.weight, self.eps, rows=self.rows)
        return add_rms_norm(self.x, self.residual, self.weight, self.eps, rows=self.rows, write_residual=False)


_weight_maps = {}
_sm_counts = {}


def _sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[key]


def _skinny():
    # (with a trace buffer set, the build that stamps its clocks: a tuning aid, compiled when first asked for)
    lib = load_cuda_library("skinny_linear.cu", {"SKINNY_TRACE": 1} if skinny_trace is not None else None)
    if not getattr(lib, "_checked", False):
        if lib.b200_skinny_params_size() != ctypes.sizeof(_SkinnyParams):
            raise KernelError("the parameter block of skinny_linear.cu and its Python mirror differ")
        lib._checked = True
    return lib


def _weight_map(weight: torch.Tensor, box_rows: int):
    key = (weight.data_ptr(), tuple(weight.shape), box_rows)
    buf = _weight_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = _skinny().b200_weight_tensor_map(buf, _p(weight), ctypes.c_longlong(weight.shape[0]),
                                              ctypes.c_longlong(weight.shape[1]), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a weight matrix could not be made (code {rc})")
        if len(_weight_maps) > 8192:
            _weight_maps.clear()
        _weight_maps[key] = buf
    return buf


def skinny_ok(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
              head_dim: int = 0) -> bool:
    """Whether the few-row kernel takes this product: bfloat16 activations and weight, at most 16 rows,
    K a multiple of 8 and at most 8 x 4032 (8 rows) or 8 x 1984 (16 rows); QKV: head size 64, 128 or 256."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    k = weight.shape[1]
    if not 0 < rows <= SKINNY_MAX_ROWS or k % 8 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if k > 8 * (4032 if rows <= 8 else 1984):
        return False
    if mode == EPI_QKV and head_dim not in (64, 128, 256):
        return False
    if mode == EPI_SWIGLU and weight.shape[0] % 2:
        return False
    return True


@contextlib.contextmanager
def graph_capture(graph: "torch.cuda.CUDAGraph"):
    """Capture the stream's work into ``graph``.

    Python's cycle collector runs first and is held off until the capture has ended.  A dead reference cycle that
    owns CUDA graphs or device memory (an engine that the caller dropped, say) is else freed at whatever allocation
    inside the capture happens to start a collection; destroying a graph or returning its memory is not permitted
    while a stream captures, and the capture ends with "operation failed due to a previous error during capture"."""
    flush_chain()
    gc.collect()
    held = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
            flush_chain()
    finally:
        if held:
            gc.enable()


def skinny_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                  qkv: Optional[dict] = None, out: Optional[torch.Tensor] = None, norm_after=None,
                  stats=None) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for at most 16 rows, in one kernel.

    ``out``: the tensor to fill (PLAIN and SWIGLU; made here when None).  ``norm_after`` = (residual, sum_out,
    stats): a PLAIN bfloat16 product also begins the add + RMSNorm that follows it: round(y + residual) goes to
    ``sum_out`` and the sums of squares per tile of columns to ``stats`` (float32 [tiles, 16]).  ``stats`` =
    (that tensor, tiles): a product whose ``x`` is a ``PendingNorm`` of such a y and residual takes the rows'
    statistics from there and reads only its own columns (``residual_out`` is then not written: it is ``sum_out``).

    ``x``: a bfloat16 tensor [rows, K], or a ``PendingNorm`` (then the residual add and the norm run as the
    prologue and ``x.residual_out`` is filled).  ``mode``: EPI_PLAIN_BF16 / EPI_PLAIN_F32: the product;
    EPI_SWIGLU: silu(gate) * up for a weight of gate rows then up rows; EPI_QKV: per-head norm, rotary
    encoding and the cache store, with ``qkv`` = the keyword arguments of ``qkv_post`` (without ``qkv``);
    the result is then ``q_out``.
    """
    _flush_held()
    if isinstance(x, PendingNorm) and x.residual is None:
        x = x.materialize()                                    # (this kernel's prologue always adds a residual)
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    _cuda(src, weight, rows_t)
    _contig(src, weight, rows_t)
    m = src.shape[0] if rows_t is None else rows_t.numel()
    n, k = weight.shape
    if src.shape[-1] != k:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    head_dim = qkv["head_dim"] if qkv else 0
    if not skinny_ok(m, weight, src.dtype, mode, head_dim):
        raise KernelError("the few-row product refuses this size or dtype")
    lib = _skinny()
    P = _SkinnyParams()
    P.x, P.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    if pending is not None:
        if pending.residual.dtype != torch.bfloat16 or pending.residual.shape != src.shape:
            raise KernelError("the residual must be bfloat16 and have the shape of x")
        P.residual = pending.residual.data_ptr()
        P.residual_out = 0 if pending.residual_out is None or stats is not None else pending.residual_out.data_ptr()
        if stats is not None:
            P.stats_in, P.stats_tiles = stats[0].data_ptr(), int(stats[1])
        P.norm_w, P.norm_w_f32, P.eps = pending.weight.data_ptr(), int(pending.weight.dtype == torch.float32), pending.eps
        if pending.weight.numel() != k or pending.weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("the norm weight must have K elements, bfloat16 or float32")
    P.M, P.N, P.K, P.mode = m, n, k, mode
    dev = src.device
    P.err = error_word(dev).data_ptr()
    P.trace = 0 if skinny_trace is None else skinny_trace.data_ptr()
    if mode == EPI_QKV:
        nh, nkv = qkv["num_heads"], qkv["num_kv_heads"]
        out = qkv["q_out"]
        kc, vc = qkv.get("k_cache"), qkv.get("v_cache")
        qw, kw = qkv.get("q_weight"), qkv.get("k_weight")
        cos, sin = qkv.get("cos"), qkv.get("sin")
        slots = qkv.get("slots")
        _cuda(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots)
        if n != (nh + 2 * nkv) * head_dim or out.shape != (m, nh * head_dim) or out.dtype != torch.bfloat16:
            raise KernelError("qkv sizes do not fit the weight")
        if slots is not None and (kc is None or kc.dtype != torch.bfloat16 or kc.shape[1] != nkv or kc.shape[3] != head_dim):
            raise KernelError("the cache must be bfloat16 [pages + 1, kv_heads, page_size, head_dim]")
        if (qw is None) != (kw is None) or (qw is not None and qw.dtype != kw.dtype):
            raise KernelError("q and k norm weights come together and share a dtype")
        P.nh, P.nkv, P.rot_dim = nh, nkv, int(qkv.get("rot_dim", 0))
        P.max_pos = 0 if cos is None else cos.shape[0]
        P.page_size = 1 if kc is None else kc.shape[2]
        P.cache_slots = 0 if kc is None else kc.shape[0] * kc.shape[2]
        P.qk_eps = float(qkv.get("eps", 0.0))
        P.q_w, P.k_w = (0 if qw is None else qw.data_ptr()), (0 if kw is None else kw.data_ptr())
        P.qk_w_f32 = int(qw is not None and qw.dtype == torch.float32)
        P.cos_table, P.sin_table = (0 if cos is None else cos.data_ptr()), (0 if sin is None else sin.data_ptr())
        P.positions = qkv["positions"].data_ptr()
        P.slots = 0 if slots is None else slots.data_ptr()
        P.k_cache, P.v_cache = (0 if kc is None else kc.data_ptr()), (0 if vc is None else vc.data_ptr())
    elif out is None:
        out = _few_row_out(m, n, mode, dev)
    if norm_after is not None:
        P.post_residual, P.post_sum_out, P.post_stats = (t.data_ptr() for t in norm_after)
    P.out = out.data_ptr()
    sms = _sm_count(dev)
    box = lib.b200_skinny_box_rows(mode, head_dim, n, sms)
    rc = lib.b200_skinny_linear(_weight_map(weight, box), ctypes.byref(P), head_dim, sms, _stream())
    _ok(rc, "skinny_linear")
    return out


def _few_row_out(m: int, n: int, mode: int, device) -> torch.Tensor:
    if mode == EPI_SWIGLU:
        return torch.empty((m, n // 2), dtype=torch.bfloat16, device=device)
    return torch.empty((m, n), dtype=torch.float32 if mode == EPI_PLAIN_F32 else torch.bfloat16, device=device)


class _StreamParams(ctypes.Structure):
    """Mirror of ``StreamParams`` in csrc/stream_linear.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("w", ctypes.c_void_p), ("M", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("mode", ctypes.c_int), ("out", ctypes.c_void_p),
                ("post_residual", ctypes.c_void_p), ("post_sum_out", ctypes.c_void_p), ("post_stats", ctypes.c_void_p),
                ("rw", ctypes.c_int), ("ks", ctypes.c_int), ("groups", ctypes.c_int), ("tiles", ctypes.c_int),
                ("xd", ctypes.c_int), ("pair", ctypes.c_int)]


def _stream_lib():
    lib = load_cuda_library("stream_linear.cu")
    if not getattr(lib, "_checked", False):
        if lib.b200_stream_params_size() != ctypes.sizeof(_StreamParams):
            raise KernelError("the parameter block of stream_linear.cu and its Python mirror differ")
        lib._checked = True
    return lib


# Few-row products on weights of at least this many bytes take the streaming kernel (every thread copies its own share
# of the weights, one CTA an SM walks over many tiles: csrc/stream_linear.cu) instead of the ring kernel
# (csrc/skinny_linear.cu), where the rows of x fit its shared memory: a rule of sizes, fixed by the environment or by
# assignment, never by a measurement.  Measured in a decode step at batch 8: 4.28 -> 3.91 ms at the Qwen3-8B sizes
# (gate/up and the head), 1.320 -> 1.308 ms at the Qwen3-0.6B sizes (the head); smaller matrices are faster on the
# ring kernel (1.41 ms with the 0.6B gate/up here).
stream_min_bytes = int(os.environ.get("LLM_INFER_B200_STREAM_MIN_BYTES", 64 << 20))
stream_pair = int(os.environ.get("LLM_INFER_B200_STREAM_PAIR", -1))


def stream_ok(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
              norm: bool = True) -> bool:
    """Whether the streaming kernel can run this product: bfloat16 activations and weight, at most 16 rows, K a
    multiple of 32; plain or SwiGLU.  Behind a norm (``norm``) the rows must fit its shared memory beside the weights
    on their way (8 rows of about 6,000 columns, 16 of about 3,000); without one, longer rows come with the weights'
    copies."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    if not 0 < rows <= SKINNY_MAX_ROWS or weight.shape[1] % 32 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if mode not in (EPI_PLAIN_BF16, EPI_PLAIN_F32, EPI_SWIGLU) or (mode == EPI_SWIGLU and weight.shape[0] % 2):
        return False
    return bool(_stream_lib().b200_stream_fits(mode, rows, weight.shape[0], weight.shape[1], int(norm)))


def stream_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                 norm: bool = True) -> bool:
    """Whether a few-row product (behind a norm or not) is routed to the streaming kernel: a weight of
    ``stream_min_bytes`` or more, and rows of x that fit the kernel's shared memory; rows that do not fit (and have no
    norm before them) only for more than 8 rows of a weight that the ring kernel would else take, since it falls off
    there (Qwen3-8B down projection, 16 rows: 22.8 against 37.4 us, a decode step at batch 16 6.36 -> 5.96 ms; with 8
    rows 20.2 against 21.3 us alone and a decode step no faster for it; the Qwen3-32B down projection is faster on
    the library: 49 against 64 us)."""
    nbytes = 2 * weight.shape[0] * weight.shape[1]
    if few_row_route != "single" or nbytes < stream_min_bytes:
        return False
    if stream_ok(rows, weight, act_dtype, mode, True):
        return True
    return not norm and rows > 8 and nbytes < single_max_bytes and stream_ok(rows, weight, act_dtype, mode, False)


def stream_tile_cols(mode: int, m: int, n: int, k: int, norm: bool) -> int:
    """Columns of the output that one tile of the streaming kernel covers for a product of ``m`` rows with a weight
    [n, k] (its tiles of statistics)."""
    return _stream_lib().b200_stream_tile_cols(mode, m, n, k, int(norm))


def stream_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None, norm_after=None, rw: int = 0, ks: int = 0,
                  xd: int = -1, pair: Optional[int] = None) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for at most 16 rows and a large weight (csrc/stream_linear.cu).

    ``x``: a bfloat16 tensor [rows, K] or a ``PendingNorm`` (with or without a residual); ``mode``: EPI_PLAIN_BF16,
    EPI_PLAIN_F32 or EPI_SWIGLU; ``norm_after`` = (residual, sum_out, stats [tiles, 16]) as for ``skinny_linear``,
    with tiles = ceil(N / ``stream_tile_cols(...)``); ``rw``, ``ks``: the launch's shape (groups of 16 weight rows a
    tile: 1 or 2; warps that split K: up to 24), 0 for the launcher's choice; ``xd``: whether the rows of x come with
    the weights' copies instead of waiting in shared memory (1, 0, or -1: where they do not fit; never behind a norm);
    ``pair``: clusters of two CTAs that stage half of the rows of x each (1, 0, or -1: where the grid fills the GPU).
    """
    _flush_held()
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    _cuda(src, weight, rows_t)
    _contig(src, weight, rows_t)
    m = src.shape[0] if rows_t is None else rows_t.numel()
    n, k = weight.shape
    if src.shape[-1] != k:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    if not stream_ok(m, weight, src.dtype, mode, pending is not None):
        raise KernelError("the streaming product refuses this size or dtype")
    P = _StreamParams()
    P.x, P.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    if pending is not None:
        w = pending.weight
        if w.numel() != k or w.dtype not in (torch.float32, torch.bfloat16) or not w.is_cuda:
            raise KernelError("the norm weight must have K elements, bfloat16 or float32, on the device")
        P.norm_w, P.norm_w_f32, P.eps = w.data_ptr(), int(w.dtype == torch.float32), pending.eps
        if pending.residual is not None:
            res = pending.residual
            if res.dtype != torch.bfloat16 or res.shape != src.shape or not res.is_contiguous():
                raise KernelError("the residual must be bfloat16, contiguous and have the shape of x")
            P.residual = res.data_ptr()
            P.residual_out = 0 if pending.residual_out is None else pending.residual_out.data_ptr()
    P.w, P.M, P.N, P.K, P.mode = weight.data_ptr(), m, n, k, mode
    if out is None:
        out = _few_row_out(m, n, mode, src.device)
    if norm_after is not None:
        P.post_residual, P.post_sum_out, P.post_stats = (t.data_ptr() for t in norm_after)
    P.out, P.rw, P.ks, P.xd = out.data_ptr(), rw, ks, xd
    P.pair = stream_pair if pair is None else pair
    rc = _stream_lib().b200_stream_linear(ctypes.byref(P), _sm_count(src.device), _stream())
    _ok(rc, "stream_linear")
    return out


# A lazy PLAIN bfloat16 product of the "single" route is held back until the next launch is known: if that is a
# product behind an add + RMSNorm of this product's result, the held product's epilogue begins the norm (the rounded
# sum and the rows' sums of squares), and the next product reads only its own columns instead of whole rows, which
# every one of its CTAs would otherwise fetch (at 4,096 columns that read took 5 of a product's 20 us).
class _Held:
    def __init__(self, x, weight, x_rows, out, stream=False):
        self.x, self.weight, self.x_rows, self.out, self.stream = x, weight, x_rows, out, stream


_held: Optional[_Held] = None


def _flush_held(norm_after=None) -> None:
    """Launch the product that is held back (with the norm that follows it begun in its epilogue, if given)."""
    global _held
    h = _held
    if h is None:
        return
    _held = None
    if h.stream:
        stream_linear(h.x, h.weight, EPI_PLAIN_BF16, x_rows=h.x_rows, out=h.out, norm_after=norm_after)
    else:
        skinny_linear(h.x, h.weight, EPI_PLAIN_BF16, x_rows=h.x_rows, out=h.out, norm_after=norm_after)


def _single_lazy(x, weight, mode, x_rows, qkv, lazy) -> torch.Tensor:
    """The "single" route of ``few_row_linear``."""
    global _held
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    m = src.shape[0] if rows_t is None else rows_t.numel()
    to_stream = mode != EPI_QKV and src.is_cuda and stream_takes(m, weight, src.dtype, mode, pending is not None)
    h = _held
    stats = None
    # (the streaming kernel gets the rows' statistics from its own loop: nothing is handed to it)
    if (h is not None and not to_stream and pending is not None and pending.x is h.out and pending.residual is not None
            and x_rows is None and pending.residual.dtype == torch.bfloat16
            and pending.residual.shape == h.out.shape and pending.residual.is_contiguous()):
        n = h.weight.shape[0]
        if h.stream:
            cols = stream_tile_cols(EPI_PLAIN_BF16, h.out.shape[0], n, h.weight.shape[1], isinstance(h.x, PendingNorm))
        else:
            cols = _skinny().b200_skinny_tile_rows(EPI_PLAIN_BF16, 0, n, _sm_count(h.out.device))
        if 0 < cols <= 128:
            tiles = -(-n // cols)
            stat_t = torch.empty((tiles, SKINNY_MAX_ROWS), dtype=torch.float32, device=h.out.device)
            sum_out = pending.residual_out if pending.residual_out is not None else torch.empty_like(pending.residual)
            _flush_held((pending.residual, sum_out, stat_t))
            stats = (stat_t, tiles)
    _flush_held()
    if (lazy and mode == EPI_PLAIN_BF16 and stats is None and (pending is None or pending.residual is not None)
            and src.is_cuda and (to_stream or skinny_ok(m, weight, src.dtype, mode))):
        _held = _Held(x, weight, x_rows, _few_row_out(m, weight.shape[0], mode, src.device), stream=to_stream)
        return _held.out
    if to_stream:
        return stream_linear(x, weight, mode, x_rows=x_rows)
    return skinny_linear(x, weight, mode, x_rows=x_rows, qkv=qkv, stats=stats)


# --------------------------------------------------------------------------- chains of few-row products
CHAIN_MAX_ROWS = 64
PRO_NONE, PRO_ADD_NORM, PRO_NORM = 0, 1, 2
# How products of few rows are routed: "single" (one kernel per product, up to 16 rows: csrc/skinny_linear.cu),
# "chain" (one persistent kernel for consecutive products, up to 64 rows: csrc/linear_chain.cu) or "library" (cuBLAS
# with the norm, rotation and activation as kernels of their own).  Fixed by the environment or by assignment,
# never by a measurement, so that two processes given the same input run the same kernels.  Measured on B200
# (decode, batch 8, context 4,096): "single" 1.42 ms a step at the Qwen3-0.6B sizes and 4.4 ms at the 8B sizes,
# "chain" 1.86 ms and 6.2 ms (its barriers and tile hand-overs cost what the launches did), so "single" is the default.
few_row_route = os.environ.get("LLM_INFER_B200_FEW_ROW", "single")
single_max_bytes = int(os.environ.get("LLM_INFER_B200_SINGLE_MAX_BYTES", 224 << 20))
# Weights up to this size are multiplied in tiles of 16 rows that one CTA owns (see csrc/linear_chain.cu).
chain_narrow_bytes = int(os.environ.get("LLM_INFER_B200_CHAIN_NARROW_BYTES", 48 << 20))


class _ChainOp(ctypes.Structure):
    """Mirror of ``ChainOp`` in csrc/linear_chain.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("stats_in", ctypes.c_void_p),
                ("stats_out", ctypes.c_void_p), ("stats_res_in", ctypes.c_void_p), ("stats_res_out", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("q_w", ctypes.c_void_p), ("k_w", ctypes.c_void_p),
                ("cos_table", ctypes.c_void_p), ("sin_table", ctypes.c_void_p), ("positions", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("cache_slots", ctypes.c_longlong), ("prologue", ctypes.c_int), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("stats_tiles", ctypes.c_int), ("M", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("mode", ctypes.c_int), ("nh", ctypes.c_int), ("nkv", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("rot_dim", ctypes.c_int), ("max_pos", ctypes.c_int),
                ("page_size", ctypes.c_int), ("qk_w_f32", ctypes.c_int), ("qk_eps", ctypes.c_float),
                ("narrow", ctypes.c_int), ("box_rows", ctypes.c_int), ("tiles", ctypes.c_int), ("kblocks", ctypes.c_int), ("per", ctypes.c_int), ("ctas", ctypes.c_int),
                ("first_cta", ctypes.c_int), ("ticket_off", ctypes.c_int)]


def _chain_lib():
    lib = load_cuda_library("linear_chain.cu")
    if not getattr(lib, "_checked", False):
        if lib.b200_chain_op_size() != ctypes.sizeof(_ChainOp):
            raise KernelError("the product block of linear_chain.cu and its Python mirror differ")
        lib.b200_chain_scratch_floats.restype = ctypes.c_longlong
        lib._checked = True
    return lib


_chain_maps = {}
_chain_state = {}
_CHAIN_TICKETS = 1 << 16


def _chain_map(weight: torch.Tensor, box_rows: int):
    key = (weight.data_ptr(), tuple(weight.shape), box_rows)
    buf = _chain_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = _chain_lib().b200_chain_weight_map(buf, _p(weight), ctypes.c_longlong(weight.shape[0]),
                                                ctypes.c_longlong(weight.shape[1]), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a weight matrix could not be made (code {rc})")
        if len(_chain_maps) > 8192:
            _chain_maps.clear()
        _chain_maps[key] = buf
    return buf


def _chain_buffers(device):
    """Scratch for partial sums (sized for 64 rows on every SM: 9.7 MB), tickets and the grid barrier's words of
    one device; made once, so that a graph may capture launches that use them."""
    key = torch.device(device).index or 0
    st = _chain_state.get(key)
    if st is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the chain kernel's buffers must exist before a graph is captured")
        floats = int(_chain_lib().b200_chain_scratch_floats(CHAIN_MAX_ROWS, _sm_count(device)))
        st = _chain_state[key] = dict(scratch=torch.empty(floats, dtype=torch.float32, device=device),
                                      tickets=torch.zeros(_CHAIN_TICKETS, dtype=torch.int32, device=device),
                                      sync=torch.zeros(_chain_lib().b200_chain_sync_words(), dtype=torch.int32,
                                                       device=device))
    return st


def _reset_chain_state(device) -> None:
    """After a wait inside the chain kernel ran out its barrier words and tickets may hold anything."""
    st = _chain_state.get(torch.device(device).index or 0)
    if st is not None:
        st["tickets"].zero_()
        st["sync"].zero_()


def chain_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                head_dim: int = 0) -> bool:
    """Whether the chain kernel takes this product: bfloat16 activations and weight, at most 64 rows, K a multiple
    of 8; QKV: a head size that divides 128."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    if not 0 < rows <= CHAIN_MAX_ROWS or weight.shape[1] % 8 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if mode == EPI_QKV and (head_dim <= 0 or 128 % head_dim):
        return False
    if mode == EPI_SWIGLU and weight.shape[0] % 2:
        return False
    return True


def few_row_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                  head_dim: int = 0, norm: bool = True) -> bool:
    """Whether a product of ``rows`` rows runs on this package's few-row kernels (with the norm before it and the
    epilogue after it fused in) rather than as a library product with those as kernels of their own.  ``norm``: the
    product may come behind a norm (False: its input is a plain tensor)."""
    if few_row_route == "chain" and chain_takes(rows, weight, act_dtype, mode, head_dim):
        return True
    if few_row_route == "library":
        return False
    if mode != EPI_QKV and stream_takes(rows, weight, act_dtype, mode, norm):
        return True
    if not skinny_ok(rows, weight, act_dtype, mode, head_dim):
        return False
    # The single-product kernel gives every CTA the rows of x to normalise and one tile of 128 weight rows; on the
    # largest layer matrices (gate/up and down at the Qwen3-32B sizes, 262 and 524 MB) the library product with the norm
    # and activation as kernels of their own was measured faster (14.8 against 18.9 ms a decode step at batch 8).
    return mode == EPI_PLAIN_F32 or 2 * weight.shape[0] * weight.shape[1] < single_max_bytes


class _Chain:
    def __init__(self, device):
        self.device = device
        self.ops, self.weights, self.keep = [], [], []
        self.by_out = {}                 # data pointer of a product's output -> (index, output tensor)
        self.stats_from = {}             # index of a product -> index of the product that leaves its rows' statistics


_chain: Optional[_Chain] = None
# For tuning: an int64 tensor [SMs, 64] on the device; every CTA's first thread then leaves the nanosecond clock there at
# eight places of every product of the next launches (start, barrier passed, row scales, x staged, products done,
# sums added, epilogue done).
chain_trace: Optional[torch.Tensor] = None
chain_stages = int(os.environ.get("LLM_INFER_B200_CHAIN_STAGES", 8))


def few_row_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                   qkv: Optional[dict] = None, lazy: bool = False) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for few rows; arguments as ``skinny_linear``.

    ``lazy`` (on the "chain" route): the product is not launched here.  It joins the products that wait, and all
    of them run in one persistent kernel when something else is about to be launched (``flush_chain``; every
    wrapper of this module does that first).  The returned tensor is filled by then: code that touches it with
    anything but this module's wrappers must call ``flush_chain()`` before.  Without ``lazy`` the product (and
    whatever waited before it) is launched before this returns."""
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    m = src.shape[0] if rows_t is None else rows_t.numel()
    head_dim = qkv["head_dim"] if qkv else 0
    if few_row_route == "chain" and chain_takes(m, weight, src.dtype, mode, head_dim):
        out = _chain_append(pending, src, rows_t, m, weight, mode, qkv)
        if not lazy:
            flush_chain()
        return out
    return _single_lazy(x, weight, mode, x_rows, qkv, lazy)


def _chain_append(pending, src, rows_t, m, weight, mode, qkv) -> torch.Tensor:
    global _chain
    _cuda_only(src, weight, rows_t)
    _contig(src, weight, rows_t)
    n, k = weight.shape
    if src.shape[-1] != k or src.dim() != 2:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    dev = src.device
    if _chain is not None and _chain.device != dev:
        flush_chain()
    if _chain is None:
        _chain = _Chain(dev)
    ch = _chain
    op = _ChainOp()
    op.x, op.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    op.M, op.N, op.K, op.mode = m, n, k, mode
    if pending is not None:
        w = pending.weight
        if w.numel() != k or w.dtype not in (torch.float32, torch.bfloat16) or not w.is_cuda:
            raise KernelError("the norm weight must have K elements, bfloat16 or float32, on the device")
        op.norm_w, op.norm_w_f32, op.eps = w.data_ptr(), int(w.dtype == torch.float32), pending.eps
        op.prologue = PRO_NORM
        if pending.residual is not None:
            res = pending.residual
            if res.dtype != torch.bfloat16 or res.shape != src.shape or not res.is_contiguous():
                raise KernelError("the residual must be bfloat16, contiguous and have the shape of x")
            op.prologue = PRO_ADD_NORM
            op.residual = res.data_ptr()
            made = ch.by_out.get(src.data_ptr())
            if made is not None and made[1] is src and ch.ops[made[0]].mode == EPI_PLAIN_BF16 \
                    and ch.ops[made[0]].stats_out is None:
                # x is the output of a product of this chain: that product's epilogue adds the residual, stores the
                # rounded sum and leaves the rows' sums of squares, so nobody has to read whole rows again
                prev = ch.ops[made[0]]
                tiles = _chain_lib().b200_chain_tiles(EPI_PLAIN_BF16, prev.N, 1)      # (narrow tiles are the most)
                stats = torch.empty(tiles * CHAIN_MAX_ROWS, dtype=torch.float32, device=dev)
                sum_out = pending.residual_out if pending.residual_out is not None else torch.empty_like(res)
                prev.stats_out, prev.stats_res_in, prev.stats_res_out = stats.data_ptr(), res.data_ptr(), sum_out.data_ptr()
                op.stats_in = stats.data_ptr()
                ch.stats_from[len(ch.ops)] = made[0]          # (how many tiles wrote them is known at the launch)
                ch.keep += [stats, sum_out]
            else:
                op.residual_out = 0 if pending.residual_out is None else pending.residual_out.data_ptr()
        ch.keep.append(pending)
    if mode == EPI_QKV:
        nh, nkv, head_dim = qkv["num_heads"], qkv["num_kv_heads"], qkv["head_dim"]
        out = qkv["q_out"]
        kc, vc = qkv.get("k_cache"), qkv.get("v_cache")
        qw, kw = qkv.get("q_weight"), qkv.get("k_weight")
        cos, sin = qkv.get("cos"), qkv.get("sin")
        slots = qkv.get("slots")
        _cuda_only(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots)
        _contig(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots)
        if n != (nh + 2 * nkv) * head_dim or out.shape != (m, nh * head_dim) or out.dtype != torch.bfloat16:
            raise KernelError("qkv sizes do not fit the weight")
        if slots is not None and (kc is None or kc.dtype != torch.bfloat16 or kc.shape[1] != nkv or kc.shape[3] != head_dim
                                  or vc is None or vc.dtype != torch.bfloat16):
            raise KernelError("the cache must be bfloat16 [pages + 1, kv_heads, page_size, head_dim]")
        if (qw is None) != (kw is None) or (qw is not None and qw.dtype != kw.dtype):
            raise KernelError("q and k norm weights come together and share a dtype")
        if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32):
            raise KernelError("rotary tables must be float32")
        op.nh, op.nkv, op.head_dim, op.rot_dim = nh, nkv, head_dim, int(qkv.get("rot_dim", 0)) if cos is not None else 0
        op.max_pos = 0 if cos is None else cos.shape[0]
        op.page_size = 1 if kc is None else kc.shape[2]
        op.cache_slots = 0 if kc is None else kc.shape[0] * kc.shape[2]
        op.qk_eps = float(qkv.get("eps", 0.0))
        op.q_w, op.k_w = (0 if qw is None else qw.data_ptr()), (0 if kw is None else kw.data_ptr())
        op.qk_w_f32 = int(qw is not None and qw.dtype == torch.float32)
        op.cos_table, op.sin_table = (0 if cos is None else cos.data_ptr()), (0 if sin is None else sin.data_ptr())
        op.positions = qkv["positions"].data_ptr()
        op.slots = 0 if slots is None else slots.data_ptr()
        op.k_cache, op.v_cache = (0 if kc is None else kc.data_ptr()), (0 if vc is None else vc.data_ptr())
        ch.keep.append(qkv)
    elif mode == EPI_SWIGLU:
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=dev)
    else:
        out = torch.empty((m, n), dtype=torch.float32 if mode == EPI_PLAIN_F32 else torch.bfloat16, device=dev)
    op.out = out.data_ptr()
    ch.ops.append(op)
    ch.weights.append(weight)
    ch.keep += [src, rows_t, out]
    ch.by_out[out.data_ptr()] = (len(ch.ops) - 1, out)
    return out


def chain_pending() -> int:
    """Products that wait in the chain."""
    return 0 if _chain is None else len(_chain.ops)


def flush_chain() -> None:
    """Launch the products that wait in the chain (at most six per launch of the persistent kernel)."""
    global _chain
    _flush_held()
    ch = _chain
    if ch is None:
        return
    _chain = None
    lib = _chain_lib()
    st = _chain_buffers(ch.device)
    most = lib.b200_chain_max_ops()
    sms = _sm_count(ch.device)
    groups = [range(at, min(at + most, len(ch.ops))) for at in range(0, len(ch.ops), most)]
    for group in groups:                                   # the kind of tile depends on the launch's largest row count
        rows = max(ch.ops[i].M for i in group)
        for i in group:
            op, w = ch.ops[i], ch.weights[i]
            op.narrow = lib.b200_chain_narrow(op.mode, op.N, op.K, rows, ctypes.c_longlong(chain_narrow_bytes))
            op.box_rows = lib.b200_chain_box_rows(op.mode, op.narrow)
    for i, source in ch.stats_from.items():
        ch.ops[i].stats_tiles = lib.b200_chain_tiles(ch.ops[source].mode, ch.ops[source].N, ch.ops[source].narrow)
    with torch.cuda.device(ch.device):
        for group in groups:
            ops_now = [ch.ops[i] for i in group]
            if sum(lib.b200_chain_tiles(o.mode, o.N, o.narrow) for o in ops_now) > _CHAIN_TICKETS:
                raise KernelError("a chain of products has more tiles than the ticket array holds")
            block = (_ChainOp * len(ops_now))(*ops_now)
            maps = ctypes.create_string_buffer(b"".join(_chain_map(ch.weights[i], ch.ops[i].box_rows).raw for i in group),
                                               128 * len(ops_now))
            rc = lib.b200_linear_chain(block, maps, len(ops_now), _p(st["scratch"]), _p(st["tickets"]), _p(st["sync"]),
                                       _p(error_word(ch.device)), _p(chain_trace), chain_stages, sms, _stream())
            _ok(rc, "linear_chain")


# --------------------------------------------------------------------------- many-row products on tcgen05
GEMM_PLAIN, GEMM_SWIGLU = 0, 1
_gemm_maps = {}


def _gemm_map(t: torch.Tensor):
    key = (t.data_ptr(), tuple(t.shape))
    buf = _gemm_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = load_cuda_library("gemm_tcgen05.cu").b200_gemm_tensor_map(buf, _p(t), ctypes.c_longlong(t.shape[0]),
                                                                       ctypes.c_longlong(t.shape[1]))
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a matrix could not be made (code {rc})")
        if len(_gemm_maps) > 8192:
            _gemm_maps.clear()
        _gemm_maps[key] = buf
    return buf


def gemm_tc_ok(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> bool:
    """bfloat16 row-major operands on the device, K a multiple of 8 (16-byte rows for TMA); SwiGLU: even N."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_cuda and weight.is_cuda
            and x.dim() == 2 and weight.dim() == 2 and x.is_contiguous() and weight.is_contiguous()
            and x.shape[1] == weight.shape[1] and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and (mode == GEMM_PLAIN or weight.shape[0] % 2 == 0))


def gemm_tc_pays(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> bool:
    """Whether the tcgen05 product is the faster way: measured on B200, the fused SwiGLU form ties or beats the
    library product followed by the activation kernel once every SM has several tiles of 128 x 256 and K is
    long (1,369 against 1,354 TFLOP/s at 2,048 x 24,576 x 4,096); on smaller shapes the library is ahead."""
    if mode != GEMM_SWIGLU or not gemm_tc_ok(x, weight, mode):
        return False
    tiles = -(-x.shape[0] // 128) * -(-(weight.shape[0] // 2) // 128)
    return x.shape[1] >= 2048 and tiles >= 4 * _sm_count(x.device)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> torch.Tensor:
    """x . weight^T on the tcgen05 tensor cores (TMA-fed, float sums in tensor memory), bfloat16 out.
    ``GEMM_SWIGLU``: weight = [gate rows; up rows]; the result is silu(x . gate^T) * (x . up^T)."""
    flush_chain()
    if not gemm_tc_ok(x, weight, mode):
        raise KernelError("the tcgen05 product takes contiguous bfloat16 [M, K] and [N, K] with K a multiple of 8")
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty((m, n // 2 if mode == GEMM_SWIGLU else n), dtype=torch.bfloat16, device=x.device)
    a_map = ctypes.create_string_buffer(128)          # activations move: their descriptor is made per call
    lib = load_cuda_library("gemm_tcgen05.cu")
    rc = lib.b200_gemm_tensor_map(a_map, _p(x), ctypes.c_longlong(m), ctypes.c_longlong(k))
    if rc != 0:
        raise KernelError(f"the TMA descriptor of the activations could not be made (code {rc})")
    rc = lib.b200_gemm_tcgen05(a_map, _gemm_map(weight), _p(out), m, n, k, mode, _p(error_word(x.device)), _stream())
    _ok(rc, "gemm_tcgen05")
    return out


# --------------------------------------------------------------------------- matrix products
def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a[M, K] . w[N, K]^T in true 32-bit on CUDA cores."""
    _cuda(a, w, out)
    _contig(a, w, out)
    if a.dtype != torch.float32 or w.dtype != torch.float32 or a.shape[1] != w.shape[1]:
        raise KernelError("gemm_f32 takes float32 [M, K] and [N, K]")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    rc = load_cuda_library("gemm_f32.cu").b200_gemm_f32(_p(a), _p(w), _p(out), m, n, k, _stream())
    _ok(rc, "gemm_f32")
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           lazy: bool = False) -> torch.Tensor:
    """x[M, K] . weight[N, K]^T, no bias.  ``lazy``: see ``few_row_linear``.

    float32 x float32: this package's 32-bit kernel.  bfloat16 x bfloat16: few rows (see ``few_row_takes``) on
    this package's few-row kernels, more on cuBLAS with float accumulation.  Mixed dtypes are multiplied in
    32-bit (the narrower operand is widened first).
    """
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32 and weight.dtype == torch.float32:
        return cast(gemm_f32(x, weight), out_dtype)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        if out_dtype in (torch.bfloat16, torch.float32) and x.dim() == 2 and x.is_contiguous() and x.is_cuda:
            mode = EPI_PLAIN_F32 if out_dtype == torch.float32 else EPI_PLAIN_BF16
            if few_row_takes(x.shape[0], weight, x.dtype, mode, norm=False):
                return few_row_linear(x, weight, mode, lazy=lazy)
        _cuda(x, weight)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, weight.t())
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if weight.dtype == torch.float32:
        return cast(gemm_f32(cast(x, torch.float32), weight), out_dtype)
    return cast(gemm_f32(x, cast(weight, torch.float32)), out_dtype)


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax takes float32 logits [rows, vocab] with unit inner stride")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    rc = load_cuda_library("sampling.cu").b200_argmax(_p(logits), ctypes.c_longlong(logits.stride(0)),
                                                      logits.shape[0], logits.shape[1], _p(out),
                                                      _p(error_word(logits.device)), _stream())
    _ok(rc, "argmax")
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``params``: uint8 [rows, 32] device tensor of packed rows (see sampling.pack_rows)."""
    _cuda(logits, params, uniforms)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample takes float32 logits [rows, vocab] with unit inner stride")
    if params.numel() * params.element_size() != logits.shape[0] * 32:
        raise KernelError("sampling parameters must hold 32 bytes per row")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    rc = load_cuda_library("sampling.cu").b200_sample(_p(logits), ctypes.c_longlong(logits.stride(0)),
                                                      logits.shape[0], logits.shape[1], _p(params), _p(out),
                                                      _p(uniforms), _p(error_word(logits.device)), _stream())
    _ok(rc, "sample")
    return out
