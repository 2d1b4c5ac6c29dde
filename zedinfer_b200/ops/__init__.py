"""Python faces of the CUDA kernels.  Every function writes into tensors the caller gives.

Nothing here runs on the CPU and nothing falls back to a library model or a library
attention; matrix products of bfloat16 operands go to cuBLAS through ``torch.mm`` where
the reference's engine calls cuBLASLt (src/backend/ops/linear/nvidia/linear_cublas.cu:201-231),
and 32-bit products go to the SIMT kernel of ``csrc/gemm_simt.cu`` so that no
reduced-precision matrix mode can slip in.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ._lib import (BF16, F32, KernelError, Library, c_float, c_int, c_ll, dtype_code, need_contiguous, need_cuda,
                   need_int32, ptr, stream)

# Library products keep float32 sums: without this cuBLAS may pick split-K kernels that add partial sums in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

_elementwise = Library("elementwise")
_gemm_simt = Library("gemm_simt")
_attention_generic = Library("attention_generic")
_sampling = Library("sampling")
_attention_mma = Library("attention_mma")
_gemm_smallm = Library("gemm_smallm")
_gemm_tcgen05 = Library("gemm_tcgen05")
_attention_tcgen05 = Library("attention_tcgen05")
SMALL_M_ROWS = 16                # the weight-streaming kernel takes up to this many rows

__all__ = ["KernelError", "embedding", "rmsnorm", "add_rmsnorm", "rope_append", "rope_table", "gemm_smallm_rope", "can_fuse_rope_product", "silu_mul", "add", "cast",
           "gemm_nt", "linear", "linear_for_residual", "gemm_smallm", "gemm_tcgen05", "gemm_tcgen05_tiles", "tcgen05_status", "status_word", "linear_silu_mul", "raise_if_tcgen05_failed", "paged_attention", "attention", "decode_attention", "decode_attention_tma", "prefill_attention", "prefill_attention_tcgen05", "argmax", "sample", "repetition_penalty", "advance_decode"]


def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(table, ids, out)
    need_int32("ids", ids)
    need_contiguous("table", table), need_contiguous("out", out), need_contiguous("ids", ids)
    n, hidden = ids.numel(), table.shape[1]
    if out.shape != (n, hidden):
        raise KernelError(f"embedding: out has shape {tuple(out.shape)}, expected {(n, hidden)}")
    _elementwise.call("zi_embedding", ptr(table), c_int(dtype_code(table.dtype)), ptr(ids), ptr(out),
                      c_int(dtype_code(out.dtype)), c_int(n), c_int(hidden), c_int(table.shape[0]), stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    need_cuda(x, w, out)
    need_contiguous("x", x), need_contiguous("w", w), need_contiguous("out", out)
    rows, hidden = x.shape
    if w.numel() != hidden or out.shape != x.shape:
        raise KernelError(f"rmsnorm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    _elementwise.call("zi_rmsnorm", ptr(x), c_int(dtype_code(x.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                      c_int(dtype_code(out.dtype)), c_int(rows), c_int(hidden), c_float(eps), stream())


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], w: torch.Tensor, eps: float,
                out: torch.Tensor, row_idx: Optional[torch.Tensor] = None, write_residual: bool = True) -> None:
    """``residual (+= delta)``, then ``out = rmsnorm(residual) * w``.  ``residual`` is float32.

    With ``row_idx`` the output row ``r`` is computed from input row ``row_idx[r]`` and the
    residual is left untouched.
    """
    need_cuda(residual, delta, w, out, row_idx)
    if residual.dtype != torch.float32:
        raise KernelError(f"add_rmsnorm: the residual stream is float32, got {residual.dtype}")
    need_contiguous("residual", residual), need_contiguous("w", w), need_contiguous("out", out)
    hidden = residual.shape[1]
    if delta is not None and delta.dim() == 3:
        # partial sums of a product whose K was cut (linear_for_residual): float32 [parts, rows, hidden]
        need_contiguous("delta", delta)
        if delta.dtype != torch.float32 or delta.shape[1:] != residual.shape:
            raise KernelError(f"add_rmsnorm: partial sums {tuple(delta.shape)} {delta.dtype} vs residual {tuple(residual.shape)}")
        if row_idx is not None:
            need_int32("row_idx", row_idx), need_contiguous("row_idx", row_idx)
        rows = row_idx.numel() if row_idx is not None else residual.shape[0]
        if w.numel() != hidden or out.shape != (rows, hidden):
            raise KernelError(f"add_rmsnorm: w {tuple(w.shape)} / out {tuple(out.shape)} do not fit {(rows, hidden)}")
        _elementwise.call("zi_add_rmsnorm_parts", ptr(residual), ptr(delta), c_int(delta.shape[0]),
                          c_ll(delta.shape[1] * hidden), ptr(w), c_int(dtype_code(w.dtype)), ptr(out),
                          c_int(dtype_code(out.dtype)), ptr(row_idx), c_int(rows), c_int(hidden), c_float(eps),
                          c_int(1 if write_residual else 0), stream())
        return
    if delta is not None:
        need_contiguous("delta", delta)
        if delta.shape != residual.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs residual {tuple(residual.shape)}")
    if row_idx is not None:
        need_int32("row_idx", row_idx), need_contiguous("row_idx", row_idx)
        rows = row_idx.numel()
    else:
        rows = residual.shape[0]
    if w.numel() != hidden or out.shape != (rows, hidden):
        raise KernelError(f"add_rmsnorm: w {tuple(w.shape)} / out {tuple(out.shape)} do not fit {(rows, hidden)}")
    _elementwise.call("zi_add_rmsnorm", ptr(residual), ptr(delta),
                      c_int(dtype_code(delta.dtype) if delta is not None else F32), ptr(w), c_int(dtype_code(w.dtype)),
                      ptr(out), c_int(dtype_code(out.dtype)), ptr(row_idx), c_int(rows), c_int(hidden), c_float(eps),
                      c_int(1 if write_residual else 0), stream())


ROPE_TABLE_MAX_TOKENS = 64       # steps of at most this many tokens rotate with the step's table of angles


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, cache: Optional[torch.Tensor], tables: torch.Tensor,
                tok_seg: torch.Tensor, pos: torch.Tensor, inv_freq: torch.Tensor, n_heads: int, n_kv_heads: int,
                head_dim: int, page_size: int, page_stride: int, kv_stride: int, write_kv: bool = True,
                cs: Optional[torch.Tensor] = None) -> None:
    """Rotate q (and k) by position and append k, v to the cache pages of each token's request.  ``cs``: the step's
    table of angles (:func:`rope_table` of ``pos`` and ``inv_freq``); steps of at most 64 tokens then read their cosines
    and sines there instead of computing them in every layer."""
    need_cuda(qkv, q_out, cache, tables, tok_seg, pos, inv_freq, cs)
    if cs is not None and (cs.dtype != torch.float32 or cs.shape != (qkv.shape[0], head_dim) or not cs.is_contiguous()):
        raise KernelError(f"rope_append: cs {tuple(cs.shape)} must be contiguous float32 [{qkv.shape[0]}, {head_dim}]")
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q_out", q_out)
    n = qkv.shape[0]
    if qkv.stride(1) != 1 or qkv.shape[1] < (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"rope_append: qkv {tuple(qkv.shape)} does not hold {n_heads}+2*{n_kv_heads} heads of {head_dim}")
    if q_out.dtype != qkv.dtype or (cache is not None and cache.dtype != qkv.dtype):
        raise KernelError("rope_append: qkv, q_out and the cache must share one dtype")
    if inv_freq.dtype != torch.float32 or inv_freq.numel() != head_dim // 2:
        raise KernelError("rope_append: inv_freq must be float32 of head_dim/2 entries")
    if write_kv and cache is None:
        raise KernelError("rope_append: write_kv needs a cache")
    _elementwise.call("zi_rope_append", ptr(qkv), ptr(q_out), ptr(cache), c_int(dtype_code(qkv.dtype)), ptr(tables),
                      ptr(tok_seg), ptr(pos), ptr(inv_freq), c_int(n), c_int(qkv.stride(0)), c_int(n_heads),
                      c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(tables.shape[1]),
                      c_ll(page_stride), c_ll(kv_stride), c_int(1 if write_kv else 0), ptr(cs), stream())


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """``out[n] = cos | sin`` of ``float(pos[n]) * inv_freq`` (float32 ``[n, head_dim]``): a step's angles, made once."""
    need_cuda(pos, inv_freq, out)
    need_int32("pos", pos)
    need_contiguous("out", out)
    if inv_freq.dtype != torch.float32 or out.dtype != torch.float32 or out.shape != (pos.numel(), 2 * inv_freq.numel()):
        raise KernelError(f"rope_table: pos {tuple(pos.shape)}, inv_freq {tuple(inv_freq.shape)}, out {tuple(out.shape)} do not agree")
    _elementwise.call("zi_rope_table", ptr(pos), ptr(inv_freq), ptr(out), c_int(pos.numel()), c_int(2 * inv_freq.numel()), stream())


def can_fuse_rope_product(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cache: Optional[torch.Tensor]) -> bool:
    """The q/k/v product of a decode step can take rotation and cache append into its epilogue."""
    return (_small_m_ok(x, w, fused="rope") and (bias is None or (bias.dtype == torch.bfloat16 and bias.data_ptr() % 16 == 0))
            and cache is not None and cache.dtype == torch.bfloat16)


def gemm_smallm_rope(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], cs: torch.Tensor, q_out: torch.Tensor,
                     cache: torch.Tensor, tables: torch.Tensor, tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int,
                     n_kv_heads: int, head_dim: int, page_size: int, page_stride: int, kv_stride: int) -> None:
    """``x @ w.T + bias`` for the stacked q/k/v weight of at most 16 tokens, rotated by position (``cs`` from
    :func:`rope_table`), q written to ``q_out`` and k, v appended to the cache pages of each token's request."""
    need_cuda(x, w, bias, cs, q_out, cache, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q_out", q_out), need_contiguous("cs", cs)
    m, k = x.shape
    if w.shape != ((n_heads + 2 * n_kv_heads) * head_dim, k) or q_out.numel() != m * n_heads * head_dim or cs.shape != (m, head_dim):
        raise KernelError(f"gemm_smallm_rope: x {tuple(x.shape)}, w {tuple(w.shape)}, q_out {tuple(q_out.shape)}, cs {tuple(cs.shape)} do not agree")
    if not can_fuse_rope_product(x, w, bias, cache) or q_out.dtype != torch.bfloat16 or cs.dtype != torch.float32:
        raise KernelError("gemm_smallm_rope: bfloat16 operands, at most 16 rows, K a multiple of 32, float32 angles")
    _gemm_smallm.call("zi_gemm_smallm_rope", ptr(x), ptr(w), ptr(bias), ptr(cs), ptr(q_out), ptr(cache), ptr(tables), ptr(tok_seg),
                      ptr(pos), c_int(m), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)), c_int(n_heads), c_int(n_kv_heads),
                      c_int(head_dim), c_int(page_size), c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(gate_up, out)
    need_contiguous("gate_up", gate_up), need_contiguous("out", out)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2) or out.dtype != gate_up.dtype:
        raise KernelError(f"silu_mul: gate_up {tuple(gate_up.shape)} vs out {tuple(out.shape)}")
    _elementwise.call("zi_silu_mul", ptr(gate_up), ptr(out), c_int(dtype_code(out.dtype)), c_int(rows),
                      c_int(two_i // 2), stream())


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> None:
    """``out = a + b`` elementwise (float32 or bfloat16 each), added in float32 with one rounding."""
    need_cuda(a, b, out)
    need_contiguous("a", a), need_contiguous("b", b), need_contiguous("out", out)
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError(f"add: shapes {tuple(a.shape)}, {tuple(b.shape)}, {tuple(out.shape)} differ")
    _elementwise.call("zi_add", ptr(a), c_int(dtype_code(a.dtype)), ptr(b), c_int(dtype_code(b.dtype)), ptr(out),
                      c_int(dtype_code(out.dtype)), c_ll(a.numel()), stream())


def cast(x: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(x, out)
    need_contiguous("x", x), need_contiguous("out", out)
    if x.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _elementwise.call("zi_cast", ptr(x), c_int(dtype_code(x.dtype)), ptr(out), c_int(dtype_code(out.dtype)),
                      c_ll(x.numel()), stream())


def gemm_nt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = a @ w.T + bias`` on the SIMT cores: float32 FMA chains in rising k, any operand types."""
    need_cuda(a, w, bias, out)
    if a.dim() != 2 or w.dim() != 2 or out.dim() != 2:
        raise KernelError("gemm_nt: operands must be matrices")
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or (bias is not None and bias.numel() != n):
        raise KernelError(f"gemm_nt: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if a.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemm_nt: rows must be contiguous")
    _gemm_simt.call("zi_gemm_nt", ptr(a), c_int(dtype_code(a.dtype)), ptr(w), c_int(dtype_code(w.dtype)), ptr(bias),
                    c_int(dtype_code(bias.dtype) if bias is not None else F32), ptr(out),
                    c_int(dtype_code(out.dtype)), c_int(m), c_int(n), c_int(k), c_ll(a.stride(0)), c_ll(w.stride(0)),
                    c_ll(out.stride(0)), stream())


# 9 to 16 rows on the weight-streaming kernel (two tiles of eight rows).  It reads the activations once per tile
# and runs three blocks to an SM instead of four, and timed back to back in a graph against the library (plus the
# kernel its epilogue would save) it wins only in these cases (us at 9 to 16 rows, streaming kernel / library):
#   K cut at least three ways, up to 16 M elements      1.5B-class down 9.5-10.2 / 13.6  (7B-class output, cut in two: 13.7 / 8.2;
#                                                       7B-class down 45 / 30; 1.5B-class output, not cut: 5.4 / 4.7)
#   q/k/v with rotation and append, up to 8 M elements  1.5B-class 5.6 / 5.0 + the rotation kernel  (7B-class 15.0 / 8.7 + it)
#   gate/up with the activation: never                  1.5B-class 17.6-18.6 / 13.5 with the activation kernel, 7B-class 58 / 49
SMALL_M_WIDE_ELEMENTS = 16 << 20
SMALL_M_WIDE_ROPE_ELEMENTS = 8 << 20
SMALL_M_WIDE_MIN_KSPLIT = 3
_ksplit_cache: Dict = {}


def _ksplit(n: int, k: int) -> int:
    key = (n, k)
    if key not in _ksplit_cache:
        _ksplit_cache[key] = int(_gemm_smallm.lib.zi_gemm_smallm_ksplit(c_int(n), c_int(k), c_int(0)))
    return _ksplit_cache[key]


def _small_m_ok(x: torch.Tensor, w: torch.Tensor, fused: Optional[str] = None) -> bool:
    """The weight-streaming kernel takes this product.  Up to 8 rows it is the fastest form measured for every
    shape tried (1.5B- to 32B-class layers, at or above the library's rate).  With 9 to 16 rows it keeps what the
    table above says; ``fused``: ``"rope"`` (rotation and cache append in its epilogue), ``"silu"`` (activation)."""
    if x.shape[0] > 8:
        elements = w.shape[0] * w.shape[1]
        if fused == "silu":
            return False
        if fused == "rope":
            if elements > SMALL_M_WIDE_ROPE_ELEMENTS:
                return False
        elif elements > SMALL_M_WIDE_ELEMENTS or x.shape[1] % 32 != 0 or _ksplit(w.shape[0], w.shape[1]) < SMALL_M_WIDE_MIN_KSPLIT:
            return False
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] <= SMALL_M_ROWS
            and x.shape[1] % 32 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_smallm(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                silu_mul: bool = False) -> None:
    """``out = x @ w.T + bias`` for at most 16 rows of ``x``: weights stream once from memory into the
    tensor cores.  ``silu_mul``: ``w`` is ``[2*I, K]`` (gate rows, then up rows) and ``out[m, j] =
    up * gate / (1 + exp(-gate))``."""
    need_cuda(x, w, bias, out)
    m, k = x.shape
    n = w.shape[0] // 2 if silu_mul else w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_smallm: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_smallm: bfloat16 operands only")
    part, counters = _smallm_scratch(x.device, n, k, silu_mul)
    _gemm_smallm.call("zi_gemm_smallm", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)), ptr(part),
                      ptr(counters), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                      c_ll(out.stride(0)), c_int(1 if silu_mul else 0), stream())


_scratch = {}


def _smallm_scratch(device, n: int, k: int, silu_mul: bool):
    """Scratch of the split-K decode product: partial sums and arrival counters.  Allocated once per device and
    grown on demand; the counters start at zero and every launch leaves them at zero.  One stream at a time."""
    lib = _gemm_smallm.lib
    lib.zi_gemm_smallm_part_floats.restype = c_ll
    need = lib.zi_gemm_smallm_part_floats(c_int(n), c_int(k), c_int(1 if silu_mul else 0))
    if need == 0:
        return None, None
    key = ("smallm", device)
    if key not in _scratch:
        # K is only split while there are fewer than 296 column tiles (N < 4736), at most 8 ways, 16 rows
        _scratch[key] = (torch.empty(8 * 16 * 4736, dtype=torch.float32, device=device),
                         torch.zeros(512, dtype=torch.int32, device=device))
    part, counters = _scratch[key]
    if part.numel() < need:
        raise KernelError(f"gemm_smallm: scratch of {part.numel()} floats is too small for N={n}, K={k}")
    return part, counters


_retired: list = []


def _grown_scratch(key, floats: int, device) -> torch.Tensor:
    """A float32 scratch buffer of at least ``floats`` entries for ``key``, grown on demand.  A CUDA graph captured
    earlier has the old buffer's address baked in and goes on writing there when it is replayed, so a buffer that is
    outgrown is never given back to the allocator: it is kept (``_retired``) for the life of the process.  Growth
    at least doubles the size, so all retired buffers together stay smaller than the live one."""
    cur = _scratch.get(key)
    if cur is None or cur.numel() < floats:
        if cur is not None:
            _retired.append(cur)
            floats = max(floats, 2 * cur.numel())
        cur = _scratch[key] = torch.empty(floats, dtype=torch.float32, device=device)
    return cur


def _tc_status(device) -> torch.Tensor:
    key = ("tc_status", device)
    if key not in _scratch:
        _scratch[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _scratch[key]


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                 swapped: Optional[bool] = None) -> None:
    """``out = x @ w.T + bias`` on the tcgen05 tensor cores (TMA-fed, accumulator in TMEM), bfloat16 operands.

    ``swapped`` puts the weights on the 128-row side of the MMA and up to 256 rows of ``x`` on the narrow side
    (decode); by default it is chosen by the number of rows.  A bounded wait that runs out inside the kernel is
    reported by :func:`tcgen05_status`.
    """
    need_cuda(x, w, bias, out)
    m, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape != (m, n) or out.stride(1) != 1 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tcgen05: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_tcgen05: bfloat16 operands only")
    if swapped is None:
        swapped = m <= 64
    _gemm_tcgen05.call("zi_gemm_tcgen05", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                       ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                       c_ll(out.stride(0)), c_int(1 if swapped else 0), stream())


_sm_count: Dict = {}


def _num_sms(device) -> int:
    if device not in _sm_count:
        _sm_count[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_count[device]


def gemm_tcgen05_tiles(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor,
                       silu_mul: bool = False, tile_width: int = 0, pairs: Optional[bool] = None) -> None:
    """``out = x @ w.T + bias`` for many rows: one persistent CTA per SM walks 128-row tiles, the accumulator
    double-buffered in TMEM so that the epilogue of a tile overlaps the products of the next.

    With ``silu_mul`` the weight is ``[gate; up]`` stacked (``[2 * n, k]``) and ``out[m, n] = silu(x.gate^T) *
    (x.up^T)``; neither half is written to memory.  ``tile_width`` (accumulator columns per tile) is chosen by
    the call when 0.  ``pairs``: two SMs share a 256-row tile and each loads only half of its weight rows
    (``cta_group::2``); the default for more than 128 rows.
    """
    need_cuda(x, w, bias, out)
    m, k = x.shape
    n = out.shape[1]
    if w.shape != ((2 * n if silu_mul else n), k) or out.shape[0] != m or out.stride(1) != 1 or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError(f"gemm_tcgen05_tiles: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)} do not agree")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or (bias is not None and bias.dtype != torch.bfloat16):
        raise KernelError("gemm_tcgen05_tiles: bfloat16 operands only")
    if pairs is None:
        pairs = m > 128
    if pairs:
        _gemm_tcgen05.call("zi_gemm_tcgen05_pairs", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                           ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                           c_ll(out.stride(0)), c_int(1 if silu_mul else 0), c_int(tile_width), stream())
        return
    _gemm_tcgen05.call("zi_gemm_tcgen05_tiles", ptr(x), ptr(w), ptr(bias), ptr(out), c_int(dtype_code(out.dtype)),
                       ptr(_tc_status(x.device)), c_int(m), c_int(n), c_int(k), c_ll(x.stride(0)), c_ll(w.stride(0)),
                       c_ll(out.stride(0)), c_int(1 if silu_mul else 0), c_int(tile_width), c_int(_num_sms(x.device)), stream())


def status_word(device) -> torch.Tensor:
    """The device word (int32 ``[1]``) in which the kernels with bounded waits report one that ran out; 0 = fine."""
    return _tc_status(torch.device(device))


def tcgen05_status(device) -> int:
    """0, or the code of the role whose bounded wait ran out (1 producer, 2 MMA issuer, 3 epilogue); resets it."""
    st = _tc_status(torch.device(device))
    v = int(st.item())
    if v:
        st.zero_()
    return v


TC_PLAIN_PRODUCTS = False        # plain bfloat16 products of many rows on the tcgen05 kernel instead of the library
TC_MIN_ROWS = 1024               # ... from this many rows, where switched on
TC_FUSED_MIN_ROWS = 128          # ... and a gate/up product with the activation in its epilogue
TC_FUSED_MIN_ROWS_LARGE = 32     # ... already from this many rows where the stacked weight has at least
TC_FUSED_LARGE_ELEMENTS = 96 << 20   # ... this many elements (7B-class layers and up: see linear_silu_mul)
_tc_launched: Dict = {}


def _tc_ok(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16)
            and out.dtype in (torch.bfloat16, torch.float32) and x.shape[1] % 8 == 0
            and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1 and x.stride(0) % 8 == 0
            and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def raise_if_tcgen05_failed(device) -> None:
    """After a step that launched tcgen05 products: synchronise and fail loudly if a bounded wait ran out."""
    device = torch.device(device)
    if _tc_launched.pop(device, False):
        code = tcgen05_status(device)
        if code:
            raise KernelError(f"gemm_tcgen05: a bounded wait ran out inside the kernel (role {code}); the step's output is not valid")


def linear_silu_mul(x: torch.Tensor, w_gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = silu(x @ gate.T + b_gate) * (x @ up.T + b_up)`` with ``w_gate_up = [gate; up]`` stacked.

    bfloat16 without bias: the activation runs in the product's epilogue (weight-streaming kernel up to 16 rows,
    tcgen05 kernel from ``TC_FUSED_MIN_ROWS``), so neither half reaches memory.  Otherwise: product, then the
    elementwise kernel.  Between 17 and 127 rows both ways are bound by streaming the weight; timed back to back in a
    graph the tcgen05 kernel is ahead from 32 rows on 7B-class layers (hidden 3,584, intermediate 18,944: 47.4
    against 51.8 us at 64 rows, 48.2 against 56.3 at 127) and level or behind on 1.5B-class layers (15.3 against 14.8
    us at 64 rows), so it takes those rows only for stacked weights of ``TC_FUSED_LARGE_ELEMENTS`` elements or more.
    """
    need_cuda(x, w_gate_up, bias, out)
    if bias is None and _small_m_ok(x, w_gate_up, fused="silu"):
        gemm_smallm(x, w_gate_up, None, out, silu_mul=True)
        return
    min_rows = TC_FUSED_MIN_ROWS_LARGE if w_gate_up.shape[0] * w_gate_up.shape[1] >= TC_FUSED_LARGE_ELEMENTS else TC_FUSED_MIN_ROWS
    if bias is None and x.shape[0] >= min_rows and out.dtype == torch.bfloat16 and _tc_ok(x, w_gate_up, None, out):
        gemm_tcgen05_tiles(x, w_gate_up, None, out, silu_mul=True)
        _tc_launched[x.device] = True
        return
    gate_up = torch.empty((x.shape[0], w_gate_up.shape[0]), dtype=out.dtype, device=x.device)
    linear(x, w_gate_up, bias, gate_up)
    silu_mul(gate_up, out)


# A product whose result goes straight into the residual stream (output and down projections), with 17 to 256 rows:
# the library's kernels for these few rows leave most of the GPU idle when the output is narrow (1.5B-class down
# product, 64 rows: 13.8 us = 2.0 TB/s).  As a batched product over RESIDUAL_K_PARTS ranges of K with float32 results
# it takes 7.8 us (7B-class: 30.8 -> 25.2 us; 0.5B-class sizes 8.9 -> 5.2; the 1.5B-class output projection 4.9 ->
# 3.8), and the norm that folds the branch into
# the stream adds the ranges on its way (add_rmsnorm), so no kernel is added.  Measured back to back in a graph;
# from 257 rows the library's own choice is as good, and at 32B-class sizes (141 M elements) nothing is gained.
RESIDUAL_K_PARTS = 4
RESIDUAL_PARTS_MIN_ROWS = 17
RESIDUAL_PARTS_MIN_K = 1024
# (most rows, most weight elements) for products with K >= 2 N (down: 1.5B-class 14.4 -> 9.7 us still at 256 rows,
# 7B-class 39.6 -> 35.6) and for the others (output projection: 7B-class 8.5 -> 8.0 us at 128 rows, but 8.8 -> 10.1 at
# 192; 32B-class, 26 M elements, 12.2 -> 13.9 at 128)
RESIDUAL_PARTS_LONG_K = (256, 80 << 20)
RESIDUAL_PARTS_SQUARE = (128, 16 << 20)


def linear_for_residual(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``x @ w.T + bias`` for a result that the next norm adds to the residual stream: either the product itself
    (``[rows, N]`` of x's type) or, where that is faster, float32 partial sums ``[parts, rows, N]`` over ranges of
    K, which :func:`add_rmsnorm` adds in order and rounds as the product would have been rounded."""
    rows, k = x.shape
    n = w.shape[0]
    max_rows, max_elements = RESIDUAL_PARTS_LONG_K if k >= 2 * n else RESIDUAL_PARTS_SQUARE
    if (bias is None and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and RESIDUAL_PARTS_MIN_ROWS <= rows <= max_rows and k >= RESIDUAL_PARTS_MIN_K
            and n * k <= max_elements and k % (8 * RESIDUAL_K_PARTS) == 0 and n % 8 == 0
            and x.is_contiguous() and w.is_contiguous()):
        need_cuda(x, w)
        p = RESIDUAL_K_PARTS
        parts = torch.empty((p, rows, n), dtype=torch.float32, device=x.device)
        torch.bmm(x.view(rows, p, k // p).permute(1, 0, 2), w.view(n, p, k // p).permute(1, 2, 0),
                  out_dtype=torch.float32, out=parts)
        return parts
    out = torch.empty((rows, n), dtype=x.dtype, device=x.device)
    linear(x, w, bias, out)
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor) -> None:
    """``out = x @ w.T + bias``; picks the kernel by operand types and the number of rows.

    * any float32 operand: the SIMT kernel (true 32-bit arithmetic);
    * bfloat16 x bfloat16 with at most 16 rows (decode steps): the weight-streaming tensor-core kernel;
    * bfloat16 x bfloat16 otherwise: cuBLAS with float32 accumulation, the library product the
      reference's engine uses as well; the output may be bfloat16 or float32.  With ``TC_PLAIN_PRODUCTS`` set,
      products of ``TC_MIN_ROWS`` rows or more run on the tcgen05 kernel (pairs of SMs) instead.  Timed back to
      back in a graph the library is ahead on plain products (2,048 rows of the 1.5B-class layer: q/k/v 12.0
      against 14.5 us, output 9.6 against 13.7, down 42.1 against 46.5; the whole 2,048-token step 5.39 against
      5.75 ms), so the tcgen05 kernel is kept for the gate/up product, where its SiLU-mul epilogue saves a kernel
      and a round trip of the activations through memory (:func:`linear_silu_mul`).
    """
    need_cuda(x, w, bias, out)
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and (bias is None or bias.dtype == torch.bfloat16):
        if _small_m_ok(x, w) and out.stride(1) == 1:
            gemm_smallm(x, w, bias, out)
            return
        if TC_PLAIN_PRODUCTS and x.shape[0] >= TC_MIN_ROWS and _tc_ok(x, w, bias, out):
            gemm_tcgen05_tiles(x, w, bias, out)
            _tc_launched[x.device] = True
            return
        if out.dtype == torch.bfloat16:
            if bias is not None:
                torch.addmm(bias, x, w.t(), out=out)
            else:
                torch.mm(x, w.t(), out=out)
        else:
            res = torch.mm(x, w.t(), out_dtype=torch.float32)
            if bias is not None:
                res += bias.float()
            out.copy_(res)
        return
    gemm_nt(x, w, bias, out)


def paged_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                    tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                    page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float) -> None:
    """Causal attention of each token over its request's cache pages (general kernel)."""
    need_cuda(q, cache, out, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out)
    if q.dtype != cache.dtype or out.dtype != q.dtype:
        raise KernelError("paged_attention: q, cache and out must share one dtype")
    n = q.shape[0]
    _attention_generic.call("zi_paged_attention", ptr(q), ptr(cache), ptr(out), c_int(dtype_code(q.dtype)),
                            ptr(tables), ptr(tok_seg), ptr(pos), c_int(n), c_int(n_heads), c_int(n_kv_heads),
                            c_int(head_dim), c_int(page_size), c_int(tables.shape[1]), c_ll(page_stride),
                            c_ll(kv_stride), c_int(window or 0), c_float(scale), stream())


PREFILL_TILE_ROWS = 128          # query rows per entry of a step's tile list


def decode_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                     tok_seg: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float) -> None:
    """One query token per request, bfloat16, tensor cores; a cluster of eight thread blocks per
    (request, key/value head) shares the context and merges through distributed shared memory."""
    need_cuda(q, cache, out, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("tok_seg", tok_seg), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out)
    n = q.shape[0]
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention: bfloat16 only")
    _attention_mma.call("zi_decode_attention", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tok_seg), ptr(pos),
                        c_int(n), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
                        c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0),
                        c_float(scale), stream())


def decode_attention_split_from() -> int:
    """The number of cached tokens from which :func:`decode_attention_tma` lets several clusters share one request's
    keys and launches the kernel that adds their parts: a step whose ``max_kv_len`` stays below it has neither."""
    return int(_attention_mma.lib.zi_decode_attention_tma_split_from())


def decode_attention_tma(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                         tok_seg: Optional[torch.Tensor], pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                         page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float,
                         max_kv_len: int = 0) -> None:
    """One query token per request, bfloat16: the cluster kernel with 32-key tiles dealt to single warps, each
    fed by TMA through the block table into a ring of its own.  Same arguments as :func:`decode_attention`;
    head_dim 64 or 128, pages of a power of two from 8 to 128 tokens.  ``max_kv_len``: an upper bound of the cached
    tokens of the step's requests; ``tok_seg`` None: token n belongs to row n of ``tables`` (every decode step of the
    engine; the kernel then asks for its first page numbers without waiting for anything).  With few requests and long contexts several clusters then share one request's
    keys and a second kernel adds their parts (0: never).  A bounded wait that runs out is reported by
    :func:`tcgen05_status`."""
    need_cuda(q, cache, out, tables, tok_seg, pos)
    need_int32("tables", tables), need_int32("pos", pos)
    if tok_seg is not None:
        need_int32("tok_seg", tok_seg)
    need_contiguous("q", q), need_contiguous("out", out)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("decode_attention_tma: bfloat16 only")
    part, part_floats = None, 0
    if max_kv_len > 0:
        lib = _attention_mma.lib
        lib.zi_decode_attention_tma_part_floats.restype = c_ll
        part_floats = int(lib.zi_decode_attention_tma_part_floats(c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads),
                                                                   c_int(head_dim), c_int(int(max_kv_len))))
        if part_floats:
            part = _grown_scratch(("decode_parts", q.device), part_floats, q.device)
    _attention_mma.call("zi_decode_attention_tma", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tok_seg), ptr(pos),
                        ptr(_tc_status(q.device)), c_int(q.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim),
                        c_int(page_size), c_int(tables.shape[1]), c_ll(cache.shape[0]), c_ll(page_stride), c_ll(kv_stride),
                        c_int(window or 0), c_float(scale), c_int(int(max_kv_len) if part_floats else 0), ptr(part),
                        c_ll(part_floats), stream())
    _tc_launched[q.device] = True


def prefill_attention(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                      tiles: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                      page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float) -> None:
    """Portions of prompts, bfloat16, ``mma.sync`` tensor-core path.  ``tiles`` int32 ``[n_tiles, 3]``: (first token,
    rows <= 128, segment); the positions of a tile's tokens are consecutive.  Takes any page size and windows."""
    need_cuda(q, cache, out, tables, tiles, pos)
    need_int32("tables", tables), need_int32("tiles", tiles), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out), need_contiguous("tiles", tiles)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("prefill_attention: bfloat16 only")
    _attention_mma.call("zi_prefill_attention", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tiles), ptr(pos),
                        c_int(tiles.shape[0]), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
                        c_int(tables.shape[1]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0),
                        c_float(scale), stream())


def prefill_attention_tcgen05(q: torch.Tensor, cache: torch.Tensor, out: torch.Tensor, tables: torch.Tensor,
                              tiles: torch.Tensor, pos: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                              page_size: int, page_stride: int, kv_stride: int, window: Optional[int], scale: float) -> None:
    """Portions of prompts, bfloat16, on tcgen05: scores and outputs accumulate in TMEM, K and V pages arrive by
    TMA through the block table.  Same arguments as :func:`prefill_attention`; head_dim 64 or 128, pages of a power
    of two from 8 to 128 tokens.  A bounded wait that runs out is reported by :func:`tcgen05_status`."""
    need_cuda(q, cache, out, tables, tiles, pos)
    need_int32("tables", tables), need_int32("tiles", tiles), need_int32("pos", pos)
    need_contiguous("q", q), need_contiguous("out", out), need_contiguous("tiles", tiles)
    if q.dtype != torch.bfloat16 or cache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("prefill_attention_tcgen05: bfloat16 only")
    _attention_tcgen05.call("zi_prefill_attention_tcgen05", ptr(q), ptr(cache), ptr(out), ptr(tables), ptr(tiles), ptr(pos),
                            ptr(_tc_status(q.device)), c_int(q.shape[0]), c_int(tiles.shape[0]), c_int(n_heads),
                            c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(tables.shape[1]),
                            c_ll(cache.shape[0]), c_ll(page_stride), c_ll(kv_stride), c_int(window or 0), c_float(scale), stream())
    _tc_launched[q.device] = True


def tcgen05_attention_ok(head_dim: int, page_size: int) -> bool:
    return head_dim in (64, 128) and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0


def attention(q: torch.Tensor, cache, out: torch.Tensor, ctx, n_heads: int, n_kv_heads: int, head_dim: int,
              window: Optional[int], scale: float) -> None:
    """Attention of a step's tokens over the cache (``cache`` is a CallCacheView, ``ctx`` a StepContext).

    Picks a kernel by dtype and by the shape of the step; all of them compute the same function.
    bfloat16 with head_dim 64 or 128 runs on the tensor cores: decode-only steps, and the single tokens at the head
    of a mixed step, on the cluster decode kernel, anything else on the tcgen05 prefill kernel (pages of 8..128 tokens) or the ``mma.sync`` prefill kernel (other
    page sizes); float32 and other head sizes on the general kernel.
    """
    tables = ctx.tables[cache.group]
    if q.dtype == torch.bfloat16 and head_dim in (64, 128):
        n = q.shape[0]
        if ctx.decode_only and tcgen05_attention_ok(head_dim, cache.page_size):
            # in a step of single tokens, token n is segment n
            decode_attention_tma(q, cache.tensor, out, tables, None, ctx.positions, n_heads, n_kv_heads, head_dim,
                                 cache.page_size, cache.page_stride, cache.kv_stride, window, scale,
                                 max_kv_len=min(ctx.max_kv_len, window) if window else ctx.max_kv_len)
            return
        if ctx.decode_only:
            decode_attention(q, cache.tensor, out, tables, ctx.tok_seg, ctx.positions, n_heads, n_kv_heads, head_dim,
                             cache.page_size, cache.page_stride, cache.kv_stride, window, scale)
            return
        tiles = ctx.extras.get("attn_tiles")
        lead = ctx.extras.get("leading_singles", 0) if tiles is not None else 0
        if lead:                                  # decoding requests beside a prompt portion: their own kernel
            if tcgen05_attention_ok(head_dim, cache.page_size):     # the leading single tokens are segments 0 .. lead - 1
                decode_attention_tma(q[:lead], cache.tensor, out[:lead], tables, None, ctx.positions[:lead], n_heads,
                                     n_kv_heads, head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale)
            else:
                decode_attention(q[:lead], cache.tensor, out[:lead], tables, ctx.tok_seg[:lead], ctx.positions[:lead], n_heads,
                                 n_kv_heads, head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale)
        if tiles is not None and tcgen05_attention_ok(head_dim, cache.page_size):
            prefill_attention_tcgen05(q, cache.tensor, out, tables, tiles, ctx.positions, n_heads, n_kv_heads, head_dim,
                                      cache.page_size, cache.page_stride, cache.kv_stride, window, scale)
            return
        if tiles is not None:
            prefill_attention(q, cache.tensor, out, tables, tiles, ctx.positions, n_heads, n_kv_heads, head_dim,
                              cache.page_size, cache.page_stride, cache.kv_stride, window, scale)
            return
    paged_attention(q, cache.tensor, out, tables, ctx.tok_seg, ctx.positions, n_heads, n_kv_heads,
                    head_dim, cache.page_size, cache.page_stride, cache.kv_stride, window, scale)


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    need_cuda(logits, out)
    need_int32("out", out)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 [rows, vocab] with contiguous rows")
    rows, vocab = logits.shape
    slices = int(_sampling.lib.zi_argmax_slices(c_int(vocab)))
    part = _grown_scratch(("argmax", logits.device), rows * slices * 2, logits.device) if slices > 1 else None
    _sampling.call("zi_argmax", ptr(logits), ptr(out), c_int(rows), c_int(vocab), c_ll(logits.stride(0)), ptr(part), stream())


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor) -> None:
    """One token per row; rows with ``temperature <= 0`` are greedy."""
    need_cuda(logits, out, temperature, top_k, top_p, uniform)
    need_int32("out", out), need_int32("top_k", top_k)
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 [rows, vocab] with contiguous rows")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("uniform", uniform)):
        if t.dtype != torch.float32 or t.numel() != rows:
            raise KernelError(f"sample: {name} must be float32 with one entry per row")
    if top_k.numel() != rows or out.numel() != rows:
        raise KernelError("sample: top_k and out need one entry per row")
    _sampling.call("zi_sample", ptr(logits), ptr(out), ptr(temperature), ptr(top_k), ptr(top_p), ptr(uniform),
                   c_int(rows), c_int(logits.shape[1]), c_ll(logits.stride(0)), stream())


def penalty_rows(logits: torch.Tensor, counts: torch.Tensor, slots: torch.Tensor, penalty: torch.Tensor) -> None:
    """The repetition penalty from a table on the device: row r of ``logits`` (float32 ``[rows, vocab]``) is penalised
    with ``penalty[r]`` once per time that the request in slot ``slots[r]`` has generated a token
    (``counts`` int32 ``[slots, vocab]``); rows with a negative slot or a penalty of 1 are left alone."""
    need_cuda(logits, counts, slots, penalty)
    need_int32("counts", counts), need_int32("slots", slots)
    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("penalty_rows: logits must be float32 [rows, vocab] with contiguous rows")
    if counts.dim() != 2 or counts.shape[1] != logits.shape[1] or counts.stride(1) != 1:
        raise KernelError(f"penalty_rows: counts {tuple(counts.shape)} do not match a vocabulary of {logits.shape[1]}")
    if penalty.dtype != torch.float32 or penalty.numel() != rows or slots.numel() != rows:
        raise KernelError("penalty_rows: slots (int32) and penalty (float32) need one entry per row")
    _sampling.call("zi_penalty_rows", ptr(logits), ptr(counts), ptr(slots), ptr(penalty), c_int(rows), c_int(logits.shape[1]),
                   c_ll(logits.stride(0)), c_ll(counts.stride(0)), stream())


def count_tokens(counts: torch.Tensor, slots: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts[slots[r], tokens[r]] += 1`` for the rows whose slot is not negative (each slot at most once)."""
    need_cuda(counts, slots, tokens)
    need_int32("counts", counts), need_int32("slots", slots), need_int32("tokens", tokens)
    if counts.dim() != 2 or counts.stride(1) != 1 or slots.numel() != tokens.numel():
        raise KernelError("count_tokens: counts [slots, vocab], one slot and one token per row")
    _sampling.call("zi_count_tokens", ptr(counts), ptr(slots), ptr(tokens), c_int(tokens.numel()), c_int(counts.shape[1]),
                   c_ll(counts.stride(0)), stream())


def count_token_list(counts_row: torch.Tensor, tokens: torch.Tensor) -> None:
    """``counts_row[t] += 1`` for every listed token (a token listed twice counts twice)."""
    need_cuda(counts_row, tokens)
    need_int32("counts_row", counts_row), need_int32("tokens", tokens)
    need_contiguous("counts_row", counts_row)
    _sampling.call("zi_count_token_list", ptr(counts_row), ptr(tokens), c_int(tokens.numel()), c_int(counts_row.numel()), stream())


def advance_decode(ids: torch.Tensor, pos: torch.Tensor, sampled: torch.Tensor, rows: Optional[int] = None) -> None:
    """Hand the chosen tokens to the next decode step: ``ids := sampled``, ``pos += 1`` for the first ``rows`` rows
    (all of ``ids`` by default).  ``pos`` is one position per token, or ``[axes, tokens]`` for a model whose tokens
    carry several position numbers: every axis moves on by one."""
    need_cuda(ids, pos, sampled)
    need_int32("ids", ids), need_int32("pos", pos), need_int32("sampled", sampled)
    n = ids.numel() if rows is None else int(rows)
    axes, per_axis = (pos.shape[0], pos.shape[1]) if pos.dim() == 2 else (1, pos.numel())
    if pos.dim() == 2 and (pos.stride(1) != 1 or (axes > 1 and pos.stride(0) < per_axis)):
        raise KernelError(f"advance_decode: positions {tuple(pos.shape)} with strides {pos.stride()}")
    if n > min(ids.numel(), per_axis, sampled.numel()):
        raise KernelError(f"advance_decode: {n} rows of ids {ids.numel()}, pos {per_axis}, sampled {sampled.numel()}")
    _sampling.call("zi_advance_decode", ptr(ids), ptr(pos), ptr(sampled), c_int(n), c_int(axes),
                   c_ll(pos.stride(0) if pos.dim() == 2 else 0), stream())


def repetition_penalty(logits_row: torch.Tensor, tokens: torch.Tensor, penalty: float) -> None:
    need_cuda(logits_row, tokens)
    need_int32("tokens", tokens)
    if logits_row.dtype != torch.float32 or logits_row.dim() != 1 or not logits_row.is_contiguous():
        raise KernelError("repetition_penalty: one contiguous float32 row")
    _sampling.call("zi_repetition_penalty", ptr(logits_row), ptr(tokens), c_int(tokens.numel()),
                   c_int(logits_row.numel()), c_float(penalty), stream())
