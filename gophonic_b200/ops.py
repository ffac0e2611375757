"""Python face of the sm_100a kernel library.

Each function checks its tensors (device, dtype, layout, sizes), passes raw pointers and the
current torch CUDA stream to the C entry point, and raises ``KernelError`` with the library's own
message if the kernel refuses the call.  Nothing here computes: there is no CPU path and no
torch fallback.  Importing this module builds the library if needed and fails if that fails.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, byref, c_float, c_int, c_int64, c_uint64, c_void_p
from typing import Optional

import torch

from .csrc import build as _build

PAGE = 64  # tokens per cache page; the kernels' GB_PAGE

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


_lib = _build.load()


def library_file() -> str:
    return _lib._name


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {dtype}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_device_index = []


def use_device(index: int) -> None:
    """Make CUDA device ``index`` the current one and the one whose stream the kernels are launched
    on.  The library serves one GPU at a time; a model opened on another device moves it there."""
    torch.cuda.set_device(index)
    _device_index[:] = [index]


def _stream() -> c_void_p:
    """torch's current CUDA stream of the library's device, as a raw handle (asked anew at every
    call: a graph capture runs on a stream of its own)."""
    if _raw_stream is not None:
        if not _device_index:
            _device_index.append(torch.cuda.current_device())
        return c_void_p(_raw_stream(_device_index[0]))
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


launches = 0  # kernels launched through this module since import (a call that launches two counts two)


def _check(rc: int, kernels: int = 1) -> None:
    global launches
    if rc != 0:
        raise KernelError(_lib.gb_last_error().decode("utf-8", "replace"))
    launches += kernels


def _need(t: torch.Tensor, name: str, dtype=None, dim=None, contiguous=True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name}: tensor is on {t.device}; kernels run on CUDA tensors only")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: dtype {t.dtype}, want {dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{name}: {t.dim()} dimensions, want {dim}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name}: tensor is not contiguous")


# ---- embedding ---------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, stats: Optional[torch.Tensor] = None,
                 next_weight: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None) -> None:
    """out[r, :] = float32(table[ids[r], :]).  With ``stats`` (float32 [>= rows, capacity]) the sum of
    squares of row r is left in stats[r, 0]: one partial sum a row.  With ``next_weight`` (float32
    [hidden]) and ``next_x`` (bfloat16 [rows, hidden]) also next_x = bf16(out * next_weight): the
    output of an RMSNorm with that weight but for each row's factor."""
    _need(table, "embed table", dim=2)
    _need(ids, "ids", torch.int32, 1)
    _need(out, "embed out", torch.float32, 2)
    rows, hidden = out.shape
    if ids.numel() != rows or table.shape[1] != hidden:
        raise KernelError(f"embed_gather: {ids.numel()} ids, table {tuple(table.shape)}, out {tuple(out.shape)}")
    stride = 0
    if stats is not None:
        _need(stats, "row statistics", torch.float32, 2)
        if stats.shape[0] < rows:
            raise KernelError(f"embed_gather: statistics for {stats.shape[0]} rows, {rows} rows")
        stride = stats.stride(0)
    ldxn = _check_next(next_weight, next_x, rows, hidden, "embed_gather")
    _check(_lib.gb_embed_gather(_ptr(table), _code(table.dtype), _ptr(ids), c_int(rows), c_int(hidden),
                                c_int(table.shape[0]), _ptr(out), _ptr(stats), c_int64(stride), _ptr(next_weight), _ptr(next_x),
                                c_int64(ldxn), _stream()))


def _check_next(next_weight, next_x, rows: int, width: int, who: str) -> int:
    if next_weight is None:
        return 0
    _need(next_weight, "next norm weight", torch.float32, 1)
    if next_x is None:
        raise KernelError(f"{who}: a norm weight is given without a tensor for the rows it scales")
    _need(next_x, "prescaled rows", torch.bfloat16, 2, contiguous=False)
    if next_weight.numel() != width or next_x.shape != (rows, width) or next_x.stride(1) != 1:
        raise KernelError(f"{who}: norm weight of {next_weight.numel()}, prescaled rows {tuple(next_x.shape)} for {rows} x {width}")
    return next_x.stride(0)


# ---- cache pages, seeded fill ------------------------------------------------------------
def block_table_set(table: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """table[slot, logical page] = physical page for the first ``n`` (slot, logical, physical)
    triples of the int32 tensor ``triples``."""
    _need(table, "block table", torch.int32, 2)
    _need(triples, "page triples", torch.int32, 1)
    if triples.numel() < 3 * n:
        raise KernelError(f"block_table_set: {triples.numel()} integers for {n} triples")
    _check(_lib.gb_block_table_set(_ptr(table), c_int(table.stride(0)), c_int(table.shape[0]), _ptr(triples), c_int(n), _stream()))


def zero_pages(planes: torch.Tensor, triples: torch.Tensor, n: int) -> None:
    """Clear, in every plane of ``planes`` [planes, pages, ...], the pages named by the third entry
    of the first ``n`` triples."""
    _need(planes, "cache planes", dim=None)
    _need(triples, "page triples", torch.int32, 1)
    if planes.dim() < 3 or triples.numel() < 3 * n:
        raise KernelError(f"zero_pages: planes {tuple(planes.shape)}, {triples.numel()} integers for {n} triples")
    es = planes.element_size()
    _check(_lib.gb_zero_pages(_ptr(planes), c_int64(planes.stride(0) * es), c_int(planes.shape[0]), c_int64(planes.stride(1) * es),
                              c_int(planes.shape[1]), _ptr(triples), c_int(n), _stream()))


def random_fill(out: torch.Tensor, key: int, c: float, mean: float) -> None:
    """The seeded fill of ``weights.random_init``: out[i] = (sum of eight 16-bit fields of two
    splitmix64 words of (key, i) - 262140) * c + mean, the same bits the numpy writer computes."""
    _need(out, "fill target")
    _check(_lib.gb_random_fill(_ptr(out), _code(out.dtype), c_int64(out.numel()), c_uint64(key & 0xFFFFFFFFFFFFFFFF), c_float(c),
                               c_float(mean), _stream()))


# ---- norm --------------------------------------------------------------------------------
def gather_tokens(ids: torch.Tensor, source: torch.Tensor) -> None:
    """ids[i] = source[ids[i]] in place (both int32 on the device)."""
    _need(ids, "ids", torch.int32, 1)
    _need(source, "token source", torch.int32, 1)
    _check(_lib.gb_gather_tokens(_ptr(ids), _ptr(source), c_int(ids.numel()), c_int(source.numel()), _stream()))


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """h += delta (if given, in place, unless ``rows`` selects); out = rmsnorm(h) * weight."""
    _need(h, "residual", torch.float32, 2)
    _need(weight, "norm weight", torch.float32, 1)
    _need(out, "norm out", dim=2)
    n = h.shape[1]
    if weight.numel() != n or out.shape[1] != n:
        raise KernelError(f"add_rmsnorm: residual width {n}, weight {weight.numel()}, out {tuple(out.shape)}")
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != h.shape:
            raise KernelError(f"add_rmsnorm: delta {tuple(delta.shape)} vs residual {tuple(h.shape)}")
    if rows is not None:
        _need(rows, "row index", torch.int32, 1)
        out_rows = rows.numel()
    else:
        out_rows = h.shape[0]
    if out.shape[0] != out_rows:
        raise KernelError(f"add_rmsnorm: out has {out.shape[0]} rows, want {out_rows}")
    _check(_lib.gb_add_rmsnorm(_ptr(h), _ptr(delta), _ptr(weight), c_float(eps), c_int(n), _ptr(out),
                               _code(out.dtype), _ptr(rows), c_int(out_rows), _stream()))


def add_rows(h: torch.Tensor, delta: torch.Tensor) -> None:
    _need(h, "residual", torch.float32, 2)
    _need(delta, "delta", torch.float32, 2)
    if delta.shape != h.shape:
        raise KernelError(f"add_rows: {tuple(delta.shape)} vs {tuple(h.shape)}")
    _check(_lib.gb_add_rows(_ptr(h), _ptr(delta), c_int(h.shape[0]), c_int(h.shape[1]), _stream()))


# ---- feed-forward activation -------------------------------------------------------------
def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleave8: bool = False) -> None:
    """out[r, i] = silu(gate[r, i]) * up[r, i]; gate and up are the two halves of ``gate_up``'s
    columns, or, with ``interleave8``, alternate in blocks of eight columns."""
    _need(gate_up, "gate_up", dim=2)
    _need(out, "swiglu out", gate_up.dtype, 2)
    rows, two_i = gate_up.shape
    if two_i % 2 or out.shape != (rows, two_i // 2):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_swiglu(_ptr(gate_up), _ptr(out), _code(out.dtype), c_int(rows), c_int(two_i // 2),
                          c_int(1 if interleave8 else 0), _stream()))


def gemm_add_accepts(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether ``gemm_add`` takes this product: a prompt-sized bfloat16 product into a float32 ``out``."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.float32 and a.dim() == 2
            and a.shape[0] >= TC5_PAIR_MIN_ROWS and w.is_contiguous() and tc5_accepts(a, w, out)
            and out.stride(0) % 4 == 0 and out.data_ptr() % 16 == 0)


def gemm_add(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out += a @ w^T in the epilogue of the tiled tcgen05 kernel (``out`` float32: the residual
    stream); the sum per element is out + product, both float32, as a separate add would give."""
    _need(a, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", torch.float32, 2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1 or not gemm_add_accepts(a, w, out):
        raise KernelError(f"gemm_add: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_gemm_tc5_pair_add(_ptr(a), _ptr(w), _ptr(out), c_int(M), c_int(N), c_int(K), c_int64(a.stride(0)),
                                     c_int64(out.stride(0)), _stream()))


def gemm_swiglu_accepts(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_swiglu`` takes this product: bfloat16 operands the tensor-core kernels accept,
    gate/up rows interleaved in blocks of eight (every one of those kernels has the fused epilogue)."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and w.shape[0] % 16 == 0 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_swiglu(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: str = "auto") -> None:
    """out[M, N/2] = silu(a Wg^T) * (a Wu^T) in one kernel, the one ``gemm`` would pick for a
    product of these sizes; ``w`` [N, K] holds gate and up rows interleaved in blocks of eight."""
    _need(a, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N // 2) or out.stride(1) != 1 or not gemm_swiglu_accepts(a, w):
        raise KernelError(f"gemm_swiglu: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if algo == "auto":
        algo = gemm_algo(M, N, K)
    if algo == "tc5_pair":
        _check(_lib.gb_gemm_tc5_pair_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                            c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5":
        _check(_lib.gb_gemm_tc5_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                       c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_decode":
        _tc5_decode(a, w, out, 1)
    elif algo == "skinny":
        _check(_lib.gb_gemm_skinny_swiglu(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                          c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    else:
        raise KernelError(f"gemm_swiglu: unknown algorithm '{algo}'")


# ---- few-row products with the residual's row-wise work folded in ------------------------
FOLD_ROWS = int(_lib.gb_dispatch_constant(c_int(5)))   # the folded products take up to this many rows


def fold_capacity(width: int) -> int:
    """Partial sums a row that a statistics buffer must have room for when ``gemm_residual`` writes a
    residual ``width`` wide: one per 16 columns (the kernel for more than 8 rows leaves one per 128)."""
    return (width + 15) // 16


def _skinny_operands_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and 0 < x.shape[0] <= FOLD_ROWS
            and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


def gemm_scaled_accepts(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``gemm_scaled`` takes this product: up to 64 bfloat16 rows against bfloat16 weights
    whose rows are 16-byte aligned."""
    return _skinny_operands_ok(x, w)


def gemm_scaled(x: torch.Tensor, eps: float, stats: torch.Tensor, stats_count: int, w: torch.Tensor, out: torch.Tensor,
                swiglu: bool = False) -> str:
    """out[r] = rs[r] * (x[r] @ w^T) with rs[r] = 1 / sqrt(sum_r / K + eps), sum_r the sum of the
    ``stats_count`` partial sums stats[r, :stats_count]: the product of RMSNorm rows whose factor was
    left out when ``x = bf16(h * norm_weight)`` was made (by ``gemm_residual`` or ``embed_gather``).
    With ``swiglu``, ``w`` holds gate and up rows interleaved in blocks of eight and
    out[M, N / 2] = silu(gate) * up.  Returns the kernel's name."""
    _need(x, "prescaled rows", torch.bfloat16, 2, contiguous=False)
    _need(stats, "row statistics", torch.float32, 2)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = x.shape
    N = w.shape[0]
    if (not gemm_scaled_accepts(x, w) or w.shape[1] != K or out.stride(1) != 1
            or out.shape != (M, N // 2 if swiglu else N) or stats.shape[0] < M or not 0 < stats_count <= stats.shape[1]):
        raise KernelError(f"gemm_scaled: x {tuple(x.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}, "
                          f"{stats_count} partial sums in {tuple(stats.shape)}")
    if _ALGO_NAMES[int(_lib.gb_gemm_scaled_algo(c_int(M), c_int(N), c_int(K), c_int(_sms())))] == "skinny":
        _check(_lib.gb_gemm_skinny_scaled(_ptr(x), c_int64(x.stride(0)), c_float(eps), _ptr(stats), c_int(stats_count),
                                          c_int64(stats.stride(0)), _ptr(w), _ptr(out), _code(out.dtype), c_int64(out.stride(0)),
                                          c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), _stream()))
        return "skinny"
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    _check(_lib.gb_gemm_tc5_decode_scaled(_ptr(x), c_int64(x.stride(0)), c_float(eps), _ptr(stats), c_int(stats_count),
                                          c_int64(stats.stride(0)), _ptr(w), _ptr(out), _code(out.dtype), c_int64(out.stride(0)),
                                          c_int(M), c_int(N), c_int(K), c_int(1 if swiglu else 0), c_int(splits), _stream()))
    return "tc5_decode"


def gemm_residual_accepts(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor) -> bool:
    return _skinny_operands_ok(x, w) and h.dtype == torch.float32 and h.stride(1) == 1


def gemm_residual(x: torch.Tensor, w: torch.Tensor, h: torch.Tensor, stats: torch.Tensor,
                  next_weight: Optional[torch.Tensor] = None, next_x: Optional[torch.Tensor] = None, behind: str = "") -> int:
    """h += x @ w^T in place (``h`` float32: the residual stream; one float32 addition per element,
    as a separate add gives) and stats[row, c] = the sum of squares of the new values of the row
    in the c-th block of columns (16 wide up to 8 rows, 128 wide above).  With ``next_weight`` also next_x = bf16(h * next_weight), the rows
    ``gemm_scaled`` takes.  ``stats`` needs ``fold_capacity(N)`` columns.  ``behind``: the kernel
    that made ``x`` (what ``gemm_scaled`` returned), if the caller knows it; a few-row kernel behind
    the tcgen05 decode kernel is launched as an ordinary kernel.  Returns the number of partial sums
    a row."""
    _need(x, "gemm a", torch.bfloat16, 2, contiguous=False)
    _need(w, "gemm w", torch.bfloat16, 2)
    _need(h, "residual", torch.float32, 2, contiguous=False)
    _need(stats, "row statistics", torch.float32, 2)
    M, K = x.shape
    N = w.shape[0]
    count = fold_capacity(N)
    if not gemm_residual_accepts(x, w, h) or w.shape[1] != K or h.shape != (M, N) or stats.shape[0] < M or stats.shape[1] < count:
        raise KernelError(f"gemm_residual: x {tuple(x.shape)}, w {tuple(w.shape)}, h {tuple(h.shape)}, statistics {tuple(stats.shape)}")
    ldxn = _check_next(next_weight, next_x, M, N, "gemm_residual")
    if gemm_algo(M, N, K) == "skinny":
        _check(_lib.gb_gemm_skinny_residual(_ptr(x), c_int64(x.stride(0)), _ptr(w), _ptr(h), c_int64(h.stride(0)), _ptr(stats),
                                            c_int64(stats.stride(0)), _ptr(next_weight), _ptr(next_x), c_int64(ldxn),
                                            c_int(M), c_int(N), c_int(K), c_int(1 if behind == "tc5_decode" else 0), _stream()))
        return count
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    made = c_int(0)
    _check(_lib.gb_gemm_tc5_decode_residual(_ptr(x), c_int64(x.stride(0)), _ptr(w), _ptr(h), c_int64(h.stride(0)), _ptr(stats),
                                            c_int64(stats.stride(0)), byref(made), _ptr(next_weight), _ptr(next_x), c_int64(ldxn),
                                            c_int(M), c_int(N), c_int(K), c_int(splits), _stream()))
    return made.value


# ---- matrix products ---------------------------------------------------------------------
def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T with fp32 multiply-add on the CUDA cores (any dtypes)."""
    _need(a, "gemm a", dim=2, contiguous=False)
    _need(w, "gemm w", dim=2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    _check(_lib.gb_gemm_simt(_ptr(a), _code(a.dtype), _ptr(w), _code(w.dtype), _ptr(out), _code(out.dtype),
                             c_int(M), c_int(N), c_int(K), c_int64(a.stride(0)), c_int64(w.stride(0)),
                             c_int64(out.stride(0)), _stream()))


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, algo: str = "auto") -> str:
    """out = a @ w^T, choosing the kernel by operand types and sizes.  Returns the kernel's name.

    bfloat16 activations with bfloat16 weights go to the tensor-core kernels (``gemm_algo``): up to
    8 rows the fragment-streaming kernel, up to 64 rows (128 or 256 for narrow outputs) the tcgen05
    decode kernel, otherwise the tiled tcgen05 kernel and from 192 rows the one that pairs two SMs
    on a tile.  Everything else,
    and operands whose rows are not 16-byte aligned, goes to the fp32 CUDA-core kernel.  float32
    operands never touch a tensor core.
    """
    _need(a, "gemm a", dim=2, contiguous=False)
    _need(w, "gemm w", dim=2)
    _need(out, "gemm out", dim=2, contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or a.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError(f"gemm: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError(f"gemm: output dtype {out.dtype}")
    if algo == "simt" or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        gemm_simt(a, w, out)
        return "simt"
    aligned = (K % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
               and a.stride(1) == 1 and w.is_contiguous())
    if not aligned:
        gemm_simt(a, w, out)
        return "simt"
    if algo == "auto":
        algo = gemm_algo(M, N, K)
    if algo == "skinny":
        _check(_lib.gb_gemm_skinny(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                   c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5":
        _check(_lib.gb_gemm_tc5(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_pair":
        _check(_lib.gb_gemm_tc5_pair(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                     c_int64(a.stride(0)), c_int64(out.stride(0)), _stream()))
    elif algo == "tc5_decode":
        _tc5_decode(a, w, out, 0)
    elif algo == "simt":
        gemm_simt(a, w, out)
    else:
        raise KernelError(f"gemm: unknown algorithm '{algo}'")
    return algo


_ALGO_NAMES = ("simt", "skinny", "tc5", "tc5_pair", "tc5_decode")


def gemm_algo(M: int, N: int, K: int) -> str:
    """The tensor-core kernel ``gemm`` picks for aligned bfloat16 operands of these sizes: up to 8 rows
    the fragment-streaming kernel, up to 64 rows (128 or 256 for narrow outputs) the tcgen05 decode
    kernel, otherwise the tiled tcgen05 kernel and from 192 rows the one that pairs two SMs on a
    tile.  The rule lives in the library (``gb_gemm_algo``), which also applies it when it
    issues a whole layer itself."""
    return _ALGO_NAMES[int(_lib.gb_gemm_algo(c_int(M), c_int(N), c_int(K), c_int(_sms())))]


# the rule's thresholds, as the library holds them: rows up to which the fragment-streaming kernel
# is used, rows up to which the tcgen05 decode kernel takes a product, rows from which two SMs are
# paired on a tile, and the output width from which the decode kernel takes every row count
SKINNY_MAX_ROWS, TC5_DECODE_MAX_ROWS, TC5_PAIR_MIN_ROWS, WIDE_OUTPUT, TC5_ATTENTION_MIN_ROWS = (
    int(_lib.gb_dispatch_constant(c_int(i))) for i in range(5))

_sm_count = {}


def _sms() -> int:
    """SMs of the library's device."""
    dev = _device_index[0] if _device_index else torch.cuda.current_device()
    if dev not in _sm_count:
        _sm_count[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _sm_count[dev]


def _tc5_decode(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epi: int) -> None:
    M, K = a.shape
    N = w.shape[0]
    splits = int(_lib.gb_gemm_tc5_decode_splits(c_int(M), c_int(N), c_int(K), c_int(_sms())))
    _check(_lib.gb_gemm_tc5_decode(_ptr(a), _ptr(w), _ptr(out), _code(out.dtype), c_int(M), c_int(N), c_int(K),
                                   c_int64(a.stride(0)), c_int64(out.stride(0)), c_int(epi), c_int(splits), _stream()))


def tc5_accepts(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tcgen05 kernel takes this product (TMA wants 16-byte rows; edges are free)."""
    K = a.shape[1]
    return K % 8 == 0 and a.stride(0) % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def is_checked_build() -> bool:
    """Whether the loaded library was compiled with bounds-checked indices (GOPHONIC_B200_CHECKED=1)."""
    return bool(_lib.gb_is_checked())


_CHECK_NAMES = {1: "a token id outside the vocabulary", 2: "a position outside the token source", 3: "a cache slot outside the block table",
                4: "a position beyond the pages of a block-table row", 5: "a block-table entry outside the cache plane",
                6: "a position beyond the rotation tables", 7: "a sequence length that does not fit", 8: "a page triple outside the table or plane"}


def checked_status():
    """None, or (where, what, value, bound, count) for the first index a kernel of the checked build
    found out of bounds since the last call (the access was skipped or redirected, nothing faulted).
    Always None in the ordinary build, whose kernels carry no checks.  Synchronises."""
    out = (c_int * 4)()
    for name in ("rows", "cache", "attention_simt", "attention_mma", "attention_tc5"):
        code = int(getattr(_lib, "gb_checked_status_" + name)(out))
        if code or out[3]:
            return name, _CHECK_NAMES.get(code, f"code {code}"), out[1], out[2], out[3]
    return None


def tc5_status() -> int:
    """0, or which role of a tcgen05 kernel gave up waiting on a barrier since the last call."""
    code = 0
    for name in ("gb_gemm_tc5_status", "gb_gemm_tc5_decode_status", "gb_attention_tc5_status"):
        code = code or int(getattr(_lib, name)())
    return code


# ---- attention ---------------------------------------------------------------------------
class _QkRopeParams(Structure):
    _fields_ = [
        ("qkv", c_void_p), ("row_stride", c_int64), ("q_w", c_void_p), ("k_w", c_void_p), ("eps", c_float),
        ("cos_t", c_void_p), ("sin_t", c_void_p), ("rot", c_int), ("table_positions", c_int),
        ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p), ("block_table", c_void_p),
        ("bt_stride", c_int), ("k_plane", c_void_p), ("v_plane", c_void_p),
        ("write_kv", c_int), ("rows", c_int), ("heads", c_int), ("kv_heads", c_int), ("d", c_int),
        ("pages", c_int), ("max_slots", c_int),
    ]


def _rope_params(qkv: torch.Tensor, heads: int, kv_heads: int, head_dim: int,
                 q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                 cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
                 row_pos: torch.Tensor, row_seq: torch.Tensor, seq_slot: torch.Tensor,
                 block_table: torch.Tensor,
                 k_plane: Optional[torch.Tensor], v_plane: Optional[torch.Tensor], write_kv: bool) -> "_QkRopeParams":
    _need(qkv, "qkv", dim=2)
    rows = qkv.shape[0]
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope: qkv {tuple(qkv.shape)} for {heads}+2x{kv_heads} heads of {head_dim}")
    for t, nm in ((q_weight, "q norm"), (k_weight, "k norm")):
        if t is not None:
            _need(t, nm, torch.float32, 1)
            if t.numel() != head_dim:
                raise KernelError(f"qk_norm_rope: {nm} weight has {t.numel()} elements, head_dim is {head_dim}")
    table_positions = 0
    if rotary_dim > 0:
        _need(cos, "rope cos", torch.float32, 2)
        _need(sin, "rope sin", torch.float32, 2)
        if cos.shape[1] != rotary_dim // 2 or sin.shape != cos.shape:
            raise KernelError(f"qk_norm_rope: angle tables {tuple(cos.shape)} for rotary width {rotary_dim}")
        table_positions = cos.shape[0]
    for t, nm in ((row_pos, "row_pos"), (row_seq, "row_seq"), (seq_slot, "seq_slot")):
        _need(t, nm, torch.int32, 1)
    _need(block_table, "block table", torch.int32, 2)
    if write_kv:
        for t, nm in ((k_plane, "key plane"), (v_plane, "value plane")):
            _need(t, nm, qkv.dtype, 4)
            if t.shape[1] != kv_heads or t.shape[2] != PAGE or t.shape[3] != head_dim:
                raise KernelError(f"qk_norm_rope: {nm} {tuple(t.shape)} for {kv_heads} kv heads of {head_dim}")
    p = _QkRopeParams(qkv.data_ptr(), qkv.stride(0), 0 if q_weight is None else q_weight.data_ptr(),
                      0 if k_weight is None else k_weight.data_ptr(), eps,
                      0 if cos is None else cos.data_ptr(), 0 if sin is None else sin.data_ptr(), rotary_dim,
                      table_positions, row_pos.data_ptr(), row_seq.data_ptr(), seq_slot.data_ptr(),
                      block_table.data_ptr(), block_table.stride(0),
                      0 if k_plane is None else k_plane.data_ptr(), 0 if v_plane is None else v_plane.data_ptr(),
                      1 if write_kv else 0, rows, heads, kv_heads, head_dim,
                      0 if k_plane is None else k_plane.shape[0], block_table.shape[0])
    return p


def qk_norm_rope_kv_write(qkv: torch.Tensor, *args) -> None:
    """Per-head RMSNorm of q and k, rotary embedding of both, q in place, k and v into the cache:
    (qkv, heads, kv_heads, head_dim, q_weight, k_weight, eps, cos, sin, rotary_dim, row_pos, row_seq,
    seq_slot, block_table, k_plane, v_plane, write_kv)."""
    p = _rope_params(qkv, *args)
    _check(_lib.gb_qk_norm_rope_kv_write(byref(p), _code(qkv.dtype), _stream()))


class _AttnParams(Structure):
    _fields_ = [
        ("q", c_void_p), ("q_row_stride", c_int64), ("out", c_void_p), ("out_row_stride", c_int64),
        ("k_plane", c_void_p), ("v_plane", c_void_p), ("block_table", c_void_p), ("bt_stride", c_int),
        ("seq_slot", c_void_p), ("seq_q_start", c_void_p), ("seq_q_len", c_void_p),
        ("seq_kv_len", c_void_p), ("nseq", c_int), ("heads", c_int), ("kv_heads", c_int), ("d", c_int),
        ("max_q_len", c_int), ("scale", c_float), ("window", c_int), ("num_splits", c_int), ("scratch", c_void_p),
        ("pages", c_int), ("max_slots", c_int),
    ]


def attention_scratch_floats(nseq: int, heads: int, head_dim: int, num_splits: int) -> int:
    return nseq * heads * num_splits * (head_dim + 2)


def _attn_params(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
                 block_table: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
                 seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor, nseq: int, max_q_len: int,
                 heads: int, kv_heads: int, head_dim: int, scale: float, window: int,
                 num_splits: int, scratch: Optional[torch.Tensor]) -> "_AttnParams":
    _need(q, "attention q", dim=2, contiguous=False)
    _need(out, "attention out", q.dtype, 2, contiguous=False)
    if q.stride(1) != 1 or out.stride(1) != 1 or q.shape[1] < heads * head_dim or out.shape[1] < heads * head_dim:
        raise KernelError(f"attention: q {tuple(q.shape)}, out {tuple(out.shape)} for {heads} heads of {head_dim}")
    for t, nm in ((k_plane, "key plane"), (v_plane, "value plane")):
        _need(t, nm, q.dtype, 4)
        if t.shape[1] != kv_heads or t.shape[2] != PAGE or t.shape[3] != head_dim:
            raise KernelError(f"attention: {nm} {tuple(t.shape)} for {kv_heads} kv heads of {head_dim}")
    for t, nm in ((seq_slot, "seq_slot"), (seq_q_start, "seq_q_start"), (seq_q_len, "seq_q_len"),
                  (seq_kv_len, "seq_kv_len")):
        _need(t, nm, torch.int32, 1)
        if t.numel() < nseq:
            raise KernelError(f"attention: {nm} has {t.numel()} entries for {nseq} sequences")
    _need(block_table, "block table", torch.int32, 2)
    if num_splits > 1:
        if scratch is None:
            raise KernelError("attention: key splits need scratch memory")
        _need(scratch, "attention scratch", torch.float32)
        if scratch.numel() < attention_scratch_floats(nseq, heads, head_dim, num_splits):
            raise KernelError("attention: scratch is too small")
    p = _AttnParams(q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_plane.data_ptr(), v_plane.data_ptr(),
                    block_table.data_ptr(), block_table.stride(0), seq_slot.data_ptr(),
                    seq_q_start.data_ptr(), seq_q_len.data_ptr(), seq_kv_len.data_ptr(), nseq, heads, kv_heads,
                    head_dim, max_q_len, scale, window, num_splits, 0 if scratch is None else scratch.data_ptr(),
                    k_plane.shape[0], block_table.shape[0])
    return p


def attention(q: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor,
              block_table: torch.Tensor, seq_slot: torch.Tensor, seq_q_start: torch.Tensor,
              seq_q_len: torch.Tensor, seq_kv_len: torch.Tensor, nseq: int, max_q_len: int,
              heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
              num_splits: int = 1, scratch: Optional[torch.Tensor] = None, algo: str = "auto") -> str:
    """Causal GQA over the paged cache.  q is a [rows, >= heads*head_dim] view (row stride free),
    out is [rows, heads*head_dim].  Returns the kernel's name."""
    p = _attn_params(q, out, k_plane, v_plane, block_table, seq_slot, seq_q_start, seq_q_len, seq_kv_len, nseq, max_q_len,
                     heads, kv_heads, head_dim, scale, window, num_splits, scratch)
    if algo == "auto":   # the library's own rule (head size, rows per sequence, alignment)
        algo = ("simt", "decode_mma", "prefill_mma", "prefill_tc5")[int(_lib.gb_attention_algo(byref(p), _code(q.dtype)))]
    nk = 2 if num_splits > 1 else 1
    if algo == "simt":
        _check(_lib.gb_attention_simt(byref(p), _code(q.dtype), _stream()), nk)
    elif algo == "decode_mma":
        _check(_lib.gb_attention_decode_mma(byref(p), _stream()), nk)
    elif algo == "prefill_mma":
        _check(_lib.gb_attention_prefill_mma(byref(p), _stream()))
    elif algo == "prefill_tc5":
        _check(_lib.gb_attention_prefill_tc5(byref(p), c_int(q.shape[0]), c_int(k_plane.shape[0]), _stream()))
    else:
        raise KernelError(f"attention: unknown algorithm '{algo}'")
    return algo


def attention_decode_rope_accepts(dtype: torch.dtype, head_dim: int, rotary_dim: int, max_q_len: int) -> bool:
    """Whether ``attention_decode_rope`` takes rows of this kind (bfloat16, one row a sequence, a head
    size the tensor-core single-token kernel takes)."""
    return dtype in (torch.float32, torch.bfloat16) and bool(_lib.gb_attention_decode_rope_accepts(_code(dtype), c_int(head_dim), c_int(rotary_dim), c_int(max_q_len)))


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, rope_args: tuple, attn_args: tuple) -> None:
    """``qk_norm_rope_kv_write(qkv, *rope_args)`` and ``attention(qkv[:, :heads * head_dim], out,
    *attn_args)`` for single-token rows in one kernel (plus the merge of key splits): the attention
    kernel norms and rotates its queries itself, takes the token's own key and value from the row and
    stores them in the cache.  The same bits as the two calls."""
    r = _rope_params(qkv, *rope_args)
    a = _attn_params(qkv[:, :r.heads * r.d], out, *attn_args)
    _check(_lib.gb_attention_decode_mma_rope(byref(a), byref(r), _stream()), 2 if a.num_splits > 1 else 1)


# ---- a whole pre-norm layer from one call ---------------------------------------------------
class PrenormLayer(Structure):
    """Sizes, constants and tensors of one pre-norm layer of attention and SwiGLU (``GbPrenormLayer``)."""
    _fields_ = [
        ("hidden", c_int), ("heads", c_int), ("kv_heads", c_int), ("head_dim", c_int), ("intermediate", c_int),
        ("mixer_norm_eps", c_float), ("ffn_norm_eps", c_float), ("qk_norm_eps", c_float), ("scale", c_float),
        ("window", c_int), ("rotary_dim", c_int), ("table_positions", c_int), ("act_dtype", c_int), ("gate_up_interleaved", c_int),
        ("mixer_norm_w", c_void_p), ("ffn_norm_w", c_void_p), ("w_qkv", c_void_p), ("w_qkv_dtype", c_int), ("w_o", c_void_p),
        ("w_o_dtype", c_int), ("w_gate_up", c_void_p), ("w_gate_up_dtype", c_int), ("w_down", c_void_p), ("w_down_dtype", c_int),
        ("q_norm_w", c_void_p), ("k_norm_w", c_void_p), ("cos_t", c_void_p), ("sin_t", c_void_p),
    ]


class _StepRows(Structure):
    _fields_ = [
        ("rows", c_int), ("nseq", c_int), ("max_q_len", c_int), ("row_pos", c_void_p), ("row_seq", c_void_p), ("seq_slot", c_void_p),
        ("seq_q_start", c_void_p), ("seq_q_len", c_void_p), ("seq_kv_len", c_void_p), ("num_splits", c_int), ("split_scratch", c_void_p),
        ("block_table", c_void_p), ("bt_stride", c_int), ("k_plane", c_void_p), ("v_plane", c_void_p), ("pages", c_int), ("write_kv", c_int),
        ("max_slots", c_int),
    ]


_lib.gb_prenorm_layer_workspace.restype = c_int64


def prenorm_layer_workspace(layer: PrenormLayer, rows: int) -> int:
    """Bytes of workspace ``prenorm_layer_forward`` needs for a step of ``rows`` rows."""
    return int(_lib.gb_prenorm_layer_workspace(byref(layer), c_int(rows)))


def prenorm_layer_forward(layer: PrenormLayer, batch, cache, h: torch.Tensor, delta: Optional[torch.Tensor],
                          workspace: torch.Tensor, num_splits: int = 1, split_scratch: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Issue every kernel of one pre-norm layer (norm, q/k/v product, q/k norm + rotation + cache
    write, attention, output projection, norm, gate/up product with SwiGLU, down projection) from one
    call into the library: the kernels, their order and their choice by size are those of the
    part-by-part path.  ``h`` is the float32 residual, updated in place; ``delta`` an addend it is
    still owed (added by the first norm).  Returns the addend the layer leaves owed (a view into
    ``workspace``), or None if its products added into the residual themselves."""
    _need(h, "residual", torch.float32, 2)
    _need(workspace, "layer workspace", torch.uint8, 1)
    rows = h.shape[0]
    if h.shape[1] != layer.hidden or rows != batch.rows:
        raise KernelError(f"prenorm_layer: residual {tuple(h.shape)} for {batch.rows} rows of {layer.hidden}")
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != h.shape:
            raise KernelError(f"prenorm_layer: delta {tuple(delta.shape)} vs residual {tuple(h.shape)}")
    if cache.k.dtype != (torch.bfloat16 if layer.act_dtype == BF16 else torch.float32):
        raise KernelError(f"prenorm_layer: the cache holds {cache.k.dtype}")
    step = _StepRows(rows, batch.nseq, batch.max_q_len, batch.row_pos.data_ptr(), batch.row_seq.data_ptr(), batch.seq_slot.data_ptr(),
                     batch.seq_q_start.data_ptr(), batch.seq_q_len.data_ptr(), batch.seq_kv_len.data_ptr(), num_splits,
                     0 if split_scratch is None else split_scratch.data_ptr(), cache.block_table.data_ptr(), cache.block_table.stride(0),
                     cache.k.data_ptr(), cache.v.data_ptr(), cache.k.shape[0], 1 if cache.writable else 0, cache.block_table.shape[0])
    out_ptr, n = c_void_p(0), c_int(0)
    _check(_lib.gb_prenorm_layer_forward(byref(layer), byref(step), _ptr(h), _ptr(delta), _ptr(workspace), c_int64(workspace.numel()),
                                         c_int(_sms()), byref(out_ptr), byref(n), _stream()), 0)
    global launches
    launches += n.value
    if not out_ptr.value:
        return None
    at = out_ptr.value - workspace.data_ptr()
    return workspace[at:at + 4 * rows * layer.hidden].view(torch.float32).view(rows, layer.hidden)


# ---- sampling ----------------------------------------------------------------------------
def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    _need(out, "argmax out", torch.int32, 1)
    if logits.stride(1) != 1 or out.numel() != logits.shape[0]:
        raise KernelError(f"argmax: logits {tuple(logits.shape)}, out {out.numel()}")
    rows, vocab = logits.shape
    if vocab > 16384:  # wide rows: many CTAs a row, merged by a second small kernel
        chunks = (vocab + 8191) // 8192
        scratch = torch.empty(2 * rows * chunks, dtype=torch.float32, device=logits.device)
        _check(_lib.gb_argmax_wide(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(out),
                                   _ptr(scratch), _stream()), 2)
        return
    _check(_lib.gb_argmax(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(out), _stream()))


def sample_scratch_bytes(rows: int, vocab: int) -> int:
    """Bytes of scratch with which ``sample`` spreads a row of a wide vocabulary over many CTAs."""
    _lib.gb_sample_scratch_bytes.restype = c_int64
    return int(_lib.gb_sample_scratch_bytes(c_int(rows), c_int(vocab)))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, draw: torch.Tensor, out: torch.Tensor, opt_row: Optional[torch.Tensor] = None,
           advance: bool = False, scratch: Optional[torch.Tensor] = None) -> None:
    """One token per row: greedy where temperature <= 0, else top-k / top-p sampling with the
    counter-based draw (seed, draw).  Row i takes its options from entry ``opt_row[i]`` of the
    option tensors (entry i without ``opt_row``); with ``advance`` the kernel adds one to the draw
    counter of every row it sampled.  ``scratch`` (uint8, ``sample_scratch_bytes``) lets rows of a
    wide vocabulary be selected by many CTAs; without it one CTA scans each row."""
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    rows = logits.shape[0]
    _need(temperature, "temperature", torch.float32, 1)
    _need(top_k, "top_k", torch.int32, 1)
    _need(top_p, "top_p", torch.float32, 1)
    _need(seed, "seed", torch.int64, 1)
    _need(draw, "draw", torch.int64, 1)
    _need(out, "sample out", torch.int32, 1)
    if out.numel() < rows:
        raise KernelError("sample: out is shorter than the batch")
    if opt_row is not None:
        _need(opt_row, "option rows", torch.int32, 1)
        if opt_row.numel() < rows:
            raise KernelError("sample: opt_row is shorter than the batch")
    else:
        for t in (temperature, top_k, top_p, seed, draw):
            if t.numel() < rows:
                raise KernelError("sample: a per-row option tensor is shorter than the batch")
    if logits.stride(1) != 1:
        raise KernelError("sample: logits rows are not contiguous")
    nbytes = 0
    if scratch is not None:
        _need(scratch, "sample scratch", torch.uint8, 1)
        nbytes = scratch.numel()
    want = sample_scratch_bytes(rows, logits.shape[1])
    wide = 0 < want <= nbytes
    _check(_lib.gb_sample(_ptr(logits), c_int(rows), c_int(logits.shape[1]), c_int64(logits.stride(0)), _ptr(opt_row),
                          _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(seed), _ptr(draw), _ptr(out),
                          c_int(1 if advance else 0), _ptr(scratch), c_int64(nbytes), _stream()), 3 if wide else 1)


def presence_penalty(logits: torch.Tensor, seen: torch.Tensor, seen_row: torch.Tensor, presence: torch.Tensor,
                     indexed: bool = False) -> None:
    """logits[r, v] -= presence for every token v set in bitmap row seen_row[r]; the penalty is
    presence[r], or presence[seen_row[r]] with ``indexed``."""
    _need(logits, "logits", torch.float32, 2, contiguous=False)
    _need(seen, "seen bitmap", torch.int32, 2)
    _need(seen_row, "seen row", torch.int32, 1)
    _need(presence, "presence", torch.float32, 1)
    rows, vocab = logits.shape
    if seen.shape[1] * 32 < vocab:
        raise KernelError("presence_penalty: bitmap is narrower than the vocabulary")
    _check(_lib.gb_presence_penalty(_ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)), _ptr(seen),
                                    c_int64(seen.stride(0)), _ptr(seen_row), _ptr(presence), c_int(1 if indexed else 0), _stream()))


def mark_seen(tokens: torch.Tensor, vocab: int, seen: torch.Tensor, seen_row: torch.Tensor) -> None:
    _need(tokens, "tokens", torch.int32, 1)
    _need(seen, "seen bitmap", torch.int32, 2)
    _need(seen_row, "seen row", torch.int32, 1)
    _check(_lib.gb_mark_seen(_ptr(tokens), c_int(tokens.numel()), c_int(vocab), _ptr(seen), c_int64(seen.stride(0)),
                             _ptr(seen_row), _stream()))


def f32_to_bf16(a: torch.Tensor, out: torch.Tensor) -> None:
    _need(a, "a", torch.float32)
    _need(out, "out", torch.bfloat16)
    if a.numel() != out.numel():
        raise KernelError("f32_to_bf16: sizes differ")
    _check(_lib.gb_f32_to_bf16(_ptr(a), _ptr(out), c_int64(a.numel()), _stream()))
