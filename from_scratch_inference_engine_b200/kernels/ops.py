"""Typed Python entry points of the hand-written CUDA kernels.

Each function checks what the kernel assumes (device, dtype, contiguity, sizes),
passes raw pointers and the current CUDA stream to the C entry point, and raises on
any non-zero return.  There is no other implementation behind these functions: on a
machine without the compiled library or without a GPU they raise.
"""

from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from ..csrc import build

DTYPE_F32, DTYPE_BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _tag(dtype: torch.dtype) -> int:
    if dtype is torch.float32:
        return DTYPE_F32
    if dtype is torch.bfloat16:
        return DTYPE_BF16
    raise KernelError(f"kernels take float32 or bfloat16 storage, not {dtype}")


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The address for a pointer argument (ctypes takes an int or None for c_void_p)."""
    return None if tensor is None else tensor.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream's handle.  Asked for at every launch (streams change under
    graph capture), so by the cheapest route torch offers."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(tensor: torch.Tensor, dtype, name: str, contiguous: bool = True) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on the GPU (the engine has no CPU path)")
    if dtype is not None and tensor.dtype is not dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if contiguous and not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


launches = 0      # kernel launches issued through this module (benchmarks read this)


def _check(code: int, what: str) -> None:
    global launches
    launches += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: argument refused by the kernel launcher")
    if code == -2:
        raise KernelError(f"{what}: size not supported by this kernel")
    raise KernelError(f"{what}: CUDA error {code}")


_core = None


def core():
    """The core kernel library, compiled at first use."""
    global _core
    if _core is None:
        lib = build.load_library("core")
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_embed_gather.argtypes = [p, p, p, i, i, i, i, p, p]
        lib.fsie_add_rmsnorm.argtypes = [p, p, p, i, p, p, i, i, f, i, i, p]
        lib.fsie_rope_kv_write.argtypes = [p, i, p, p, i, p, p, p, ll, i, i, i, i, i, i, i, i, p, p]
        lib.fsie_swiglu.argtypes = [p, p, ll, i, i, p]
        lib.fsie_place_tokens.argtypes = [p, p, p, p, i, p]
        lib.fsie_gemm_f32.argtypes = [p, p, p, p, i, i, i, i, i, i, i, p]
        lib.fsie_gemm_f32_rows_limit.argtypes = []
        lib.fsie_gemm_f32_rows_limit.restype = i
        lib.fsie_attn_generic.argtypes = [p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                          i, i, i, i, i, i, f, i, p]
        lib.fsie_attn_tiles.argtypes = [p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                        i, i, i, i, i, i, f, i, i, i, p]
        lib.fsie_attn_tiles.restype = i
        lib.fsie_attn_generic_rows.argtypes = []
        lib.fsie_attn_rows16_rows.argtypes = []
        lib.fsie_attn_rows16_rows.restype = i
        lib.fsie_attn_rows16_takes.argtypes = [i]
        lib.fsie_attn_rows16_takes.restype = i
        lib.fsie_argmax.argtypes = [p, i, i, p, p]
        lib.fsie_argmax_staged.argtypes = [p, i, i, p, p, i, p]
        lib.fsie_sample.argtypes = [p, i, i, p, p, p, p, p, p]
        for name in ("fsie_embed_gather", "fsie_add_rmsnorm", "fsie_rope_kv_write", "fsie_swiglu",
                     "fsie_gemm_f32", "fsie_attn_generic", "fsie_attn_generic_rows",
                     "fsie_argmax", "fsie_argmax_staged", "fsie_sample"):
            getattr(lib, name).restype = ctypes.c_int
        _core = lib
    return _core


# ------------------------------------------------------------------------- embedding
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor,
                 error: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]] widened to float32; an id outside the table sets error[0]."""
    _need(ids, torch.int32, "ids")
    _need(table, None, "table")
    _need(out, torch.float32, "out")
    _need(error, torch.int32, "error")
    tokens, (vocab, hidden) = ids.numel(), table.shape
    if out.shape[-1] != hidden or out.numel() < tokens * hidden:
        raise KernelError("embed_gather: out is too small")
    _check(core().fsie_embed_gather(_ptr(ids), _ptr(table), _ptr(out), tokens, hidden, vocab,
                                    _tag(table.dtype), _ptr(error), _stream()), "embed_gather")
    return out


# ---------------------------------------------------------------------- add + RMSNorm
def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None,
                write_x: bool = True) -> torch.Tensor:
    """x (float32 residual) += delta; out = rmsnorm(x) * gain in out's dtype.

    With `rows` (int32 indices) only those rows are normed, into out[0..len(rows)), and
    x is left untouched unless write_x.
    """
    _need(x, torch.float32, "x")
    _need(out, None, "out")
    hidden = x.shape[-1]
    if delta is not None:
        _need(delta, out.dtype, "delta")
        if delta.shape[-1] != hidden:
            raise KernelError("add_rmsnorm: delta width differs from x")
    _need(gain, None, "gain")
    if gain.numel() != hidden:
        raise KernelError("add_rmsnorm: gain width differs from x")
    if gain.dtype not in (torch.float32, out.dtype):
        raise KernelError(f"add_rmsnorm: gain must be float32 or {out.dtype}")
    if rows is not None:
        _need(rows, torch.int32, "rows")
        count = rows.numel()
    else:
        count = x.numel() // hidden
    if out.numel() < count * hidden:
        raise KernelError("add_rmsnorm: out is too small")
    _check(core().fsie_add_rmsnorm(_ptr(x), _ptr(delta), _ptr(gain),
                                   int(gain.dtype is torch.float32), _ptr(out), _ptr(rows), count,
                                   hidden, float(eps), int(write_x), _tag(out.dtype), _stream()),
           "add_rmsnorm")
    return out


# ------------------------------------------------------- rotary + paged cache write
def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos_sin: torch.Tensor,
                  slot_of: Optional[torch.Tensor], k_pages: Optional[torch.Tensor],
                  v_pages: Optional[torch.Tensor], page_stride: int, page_size: int,
                  heads: int, kv_heads: int, head_dim: int, rotary_dim: int,
                  error: torch.Tensor) -> None:
    """Rotate q in place in the fused projection rows; rotate k and store k, v in their pages.

    k_pages / v_pages are views whose first element is page 0 of this cache entry;
    page p of it starts page_stride elements further per page.
    """
    _need(qkv, None, "qkv")
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    tokens, ld = qkv.shape
    if ld < (heads + 2 * kv_heads) * head_dim:
        raise KernelError("rope_kv_write: projection rows are narrower than q, k and v")
    if rotary_dim > 0 and cos_sin.shape[-1] != rotary_dim:
        raise KernelError("rope_kv_write: cos/sin table width differs from rotary_dim")
    write = k_pages is not None
    if write:
        _need(slot_of, torch.int32, "slot_of")
        if k_pages.dtype is not qkv.dtype or v_pages.dtype is not qkv.dtype:
            raise KernelError("rope_kv_write: cache dtype differs from the projection dtype")
    _check(core().fsie_rope_kv_write(_ptr(qkv), ld, _ptr(positions), _ptr(cos_sin),
                                     cos_sin.shape[0], _ptr(slot_of), _ptr(k_pages), _ptr(v_pages),
                                     page_stride, page_size, tokens, heads, kv_heads, head_dim,
                                     rotary_dim, int(write), _tag(qkv.dtype), _ptr(error),
                                     _stream()), "rope_kv_write")


# ----------------------------------------------------------------------------- SwiGLU
def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i]."""
    _need(gate_up, None, "gate_up")
    _need(out, gate_up.dtype, "out")
    tokens, two_inter = gate_up.shape
    inter = two_inter // 2
    if two_inter != 2 * inter or out.numel() < tokens * inter:
        raise KernelError("swiglu: shapes do not fit")
    _check(core().fsie_swiglu(_ptr(gate_up), _ptr(out), tokens, inter, _tag(out.dtype), _stream()),
           "swiglu")
    return out


def place_tokens(ids: torch.Tensor, dst_and_row: torch.Tensor, chosen: torch.Tensor) -> None:
    """ids[dst[i]] = chosen[row[i]] for dst_and_row = [dst (n), row (n)], all int32 on the device."""
    for name, t in (("ids", ids), ("dst_and_row", dst_and_row), ("chosen", chosen)):
        _need(t, torch.int32, name)
    n = dst_and_row.numel() // 2
    _check(core().fsie_place_tokens(_ptr(ids), _ptr(dst_and_row), _ptr(dst_and_row[n:]),
                                    _ptr(chosen), n, _stream()), "place_tokens")


# --------------------------------------------------------------------- float32 product
GEMM_F32_KINDS = {"auto": 0, "rows": 1, "tiles": 2, "plain": 3}


def gemm_f32_rows_limit() -> int:
    """Rows of x up to which the float32 product takes its few-rows kernel."""
    return int(core().fsie_gemm_f32_rows_limit())


def gemm_f32(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
             out: Optional[torch.Tensor] = None, kind: str = "auto",
             rows_per_warp: int = 0) -> torch.Tensor:
    """out = x @ weight.T (+ bias), all float32, plain FFMA (no tensor-core mode).  `kind`
    names one of the three kernels (few rows, tiles, plain) instead of the choice by size;
    `rows_per_warp` (1, 2, 4) fixes how many rows of the weight a warp of the few-rows kernel
    owns instead of the choice by size."""
    _need(x, torch.float32, "x", contiguous=False)
    _need(weight, torch.float32, "weight")
    if x.dim() != 2 or x.stride(1) != 1:
        raise KernelError("gemm_f32: x must be 2-D with unit inner stride")
    m, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k:
        raise KernelError("gemm_f32: inner sizes differ")
    if bias is not None:
        _need(bias, torch.float32, "bias")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    _need(out, torch.float32, "out", contiguous=False)
    if out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError("gemm_f32: out must be [rows of x, rows of weight] with unit inner stride")
    _check(core().fsie_gemm_f32(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), m, n, k,
                                x.stride(0), out.stride(0), GEMM_F32_KINDS[kind], int(rows_per_warp),
                                _stream()),
           "gemm_f32")
    return out


# -------------------------------------------------------------------------- attention
def attention_rows_per_tile() -> int:
    return int(core().fsie_attn_generic_rows())


def attention_generic(q: torch.Tensor, q_ld: int, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      page_stride: int, page_size: int, block_tables: torch.Tensor,
                      tile_item: torch.Tensor, tile_row0: torch.Tensor, num_tiles: int,
                      item_qstart: torch.Tensor, item_qlen: torch.Tensor, item_pos0: torch.Tensor,
                      out: torch.Tensor, tokens: int, heads: int, kv_heads: int, head_dim: int,
                      window: int, scale: float, nsplit: int = 1,
                      part_o: Optional[torch.Tensor] = None,
                      part_ml: Optional[torch.Tensor] = None, rows16: bool = False,
                      merge: bool = True) -> torch.Tensor:
    """The 32-bit attention over tiles of up to 32 query rows (any storage, any head size up to
    256), or with `rows16` over tiles of up to 16 rows by the kernel for few rows (float storage,
    head sizes in steps of 4).  `merge=False` leaves the partial results of split key ranges
    unmerged: a step whose tiles go out in several launches merges with the last."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0)):
        _need(t, torch.int32, name)
    _need(q, None, "q", contiguous=False)
    _need(out, q.dtype, "out")
    if k_pages.dtype is not q.dtype or v_pages.dtype is not q.dtype:
        raise KernelError("attention: cache dtype differs from q")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention: split scratch is too small")
    _check(core().fsie_attn_tiles(_ptr(q), q_ld, _ptr(k_pages), _ptr(v_pages), page_stride,
                                  page_size, _ptr(block_tables), block_tables.stride(0),
                                  _ptr(tile_item), _ptr(tile_row0), num_tiles,
                                  _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0),
                                  _ptr(out), out.stride(0), _ptr(part_o), _ptr(part_ml), tokens,
                                  heads, kv_heads, head_dim, window, nsplit, float(scale),
                                  _tag(q.dtype), int(rows16), int(merge), _stream()),
           "attention_generic")
    return out


def attention_rows16_fits(dtype: torch.dtype, head_dim: int, page_stride: int) -> bool:
    """Whether the 32-bit attention kernel for tiles of up to 16 rows takes this cache."""
    return (dtype is torch.float32 and page_stride % 4 == 0
            and bool(core().fsie_attn_rows16_takes(int(head_dim))))


def attention_rows16_rows() -> int:
    return int(core().fsie_attn_rows16_rows())


_attn_mma = {}


def attn_mma(head_dim: int):
    """The tensor-core attention library for one head size, compiled at first use."""
    if head_dim not in _attn_mma:
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"tensor-core attention takes head sizes 16..256 in steps of 16, "
                              f"not {head_dim}")
        lib = build.load_library("attn_mma", (f"-DHEAD_DIM={head_dim}",))
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_attn_mma.argtypes = [i, p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                      i, i, i, i, i, i, f, p, i, p]
        lib.fsie_attn_mma.restype = i
        lib.fsie_attn_mma_rows.argtypes = [i]
        lib.fsie_attn_mma_rows.restype = i
        _attn_mma[head_dim] = lib
    return _attn_mma[head_dim]


ATTENTION_ROW_CLASSES = (16, 32, 64)      # rows per tile of row class 0, 1, 2


def attention_mma(row_class: int, q: torch.Tensor, q_ld: int, k_pages: torch.Tensor,
                  v_pages: torch.Tensor, page_stride: int, page_size: int,
                  block_tables: torch.Tensor, tile_item: torch.Tensor, tile_row0: torch.Tensor,
                  num_tiles: int, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                  item_pos0: torch.Tensor, out: torch.Tensor, tokens: int, heads: int,
                  kv_heads: int, head_dim: int, window: int, scale: float, nsplit: int = 1,
                  part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                  combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                  ) -> torch.Tensor:
    """bfloat16 attention of one row class (tiles of 16, 32 or 64 rows) on the tensor cores."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    if k_pages.dtype is not torch.bfloat16 or v_pages.dtype is not torch.bfloat16:
        raise KernelError("attention_mma: the cache must be bfloat16")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_mma: split scratch is too small")
        if combine_tokens is not None:
            _need(combine_tokens, torch.int32, "combine_tokens")
    _check(attn_mma(head_dim).fsie_attn_mma(
        row_class, _ptr(q), q_ld, _ptr(k_pages), _ptr(v_pages), page_stride, page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _stream()), "attention_mma")
    return out


_attn_tc = {}
ATTENTION_TC_PAGES = (8, 16, 32, 64, 128)
ATTENTION_TC_HEAD_DIMS = (64, 128)
ATTENTION_TC_ROWS = 256
ATTENTION_TC_DECODE_HEAD_DIMS = (128,)      # tiles of up to 16 rows: attention_tc_decode


def attn_tc(head_dim: int):
    """The tcgen05 attention library (prompt portions) for one head size (64 or 128)."""
    if head_dim not in _attn_tc:
        if head_dim not in ATTENTION_TC_HEAD_DIMS:
            raise KernelError(f"tcgen05 attention takes head sizes 64 and 128, not {head_dim}")
        lib = build.load_library("attn_tc", (f"-DHEAD_DIM={head_dim}",))
        i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_attn_tc_map_bytes.argtypes = []
        lib.fsie_attn_tc_pages_map.argtypes = [p, p, ll, i, i]
        lib.fsie_attn_tc.argtypes = [p, i, i, p, i, i, p, i, p, p, i, p, p, p, p, i, p, p,
                                     i, i, i, i, i, i, f, p, i, p, p]
        lib.fsie_attn_tc_decode.argtypes = lib.fsie_attn_tc.argtypes
        lib.fsie_attn_tc_decode_rows.argtypes = []
        for name in ("fsie_attn_tc_map_bytes", "fsie_attn_tc_pages_map", "fsie_attn_tc",
                     "fsie_attn_tc_decode", "fsie_attn_tc_decode_rows"):
            getattr(lib, name).restype = i
        _attn_tc[head_dim] = lib
    return _attn_tc[head_dim]


class PagesMap:
    """TMA descriptor of one cache group's pages [pages, entries, 2, kv_heads, slots, head_dim]
    (boxes of one page x 64 columns, 128-byte swizzle), as the tcgen05 attention kernels read it."""

    def __init__(self, pages: torch.Tensor, kind: str = "tc"):
        _need(pages, torch.bfloat16, "pages")
        num_pages, entries, two, kv_heads, page_size, head_dim = pages.shape
        if two != 2:
            raise KernelError("pages must be [pages, entries, 2, kv_heads, slots, head_dim]")
        self.pages, self.entries, self.page_size, self.head_dim = pages, entries, page_size, head_dim
        rows = num_pages * entries * 2 * kv_heads * page_size
        if kind != "tc":
            raise KernelError(f"PagesMap: unknown kind '{kind}'")
        lib = attn_tc(head_dim)
        size, encode = lib.fsie_attn_tc_map_bytes(), lib.fsie_attn_tc_pages_map
        self.buffer = ctypes.create_string_buffer(size + 64)
        offset = (-ctypes.addressof(self.buffer)) % 64
        self.ptr = ctypes.c_void_p(ctypes.addressof(self.buffer) + offset)
        _check(encode(self.ptr, _ptr(pages), rows, head_dim, page_size), "attention pages map")


def attention_tc(pages_map: PagesMap, entry: int, q: torch.Tensor, q_ld: int,
                 block_tables: torch.Tensor, tile_item: torch.Tensor, tile_row0: torch.Tensor,
                 num_tiles: int, item_qstart: torch.Tensor, item_qlen: torch.Tensor,
                 item_pos0: torch.Tensor, out: torch.Tensor, tokens: int, heads: int,
                 kv_heads: int, window: int, scale: float, error: torch.Tensor, nsplit: int = 1,
                 part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                 combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                 ) -> torch.Tensor:
    """bfloat16 attention of prompt portions (tiles of 128 query rows) with tcgen05.mma."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("error", error)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    head_dim = pages_map.head_dim
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_tc: split scratch is too small")
    _check(attn_tc(head_dim).fsie_attn_tc(
        pages_map.ptr, pages_map.entries, entry, _ptr(q), q_ld, pages_map.page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _ptr(error), _stream()), "attention_tc")
    return out


def attention_tc_decode(pages_map: PagesMap, entry: int, q: torch.Tensor, q_ld: int,
                        block_tables: torch.Tensor, tile_item: torch.Tensor,
                        tile_row0: torch.Tensor, num_tiles: int, item_qstart: torch.Tensor,
                        item_qlen: torch.Tensor, item_pos0: torch.Tensor, out: torch.Tensor,
                        tokens: int, heads: int, kv_heads: int, window: int, scale: float,
                        error: torch.Tensor, nsplit: int = 1,
                        part_o: Optional[torch.Tensor] = None,
                        part_ml: Optional[torch.Tensor] = None,
                        combine_tokens: Optional[torch.Tensor] = None, num_combine: int = 0
                        ) -> torch.Tensor:
    """bfloat16 attention of decoded tokens (tiles of up to 16 query rows, head size 128) with
    tcgen05.mma: the keys of a tile are the M side."""
    for name, t in (("block_tables", block_tables), ("tile_item", tile_item),
                    ("tile_row0", tile_row0), ("item_qstart", item_qstart),
                    ("item_qlen", item_qlen), ("item_pos0", item_pos0), ("error", error)):
        _need(t, torch.int32, name)
    _need(q, torch.bfloat16, "q", contiguous=False)
    _need(out, torch.bfloat16, "out")
    head_dim = pages_map.head_dim
    if head_dim not in ATTENTION_TC_DECODE_HEAD_DIMS:
        raise KernelError(f"attention_tc_decode takes head size 128, not {head_dim}")
    if nsplit > 1:
        _need(part_o, torch.float32, "part_o")
        _need(part_ml, torch.float32, "part_ml")
        if part_o.numel() < nsplit * tokens * heads * head_dim or \
                part_ml.numel() < nsplit * tokens * heads * 2:
            raise KernelError("attention_tc_decode: split scratch is too small")
    _check(attn_tc(head_dim).fsie_attn_tc_decode(
        pages_map.ptr, pages_map.entries, entry, _ptr(q), q_ld, pages_map.page_size,
        _ptr(block_tables), block_tables.stride(0), _ptr(tile_item), _ptr(tile_row0), num_tiles,
        _ptr(item_qstart), _ptr(item_qlen), _ptr(item_pos0), _ptr(out), out.stride(0),
        _ptr(part_o), _ptr(part_ml), tokens, heads, kv_heads, head_dim, window, nsplit,
        float(scale), _ptr(combine_tokens), num_combine, _ptr(error), _stream()),
        "attention_tc_decode")
    return out


# ------------------------------------------------- tcgen05 product for few tokens
_gemm_decode = None


def gemm_decode_lib():
    global _gemm_decode
    if _gemm_decode is None:
        lib = build.load_library("gemm_decode")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_tensor_map_bytes.argtypes = []
        lib.fsie_gemm_decode_weight_map.argtypes = [p, p, ll, ll, i]
        lib.fsie_gemm_decode.argtypes = [p, p, i, p, i, p, i, i, i, i, i, i, p, p]
        for name in ("fsie_tensor_map_bytes", "fsie_gemm_decode_weight_map", "fsie_gemm_decode"):
            getattr(lib, name).restype = i
        _gemm_decode = lib
    return _gemm_decode


GEMM_DECODE_MAX_TOKENS = 64


class DecodeWeight:
    """A bfloat16 weight [rows, K] prepared for `gemm_decode`: its TMA descriptor.
    For SwiGLU the weight holds the gate rows and then as many up rows."""

    def __init__(self, weight: torch.Tensor, swiglu: bool = False):
        _need(weight, torch.bfloat16, "weight")
        rows, k = weight.shape
        if k % 8:
            raise KernelError("gemm_decode: K must be a multiple of 8")
        if swiglu and rows % 2:
            raise KernelError("gemm_decode: a SwiGLU weight holds gate rows and as many up rows")
        lib = gemm_decode_lib()
        self.weight, self.swiglu, self.k = weight, swiglu, k
        self.n = rows // 2 if swiglu else rows
        self.map = ctypes.create_string_buffer(lib.fsie_tensor_map_bytes() + 64)
        offset = (-ctypes.addressof(self.map)) % 64
        self.map_ptr = ctypes.c_void_p(ctypes.addressof(self.map) + offset)
        _check(lib.fsie_gemm_decode_weight_map(self.map_ptr, _ptr(weight), rows, k,
                                               64 if swiglu else 128), "gemm_decode weight map")


def gemm_decode_splits(tiles: int, k: int, sm_count: int) -> int:
    """Blocks of a cluster that share the k range of one tile: enough to occupy the GPU."""
    splits = 1
    while splits < 8 and tiles * splits < sm_count and (k // 64) // (splits * 2) >= 4:
        splits *= 2
    return splits


def gemm_decode(weight: DecodeWeight, x: torch.Tensor, out: torch.Tensor,
                bias: Optional[torch.Tensor], error: torch.Tensor, splits: int = 1) -> torch.Tensor:
    """out[T, N] = x[T, K] @ w.T (+ bias), or silu(x @ gate.T) * (x @ up.T); T <= 64; out is
    bfloat16 or float32."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out")
    tokens, k = x.shape
    if k != weight.k or x.stride(1) != 1 or tokens > GEMM_DECODE_MAX_TOKENS:
        raise KernelError("gemm_decode: x does not fit the weight (or more than 64 tokens)")
    if out.shape[0] < tokens or out.shape[1] != weight.n or out.dtype not in (torch.bfloat16,
                                                                            torch.float32):
        raise KernelError("gemm_decode: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    _check(gemm_decode_lib().fsie_gemm_decode(
        weight.map_ptr, _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), tokens,
        weight.n, k, int(weight.swiglu), int(out.dtype is torch.float32), splits, _ptr(error),
        _stream()), "gemm_decode")
    return out


_gemm_skinny = None
GEMM_SKINNY_MAX_TOKENS = 16


def gemm_skinny_fits(tokens: int, k: int) -> bool:
    """Whether `gemm_skinny` takes a product of `tokens` rows over `k`."""
    return 0 < tokens <= GEMM_SKINNY_MAX_TOKENS and k % 32 == 0


def gemm_skinny_lib():
    global _gemm_skinny
    if _gemm_skinny is None:
        lib = build.load_library("gemm_skinny")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_gemm_skinny.argtypes = [p, p, ll, p, ll, p, i, i, i, i, p]
        lib.fsie_gemm_skinny.restype = i
        lib.fsie_gemm_skinny_qkv_rope.argtypes = [p, p, ll, p, ll, p, i, i, p, p, i, p, p, p, ll, i,
                                                  i, i, i, p, p]
        lib.fsie_gemm_skinny_qkv_rope.restype = i
        _gemm_skinny = lib
    return _gemm_skinny


def gemm_skinny_qkv_rope(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor,
                         bias: Optional[torch.Tensor], positions: torch.Tensor,
                         cos_sin: torch.Tensor, slot_of: Optional[torch.Tensor],
                         k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                         page_stride: int, page_size: int, heads: int, kv_heads: int,
                         head_dim: int, error: torch.Tensor) -> torch.Tensor:
    """The q, k, v product of up to 16 tokens with the rotation of q and k and the cache write in
    its epilogue: rotated queries into out[:, :heads * head_dim] (bfloat16; the key and value
    columns of `out` are not written), rotated keys and the values into the pages (not when
    k_pages is None).  The whole head is rotated: cos_sin is [positions, head_dim]."""
    lib = gemm_skinny_lib()
    _need(weight, torch.bfloat16, "weight")
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, torch.bfloat16, "out", contiguous=False)
    _need(positions, torch.int32, "positions")
    _need(cos_sin, torch.float32, "cos_sin")
    _need(error, torch.int32, "error")
    tokens, k = x.shape
    n = (heads + 2 * kv_heads) * head_dim
    if weight.shape != (n, k) or x.stride(1) != 1 or not gemm_skinny_fits(tokens, k):
        raise KernelError("gemm_skinny_qkv_rope: x does not fit the weight, or the sizes are beyond the kernel")
    if head_dim % 16 or cos_sin.shape[-1] != head_dim:
        raise KernelError("gemm_skinny_qkv_rope: needs a head size in steps of 16, rotated as a whole")
    if out.shape[0] != tokens or out.shape[1] < heads * head_dim or out.stride(1) != 1:
        raise KernelError("gemm_skinny_qkv_rope: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    if k_pages is not None:
        _need(slot_of, torch.int32, "slot_of")
        if k_pages.dtype is not torch.bfloat16 or v_pages.dtype is not torch.bfloat16:
            raise KernelError("gemm_skinny_qkv_rope: the cache must be bfloat16")
    _check(lib.fsie_gemm_skinny_qkv_rope(
        _ptr(weight), _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), tokens, k,
        _ptr(positions), _ptr(cos_sin), cos_sin.shape[0], _ptr(slot_of), _ptr(k_pages),
        _ptr(v_pages), page_stride, page_size, heads, kv_heads, head_dim, _ptr(error), _stream()),
        "gemm_skinny_qkv_rope")
    return out


def gemm_skinny(weight: torch.Tensor, x: torch.Tensor, out: torch.Tensor,
                bias: Optional[torch.Tensor]) -> torch.Tensor:
    """out[T, N] = x[T, K] @ weight.T (+ bias) for T <= 16: no pipeline to fill, every lane asks
    for its weights straight from global memory (for matrices so small that set-up would
    dominate).  out is bfloat16 or float32."""
    gemm_skinny_lib()
    _need(weight, torch.bfloat16, "weight")
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out", contiguous=False)
    tokens, k = x.shape
    n = weight.shape[0]
    if weight.shape[1] != k or x.stride(1) != 1 or not gemm_skinny_fits(tokens, k):
        raise KernelError("gemm_skinny: x does not fit the weight, or the sizes are beyond the kernel")
    if out.shape[0] != tokens or out.shape[1] != n or out.stride(1) != 1 or \
            out.dtype not in (torch.bfloat16, torch.float32):
        raise KernelError("gemm_skinny: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
    _check(_gemm_skinny.fsie_gemm_skinny(_ptr(weight), _ptr(x), x.stride(0), _ptr(out), out.stride(0),
                                         _ptr(bias), tokens, n, k, int(out.dtype is torch.float32),
                                         _stream()), "gemm_skinny")
    return out


_gemm_tiles = None


def gemm_tiles_lib():
    global _gemm_tiles
    if _gemm_tiles is None:
        lib = build.load_library("gemm_tiles")
        i, ll, p = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p
        lib.fsie_gemm_tiles_map_bytes.argtypes = []
        lib.fsie_gemm_tiles_weight_map.argtypes = [p, p, ll, ll]
        lib.fsie_gemm_tiles.argtypes = [p, p, ll, p, ll, p, i, i, i, i, i, i, p, ll, p, i, p, p]
        lib.fsie_gemm_tiles_workspace.argtypes = [i, i, i, i, i, ctypes.POINTER(ll), ctypes.POINTER(i)]
        lib.fsie_gemm_tiles_pairs.argtypes = []
        for name in ("fsie_gemm_tiles_map_bytes", "fsie_gemm_tiles_weight_map", "fsie_gemm_tiles",
                     "fsie_gemm_tiles_pairs", "fsie_gemm_tiles_workspace"):
            getattr(lib, name).restype = i
        pairs = lib.fsie_gemm_tiles_pairs()       # also sets the kernels up, outside any capture
        if pairs <= 0:
            raise KernelError(f"gemm_tiles: pairs of blocks cannot be launched here (code {pairs})")
        lib.pairs = pairs
        _gemm_tiles = lib
    return _gemm_tiles


def gemm_tiles_count(rows: int, n: int, swiglu: bool) -> int:
    """Output tiles of `gemm_tiles` for a product of `rows` tokens and `n` output features."""
    return -(-rows // 256) * -(-n // (128 if swiglu else 256))


class TiledWeight:
    """A bfloat16 weight [rows, K] prepared for `gemm_tiles`: its TMA descriptor (boxes of 128
    rows).  For SwiGLU the weight holds the gate rows and then as many up rows."""

    def __init__(self, weight: torch.Tensor, swiglu: bool = False):
        _need(weight, torch.bfloat16, "weight")
        rows, k = weight.shape
        if k % 8:
            raise KernelError("gemm_tiles: K must be a multiple of 8")
        if swiglu and rows % 2:
            raise KernelError("gemm_tiles: a SwiGLU weight holds gate rows and as many up rows")
        lib = gemm_tiles_lib()
        self.weight, self.swiglu, self.k = weight, swiglu, k
        self.n = rows // 2 if swiglu else rows
        self.map = ctypes.create_string_buffer(lib.fsie_gemm_tiles_map_bytes() + 64)
        offset = (-ctypes.addressof(self.map)) % 64
        self.map_ptr = ctypes.c_void_p(ctypes.addressof(self.map) + offset)
        _check(lib.fsie_gemm_tiles_weight_map(self.map_ptr, _ptr(weight), rows, k),
               "gemm_tiles weight map")


def gemm_tiles_workspace(rows: int, n: int, k: int, swiglu: bool, blocks: int) -> Tuple[int, int]:
    """(floats of workspace, ints of counters) with which `gemm_tiles` shares the tiles of a
    partial last round out among all pairs of blocks; (0, 0) where it has none to share."""
    floats, counters = ctypes.c_longlong(0), ctypes.c_int(0)
    code = gemm_tiles_lib().fsie_gemm_tiles_workspace(rows, n, k, int(swiglu), blocks,
                                                      ctypes.byref(floats), ctypes.byref(counters))
    if code != 0:
        raise KernelError(f"gemm_tiles_workspace failed with code {code}")
    return int(floats.value), int(counters.value)


def gemm_tiles(weight: TiledWeight, x: torch.Tensor, out: torch.Tensor,
               bias: Optional[torch.Tensor], error: torch.Tensor, blocks: int,
               workspace: Optional[torch.Tensor] = None,
               counters: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w.T (+ bias), or silu(x @ gate.T) * (x @ up.T), any M; out is
    bfloat16 (or float32 for the plain product).  `blocks`: size of the persistent grid.
    workspace (float32) and counters (int32, zero before the first call; every call leaves them
    zero) of the sizes `gemm_tiles_workspace` names let the kernel share out the tiles of a
    partial last round; without them every tile is summed by one pair of blocks."""
    _need(x, torch.bfloat16, "x", contiguous=False)
    _need(out, None, "out", contiguous=False)
    rows, k = x.shape
    if k != weight.k or x.stride(1) != 1 or x.stride(0) % 8:
        raise KernelError("gemm_tiles: x does not fit the weight (rows must start on 16 bytes)")
    if (out.shape[0] != rows or out.shape[1] != weight.n or out.stride(1) != 1
            or out.dtype not in (torch.bfloat16, torch.float32)
            or (weight.swiglu and out.dtype is torch.float32)):
        raise KernelError("gemm_tiles: out does not fit")
    if bias is not None:
        _need(bias, torch.bfloat16, "bias")
        if weight.swiglu or bias.numel() != weight.n:
            raise KernelError("gemm_tiles: bias does not fit")
    if workspace is not None:
        _need(workspace, torch.float32, "workspace")
        _need(counters, torch.int32, "counters")
    _check(gemm_tiles_lib().fsie_gemm_tiles(
        weight.map_ptr, _ptr(x), x.stride(0), _ptr(out), out.stride(0), _ptr(bias), rows,
        weight.n, k, int(weight.swiglu), int(out.dtype is torch.float32), blocks,
        _ptr(workspace), workspace.numel() if workspace is not None else 0,
        _ptr(counters), counters.numel() if counters is not None else 0, _ptr(error),
        _stream()), "gemm_tiles")
    return out


# --------------------------------------------------------------------------- sampling
ARGMAX_PARTS = 64      # blocks per row of the two-stage argmax
_argmax_scratch: Dict[int, torch.Tensor] = {}


def argmax(logits: torch.Tensor, out: torch.Tensor,
           scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = index of the largest logit of row r, ties to the smallest index.  A wide row is
    reduced by ARGMAX_PARTS blocks and a second small kernel (in `scratch`, float32, at least
    2 * rows * ARGMAX_PARTS elements; the module keeps one per device when none is given -
    pass your own inside a stream capture); a narrow row by one block."""
    _need(logits, torch.float32, "logits")
    _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    if vocab >= 8192:
        need = 2 * rows * ARGMAX_PARTS
        if scratch is None:
            key = logits.device.index or 0
            scratch = _argmax_scratch.get(key)
            if scratch is None or scratch.numel() < need:
                scratch = _argmax_scratch[key] = torch.empty(max(need, 1 << 16), dtype=torch.float32,
                                                             device=logits.device)
        _need(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError("argmax: scratch is too small")
        # enough blocks to fill the GPU several times over, each with more than a few loads per thread
        parts = max(4, min(ARGMAX_PARTS, 2048 // rows))
        _check(core().fsie_argmax_staged(_ptr(logits), rows, vocab, _ptr(out), _ptr(scratch),
                                         parts, _stream()), "argmax")
        return out
    _check(core().fsie_argmax(_ptr(logits), rows, vocab, _ptr(out), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits, torch.float32, "logits")
    _need(temperature, torch.float32, "temperature")
    _need(top_k, torch.int32, "top_k")
    _need(top_p, torch.float32, "top_p")
    _need(uniform, torch.float32, "uniform")
    _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    _check(core().fsie_sample(_ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k),
                              _ptr(top_p), _ptr(uniform), _ptr(out), _stream()), "sample")
    return out
