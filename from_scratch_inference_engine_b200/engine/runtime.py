"""What the parts get from the engine: device, compute dtype, matrix products, shared tables."""

from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn.functional as F

from ..kernels import ops

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
          "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype '{name}' (bfloat16 or float32)") from None


class Runtime:
    """Device and precision of one engine, and which kernel multiplies which step.

    bfloat16: steps of few tokens take the engine's few-token products (tcgen05 for the large
    matrices up to 32 tokens, a set-up-free mma.sync kernel for the small ones up to 16), steps with enough
    256 x 256 output tiles to fill the GPU take the engine's tiled tcgen05 product, and the
    steps in between take the library product (cuBLAS through torch, bf16 operands, 32-bit
    accumulation), as the reference engine uses the library for its products
    (src/cuda/device.cu:322-357).  float32: every product by the engine's own FFMA kernel,
    no tensor-core mode.  Everything that is not a plain matrix product is a kernel of
    this package in both modes.
    """

    def __init__(self, device="cuda:0", dtype=torch.bfloat16, max_positions: int = 0,
                 few_token_min_elements: int = 32 * 1024 * 1024, products: str = "own",
                 tiled_min_tiles: Optional[int] = None,
                 decode_tcgen05_min_blocks: Optional[int] = None, few_token_limit: int = 32,
                 share_tiles: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: this engine has no CPU path")
        self.device = torch.device(device)
        self.dtype = parse_dtype(dtype)
        self.max_positions = int(max_positions)
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self._tables: Dict[object, torch.Tensor] = {}
        self._buffers: Dict[object, torch.Tensor] = {}
        self._f32_out: Optional[bool] = None
        # device-side error flag that kernels set when they refuse an input or give up a wait
        self.error = torch.zeros(1, dtype=torch.int32, device=self.device)
        # weights prepared for the tcgen05 product of steps with few tokens, by storage address
        self._few_token_weights: Dict[int, ops.DecodeWeight] = {}
        if not 1 <= few_token_limit <= ops.GEMM_DECODE_MAX_TOKENS:
            raise ValueError(f"few_token_limit must lie in 1..{ops.GEMM_DECODE_MAX_TOKENS}")
        # steps of up to this many tokens take that product (32: inside a decode step of 24 tokens
        # it measured 2.5 % ahead of the library, at 32 level with it, at 64 4 % behind; up to 64 is
        # possible and is what measurements of that choice set)
        self.few_token_limit = int(few_token_limit)
        self.few_token_limit_fused = int(few_token_limit)    # ... the same with the fused SwiGLU
        self.few_token_min_elements = few_token_min_elements   # ... for matrices at least this large
        # "own": steps of many tokens take the tiled tcgen05 product (fused bias / SwiGLU) where
        # its tiles fill the GPU; "library": they take the library product
        if products not in ("own", "library"):
            raise ValueError("products must be 'own' or 'library'")
        self.products = products
        self.tiled_min_tiles = tiled_min_tiles       # None: as many tiles as pairs of SMs run at once
        # decode steps of up to 64 tokens that the few-token products do not take keep the library
        # product: alone the tiled kernel ties with it there, inside a captured decode step it
        # measured 6 % slower (batch 64); a test that forces the tiled product gets it for every step
        # that is beyond the set-up-free kernel
        self.tiled_min_rows = 65 if tiled_min_tiles is None else ops.GEMM_SKINNY_MAX_TOKENS + 1
        # matrices that may take the tiled product: storage address -> (weight, swiglu) until a step
        # qualifies, then its descriptor (made, and the kernel library compiled, only then)
        self._tiled_weights: Dict[int, object] = {}
        # decoded tokens take the tcgen05 attention kernel when their (request, kv head) pairs
        # number at least this many (None: 1.6 per SM - measured at 4,096-token contexts: behind
        # the mma.sync kernel by 9 % at 192 pairs on 148 SMs, ahead by 15 % at 256)
        self.decode_tcgen05_min_blocks = (int(1.6 * self.sm_count) if decode_tcgen05_min_blocks is None
                                          else int(decode_tcgen05_min_blocks))
        # steps of few tokens rotate q, k and write k, v in the q, k, v product's epilogue
        self.fused_qkv_rope = True
        # the tiled product shares a partial last round of tiles out among all pairs of blocks
        self.share_tiles = bool(share_tiles)
        # its counters (eight per shared tile, fewer tiles than pairs of SMs): made now, so that a
        # step that is being captured into a graph never allocates them
        self._tiles_counters = torch.zeros(8 * max(self.sm_count // 2, 1) + 8, dtype=torch.int32,
                                           device=self.device)
        # bf16 products must accumulate in 32-bit all the way
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

    def buffer(self, tag: Optional[str], rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """[rows, cols] of working memory for one operation's result.

        With a `tag` the memory is kept and handed out again to whoever asks under the same tag
        (grown when more is needed): a step's operations run one after the other on one stream,
        so a result may live in the same place as the result of the same operation of the
        layer before it, and nothing is asked of the allocator per operation.  The caller
        guarantees that the earlier result under the tag is dead when it asks again.  Without a
        tag, and while a CUDA graph is being captured (whose memory must be the graph's own),
        the memory is fresh."""
        if tag is None or torch.cuda.is_current_stream_capturing():
            return torch.empty((rows, cols), dtype=dtype, device=self.device)
        key = (tag, dtype)
        have = self._buffers.get(key)
        if have is None or have.numel() < rows * cols:
            have = torch.empty(max(rows * cols, 1), dtype=dtype, device=self.device)
            self._buffers[key] = have
        return have[:rows * cols].view(rows, cols)

    def reset_after_fault(self) -> None:
        """After a kernel has set the error flag: a tiled product that gave up may have left the
        counters of its shared tiles above zero, where the next launch expects zero."""
        self._tiles_counters.zero_()

    def pages_map(self, pages: torch.Tensor):
        """TMA descriptor of a cache group's page tensor (made once per tensor), or None when
        the tcgen05 attention kernels do not take its head size or page size."""
        key = ("pages_map", pages.data_ptr())
        if key not in self._tables:
            head_dim, page_size = pages.shape[-1], pages.shape[-2]
            ok = (pages.dtype is torch.bfloat16 and head_dim in ops.ATTENTION_TC_HEAD_DIMS
                  and page_size in ops.ATTENTION_TC_PAGES)
            self._tables[key] = ops.PagesMap(pages, "tc") if ok else None
        return self._tables[key]

    def shared_table(self, key, make: Callable[[], torch.Tensor]) -> torch.Tensor:
        """A constant table on the device, built once per distinct key."""
        if key not in self._tables:
            self._tables[key] = make().to(self.device).contiguous()
        return self._tables[key]

    def prepare_weight(self, weight: torch.Tensor, swiglu: bool = False) -> None:
        """Called by a part at bind for a matrix it will multiply activations with.  Large
        bfloat16 matrices get a TMA descriptor for the tcgen05 product that steps of few
        tokens use (the library product is kept where it measured faster: small matrices)."""
        if self.dtype is not torch.bfloat16 or weight.dtype is not torch.bfloat16:
            return
        rows, k = weight.shape
        if k % 8 or (swiglu and rows % 2):
            return
        if self.products == "own":
            self._tiled_weights[weight.data_ptr()] = (weight, swiglu)
        if rows * k >= self.few_token_min_elements:
            self._few_token_weights[weight.data_ptr()] = ops.DecodeWeight(weight, swiglu)

    def _tiled(self, x: torch.Tensor, weight: torch.Tensor) -> Optional["ops.TiledWeight"]:
        """The weight's descriptor for the tiled product when this step is one for it: more
        tokens than the few-token product takes, and enough tiles to give every pair of SMs
        one (with fewer, the library's smaller tiles or split k stream the weight faster)."""
        prepared = self._tiled_weights.get(weight.data_ptr())
        if prepared is None or x.shape[0] < self.tiled_min_rows or x.stride(0) % 8 or x.data_ptr() % 16:
            return None
        known = isinstance(prepared, ops.TiledWeight)
        swiglu = prepared.swiglu if known else prepared[1]
        n = prepared.n if known else prepared[0].shape[0] // (2 if swiglu else 1)
        least = self.sm_count // 2 if self.tiled_min_tiles is None else self.tiled_min_tiles
        if ops.gemm_tiles_count(x.shape[0], n, swiglu) < least:
            return None
        if not known:
            prepared = self._tiled_weights[weight.data_ptr()] = ops.TiledWeight(prepared[0], swiglu)
        return prepared

    def _tiled_product(self, prepared, x, bias, out_dtype, tag=None) -> torch.Tensor:
        out = self.buffer(tag, x.shape[0], prepared.n, out_dtype)
        # where the tiles leave a partial last round, the kernel shares that round's tiles out among
        # all pairs of blocks and needs room for their partial sums (kept, grown when more is needed)
        floats, counters = ops.gemm_tiles_workspace(x.shape[0], prepared.n, prepared.k, prepared.swiglu,
                                                    self.sm_count) if self.share_tiles else (0, 0)
        workspace = None
        if floats and counters <= self._tiles_counters.numel():
            workspace = self.buffer("gemm_tiles.parts", 1, floats, torch.float32).view(-1)
        return ops.gemm_tiles(prepared, x, out, bias, self.error, self.sm_count, workspace,
                              self._tiles_counters if workspace is not None else None)

    def _few_tokens(self, x: torch.Tensor, weight: torch.Tensor) -> Optional["ops.DecodeWeight"]:
        if x.shape[0] > max(self.few_token_limit, self.few_token_limit_fused) or x.stride(0) % 8:
            return None
        prepared = self._few_token_weights.get(weight.data_ptr())
        if prepared is None:
            return None
        limit = self.few_token_limit_fused if prepared.swiglu else self.few_token_limit
        return prepared if x.shape[0] <= limit else None

    def _few_token_product(self, prepared, x, bias, out_dtype, tag=None) -> torch.Tensor:
        out = self.buffer(tag, x.shape[0], prepared.n, out_dtype)
        tiles = -(-prepared.n // (64 if prepared.swiglu else 128))
        splits = ops.gemm_decode_splits(tiles, prepared.k, self.sm_count)
        return ops.gemm_decode(prepared, x, out, bias, self.error, splits)

    def linear(self, x: torch.Tensor, weight: torch.Tensor,
               bias: Optional[torch.Tensor], tag: Optional[str] = None) -> torch.Tensor:
        """x @ weight.T (+ bias) in the compute dtype.  `tag`: see `buffer` (the result may then
        live where the last result under that tag lived)."""
        if self.dtype is torch.float32:
            return ops.gemm_f32(x, weight, bias, self.buffer(tag, x.shape[0], weight.shape[0], torch.float32))
        prepared = self._few_tokens(x, weight)
        if prepared is not None and not prepared.swiglu:
            return self._few_token_product(prepared, x, bias, torch.bfloat16, tag)
        tiled = self._tiled(x, weight)
        if tiled is not None and not tiled.swiglu:
            return self._tiled_product(tiled, x, bias, torch.bfloat16, tag)
        if self._skinny(x, weight):
            return ops.gemm_skinny(weight, x, self.buffer(tag, x.shape[0], weight.shape[0], torch.bfloat16), bias)
        if tag is None or x.dtype is not torch.bfloat16:
            return F.linear(x, weight, bias)
        out = self.buffer(tag, x.shape[0], weight.shape[0], torch.bfloat16)
        if bias is None:
            return torch.mm(x, weight.t(), out=out)
        return torch.addmm(bias, x, weight.t(), out=out)

    def _skinny(self, x: torch.Tensor, weight: torch.Tensor) -> bool:
        """Whether the set-up-free product takes this step: few tokens, and a matrix that the
        tcgen05 few-token product was not prepared for (a small one)."""
        return (self.products == "own" and ops.gemm_skinny_fits(x.shape[0], x.shape[1])
                and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                and weight.dtype is torch.bfloat16 and weight.is_contiguous())

    def qkv_rotated_and_cached(self, x: torch.Tensor, weight: torch.Tensor,
                               bias: Optional[torch.Tensor], positions: torch.Tensor,
                               cos_sin: torch.Tensor, slot_of, k_pages, v_pages, page_stride: int,
                               page_size: int, heads: int, kv_heads: int, head_dim: int,
                               rotary_dim: int) -> Optional[torch.Tensor]:
        """The q, k, v product of an attention layer together with the rotation of q and k and
        the write of k and v into the pages, where one kernel does all three (steps of few
        tokens against a matrix that the set-up-free product takes, whole heads rotated);
        else None, and the caller runs the product and `ops.rope_kv_write` one after the other.
        Returns [tokens, q + k + v width] of which only the query columns are filled."""
        if not (self.dtype is torch.bfloat16 and self.fused_qkv_rope and rotary_dim == head_dim
                and head_dim % 16 == 0 and self._few_tokens(x, weight) is None
                and self._skinny(x, weight)
                and weight.shape[0] == (heads + 2 * kv_heads) * head_dim):
            return None
        out = self.buffer("qkv", x.shape[0], weight.shape[0], torch.bfloat16)
        return ops.gemm_skinny_qkv_rope(weight, x, out, bias, positions, cos_sin, slot_of, k_pages,
                                        v_pages, page_stride, page_size, heads, kv_heads, head_dim,
                                        self.error)

    def linear_swiglu(self, x: torch.Tensor, gate_up: torch.Tensor,
                      tag: Optional[str] = None) -> torch.Tensor:
        """silu(x @ gate.T) * (x @ up.T) for the stacked weight [gate rows; up rows]: one fused
        kernel for steps of few tokens, else the library product and the SwiGLU kernel."""
        prepared = self._few_tokens(x, gate_up) if self.dtype is torch.bfloat16 else None
        if prepared is not None and prepared.swiglu:
            return self._few_token_product(prepared, x, None, torch.bfloat16, tag)
        tiled = self._tiled(x, gate_up) if self.dtype is torch.bfloat16 else None
        if tiled is not None and tiled.swiglu:
            return self._tiled_product(tiled, x, None, torch.bfloat16, tag)
        wide = None if tag is None else tag + ".gate_up"
        both = self.linear(x, gate_up, None, wide) if prepared is None else F.linear(x, gate_up)
        act = self.buffer(tag, x.shape[0], gate_up.shape[0] // 2, both.dtype)
        return ops.swiglu(both, act)

    def linear_f32_out(self, x: torch.Tensor, weight: torch.Tensor,
                       tag: Optional[str] = None) -> torch.Tensor:
        """x @ weight.T with a float32 result (the logits)."""
        if self.dtype is torch.float32:
            return ops.gemm_f32(x, weight, None, self.buffer(tag, x.shape[0], weight.shape[0], torch.float32))
        prepared = self._few_tokens(x, weight)
        if prepared is not None and not prepared.swiglu:
            return self._few_token_product(prepared, x, None, torch.float32, tag)
        tiled = self._tiled(x, weight)
        if tiled is not None and not tiled.swiglu:
            return self._tiled_product(tiled, x, None, torch.float32, tag)
        if self._skinny(x, weight):
            return ops.gemm_skinny(weight, x, self.buffer(tag, x.shape[0], weight.shape[0], torch.float32), None)
        if self._f32_out is None:
            try:
                torch.mm(x[:1], weight[:8].t(), out_dtype=torch.float32)
                self._f32_out = True
            except (TypeError, RuntimeError):
                self._f32_out = False
        if self._f32_out:
            return torch.mm(x, weight.t(), out_dtype=torch.float32)
        # this torch cannot give a float32 result from bfloat16 operands: rounding the logits
        # to bfloat16 on the way would break the rule that logits are 32-bit, so the rows go
        # through the engine's own products sixteen at a time where those take the matrix,
        # else through a float32 product over slabs of the matrix (slow, and said so once)
        part = x[:self.few_token_limit]
        if x.shape[0] > self.few_token_limit and (
                self._few_tokens(part, weight) is not None or self._skinny(part, weight)):
            return torch.cat([self.linear_f32_out(x[r:r + self.few_token_limit], weight)
                              for r in range(0, x.shape[0], self.few_token_limit)])
        if not getattr(self, "_warned_f32_out", False):
            self._warned_f32_out = True
            import warnings
            warnings.warn("torch.mm(out_dtype=float32) is not available: float32 logits are "
                          "computed by a float32 product over slabs of the output head")
        xf = x.float()
        return torch.cat([xf @ weight[r:r + 8192].float().t()
                          for r in range(0, weight.shape[0], 8192)], dim=1)
