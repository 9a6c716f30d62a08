"""Grouped-query attention over the paged cache."""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..cache.manager import CacheNeed
from ..config.spec import PartSpec
from ..kernels import ops
from ..weights.tensor_spec import TensorSpec
from .base import LayerCache, Mixer, build_part, register_part


MAX_KEY_SPLITS = 64        # what the kernels that merge partial results take


def attention_splits(blocks: int, longest: int, sms: int, even_work: bool,
                     blocks_per_sm: int = 2, decode_slots: int = 3, decode_fixed: int = 270,
                     merge_cost: int = 350, tile_keys: int = 64, merge_step: int = 28) -> int:
    """Into how many key ranges to split each tile (at most 64, each at least 128 keys).

    Tiles of decoded tokens all have the same work, so the time is waves x (fixed cost of a
    block + the keys of a range) + the launch that merges the ranges.  A range is a whole number
    of the kernel's key tiles (`tile_keys`: 64 for the mma.sync kernel, 128 for the tcgen05 one),
    so the candidates are tiles per range, two at least, and the count is what covers the
    longest context with that many - 4,091 keys in ranges of two tiles are 32 ranges, none
    empty, where 29 or 31 ranges would have been three tiles each.  Costs are in keys (a
    64-key tile takes about 2 us): measured at context 4,096 the fixed cost of an mma.sync block
    is about 270 keys and three blocks fit on an SM (tcgen05 kernel for decoded tokens: 530
    keys, two blocks: `decode_fixed`, `decode_slots`); the merge costs `merge_cost` (5 us after
    the mma.sync kernel at batch 8, 17 us after the tcgen05 kernel with 200 requests) and
    `merge_step` more for every eight ranges beyond sixteen (it reads eight at a time), less
    for eight or fewer.  Chosen this way a decode step at contexts of 4,090 takes 2.86 instead
    of 2.91 ms at batch 1, 3.00 instead of 3.05 ms at batch 4, and as before at batch 8.
    Tiles of a prompt have uneven work and are split only when there are fewer of them than
    block slots (`blocks_per_sm` per SM; the tcgen05 kernel has one, and its partial results
    cost more than a little idling, so it splits only to fill slots that would stay empty)."""
    if not even_work:
        slots = blocks_per_sm * sms
        if blocks >= slots:
            return 1
        wanted = slots // blocks if blocks_per_sm == 1 else -(-slots // blocks)
        return max(1, min(wanted, longest // 128, MAX_KEY_SPLITS))
    slots = decode_slots * sms
    best, best_cost = 1, -(-blocks // slots) * (decode_fixed + longest)
    least = max(2, -(-128 // tile_keys))                # tiles of a range: 128 keys at least
    for tiles in range(-(-longest // tile_keys) - 1, least - 1, -1):
        n = -(-longest // (tiles * tile_keys))
        if n < 2 or n > MAX_KEY_SPLITS:
            continue
        cost = -(-blocks * n // slots) * (decode_fixed + tiles * tile_keys) \
            + merge_cost + merge_step * (-(-n // 8) - 2)
        if cost < best_cost:
            best, best_cost = n, cost
    return best


@register_part("mixer", "gqa_attention")
class GqaAttention(Mixer):
    """q, k, v projections (optional bias), position encoding on q and k, causal attention of
    each query head over the kv head of its group (head h uses kv head h // group), output
    projection without bias.  Scale 1/sqrt(head_dim); keys 0..position inclusive, or the last
    `window` of them.  Reference: src/model/model.cpp:111-132, src/model/nn.cpp:151-226.

    The three projections are one matrix product over the concatenated weight
    [q_width + 2 kv_width, hidden], made at bind.
    """

    capturable = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, qkv_bias: bool, position: PartSpec, window: int = 0):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is beyond the attention kernels (256)")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.qkv_bias, self.window = head_dim, bool(qkv_bias), int(window)
        self.q_width, self.kv_width = num_heads * head_dim, num_kv_heads * head_dim
        self.position = build_part("position", position, prefix)
        if self.position.rotary_dim > head_dim:
            raise ValueError("rotary_dim exceeds head_dim")
        self.scale = 1.0 / math.sqrt(head_dim)
        self.w_qkv = self.b_qkv = self.w_o = None

    def tensor_specs(self) -> List[TensorSpec]:
        p, h = self.prefix, self.hidden_size
        specs = [TensorSpec(p + "q_proj.weight", (self.q_width, h)),
                 TensorSpec(p + "k_proj.weight", (self.kv_width, h)),
                 TensorSpec(p + "v_proj.weight", (self.kv_width, h)),
                 TensorSpec(p + "o_proj.weight", (h, self.q_width))]
        if self.qkv_bias:
            specs += [TensorSpec(p + "q_proj.bias", (self.q_width,)),
                      TensorSpec(p + "k_proj.bias", (self.kv_width,)),
                      TensorSpec(p + "v_proj.bias", (self.kv_width,))]
        return specs + self.position.tensor_specs()

    def cache_need(self) -> Optional[CacheNeed]:
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def bind(self, tensors: Dict[str, torch.Tensor], runtime) -> None:
        self.runtime = runtime
        p = self.prefix
        self.w_qkv = torch.cat([tensors[p + f"{n}_proj.weight"] for n in "qkv"]).contiguous()
        self.b_qkv = (torch.cat([tensors[p + f"{n}_proj.bias"] for n in "qkv"]).contiguous()
                      if self.qkv_bias else None)
        self.w_o = tensors[p + "o_proj.weight"].contiguous()
        runtime.prepare_weight(self.w_qkv)
        runtime.prepare_weight(self.w_o)
        self.position.bind(tensors, runtime)

    def forward(self, ctx, y: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        rt = self.runtime
        tokens = y.shape[0]
        group = ctx.groups[cache.group]
        rope = (ctx.positions, self.position.table,
                group.slot_of if cache.writes else None,
                cache.k_pages if cache.writes else None,
                cache.v_pages if cache.writes else None,
                cache.page_stride, group.page_size, self.num_heads, self.num_kv_heads,
                self.head_dim, self.position.rotary_dim)
        qkv = rt.qkv_rotated_and_cached(y, self.w_qkv, self.b_qkv, *rope)
        if qkv is None:
            qkv = rt.linear(y, self.w_qkv, self.b_qkv, "qkv")
            ops.rope_kv_write(qkv, *rope, ctx.error)
        # working memory shared by all attention layers of a model: a layer's q, k, v and its
        # attention output are dead when the next attention layer runs
        out = rt.buffer("attention.out", tokens, self.q_width, qkv.dtype)
        self._attend(ctx, qkv, group, cache, out)
        return rt.linear(out, self.w_o, None, "attention.o")

    def _attend(self, ctx, qkv: torch.Tensor, group, cache: LayerCache, out: torch.Tensor) -> None:
        """Attention of the step's tokens over the pages.  Work is cut into tiles of query
        rows, a row being a (token, head of the group) pair; a tile's key range is split
        over several blocks when the batch alone would not fill the GPU.  bfloat16 runs on
        the tensor cores (one launch per row class present in the batch: single decoded
        tokens, short portions, long portions); float32 runs the 32-bit kernel."""
        tokens = qkv.shape[0]
        group_size = self.num_heads // self.num_kv_heads
        sms = ctx.runtime.sm_count

        def splits(blocks: int, longest: int, even_work: bool = False, blocks_per_sm: int = 2) -> int:
            return attention_splits(blocks, longest, sms, even_work, blocks_per_sm)

        common = (cache.k_pages, cache.v_pages, cache.page_stride, group.page_size,
                  group.block_tables)
        if qkv.dtype is torch.bfloat16 and self.head_dim % 16 == 0:
            # prompt portions (the last row class) run on tcgen05 in tiles of 256 rows where the
            # head size and the page size allow it
            pages_map = ctx.runtime.pages_map(cache.pages) if cache.pages is not None else None
            class_rows = ops.ATTENTION_ROW_CLASSES
            if pages_map is not None:
                class_rows = class_rows[:-1] + (ops.ATTENTION_TC_ROWS,)
            for row_class, tiles, class_tokens, count, longest in \
                    ctx.attention_row_classes(group_size, class_rows):
                on_tcgen05 = pages_map is not None and row_class == len(class_rows) - 1
                # decoded tokens: from about 1.6 blocks per SM before any split the tcgen05 kernel
                # (a tile's keys as the M side) is ahead of the mma.sync one, below that behind
                decode_tcgen05 = (pages_map is not None and row_class == 0
                                  and self.head_dim in ops.ATTENTION_TC_DECODE_HEAD_DIMS
                                  and tiles.count * self.num_kv_heads
                                  >= ctx.runtime.decode_tcgen05_min_blocks)
                if decode_tcgen05:
                    nsplit = attention_splits(tiles.count * self.num_kv_heads, longest, sms, True,
                                              decode_slots=2, decode_fixed=530, merge_cost=1300,
                                              tile_keys=128)
                else:
                    nsplit = splits(tiles.count * self.num_kv_heads, longest, row_class == 0,
                                    1 if on_tcgen05 else 2)
                part_o = part_ml = None
                if nsplit > 1:
                    part_o = ctx.scratch("attention.part_o", nsplit * tokens * self.q_width)
                    part_ml = ctx.scratch("attention.part_ml", nsplit * tokens * self.num_heads * 2)
                if decode_tcgen05:
                    ops.attention_tc_decode(pages_map, cache.entry_index, qkv, qkv.stride(0),
                                            group.block_tables, tiles.item, tiles.row0,
                                            tiles.count, ctx.item_qstart, ctx.item_qlen,
                                            ctx.item_pos0, out, tokens, self.num_heads,
                                            self.num_kv_heads, self.window, self.scale,
                                            ctx.error, nsplit, part_o, part_ml, class_tokens,
                                            count)
                    continue
                if on_tcgen05:
                    ops.attention_tc(pages_map, cache.entry_index, qkv, qkv.stride(0),
                                     group.block_tables, tiles.item, tiles.row0, tiles.count,
                                     ctx.item_qstart, ctx.item_qlen, ctx.item_pos0, out, tokens,
                                     self.num_heads, self.num_kv_heads, self.window, self.scale,
                                     ctx.error, nsplit, part_o, part_ml, class_tokens, count)
                    continue
                ops.attention_mma(row_class, qkv, qkv.stride(0), *common, tiles.item, tiles.row0,
                                  tiles.count, ctx.item_qstart, ctx.item_qlen, ctx.item_pos0, out,
                                  tokens, self.num_heads, self.num_kv_heads, self.head_dim,
                                  self.window, self.scale, nsplit, part_o, part_ml,
                                  class_tokens, count)
            return
        # 32-bit arithmetic on CUDA cores: requests of up to 16 query rows (decoded tokens, short
        # portions) take the kernel in which every warp works on such a tile, the others the
        # kernel for tiles of 32 rows; one choice of key splits and one merge for both
        if ops.attention_rows16_fits(qkv.dtype, self.head_dim, cache.page_stride):
            classes = ctx.attention_row_classes(group_size, (ops.attention_rows16_rows(),
                                                             ops.attention_rows_per_tile()))
            launches = [(row_class == 0, tiles) for row_class, tiles, _, _, _ in classes]
        else:
            launches = [(False, ctx.attention_tiles(group_size, ops.attention_rows_per_tile()))]
        blocks = sum(tiles.count for _, tiles in launches) * self.num_kv_heads
        decoding = all(rows16 for rows16, _ in launches)
        nsplit = splits(blocks, ctx.max_context, even_work=decoding, blocks_per_sm=2)
        part_o = part_ml = None
        if nsplit > 1:
            part_o = ctx.scratch("attention.part_o", nsplit * tokens * self.q_width)
            part_ml = ctx.scratch("attention.part_ml", nsplit * tokens * self.num_heads * 2)
        for index, (rows16, tiles) in enumerate(launches):
            ops.attention_generic(qkv, qkv.stride(0), *common, tiles.item, tiles.row0, tiles.count,
                                  ctx.item_qstart, ctx.item_qlen, ctx.item_pos0, out, tokens,
                                  self.num_heads, self.num_kv_heads, self.head_dim, self.window,
                                  self.scale, nsplit, part_o, part_ml, rows16=rows16,
                                  merge=index == len(launches) - 1)
