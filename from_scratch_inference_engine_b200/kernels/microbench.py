"""Times single kernels at given sizes and prints achieved GB/s or TFLOP/s.

    python -m from_scratch_inference_engine_b200.kernels.microbench KERNEL [options]

KERNEL: attention_decode, attention_prefill, add_rmsnorm, rope_kv_write, swiglu, argmax,
sample, linear (the library product as the engine calls it), gemm_f32, gemm_decode,
gemm_decode_swiglu, gemm_tiles, gemm_tiles_swiglu (the engine's own tcgen05 products).

Each kernel is timed with CUDA events over --iters launches after --warmup launches; between
launches a buffer larger than L2 is read so that inputs come from HBM (read, not written:
dirty lines would be written back during the timed kernel).  One JSON line
per run: time, algorithmic bytes and flops, achieved rates and their fraction of the peaks
in MEASURED_PEAKS.json at the repository root (or of 6,650 GB/s and 1,590 TFLOP/s when that
file is absent).  The same command under `ncu` profiles exactly this kernel at this size.
"""

from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch

from . import ops

ROOT = Path(__file__).resolve().parents[2]


def peaks():
    values = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                value = data.get(key) if isinstance(data, dict) else None
                if isinstance(value, dict):        # a record with the figure inside
                    value = next((value[k] for k in ("value", "median", "mean") if k in value), None)
                if isinstance(value, (int, float)) and value > 0:
                    values[key] = float(value)
                    values["source"] = "measured"
        except (OSError, ValueError, TypeError):
            pass
    return values


class Timer:
    def __init__(self, warmup: int, iters: int, flush: bool = True):
        self.warmup, self.iters = warmup, iters
        self.flush = torch.zeros(256 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.view(torch.int32).sum()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end))
        times.sort()
        return times[len(times) // 2]          # median, ms


def paged_inputs(batch, new, past, heads, kv_heads, hd, page, dtype):
    """Random pages, shuffled block tables and queries for `batch` requests with `past`
    cached tokens and `new` tokens each."""
    g = torch.Generator(device="cuda").manual_seed(0)
    total = past + new
    blocks = -(-total // page)
    pages = torch.randn((batch * blocks + 1, 1, 2, kv_heads, page, hd), generator=g, device="cuda",
                        dtype=torch.float32).to(dtype)
    order = torch.randperm(batch * blocks, generator=g, device="cuda").to(torch.int32)
    tables = order.view(batch, blocks).contiguous()
    q = torch.randn((batch * new, (heads + 2 * kv_heads) * hd), generator=g, device="cuda",
                    dtype=torch.float32).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    return pages, tables, q, i32([i * new for i in range(batch)]), i32([new] * batch), \
        i32([past] * batch)


def run_attention(args, timer, decode: bool):
    heads, kv_heads, hd, page = args.heads, args.kv_heads, args.head_dim, args.page
    new = 1 if decode else args.tokens
    past = args.context - new
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    pages, tables, q, qstart, qlen, pos0 = paged_inputs(args.batch, new, past, heads, kv_heads, hd,
                                                        page, dtype)
    group = heads // kv_heads
    tokens = args.batch * new
    out = torch.empty((tokens, heads * hd), dtype=dtype, device="cuda")
    rows = new * group
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    if dtype is torch.bfloat16:
        row_class = next((c for c, r in enumerate(ops.ATTENTION_ROW_CLASSES) if rows <= r), 2)
        per_tile = ops.ATTENTION_ROW_CLASSES[row_class]
        if args.variant == "tc" and row_class == 2:
            per_tile = ops.ATTENTION_TC_ROWS
    else:
        rows16 = args.variant == "rows16" and rows <= ops.attention_rows16_rows()
        row_class, per_tile = -1, ops.attention_rows16_rows() if rows16 else ops.attention_rows_per_tile()
    tile_item, tile_row0 = [], []
    for i in range(args.batch):
        for r0 in range(0, rows, per_tile):
            tile_item.append(i)
            tile_row0.append(r0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    # as the engine lists them: the tiles that see the most keys first
    by_keys = sorted(range(len(tile_item)), key=lambda n: -(past + (min(tile_row0[n] + per_tile, rows) - 1) // group))
    tile_item, tile_row0 = [tile_item[n] for n in by_keys], [tile_row0[n] for n in by_keys]
    tile_item, tile_row0 = i32(tile_item), i32(tile_row0)
    nsplit = args.nsplit
    if nsplit <= 0:
        from ..parts.attention import attention_splits
        nsplit = attention_splits(tile_item.numel() * kv_heads, args.context, sms, decode,
                                  1 if args.variant == "tc" and row_class == 2 else 2)
    part_o = torch.empty(max(1, nsplit * tokens * heads * hd), device="cuda")
    part_ml = torch.empty(max(1, nsplit * tokens * heads * 2), device="cuda")
    scale = 1.0 / math.sqrt(hd)

    use_tc = args.variant == "tc" and row_class == 2
    use_tcd = args.variant == "tc" and row_class == 0 and hd in ops.ATTENTION_TC_DECODE_HEAD_DIMS
    if use_tc or use_tcd:
        pages_map = ops.PagesMap(pages, "tc")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")

    def launch():
        if use_tcd:
            ops.attention_tc_decode(pages_map, 0, q, q.stride(0), tables, tile_item, tile_row0,
                                    tile_item.numel(), qstart, qlen, pos0, out, tokens, heads,
                                    kv_heads, 0, scale, error, nsplit, part_o, part_ml, None, 0)
        elif use_tc:
            ops.attention_tc(pages_map, 0, q, q.stride(0), tables, tile_item, tile_row0,
                             tile_item.numel(), qstart, qlen, pos0, out, tokens, heads, kv_heads,
                             0, scale, error, nsplit, part_o, part_ml, None, 0)
        elif row_class >= 0:
            ops.attention_mma(row_class, q, q.stride(0), pages[:, 0, 0], pages[:, 0, 1],
                              pages.stride(0), page, tables, tile_item, tile_row0,
                              tile_item.numel(), qstart, qlen, pos0, out, tokens, heads, kv_heads,
                              hd, 0, scale, nsplit, part_o, part_ml, None, 0)
        else:
            ops.attention_generic(q, q.stride(0), pages[:, 0, 0], pages[:, 0, 1], pages.stride(0),
                                  page, tables, tile_item, tile_row0, tile_item.numel(), qstart,
                                  qlen, pos0, out, tokens, heads, kv_heads, hd, 0, scale, nsplit,
                                  part_o, part_ml, rows16=rows16)
    ms = timer(launch)
    extra = {}
    elem = 2 if dtype is torch.bfloat16 else 4
    kv_bytes = args.batch * args.context * 2 * kv_heads * hd * elem
    io_bytes = kv_bytes + 2 * tokens * heads * hd * elem
    # causal: query t of a portion sees past + t + 1 keys
    pairs = args.batch * (new * past + new * (new + 1) / 2)
    flops = 4.0 * heads * hd * pairs
    if use_tc or use_tcd:
        extra["error"] = int(error.item())
    extra.update({"nsplit": nsplit, "tiles": tile_item.numel(),
                  "variant": ("tc" if use_tc else "tc_decode" if use_tcd else "mma")
                  if row_class >= 0 else ("rows16" if rows16 else "generic")})
    return ms, io_bytes, flops, extra


def run(args):
    timer = Timer(args.warmup, args.iters, not args.no_flush)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    elem = 2 if dtype is torch.bfloat16 else 4
    extra = {}
    g = torch.Generator(device="cuda").manual_seed(0)
    rand = lambda *shape: torch.randn(shape, generator=g, device="cuda", dtype=torch.float32)
    if args.kernel in ("attention_decode", "attention_prefill"):
        ms, nbytes, flops, extra = run_attention(args, timer, args.kernel == "attention_decode")
    elif args.kernel == "add_rmsnorm":
        x, delta = rand(args.tokens, args.hidden), rand(args.tokens, args.hidden).to(dtype)
        gain, y = rand(args.hidden).to(dtype), torch.empty((args.tokens, args.hidden), dtype=dtype,
                                                           device="cuda")
        ms = timer(lambda: ops.add_rmsnorm(x, delta, gain, 1e-6, y))
        nbytes, flops = args.tokens * args.hidden * (8 + 2 * elem), 4.0 * args.tokens * args.hidden
    elif args.kernel == "swiglu":
        gu = rand(args.tokens, 2 * args.inter).to(dtype)
        act = torch.empty((args.tokens, args.inter), dtype=dtype, device="cuda")
        ms = timer(lambda: ops.swiglu(gu, act))
        nbytes, flops = 3 * args.tokens * args.inter * elem, 8.0 * args.tokens * args.inter
    elif args.kernel == "rope_kv_write":
        from ..parts.rope import rotary_table
        heads, kv_heads, hd, page = args.heads, args.kv_heads, args.head_dim, args.page
        qkv = rand(args.tokens, (heads + 2 * kv_heads) * hd).to(dtype)
        table = torch.from_numpy(rotary_table(1e6, hd, args.tokens + 1)).cuda()
        pages = torch.zeros((args.tokens // page + 1, 1, 2, kv_heads, page, hd), dtype=dtype,
                            device="cuda")
        pos = torch.arange(args.tokens, dtype=torch.int32, device="cuda")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        ms = timer(lambda: ops.rope_kv_write(qkv, pos, table, pos, pages[:, 0, 0], pages[:, 0, 1],
                                             pages.stride(0), page, heads, kv_heads, hd, hd, error))
        nbytes = args.tokens * hd * elem * (2 * heads + 4 * kv_heads)
        flops = 6.0 * args.tokens * (heads + kv_heads) * hd
    elif args.kernel in ("argmax", "sample"):
        logits = rand(args.tokens, args.vocab)
        out = torch.empty(args.tokens, dtype=torch.int32, device="cuda")
        if args.kernel == "argmax":
            scratch = torch.empty(2 * args.tokens * ops.ARGMAX_PARTS, device="cuda")
            ms = timer(lambda: ops.argmax(logits, out, scratch))
        else:
            ones = torch.ones(args.tokens, device="cuda")
            k = torch.full((args.tokens,), args.top_k, dtype=torch.int32, device="cuda")
            u = torch.rand(args.tokens, generator=g, device="cuda")
            ms = timer(lambda: ops.sample(logits, ones * 0.8, k, ones * args.top_p, u, out))
        nbytes, flops = args.tokens * args.vocab * 4, float(args.tokens * args.vocab)
    elif args.kernel in ("gemm_decode", "gemm_decode_swiglu"):
        m, n, k = args.tokens, args.n, args.k
        swiglu = args.kernel == "gemm_decode_swiglu"
        x, w = rand(m, k).to(dtype), (rand(2 * n if swiglu else n, k) / math.sqrt(k)).to(dtype)
        weight = ops.DecodeWeight(w, swiglu=swiglu)
        out = torch.empty((m, n), dtype=dtype, device="cuda")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        tiles = -(-n // (64 if swiglu else 128))
        splits = args.nsplit if args.nsplit > 0 else ops.gemm_decode_splits(tiles, k, sms)
        ms = timer(lambda: ops.gemm_decode(weight, x, out, None, error, splits))
        extra = {"splits": splits, "error": int(error.item())}
        nbytes, flops = (m * k + w.shape[0] * k + m * n) * elem, 2.0 * m * w.shape[0] * k
    elif args.kernel == "gemm_skinny":
        m, n, k = args.tokens, args.n, args.k
        x, w = rand(m, k).to(dtype), (rand(n, k) / math.sqrt(k)).to(dtype)
        out = torch.empty((m, n), dtype=dtype, device="cuda")
        ms = timer(lambda: ops.gemm_skinny(w, x, out, None))
        nbytes, flops = (m * k + n * k + m * n) * elem, 2.0 * m * n * k
    elif args.kernel in ("gemm_tiles", "gemm_tiles_swiglu"):
        m, n, k = args.tokens, args.n, args.k
        swiglu = args.kernel == "gemm_tiles_swiglu"
        # outputs of unit scale, as a layer sees them (the activation's exp stays in range)
        x, w = rand(m, k).to(dtype), (rand(2 * n if swiglu else n, k) / math.sqrt(k)).to(dtype)
        weight = ops.TiledWeight(w, swiglu=swiglu)
        out = torch.empty((m, n), dtype=dtype, device="cuda")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        floats, ints = (0, 0) if args.variant == "whole_tiles" else \
            ops.gemm_tiles_workspace(m, n, k, swiglu, sms)
        workspace = torch.empty(floats, dtype=torch.float32, device="cuda") if floats else None
        counters = torch.zeros(max(ints, 1), dtype=torch.int32, device="cuda") if floats else None
        ms = timer(lambda: ops.gemm_tiles(weight, x, out, None, error, sms, workspace, counters))
        extra = {"error": int(error.item()), "workspace_floats": floats,
                 "counters_left": int(counters.abs().sum().item()) if floats else 0}
        nbytes, flops = (m * k + w.shape[0] * k + m * n) * elem, 2.0 * m * w.shape[0] * k
    elif args.kernel in ("linear", "gemm_f32"):
        m, n, k = args.tokens, args.n, args.k
        if args.kernel == "linear":
            x, w = rand(m, k).to(dtype), rand(n, k).to(dtype)
            ms = timer(lambda: torch.nn.functional.linear(x, w))
        else:
            x, w = rand(m, k), rand(n, k)
            ms = timer(lambda: ops.gemm_f32(x, w, None, kind=args.f32_kind, rows_per_warp=args.f32_rows_per_warp))
            elem = 4
            extra = {"frac_ffma": round(2.0 * m * n * k / (ms * 1e-3) / 74.4e12, 3), "f32_kind": args.f32_kind}
        nbytes, flops = (m * k + n * k + m * n) * elem, 2.0 * m * n * k
    else:
        raise SystemExit(f"unknown kernel {args.kernel}")
    peak = peaks()
    gbs, tflops = nbytes / (ms * 1e-3) / 1e9, flops / (ms * 1e-3) / 1e12
    record = {"kernel": args.kernel, "dtype": args.dtype, "ms": round(ms, 5), "bytes": int(nbytes),
              "flops": flops, "GB/s": round(gbs, 1), "TFLOP/s": round(tflops, 2),
              "frac_hbm": round(gbs / peak["hbm_gbs"], 3),
              "frac_bf16": round(tflops / peak["bf16_tflops"], 3), "peaks": peak["source"],
              "sizes": {k: v for k, v in vars(args).items()
                        if k not in ("kernel", "dtype", "warmup", "iters", "no_flush", "f32_kind", "f32_rows_per_warp")}}
    record.update(extra)
    print(json.dumps(record))


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("kernel")
    parser.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=28)
    parser.add_argument("--kv-heads", type=int, default=4)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page", type=int, default=16)
    parser.add_argument("--hidden", type=int, default=3584)
    parser.add_argument("--inter", type=int, default=18944)
    parser.add_argument("--vocab", type=int, default=152064)
    parser.add_argument("--n", type=int, default=37888)
    parser.add_argument("--k", type=int, default=3584)
    parser.add_argument("--nsplit", type=int, default=0, help="0 = the engine's choice")
    parser.add_argument("--variant", default="mma", choices=["mma", "tc", "rows16", "whole_tiles"],
                        help="bfloat16 attention: mma.sync with cp.async loads, or tcgen05; float32 "
                             "attention: rows16 takes the kernel for tiles of up to 16 rows; gemm_tiles: "
                             "whole_tiles leaves a partial last round of tiles to the pairs it falls to")
    parser.add_argument("--f32-kind", default="auto", choices=["auto", "rows", "tiles", "plain"],
                        help="gemm_f32: which of the float32 kernels (frac_ffma is of the nominal "
                             "74.4 TFLOP/s: 148 SMs x 128 lanes x 2 x 1.965 GHz)")
    parser.add_argument("--f32-rows-per-warp", type=int, default=0, choices=[0, 1, 2, 4])
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--no-flush", action="store_true")
    args = parser.parse_args(argv)
    run(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
