"""Each CUDA kernel alone against a plain PyTorch reference, at sizes other than the
engine's test models (the reference does the same for its kernels,
tests/cpp/test_cuda_kernels.cpp:26-235)."""

import math
import random

import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 2e-5 if dtype is torch.float32 else 1.6e-2       # bf16: 2^-8 relative + slack


@pytest.fixture(scope="module")
def ops():
    from from_scratch_inference_engine_b200.kernels import ops
    ops.core()
    return ops


def dev(t, dtype=None):
    t = t.to("cuda")
    return t if dtype is None else t.to(dtype)


# --------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(ops, dtype):
    torch.manual_seed(0)
    for hidden in (300, 301, 3584):
        table = dev(torch.randn(1000, hidden), dtype)
        ids = dev(torch.tensor([0, 999, 5, 5, 123], dtype=torch.int32))
        out = torch.empty(5, hidden, device="cuda")
        error = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.embed_gather(ids, table, out, error)
        assert torch.equal(out, table[ids.long()].float()) and error.item() == 0
        ops.embed_gather(dev(torch.tensor([3, 1000], dtype=torch.int32)), table, out, error)
        assert error.item() == 1 and out[1].abs().max().item() == 0.0     # refused, not read


# ----------------------------------------------------------------------- add + RMSNorm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [64, 777, 3584, 9000, 8 * 1500, 8 * 3000, 8 * 5000])
def test_add_rmsnorm(ops, dtype, hidden):
    torch.manual_seed(1)
    rows, eps = 7, 1e-5
    x0 = torch.randn(rows, hidden) * 3
    delta = (torch.randn(rows, hidden) * 0.5).to(dtype)
    gain = (1 + 0.1 * torch.randn(hidden))
    for gain_dtype in {torch.float32, dtype}:
        x = dev(x0.clone())
        y = torch.empty(rows, hidden, dtype=dtype, device="cuda")
        g = gain.to(gain_dtype)
        ops.add_rmsnorm(x, dev(delta), dev(g), eps, y)
        summed = x0.double() + delta.double()
        want = plain.rms_norm(summed, g.double(), eps)
        assert torch.allclose(x.cpu().double(), summed, atol=1e-6)          # residual in 32-bit
        err = (y.cpu().double() - want).abs().max().item()
        assert err < tol(dtype) * want.abs().max().item()
    # no delta; rows gathered; x untouched
    x = dev(x0.clone())
    pick = dev(torch.tensor([6, 0, 3], dtype=torch.int32))
    y = torch.empty(3, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(x, dev(delta), dev(gain), eps, y, rows=pick, write_x=False)
    want = plain.rms_norm(x0.double() + delta.double(), gain.double(), eps)[[6, 0, 3]]
    assert torch.equal(x.cpu(), x0)
    assert (y.cpu().double() - want).abs().max().item() < tol(dtype) * want.abs().max().item()


# ----------------------------------------------------- rotary encoding + cache write
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,rotary,theta", [(5, 5, 16, 16, 1e4), (6, 2, 48, 32, 5e5),
                                                            (7, 1, 128, 128, 1e6), (3, 3, 20, 12, 1e4),
                                                            (28, 4, 128, 64, 1e6)])
def test_rope_kv_write(ops, dtype, heads, kv_heads, hd, rotary, theta):
    from from_scratch_inference_engine_b200.parts.rope import rotary_table
    torch.manual_seed(2)
    tokens, page_size, num_pages, entries = 9, 4, 11, 2
    positions = [0, 1, 2, 3, 17, 4095, 30000, 31, 32]
    width = (heads + 2 * kv_heads) * hd
    qkv0 = torch.randn(tokens, width).to(dtype)
    qkv = dev(qkv0.clone())
    table = dev(torch.from_numpy(rotary_table(theta, rotary, 30001)))
    pages = torch.zeros(num_pages, entries, 2, kv_heads, page_size, hd, dtype=dtype, device="cuda")
    slots = [5 * page_size + 0, 5 * page_size + 1, 2 * page_size + 3, 0, 10 * page_size + 2,
             -1, 7 * page_size + 1, 3 * page_size + 0, 3 * page_size + 1]
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.rope_kv_write(qkv, dev(torch.tensor(positions, dtype=torch.int32)), table,
                      dev(torch.tensor(slots, dtype=torch.int32)), pages[:, 1, 0], pages[:, 1, 1],
                      pages.stride(0), page_size, heads, kv_heads, hd, rotary, error)
    assert error.item() == 0

    def rotate(x, n):      # plain rope over the first `rotary` dims of each head
        xh = x.double().reshape(tokens, n, hd)
        rot = plain.rope(xh[..., :rotary].reshape(tokens, n * rotary), n, rotary, theta, positions)
        return torch.cat([rot.reshape(tokens, n, rotary), xh[..., rotary:]], -1)
    q_want = rotate(qkv0[:, :heads * hd], heads)
    k_want = rotate(qkv0[:, heads * hd:(heads + kv_heads) * hd], kv_heads)
    v_want = qkv0[:, (heads + kv_heads) * hd:].double().reshape(tokens, kv_heads, hd)
    got_q = qkv[:, :heads * hd].cpu().double().reshape(tokens, heads, hd)
    assert (got_q - q_want).abs().max().item() < tol(dtype) * q_want.abs().max().item()
    cache = pages.cpu().double()
    assert cache[:, 0].abs().max().item() == 0.0                      # the other entry is untouched
    written = 0
    for t, slot in enumerate(slots):
        if slot < 0:
            continue
        page, off = divmod(slot, page_size)
        assert (cache[page, 1, 0, :, off] - k_want[t]).abs().max().item() \
            < tol(dtype) * k_want.abs().max().item()
        assert torch.equal(cache[page, 1, 1, :, off], v_want[t])
        written += 1
    assert (cache[:, 1, 0].abs().sum((1, 3)) > 0).sum().item() == written   # nothing else written
    # a position beyond the table is refused
    ops.rope_kv_write(qkv, dev(torch.tensor([40000] * tokens, dtype=torch.int32)), table, None,
                      None, None, 0, page_size, heads, kv_heads, hd, rotary, error)
    assert error.item() == 2


# ------------------------------------------------------------------------------ SwiGLU
@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(ops, dtype):
    torch.manual_seed(3)
    for inter in (333, 18944 // 8, 8):
        gu = (torch.randn(13, 2 * inter) * 3).to(dtype)
        out = torch.empty(13, inter, dtype=dtype, device="cuda")
        ops.swiglu(dev(gu), out)
        want = plain.silu_mul(gu[:, :inter].double(), gu[:, inter:].double())
        assert (out.cpu().double() - want).abs().max().item() < tol(dtype) * want.abs().max().item()


# ---------------------------------------------------------------------- float32 product
GEMM_F32_SIZES = [(1, 7, 5), (37, 101, 203), (64, 64, 16), (130, 70, 1000), (1, 96, 512),
                  (8, 4608, 3584), (16, 3584, 1000), (13, 77, 132), (40, 300, 644), (64, 1024, 2048),
                  (200, 130, 260), (129, 257, 516), (2048, 512, 384)]


@pytest.mark.parametrize("kind", ["auto", "rows", "tiles", "plain"])
@pytest.mark.parametrize("m,n,k", GEMM_F32_SIZES)
def test_gemm_f32(ops, m, n, k, kind):
    """The three float32 kernels (few rows, tiles, plain) and the choice among them, each
    against the 64-bit product, with and without bias, at sizes that are no multiples of
    their tiles."""
    from from_scratch_inference_engine_b200.kernels.ops import KernelError
    torch.manual_seed(4)
    x, w, b = torch.randn(m, k), torch.randn(n, k), torch.randn(n)
    want = x.double() @ w.double().T + b.double()
    takes = {"auto": True, "plain": True, "tiles": k % 4 == 0,
             "rows": k % 4 == 0 and m <= ops.gemm_f32_rows_limit()}[kind]
    if not takes:
        with pytest.raises(KernelError):
            ops.gemm_f32(dev(x), dev(w), dev(b), kind=kind)
        return
    bound = 1e-5 * math.sqrt(k) * 4
    got = ops.gemm_f32(dev(x), dev(w), dev(b), kind=kind)
    assert (got.cpu().double() - want).abs().max().item() < bound
    got = ops.gemm_f32(dev(x), dev(w), None, kind=kind)
    assert (got.cpu().double() - (want - b.double())).abs().max().item() < bound
    # a row's result does not depend on the other rows of the launch (same kernel)
    alone = ops.gemm_f32(dev(x[m // 2:m // 2 + 1]), dev(w), dev(b), kind=kind)
    both = ops.gemm_f32(dev(x), dev(w), dev(b), kind=kind)
    if kind != "auto" or (m <= ops.gemm_f32_rows_limit()) or k % 4:
        assert torch.equal(alone[0], both[m // 2])
    else:       # the single row took the few-rows kernel, the batch the tiles: another order of the sums
        assert (alone[0] - both[m // 2]).abs().max().item() < bound
    # x as a view with a row stride (rows of a wider matrix), output into a wider matrix
    if k % 4 == 0 and kind != "plain":
        wide = torch.randn(m, k + 8)
        out = torch.full((m, n + 3), float("nan"), device="cuda")
        ops.gemm_f32(dev(wide)[:, 4:4 + k], dev(w), dev(b), out=out[:, :n], kind=kind)
        again = wide[:, 4:4 + k].double() @ w.double().T + b.double()
        assert (out[:, :n].cpu().double() - again).abs().max().item() < bound
        assert torch.isnan(out[:, n:]).all()


# --------------------------------------------------------------------------- attention
class PagedCase:
    """Requests with history and new tokens over shuffled pages, and the plain answer."""

    def __init__(self, dtype, heads, kv_heads, hd, page_size, items, window=0, seed=0,
                 peak=None):
        g = torch.Generator().manual_seed(seed)
        self.heads, self.kv_heads, self.hd, self.page_size, self.window = \
            heads, kv_heads, hd, page_size, window
        self.items = items                                   # [(past, new)]
        total_pages = sum(-(-(p + n) // page_size) for p, n in items) + 3
        order = list(range(total_pages))
        random.Random(seed).shuffle(order)
        self.pages = torch.zeros(total_pages, 1, 2, kv_heads, page_size, hd, dtype=dtype)
        width = max(-(-(p + n) // page_size) for p, n in items)
        self.tables = torch.full((len(items), width), -1, dtype=torch.int32)
        qs, self.want = [], []
        for i, (past, new) in enumerate(items):
            total = past + new
            k = torch.randn(total, kv_heads * hd, generator=g).to(dtype)
            v = torch.randn(total, kv_heads * hd, generator=g).to(dtype)
            q = torch.randn(new, heads * hd, generator=g).to(dtype)
            if peak is not None:
                # one far key stands out for the last query: scale the pair so its score wins
                key_at = peak(past, new)
                q[-1] = q[-1] * 0 + 1.0
                k[key_at] = k[key_at] * 0 + 3.0
            blocks = -(-total // page_size)
            mine = [order.pop() for _ in range(blocks)]
            self.tables[i, :blocks] = torch.tensor(mine, dtype=torch.int32)
            for t in range(total):
                page, off = mine[t // page_size], t % page_size
                self.pages[page, 0, 0, :, off] = k[t].reshape(kv_heads, hd)
                self.pages[page, 0, 1, :, off] = v[t].reshape(kv_heads, hd)
            if window > 0:      # pages the window has left behind are gone
                for b in range(max(0, past - window + 1) // page_size):
                    self.pages[mine[b]] = float("nan")
                    self.tables[i, b] = -1
            qs.append(q)
            self.want.append(plain.attention(q.double(), k.double(), v.double(), heads, kv_heads,
                                             hd, query_offset=past, window=window))
        self.q = torch.cat(qs)
        self.want = torch.cat(self.want)

    def run(self, ops, nsplit=1, rows16=False):
        """The 32-bit kernels; with rows16 the requests of up to 16 query rows go to the kernel
        for few rows first (unmerged) and the others follow, as the engine launches them."""
        group = self.heads // self.kv_heads
        rows = ops.attention_rows_per_tile()
        tile_item, tile_row0, qstart = [], [], []
        few_item, few_row0 = [], []
        at = 0
        for i, (past, new) in enumerate(self.items):
            qstart.append(at)
            at += new
            if rows16 and new * group <= ops.attention_rows16_rows():
                few_item.append(i)
                few_row0.append(0)
                continue
            for r0 in range(0, new * group, rows):
                tile_item.append(i)
                tile_row0.append(r0)
        i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
        pages = dev(self.pages)
        q = dev(self.q)
        tokens = q.shape[0]
        out = torch.full((tokens, self.heads * self.hd), float("nan"), dtype=q.dtype, device="cuda")
        part_o = part_ml = None
        if nsplit > 1:
            part_o = torch.full((nsplit * tokens * self.heads * self.hd,), float("nan"),
                                device="cuda")
            part_ml = torch.full((nsplit * tokens * self.heads * 2,), float("nan"), device="cuda")
        if few_item:
            ops.attention_generic(q, q.stride(0), pages[:, 0, 0], pages[:, 0, 1], pages.stride(0),
                                  self.page_size, dev(self.tables), i32(few_item), i32(few_row0),
                                  len(few_item), i32(qstart), i32([n for _, n in self.items]),
                                  i32([p for p, _ in self.items]), out, tokens, self.heads,
                                  self.kv_heads, self.hd, self.window, 1.0 / math.sqrt(self.hd),
                                  nsplit, part_o, part_ml, rows16=True, merge=False)
        ops.attention_generic(q, q.stride(0), pages[:, 0, 0], pages[:, 0, 1], pages.stride(0),
                              self.page_size, dev(self.tables), i32(tile_item), i32(tile_row0),
                              len(tile_item), i32(qstart), i32([n for _, n in self.items]),
                              i32([p for p, _ in self.items]), out, tokens, self.heads,
                              self.kv_heads, self.hd, self.window, 1.0 / math.sqrt(self.hd),
                              nsplit, part_o, part_ml)
        return out.cpu().double()


    def run_mma(self, ops, nsplit=1, tc=False, tc_decode=False):
        """The tensor-core kernels: requests sorted into row classes as the engine does."""
        group = self.heads // self.kv_heads
        i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
        qstart, at = [], 0
        for _, new in self.items:
            qstart.append(at)
            at += new
        pages, q = dev(self.pages), dev(self.q)
        tokens = q.shape[0]
        out = torch.full((tokens, self.heads * self.hd), float("nan"), dtype=q.dtype, device="cuda")
        part_o = part_ml = None
        if nsplit > 1:
            part_o = torch.full((nsplit * tokens * self.heads * self.hd,), float("nan"), device="cuda")
            part_ml = torch.full((nsplit * tokens * self.heads * 2,), float("nan"), device="cuda")
        classes = ops.ATTENTION_ROW_CLASSES
        if tc:      # prompt portions in tiles of 128 rows through the tcgen05 kernel
            classes = classes[:2] + (ops.ATTENTION_TC_ROWS,)
        for c, per_tile in enumerate(classes):
            tile_item, tile_row0, toks = [], [], []
            for i, (_, new) in enumerate(self.items):
                rows = new * group
                fits = [k for k, r in enumerate(classes) if rows <= r]
                if (fits[0] if fits else len(classes) - 1) != c:
                    continue
                toks += list(range(qstart[i], qstart[i] + new))
                for r0 in range(0, rows, per_tile):
                    tile_item.append(i)
                    tile_row0.append(r0)
            if not tile_item:
                continue
            if tc and c == 2:
                error = torch.zeros(1, dtype=torch.int32, device="cuda")
                ops.attention_tc(ops.PagesMap(pages, "tc"), 0, q, q.stride(0), dev(self.tables),
                                 i32(tile_item), i32(tile_row0), len(tile_item), i32(qstart),
                                 i32([n for _, n in self.items]), i32([p for p, _ in self.items]),
                                 out, tokens, self.heads, self.kv_heads, self.window,
                                 1.0 / math.sqrt(self.hd), error, nsplit, part_o, part_ml,
                                 i32(toks), len(toks))
                assert error.item() == 0
                continue
            if tc_decode and c == 0:
                error = torch.zeros(1, dtype=torch.int32, device="cuda")
                ops.attention_tc_decode(ops.PagesMap(pages, "tc"), 0, q, q.stride(0),
                                        dev(self.tables), i32(tile_item), i32(tile_row0),
                                        len(tile_item), i32(qstart),
                                        i32([n for _, n in self.items]),
                                        i32([p for p, _ in self.items]), out, tokens, self.heads,
                                        self.kv_heads, self.window, 1.0 / math.sqrt(self.hd),
                                        error, nsplit, part_o, part_ml, i32(toks), len(toks))
                assert error.item() == 0
                continue
            ops.attention_mma(c, q, q.stride(0), pages[:, 0, 0], pages[:, 0, 1], pages.stride(0),
                              self.page_size, dev(self.tables), i32(tile_item), i32(tile_row0),
                              len(tile_item), i32(qstart), i32([n for _, n in self.items]),
                              i32([p for p, _ in self.items]), out, tokens, self.heads,
                              self.kv_heads, self.hd, self.window, 1.0 / math.sqrt(self.hd),
                              nsplit, part_o, part_ml, i32(toks), len(toks))
        return out.cpu().double()


def assert_rows_close(got, want, case, dtype):
    """Every (token, head) row against its own size: the output of a token over thousands of
    random keys is an average near zero (about 0.05), a first token's output is one value
    vector (about 3) - a bound taken from the largest value anywhere would let the small rows
    be anything."""
    got = got.reshape(-1, case.heads, case.hd)
    want = want.reshape(-1, case.heads, case.hd)
    assert got.shape == want.shape and torch.isfinite(got).all()
    error = (got - want).abs().amax(-1)
    bound = tol(dtype) * want.abs().amax(-1)
    worst = (error / bound).max().item()
    assert worst < 1.0, f"worst row at {worst:.2f} of its bound (token, head) = " \
                        f"{divmod((error / bound).argmax().item(), case.heads)}"


def run_kernel(case, ops, kernel, nsplit=1):
    if kernel == "tc":
        if case.hd not in ops.ATTENTION_TC_HEAD_DIMS or case.page_size not in ops.ATTENTION_TC_PAGES:
            pytest.skip("the tcgen05 kernel takes head sizes 64 and 128 and pages of 8..128")
        return case.run_mma(ops, nsplit, tc=True)
    if kernel == "rows16":
        if not ops.attention_rows16_fits(torch.float32, case.hd, case.hd):
            pytest.skip("the kernel for few rows is compiled for head sizes 32, 64, 96, 128 and 256")
        return case.run(ops, nsplit, rows16=True)
    return case.run_mma(ops, nsplit) if kernel == "mma" else case.run(ops, nsplit)


KERNELS = [("generic", torch.float32), ("generic", torch.bfloat16), ("rows16", torch.float32),
           ("mma", torch.bfloat16), ("tc", torch.bfloat16)]


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("heads,kv_heads,hd,page_size", [
    (4, 4, 16, 4), (6, 2, 48, 8), (7, 1, 80, 16), (28, 4, 128, 16), (3, 1, 256, 32),
    (40, 1, 32, 5), (8, 2, 64, 8), (5, 1, 192, 64), (28, 4, 128, 32)])
def test_attention_sizes(ops, kernel, dtype, heads, kv_heads, hd, page_size):
    case = PagedCase(dtype, heads, kv_heads, hd, page_size,
                     items=[(0, 37), (45, 1), (19, 6), (0, 1), (63, 2), (130, 70)], seed=heads)
    got = run_kernel(case, ops, kernel)
    assert_rows_close(got, case.want, case, dtype)


@pytest.mark.parametrize("kernel,dtype", [k for k in KERNELS if k[0] != "generic" or k[1] is torch.float32])
def test_attention_long_context(ops, kernel, dtype):
    """Thousands of keys over hundreds of shuffled pages: a long prompt portion on top of a long
    history, a decoded token, and a whole prompt, with and without split key ranges."""
    case = PagedCase(dtype, 4, 2, 64, 16, items=[(3000, 300), (4100, 1), (0, 700)], seed=12)
    for nsplit in (1, 7, 64):            # 64: ranges of 128 keys (mma.sync kernel 64), more than 32 of them hold keys
        got = run_kernel(case, ops, kernel, nsplit)
        assert_rows_close(got, case.want, case, dtype)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("nsplit", [2, 5, 32, 37, 64])
def test_attention_split_keys(ops, kernel, dtype, nsplit):
    case = PagedCase(dtype, 14, 2, 64, 16, items=[(700, 1), (0, 3), (301, 1), (33, 2), (400, 20)],
                     seed=5)
    whole, split = run_kernel(case, ops, kernel, 1), run_kernel(case, ops, kernel, nsplit)
    assert_rows_close(split, case.want, case, dtype)
    assert_rows_close(whole, case.want, case, dtype)


@pytest.mark.parametrize("hd", [16, 48, 80, 112, 160, 256])
@pytest.mark.parametrize("nsplit", [9, 17, 33])
def test_attention_split_keys_at_other_head_sizes(ops, hd, nsplit):
    """The merge of more than eight key ranges at head sizes that are no multiple of 64 (its
    threads hold two dimensions each, so the last warp's lanes are not all in use)."""
    case = PagedCase(torch.bfloat16, 6, 2, hd, 16, items=[(1300, 1), (0, 3), (2200, 1), (700, 20)], seed=13)
    assert_rows_close(run_kernel(case, ops, "mma", nsplit), case.want, case, torch.bfloat16)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("key_at", ["first", "page_edge", "far", "self"])
def test_attention_finds_one_far_key_among_hundreds(ops, kernel, dtype, key_at):
    pick = {"first": lambda p, n: 0, "page_edge": lambda p, n: 16 * 7 - 1,
            "far": lambda p, n: 131, "self": lambda p, n: p + n - 1}[key_at]
    case = PagedCase(dtype, 8, 2, 64, 16, items=[(600, 1), (500, 5)], seed=6, peak=pick)
    # the scaled pair has score 3 * 64 / 8 = 24 over scores of order 1: the last query's
    # output is that key's value, so a wrong page or offset shows at full size
    got = run_kernel(case, ops, kernel, nsplit=1)
    assert_rows_close(got, case.want, case, dtype)
    got = run_kernel(case, ops, kernel, nsplit=4)
    assert_rows_close(got, case.want, case, dtype)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("window", [1, 16, 21])
def test_attention_window_edge(ops, kernel, dtype, window):
    # the key just outside the window carries the peak: it must not be seen;
    # pages wholly behind the window hold NaN and have no table entry
    outside = lambda p, n: p + n - 1 - window
    case = PagedCase(dtype, 6, 3, 32, 8, items=[(90, 1), (64, 7), (0, 30)], window=window,
                     seed=7, peak=outside if window < 30 else None)
    got = run_kernel(case, ops, kernel)
    assert torch.isfinite(got).all()
    assert_rows_close(got, case.want, case, dtype)
    inside = lambda p, n: p + n - window
    case = PagedCase(dtype, 6, 3, 32, 8, items=[(90, 1), (64, 7)], window=window, seed=8,
                     peak=inside)
    got = run_kernel(case, ops, kernel, nsplit=2)
    assert_rows_close(got, case.want, case, dtype)


@pytest.mark.parametrize("kernel,dtype", KERNELS)
@pytest.mark.parametrize("window,nsplit", [(26, 2), (150, 2), (300, 3)])
def test_attention_window_with_split_keys(ops, kernel, dtype, window, nsplit):
    """A window that does not start on a tile of keys, cut into key ranges.  No key stands out
    here: every key of the window counts alike, so a key that two ranges see (ranges that
    overlap once they are rounded to tiles) or that none sees moves the result."""
    case = PagedCase(dtype, 8, 2, 128, 16, items=[(700, 1), (450, 40), (0, 350), (131, 2)],
                     window=window, seed=11)
    assert_rows_close(run_kernel(case, ops, kernel, nsplit), case.want, case, dtype)


@pytest.mark.parametrize("window,nsplit", [(150, 2), (300, 3), (1000, 4)])
def test_attention_tc_decode_window_with_split_keys(ops, window, nsplit):
    case = PagedCase(torch.bfloat16, 14, 2, 128, 16, items=[(700, 1), (1450, 1), (131, 2), (2000, 1)],
                     window=window, seed=12)
    assert_rows_close(case.run_mma(ops, nsplit, tc_decode=True), case.want, case, torch.bfloat16)


@pytest.mark.parametrize("heads,kv_heads,page_size", [(28, 4, 16), (40, 8, 32), (16, 1, 8), (3, 3, 128),
                                                      (12, 2, 64)])
def test_attention_tc_decode_sizes(ops, heads, kv_heads, page_size):
    """The tcgen05 kernel for tiles of up to 16 rows (head size 128): decoded tokens over short and
    long histories, two-token portions, first tokens, beside requests of the other row classes."""
    group = heads // kv_heads
    items = [(45, 1), (0, 1), (127, 1), (128, 1), (1300, 1), (63, max(1, 16 // group)), (130, 70), (0, 37)]
    case = PagedCase(torch.bfloat16, heads, kv_heads, 128, page_size, items=items, seed=heads)
    for nsplit in (1, 3):
        got = case.run_mma(ops, nsplit, tc_decode=True)
        assert_rows_close(got, case.want, case, torch.bfloat16)


def test_attention_tc_decode_long_contexts_with_the_engine_s_split(ops):
    """Sixteen requests of 3,900-4,100 keys over four kv heads: 64 (request, kv head) pairs, for
    which the engine would split each key range in four for this kernel."""
    from from_scratch_inference_engine_b200.parts.attention import attention_splits
    items = [(3900 + 13 * i, 1) for i in range(16)]
    case = PagedCase(torch.bfloat16, 28, 4, 128, 16, items=items, seed=31)
    nsplit = attention_splits(16 * 4, 4100, 148, True, decode_slots=2, decode_fixed=530, merge_cost=1300)
    assert nsplit == 4
    for n in (1, nsplit):
        assert_rows_close(case.run_mma(ops, n, tc_decode=True), case.want, case, torch.bfloat16)
    assert_rows_close(case.run_mma(ops, nsplit), case.want, case, torch.bfloat16)     # mma.sync kernel


@pytest.mark.parametrize("key_at", ["first", "page_edge", "far", "self"])
def test_attention_tc_decode_finds_one_far_key(ops, key_at):
    pick = {"first": lambda p, n: 0, "page_edge": lambda p, n: 16 * 7 - 1,
            "far": lambda p, n: 131, "self": lambda p, n: p + n - 1}[key_at]
    case = PagedCase(torch.bfloat16, 14, 2, 128, 16, items=[(600, 1), (500, 2)], seed=6, peak=pick)
    for nsplit in (1, 4):
        got = case.run_mma(ops, nsplit, tc_decode=True)
        assert_rows_close(got, case.want, case, torch.bfloat16)


@pytest.mark.parametrize("window", [1, 16, 21, 200])
def test_attention_tc_decode_window_edge(ops, window):
    outside = lambda p, n: max(0, p + n - 1 - window)
    case = PagedCase(torch.bfloat16, 6, 3, 128, 8, items=[(290, 1), (64, 7), (700, 1)], window=window,
                     seed=7, peak=outside)
    got = case.run_mma(ops, tc_decode=True)
    assert torch.isfinite(got).all()
    assert_rows_close(got, case.want, case, torch.bfloat16)
    inside = lambda p, n: max(0, p + n - window)
    case = PagedCase(torch.bfloat16, 6, 3, 128, 8, items=[(290, 1), (64, 7)], window=window, seed=8,
                     peak=inside)
    got = case.run_mma(ops, nsplit=2, tc_decode=True)
    assert_rows_close(got, case.want, case, torch.bfloat16)


def test_attention_refuses_what_it_cannot_take(ops):
    from from_scratch_inference_engine_b200.kernels.ops import KernelError
    case = PagedCase(torch.float32, 2, 2, 16, 4, items=[(0, 2)])
    case.hd = 272
    with pytest.raises(KernelError):
        case.run(ops)
    with pytest.raises(KernelError, match="head sizes"):
        ops.attn_mma(24)


# ---------------------------------------------------------------------------- sampling
def test_argmax_ties_go_to_the_smallest_index(ops):
    logits = torch.zeros(3, 151936)
    logits[0, [70000, 5, 150000]] = 4.0
    logits[1, 151935] = 1.0
    logits[2] = -1.0
    out = torch.empty(3, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), out)
    assert out.tolist() == [5, 151935, 0]
    staged = torch.full((3,), -7, dtype=torch.int32, device="cuda")
    ops.argmax(dev(logits), staged, torch.empty(2 * 3 * ops.ARGMAX_PARTS, device="cuda"))
    assert staged.tolist() == [5, 151935, 0]
    torch.manual_seed(9)
    wide = torch.randn(5, 100003)
    ops.argmax(dev(wide), staged.new_empty(5), None)
    got = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.argmax(dev(wide), got, torch.empty(2 * 5 * ops.ARGMAX_PARTS, device="cuda"))
    assert got.tolist() == wide.argmax(-1).tolist()


@pytest.mark.parametrize("vocab", [1000, 151936])
def test_sample_matches_plain_sampler(ops, vocab):
    rng = random.Random(vocab)
    torch.manual_seed(vocab)
    cases = []
    for temperature in (0.7, 1.0, 1.5):
        for top_k in (0, 1, 5, 50):
            for top_p in (1.0, 0.9, 0.3):
                cases.append((temperature, top_k, top_p, rng.random()))
    cases += [(1.0, 0, 1.0, 0.0), (1.0, 0, 1.0, 0.99999994), (0.8, 3, 0.95, 0.5)]
    logits = torch.randn(len(cases), vocab) * 3
    logits[:, 17] = logits[:, 400]                 # ties inside every row
    logits[3, :] = 0.25                            # a row of equal logits
    f32 = lambda v: dev(torch.tensor(v, dtype=torch.float32))
    out = torch.empty(len(cases), dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), f32([c[0] for c in cases]),
               dev(torch.tensor([c[1] for c in cases], dtype=torch.int32)),
               f32([c[2] for c in cases]), f32([c[3] for c in cases]), out)
    got = out.tolist()
    mismatches = 0
    for r, (temperature, top_k, top_p, u) in enumerate(cases):
        want = plain.sample(logits[r].tolist(), temperature, top_k, top_p,
                            float(np.float32(u)))
        if got[r] != want:
            # allowed only when u lands within float32 rounding of a step of the CDF: the
            # running probability between the two tokens is then below 2e-6
            order = sorted(range(vocab), key=lambda i: (-logits[r, i].item(), i))
            w = np.exp((logits[r, order].double().numpy() - logits[r].max().item())
                       / temperature)
            cdf = np.cumsum(w) / w.sum()
            lo, hi = sorted((order.index(got[r]), order.index(want)))
            assert cdf[hi] - cdf[lo] < 2e-6, (r, cases[r], got[r], want)
            mismatches += 1
    assert mismatches <= 2


def test_sample_frequencies(ops):
    """2,000 draws from three tokens with probabilities 0.7 / 0.2 / 0.1."""
    probs = torch.tensor([0.2, 0.7, 0.1])
    logits = probs.log().repeat(2000, 1)
    rng = random.Random(1)
    u = torch.tensor([rng.random() for _ in range(2000)], dtype=torch.float32)
    out = torch.empty(2000, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(torch.ones(2000)), dev(torch.zeros(2000, dtype=torch.int32)),
               dev(torch.ones(2000)), dev(u), out)
    counts = torch.bincount(out.cpu().long(), minlength=3).tolist()
    assert abs(counts[1] - 1400) < 90 and abs(counts[0] - 400) < 70 and abs(counts[2] - 200) < 55


# -------------------------------------------------------- tcgen05 product for few tokens
@pytest.mark.parametrize("tokens", [1, 8, 16, 17, 33, 64])
@pytest.mark.parametrize("n,k,splits", [(384, 512, 1), (200, 136, 1), (256, 1024, 2), (128, 2048, 8),
                                        (3584, 3584, 4)])
def test_gemm_decode_tcgen05(ops, tokens, n, k, splits):
    torch.manual_seed(tokens + n)
    x = dev(torch.randn(tokens, k), torch.bfloat16)
    w = dev(torch.randn(n, k) / math.sqrt(k), torch.bfloat16)
    bias = dev(torch.randn(n), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = x.double() @ w.double().T
    weight = ops.DecodeWeight(w)
    out = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_decode(weight, x, out, None, error, splits)
    assert error.item() == 0
    assert (out.double() - want).abs().max().item() < 1.6e-2 * want.abs().max().item()
    out32 = torch.full((tokens, n), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemm_decode(weight, x, out32, bias, error, splits)
    assert error.item() == 0
    assert (out32.double() - want - bias.double()).abs().max().item() < 2e-3 * want.abs().max().item()


@pytest.mark.parametrize("tokens,inter,k,splits", [(8, 320, 512, 1), (3, 100, 264, 1), (64, 192, 1024, 4),
                                                   (8, 18944, 3584, 1)])
def test_gemm_decode_swiglu_epilogue(ops, tokens, inter, k, splits):
    torch.manual_seed(inter)
    x = dev(torch.randn(tokens, k), torch.bfloat16)
    w = dev(torch.randn(2 * inter, k) / math.sqrt(k), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    gate_up = (x.double() @ w.double().T).to(torch.bfloat16).double()      # rounded as the library path
    want = plain.silu_mul(gate_up[:, :inter], gate_up[:, inter:])
    out = torch.full((tokens, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_decode(ops.DecodeWeight(w, swiglu=True), x, out, None, error, splits)
    assert error.item() == 0
    assert (out.double() - want).abs().max().item() < 2.5e-2 * want.abs().max().item()


# -------------------------------------------------------- tcgen05 product for many tokens
@pytest.mark.parametrize("rows", [1, 100, 129, 256, 300, 700])
@pytest.mark.parametrize("n,k,blocks", [(384, 512, 148), (200, 136, 148), (520, 72, 2), (1288, 1024, 3)])
def test_gemm_tiles_tcgen05(ops, rows, n, k, blocks):
    """Tiles of 256 x 256 with ragged edges in every direction; with fewer blocks than tiles a
    block walks over several tiles and reuses its stages and its tensor memory."""
    torch.manual_seed(rows + n)
    x_full = dev(torch.randn(rows, k + 8), torch.bfloat16)
    x = x_full[:, :k]                                          # rows 16 bytes further apart than k
    w = dev(torch.randn(n, k) / math.sqrt(k), torch.bfloat16)
    bias = dev(torch.randn(n), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = x.double() @ w.double().T
    weight = ops.TiledWeight(w)
    out_full = torch.full((rows, n + 8), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tiles(weight, x, out_full[:, :n], None, error, blocks)
    assert error.item() == 0
    assert torch.isnan(out_full[:, n:]).all()                  # nothing beyond the last column
    assert (out_full[:, :n].double() - want).abs().max().item() < 1.6e-2 * want.abs().max().item()
    out32 = torch.full((rows, n), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemm_tiles(weight, x, out32, bias, error, blocks)
    assert error.item() == 0
    assert (out32.double() - want - bias.double()).abs().max().item() < 2e-3 * want.abs().max().item()


@pytest.mark.parametrize("rows,inter,k,blocks", [(300, 320, 512, 148), (77, 100, 264, 148), (513, 712, 128, 4),
                                                 (256, 18944, 3584, 148)])
def test_gemm_tiles_swiglu_epilogue(ops, rows, inter, k, blocks):
    torch.manual_seed(inter)
    x = dev(torch.randn(rows, k), torch.bfloat16)
    w = dev(torch.randn(2 * inter, k) / math.sqrt(k), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    gate_up = (x.double() @ w.double().T).to(torch.bfloat16).double()      # rounded as the unfused path
    want = plain.silu_mul(gate_up[:, :inter], gate_up[:, inter:])
    out = torch.full((rows, inter), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tiles(ops.TiledWeight(w, swiglu=True), x, out, None, error, blocks)
    assert error.item() == 0
    assert (out.double() - want).abs().max().item() < 2.5e-2 * want.abs().max().item()


@pytest.mark.parametrize("rows,n,k,blocks,swiglu,shares", [
    (700, 1288, 6144, 10, False, True),     # 18 tiles on 5 pairs: 3 tiles shared out among 5
    (2048, 3584, 4096, 148, False, True),   # 112 tiles on 74 pairs: 38 shared out among 74, k-blocks cut 2 and 3 ways
    (2048, 3584, 512, 148, False, False),   # the same with a k so short that sharing would not pay
    (300, 2000, 2056, 148, False, False),   # fewer tiles than pairs never share; ragged k
    (1000, 520, 1536, 12, False, False),    # 12 tiles on 6 pairs: a full last round
    (515, 1100, 6152, 20, True, True),      # SwiGLU: 27 tiles on 10 pairs, 7 shared; ragged everywhere
    (2300, 300, 4096, 16, False, True),     # 18 tiles on 8 pairs: 2 shared three ways each
])
def test_gemm_tiles_shares_a_partial_last_round(ops, rows, n, k, blocks, swiglu, shares):
    """With a workspace the tiles that do not fill a last round are cut along k among all pairs
    and the parts are added by whoever comes last, in the order of the shares: the result is
    the same on every run, equals the product, and the counters are left at zero."""
    torch.manual_seed(rows + n)
    x = dev(torch.randn(rows, k), torch.bfloat16)
    w = dev(torch.randn((2 if swiglu else 1) * n, k) / math.sqrt(k), torch.bfloat16)
    bias = None if swiglu else dev(torch.randn(n), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    full = x.double() @ w.double().T
    if swiglu:
        full = full.to(torch.bfloat16).double()
        want = plain.silu_mul(full[:, :n], full[:, n:])
    else:
        want = full + bias.double()
    weight = ops.TiledWeight(w, swiglu=swiglu)
    floats, ints = ops.gemm_tiles_workspace(rows, n, k, swiglu, blocks)
    assert (floats > 0) == shares
    workspace = torch.full((max(floats, 1),), float("nan"), dtype=torch.float32, device="cuda")
    counters = torch.zeros(max(ints, 1), dtype=torch.int32, device="cuda")
    outs = []
    for _ in range(3):
        out = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.gemm_tiles(weight, x, out, bias, error, blocks, workspace, counters)
        assert error.item() == 0 and counters.abs().sum().item() == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    bound = (2.5e-2 if swiglu else 1.6e-2) * want.abs().max().item()
    assert (outs[0].double() - want).abs().max().item() < bound
    # the same tiles summed by one pair each differ from the shared ones by the order of the sums only
    whole = torch.full((rows, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_tiles(weight, x, whole, bias, error, blocks)
    assert (whole.double() - outs[0].double()).abs().max().item() <= 1.6e-2 * want.abs().max().item()
    if not swiglu:
        out32 = torch.full((rows, n), float("nan"), dtype=torch.float32, device="cuda")
        ops.gemm_tiles(weight, x, out32, None, error, blocks, workspace, counters)
        assert (out32.double() - full).abs().max().item() < 2e-3 * full.abs().max().item()


def test_gemm_tiles_workspace_is_asked_for_only_where_a_round_is_partial(ops):
    assert ops.gemm_tiles_workspace(2048, 3584, 18944, False, 148)[0] > 0          # 112 tiles, 74 pairs
    assert ops.gemm_tiles_workspace(2048, 18944, 3584, True, 148) == (0, 0)        # 1,184 tiles: 16 full rounds
    assert ops.gemm_tiles_workspace(256, 256, 4096, False, 148) == (0, 0)          # one tile


@pytest.mark.parametrize("rows,blocks", [(2600, 148), (2600, 6), (4200, 10), (2049, 148)])
def test_gemm_tiles_bands_of_row_tiles(ops, rows, blocks):
    """More than eight tiles of rows: the tiles are walked in bands of eight row tiles, the
    last band lower than the others.  Every output must be written once and be the right one."""
    torch.manual_seed(rows)
    n, k = 520, 136
    x = dev(torch.randn(rows, k), torch.bfloat16)
    w = dev(torch.randn(n, k) / math.sqrt(k), torch.bfloat16)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.full((rows, n), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemm_tiles(ops.TiledWeight(w), x, out, None, error, blocks)
    want = x.double() @ w.double().T
    assert error.item() == 0 and torch.isfinite(out).all()
    assert (out.double() - want).abs().max().item() < 2e-3 * want.abs().max().item()


def test_gemm_tiles_one_key_block_stands_out(ops):
    """One k-block of one row tile carries the whole result: a stage that is read too early,
    too late or for the wrong tile shows as a gross error, not as noise."""
    rows, n, k = 600, 512, 1024
    x = torch.zeros(rows, k)
    w = torch.zeros(n, k)
    x[:, 640:704] = torch.randn(rows, 64)
    w[:, 640:704] = torch.randn(n, 64)
    x[300:, :64] = 1.0                                         # rows of the second tile also see k-block 0
    w[:, :64] = 0.5
    error = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty((rows, n), dtype=torch.float32, device="cuda")
    ops.gemm_tiles(ops.TiledWeight(dev(w, torch.bfloat16)), dev(x, torch.bfloat16), out, None, error, 2)
    want = dev(x, torch.bfloat16).double() @ dev(w, torch.bfloat16).double().T
    assert error.item() == 0
    assert (out.double() - want).abs().max().item() < 1e-3 * want.abs().max().item()


# -------------------------------------------------------- product without set-up for small matrices
@pytest.mark.parametrize("tokens", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(384, 512), (200, 96), (37, 1024), (4608, 3584), (3584, 512), (4001, 64),
                                 (9000, 96)])
def test_gemm_skinny(ops, tokens, n, k):
    """Rows of w in blocks of 16 (a ragged last block), k in chunks of 32 taken in turn by the
    warps (fewer chunks than warps at k = 96), tokens padded to 8 or 16."""
    torch.manual_seed(tokens * 1000 + n)
    x_full = dev(torch.randn(tokens, k + 8), torch.bfloat16)
    x = x_full[:, :k]
    w = dev(torch.randn(n, k) / math.sqrt(k), torch.bfloat16)
    bias = dev(torch.randn(n), torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny(w, x, out, None)
    assert (out.double() - want).abs().max().item() < 1.6e-2 * want.abs().max().item()
    out32 = torch.full((tokens, n), float("nan"), dtype=torch.float32, device="cuda")
    ops.gemm_skinny(w, x, out32, bias)
    assert (out32.double() - want - bias.double()).abs().max().item() < 2e-3 * want.abs().max().item()


@pytest.mark.parametrize("tokens", [1, 7, 16])
@pytest.mark.parametrize("heads,kv_heads,hd,k,page_size,bias", [
    (28, 4, 128, 512, 16, True), (6, 2, 48, 96, 8, False), (5, 1, 16, 64, 4, True), (3, 3, 80, 160, 32, True)])
def test_gemm_skinny_with_rotation_and_cache_write(ops, tokens, heads, kv_heads, hd, k, page_size, bias):
    """The q, k, v product with the rotation and the cache write in its epilogue gives what the
    product followed by rope_kv_write gives: rotated queries, rotated keys and values in the slots
    (one token has no slot: nothing of it may be stored), other slots untouched."""
    from from_scratch_inference_engine_b200.parts.rope import rotary_table
    torch.manual_seed(tokens * 100 + heads)
    n = (heads + 2 * kv_heads) * hd
    x = dev(torch.randn(tokens, k), torch.bfloat16)
    w = dev(torch.randn(n, k) / math.sqrt(k), torch.bfloat16)
    b = dev(torch.randn(n), torch.bfloat16) if bias else None
    table = dev(torch.from_numpy(rotary_table(10000.0, hd, 300)))
    positions = dev(torch.randint(0, 300, (tokens,), dtype=torch.int32))
    num_pages = 9
    slots = torch.randperm(num_pages * page_size)[:tokens].to(torch.int32)
    if tokens > 2:
        slots[1] = -1
    slots = dev(slots)
    error = torch.zeros(1, dtype=torch.int32, device="cuda")

    def pages():
        return torch.full((num_pages, 1, 2, kv_heads, page_size, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    want_pages, got_pages = pages(), pages()
    want = torch.empty((tokens, n), dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny(w, x, want, b)
    ops.rope_kv_write(want, positions, table, slots, want_pages[:, 0, 0], want_pages[:, 0, 1],
                      want_pages.stride(0), page_size, heads, kv_heads, hd, hd, error)
    got = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny_qkv_rope(w, x, got, b, positions, table, slots, got_pages[:, 0, 0], got_pages[:, 0, 1],
                             got_pages.stride(0), page_size, heads, kv_heads, hd, error)
    assert error.item() == 0

    def same(a, b):      # to one rounding of bfloat16 (the two kernels may contract a * c - b * s differently)
        return (a.float() - b.float()).abs().max().item() <= 2.0 ** -7 * b.float().abs().max().item()
    assert same(got[:, :heads * hd], want[:, :heads * hd])
    assert same(got_pages, want_pages)
    assert torch.equal(got_pages == 7.0, want_pages == 7.0)       # the same slots were written
    # without pages: queries only
    got = torch.full((tokens, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_skinny_qkv_rope(w, x, got, b, positions, table, None, None, None, 0, page_size, heads, kv_heads,
                             hd, error)
    assert same(got[:, :heads * hd], want[:, :heads * hd])


def test_gemm_skinny_one_element_stands_out(ops):
    """A single k position of a single row and token carries the result: a lane that pairs the
    wrong 16 bytes of x with its weights shows at once."""
    tokens, k = 7, 256
    for n, kk, row, token in ((64, 0, 0, 0), (64, 37, 9, 3), (64, 255, 63, 6), (64, 130, 24, 5),
                              (3584, 77, 24, 2), (3584, 200, 3583, 6), (3584, 1, 1816, 0)):
        x = torch.zeros(tokens, k)
        w = torch.zeros(n, k)
        x[token, kk] = 3.0
        w[row, kk] = 0.5
        out = torch.empty((tokens, n), dtype=torch.float32, device="cuda")
        ops.gemm_skinny(dev(w, torch.bfloat16), dev(x, torch.bfloat16), out, None)
        want = torch.zeros(tokens, n)
        want[token, row] = 1.5
        assert torch.equal(out.cpu(), want), (kk, row, token)
