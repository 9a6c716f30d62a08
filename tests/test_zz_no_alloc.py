"""The attention entry point for callers that cannot allocate device memory.

`fsie_attn_generic_static_scratch` keeps the partial results of a split key range in a
fixed array inside the library instead of buffers from the caller - for a process whose
GPU memory is all given to the page pool already, for a step loop that must not take the
device-wide synchronisation of cudaMalloc and cudaFree, and for a C program that uses
the library without torch.  This test calls it the way such a caller does: through the
exported C symbol of the shared object, with raw pointers, and checks its output against
the ordinary entry point (whose scratch the test allocates) on two calls in a row with
different inputs, since the array keeps what the last call left in it.

It is collected last on purpose: a run that stops at the first failure has then already
run every other test.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20
TOO_SMALL = -3


@pytest.fixture(scope="module")
def lib():
    from from_scratch_inference_engine_b200.csrc import build
    handle = ctypes.CDLL(str(build.library_path("core")))
    i, f, ll, p = ctypes.c_int, ctypes.c_float, ctypes.c_longlong, ctypes.c_void_p
    handle.fsie_attn_generic_static_scratch.argtypes = [
        p, i, p, p, ll, i, p, i, p, p, i, p, p, p, p, i, i, i, i, i, i, i, f, i, p]
    handle.fsie_attn_generic_static_scratch.restype = i
    handle.fsie_attn_static_scratch_floats.argtypes = [i, i, i, i]
    handle.fsie_attn_static_scratch_floats.restype = ll
    handle.fsie_attn_static_scratch_error.argtypes = [i]
    handle.fsie_attn_static_scratch_error.restype = ctypes.c_char_p
    return handle


def call_both(lib, case, nsplit):
    """Outputs of the ordinary entry point and of the static-scratch one for one case."""
    from from_scratch_inference_engine_b200.kernels import ops
    want = case.run(ops, nsplit)                       # ordinary entry, scratch from torch
    group = case.heads // case.kv_heads
    rows = ops.attention_rows_per_tile()
    tile_item, tile_row0, qstart, at = [], [], [], 0
    for index, (_, new) in enumerate(case.items):
        qstart.append(at)
        at += new
        for r0 in range(0, new * group, rows):
            tile_item.append(index)
            tile_row0.append(r0)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    pages, q, tables = case.pages.cuda(), case.q.cuda(), case.tables.cuda()
    meta = [i32(tile_item), i32(tile_row0), i32(qstart), i32([n for _, n in case.items]),
            i32([p for p, _ in case.items])]
    tokens = q.shape[0]
    out = torch.full((tokens, case.heads * case.hd), float("nan"), dtype=q.dtype, device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    code = lib.fsie_attn_generic_static_scratch(
        ptr(q), q.stride(0), ptr(pages[:, 0, 0]), ptr(pages[:, 0, 1]), pages.stride(0),
        case.page_size, ptr(tables), tables.stride(0), ptr(meta[0]), ptr(meta[1]),
        len(tile_item), ptr(meta[2]), ptr(meta[3]), ptr(meta[4]), ptr(out), out.stride(0),
        tokens, case.heads, case.kv_heads, case.hd, case.window, nsplit,
        1.0 / math.sqrt(case.hd), 0 if q.dtype is torch.float32 else 1,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return code, out.cpu().double(), want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_matches_the_ordinary_one_twice_in_a_row(lib, dtype):
    from test_gpu_kernels import PagedCase, assert_rows_close
    first = PagedCase(dtype, 14, 2, 64, 16, items=[(700, 1), (0, 3), (301, 1), (33, 2)], seed=21)
    second = PagedCase(dtype, 14, 2, 64, 16, items=[(90, 2), (512, 1), (5, 1)], seed=22)
    for case, nsplit in ((first, 6), (second, 3), (second, 1)):
        need = lib.fsie_attn_static_scratch_floats(case.q.shape[0], case.heads, case.hd, nsplit)
        assert need <= SCRATCH_FLOATS
        code, got, want = call_both(lib, case, nsplit)
        assert code == 0, lib.fsie_attn_static_scratch_error(code).decode()
        assert torch.isfinite(got).all()
        assert_rows_close(got, want, case, dtype)               # against the ordinary entry
        assert_rows_close(got, case.want, case, dtype)          # and against the plain answer


def test_static_scratch_entry_refuses_what_does_not_fit(lib):
    from test_gpu_kernels import PagedCase
    case = PagedCase(torch.float32, 32, 2, 128, 16, items=[(40, 40)], seed=23)
    nsplit = 8          # 8 * 40 * 32 * 130 floats = 1,331,200 > 1,048,576
    assert lib.fsie_attn_static_scratch_floats(40, 32, 128, nsplit) > SCRATCH_FLOATS
    code, got, _ = call_both(lib, case, nsplit)
    assert code == TOO_SMALL
    assert b"more split scratch" in lib.fsie_attn_static_scratch_error(code)
    assert torch.isnan(got).all()                               # nothing ran


def test_static_scratch_entry_at_exactly_its_limit_and_without_allocating(lib):
    """8 splits x 128 tokens x 16 heads x (62 + 2) floats are exactly the 1,048,576 the
    array holds.  The device's free memory is read before and after a repeated call: a caller
    that has no memory left to give must not lose any to this entry point."""
    from test_gpu_kernels import PagedCase, assert_rows_close
    case = PagedCase(torch.float32, 16, 2, 62, 16, items=[(300, 100), (900, 28)], seed=24)
    assert lib.fsie_attn_static_scratch_floats(128, 16, 62, 8) == SCRATCH_FLOATS
    code, got, want = call_both(lib, case, 8)              # first call: set-up may happen here
    assert code == 0, lib.fsie_attn_static_scratch_error(code).decode()
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    code, again, _ = call_both(lib, case, 8)
    free_after, _ = torch.cuda.mem_get_info()
    # what torch itself reserved for the test's own tensors is not the entry point's doing
    grown_by_torch = torch.cuda.memory_reserved() - reserved_before
    assert free_before - free_after <= grown_by_torch
    for out in (got, again):
        assert_rows_close(out, want, case, torch.float32)
        assert_rows_close(out, case.want, case, torch.float32)
    # one more split does not fit, and absurd sizes are cut off instead of wrapping around
    assert lib.fsie_attn_static_scratch_floats(128, 16, 62, 9) > SCRATCH_FLOATS
    assert lib.fsie_attn_static_scratch_floats(2**31 - 1, 2**31 - 1, 2**31 - 3, 2**31 - 1) == SCRATCH_FLOATS + 1
    assert lib.fsie_attn_static_scratch_floats(-5, 4, 64, 2) == -1
