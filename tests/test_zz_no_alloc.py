"""The allocation-free entry point of split-context decode attention, called through its
exported C symbol, against the ordinary entry point (which takes scratch from the caller).

Some hosts of the kernel library cannot allocate device memory where they call it: inside a
stream capture, in a loop with a fixed memory budget, or from a foreign runtime that can only
pass pointers it already owns.  For them the library keeps a fixed 4 MiB scratch array of its
own.  This test calls the symbol twice in a row with different inputs: the array is shared by
all calls and keeps the previous call's contents, which must not leak into the next result.
It runs last, alone in a fresh process or after every other test.
"""
import ctypes
import math
import random

import pytest
import torch

from citlali_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(seed, lengths, nq, nkv, d, page=64):
    g = torch.Generator().manual_seed(seed)
    B = len(lengths)
    pages_per = [(n + page - 1) // page for n in lengths]
    total = sum(pages_per) + 2
    order = list(range(total)); random.Random(seed).shuffle(order)
    table = torch.zeros(B, max(pages_per) + 1, dtype=torch.int32)
    nxt = 0
    for b, n in enumerate(pages_per):
        for i in range(n):
            table[b, i] = order[nxt]; nxt += 1
    kp = torch.randn(total, nkv, page, d, generator=g).to(torch.bfloat16).to(DEV)
    vp = torch.randn(total, nkv, page, d, generator=g).to(torch.bfloat16).to(DEV)
    q = (torch.randn(B, nq * d, generator=g) * 2).to(torch.bfloat16).to(DEV)
    slots = torch.arange(B, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lengths], dtype=torch.int32, device=DEV)
    return q, kp, vp, table.to(DEV), slots, pos


def _no_alloc(lib, q, kp, vp, table, slots, pos, out, nq, nkv, d, page, max_positions, window=0):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    i = ctypes.c_int
    return lib.citlali_attention_decode_no_alloc(
        p(q), i(q.shape[1]), p(kp), p(vp), p(table), i(table.shape[1]), p(slots), p(pos), p(out), i(out.shape[1]),
        i(out.shape[0]), i(nq), i(nkv), i(d), i(page), i(window), i(max_positions), ctypes.c_float(1.0 / math.sqrt(d)),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_no_alloc_entry_point_matches_the_ordinary_one_on_two_calls_in_a_row():
    lib = ops.lib()
    assert hasattr(lib, "citlali_attention_decode_no_alloc")
    nq, nkv, d = 8, 2, 64
    # pages of 16 keys take the kernel pair that keeps per-chunk partials in the scratch array; pages of 64 take the
    # cluster kernel, which leaves the array alone.  Within each pair the second call sees what the first one left.
    # The last two calls attend to a window of keys only (chunks before the window are skipped).  Both entry
    # points run the same kernels on the same inputs, so the results are equal bit for bit.
    for seed, lengths, page, window in ((1, [700, 3, 257, 64], 16, 0), (2, [5, 130, 1, 300], 16, 0),
                                        (3, [700, 3, 257, 64], 64, 0), (4, [5, 130, 1, 300], 64, 0),
                                        (5, [700, 3, 257, 64], 16, 100), (6, [5, 130, 1, 300], 64, 37)):
        q, kp, vp, table, slots, pos = _case(seed, lengths, nq, nkv, d, page)
        max_positions = table.shape[1] * page
        want = torch.empty(len(lengths), nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_decode(q, q.shape[1], kp, vp, table, slots, pos, want, nq, nkv, d, page, window, max_positions,
                             1.0 / math.sqrt(d))
        got = torch.full_like(want, float("nan"))
        rc = _no_alloc(lib, q, kp, vp, table, slots, pos, got, nq, nkv, d, page, max_positions, window)
        assert rc == 0, lib.citlali_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call with seed {seed}: the two entry points differ"


def test_no_alloc_entry_point_at_the_edge_of_its_array():
    """The largest call the array holds is accepted and right; one chunk more is refused.  (A call's need is
    a multiple of head size + 2, which divides no power of two for a legal head size: no call needs exactly
    the array's 2^20 floats.  2 rows x 13 heads x 611 chunks x 66 is 100 floats short of it.)"""
    lib = ops.lib()
    lib.citlali_attention_decode_scratch_floats.restype = ctypes.c_size_t
    nq, nkv, d, page = 13, 13, 64, 16
    chunks = 611
    max_positions = chunks * 2 * page
    i = ctypes.c_int
    assert lib.citlali_attention_decode_scratch_floats(i(2), i(nq), i(d), i(page), i(max_positions)) == (1 << 20) - 100
    assert lib.citlali_attention_decode_scratch_floats(i(2), i(nq), i(d), i(page), i(max_positions + 1)) > (1 << 20)
    q, kp, vp, table, slots, pos = _case(7, [max_positions, 301], nq, nkv, d, page)
    want = torch.empty(2, nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(q, q.shape[1], kp, vp, table, slots, pos, want, nq, nkv, d, page, 0, max_positions,
                         1.0 / math.sqrt(d))
    got = torch.full_like(want, float("nan"))
    rc = _no_alloc(lib, q, kp, vp, table, slots, pos, got, nq, nkv, d, page, max_positions)
    assert rc == 0, lib.citlali_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    out = torch.zeros_like(want)
    rc = _no_alloc(lib, q, kp, vp, table, slots, pos, out, nq, nkv, d, page, max_positions + 1)
    assert rc < 0 and "built-in array holds 1048576" in lib.citlali_last_error().decode()
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0


def test_no_alloc_entry_point_refuses_what_exceeds_its_array():
    lib = ops.lib()
    nq, nkv, d, page = 32, 8, 128, 64
    q, kp, vp, table, slots, pos = _case(3, [10, 20], nq, nkv, d, page)
    out = torch.zeros(2, nq * d, dtype=torch.bfloat16, device=DEV)
    rc = _no_alloc(lib, q, kp, vp, table, slots, pos, out, nq, nkv, d, page, 1 << 20)      # a million positions
    assert rc < 0 and "built-in array holds 1048576" in lib.citlali_last_error().decode()
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0                                           # nothing was launched
