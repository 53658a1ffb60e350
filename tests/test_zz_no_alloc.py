"""GPU: the allocation-free fp32 sum (booth_sm100_reduce_f32_noalloc).

Some callers cannot allocate device memory when they need the sum (a frozen
memory pool, a real-time loop, a plug-in whose host owns the GPU's memory), so
this entry point takes no device handle and keeps its scratch in an array built
into the library. It must agree with the regular booth_sm100_reduce_f32 within
the tolerance the reduction tests use, on consecutive calls (the built-in array
is reused and keeps the previous call's contents).

This file is collected last on purpose: a run that stops at the first failure
has then already run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL = 1e-6


def regular(dev, p, n):
    out = dev.alloc(8)
    dev.reduce_f32(p, n, out)
    v = float(dev.download(out, 1, np.float64)[0])
    dev.free(out)
    return v


def noalloc(sm, dev, p, n, out):
    # On the device's own stream, so the call is ordered after the upload of the
    # input and before the copy that reads the result back.
    rc = sm.lib().booth_sm100_reduce_f32_noalloc(p, n, out, dev.stream)
    assert rc == sm.OK
    return float(dev.download(out, 1, np.float64)[0])


def test_two_calls_in_a_row_match_the_regular_entry_point(sm, dev):
    out = dev.alloc(8)
    for n, seed in (((1 << 22) + 5, 21), (300001, 22)):          # two calls, back to back, different sizes
        v = sm.fill_host(n, seed, 1, 1)
        p = dev.upload(v)
        want = regular(dev, p, n)
        got = noalloc(sm, dev, p, n, out)
        assert abs(got - want) <= REL * abs(want), (n, got, want)
        assert abs(got - float(v.astype(np.float64).sum())) <= REL * abs(want)
        # same input again: the array still holds the previous call's segment sums
        assert noalloc(sm, dev, p, n, out) == got
        dev.free(p)
    dev.free(out)


def test_small_ragged_and_unaligned_inputs(sm, dev):
    out = dev.alloc(8)
    v = sm.fill_host(70003, 23, 1, 1)
    p = dev.upload(v)
    for off, n in ((0, 0), (0, 1), (1, 5), (3, 70000), (0, 65536), (2, 262145 - 200000)):
        want = float(v[off:off + n].astype(np.float64).sum())
        got = noalloc(sm, dev, p + 4 * off, n, out)
        assert abs(got - want) <= REL * max(abs(want), 1e-30), (off, n)
    dev.free(p); dev.free(out)


def test_sizes_beyond_the_built_in_scratch_are_refused(sm, dev):
    out = dev.alloc(8)
    p = dev.alloc(1024)
    L = sm.lib()
    assert L.booth_sm100_reduce_f32_noalloc(p, (1 << 30) + 1, out, None) == sm.ERR_ARG
    assert L.booth_sm100_reduce_f32_noalloc(p, -1, out, None) == sm.ERR_ARG
    assert L.booth_sm100_reduce_f32_noalloc(p, 16, 0, None) == sm.ERR_ARG
    # a result address that is not 8-byte aligned would fault on the device: refused on the host
    assert L.booth_sm100_reduce_f32_noalloc(p, 16, out + 4, None) == sm.ERR_ARG
    assert L.booth_sm100_reduce_f32_noalloc(p + 2, 16, out, None) == sm.ERR_ARG
    assert L.booth_sm100_reduce_f32_noalloc(0, 16, out, None) == sm.ERR_ARG
    dev.free(p); dev.free(out)


def test_full_capacity(sm, dev):
    """n = 2^30, the most the built-in scratch takes (4096 segments)."""
    n = 1 << 30
    p = dev.alloc(n * 4)
    dev.fill(p, 0, n, 0xB0070002, 1, 1)
    out = dev.alloc(8)
    want = regular(dev, p, n)
    got = noalloc(sm, dev, p, n, out)
    assert abs(got - want) <= REL * want
    dev.free(p); dev.free(out)
