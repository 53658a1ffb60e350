"""GPU parity: the global sum. int32 is bit-exact (wrapping), fp32 within 1e-6
relative of the CPU checker's chunked sum."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

SIZES = [0, 1, 2, 3, 4, 5, 31, 32, 33, 255, 256, 257, 4095, 4096, 4097, 65535, (1 << 20) + 7, (1 << 24) + 1]
REL = 1e-6


def wrap32(s):
    s &= 0xFFFFFFFF
    return s - (1 << 32) if s >= (1 << 31) else s


def gpu_sum_i32(dev, p, n):
    out = dev.alloc(8)
    dev.reduce_i32(p, n, out)
    v = int(dev.download(out, 1, np.int32)[0])
    dev.free(out)
    return v


def gpu_sum_f32(dev, p, n):
    out = dev.alloc(8)
    dev.reduce_f32(p, n, out)
    v = float(dev.download(out, 1, np.float64)[0])
    dev.free(out)
    return v


@pytest.mark.parametrize("n", SIZES)
def test_int32_sum_bit_exact(sm, dev, oracle_lib, n):
    v = sm.fill_host(max(n, 1), 0xB0070002, 0, 2)[:n].copy()
    p = dev.upload(v) if n else dev.alloc(4)
    got = gpu_sum_i32(dev, p, n)
    want = oracle_lib.reduce_i32(v) if n else 0
    assert got == want
    assert got == wrap32(int(np.sum(v.astype(np.int64))))
    dev.free(p)


def test_int32_sum_wraps_like_the_reference(sm, dev, oracle_lib):
    v = np.full(1 << 16, 2 ** 31 - 1, np.int32)          # sum overflows many times
    p = dev.upload(v)
    assert gpu_sum_i32(dev, p, v.size) == oracle_lib.reduce_i32(v)
    dev.free(p)


@pytest.mark.parametrize("n", SIZES[1:])
def test_fp32_sum_within_1e6(sm, dev, oracle_lib, n):
    v = sm.fill_host(n, 0xB0070002, 1, 1)
    p = dev.upload(v)
    got = gpu_sum_f32(dev, p, n)
    want = oracle_lib.reduce_f32(v)
    truth = oracle_lib.sum_f64(v)
    assert abs(np.float32(got) - np.float32(want)) <= REL * abs(want)
    assert abs(got - truth) <= REL * abs(truth)
    dev.free(p)


def test_unaligned_input_and_repeat_launches(sm, dev, oracle_lib):
    n = 100003
    vi = sm.fill_host(n + 3, 11, 0, 2)
    vf = sm.fill_host(n + 3, 11, 1, 1)
    pi, pf = dev.upload(vi), dev.upload(vf)
    for rep in range(3):                     # the arrival counter must return to zero
        for off in (0, 1, 2, 3):
            assert gpu_sum_i32(dev, pi + 4 * off, n) == oracle_lib.reduce_i32(vi[off:off + n].copy())
            want = oracle_lib.reduce_f32(vf[off:off + n].copy())
            assert abs(gpu_sum_f32(dev, pf + 4 * off, n) - want) <= REL * abs(want)
    dev.free(pi); dev.free(pf)


def test_reference_fixture_ones(sm, dev):
    # tests/build/gpu_reduce.c:33-60: a[i] = 1 sums to N
    for n in (16, 1024, 100000):
        p = dev.upload(np.ones(n, np.float32))
        assert gpu_sum_f32(dev, p, n) == float(n)
        q = dev.upload(np.ones(n, np.int32))
        assert gpu_sum_i32(dev, q, n) == n
        dev.free(p); dev.free(q)


def test_reproducible(sm, dev):
    n = (1 << 22) + 5
    p = dev.alloc(n * 4)
    dev.fill(p, 0, n, 77, 0, 1)
    a = gpu_sum_f32(dev, p, n)
    assert all(gpu_sum_f32(dev, p, n) == a for _ in range(3))
    dev.free(p)


def test_full_size_2_30(sm, dev, oracle_lib):
    """N = 2^30, both variants, against the CPU checker on the same stream."""
    n = 1 << 30
    p = dev.alloc(n * 4)
    dev.fill(p, 0, n, 0xB0070002, 0, 2)
    got_i = gpu_sum_i32(dev, p, n)
    host = sm.fill_host(n, 0xB0070002, 0, 2, threads=oracle_lib.cores)
    assert got_i == oracle_lib.reduce_i32(host)
    dev.fill(p, 0, n, 0xB0070002, 1, 1)
    got_f = gpu_sum_f32(dev, p, n)
    host = sm.fill_host(n, 0xB0070002, 1, 1, threads=oracle_lib.cores)
    want = oracle_lib.reduce_f32(host)
    truth = oracle_lib.sum_f64(host)
    assert abs(np.float32(got_f) - np.float32(want)) <= REL * abs(want)
    assert abs(got_f - truth) <= REL * abs(truth)
    dev.free(p)


def test_bad_addresses_are_refused_on_the_host(sm, dev):
    """A result address that is not aligned to the result's size, or a NULL input
    with n > 0, would fault on the device; the calls return SM100_ERR_ARG before
    any GPU work and the device stays usable."""
    x, out = dev.alloc(4096), dev.alloc(64)
    L = sm.lib()
    assert L.booth_sm100_reduce_f32(dev.handle, x, 100, out + 4) == sm.ERR_ARG
    assert L.booth_sm100_reduce_i32(dev.handle, x, 100, out + 2) == sm.ERR_ARG
    assert L.booth_sm100_reduce_f32(dev.handle, 0, 100, out) == sm.ERR_ARG
    assert L.booth_sm100_reduce_i32(dev.handle, x + 1, 100, out) == sm.ERR_ARG
    assert L.booth_sm100_asian(dev.handle, sm.asian_params(), 0, 1000, out + 4) == sm.ERR_ARG
    dev.zero(x, 4096)
    dev.reduce_i32(x, 1024, out + 4)                     # 4-byte alignment is enough for the int32 sum
    assert int(dev.download(out + 4, 1, np.int32)[0]) == 0
    dev.free(x); dev.free(out)
