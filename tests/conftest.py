"""Shared fixtures. Tests marked ``gpu`` need a B200 and call the product through
its C ABI; everything else runs on a CPU-only machine."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def sm():
    import booth_b200
    if not os.path.exists(booth_b200.LIB_PATH):
        from booth_b200 import build
        build.build()
    booth_b200.lib()
    return booth_b200


@pytest.fixture(scope="session")
def oracle_lib():
    """The CPU checker: the reference compiler's own objects when they are built,
    else the C restatement."""
    import oracle
    return oracle.load()


@pytest.fixture(scope="session")
def dev(sm):
    """One device for the whole session. No skip: a GPU test without a working
    B200 path must fail, not pass silently."""
    d = sm.Device(0)
    yield d
    d.close()


def philox_np(ctr, seed, stream):
    """Philox4x32-10 in numpy: counter (ctr low, ctr high, 0, 0), key (seed, stream).
    Independent restatement used to pin the C and CUDA generators."""
    ctr = np.asarray(ctr, dtype=np.uint64)
    c0 = (ctr & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (ctr >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = np.uint64(seed), np.uint64(stream)
    M0, M1, MASK = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & MASK
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ k1) & MASK
        c0, c1, c2, c3 = n0, p1 & MASK, n2, p0 & MASK
        k0 = (k0 + np.uint64(0x9E3779B9)) & MASK
        k1 = (k1 + np.uint64(0xBB67AE85)) & MASK
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def fill_np(first, n, seed, stream, kind):
    """numpy statement of the seeded input stream (include/booth_sm100.h)."""
    idx = np.arange(first, first + n, dtype=np.uint64)
    words = philox_np(idx >> np.uint64(2), seed, stream)
    x = words[np.arange(n), (idx & np.uint64(3)).astype(np.int64)]
    if kind == 2:
        return (x % np.uint32(2001)).astype(np.int32) - np.int32(1000)
    u = (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)
    return (np.float32(2) * u - np.float32(1)) if kind == 0 else u
