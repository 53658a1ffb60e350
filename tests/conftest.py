"""Shared fixtures. Tests marked ``gpu`` need a B200 and call the product through
its C ABI; everything else runs on a CPU-only machine."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
# The reference tree, when present: BOOTH_REF, else a checkout named "reference"
# beside this repository. Tests that need it skip their reference half without it.
REFERENCE = os.environ.get("BOOTH_REF") or os.path.join(os.path.dirname(ROOT), "reference")


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


# Known-answer vectors of Philox4x32-10 as published with the Random123 library
# (Salmon, Moraes, Dror, Shaw, SC'11; its kat_vectors file): (counter, key, output).
PHILOX_KAT = (
    ((0x00000000, 0x00000000, 0x00000000, 0x00000000), (0x00000000, 0x00000000),
     (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
    ((0xffffffff, 0xffffffff, 0xffffffff, 0xffffffff), (0xffffffff, 0xffffffff),
     (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
    ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
     (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
)


def philox_np(ctr, seed, stream, c2=0, c3=0):
    """Philox4x32-10 in numpy: counter (ctr low, ctr high, c2, c3), key (seed, stream).
    Independent restatement used to pin the C and CUDA generators."""
    ctr = np.asarray(ctr, dtype=np.uint64)
    c0 = (ctr & np.uint64(0xFFFFFFFF)).astype(np.uint64)
    c1 = (ctr >> np.uint64(32)).astype(np.uint64)
    c2 = np.zeros_like(c0) + np.uint64(c2)
    c3 = np.zeros_like(c0) + np.uint64(c3)
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
    if kind == 3:
        return x
    u = (x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)
    return (np.float32(2) * u - np.float32(1)) if kind == 0 else u
