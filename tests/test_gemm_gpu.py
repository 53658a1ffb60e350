"""GPU parity: fp32 GEMM (3xTF32 on tcgen05) against the CPU checker's tiled
matmul (tests/tri_matmul_k.py called tile by tile). Relative Frobenius error
<= 1e-5 over the compared rows."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 1e-5


def rel_fro(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want.astype(np.float64)) /
                 np.linalg.norm(want.astype(np.float64)))


def gpu_gemm(dev, a, b):
    M, K = a.shape
    _, N = b.shape
    da, db, dc = dev.upload(a), dev.upload(b), dev.alloc(M * N * 4)
    dev.gemm(dc, da, db, M, N, K)
    dev.sync()
    c = dev.download(dc, (M, N), np.float32)
    for p in (da, db, dc):
        dev.free(p)
    return c


def inputs(sm, M, N, K, seed=0xB0070003):
    a = sm.fill_host(M * K, seed, 0, 0).reshape(M, K)
    b = sm.fill_host(K * N, seed, 1, 0).reshape(K, N)
    return a, b


@pytest.mark.parametrize("M,N,K", [(128, 256, 32), (128, 256, 64), (128, 256, 96), (256, 512, 256),
                                   (384, 256, 1024), (512, 768, 512)])
def test_gemm_matches_cpu_checker(sm, dev, oracle_lib, M, N, K):
    a, b = inputs(sm, M, N, K)
    got = gpu_gemm(dev, a, b)
    want = oracle_lib.matmul(a, b)
    assert rel_fro(got, want) <= TOL
    # inject-must-fail: one wrong element in a 128x256 result is visible at this tolerance
    bad = got.copy()
    bad[M // 2, N // 3] += np.float32(1.0)
    assert rel_fro(bad, want) > TOL


def test_gemm_layout_identity_and_one_hot(sm, dev):
    """Catches a swapped operand, a transposed tile or a swizzle mismatch exactly."""
    M, N, K = 128, 256, 256
    a = sm.fill_host(M * K, 17, 0, 0).reshape(M, K)
    eye = np.eye(K, N, dtype=np.float32)
    got = gpu_gemm(dev, a, eye)
    assert np.allclose(got, a, rtol=0, atol=2e-7)
    # B = shifted permutation with distinct weights
    perm = np.zeros((K, N), np.float32)
    cols = (np.arange(K) * 7 + 3) % N
    perm[np.arange(K), cols] = np.arange(1, K + 1, dtype=np.float32)
    got = gpu_gemm(dev, a, perm)
    want = (a.astype(np.float64) @ perm.astype(np.float64))
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)


def test_gemm_argument_errors(sm, dev):
    p = dev.alloc(1 << 20)
    for M, N, K in ((0, 256, 32), (128, -1, 32), (128, 256, 0)):
        with pytest.raises(sm.Sm100Error) as e:
            dev.gemm(p, p, p, M, N, K)
        assert e.value.code == sm.ERR_ARG
    with pytest.raises(sm.Sm100Error):
        dev.gemm(0, p, p, 128, 256, 32)
    dev.free(p)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (4, 4, 4), (100, 200, 50), (129, 257, 33), (128, 256, 30),
                                   (300, 1000, 514), (1000, 1000, 1000), (2500, 260, 64), (2100, 301, 99),
                                   (2049, 515, 258), (768, 130, 4100),
                                   # a tail dealt out by K chunks whose last chunk is short (K pads to 4128 = 32 chunks + 1 block)
                                   (512, 4096, 4100)])
def test_gemm_any_size(sm, dev, oracle_lib, M, N, K):
    """Sizes that are not whole tiles: the planes are zero-padded in the workspace
    and only the M x N that exist are stored (the memory after C stays untouched).
    The CPU checker's 4x4x2 tiles need M, N % 4 == 0 and K % 2 == 0; other sizes are
    checked against a double-precision product."""
    a, b = inputs(sm, M, N, K, seed=77)
    da, db = dev.upload(a), dev.upload(b)
    guard = 64
    dc = dev.alloc((M * N + guard) * 4)
    sentinel = np.full(M * N + guard, -7.5, np.float32)
    dev.h2d(dc, sentinel)
    dev.gemm(dc, da, db, M, N, K)
    dev.sync()
    raw = dev.download(dc, M * N + guard, np.float32)
    got = raw[:M * N].reshape(M, N)
    assert np.all(raw[M * N:] == np.float32(-7.5))
    if M % 4 == 0 and N % 4 == 0 and K % 2 == 0:
        want = oracle_lib.matmul(a, b)
    else:
        want = (a.astype(np.float64) @ b.astype(np.float64))
    assert rel_fro(got, want) <= TOL
    for p in (da, db, dc):
        dev.free(p)


@pytest.mark.parametrize("M,size", [(4096, 4096), (8192, 8192), (512, 4096), (1024, 8192)])
def test_gemm_full_size_sampled_rows(sm, dev, oracle_lib, M, size):
    """N = K in {4096, 8192} with M = N (one GPU) and with the row blocks one of
    eight GPUs holds (512 x 4096 x 4096, 1024 x 8192 x 8192; the second of them, so
    A starts at row M of the global matrix): inputs generated on the device from the
    seeded stream, the CPU checker computes a seeded sample of 64 four-row blocks
    (256 rows) of C from the same stream generated on the host (rows of C are
    independent given B)."""
    N = K = size
    row0 = 0 if M == size else M                       # the shard's first row of the global A
    da, db, dc = dev.alloc(M * K * 4), dev.alloc(K * N * 4), dev.alloc(M * N * 4)
    dev.fill(da, row0 * K, M * K, 0xB0070003, 0, 0)
    dev.fill(db, 0, K * N, 0xB0070003, 1, 0)
    dev.zero(dc, M * N * 4)
    dev.gemm(dc, da, db, M, N, K)
    dev.sync()
    rng = np.random.default_rng(size + M)
    rows4 = np.sort(rng.choice(M // 4, size=64, replace=False)).astype(np.int32)
    b = sm.fill_host(K * N, 0xB0070003, 1, 0, threads=16).reshape(K, N)
    a = np.concatenate([sm.fill_host(4 * K, 0xB0070003, 0, 0, first=(row0 + 4 * int(r)) * K) for r in rows4]).reshape(256, K)
    want = oracle_lib.matmul(a, b)
    got = np.concatenate([dev.download(dc + 4 * int(r) * N * 4, (4, N), np.float32) for r in rows4])
    assert rel_fro(got, want) <= TOL
    # teeth: the same comparison notices one row block of C shifted by one block
    assert rel_fro(np.roll(got, 4, axis=0), want) > 100 * TOL
    for p in (da, db, dc):
        dev.free(p)


@pytest.mark.parametrize("clusters,shapes", [
    ("5", [(512, 768, 4096), (1024, 1024, 2048)]),     # one tail tile shared by five clusters; a tail too short to divide
    ("3", [(512, 1024, 8192), (768, 512, 1024)]),      # two tail tiles over three clusters: partial first, then owner
    ("7", [(768, 1280, 4096)]),                        # two full waves and one shared tile
])
def test_persistent_form_with_few_clusters(sm, clusters, shapes):
    """The persistent contraction's scheduling paths at sizes a test can afford: with
    the number of clusters held down (BOOTH_SM100_GEMM_CLUSTERS) a few hundred rows
    already make several waves and a tail whose K chunks are dealt out over clusters,
    including tiles shared by more than two of them and clusters that first hand a
    partial sum over and then own the next tile. Checked against a float64 product,
    for repeatability, and against the one-tile-per-cluster form (same tolerance)."""
    code = r"""
import os, sys, numpy as np, booth_b200 as sm
shapes = %r
d = sm.Device(0)
for (M, N, K) in shapes:
    a = sm.fill_host(M * K, 31, 0, 0).reshape(M, K); b = sm.fill_host(K * N, 31, 1, 0).reshape(K, N)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    da, db, dc = d.upload(a), d.upload(b), d.alloc(M * N * 4)
    outs = []
    # the persistent form twice, then one tile per cluster
    for persist in ("1", "1", "0"):
        os.environ["BOOTH_SM100_GEMM_PERSIST"] = persist
        d.zero(dc, M * N * 4)
        d.gemm(dc, da, db, M, N, K); d.sync()
        outs.append(d.download(dc, (M, N), np.float32))
    rel = [float(np.linalg.norm(o.astype(np.float64) - ref) / np.linalg.norm(ref)) for o in outs]
    print((M, N, K), "rel", ["%%.2e" %% r for r in rel], "ok", all(r <= 1e-5 for r in rel),
          "repeatable", bool(np.array_equal(outs[0], outs[1])),
          "forms agree", float(np.abs(outs[0] - outs[2]).max()) <= 1e-5 * float(np.abs(ref).max()))
    for p in (da, db, dc): d.free(p)
d.close()
""" % (shapes,)
    import subprocess, sys
    from conftest import ROOT
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=300, env=dict(os.environ, BOOTH_SM100_GEMM_CLUSTERS=clusters))
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("(")]
    assert len(lines) == len(shapes)
    for ln in lines:
        assert "ok True repeatable True forms agree True" in ln, ln


@pytest.mark.parametrize("seed,clusters", [(11, ""), (12, "13"), (13, "3")])
def test_random_shapes_against_a_double_precision_product(sm, seed, clusters):
    """Seeded random shapes (rows that make one to twelve tile rows, ragged widths, K from
    one block to several dozen chunks) through whatever contraction form the library picks,
    with the GPU's own number of clusters and with it held down: relative Frobenius error
    <= 1e-5 against a float64 product, and the call that keeps B's planes gives the same bits."""
    code = r"""
import os, numpy as np, booth_b200 as sm
rng = np.random.default_rng(%d)
d = sm.Device(0)
for it in range(8):
    M = int(rng.choice([256, 512, 768, 1024, 1280, 2048, 2304, 2500, 3000, 2049]))
    N = int(rng.integers(1, 12)) * 256 - int(rng.choice([0, 0, 0, 1, 7, 100]))
    K = int(rng.choice([32, 96, 128, 500, 512, 1000, 1024, 2048, 3000, 4096, 4100, 6144]))
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32); b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    da, db, dc = d.upload(a), d.upload(b), d.alloc(M * N * 4)
    d.gemm(dc, da, db, M, N, K); d.sync()
    c = d.download(dc, (M, N), np.float32)
    d.gemm(dc, da, db, M, N, K, b_unchanged=True); d.sync()
    c2 = d.download(dc, (M, N), np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    rel = float(np.linalg.norm(c - ref) / np.linalg.norm(ref))
    print("case", (M, N, K), "rel %%.2e" %% rel, "ok", rel <= 1e-5 and bool(np.array_equal(c, c2)))
    for p in (da, db, dc): d.free(p)
d.close()
""" % seed
    import subprocess, sys
    from conftest import ROOT
    env = dict(os.environ)
    if clusters:
        env["BOOTH_SM100_GEMM_CLUSTERS"] = clusters
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout + res.stderr
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("case")]
    assert len(lines) == 8 and all(ln.endswith("ok True") for ln in lines), res.stdout


@pytest.mark.parametrize("sa,sb", [(1e-20, 1e15), (1e30, 1e5), (1.0, 1e-30), (1e-15, 1e-15)])
def test_operand_scales_and_non_finite_values(sm, dev, sa, sb):
    """The split into a TF32 value and a TF32 remainder must hold over fp32's range, not
    only for U[-1,1): operands scaled far down and far up (products and remainders stay
    normal numbers) keep the 1e-5 relative Frobenius bound against a float64 product. An
    infinity in A turns the row of C it reaches into non-finite values (NaN: the remainder
    of an infinity is inf - inf) and leaves every other row as it was."""
    rng = np.random.default_rng(77)
    M, N, K = 512, 512, 640
    a = (rng.uniform(-1, 1, (M, K)) * sa).astype(np.float32)
    b = (rng.uniform(-1, 1, (K, N)) * sb).astype(np.float32)
    da, db, dc = dev.upload(a), dev.upload(b), dev.alloc(M * N * 4)
    dev.gemm(dc, da, db, M, N, K); dev.sync()
    c = dev.download(dc, (M, N), np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.all(np.isfinite(c))
    assert np.linalg.norm(c - ref) / np.linalg.norm(ref) <= 1e-5
    a[7, 100] = np.inf
    dev.h2d(da, a)
    dev.gemm(dc, da, db, M, N, K); dev.sync()
    c2 = dev.download(dc, (M, N), np.float32)
    assert not np.any(np.isfinite(c2[7]))
    keep = np.arange(M) != 7
    assert np.array_equal(c2[keep], c[keep])
    for p in (da, db, dc): dev.free(p)


@pytest.mark.parametrize("pair", ["1", "0"])
def test_barrier_wait_limit_reports_instead_of_hanging(sm, pair):
    """Failure detection without a fault: with the TMA producer kept silent (a
    host-side flag of the call) nothing ever signals the "operands ready" barrier, so the MMA
    issuer's and the epilogue's bounded waits run out (limit 50 ms here), the
    kernel records which wait gave up, frees its tensor memory and returns; the
    host reads the status at the next call that waits. The device stays usable.
    512 x 512 rows run the persistent pair form (pair = "1") or the one-CTA form."""
    code = r"""
import os, numpy as np, booth_b200 as sm
d = sm.Device(0)
M = N = 512; K = 256
a = sm.fill_host(M * K, 5, 0, 0); b = sm.fill_host(K * N, 5, 1, 0)
da, db, dc = d.upload(a), d.upload(b), d.alloc(M * N * 4)
d.gemm_wait_limit(50)
d.gemm(dc, da, db, M, N, K, flags=sm.GEMM_TEST_SILENT_PRODUCER)
try:
    d.download(dc, 4, np.float32); print("no error reported")       # any call that waits reports it
except sm.Sm100Error as e:
    print("reported:", e)
d.gemm_wait_limit(4000)
d.gemm(dc, da, db, M, N, K); d.sync()
c = d.download(dc, (M, N), np.float32).astype(np.float64)
ref = a.reshape(M, K).astype(np.float64) @ b.reshape(K, N).astype(np.float64)
print("after: rel", np.linalg.norm(c - ref) / np.linalg.norm(ref) < 1e-5)
d.close()
"""
    import subprocess, sys
    from conftest import ROOT
    res = subprocess.run([sys.executable, "-c", code], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                         text=True, timeout=120, env=dict(os.environ, BOOTH_SM100_GEMM_2CTA=pair))
    assert res.returncode == 0, res.stdout + res.stderr
    assert "reported:" in res.stdout and "gave up waiting on a barrier (code 2" in res.stdout + res.stderr
    assert "after: rel True" in res.stdout


def test_gemm_reuses_the_planes_of_an_unchanged_b_only_when_it_may(sm, dev, oracle_lib):
    """booth_sm100_gemm_ex with BOOTH_GEMM_B_UNCHANGED: same result as the full call
    when B is unchanged; the flag is ignored when the pointer or the shape differ;
    and it does what it says when the caller lies (the old B is used), which shows
    the planes really were reused."""
    M, N, K = 256, 512, 160
    a = sm.fill_host(M * K, 71, 0, 0).reshape(M, K)
    b1 = sm.fill_host(K * N, 71, 1, 0).reshape(K, N)
    b2 = sm.fill_host(K * N, 71, 2, 0).reshape(K, N)
    da, db, db2, dc = dev.upload(a), dev.upload(b1), dev.upload(b2), dev.alloc(M * N * 4)
    want1 = oracle_lib.matmul(a, b1).astype(np.float64)
    want2 = oracle_lib.matmul(a, b2).astype(np.float64)

    def run(bptr, flag, n=N):
        dev.zero(dc, M * N * 4)
        dev.gemm(dc, da, bptr, M, n, K, b_unchanged=flag)
        dev.sync()
        return dev.download(dc, (M, N), np.float32).astype(np.float64)

    def close(got, want):
        return np.linalg.norm(got - want) <= 1e-5 * np.linalg.norm(want)

    assert close(run(db, True), want1)            # nothing to reuse yet: splits B
    assert close(run(db, True), want1)            # reuses
    assert close(run(db2, True), want2)           # other pointer: flag ignored
    assert close(run(db2, True), want2)
    dev.h2d(db2, b1)                              # B changes behind the library's back ...
    assert close(run(db2, True), want2)           # ... and the flag keeps the old planes, as documented
    assert close(run(db2, False), want1)          # the plain call sees the new contents
    for p in (da, db, db2, dc):
        dev.free(p)
