"""GPU parity: the Asian-option Monte Carlo pricer against the CPU checker on the
same Philox stream. Prices within 1e-5 relative; the geometric price also
against its closed form."""
import math

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL = 1e-5
DISC = math.exp(-0.05)


def closed_form_geometric(s0=100.0, k=100.0, r=0.05, sigma=0.2, T=1.0, n=252):
    mu = (r - 0.5 * sigma * sigma) * T * (n + 1) / (2.0 * n)
    var = sigma * sigma * T * (n + 1) * (2 * n + 1) / (6.0 * n * n)
    sg = math.sqrt(var)
    d2 = (math.log(s0 / k) + mu) / sg
    d1 = d2 + sg
    N = lambda x: 0.5 * (1.0 + math.erf(x / math.sqrt(2.0)))
    return math.exp(-r * T) * (s0 * math.exp(mu + 0.5 * var) * N(d1) - k * N(d2))


def gpu_sums(dev, params, path0, npaths):
    out = dev.alloc(32)
    dev.asian(params, path0, npaths, out)
    v = dev.download(out, 4, np.float64)
    dev.free(out)
    return v


@pytest.mark.parametrize("precise", [1, 0])
def test_price_matches_cpu_checker(sm, dev, oracle_lib, precise):
    npaths = 1 << 18
    prm = sm.asian_params(precise=precise)
    s = gpu_sums(dev, prm, 0, npaths)
    oa, og = oracle_lib.asian(prm, 0, npaths)
    assert abs(s[0] - oa) <= REL * oa, (s[0] / npaths * DISC, oa / npaths * DISC)
    assert abs(s[1] - og) <= REL * og, (s[1] / npaths * DISC, og / npaths * DISC)


@pytest.mark.parametrize("precise", [1, 0])
def test_per_path_payoffs(sm, dev, oracle_lib, precise):
    npaths = 1 << 14
    prm = sm.asian_params(precise=precise)
    da, dg = dev.alloc(npaths * 4), dev.alloc(npaths * 4)
    dev.asian_paths(prm, 123456789, npaths, da, dg)
    ga, gg = dev.download(da, npaths, np.float32), dev.download(dg, npaths, np.float32)
    _, _, oa, og = oracle_lib.asian(prm, 123456789, npaths, per_path=True)
    # A path's payoff is about 100*(relative error of S): transcendental
    # implementations differ by a few ulp per step, so per path we only ask for
    # agreement to 2e-3 absolute on a price of order 100; the mean must agree
    # far more tightly (the 1e-5 test above).
    assert np.max(np.abs(ga - oa)) < 2e-3 and np.max(np.abs(gg - og)) < 2e-3
    assert np.count_nonzero((ga > 0) != (oa > 0)) <= 2
    # the reduced sums are the per-path payoffs added in double
    s = gpu_sums(dev, prm, 123456789, npaths)
    assert abs(s[0] - ga.astype(np.float64).sum()) <= 1e-9 * s[0]
    assert abs(s[1] - gg.astype(np.float64).sum()) <= 1e-9 * s[1]
    assert abs(s[2] - (ga.astype(np.float64) ** 2).sum()) <= 1e-9 * s[2]
    dev.free(da); dev.free(dg)


def test_disjoint_subsequences_add_up(sm, dev):
    prm = sm.asian_params()
    n = 100000
    whole = gpu_sums(dev, prm, 0, n)
    parts = sum(gpu_sums(dev, prm, lo, hi - lo) for lo, hi in ((0, 33333), (33333, 70001), (70001, n)))
    assert np.allclose(whole, parts, rtol=1e-12, atol=0)
    assert np.all(gpu_sums(dev, prm, 0, 0) == 0)


def test_geometric_price_vs_closed_form(sm, dev):
    npaths = 1 << 22
    prm = sm.asian_params()
    s = gpu_sums(dev, prm, 0, npaths)
    mean = s[1] / npaths
    var = s[3] / npaths - mean * mean
    se = DISC * math.sqrt(var / npaths)
    price = DISC * mean
    cf = closed_form_geometric()
    assert abs(cf - 5.5655) < 1e-3
    assert abs(price - cf) < 4 * se, (price, cf, se)
    # arithmetic average >= geometric average, path by path, hence in the mean
    assert s[0] > s[1]


def test_path_index_above_2_32(sm, dev, oracle_lib):
    prm = sm.asian_params(precise=1)
    p0 = (1 << 32) + 5
    s = gpu_sums(dev, prm, p0, 4096)
    oa, og = oracle_lib.asian(prm, p0, 4096)
    assert abs(s[0] - oa) <= 1e-4 * oa and abs(s[1] - og) <= 1e-4 * og


@pytest.mark.parametrize("precise", [1, 0])
@pytest.mark.parametrize("kw", [
    dict(nstep=4), dict(nstep=12, sigma=0.8), dict(nstep=1000, sigma=0.05),            # few / many monitoring steps
    dict(sigma=0.0),                                                                   # no noise: every path is the same
    dict(strike=60.0), dict(strike=140.0, sigma=0.4),                                  # deep in and out of the money
    dict(s0=0.5, strike=0.5, r=0.0), dict(s0=2.5e4, strike=2.4e4, r=0.11, T=3.0),      # other scales and horizons
    dict(k0=7, k1=0xFFFFFFFF),                                                         # another key
])
def test_other_contracts_and_step_counts(sm, dev, oracle_lib, precise, kw):
    """The benchmark prices one contract (S0 = K = 100, 252 steps); the kernel takes any.
    Other step counts (any multiple of 4), volatilities down to zero, strikes far from the
    money, other scales, rates, horizons and Philox keys against the CPU checker on the same
    stream: both sums within 1e-5 relative (within 1e-7 of the notional where a payoff sum
    is nearly zero)."""
    npaths = 1 << 15
    prm = sm.asian_params(precise=precise, **kw)
    s = gpu_sums(dev, prm, 1000, npaths)
    oa, og = oracle_lib.asian(prm, 1000, npaths)
    floor = 1e-7 * npaths * float(prm.s0)
    if kw.get("sigma") == 0.0 and not precise:
        # Without noise every step multiplies the price by the same factor, and the CPU statement's
        # fp32 chain s *= exp(x) then rounds the same way 252 times: its arithmetic price is 2.6e-4
        # off the exact value (2.55302 against 2.552366 here). The MUFU flavour rebuilds the price from
        # its running logarithm and does not share that drift, so it is held against the exact value
        # (computed in double from the same fp32 drift), and the checker's own distance is recorded.
        n, d = prm.nstep, float(prm.drift)
        exact_a = npaths * (float(prm.s0) * sum(math.exp(d * j) for j in range(1, n + 1)) / n - float(prm.strike))
        exact_g = npaths * (float(prm.s0) * math.exp(d * (n + 1) / 2.0) - float(prm.strike))
        assert abs(s[0] - exact_a) <= REL * exact_a and abs(s[1] - exact_g) <= REL * exact_g
        assert abs(oa - exact_a) > 10 * abs(s[0] - exact_a)
        return
    assert abs(s[0] - oa) <= max(REL * oa, floor), (kw, s[0] / npaths, oa / npaths)
    assert abs(s[1] - og) <= max(REL * og, floor), (kw, s[1] / npaths, og / npaths)
    assert oa >= og - floor                       # arithmetic mean >= geometric mean, also on the checker's side


def test_step_counts_that_are_not_multiples_of_four_are_refused(sm, dev):
    out = dev.alloc(32)
    for nstep in (0, 1, 250, -4):
        prm = sm.asian_params(nstep=max(nstep, 1))
        prm.nstep = nstep
        with pytest.raises(sm.Sm100Error) as e:
            dev.asian(prm, 0, 16, out)
        assert e.value.code == sm.ERR_ARG
    dev.free(out)


@pytest.mark.parametrize("precise", [1, 0])
def test_same_bits_run_to_run(sm, dev, precise):
    """No float atomics anywhere: per-thread double sums, a shuffle tree, and the block
    that draws the last ticket adds the block partials in index order. Two runs of the
    same launch give the same four doubles, bit for bit."""
    prm = sm.asian_params(precise=precise)
    first = gpu_sums(dev, prm, 12345, 300001)
    for _ in range(3):
        assert np.array_equal(gpu_sums(dev, prm, 12345, 300001).view(np.uint64), first.view(np.uint64))


def test_pipe_probe_kernels_run_and_order_as_expected(sm, dev):
    """The three probe kernels of the image (kernels/pipe_probe.cu) that bench.py times for the
    pricer's second roofline: they load by name, run, leave their scratch word alone (they
    write only on an impossible sum), and the two instruction groups together take longer
    than either alone but less than one after the other."""
    import ctypes as C
    L = sm.lib()
    scratch = dev.alloc(64)
    dev.zero(scratch, 64)
    ms = {}
    for name in ("probe_mufu", "probe_imad_wide", "probe_mufu_imad_wide"):
        k = sm.Kern()
        assert L.sm100_rt_load_builtin(dev.handle, name.encode(), C.byref(k)) == 0
        vals = [C.c_uint64(scratch), C.c_int(512), C.c_float(0.999), C.c_uint32(12345)]
        argv = (C.c_void_p * len(vals))(*[C.cast(C.byref(v), C.c_void_p) for v in vals])
        grid = dev.sm_count * 8
        for _ in range(2):
            assert L.sm100_rt_launch(dev.handle, C.byref(k), grid, 1, 1, 256, 1, 1, 0, argv) == 0
        dev.sync(); dev.tic()
        for _ in range(4):
            assert L.sm100_rt_launch(dev.handle, C.byref(k), grid, 1, 1, 256, 1, 1, 0, argv) == 0
        ms[name] = dev.toc() / 4
        L.sm100_rt_unload(dev.handle, C.byref(k))
    assert np.all(dev.download(scratch, 16, np.uint32) == 0)
    both, a, b = ms["probe_mufu_imad_wide"], ms["probe_mufu"], ms["probe_imad_wide"]
    assert both > 0.95 * max(a, b) and both < 1.05 * (a + b), ms
    dev.free(scratch)
