"""The numeric manifest (tests/numeric): two-axis verdicts in the style of the
reference's tests/numeric/run_numeric.py, with inject-must-fail teeth."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

RUN = [sys.executable, os.path.join(ROOT, "tests", "numeric", "run_numeric.py")]


def run(*args):
    return subprocess.run(RUN + list(args), cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                          text=True, timeout=1800)


def test_cpu_backend_matches_committed_baseline(sm):
    res = run("--backends", "cpu")
    assert res.returncode == 0, res.stdout
    assert "all ok" in res.stdout and "FAIL" not in res.stdout
    assert "no baseline" not in res.stdout            # every CPU line is pinned by baseline.json


@pytest.mark.gpu
def test_sm100_against_cpu_and_baseline(sm):
    res = run("--backends", "cpu,sm100")
    assert res.returncode == 0, res.stdout
    assert res.stdout.count(" ok   sm100") >= 18 and "FAIL" not in res.stdout


@pytest.mark.gpu
def test_inject_must_fail(sm):
    # tests/diff/run_diff.sh:32-33: a corrupted element has to be noticed, for every workload
    res = run("--backends", "cpu,sm100", "--inject")
    assert res.returncode == 1
    for w in ("vadd", "saxpy", "reduce_i32", "reduce_f32", "gemm", "asian"):
        assert "FAIL sm100  %s/" % w in res.stdout, (w, res.stdout)
    assert "FAIL cpu" not in res.stdout


@pytest.mark.gpu
def test_full_size_cases(sm):
    res = run("--backends", "cpu,sm100", "--full")
    assert res.returncode == 0, res.stdout
    assert "saxpy/n=268435456" in res.stdout and "gemm/k=8192,m=8192,n=8192,rows4=64" in res.stdout


@pytest.mark.gpu
def test_reference_ptx_backend_against_cpu_and_baseline(sm):
    # the counterpart of the reference runner's "nvidia" backend (tests/numeric/run_numeric.py:230-296):
    # what the reference compiler emits for the GPU, run here, against what it emits for x86-64
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "ptx", "saxpy.ptx")):
        pytest.skip("oracle/_ref/ptx was not built (the reference tree was absent at build time)")
    res = run("--backends", "cpu,nvptx")
    assert res.returncode == 0, res.stdout
    assert res.stdout.count(" ok   nvptx") >= 14 and "FAIL" not in res.stdout
    assert "no baseline" not in res.stdout
