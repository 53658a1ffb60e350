"""World-size-2 run of the host-side multi-GPU logic on CPU (gloo): the rank
plumbing of bench.py and the rule that contiguous shards, reduced per rank and
summed across ranks, give the unsharded result. The per-rank arithmetic is done
by the CPU checker here, the cross-rank sum by gloo in place of NCCL."""
import os
import socket
import subprocess
import sys

from conftest import ROOT

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["BOOTH_ROOT"])
import numpy as np, torch, torch.distributed as dist
import bench, booth_b200 as sm, oracle
ranks = bench.Ranks(2)
assert ranks.world == 2 and ranks.rank in (0, 1)
orc = oracle.load("port")
n = 1000003
lo, hi = sm.shard_range(n, ranks.rank, ranks.world)
# every rank generates only its own contiguous range of the global seeded stream
vi = sm.fill_host(hi - lo, 99, 0, 2, first=lo)
vf = sm.fill_host(hi - lo, 99, 1, 1, first=lo)
part = torch.tensor([orc.reduce_i32(vi)], dtype=torch.int64)
dist.all_reduce(part)
partf = torch.tensor([orc.reduce_f32(vf)], dtype=torch.float64)
dist.all_reduce(partf)
whole_i = orc.reduce_i32(sm.fill_host(n, 99, 0, 2))
whole_f = orc.reduce_f32(sm.fill_host(n, 99, 1, 1))
assert int(part[0]) == whole_i, (int(part[0]), whole_i)
assert abs(float(partf[0]) - whole_f) <= 1e-6 * whole_f   # chunk boundaries move with the shard
# Monte Carlo: disjoint path ranges add up to the whole
prm = sm.asian_params()
npaths = 4096
a, g = orc.asian(prm, ranks.rank * npaths, npaths)
t = torch.tensor([a, g], dtype=torch.float64); dist.all_reduce(t)
wa, wg = orc.asian(prm, 0, 2 * npaths)
assert abs(float(t[0]) - wa) <= 1e-12 * wa and abs(float(t[1]) - wg) <= 1e-12 * wg
# The benchmark's own parity plumbing, as bench.py uses it at N > 1: every rank sums its shard of
# the global stream piece by piece with the checker's generator (no product code), the wrapped
# int32 partial sums and the double partial sums travel through Ranks.sum, and the totals equal the
# checker's sums of the whole stream generated in one go.
m = 1 << 18
first = ranks.rank * m
acc_i, acc_f = 0, 0.0
for off in range(0, m, 1 << 16):
    acc_i = bench.wrap32(acc_i + orc.reduce_i32(orc.fill(1 << 16, 5, 0, 2, first=first + off)))
    acc_f += orc.reduce_f32(orc.fill(1 << 16, 5, 1, 1, first=first + off))
tot_i = bench.wrap32(int(ranks.sum([acc_i], integer=True)[0]))
tot_f = ranks.sum([acc_f])[0]
assert tot_i == orc.reduce_i32(orc.fill(2 * m, 5, 0, 2)), tot_i
assert abs(tot_f - orc.reduce_f32(orc.fill(2 * m, 5, 1, 1))) <= 1e-12 * tot_f
assert bench.wrap32(0x7FFFFFFF + 1) == -(1 << 31) and bench.wrap32(-(1 << 31) - 1) == 0x7FFFFFFF
assert ranks.gather(1.5 + ranks.rank) == [1.5, 2.5]
# the checker's generator and the library's give the same stream
assert np.array_equal(orc.fill(1000, 99, 0, 2, first=lo), vi[:1000])
# plumbing: max over ranks, byte broadcast, barrier
assert ranks.max(10.0 + ranks.rank) == 11.0
blob = ranks.bcast_bytes(bytes(range(128)) if ranks.rank == 0 else None)
assert blob == bytes(range(128))
ranks.barrier()
ranks.close()
print("rank %d ok" % ranks.rank)
'''


def test_two_ranks_on_cpu(sm, tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), BOOTH_ROOT=ROOT)
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for rank, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, out
        assert "rank %d ok" % rank in out


def test_wrong_world_size_is_refused(sm):
    """bench.py --gpus N must be launched with WORLD_SIZE == N (host-detected error, exit code 2)."""
    env = dict(os.environ, WORLD_SIZE="1", RANK="0")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", "2"], env=env,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=120)
    assert res.returncode == 2 and "WORLD_SIZE" in res.stderr
