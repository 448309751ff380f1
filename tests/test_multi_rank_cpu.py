"""The multi-GPU path's host logic on CPU ranks (gloo, world size 2): sequence sharding with no data-path collective,
whole-job throughput = units summed over ranks / the slowest rank's time.  The GPUs' part of a rank is the same
single-GPU step the other tests cover; ranks exchange only the scalars reduced here."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import json, os, sys
sys.path.insert(0, %r)
import bench
rank, local_rank, world = bench.dist_env()
d = bench.Dist(world, local_rank, backend="gloo")
contexts = [6000, 128000, 300, 9000, 45000, 1200, 64000, 7000, 2500, 31000]
shards = bench.shard_sequences(contexts, world)
mine = shards[rank]
rows = 10 * len(mine)                      # ten rows a sequence
ms = 5.0 * (rank + 1)                      # the second rank is slower
d.barrier()
agg = bench.aggregate(d, rows, len(mine), ms * 4, 4)
per_rank = [d.select(r, rows) for r in range(world)]      # what the 64-sequence report lists per rank
d.barrier()
if rank == 0:
    print(json.dumps({"shards": shards, "agg": agg, "per_rank_rows": per_rank,
                      "churn_mine": [len(bench.workload("churn64", r, 1000)) for r in range(world)]}))
d.close()
"""


def test_shard_sequences_balances_kv_and_keeps_every_sequence_once():
    sys.path.insert(0, ROOT)
    import bench
    rng = np.random.default_rng(0)
    contexts = [int(min(131072, max(1, rng.lognormal(np.log(6000), 1.0)))) for _ in range(64)]
    for world in (1, 2, 4, 8):
        shards = bench.shard_sequences(contexts, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [sum(contexts[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(contexts)
    assert bench.shard_sequences([5, 5], 4) == [[0], [1], [], []]
    # with the trees' rows the estimated step time is balanced instead: one 128k-token sequence no longer has a GPU to itself
    rows = [int(n) for n in rng.integers(1, 33, 64)]
    cost = lambda s: bench.shard_cost(contexts, rows, s)
    for world in (2, 4, 8):
        by_kv, by_cost = bench.shard_sequences(contexts, world), bench.shard_sequences(contexts, world, rows=rows)
        assert sorted(i for s in by_cost for i in s) == list(range(64))
        assert max(map(cost, by_cost)) <= max(map(cost, by_kv)) + 1e-9


def test_two_gloo_ranks_aggregate_like_the_bench():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29653")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29653", "-c", WORKER % ROOT]
    # torch.distributed.run wants a script path: write the worker beside the test's temp dir
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "worker.py")
        open(path, "w").write(WORKER % ROOT)
        cmd = cmd[:-2] + [path]
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    got = json.loads(line)
    shards = got["shards"]
    assert sorted(i for s in shards for i in s) == list(range(10)) and len(shards) == 2
    # 10 sequences x 10 rows, 4 steps, the slower rank took 40 ms in all
    assert abs(got["agg"]["rows_per_s"] - 100 * 4 / 0.040) < 1e-6
    assert abs(got["agg"]["ms_per_step"] - 10.0) < 1e-9
    assert got["per_rank_rows"] == [10 * len(s) for s in shards]
    # the bench's 64-sequence workload is sharded by the same rule: both ranks' shares make up the 64 sequences
    assert sum(got["churn_mine"]) == 64 and min(got["churn_mine"]) > 0
