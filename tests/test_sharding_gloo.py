"""The N > 1 host logic on CPU: two gloo ranks shard the rows of a small Linear+GELU stack, each
computes its slice with the CPU oracle (standing in for the per-rank GPU replica), and the gathered
result must equal the single-rank result bit for bit; the timing reduction must be the max."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from mimir_framework_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_are_disjoint_and_cover():
    for total in (0, 1, 7, 64, 65537):
        for world in (1, 2, 3, 8):
            r = [sharding.shard_range(total, world, k) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == total
            assert all(r[k][1] == r[k + 1][0] for k in range(world - 1))
            sizes = [e - b for b, e in r]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)


WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, os.environ["REPO_ROOT"])
    from mimir_framework_b200 import configs, sharding
    from oracle import port
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rows, k = 37, 64
    x = configs.linear_gelu_stack_input(rows, k)
    weights = configs.linear_gelu_stack_weights(k)
    b, e = sharding.shard_range(rows, world, rank)
    local = port.run_graph(configs.linear_gelu_stack(e - b, k), weights, {"x": x[b:e].ravel()}).reshape(e - b, k)
    t = sharding.reduce_max(0.5 + rank)
    full = sharding.gather_rows(local, rows)
    if rank == 0:
        want = port.run_graph(configs.linear_gelu_stack(rows, k), weights, {"x": x.ravel()}).reshape(rows, k)
        assert np.array_equal(full, want), "gathered rows differ from the single-rank result"
        assert t == 0.5 + world - 1, t
        print("OK", world)
    else:
        assert full is None
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_rank_gloo_shard_and_gather(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port_no = s.getsockname()[1]
    env = dict(os.environ, REPO_ROOT=ROOT, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port_no), str(script)], capture_output=True, text=True, env=env, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "OK 2" in r.stdout
