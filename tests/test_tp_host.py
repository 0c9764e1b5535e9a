"""Host-side logic of the tensor-parallel path on CPU: two gloo ranks exchange their (fake) buffer
handles and agree on the shard layout.  No GPU, no kernel."""
import os
import subprocess
import sys
import textwrap

from conftest import ROOT

WORKER = textwrap.dedent('''
    import importlib, os, sys
    sys.path.insert(0, os.environ["MOE_ROOT"])
    import torch.distributed as dist
    pkg = importlib.import_module("gpt-oss_b200")
    tp = importlib.import_module("gpt-oss_b200.tp")
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    blob = bytes([rank * 16 + (i % 16) for i in range(192)])
    got = tp.exchange_blobs(blob)
    assert len(got) == world
    for r, b in enumerate(got):
        assert b == bytes([r * 16 + (i % 16) for i in range(192)]), r
    # every rank derives the same shard table and the shards tile the intermediate dimension
    table = [pkg.shard_range(2880, world, r) for r in range(world)]
    flat = [None] * world
    dist.all_gather_object(flat, table)
    assert all(t == table for t in flat)
    assert table[0][0] == 0 and sum(n for _, n in table) == 2880
    assert all(table[i][0] + table[i][1] == table[i + 1][0] for i in range(world - 1))
    assert tp.tp_groups(8, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    dist.barrier()
    print("host ok", rank)
''')


def test_two_gloo_ranks_exchange_handles_and_shards(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MOE_ROOT=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29531", str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert res.stdout.count("host ok") == 2
