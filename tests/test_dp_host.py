"""Host side of the data-parallel step on CPU: two `gloo` ranks shard a batch and sum their
gradient buckets; every rank ends with the same sums (the reference's property that replicas stay
equal after a step, test/fixtures/devices.jl `shards_sgd!`)."""
import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import torch, torch.distributed as dist
    import __graft_entry__ as entry
    mlp = entry.load_package().mlp
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo")
    lo, hi = mlp.shard_rows(8, rank, world)
    assert (hi - lo) * world == 8 and lo == rank * 4
    data = torch.arange(8 * 3, dtype=torch.float32).reshape(8, 3)
    # "gradients" of each layer from this rank's shard
    buckets = [data[lo:hi].sum(dim=0).clone() * (layer + 1) for layer in range(3)]
    marks = mlp.sum_over_replicas(torch, buckets)
    assert marks == [None, None, None]
    for layer, b in enumerate(buckets):
        assert torch.equal(b, data.sum(dim=0) * (layer + 1)), (rank, layer, b)
    try:
        mlp.shard_rows(9, rank, world)
        raise SystemExit("an uneven split was accepted")
    except ValueError:
        pass
    dist.barrier()
    dist.destroy_process_group()
    os.write(1, ("rank " + str(rank) + " ok" + chr(10)).encode())
""")


def test_two_gloo_ranks_sum_their_buckets(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", str(script)]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert "rank 0 ok" in out.stdout and "rank 1 ok" in out.stdout
