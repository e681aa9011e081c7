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
    # the flat gradient buffer of a 4-layer step: each bucket a contiguous range, summed in one call
    sizes = (6, 10, 10, 10, 3)
    order, offsets, total, groups = mlp.flat_layout(sizes, fused=False)
    flat = torch.zeros(total)
    for i in range(4):
        w_at, b_at = offsets[i]
        flat[w_at: w_at + sizes[i] * sizes[i + 1]] = float((rank + 1) * (i + 1))
        flat[b_at: b_at + sizes[i + 1]] = float((rank + 1) * 10 * (i + 1))
    mlp.sum_over_replicas(torch, [flat[a:b] for a, b, _ in groups])
    for i in range(4):
        w_at, b_at = offsets[i]
        assert (flat[w_at: w_at + sizes[i] * sizes[i + 1]] == 3.0 * (i + 1)).all()
        assert (flat[b_at: b_at + sizes[i + 1]] == 30.0 * (i + 1)).all()
    used = sum(sizes[i] * sizes[i + 1] + sizes[i + 1] for i in range(4))
    assert (flat != 0).sum().item() == used           # the aligning gaps stayed zero
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


def test_flat_layout(pkg):
    """Every array on a 16-byte boundary, nothing overlapping, buckets contiguous and covering everything;
    the middle layers first (one bucket each, in the order the backward forms them), the two ends together."""
    mlp = pkg.mlp
    sizes = (1024, 4096, 4096, 4096, 1024)
    order, offsets, total, buckets = mlp.flat_layout(sizes, fused=False)
    assert order == [2, 1, 0, 3]
    assert [layers for _, _, layers in buckets] == [(2,), (1,), (0, 3)]
    taken = []
    for i in range(4):
        w_at, b_at = offsets[i]
        assert w_at % 8 == 0 and b_at % 8 == 0
        taken += [(w_at, w_at + sizes[i] * sizes[i + 1]), (b_at, b_at + sizes[i + 1])]
    taken.sort()
    assert all(a[1] <= b[0] for a, b in zip(taken, taken[1:])) and taken[-1][1] <= total
    assert buckets[0][0] == 0 and buckets[-1][1] == total
    assert all(a[1] == b[0] for a, b in zip(buckets, buckets[1:]))
    # odd sizes: gaps appear, arrays stay aligned
    order, offsets, total, buckets = mlp.flat_layout((10, 7, 3), fused=True)
    assert order == [0, 1] and offsets[0] == (0, 72) and offsets[1] == (80, 104) and total == 112
    assert [layers for _, _, layers in buckets] == [(1,), (0,)]
    # the exchange points of the schedule: each bucket right after the last of its layers' gradients
    class Fake:
        pass
    step = Fake()
    step.L, step.fuse_update, step.buckets, step.link = 4, False, mlp.flat_layout(sizes, False)[3], None
    plan = mlp.MLPStep._schedule(step)
    assert plan == [("below", 3), ("grads", 2), ("exchange", 0), ("below", 2), ("grads", 1), ("exchange", 1),
                    ("below", 1), ("grads", 3), ("grads", 0), ("exchange", 2)]
    # with the fused exchange (it writes the new weights at once) a layer's exchange waits for the layer below
    step.link = object()
    plan = mlp.MLPStep._schedule(step)
    assert plan == [("below", 3), ("below", 2), ("grads", 2), ("exchange", 0), ("below", 1), ("grads", 1), ("exchange", 1),
                    ("grads", 3), ("grads", 0), ("exchange", 2)]
