"""Two-rank run on CPU (gloo) of the benchmark's multi-GPU plumbing: every rank builds its
own shard or replica, nothing is exchanged except the barrier and the reductions of the
timing, and the aggregate is what bench.py reports."""

import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench
    from oracle import torch_oracle
    import workloads

    assert bench.dist_env() == (rank, rank, world)
    wl = workloads.WORKLOADS["layer_norm"]
    # strong-scaling shard of one configuration
    shard = wl.make(rank, world, "cpu", scale=8)
    res = wl.run(shard, torch_oracle)
    # weak-scaling replica (what bench.py times): same size on every rank, different data
    workloads.set_replica(rank)
    replica = wl.make(0, 1, "cpu", scale=8)
    workloads.set_replica(0)
    t_max = bench.reduce_max(1.0 + rank, world, torch.device("cpu"))
    work = bench.reduce_sum(wl.work(replica), world, torch.device("cpu"))
    bench.barrier(world)
    gathered = [None] * world
    dist.all_gather_object(gathered, (shard["x"], res["dx"], replica["x"][0, :4].tolist()))
    if rank == 0:
        torch.save({"t_max": t_max, "work": work, "gathered": gathered}, out)
    dist.destroy_process_group()


def test_two_ranks_gloo(tmp_path):
    out = str(tmp_path / "out.pt")
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out, weights_only=False)
    assert got["t_max"] == 2.0  # max over ranks
    sys.path.insert(0, ROOT)
    from oracle import torch_oracle
    import workloads

    wl = workloads.WORKLOADS["layer_norm"]
    whole = wl.make(0, 1, "cpu", scale=8)
    assert got["work"] == 2 * wl.work(whole)  # two full-size replicas
    ref = wl.run(whole, torch_oracle)
    xs = torch.cat([g[0] for g in got["gathered"]])
    dxs = torch.cat([g[1] for g in got["gathered"]])
    assert torch.equal(xs, whole["x"])  # shards concatenate to the single-rank problem
    assert torch.allclose(dxs, ref["dx"], rtol=1e-6, atol=1e-6)  # rows are independent
    assert got["gathered"][0][2] != got["gathered"][1][2]  # replicas differ between ranks
