"""The N>1 path on CPU: two gloo ranks shard a global batch, each works on its own slice
(the oracle stands in for the kernels here), nothing but timings is exchanged."""

from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp


def test_shard_batch_partitions_exactly():
    from deformops_b200.sharding import shard_batch

    for world in (1, 2, 3, 4, 8):
        for gb in (0, 1, 7, 8, 64):
            shards = [shard_batch(gb, world, r) for r in range(world)]
            assert sum(s.batch for s in shards) == gb
            cursor = 0
            for s in shards:
                assert s.first_sample == cursor
                cursor += s.batch
            assert max(s.batch for s in shards) - min(s.batch for s in shards) <= 1
    assert [shard_batch(64, 8, r).batch for r in range(8)] == [8] * 8
    with pytest.raises(ValueError):
        shard_batch(4, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, global_batch: int, out_dir: str):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.set_num_threads(1)
    from deformops_b200.sharding import barrier, init_from_env, max_over_ranks, shard_batch
    from deformops_b200.workloads import make_workload
    from oracle import msda_oracle as orc

    r, w, _ = init_from_env(backend="gloo")
    assert (r, w) == (rank, world)
    shard = shard_batch(global_batch, world, rank)
    cfg = dict(batch=global_batch, levels=[(8, 8), (4, 4)], heads=2, head_dim=8, points=2,
               dtype=torch.float32)
    mine = make_workload(cfg, batch=shard.batch, first_sample=shard.first_sample, seed=5)
    barrier()
    out = orc.forward(mine.value, mine.spatial_shapes, mine.level_start_index,
                      mine.sampling_locations, mine.attention_weights, precision="f32")
    # per-rank "device time": rank 1 is the slow one; everyone must see its time
    times = max_over_ranks([1.0 + rank, 10.0 - rank])
    assert times == [float(world), 10.0]
    np.save(os.path.join(out_dir, f"out_{rank}.npy"), out)
    np.save(os.path.join(out_dir, f"val_{rank}.npy"), mine.value.numpy())
    barrier()
    torch.distributed.destroy_process_group()


def test_two_gloo_ranks_match_the_unsharded_batch(tmp_path):
    from deformops_b200.workloads import make_workload
    from oracle import msda_oracle as orc

    world, global_batch = 2, 5
    mp.spawn(_worker, args=(world, _free_port(), global_batch, str(tmp_path)), nprocs=world,
             join=True)
    cfg = dict(batch=global_batch, levels=[(8, 8), (4, 4)], heads=2, head_dim=8, points=2,
               dtype=torch.float32)
    whole = make_workload(cfg, seed=5)
    expect = orc.forward(whole.value, whole.spatial_shapes, whole.level_start_index,
                         whole.sampling_locations, whole.attention_weights, precision="f32")
    got = np.concatenate([np.load(tmp_path / f"out_{r}.npy") for r in range(world)])
    vals = np.concatenate([np.load(tmp_path / f"val_{r}.npy") for r in range(world)])
    # a rank's slice is bit-identical to the same samples of the unsharded batch
    assert np.array_equal(vals, whole.value.numpy())
    assert np.array_equal(got, expect)
