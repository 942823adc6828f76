"""Data-parallel scheme on CPU ranks (gloo, world size 2): each rank differentiates its half of the
batch with the loss seed 1/world; the sum of the ranks' gradients must equal the full-batch
gradient, and the averaged shard losses the full-batch loss.  This is the host-side contract the
GPU ranks follow (bench.py, nn.Model with a communicator); no GPU is involved."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dims, batch = [20, 16, 12, 5], 64
    rng = np.random.default_rng(0)                       # same seed on every rank: replicated parameters, one global batch
    ws = [rng.standard_normal((dims[i + 1], dims[i])).astype(np.float32) * 0.3 for i in range(3)]
    bs = [rng.standard_normal(dims[i + 1]).astype(np.float32) * 0.1 for i in range(3)]
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    labels = rng.integers(0, dims[-1], batch)
    rows = batch // world
    shard = slice(rank * rows, (rank + 1) * rows)
    # seed 1/world with the local count == count override to the global batch
    loss, grads, _ = oracle.mlp_gradients(x[shard], labels[shard], ws, bs, "ce", count=batch)
    flat = torch.from_numpy(np.concatenate([g.reshape(-1) for g in grads]))
    dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    loss_t = torch.tensor([float(loss)], dtype=torch.float64)
    dist.all_reduce(loss_t, op=dist.ReduceOp.SUM)
    if rank == 0:
        full_loss, full_grads, _ = oracle.mlp_gradients(x, labels, ws, bs, "ce")
        want = np.concatenate([g.reshape(-1) for g in full_grads])
        got = flat.numpy()
        np.save(os.path.join(result_dir, "err.npy"), np.array([np.abs(got - want).max(), np.abs(want).max(),
                                                               abs(loss_t.item() / world - float(full_loss))]))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_gradients_sum_to_the_full_batch_gradient(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    err, scale, loss_err = np.load(tmp_path / "err.npy")
    assert err <= 4e-7 * scale + 1e-9                       # split contraction: a few ulp of the largest entry
    assert loss_err <= 2e-6


def test_seed_scaling_is_exact_for_power_of_two_worlds():
    # scale = seed / rows with seed = 1/world and rows = batch/world equals 1/batch exactly
    for world in (1, 2, 4, 8):
        batch = 65536
        seed = np.float32(1.0 / world)
        assert seed / np.float32(batch // world) == np.float32(1.0) / np.float32(batch)
