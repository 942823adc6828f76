"""Data-parallel training on 2, 4 and 8 B200s (as many as the box has; skipped with one): after every
one of 20 Adam steps the ranks must hold identical parameters, and those must match a single-rank
run on the whole batch within the GEMM tolerance."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, json
import numpy as np
sys.path.insert(0, os.environ["SYN_ROOT"])
import torch, torch.distributed as dist
from synaptik_b200 import native, nn
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
ctx = native.Context(local)
holder = [native.comm_unique_id() if rank == 0 else None]
dist.broadcast_object_list(holder, src=0)
comm = native.Comm(ctx, world, rank, holder[0]) if world > 1 else None
dims, batch = [784, 512, 256, 10], 1024
ctx.set_option("gemm_engine", 2)
if os.environ.get("SYN_CHUNK"):
    ctx.set_option("gemm_chunk", int(os.environ["SYN_CHUNK"]))
tag = os.environ.get("SYN_TAG") or f"w{world}"
model = nn.Model(dims, ctx, seed=9, comm=comm, world_size=world)
model.configure_training("ce", nn.Adam(1e-3))
rng = np.random.default_rng(5)
x = rng.uniform(0, 1, (batch, dims[0])).astype(np.float32)
labels = rng.integers(0, 10, batch)
rows = batch // world
# before any step: the all-reduced gradients of the ranks' slices are the gradient of the whole batch
_, first_gradients = model.gradients(x[rank * rows:(rank + 1) * rows], labels[rank * rows:(rank + 1) * rows])
if rank == 0:
    np.save(os.environ["SYN_OUT"] + f".{tag}.start.npy", np.concatenate([p.reshape(-1) for p in model.parameters()]))
    np.save(os.environ["SYN_OUT"] + f".{tag}.grads.npy", np.concatenate([g.reshape(-1) for g in first_gradients]))
losses, history, same = [], [], True
for step in range(20):
    losses.append(model.train(x[rank * rows:(rank + 1) * rows], labels[rank * rows:(rank + 1) * rows]))
    params = np.concatenate([p.reshape(-1) for p in model.parameters()])
    history.append(params)
    t = torch.from_numpy(params).cuda()
    gathered = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    same = same and all(bool(torch.equal(gathered[0], g)) for g in gathered)
l = torch.tensor(losses, dtype=torch.float64, device="cuda")
dist.all_reduce(l)
if rank == 0:
    np.save(os.environ["SYN_OUT"] + f".{tag}.npy", np.stack(history))
    json.dump({"replicas_identical": same, "losses": (l / world).tolist()}, open(os.environ["SYN_OUT"] + f".{tag}.json", "w"))
model.close()
if comm is not None: comm.close()
dist.destroy_process_group()
'''


def _run(world, out, port, tag="", chunk=""):
    env = dict(os.environ, SYN_ROOT=ROOT, SYN_OUT=out, NCCL_NVLS_ENABLE="0", SYN_TAG=tag, SYN_CHUNK=chunk)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-c", WORKER]
    script = out + ".worker.py"
    open(script, "w").write(WORKER)
    cmd = cmd[:-2] + [script]
    subprocess.run(cmd, env=env, check=True, timeout=600)


def test_ranks_match_one_rank_after_every_step(tmp_path):
    import torch
    available = torch.cuda.device_count()
    if available < 2:
        pytest.skip("needs two GPUs")
    out = str(tmp_path / "dp")
    _run(1, out, 29731)
    from helpers import report, trajectory_distance
    one = np.load(out + ".w1.npy")                      # [steps, parameters]
    start = np.load(out + ".w1.start.npy")
    info1 = json.load(open(out + ".w1.json"))
    # what a rounding-level change does to 20 Adam steps, measured rather than assumed: the same single rank with
    # FP32 partial sums of 256 instead of 512 contraction steps (the weight gradients then are four partial sums
    # of 256 rows, the very split four ranks make)
    _run(1, out, 29733, tag="reordered", chunk="256")
    reordered = np.load(out + ".reordered.npy")
    info_reordered = json.load(open(out + ".reordered.json"))
    floor = [trajectory_distance(reordered[step], one[step], start, 1e-3, step + 1) for step in range(one.shape[0])]
    report("data_parallel_rounding_floor", floor)
    for world in [w for w in (2, 4, 8) if w <= available]:
        _run(world, out, 29731 + 2 * world)
        many = np.load(out + f".w{world}.npy")
        info = json.load(open(out + f".w{world}.json"))
        assert info["replicas_identical"], world
        # step 0: a wrong reduction (scale, a missing bucket, a stale buffer) shows at once in the gradients,
        # which must agree with the single-rank gradient of the whole batch to GEMM rounding
        g1, gn = np.load(out + ".w1.grads.npy").astype(np.float64), np.load(out + f".w{world}.grads.npy").astype(np.float64)
        assert np.linalg.norm(g1 - gn) <= 2e-5 * np.linalg.norm(g1), (world, np.linalg.norm(g1 - gn) / np.linalg.norm(g1))
        # then every step: two summation orders drift apart slowly (Adam turns gradient rounding near zero
        # into fractions of lr); bounded as whole trajectories, since 2 * lr * step per entry would hold
        # for any two runs
        table = []
        for step in range(one.shape[0]):
            d = trajectory_distance(many[step], one[step], start, 1e-3, step + 1)
            table.append(d)
            # measured on 2 ranks: identical to 5e-8 after 20 steps (the forward passes are the single rank's bit for
            # bit, and two partial sums of 512 rows are exactly the single rank's two promoted partials).  More
            # ranks round the weight gradients differently, entries whose gradient is near zero take Adam steps of
            # opposite sign, the ReLU gates follow, and the trajectories part as fast as the reordered single rank's
            # does (measured on 4 ranks: relative L2 2.3e-3 at step 7, 2.4e-2 at step 14): bounded by three times that
            f = floor[step]
            if world == 2:
                ok = d["relative_l2"] <= 0.01 and d["share_apart"] <= 1e-3 and d["mean"] <= 2e-6 * (step + 1) and d["max"] <= 1e-3
            else:
                ok = d["relative_l2"] <= 3 * f["relative_l2"] + 0.01 and d["share_apart"] <= 3 * f["share_apart"] + 1e-3 \
                    and d["mean"] <= 3 * f["mean"] + 2e-6 * (step + 1) and d["max"] <= 3 * f["max"] + 1e-3
            assert ok, (world, step, d, f)
        report(f"data_parallel_world{world}", table)
        l1, ln = np.asarray(info1["losses"]), np.asarray(info["losses"])
        slack = 0.0 if world == 2 else 3 * np.abs(np.asarray(info_reordered["losses"]) - l1).max()
        assert np.all(np.abs(ln - l1) <= 2e-4 * np.abs(l1) + slack), (world, np.abs(ln - l1).max(), slack)
