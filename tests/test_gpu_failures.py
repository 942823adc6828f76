"""Failure semantics on a B200, all through the C ABI and none of them by misusing the GPU: a step that
fails leaves no trace (the reference stages, validates and commits: TrainingSession.java:1151-1171,
TrainingParameter.java:391-409), device-side waits give up in an orderly way, a prefetch never
overtakes a run, and a collective that does not answer ends with COMM_FAILED after a host deadline.
The peer that does not answer is a stand-in NCCL library whose all-reduce parks a sleeping HOST
function on the stream: the GPU itself is idle the whole time."""
import os
import subprocess
import sys
import time

import numpy as np
import pytest

from synaptik_b200 import native, nn, program
from synaptik_b200.program import F32, GraphBuilder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ctx():
    c = native.Context(0)
    yield c
    c.close()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def optimizer_snapshot(opt, params, shapes):
    state = {"steps": opt.steps(), "runs": opt.accumulated_runs(), "p": [bits(b.download(np.float32, s)) for b, s in zip(params, shapes)]}
    for slot in (0, 1, 2):
        try:
            state[slot] = [bits(opt.state(i, slot)) for i in range(len(params))]
        except native.NativeFailure:        # SGD has no second moment
            state[slot] = None
    return state


def assert_same_state(a, b):
    assert a["steps"] == b["steps"] and a["runs"] == b["runs"]
    for x, y in zip(a["p"], b["p"]):
        assert np.array_equal(x, y)
    for slot in (0, 1, 2):
        if a[slot] is None:
            assert b[slot] is None
            continue
        for x, y in zip(a[slot], b[slot]):
            assert np.array_equal(x, y)


@pytest.mark.parametrize("kind,hyper", [(native.ADAM, [1e-3, 0.9, 0.999, 1e-8, 0.0]), (native.ADAMW, [1e-3, 0.9, 0.999, 1e-8, 0.01]),
                                        (native.SGD, [0.01, 0.9, 0.0, 0.0, 0.0]), (native.SGD, [0.01, 0.0, 0.0, 0.0, 0.0])])
def test_a_non_finite_update_leaves_every_array_and_counter_as_it_was(ctx, oracle, kind, hyper):
    rng = np.random.default_rng(3)
    shapes = [(300, 41), (41,)]
    values = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    params = [ctx.upload(v) for v in values]
    grads_ok = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    opt = native.Optimizer(ctx, kind, hyper, params, [int(np.prod(s)) for s in shapes])
    g_ok = [ctx.upload(g) for g in grads_ok]
    opt.step(g_ok)
    opt.run(native.Optimizer.ACCUMULATE, g_ok)               # a pending sum is part of the state too
    before = optimizer_snapshot(opt, params, shapes)
    poisoned = [g.copy() for g in grads_ok]
    poisoned[0][137, 5] = np.inf                             # one element of one tensor; the other tensor is clean
    g_bad = [ctx.upload(g) for g in poisoned]
    for mode in (native.Optimizer.RESET_AND_STEP, native.Optimizer.ACCUMULATE_AND_STEP, native.Optimizer.ACCUMULATE):
        with pytest.raises(native.NativeFailure) as failure:
            opt.run(mode, g_bad)
        assert failure.value.status == 11
        assert_same_state(before, optimizer_snapshot(opt, params, shapes))
    # an overflowing pending sum is refused the same way
    huge = [ctx.upload(np.full(s, 3e38, dtype=np.float32)) for s in shapes]
    fresh = native.Optimizer(ctx, kind, hyper, params, [int(np.prod(s)) for s in shapes])
    fresh.run(native.Optimizer.ACCUMULATE, huge)
    held = optimizer_snapshot(fresh, params, shapes)
    with pytest.raises(native.NativeFailure):
        fresh.run(native.Optimizer.ACCUMULATE, huge)
    assert_same_state(held, optimizer_snapshot(fresh, params, shapes))
    fresh.close()
    # and the optimizer carries on from the untouched state exactly like one that never saw the failure
    twin_params = [ctx.upload(np.frombuffer(p.tobytes(), np.float32).reshape(s)) for p, s in zip(before["p"], shapes)]
    twin = native.Optimizer(ctx, kind, hyper, twin_params, [int(np.prod(s)) for s in shapes])
    for i in range(len(shapes)):
        for slot in (0, 1, 2):
            if before[slot] is not None and (slot != 1 or kind != native.SGD) and (slot != 0 or kind != native.SGD or hyper[1] != 0.0):
                twin.restore(i, slot, before[slot][i].view(np.float32), before["steps"])
    twin.set_progress(before["steps"], before["runs"])
    opt.run(native.Optimizer.ACCUMULATE_AND_STEP, g_ok)
    twin.run(native.Optimizer.ACCUMULATE_AND_STEP, g_ok)
    assert_same_state(optimizer_snapshot(opt, params, shapes), optimizer_snapshot(twin, twin_params, shapes))
    opt.close(); twin.close()


def test_a_label_out_of_range_voids_the_step_and_every_step_enqueued_after_it(ctx):
    dims, batch = [48, 64, 10], 128
    rng = np.random.default_rng(9)
    model = nn.Model(dims, ctx, seed=2)
    model.configure_training("ce", nn.Adam(1e-3))
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    labels = rng.integers(0, 10, batch).astype(np.int32)
    model.train(x, labels)
    exe, xbuf, tbuf, seed, loss, grads = model.training_state(batch)
    opt = model._optimizer
    shapes = model.param_shapes
    inputs, outputs = [xbuf, tbuf, seed] + model.param_buffers, [loss] + grads
    bad = labels.copy()
    bad[77] = 10
    bad_buf = ctx.upload(bad)
    # synchronous form: the run reports the label
    before = optimizer_snapshot(opt, model.param_buffers, shapes)
    with pytest.raises(native.NativeFailure) as failure:
        exe.run([xbuf, bad_buf, seed] + model.param_buffers, outputs)
    assert failure.value.status == 5
    assert_same_state(before, optimizer_snapshot(opt, model.param_buffers, shapes))
    # enqueue-only form: good step, bad step, good step, then one finish.  Only the first counts.
    xbuf.upload(x); tbuf.upload(labels)
    exe.enqueue(inputs, outputs); opt.step_enqueue(grads); opt.finish()
    after_one = optimizer_snapshot(opt, model.param_buffers, shapes)
    # rewind by restoring the state, then replay the three steps without finishing in between
    for buf, old in zip(model.param_buffers, before["p"]):
        buf.upload(old.view(np.float32))
    for i in range(len(shapes)):
        opt.restore(i, 0, before[0][i].view(np.float32), before["steps"])
        opt.restore(i, 1, before[1][i].view(np.float32), before["steps"])
    opt.set_progress(before["steps"], before["runs"])
    exe.enqueue(inputs, outputs); opt.step_enqueue(grads)
    exe.enqueue([xbuf, bad_buf, seed] + model.param_buffers, outputs); opt.step_enqueue(grads)
    exe.enqueue(inputs, outputs); opt.step_enqueue(grads)
    assert opt.steps() == before["steps"] + 3              # enqueued steps are counted until the verdict
    with pytest.raises(native.NativeFailure) as failure:
        opt.finish()
    assert failure.value.status == 5
    assert_same_state(after_one, optimizer_snapshot(opt, model.param_buffers, shapes))
    # the context is clean again: a further good step works and moves the parameters
    exe.enqueue(inputs, outputs); opt.step_enqueue(grads); opt.finish()
    assert opt.steps() == before["steps"] + 2
    assert not np.array_equal(after_one["p"][0], bits(model.param_buffers[0].download(np.float32, shapes[0])))
    bad_buf.close()
    model.close()


def test_a_device_side_wait_that_runs_out_reports_timeout_and_the_context_lives_on(ctx):
    start = time.perf_counter()
    with pytest.raises(native.NativeFailure) as failure:
        ctx.wait_probe(2000)                                # a 2 ms limit on a barrier nothing signals
    assert failure.value.status == 14
    assert time.perf_counter() - start < 1.0
    # the next ordinary run on the same context succeeds and is clean
    g = GraphBuilder()
    a, b = g.feed(F32, (64, 32)), g.feed(F32, (32, 16))
    g.publish(g.matmul(a, b))
    rng = np.random.default_rng(0)
    av, bv = rng.integers(-3, 4, (64, 32)).astype(np.float32), rng.integers(-3, 4, (32, 16)).astype(np.float32)
    exe = native.Executable(ctx, g.build())
    ins, out = [ctx.upload(av), ctx.upload(bv)], ctx.buffer(64 * 16 * 4)
    exe.run(ins, [out])
    assert np.array_equal(out.download(np.float32, (64, 16)), av @ bv)
    exe.close()


def test_the_first_prefetch_into_a_buffer_waits_for_runs_already_enqueued(ctx):
    # upload, enqueue without finishing, then the FIRST prefetch of other data into the same input
    # buffer: every run enqueued before the prefetch must still see the old data
    m, k, n = 8192, 1024, 1024
    rng = np.random.default_rng(4)
    g = GraphBuilder()
    x, w, b = g.feed(F32, (m, k)), g.feed(F32, (n, k)), g.feed(F32, (n,))
    _, z = g.linear(x, w, b)
    g.publish(g.relu(z))
    exe = native.Executable(ctx, g.build())
    old = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    new = native.PinnedArray((m, k), np.float32)
    new.array[...] = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    xb, wb, bb = ctx.upload(old), ctx.upload(rng.uniform(-0.05, 0.05, (n, k)).astype(np.float32)), ctx.upload(np.zeros(n, np.float32))
    out_a, out_b = ctx.buffer(m * n * 4), ctx.buffer(m * n * 4)
    exe.run([xb, wb, bb], [out_a])
    want = out_a.download(np.float32, (m, n))
    for _ in range(6):                                       # a queue of runs that all read the old data
        exe.enqueue([xb, wb, bb], [out_b])
    xb.prefetch(new.pointer, new.nbytes)                     # copy stream; must start after the six runs
    exe.finish()
    assert np.array_equal(bits(out_b.download(np.float32, (m, n))), bits(want))
    exe.run([xb, wb, bb], [out_b])                           # and a run enqueued after it sees the new data
    assert not np.array_equal(bits(out_b.download(np.float32, (m, n))), bits(want))
    assert np.array_equal(xb.download(np.float32, (m, k)), new.array)
    exe.close(); new.close()


def test_a_chained_product_with_one_accumulator_and_contraction_slices_runs(ctx):
    # X W1 W2 with a long contraction, FP32 promotion off: the second product may split its contraction
    # into slices, and a sliced product cannot also write operand planes from its epilogue
    m, k, n = 512, 4096, 4096
    rng = np.random.default_rng(6)
    g = GraphBuilder()
    x, w1, w2 = g.feed(F32, (m, k)), g.feed(F32, (k, n)), g.feed(F32, (n, 256))
    g.publish(g.matmul(g.matmul(x, w1), w2))
    ctx.set_option("gemm_engine", 2); ctx.set_option("gemm_promote", 0); ctx.set_option("gemm_slices", 1)
    try:
        exe = native.Executable(ctx, g.build())
    finally:
        ctx.set_option("gemm_engine", 0); ctx.set_option("gemm_promote", 1)
    xv = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w1v = rng.uniform(-0.03, 0.03, (k, n)).astype(np.float32)
    w2v = rng.uniform(-0.03, 0.03, (n, 256)).astype(np.float32)
    ins, out = [ctx.upload(a) for a in (xv, w1v, w2v)], ctx.buffer(m * 256 * 4)
    exe.run(ins, [out])
    got = out.download(np.float32, (m, 256))
    ref = (xv.astype(np.float64) @ w1v.astype(np.float64)) @ w2v.astype(np.float64)
    assert np.abs(got - ref).max() <= 2e-4 * np.abs(ref).max()
    exe.close()


FAKE_WORKER = r'''
import os, sys, time
import numpy as np
sys.path.insert(0, os.environ["SYN_ROOT"])
from synaptik_b200 import native, nn
ctx = native.Context(0)
ctx.set_option("comm_timeout_ms", 300)
comm = native.Comm(ctx, 1, 0, native.comm_unique_id())
buf = ctx.upload(np.arange(1024, dtype=np.float32))
start = time.perf_counter()
try:
    comm.allreduce_sum(buf, 1024)
    status = 0
except native.NativeFailure as failure:
    status = failure.status
waited = time.perf_counter() - start
print("first all-reduce: status", status, "after", round(waited, 4), "s", flush=True)
assert status == 15, status
limit = float(os.environ["SYN_EXPECT_WITHIN"])
assert waited < limit, waited
if os.environ.get("FAKE_NCCL_ASYNC_ERROR") != "1":
    assert waited >= 0.3, waited                         # the deadline, not an early return
# the communicator is gone for good, the context is not
try:
    comm.allreduce_sum(buf, 1024)
    raise SystemExit("a dead communicator answered")
except native.NativeFailure as failure:
    assert failure.status == 15
assert np.array_equal(buf.download(np.float32, (1024,)), np.arange(1024, dtype=np.float32))
# a training step whose gradients sit behind a collective that is given up is void
comm2 = native.Comm(ctx, 1, 0, native.comm_unique_id())
model = nn.Model([32, 48, 10], ctx, seed=1, comm=comm2, world_size=1)
model.configure_training("ce", nn.Adam(1e-3))
rng = np.random.default_rng(0)
x = rng.standard_normal((64, 32)).astype(np.float32)
labels = rng.integers(0, 10, 64)
before = [p.copy() for p in model.parameters()]
exe, xbuf, tbuf, seed, loss, grads = model.training_state(64)
xbuf.upload(x); tbuf.upload(labels.astype(np.int32))
exe.enqueue([xbuf, tbuf, seed] + model.param_buffers, [loss] + grads)      # four all-reduces that never finish
model._optimizer.step_enqueue(grads)                                        # the update queued behind them
assert model.optimizer_steps() == 1
try:
    model._optimizer.finish()
    raise SystemExit("the step went through")
except native.NativeFailure as failure:
    assert failure.status == 15, failure.status
for a, b in zip(before, model.parameters()):
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
assert model.optimizer_steps() == 0
model.close(); comm2.close(); comm.close(); ctx.close()
print("ok")
'''


def build_fake_nccl(folder) -> str:
    out = os.path.join(str(folder), "libfake_nccl.so")
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-o", out, os.path.join(ROOT, "tests", "fake_nccl.c"), "-ldl"], check=True)
    return out


@pytest.mark.parametrize("async_error", ["0", "1"])
def test_a_collective_that_never_answers_ends_with_comm_failed(tmp_path, async_error):
    fake = build_fake_nccl(tmp_path)
    script = tmp_path / "worker.py"
    script.write_text(FAKE_WORKER)
    # the stall is host-side and far longer than the deadline; with an asynchronous error reported the
    # wait ends at once instead of at the deadline
    # (limits with room for the one-off delays of a process's first launches on a fresh machine: the deadline is
    # 0.3 s, the stall 4 s)
    env = dict(os.environ, SYN_ROOT=ROOT, SYNAPTIK_NCCL_LIBRARY=fake, FAKE_NCCL_STALL_MS="4000", FAKE_NCCL_ASYNC_ERROR=async_error,
               SYN_EXPECT_WITHIN="3.0" if async_error == "0" else "1.5")
    done = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0 and "ok" in done.stdout, done.stdout + done.stderr


def test_products_give_way_to_a_co_tenant_without_changing_their_result(ctx):
    """While other blocks hold a third of the SMs (as a collective's do), the two-SM kernel's pairs take fewer
    tiles each; the product must come out bit for bit as on a free GPU."""
    from synaptik_b200.program import GraphBuilder, F32
    rng = np.random.default_rng(11)
    m, k, n = 4096, 1024, 2048
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    g = GraphBuilder()
    xv, wv = g.feed(F32, (m, k)), g.feed(F32, (n, k))
    g.publish(g.linear(xv, wv, None)[1])
    ctx.set_option("gemm_engine", 2)
    try:
        exe = native.Executable(ctx, g.build())
    finally:
        ctx.set_option("gemm_engine", 0)
    assert "tcgen05" in exe.describe()
    feeds = [ctx.buffer(a.nbytes) for a in (x, w)]
    for b, a in zip(feeds, (x, w)):
        b.upload(a)
    out = ctx.buffer(m * n * 4)
    exe.run(feeds, [out])
    free = out.download(np.float32, (m, n)).copy()
    for blocks in (16, 48, 100):
        ctx.occupy(blocks, 20000)                   # 20 ms: longer than the product
        exe.run(feeds, [out])
        assert np.array_equal(out.download(np.float32, (m, n)), free), blocks
    ctx.synchronize()
    exe.close()


def test_a_single_wave_weight_gradient_is_planned_again_in_slices_under_a_communicator(ctx):
    """A product of at most one tile per SM pair cannot give way to a collective's blocks; attaching a communicator
    plans it again with its contraction in slices (one more launch: the kernel that adds the slices)."""
    import torch  # noqa: F401  (brings the process's NCCL with it)
    try:
        comm = native.Comm(ctx, 1, 0, native.comm_unique_id())
    except native.NativeFailure:
        pytest.skip("no NCCL in this process")
    rows, k, n = 4096, 784, 4096
    rng = np.random.default_rng(12)
    x = rng.uniform(0, 1, (rows, k)).astype(np.float32)
    dz = rng.standard_normal((rows, n)).astype(np.float32)
    g = GraphBuilder()
    xv, dzv = g.feed(F32, (rows, k)), g.feed(F32, (rows, n))
    g.publish(g.matmul(g.permute(xv, (1, 0)), dzv))                 # [k, n]: 4 x 16 tiles of 256 x 256 on 74 pairs
    ctx.set_option("gemm_engine", 2)
    try:
        exe = native.Executable(ctx, g.build())
    finally:
        ctx.set_option("gemm_engine", 0)
    feeds, out = [ctx.upload(x), ctx.upload(dz)], ctx.buffer(k * n * 4)
    exe.run(feeds, [out])
    whole, launches = out.download(np.float32, (k, n)).copy(), exe.launch_count()
    exe.attach_comm(comm, [0])
    exe.run(feeds, [out])
    sliced = out.download(np.float32, (k, n))
    assert exe.launch_count() == launches + 1
    ref = x.astype(np.float64).T @ dz.astype(np.float64)
    bound = (8 + 512 / 4) * 2.0 ** -24 * (np.abs(x.astype(np.float64)).T @ np.abs(dz.astype(np.float64)))
    assert np.all(np.abs(sliced - ref) <= bound) and np.all(np.abs(whole - ref) <= bound)
    exe.attach_comm(None)
    exe.close(); comm.close()
