"""Parity at the benchmark configurations' full sizes, where the CPU checker cannot compute the
whole result in seconds: sampled rows / blocks against binary64 arithmetic, plus properties that do
not depend on the size (exact power-of-two scaling, a checksum of checksums, gradient rows that sum
to zero, index outputs bit-exact).  Everything goes through the C ABI."""
import numpy as np
import pytest

from helpers import run_image
from synaptik_b200 import native
from synaptik_b200.program import F32, I32, GraphBuilder

pytestmark = pytest.mark.gpu

TWO_M24 = 2.0 ** -24


@pytest.fixture(scope="module")
def ctx():
    c = native.Context(0)
    yield c
    c.close()


def dense_layer_graph(m, k, n):
    """Y = relu(X W^T + b) with dX, dW, db for an upstream gradient (the standalone fused dense layer)."""
    g = GraphBuilder()
    x, w, b, dy = g.feed(F32, (m, k)), g.feed(F32, (n, k)), g.feed(F32, (n,)), g.feed(F32, (m, n))
    wt, z = g.linear(x, w, b)
    g.publish(g.relu(z))
    dz = g.relu_backward(z, dy)
    dx, dw, db = g.linear_backward(x, wt, dz, need_dx=True)
    for v in (dx, dw, db):
        g.publish(v)
    return g


def tc_bound(abs_products_sum, k):
    # the tensor-core tolerance of the parity suite: (8 + min(K, 512) / 4) * 2^-24 * sum |a b|
    return (8.0 + min(k, 512) / 4.0) * TWO_M24 * abs_products_sum + 1e-30


@pytest.mark.parametrize("m,k,n", [(4096, 1024, 1024), (65536, 4096, 4096)])
def test_dense_layer_forward_and_backward_at_full_size(ctx, m, k, n):
    rng = np.random.default_rng(m + k)
    bound = np.sqrt(6.0 / (k + n))
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = rng.uniform(-bound, bound, (n, k)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, n).astype(np.float32)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    y, dx, dw, db = run_image(ctx, dense_layer_graph(m, k, n), [x, w, b, dy])

    rows = rng.choice(m, 48, replace=False)
    x64, w64 = x[rows].astype(np.float64), w.astype(np.float64)
    z_ref = x64 @ w64.T + b.astype(np.float64)
    z_tol = tc_bound(np.abs(x64) @ np.abs(w64).T, k) + 2 * TWO_M24 * np.abs(z_ref)     # + the bias rounding
    # forward: the stored activation of the sampled rows
    assert np.all(np.abs(y[rows] - np.maximum(z_ref, 0.0)) <= z_tol)
    assert np.all(y >= 0.0) and np.all(np.isfinite(y))
    # dX on the device's own gates (a pre-activation within rounding of zero may gate either way)
    dz64 = np.where(y[rows] > 0.0, dy[rows], 0.0).astype(np.float64)
    dx_ref = dz64 @ w64
    assert np.all(np.abs(dx[rows] - dx_ref) <= tc_bound(np.abs(dz64) @ np.abs(w64), n))
    # dW and db: a 64 x 64 block and 256 columns, contraction over the whole batch, device gates
    cols_n, cols_k = rng.choice(n, 64, replace=False), rng.choice(k, 64, replace=False)
    dz_cols = np.where(y[:, cols_n] > 0.0, dy[:, cols_n], 0.0).astype(np.float64)
    x_cols = x[:, cols_k].astype(np.float64)
    dw_ref = dz_cols.T @ x_cols
    assert np.all(np.abs(dw[np.ix_(cols_n, cols_k)] - dw_ref) <= tc_bound(np.abs(dz_cols).T @ np.abs(x_cols), m))
    db_ref = dz_cols.sum(axis=0)
    assert np.all(np.abs(db[cols_n] - db_ref) <= 1.5 * TWO_M24 * np.abs(db_ref) + 1e-30)       # binary64 sums, one rounding
    # size-independent check of every output element: a checksum of checksums.  sum_r dX[r, :] must equal
    # (sum_r dZ[r, :]) W, and sum over everything of dW equals (column sums of dZ) . (column sums of X)
    dz_all = np.where(y > 0.0, dy, np.float32(0.0))
    col_dz = dz_all.sum(axis=0, dtype=np.float64)
    lhs = dx.sum(axis=0, dtype=np.float64)
    rhs = col_dz @ w64
    scale = np.abs(dz_all).sum(axis=0, dtype=np.float64) @ np.abs(w64)
    assert np.all(np.abs(lhs - rhs) <= 64 * TWO_M24 * scale)
    total_dw = dw.sum(dtype=np.float64)
    # (the dW checksum: sum_ij dW[i, j] = sum_r (sum_i dZ[r, i]) (sum_j X[r, j]))
    per_row = dz_all.sum(axis=1, dtype=np.float64) * x.sum(axis=1, dtype=np.float64)
    budget = (np.abs(dz_all).sum(axis=1, dtype=np.float64) * np.abs(x).sum(axis=1, dtype=np.float64)).sum()
    assert abs(total_dw - per_row.sum()) <= 64 * TWO_M24 * budget


def test_power_of_two_scaling_is_exact_at_full_size(ctx):
    # scaling an operand by a power of two scales every split plane, product and partial sum exactly, so
    # the tensor-core product of (4 X) must be 4 times the product of X bit for bit: a check of every
    # element of a 65536 x 4096 result that needs no reference arithmetic
    m, k, n = 65536, 1024, 4096
    rng = np.random.default_rng(11)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = rng.uniform(-0.05, 0.05, (n, k)).astype(np.float32)

    def product(a):
        g = GraphBuilder()
        xv, wv = g.feed(F32, (m, k)), g.feed(F32, (n, k))
        g.publish(g.matmul(xv, g.permute(wv, (1, 0))))
        (out,) = run_image(ctx, g, [a, w])
        return out

    base = product(x)
    assert np.array_equal(product(x * np.float32(4.0)), base * np.float32(4.0))


def test_classifier_head_at_full_size(ctx):
    rows, classes = 65536, 1000
    rng = np.random.default_rng(7)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = rng.integers(0, classes, rows).astype(np.int32)
    g = GraphBuilder()
    lv, yv, sv = g.feed(F32, (rows, classes)), g.feed(I32, (rows,)), g.feed(F32, ())
    g.publish(g.index_cross_entropy(lv, yv))
    g.publish(g.index_cross_entropy_backward(lv, yv, sv))
    g.publish(g.arg_max(lv, 1))
    loss, grad, best = run_image(ctx, g, [logits, labels, np.array(1.0, dtype=np.float32)])
    # index output: bit-exact against first-index arg-max over every row
    assert np.array_equal(best, np.argmax(logits, axis=1).astype(np.int64))
    # loss against binary64 log-sum-exp over every row
    l64 = logits.astype(np.float64)
    mx = l64.max(axis=1)
    lse = mx + np.log(np.exp(l64 - mx[:, None]).sum(axis=1))
    ref_loss = float((lse - l64[np.arange(rows), labels]).mean())
    assert abs(float(loss) - ref_loss) <= 1e-6 * abs(ref_loss)
    # gradient: every row sums to zero up to rounding (softmax minus one-hot), the label entry is
    # the only negative one, and sampled rows match binary64 arithmetic to 4 ulp of the row's largest entry
    row_sums = grad.sum(axis=1, dtype=np.float64)
    assert np.all(np.abs(row_sums) <= 64 * TWO_M24 / rows)
    assert np.all(grad[np.arange(rows), labels] < 0.0)
    assert int((grad < 0.0).sum()) == rows
    sample = rng.choice(rows, 64, replace=False)
    p = np.exp(l64[sample] - lse[sample][:, None])
    p[np.arange(len(sample)), labels[sample]] -= 1.0
    ref_grad = p / rows
    tol = 4 * TWO_M24 * np.abs(ref_grad).max(axis=1, keepdims=True) + 4 * TWO_M24 * np.abs(ref_grad)
    assert np.all(np.abs(grad[sample] - ref_grad) <= tol)


def test_classifier_inference_at_full_size(ctx):
    # the benchmark inference configuration: 784-4096-4096-4096-10, batch 8192 per GPU, arg-max published
    from synaptik_b200 import nn
    dims, batch = [784, 4096, 4096, 4096, 10], 8192
    rng = np.random.default_rng(21)
    model = nn.Model(dims, ctx, seed=3)
    # biases start at zero in the reference's initialisation; give them values so the epilogue is exercised
    params = model.parameters()
    for i in range(1, len(params), 2):
        params[i] = rng.uniform(-0.1, 0.1, params[i].shape).astype(np.float32)
    model.load_parameters(params)
    x = rng.uniform(0, 1, (batch, dims[0])).astype(np.float32)
    logits, best = model.compute(x, arg_max=True)
    # binary64 forward pass of sampled rows with the model's own parameters
    sample = rng.choice(batch, 32, replace=False)
    h = x[sample].astype(np.float64)
    weights, biases = params[0::2], params[1::2]
    for layer, (w, b) in enumerate(zip(weights, biases)):
        h = h @ w.astype(np.float64).T + b.astype(np.float64)
        if layer + 1 < len(weights):
            h = np.maximum(h, 0.0)
    assert np.all(np.abs(logits[sample] - h) <= 2e-5 * np.abs(h).max())
    # index output: bit-exact arg-max of the device's own logits, over every row
    assert np.array_equal(best, np.argmax(logits, axis=1).astype(np.int64))
    model.close()


def test_full_width_classifier_training_against_the_openblas_cpu_tier_for_20_steps(ctx, oracle):
    # The benchmark network at its own width, 784-4096-4096-4096-10 with softmax cross entropy and Adam
    # (1e-3, 0.9, 0.999, 1e-8), 20 steps from a fixed seed on a 2048-row batch, parameters compared after
    # EVERY step against the reference-shaped CPU step (OpenBLAS sgemm called the way the reference's CPU
    # backend calls it, plus its scalar loops).
    #
    # What two correct FP32 implementations can be expected to agree on here is set by the optimizer and the
    # ReLU gates, not by the kernels' rounding: Adam's first step moves every entry by about lr * sign(g), a
    # hidden pre-activation within rounding of zero gates one way or the other depending on the order of the
    # additions, one such gate changes that sample's contribution to every gradient below it, and this
    # configuration's second step sends the loss from 2.3 to about 20 before it recovers, which amplifies
    # every difference.  So the device is held to the noise floor of the CPU tier itself.  The same CPU step
    # is run a second time on an equivalent problem: batch rows, input features and hidden units consistently
    # permuted (the network computes the same function; only the order of the additions inside every
    # product changes), and its parameters are permuted back.  That is a second, equally valid FP32
    # trajectory, and the device may be at most three times as far from the CPU run as that one is, plus a
    # constant for the gates the less exact product flips early on.  Absolute caps far below what unrelated
    # trajectories show (relative L2 near 1.4, more than half of the entries apart) back this up.
    from helpers import report, trajectory_distance
    from synaptik_b200 import nn
    import os
    dims, batch, steps, lr = [784, 4096, 4096, 4096, 10], 2048, 20, 1e-3
    rng = np.random.default_rng(2024)
    x = rng.random((batch, dims[0]), dtype=np.float32)
    labels = rng.integers(0, 10, batch).astype(np.int32)
    order = rng.permutation(batch)
    perms = [rng.permutation(dims[0])] + [rng.permutation(d) for d in dims[1:-1]] + [np.arange(dims[-1])]
    inverse = [np.argsort(p) for p in perms]
    x_other, labels_other = np.ascontiguousarray(x[order][:, perms[0]]), np.ascontiguousarray(labels[order])
    model = nn.Model(dims, ctx, seed=17)
    model.configure_training("ce", nn.Adam(lr, 0.9, 0.999, 1e-8))
    start = model.parameters()

    def cpu_state(permuted):
        weights = [p.copy() for p in start[0::2]]
        biases = [p.copy() for p in start[1::2]]
        if permuted:
            weights = [np.ascontiguousarray(w[perms[l + 1]][:, perms[l]]) for l, w in enumerate(weights)]
            biases = [np.ascontiguousarray(b[perms[l + 1]]) for l, b in enumerate(biases)]
        return (weights, biases, [np.zeros(p.size, dtype=np.float32) for p in start], [np.zeros(p.size, dtype=np.float32) for p in start])

    def restored(state):            # the permuted problem's parameters in the original order
        weights = [w[inverse[l + 1]][:, inverse[l]] for l, w in enumerate(state[0])]
        biases = [b[inverse[l + 1]] for l, b in enumerate(state[1])]
        return [a for pair in zip(weights, biases) for a in pair]

    cpu, other = cpu_state(False), cpu_state(True)
    oracle.baseline_bind_openblas()
    threads = os.cpu_count() or 1
    table = []
    for step in range(1, steps + 1):
        device_loss = model.train(x, labels)
        losses = []
        for (weights, biases, m1, m2), (xs, ls) in ((cpu, (x, labels)), (other, (x_other, labels_other))):
            _, loss, _ = oracle.baseline_mlp_step(dims, xs, ls, weights, biases, m1, m2, train=True, count_total=batch,
                                                  adam_step=step, lr=lr, threads=threads)
            losses.append(float(loss))
        flat = lambda state: [a for pair in zip(state[0], state[1]) for a in pair]
        device = [trajectory_distance(g, c, s, lr, step) for g, c, s in zip(model.parameters(), flat(cpu), start)]
        floor = [trajectory_distance(o, c, s, lr, step) for o, c, s in zip(restored(other), flat(cpu), start)]
        table.append({"step": step, "device_loss": device_loss, "cpu_loss": losses[0], "cpu_reordered_loss": losses[1],
                      "device_vs_cpu": device, "cpu_reordered_vs_cpu": floor})
        report("full_width_training_20_steps", table)
    # Measured: the reordered CPU run stays within 1e-4 (relative L2) of
    # the CPU run for the first two steps and reaches 0.10 after twenty, the device starts at 0.04 and reaches
    # 0.19.  The device's head start is the 3xTF32 product: its error (about one unit of 2^-24 sum|a b|, see
    # the GEMM bound) is some twenty times that of OpenBLAS's blocked FMA sums, so about twenty times as many
    # pre-activations land on the other side of zero in the first steps (a handful per layer among 8.4
    # million); each such gate changes its sample's contribution to every gradient below.  From step 7 on the
    # device is 3 to 6 times as far from the CPU run as the reordered CPU run is.
    for row in table:
        step = row["step"]
        loss_floor = abs(row["cpu_reordered_loss"] - row["cpu_loss"])
        assert abs(row["device_loss"] - row["cpu_loss"]) <= 3 * loss_floor + 2e-3 * abs(row["cpu_loss"]), row
        for index, (d, f) in enumerate(zip(row["device_vs_cpu"], row["cpu_reordered_vs_cpu"])):
            assert d["relative_l2"] <= 3 * f["relative_l2"] + 0.06, (step, index, d, f)
            assert d["share_apart"] <= 3 * f["share_apart"] + 0.025, (step, index, d, f)
            assert d["mean"] <= 3 * f["mean"] + 0.01 * lr * step, (step, index, d, f)
            assert d["relative_l2"] <= 0.4 and d["share_apart"] <= 0.1, (step, index, d)
    assert model.optimizer_steps() == steps
    model.close()
