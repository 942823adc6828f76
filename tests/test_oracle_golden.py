"""Pins the CPU checker against the reference's own known-answer tests (no GPU needed)."""
import json
import math
import os

import numpy as np
import pytest

import golden_cases

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))


def _vals(seq):
    return np.array([float(v) for v in seq], dtype=np.float32)


def test_matmul_integer_known_answers(oracle):
    for key in ("matmul_int_2x3x2", "matmul_qualifier_smoke"):
        g = GOLDEN[key]
        a = np.array(g["a"], dtype=np.float32)
        b = np.array(g["b"], dtype=np.float32)
        assert np.array_equal(oracle.matmul(a, b), np.array(g["c"], dtype=np.float32)), key
    # transposed-output form of the same product (CpuOpenBlasRouteConformanceTest.java:315)
    g = GOLDEN["matmul_int_2x3x2"]
    a = np.array(g["a"], dtype=np.float32)
    b = np.array(g["b"], dtype=np.float32)
    assert np.array_equal(oracle.matmul(b.T, a.T).ravel(), np.array([58, 139, 64, 154], dtype=np.float32))


def test_matmul_mod5_exact_and_views(oracle):
    g = GOLDEN["matmul_mod5"]
    m, k, n = g["m"], g["k"], g["n"]
    a = (np.arange(m * k) % 5 - 2).astype(np.float32).reshape(m, k)
    b = (np.arange(k * n) % 5 - 2).astype(np.float32).reshape(k, n)
    expect = (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)
    assert np.array_equal(oracle.matmul(a, b), expect)
    # a permuted (strided) right operand, as Linear hands W[N,K] to MATMUL as a [K,N] view
    w = np.ascontiguousarray(b.T)
    assert np.array_equal(oracle.matmul(a, w.T), expect)
    # K == 1 is a single product
    assert np.array_equal(oracle.matmul(a[:, :1], b[:1, :]), a[:, :1] * b[:1, :])


def test_matmul_is_sequential_not_pairwise(oracle):
    # 1e8 + 1 - 1e8 in ascending k order: the 1 is absorbed; a pairwise or FMA tree would differ
    a = np.array([[1e8, 1.0, -1e8]], dtype=np.float32)
    b = np.ones((3, 1), dtype=np.float32)
    assert oracle.matmul(a, b)[0, 0] == 0.0


def test_softmax_known_answers(oracle):
    g = GOLDEN["softmax_123"]
    p = oracle.softmax(_vals(g["x"])[None, :])[0]
    assert np.allclose(p, _vals(g["p"]), atol=g["tol"], rtol=0)
    assert np.array_equal(oracle.softmax(_vals(GOLDEN["softmax_1000_1000"]["x"])[None, :])[0], _vals([0.5, 0.5]))
    p = oracle.softmax(_vals(GOLDEN["softmax_neginf_1000"]["x"])[None, :])[0]
    assert p[0] == 0.0 and not np.signbit(p[0]) and math.isnan(p[1])
    assert np.array_equal(oracle.softmax(_vals(GOLDEN["softmax_0_m1000"]["x"])[None, :])[0], _vals([1.0, 0.0]))
    p = oracle.softmax(_vals(["inf", 1.0, "inf"])[None, :])[0]
    assert math.isnan(p[0]) and p[1] == 0.0 and math.isnan(p[2])


def test_log_softmax_known_answers(oracle):
    for key in ("log_softmax_0_m1000", "log_softmax_extreme", "log_softmax_0_0", "log_softmax_inf_1"):
        g = GOLDEN[key]
        y, expect = oracle.log_softmax(_vals(g["x"])[None, :])[0], _vals(g["y"])
        assert np.array_equal(y, expect, equal_nan=True), key
    assert not np.signbit(oracle.log_softmax(_vals([0, -1000])[None, :])[0, 0])
    g = GOLDEN["log_softmax_columns"]
    for x, y in zip(g["x"], g["y"]):
        assert np.allclose(oracle.log_softmax(_vals(x)[None, :])[0], _vals(y), atol=g["tol"], rtol=0)


def test_categorical_loss_known_answers(oracle):
    g = GOLDEN["dense_ce_0_0"]
    per_row, mean = oracle.dense_cross_entropy(np.array(g["logits"], dtype=np.float32), np.array(g["target"], dtype=np.float32), "mean")
    assert mean == np.float32(2.0) * np.float32(g["loss"] / 2) and per_row[0] == mean
    g = GOLDEN["index_ce_0_0"]
    assert oracle.index_cross_entropy(np.array(g["logits"], dtype=np.float32), g["labels"])[1] == np.float32(g["loss"])
    # an ignore index: the ignored row is skipped before its bounds are looked at and is not counted
    logits = np.zeros((3, 2), dtype=np.float32)
    per_row, mean = oracle.index_cross_entropy_ignore(logits, [1, 7, 0], 7, "mean")
    assert np.array_equal(per_row, np.array([g["loss"], 0.0, g["loss"]], dtype=np.float32)) and mean == np.float32(g["loss"])
    assert oracle.index_cross_entropy_ignore(logits, [1, 7, 0], 7, "sum")[1] == np.float32(2.0) * np.float32(g["loss"])
    assert np.isnan(oracle.index_cross_entropy_ignore(logits, [7, 7, 7], 7, "mean")[1])
    # without rows to ignore the two forward checkers agree, and so do the two gradient checkers
    rng = np.random.default_rng(5)
    x = rng.standard_normal((33, 17)).astype(np.float32)
    labels = rng.integers(0, 17, 33)
    assert np.array_equal(oracle.index_cross_entropy_ignore(x, labels, -1, "mean")[0], oracle.index_cross_entropy(x, labels)[0])
    assert np.array_equal(oracle.index_cross_entropy_ignore_backward(x, labels, -1), oracle.index_cross_entropy_backward(x, labels))
    # a one-hot dense target is the index loss, row by row
    hot = np.zeros_like(x)
    hot[np.arange(33), labels] = 1.0
    assert np.array_equal(oracle.dense_cross_entropy(x, hot, "none")[0], oracle.index_cross_entropy(x, labels)[0])
    assert np.array_equal(oracle.dense_cross_entropy_backward(x, hot), oracle.index_cross_entropy_backward(x, labels))


def test_loss_gradient_chains_are_the_derivatives_of_their_losses(oracle):
    # the reference's tests hold no FLOAT32 known answers for these gradient node lists, so the restatements
    # are checked against central differences of the binary64 loss they differentiate
    rng = np.random.default_rng(21)
    x = rng.standard_normal((6, 9)).astype(np.float32)
    labels = np.array([3, -100, 0, 8, -100, 5])
    target = rng.random((6, 9)).astype(np.float32)
    target[rng.random((6, 9)) < 0.4] = 0.0
    target[2] = 0.0

    def lse(z):
        m = z.max(axis=1, keepdims=True)
        return (m + np.log(np.exp(z - m).sum(axis=1, keepdims=True)))[:, 0]

    def index_loss(z, reduction):
        active = labels != -100
        rows = lse(z)[active] - z[active, labels[active]]
        return rows.mean() if reduction == "mean" else rows.sum()

    def dense_loss(z, reduction):
        rows = (target.astype(np.float64) * (lse(z)[:, None] - z)).sum(axis=1)
        return rows.mean() if reduction == "mean" else rows.sum()

    def central(loss, reduction):
        z = x.astype(np.float64)
        grad = np.zeros_like(z)
        for i in range(z.shape[0]):
            for j in range(z.shape[1]):
                hi, lo = z.copy(), z.copy()
                hi[i, j] += 1e-5
                lo[i, j] -= 1e-5
                grad[i, j] = (loss(hi, reduction) - loss(lo, reduction)) / 2e-5
        return grad

    for reduction in ("mean", "sum"):
        got = oracle.index_cross_entropy_ignore_backward(x, labels, -100, 1.0, reduction)
        assert np.abs(got - central(index_loss, reduction)).max() <= 1e-5
        got = oracle.dense_cross_entropy_backward(x, target, 1.0, reduction)
        assert np.abs(got - central(dense_loss, reduction)).max() <= 1e-5
    # per-row cotangents (reduction NONE): each row's derivative scaled by its own cotangent
    seed = rng.standard_normal(6).astype(np.float32)
    got = oracle.index_cross_entropy_ignore_backward(x, labels, -100, seed, "none")
    assert np.abs(got - central(index_loss, "sum") * seed[:, None]).max() <= 1e-5
    got = oracle.dense_cross_entropy_backward(x, target, seed, "none")
    assert np.abs(got - central(dense_loss, "sum") * seed[:, None]).max() <= 1e-5
    # softmax and log-softmax: y and the upstream gradient give the vector-Jacobian product
    up = rng.standard_normal(x.shape).astype(np.float32)
    z = x.astype(np.float64)
    p = np.exp(z - lse(z)[:, None])
    want = p * (up - (up * p).sum(axis=1, keepdims=True))
    assert np.abs(oracle.softmax_backward(oracle.softmax(x), up, False) - want).max() <= 1e-6
    want = up - p * up.sum(axis=1, keepdims=True)
    assert np.abs(oracle.softmax_backward(oracle.log_softmax(x), up, True) - want).max() <= 2e-6


def test_activation_gradient_chains_are_the_derivatives_of_their_activations(oracle):
    # the five activation gradient rules against central differences of the binary64 functions
    x = np.linspace(-4.0, 4.0, 33).astype(np.float32)
    up = np.full_like(x, 1.5)
    z = x.astype(np.float64)
    erf = np.vectorize(math.erf)
    functions = {
        "tanh": np.tanh,
        "sigmoid": lambda v: 1.0 / (1.0 + np.exp(-v)),
        "silu": lambda v: v / (1.0 + np.exp(-v)),
        "gelu": lambda v: 0.5 * v * (1.0 + erf(v / math.sqrt(2.0))),
        "gelu_tanh": lambda v: 0.5 * v * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (v + 0.044715 * v ** 3))),
    }
    for kind, f in functions.items():
        want = 1.5 * (f(z + 1e-6) - f(z - 1e-6)) / 2e-6
        y = getattr(oracle, kind)(x)
        got = oracle.activation_backward(kind, y, up, x)
        assert np.abs(got - want).max() <= 2e-6, kind


def test_relu_special_values(oracle):
    y = oracle.relu(_vals([-1.0, -0.0, 0.0, 2.5, "-inf", "inf", "nan"]))
    assert list(y[:6]) == [0.0, 0.0, 0.0, 2.5, 0.0, float("inf")] and math.isnan(y[6])
    assert not np.signbit(y[1])


def test_argmax_rules(oracle):
    nan = float("nan")
    rows = np.array([[1, 3, 3, 2], [-0.0, 0.0, 0.0, -0.0], [0.0, -0.0, 0.0, 0.0], [1, nan, 5, nan],
                     [-np.inf, -np.inf, -np.inf, -np.inf]], dtype=np.float32)
    assert list(oracle.argmax(rows)) == [1, 1, 0, 1, 0]


def test_exact_sum_rounds_once(oracle):
    # 2^24 + 1 + 1: sequential float addition loses both ones, the exact sum keeps them
    x = np.array([16777216.0, 1.0, 1.0], dtype=np.float32)
    assert oracle.exact_sum(x) == 16777218.0
    rng = np.random.default_rng(7)
    for scale in (1e-30, 1.0, 1e30):
        v = (rng.standard_normal(4097) * scale).astype(np.float32)
        assert oracle.exact_sum(v) == np.float32(math.fsum(float(t) for t in v))
    tie = np.array([1.0, 2.0 ** -24], dtype=np.float32)           # exact tie rounds to even
    assert oracle.exact_sum(tie) == 1.0
    assert oracle.exact_sum(np.array([1.0, 2.0 ** -24, 2.0 ** -40], dtype=np.float32)) == np.float32(1.0 + 2.0 ** -23)
    assert oracle.exact_sum(np.array([1e-45, -1e-45, 3e-45], dtype=np.float32)) == np.float32(3e-45)
    assert math.isnan(oracle.exact_sum(np.array([np.inf, -np.inf], dtype=np.float32)))


def test_index_cross_entropy_and_label_check(oracle):
    logits = np.array([[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]], dtype=np.float32)
    per_row, mean = oracle.index_cross_entropy(logits, [2, 0])
    assert abs(per_row[0] - (-math.log(0.66524096))) < 1e-6
    assert abs(per_row[1] - math.log(3.0)) < 1e-6
    assert mean == np.float32((per_row[0] + per_row[1]) / np.float32(2))
    try:
        oracle.index_cross_entropy(logits, [3, 0])
    except ValueError:
        pass
    else:
        raise AssertionError("out-of-range label must be rejected")
    d = oracle.index_cross_entropy_backward(logits, [2, 0])
    p = oracle.softmax(logits)
    hot = np.array([[0, 0, 1], [1, 0, 0]], dtype=np.float32)
    assert np.allclose(d, (p - hot) / 2, atol=1e-7)
    assert abs(float(d.sum())) < 1e-6


def test_mse_exact_count_quotient(oracle):
    p = np.array([1.0, 2.0, 4.0], dtype=np.float32)
    t = np.array([0.0, 0.0, 0.0], dtype=np.float32)
    assert oracle.mse(p, t) == np.float32(21.0 / 3.0)
    assert oracle.mse(p[:3] * 0 + 1, t) == np.float32(1.0)
    one_third = oracle.mse(np.array([1.0, 0.0, 0.0], dtype=np.float32), t)
    assert one_third == np.float32(1.0 / 3.0)
    assert np.array_equal(oracle.mse_backward(p, t), (p * 2) * np.float32(np.float32(1.0) / np.float32(3.0)))


def test_sgd_scalar_training_trace(oracle):
    g = GOLDEN["sgd_scalar_trace"]
    w = np.array([g["w0"]], dtype=np.float32)
    for step, s in enumerate(g["steps"]):
        error = np.float32(w[0] * np.float32(s["x"]) - np.float32(s["t"]))
        loss = np.float32(error * error)
        assert abs(loss - s["loss"]) <= g["tol"]
        grad = np.array([np.float32(2) * error * np.float32(s["x"])], dtype=np.float32)
        assert oracle.sgd(w, grad, lr=g["lr"], completed_steps=step)
        assert abs(w[0] - s["w_after"]) <= g["tol"]


def test_one_linear_model_journey(oracle):
    g = GOLDEN["one_linear_model"]
    w = np.array([[g["w0"]]], dtype=np.float32)
    x3 = np.array([[3.0]], dtype=np.float32)
    assert oracle.matmul(x3, w.T)[0, 0] == g["compute_3"]
    for key, probe, expect in (("train_1", 2.0, g["compute_2_after"]), ("train_2", 4.0, g["compute_4_after"])):
        s = g[key]
        x = np.array([[s["x"]]], dtype=np.float32)
        pred = oracle.matmul(x, w.T)
        error = pred - np.float32(s["t"])
        assert abs(float((error * error).sum()) - s["loss"]) <= g["tol"]
        dw = oracle.matmul((np.float32(2) * error).T, x)
        flat = w.reshape(-1)
        assert oracle.sgd(flat, dw.reshape(-1), lr=0.1)
        assert abs(oracle.matmul(np.array([[probe]], dtype=np.float32), w.T)[0, 0] - expect) <= g["tol"]


def test_adam_tracks_the_reference_double_oracle(oracle):
    g = GOLDEN["adam_oracle_3_steps"]
    for decoupled in (False, True):
        p = np.array([g["p0"]], dtype=np.float32)
        m = np.zeros(1, dtype=np.float32)
        v = np.zeros(1, dtype=np.float32)
        o_first = o_second = 0.0
        for step in range(1, 4):
            represented = float(p[0])
            published = 2.0 * represented
            grad = np.array([np.float32(2) * p[0]], dtype=np.float32)
            assert oracle.adam(p, grad, m, v, step, lr=g["lr"], beta1=g["beta1"], beta2=g["beta2"],
                               eps=g["eps"], weight_decay=g["weight_decay"], decoupled=decoupled)
            gradient = published if decoupled else published + 0.2 * represented
            o_first = 0.5 * o_first + 0.5 * gradient
            o_second = 0.25 * o_second + 0.75 * gradient * gradient
            c_first = o_first / (1.0 - 0.5 ** step)
            c_second = o_second / (1.0 - 0.25 ** step)
            base = represented * (1.0 - 0.1 * 0.2) if decoupled else represented
            o_parameter = base - 0.1 * c_first / (math.sqrt(c_second) + 0.01)
            assert abs(p[0] - o_parameter) <= g["tol_parameter"]
            assert abs(m[0] - o_first) <= g["tol_first"]
            assert abs(v[0] - o_second) <= g["tol_second"]


def test_adam_scales_before_dividing(oracle):
    g = GOLDEN["adam_scale_before_divide"]
    f = np.float32
    gradient = f(g["gradient"])
    rate = f(g["lr"])
    first_moment = f(0.5) * gradient
    second_step_moment = f(0.5) * first_moment
    corrected = second_step_moment / f(0.75)
    with np.errstate(over="ignore"):
        assert np.isinf(corrected / rate)
    update = (rate * corrected) / rate
    assert np.isfinite(update)
    for decoupled in (False, True):
        p = np.array([1.0], dtype=np.float32)
        m = np.zeros(1, dtype=np.float32)
        v = np.zeros(1, dtype=np.float32)
        # step 1: second moment is g*g = inf in binary32 -> the reference rejects?  No: beta2 = 0
        # gives v = g*g = 1e38 (finite); sqrt = 1e19; update = (lr*g)/(1e19+eps) = lr -> p stays 1.
        assert oracle.adam(p, np.array([gradient]), m, v, 1, lr=g["lr"], beta1=g["beta1"],
                           beta2=g["beta2"], eps=g["eps"], decoupled=decoupled)
        assert p[0] == f(1.0) and m[0] == first_moment and v[0] == gradient * gradient
        assert oracle.adam(p, np.array([0.0], dtype=np.float32), m, v, 2, lr=g["lr"], beta1=g["beta1"],
                           beta2=g["beta2"], eps=g["eps"], decoupled=decoupled)
        assert p[0] == f(1.0) - update and m[0] == second_step_moment and v[0] == 0.0


def test_mlp_gradients_match_float64_autodiff(oracle):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((16, 5)).astype(np.float32)
    ws = [rng.standard_normal((7, 5)).astype(np.float32) * 0.5, rng.standard_normal((3, 7)).astype(np.float32) * 0.5]
    bs = [rng.standard_normal(7).astype(np.float32) * 0.1, rng.standard_normal(3).astype(np.float32) * 0.1]
    labels = rng.integers(0, 3, 16)
    loss, grads, logits = oracle.mlp_gradients(x, labels, ws, bs, "ce")
    # independent float64 evaluation
    x64 = x.astype(np.float64)
    z1 = x64 @ ws[0].T.astype(np.float64) + bs[0]
    a1 = np.maximum(z1, 0)
    z2 = a1 @ ws[1].T.astype(np.float64) + bs[1]
    e = np.exp(z2 - z2.max(1, keepdims=True))
    p = e / e.sum(1, keepdims=True)
    ref_loss = -np.log(p[np.arange(16), labels]).mean()
    d2 = p.copy()
    d2[np.arange(16), labels] -= 1
    d2 /= 16
    dw2, db2 = d2.T @ a1, d2.sum(0)
    d1 = (d2 @ ws[1].astype(np.float64)) * (z1 > 0)
    dw1, db1 = d1.T @ x64, d1.sum(0)
    assert abs(loss - ref_loss) < 1e-6
    for got, ref in zip(grads, (dw1, db1, dw2, db2)):
        assert np.allclose(got, ref, atol=2e-6, rtol=1e-5)


def test_pending_gradient_sum_is_all_or_nothing(oracle):
    # TrainingParameter.stageAccumulation (TrainingParameter.java:373-390): one binary32 addition per
    # element, committed only when every candidate is finite
    acc = np.array([1.0, 2.0 ** -24, 3.0e38], np.float32)
    assert oracle.accumulate(acc, np.array([2.0 ** -24, 2.0 ** -24, 0.0], np.float32))
    assert np.array_equal(acc, np.array([1.0, 2.0 ** -23, 3.0e38], np.float32))     # 1 + 2^-24 rounds to even
    before = acc.copy()
    assert not oracle.accumulate(acc, np.array([0.0, 0.0, 3.0e38], np.float32))   # overflow: rejected
    assert np.array_equal(acc, before)


def test_tanh_and_sigmoid_special_values(oracle):
    # the reference's tests hold no FLOAT32 known answers for these two; the values below follow from the
    # definition (binary64 function, one narrowing: CpuScalarReferenceKernel.java:1729-1742)
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 20.0, -20.0, -104.0], np.float32)
    t, s = oracle.tanh(x), oracle.sigmoid(x)
    assert t[0] == 0.0 and not np.signbit(t[0]) and t[1] == 0.0 and np.signbit(t[1])
    assert t[2] == 1.0 and t[3] == -1.0 and np.isnan(t[4]) and t[5] == 1.0 and t[6] == -1.0
    assert s[0] == 0.5 and s[1] == 0.5 and s[2] == 1.0 and s[3] == 0.0 and np.isnan(s[4]) and s[5] == 1.0
    assert s[6] == np.float32(np.exp(-20.0) / (1.0 + np.exp(-20.0))) and s[7] == 0.0       # underflows past the subnormals
    y = oracle.tanh(np.array([0.5], np.float32))
    assert oracle.activation_backward("tanh", y, np.array([2.0], np.float32))[0] == np.float32(2.0) * (np.float32(1.0) - y[0] * y[0])


def test_silu_special_values(oracle):
    # CpuScalarReferenceKernel.silu (:1236-1241): -inf gives -0, +inf stays +inf, NaN stays NaN, x = 0 gives 0
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0], np.float32)
    y = oracle.silu(x)
    assert y[0] == 0.0 and y[1] == 0.0 and np.signbit(y[1]) and y[2] == np.inf
    assert y[3] == 0.0 and np.signbit(y[3]) and np.isnan(y[4])
    assert y[5] == np.float32(1.0 / (1.0 + np.exp(-1.0)))
    g = oracle.activation_backward("silu", None, np.array([3.0, 3.0], np.float32), np.array([np.inf, -np.inf], np.float32))
    assert g[0] == 3.0 and g[1] == 0.0


def test_gelu_tanh_special_values_and_coefficients(oracle):
    # CpuScalarReferenceKernel.geluTanhApproximation (:1224-1229): -inf gives -0, +inf stays +inf, 0 gives 0;
    # the gradient rule's FLOAT32 coefficients are the bit patterns of ElementwiseGradientRules.java:370-378
    x = np.array([0.0, np.inf, -np.inf, np.nan, 1.0], np.float32)
    y = oracle.gelu_tanh(x)
    assert y[0] == 0.0 and y[1] == np.inf and y[2] == 0.0 and np.signbit(y[2]) and np.isnan(y[3])
    want = 0.5 * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (1.0 + 0.044715)))
    assert y[4] == np.float32(want)
    assert oracle._coefficient(0x3F000000) == np.float32(0.5) and oracle._coefficient(0x3D372713) == np.float32(0.044715)
    assert oracle._coefficient(0x3F4C422A) == np.float32(np.sqrt(2.0 / np.pi))
    assert oracle._coefficient(0x3E095D4F) == np.float32(3 * 0.044715)
    g = oracle.activation_backward("gelu_tanh", None, np.array([3.0, 3.0, 2.0], np.float32), np.array([np.inf, -np.inf, 0.0], np.float32))
    assert g[0] == 3.0 and g[1] == 0.0 and g[2] == 1.0            # d/dx at 0 is 1/2, times g = 2


def test_erf_and_exact_gelu_special_values(oracle):
    g = GOLDEN["erf_special_values"]
    y, want = oracle.erf(_vals(g["x"])), _vals(g["y"])
    assert np.isnan(y[0]) and y[1] == 1.0 and y[2] == -1.0 and y[3] == 0.0 and np.signbit(y[3])
    assert abs(float(y[4]) - float(want[4])) <= g["tol"]
    # the reference returns +-1 from |x| = 6 on (CpuScalarReferenceKernel.java:1258); so does erf in binary64
    assert np.array_equal(oracle.erf(_vals([6.0, -6.0, 7.5])), _vals([1.0, -1.0, 1.0]))
    # exact GELU (CpuScalarEmitter.java:441-452): -inf gives -0, +inf stays +inf, signed zeros kept
    x = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0], np.float32)
    y = oracle.gelu(x)
    assert y[0] == 0.0 and not np.signbit(y[0]) and y[1] == 0.0 and np.signbit(y[1])
    assert y[2] == np.inf and y[3] == 0.0 and np.signbit(y[3]) and np.isnan(y[4])
    assert y[5] == np.float32(0.5 * (1.0 + math.erf(1.0 / math.sqrt(2.0))))
    # gradient rule coefficients (ElementwiseGradientRules.java:370-378) and its infinity selection
    assert oracle._coefficient(0x3F3504F3) == np.float32(1.0 / math.sqrt(2.0))
    assert oracle._coefficient(0x3ECC422A) == np.float32(1.0 / math.sqrt(2.0 * math.pi)) and oracle._coefficient(0xBF000000) == -0.5
    grad = oracle.activation_backward("gelu", None, np.array([3.0, 3.0, 2.0], np.float32), np.array([np.inf, -np.inf, 0.0], np.float32))
    assert grad[0] == 3.0 and grad[1] == 0.0 and grad[2] == 1.0            # d/dx at 0 is 1/2, times g = 2


def test_clamp_signed_zero_and_nan_rules(oracle):
    # documented on Tensor.clamp (Tensor.java:2325-2331): NaN input gives NaN; bounds [-0, +0] keep -0 for
    # negative inputs and -0, +0 for positive inputs and +0; bounds [+0, -0] give -0 for every non-NaN input
    x = np.array([-3.0, -0.0, 0.0, 2.0, np.nan], np.float32)
    a = oracle.clamp(x, -0.0, 0.0)
    assert list(np.signbit(a[:4])) == [True, True, False, False] and not a[:4].any() and np.isnan(a[4])
    b = oracle.clamp(x, 0.0, -0.0)
    assert all(np.signbit(b[:4])) and not b[:4].any() and np.isnan(b[4])
    assert list(oracle.clamp(np.array([-5.0, 0.25, 9.0], np.float32), -1.0, 1.5)) == [-1.0, 0.25, 1.5]
    g = oracle.clamp_backward(np.array([-2.0, -1.0, 0.0, 1.5, 2.0], np.float32), np.full(5, 4.0, np.float32), -1.0, 1.5)
    assert list(g) == [0.0, 2.0, 4.0, 2.0, 0.0]


def test_squared_error_reductions(oracle):
    # CpuLossReferenceKernel.meanSquaredError (:67-87): NONE keeps (p - t)^2 per element, SUM adds them in
    # increasing order in binary32, MEAN divides that sum by the count exactly
    p = np.array([1.0, 2.0, 4.0, 1.0], np.float32)
    t = np.array([0.0, 0.0, 1.0, 1.0 + 2.0 ** -12], np.float32)
    assert list(oracle.squared_error(p, t, "none")) == [1.0, 4.0, 9.0, 2.0 ** -24]
    assert oracle.squared_error(p, t, "sum") == np.float32(14.0)            # 14 + 2^-24 rounds back to 14
    assert oracle.mse(p, t) == np.float32(3.5)


class CheckerBackend:
    """The CPU checker behind the interface of golden_cases."""

    def __init__(self, oracle):
        self.o = oracle

    def softmax(self, x, log):
        return self.o.log_softmax(x) if log else self.o.softmax(x)

    def softmax_backward(self, y, g, log):
        with np.errstate(all="ignore"):
            return self.o.softmax_backward(y, g, log)

    def softmax_with_backward(self, x, g, log):
        y = self.softmax(x, log)
        return y, self.softmax_backward(y, g, log)

    def index_ce(self, logits, labels, reduction, ignore, label_dtype):
        ignore = -(2 ** 40) if ignore is None else ignore           # a value no label takes
        per_row, reduced = self.o.index_cross_entropy_ignore(logits, labels, ignore, reduction)
        return per_row if reduction == "none" else reduced

    def index_ce_backward(self, logits, labels, seed, reduction, ignore, label_dtype):
        ignore = -(2 ** 40) if ignore is None else ignore
        with np.errstate(all="ignore"):
            return self.o.index_cross_entropy_ignore_backward(logits, labels, ignore, seed, reduction)

    def dense_ce(self, logits, target, reduction):
        per_row, reduced = self.o.dense_cross_entropy(logits, target, reduction)
        return per_row if reduction == "none" else reduced

    def dense_ce_backward(self, logits, target, seed, reduction):
        with np.errstate(all="ignore"):
            return self.o.dense_cross_entropy_backward(logits, target, seed, reduction)

    def unary(self, name, x):
        return {"erf": self.o.erf, "gelu": self.o.gelu}[name](x)


@pytest.mark.parametrize("check", golden_cases.ALL_CHECKS, ids=lambda f: f.__name__)
def test_reference_held_gradient_rule_vectors(oracle, check):
    check(CheckerBackend(oracle))


class LowCheckerBackend:
    """The CPU checker's 16-bit storage functions behind the interface of golden_cases."""

    def __init__(self, oracle):
        self.o = oracle

    def low_matmul(self, kind, a_bits, b_bits):
        return self.o.low_encode(kind, self.o.matmul(self.o.low_decode(kind, np.ascontiguousarray(a_bits)), self.o.low_decode(kind, np.ascontiguousarray(b_bits))))

    def low_unary(self, kind, name, bits):
        return self.o.low_encode(kind, self.o.low_activation(name, self.o.low_decode(kind, bits)))


@pytest.mark.parametrize("check", golden_cases.LOW_CHECKS, ids=lambda f: f.__name__)
def test_reference_held_low_precision_vectors(oracle, check):
    check(LowCheckerBackend(oracle))
