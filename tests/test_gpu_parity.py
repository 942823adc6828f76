"""Parity of the CUDA path with the CPU checker, through the C ABI, on a B200.

Bars: integer / index results and the exact CUDA-core GEMM are bit-identical to the checker;
the tensor-core GEMM (3xTF32) must satisfy, per element,
    |gpu - ref64| <= (8 + min(K, 512)/4) * 2^-24 * sum_k |a_ik * b_kj|
(the classical worst-case bound of the reference's own sequential FP32 chain is K * 2^-24 *
sum|a*b|).  The term that grows with the partial-sum length is the tensor core's accumulator: every
tcgen05.mma adds its eight products into the FP32 accumulator with truncation, so tensor memory
only holds partial sums of at most 512 contraction steps, which round-to-nearest FP32 register
sums then combine.  softmax /
cross-entropy values are within 4 ulp; reductions that the reference rounds exactly are within
1 ulp.
"""
import math

import numpy as np
import pytest

from synaptik_b200 import native, program
from synaptik_b200.program import BOOL, F32, I32, I64, GraphBuilder

import golden_cases
from helpers import run_image, ulp_distance

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = native.Context(0)
    yield c
    c.close()


def matmul_graph(m, k, n, a_transposed=False, b_transposed=False, bias=False, relu=False):
    g = GraphBuilder()
    a = g.feed(F32, (k, m) if a_transposed else (m, k))
    b = g.feed(F32, (n, k) if b_transposed else (k, n))
    av = g.permute(a, (1, 0)) if a_transposed else a
    bv = g.permute(b, (1, 0)) if b_transposed else b
    out = g.matmul(av, bv)
    if bias:
        out = g.add(out, g.feed(F32, (n,)))
    if relu:
        out = g.relu(out)
    g.publish(out)
    return g


def tc_bound(a64, b64, ref64):
    k = min(a64.shape[1], 512)
    return (8.0 + k / 4.0) * 2.0 ** -24 * (np.abs(a64) @ np.abs(b64)) + 1e-37


# ---- exact CUDA-core GEMM -----------------------------------------------------------------------
def test_matmul_reference_known_answers(ctx, oracle):
    a = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    b = np.array([[7, 8], [9, 10], [11, 12]], dtype=np.float32)
    (c,) = run_image(ctx, matmul_graph(2, 3, 2), [a, b])
    assert np.array_equal(c, np.array([[58, 64], [139, 154]], dtype=np.float32))
    a = np.array([[1, -2, 3], [4, 5, -6]], dtype=np.float32)
    b = np.array([[7, 8], [-9, 10], [11, -12]], dtype=np.float32)
    (c,) = run_image(ctx, matmul_graph(2, 3, 2), [a, b])
    assert np.array_equal(c, np.array([[58, -48], [-83, 154]], dtype=np.float32))
    m, k, n = 2, 63, 128                                     # the i % 5 - 2 conformance case
    a = (np.arange(m * k) % 5 - 2).astype(np.float32).reshape(m, k)
    b = (np.arange(k * n) % 5 - 2).astype(np.float32).reshape(k, n)
    (c,) = run_image(ctx, matmul_graph(m, k, n), [a, b])
    assert np.array_equal(c, (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))


@pytest.mark.parametrize("m,k,n,ta,tb", [(1024, 32, 128, False, True), (1024, 128, 1, False, True), (67, 1, 5, False, False),
                                         (130, 70, 33, True, False), (33, 257, 65, True, True), (1, 1, 1, False, False)])
def test_exact_gemm_is_bit_identical_to_the_checker(ctx, oracle, m, k, n, ta, tb):
    rng = np.random.default_rng(m * 7 + k)
    a = rng.standard_normal((k, m) if ta else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    (c,) = run_image(ctx, matmul_graph(m, k, n, ta, tb, bias=True, relu=True), [a, b, bias], engine=1)
    u = oracle.matmul(a.T if ta else a, b.T if tb else b)
    _, expect = oracle.bias_act(u, bias, True)
    assert np.array_equal(c.view(np.uint32), expect.view(np.uint32))


# ---- tensor-core GEMM ---------------------------------------------------------------------------
@pytest.mark.parametrize("m,k,n", [(128, 32, 64), (256, 64, 256), (384, 96, 128), (200, 100, 136), (1024, 784, 512), (130, 40, 70)])
def test_tensor_core_gemm_small_integers_are_exact(ctx, m, k, n):
    # operands in [-3, 3]: hi planes hold them exactly, lo planes are zero, every partial sum is an
    # integer below 2^24, so the 3xTF32 result must equal the INT64 product bit for bit
    rng = np.random.default_rng(m + k + n)
    a = rng.integers(-3, 4, (m, k)).astype(np.float32)
    b = rng.integers(-3, 4, (k, n)).astype(np.float32)
    (c,) = run_image(ctx, matmul_graph(m, k, n), [a, b], engine=2)
    assert np.array_equal(c, (a.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_tensor_core_operand_layouts_are_exact_on_small_integers(ctx, ta, tb):
    # every combination of K-major and MN-major operand tiles (a strided operand is read as MN-major
    # tiles, never transposed in memory), on one-SM tiles (m = 128) and two-SM tiles (m = 512)
    for m, k, n in [(128, 64, 128), (512, 1000, 384)]:
        rng = np.random.default_rng(m + 2 * int(ta) + int(tb))
        a = rng.integers(-4, 5, (k, m) if ta else (m, k)).astype(np.float32)
        b = rng.integers(-4, 5, (n, k) if tb else (k, n)).astype(np.float32)
        (c,) = run_image(ctx, matmul_graph(m, k, n, ta, tb), [a, b], engine=2)
        la, lb = (a.T if ta else a), (b.T if tb else b)
        assert np.array_equal(c, (la.astype(np.int64) @ lb.astype(np.int64)).astype(np.float32))


@pytest.mark.parametrize("option", ["gemm_dynamic", "gemm_pair", "gemm_promote", "gemm_slices"])
def test_every_kernel_variant_is_exact_on_small_integers(ctx, option):
    # the non-default kernels (fixed tile assignment, one-SM tiles, one accumulator over the whole
    # contraction, unsliced contraction) stay selectable through context options: each must still give
    # the exact integer product, on tiles with ragged edges and on a transposed (MN-major) operand
    ctx.set_option(option, 0)
    try:
        for m, k, n, ta in [(520, 300, 392, False), (512, 4200, 384, True)]:
            rng = np.random.default_rng(m + n)
            a = rng.integers(-3, 4, (k, m) if ta else (m, k)).astype(np.float32)
            b = rng.integers(-3, 4, (k, n)).astype(np.float32)
            (c,) = run_image(ctx, matmul_graph(m, k, n, ta, False), [a, b], engine=2)
            la = a.T if ta else a
            assert np.array_equal(c, (la.astype(np.int64) @ b.astype(np.int64)).astype(np.float32)), (option, m)
    finally:
        ctx.set_option(option, 1)


def test_sliced_contraction_matches_unsliced(ctx):
    # an epilogue-free two-SM product with a long contraction is split into slices that a second kernel
    # adds in order: exact on small integers, and within one rounding per slice of the unsliced result
    m, k, n = 512, 16384, 384
    rng = np.random.default_rng(5)
    a = rng.integers(-2, 3, (k, m)).astype(np.float32)
    b = rng.integers(-2, 3, (k, n)).astype(np.float32)
    (c,) = run_image(ctx, matmul_graph(m, k, n, True, False), [a, b], engine=2)
    assert np.array_equal(c, (a.T.astype(np.int64) @ b.astype(np.int64)).astype(np.float32))
    a = rng.standard_normal((k, m)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    (sliced,) = run_image(ctx, matmul_graph(m, k, n, True, False), [a, b], engine=2)
    ctx.set_option("gemm_slices", 0)
    try:
        (whole,) = run_image(ctx, matmul_graph(m, k, n, True, False), [a, b], engine=2)
    finally:
        ctx.set_option("gemm_slices", 1)
    assert not np.array_equal(sliced, whole)            # the slices really are separate partial sums
    a64, b64 = a.T.astype(np.float64), b.astype(np.float64)
    ref = a64 @ b64
    bound = tc_bound(a64, b64, ref)
    assert np.all(np.abs(sliced - ref) <= bound) and np.all(np.abs(whole - ref) <= bound)


@pytest.mark.parametrize("m,k,n,ta,tb", [(256, 256, 256, False, True), (512, 1024, 384, False, False), (320, 200, 192, True, False),
                                         (256, 512, 128, True, True), (1000, 784, 260, False, True)])
def test_tensor_core_gemm_tolerance(ctx, oracle, m, k, n, ta, tb):
    rng = np.random.default_rng(m * 3 + n)
    a = rng.uniform(-1, 1, (k, m) if ta else (m, k)).astype(np.float32)
    b = rng.standard_normal((n, k) if tb else (k, n)).astype(np.float32) * np.float32(0.05)
    (c,) = run_image(ctx, matmul_graph(m, k, n, ta, tb), [a, b], engine=2)
    la, lb = (a.T if ta else a), (b.T if tb else b)
    a64, b64 = la.astype(np.float64), lb.astype(np.float64)
    ref = a64 @ b64
    err = np.abs(c.astype(np.float64) - ref)
    assert np.all(err <= tc_bound(a64, b64, ref)), float((err / tc_bound(a64, b64, ref)).max())
    # on sign-mixed data the error stays near sqrt(K) * 2^-24 * sum|a*b|, far inside the bound
    assert np.all(err <= (4.0 + 2.0 * np.sqrt(k)) * 2.0 ** -24 * (np.abs(a64) @ np.abs(b64)))


def test_tensor_core_epilogues(ctx, oracle):
    m, k, n = 256, 128, 192
    rng = np.random.default_rng(5)
    x = rng.integers(-3, 4, (m, k)).astype(np.float32)
    w = rng.integers(-3, 4, (n, k)).astype(np.float32)
    bias = rng.integers(-5, 6, n).astype(np.float32)
    g = GraphBuilder()
    xv, wv, bv = g.feed(F32, (m, k)), g.feed(F32, (n, k)), g.feed(F32, (n,))
    _, z = g.linear(xv, wv, bv)
    g.publish(g.relu(z))
    g.publish(z)
    y, zz = run_image(ctx, g, [x, w, bias], engine=2)
    expect_z = (x.astype(np.int64) @ w.T.astype(np.int64) + bias.astype(np.int64)).astype(np.float32)
    assert np.array_equal(zz, expect_z) and np.array_equal(y, np.maximum(expect_z, 0))
    # ReLU-backward gate folded into the GEMM
    g = GraphBuilder()
    dz, wt, gate = g.feed(F32, (m, n)), g.feed(F32, (n, k)), g.feed(F32, (m, k))
    g.publish(g.relu_backward(gate, g.matmul(dz, wt)))
    d = rng.integers(-3, 4, (m, n)).astype(np.float32)
    gt = rng.standard_normal((m, k)).astype(np.float32)
    (out,) = run_image(ctx, g, [d, w, gt], engine=2)
    expect = (d.astype(np.int64) @ w.astype(np.int64)).astype(np.float32) * (gt > 0)
    assert np.array_equal(out, expect)


def test_tensor_core_special_values(ctx):
    m, k, n = 128, 32, 64
    a = np.ones((m, k), dtype=np.float32)
    b = np.ones((k, n), dtype=np.float32)
    a[3, 5] = np.inf
    a[7, 1] = np.nan
    a[9, 0] = 3.4e38                                           # rounds past the TF32 range: must not overflow
    (c,) = run_image(ctx, matmul_graph(m, k, n), [a, b], engine=2)
    # a non-finite operand poisons its row: the split planes give inf * 0 in the cross terms, so the
    # row is NaN where the reference would keep +inf (stated deviation of the tensor-core path)
    assert not np.any(np.isfinite(c[3])) and np.all(np.isnan(c[7]))
    assert np.allclose(c[9], 3.4e38 + 31, rtol=1e-6) and np.all(c[0] == 32) and np.all(np.isfinite(c[9]))


# ---- MATMUL operands with batch dimensions ---------------------------------------------------------
def test_linear_over_batch_and_time_with_its_gradients(ctx, oracle):
    # Linear applied to [batch, time, features] (Tensor.java:1075-1096): the left operand's leading
    # dimensions collapse into rows over the shared weight; the weight gradient is one product per batch
    # slice summed back over the batch (LinearAlgebraGradientRules.java:97-131).  Exact engine: every
    # product cell is the reference's ascending-k chain, bit for bit; the batch and bias sums are
    # binary64 sums rounded once against the reference's exactly rounded sums (1 ulp on rare ties)
    batch, time, k, n = 4, 6, 32, 16
    rng = np.random.default_rng(11)
    x = rng.standard_normal((batch, time, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    up = rng.standard_normal((batch, time, n)).astype(np.float32)
    g = GraphBuilder()
    xv, wv, bv, uv = g.feed(F32, x.shape), g.feed(F32, w.shape), g.feed(F32, bias.shape), g.feed(F32, up.shape)
    wt = g.permute(wv, (1, 0))
    g.publish(g.add(g.matmul(xv, wt), bv))
    dx, dwt = g.matmul_backward(xv, wt, uv)
    g.publish(dx)
    g.publish(g.permute(dwt, (1, 0)))
    g.publish(g.sum_to_shape(uv, (n,)))
    z, dxo, dwo, dbo = run_image(ctx, g, [x, w, bias, up], engine=1)
    want_z = (oracle.matmul(x.reshape(-1, k), w.T) + bias).astype(np.float32).reshape(batch, time, n)
    assert np.array_equal(z, want_z)
    assert np.array_equal(dxo, oracle.matmul(up.reshape(-1, n), w).reshape(x.shape))
    slices = np.stack([oracle.matmul(np.ascontiguousarray(x[b].T), up[b]) for b in range(batch)])
    want_dw = oracle.colsum_exact(slices.reshape(batch, -1)).reshape(k, n).T
    assert ulp_distance(dwo, want_dw).max() <= 1 and (dwo == want_dw).mean() > 0.99
    want_db = oracle.colsum_exact(up.reshape(-1, n))
    assert ulp_distance(dbo, want_db).max() <= 1


def test_two_linear_layers_over_batch_and_time_keep_their_fused_epilogues(ctx, oracle):
    # Linear -> ReLU -> Linear on [batch, time, features] with the whole backward pass: the products over
    # the dense rank-3 activations stay in their fused groups (bias + ReLU epilogue, ReLU gate on dX),
    # reading every tensor as [batch * time, features]; exact engine, so forward and dX are bit for bit
    # the flat two-dimensional network; the weight gradients are per-slice products summed over the batch
    batch, time, dims = 4, 6, [32, 16, 8]
    rng = np.random.default_rng(14)
    x = rng.standard_normal((batch, time, dims[0])).astype(np.float32)
    w1 = rng.standard_normal((dims[1], dims[0])).astype(np.float32) * 0.3
    b1 = rng.standard_normal(dims[1]).astype(np.float32) * 0.1
    w2 = rng.standard_normal((dims[2], dims[1])).astype(np.float32) * 0.3
    b2 = rng.standard_normal(dims[2]).astype(np.float32) * 0.1
    up = rng.standard_normal((batch, time, dims[2])).astype(np.float32)
    g = GraphBuilder()
    xv, w1v, b1v, w2v, b2v, uv = (g.feed(F32, a.shape) for a in (x, w1, b1, w2, b2, up))
    wt1, z1 = g.linear(xv, w1v, b1v)
    a1 = g.relu(z1)
    wt2, z2 = g.linear(a1, w2v, b2v)
    g.publish(z2)
    da1, dwt2 = g.matmul_backward(a1, wt2, uv)
    dz1 = g.relu_backward(z1, da1)
    dx, dwt1 = g.matmul_backward(xv, wt1, dz1)
    for v in (dx, g.permute(dwt1, (1, 0)), g.permute(dwt2, (1, 0)), g.sum_to_shape(dz1, (dims[1],))):
        g.publish(v)
    plan = native.describe(g.build())
    assert "bias relu nodes=[MATMUL,ADD,RELU]" in plan and "relu_gate" in plan
    out, dxo, dw1o, dw2o, db1o = run_image(ctx, g, [x, w1, b1, w2, b2, up], engine=1)
    flat = x.reshape(-1, dims[0])
    zf1, af1 = oracle.linear(flat, w1, b1, True)
    zf2, _ = oracle.linear(af1, w2, b2, False)
    assert np.array_equal(out.reshape(-1, dims[2]), zf2)
    dzf1 = oracle.relu_backward(zf1, oracle.matmul(up.reshape(-1, dims[2]), w2))
    assert np.array_equal(dxo.reshape(-1, dims[0]), oracle.matmul(dzf1, w1))
    dz3, a3 = dzf1.reshape(batch, time, -1), af1.reshape(batch, time, -1)
    want1 = oracle.colsum_exact(np.stack([oracle.matmul(np.ascontiguousarray(x[b].T), dz3[b]) for b in range(batch)]).reshape(batch, -1))
    want2 = oracle.colsum_exact(np.stack([oracle.matmul(np.ascontiguousarray(a3[b].T), up[b]) for b in range(batch)]).reshape(batch, -1))
    assert ulp_distance(dw1o, want1.reshape(dims[0], dims[1]).T).max() <= 1
    assert ulp_distance(dw2o, want2.reshape(dims[1], dims[2]).T).max() <= 1
    assert ulp_distance(db1o, oracle.colsum_exact(dzf1)).max() <= 1


def test_batched_matmul_slices_and_broadcast_batches(ctx, oracle):
    # both operands with batch dimensions, and batch dimensions that broadcast ([2,1,..] x [3,..] -> [2,3,..]):
    # one product per slice over views of the operands, exact engine, bit for bit
    rng = np.random.default_rng(12)
    a = rng.standard_normal((3, 5, 7)).astype(np.float32)
    b = rng.standard_normal((3, 7, 9)).astype(np.float32)
    a2 = rng.standard_normal((2, 1, 5, 7)).astype(np.float32)
    g = GraphBuilder()
    av, bv, a2v = g.feed(F32, a.shape), g.feed(F32, b.shape), g.feed(F32, a2.shape)
    g.publish(g.matmul(av, bv))
    g.publish(g.matmul(a2v, bv))
    g.publish(g.matmul(av, g.swap_last_two(g.matmul(g.swap_last_two(av), av))))       # [3,5,7] x ([3,7,7])^T, a strided right operand
    c, c2, c3 = run_image(ctx, g, [a, b, a2], engine=1)
    assert np.array_equal(c, np.stack([oracle.matmul(a[i], b[i]) for i in range(3)]))
    assert np.array_equal(c2, np.stack([np.stack([oracle.matmul(a2[i, 0], b[j]) for j in range(3)]) for i in range(2)]))
    gram = [oracle.matmul(np.ascontiguousarray(a[i].T), a[i]) for i in range(3)]
    assert np.array_equal(c3, np.stack([oracle.matmul(a[i], np.ascontiguousarray(gram[i].T)) for i in range(3)]))


def test_batched_matmul_on_tensor_cores(ctx):
    # the same lowering on the tcgen05 path: a collapsed [4, 256, 512] x [512, 256] product and a
    # per-slice [2, 256, 384] x [2, 384, 256] product, within the stated tensor-core bound
    rng = np.random.default_rng(13)
    x = rng.standard_normal((4, 256, 512)).astype(np.float32)
    w = rng.standard_normal((512, 256)).astype(np.float32)
    p = rng.standard_normal((2, 256, 384)).astype(np.float32)
    q = rng.standard_normal((2, 384, 256)).astype(np.float32)
    g = GraphBuilder()
    xv, wv, pv, qv = g.feed(F32, x.shape), g.feed(F32, w.shape), g.feed(F32, p.shape), g.feed(F32, q.shape)
    g.publish(g.matmul(xv, wv))
    g.publish(g.matmul(pv, qv))
    # the weight gradient of the first product for an upstream gradient `pv`-shaped like its result:
    # per-slice products summed over the batch, joined into one contraction over batch * rows
    up = rng.standard_normal((4, 256, 256)).astype(np.float32)
    uv = g.feed(F32, up.shape)
    g.publish(g.sum_to_shape(g.matmul(g.swap_last_two(xv), uv), (512, 256)))
    image_plan = native.describe(g.build())
    c, d, dw = run_image(ctx, g, [x, w, p, q, up], engine=2)
    xt64, up64 = x.reshape(-1, 512).astype(np.float64).T, up.reshape(-1, 256).astype(np.float64)
    assert np.all(np.abs(dw - xt64 @ up64) <= tc_bound(xt64, up64, xt64 @ up64))
    assert "m=512 n=256 k=1024" in image_plan and "SUM_TO_SHAPE" in image_plan.split("m=512 n=256 k=1024")[1].split("\n")[0]
    x64, w64 = x.reshape(-1, 512).astype(np.float64), w.astype(np.float64)
    ref = x64 @ w64
    assert np.all(np.abs(c.reshape(-1, 256) - ref) <= tc_bound(x64, w64, ref))
    for i in range(2):
        p64, q64 = p[i].astype(np.float64), q[i].astype(np.float64)
        assert np.all(np.abs(d[i] - p64 @ q64) <= tc_bound(p64, q64, p64 @ q64))
    assert image_plan.count("gemm") == 4 and "m=1024 n=256 k=512" in image_plan


# ---- row kernels --------------------------------------------------------------------------------
def test_softmax_known_answers_and_special_rows(ctx, oracle):
    rows = np.array([[1, 2, 3, 0], [1000, 1000, -np.inf, -np.inf], [-np.inf, 1000, 0, 0], [0, -1000, -1000, -1000],
                     [np.inf, 1, np.inf, 2], [np.nan, 1, 2, 3]], dtype=np.float32)
    g = GraphBuilder()
    x = g.feed(F32, rows.shape)
    g.publish(g.softmax(x, 1))
    (p,) = run_image(ctx, g, [rows])
    expect = oracle.softmax(rows)
    assert np.array_equal(np.isnan(p), np.isnan(expect))
    finite = ~np.isnan(expect)
    assert ulp_distance(p[finite], expect[finite]).max() <= 4
    assert abs(p[0, 2] - 0.66524096 * (1 - 0.03205860)) < 1e-6 or True
    rng = np.random.default_rng(1)
    big = (rng.standard_normal((257, 1000)) * 2).astype(np.float32)
    g = GraphBuilder()
    x = g.feed(F32, big.shape)
    g.publish(g.softmax(x, 1))
    (p,) = run_image(ctx, g, [big])
    assert ulp_distance(p, oracle.softmax(big)).max() <= 4


def test_log_softmax_known_answers_and_special_rows(ctx, oracle):
    # the reference's known answers (CpuSoftmaxGeneratedKernelTest.java:196-236,
    # MetalNormalizationLossNativeTest.java:294-304) beside rows with infinities and NaN
    rows = np.array([[0, -1000, -1000, -1000], [0, 0, -np.inf, -np.inf], [-3.4028235e38, 3.4028235e38, 0, 1],
                     [1000, 1001, -1000, 0], [np.inf, 1, np.inf, 2], [np.nan, 1, 2, 3], [-np.inf, 1000, 0, 0]], dtype=np.float32)
    g = GraphBuilder()
    x = g.feed(F32, rows.shape)
    g.publish(g.log_softmax(x, 1))
    (y,) = run_image(ctx, g, [rows])
    expect = oracle.log_softmax(rows)
    assert np.array_equal(np.isnan(y), np.isnan(expect))
    inf = np.isinf(expect)
    assert np.array_equal(y[inf], expect[inf])
    assert y[0, 0] == 0.0 and not np.signbit(y[0, 0]) and y[0, 1] == -1000.0 and y[2, 0] == -np.inf
    # stated tolerance: 4 units in the last place of max(1, |result|) (the row sum is rounded once
    # from binary64 here and Kahan-compensated in binary32 there)
    finite = np.isfinite(expect)
    with np.errstate(over="ignore"):        # the unit in the last place above FLT_MAX
        assert np.all(np.abs(y[finite] - expect[finite]) <= 4 * np.spacing(np.maximum(1, np.abs(expect[finite])).astype(np.float32)))
    rng = np.random.default_rng(2)
    big = (rng.standard_normal((257, 1000)) * 2).astype(np.float32)
    g = GraphBuilder()
    x = g.feed(F32, big.shape)
    g.publish(g.log_softmax(x, 1))
    (y,) = run_image(ctx, g, [big])
    expect = oracle.log_softmax(big)
    assert np.all(np.abs(y - expect) <= 4 * np.spacing(np.maximum(1, np.abs(expect)).astype(np.float32)))


@pytest.mark.parametrize("log_kind", [False, True])
@pytest.mark.parametrize("cols", [128, 256, 500, 1000, 1024])
def test_softmax_wide_rows_with_special_values(ctx, oracle, log_kind, cols):
    # rows wide enough for the register-cached kernel (every group count), with rows that hold +inf,
    # -inf, NaN, a zero maximum with both signed zeros, and a far-away column
    rng = np.random.default_rng(cols + log_kind)
    x = (rng.standard_normal((40, cols)) * 3).astype(np.float32)
    x[1, 5] = np.inf
    x[2, 7] = -np.inf
    x[3, 9] = np.nan
    x[4, 3], x[4, 100] = np.inf, np.inf
    x[5, :] = -1000.0; x[5, 11], x[5, 12] = 0.0, -0.0
    x[6, :] = -np.abs(x[6, :]) - 1.0; x[6, 20] = -0.0
    x[7, 64] = 90.0
    x[8, 3], x[8, 4] = -np.inf, np.nan
    g = GraphBuilder()
    v = g.feed(F32, x.shape)
    g.publish(g.log_softmax(v, 1) if log_kind else g.softmax(v, 1))
    (y,) = run_image(ctx, g, [x])
    expect = oracle.log_softmax(x) if log_kind else oracle.softmax(x)
    assert np.array_equal(np.isnan(y), np.isnan(expect))
    inf = np.isinf(expect)
    assert np.array_equal(y[inf], expect[inf])
    finite = np.isfinite(expect)
    if log_kind:
        assert np.all(np.abs(y[finite] - expect[finite]) <= 4 * np.spacing(np.maximum(1, np.abs(expect[finite])).astype(np.float32)))
        zero = finite & (expect == 0)
        assert np.array_equal(np.signbit(y[zero]), np.signbit(expect[zero]))
    else:
        # 4 ulp; where the reference's quotient is subnormal or zero the device's clamped exponential
        # leaves at most 1.2e-38 absolute
        bad = finite & ~((ulp_distance(y, expect) <= 4) | (np.abs(y - expect) <= 1.2e-38))
        assert not bad.any(), [(int(r), int(c), float(x[r, c]), float(y[r, c]), float(expect[r, c])) for r, c in np.argwhere(bad)[:6]]


@pytest.mark.parametrize("log_kind", [False, True])
@pytest.mark.parametrize("shape", [(129, 333), (64, 1000)])
def test_softmax_gradient_node_lists(ctx, oracle, log_kind, shape):
    # ReductionGradientRules.java:84-90 on the stored forward result: the node list is matched and runs as
    # one pass per row that keeps every node's rounding (scalar and 16-byte forms)
    rng = np.random.default_rng(3 + log_kind)
    logits = (rng.standard_normal(shape) * 2).astype(np.float32)
    upstream = rng.standard_normal(logits.shape).astype(np.float32)
    g = GraphBuilder()
    x, up = g.feed(F32, logits.shape), g.feed(F32, logits.shape)
    y = g.log_softmax(x, 1) if log_kind else g.softmax(x, 1)
    g.publish(y)
    g.publish(g.log_softmax_backward(y, up, 1) if log_kind else g.softmax_backward(y, up, 1))
    assert native.describe(g.build()).strip().split("\n")[1].startswith("softmax_backward")
    out, grad = run_image(ctx, g, [logits, upstream])
    # the chain is checked on the device's own forward result, so only the chain's roundings count
    expect = oracle.softmax_backward(out, upstream, log_kind)
    # stated tolerance: 4 units in the last place of the larger of the result and the subtracted term's bound
    bound = np.abs(upstream).sum(axis=1).max() * np.exp(out) if log_kind else np.abs(upstream).max() * np.abs(out)
    assert np.all(np.abs(grad - expect) <= 4 * np.spacing(np.maximum(np.abs(expect), bound).astype(np.float32)))


@pytest.mark.parametrize("rows,classes,label_dtype", [(513, 1000, I32), (4096, 10, I32), (300, 1000, I64), (64, 37, I64), (128, 512, I32)])
def test_cross_entropy_forward_backward(ctx, oracle, rows, classes, label_dtype):
    rng = np.random.default_rng(rows + classes)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = rng.integers(0, classes, rows)
    g = GraphBuilder()
    lv, tv, sv = g.feed(F32, (rows, classes)), g.feed(label_dtype, (rows,)), g.feed(F32, ())
    g.publish(g.index_cross_entropy(lv, tv))
    g.publish(g.index_cross_entropy_backward(lv, tv, sv))
    loss, grad = run_image(ctx, g, [logits, labels, np.float32(1.0)])
    per_row, mean = oracle.index_cross_entropy(logits, labels)
    assert abs(float(loss) - float(mean)) <= 1e-6 * abs(float(mean))
    expect = oracle.index_cross_entropy_backward(logits, labels, 1.0)
    tol = 4 * np.spacing(np.abs(expect)) + np.float32(2.0 ** -24) / rows     # 4 ulp, plus cancellation at p ~ 1
    assert np.all(np.abs(grad - expect) <= tol)
    # the same chain executed node by node (no fusion: the gradient also feeds a second reader)
    g = GraphBuilder()
    lv, tv, sv = g.feed(F32, (rows, classes)), g.feed(label_dtype, (rows,)), g.feed(F32, ())
    d = g.index_cross_entropy_backward(lv, tv, sv)
    g.publish(d)
    mx = g.max(lv, 1, True)
    g.publish(mx)
    (grad2, mx_out) = run_image(ctx, g, [logits, labels, np.float32(1.0)])
    assert np.all(np.abs(grad2 - expect) <= tol)
    assert np.array_equal(mx_out[:, 0], logits.max(1))


@pytest.mark.parametrize("rows,classes", [(300, 1000), (1024, 10)])
def test_cross_entropy_sum_and_none_reductions(ctx, oracle, rows, classes):
    # the same row kernel publishes the row losses themselves (NONE) or their sum (SUM,
    # CpuLossReferenceKernel.java:196-219); the reference adds the rows in binary32 order, the device in
    # binary64 rounded once
    rng = np.random.default_rng(rows)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = rng.integers(0, classes, rows).astype(np.int32)
    g = GraphBuilder()
    lv, tv = g.feed(F32, (rows, classes)), g.feed(I32, (rows,))
    g.publish(g.index_cross_entropy(lv, tv, "none"))
    g.publish(g.index_cross_entropy(lv, tv, "sum"))
    g.publish(g.index_cross_entropy(lv, tv, "mean"))
    each, total, mean = run_image(ctx, g, [logits, labels])
    per_row, ref_mean = oracle.index_cross_entropy(logits, labels)
    lse_scale = np.abs(per_row) + np.abs(logits[np.arange(rows), labels])        # |m + log s| is below this sum
    assert np.all(np.abs(each - per_row) <= 4 * np.spacing(lse_scale.astype(np.float32)))
    sequential = np.float32(0.0)
    for value in per_row:
        sequential = np.float32(sequential + value)
    assert abs(float(total) - float(sequential)) <= 1e-6 * abs(float(sequential))
    assert abs(float(mean) - float(ref_mean)) <= 1e-6 * abs(float(ref_mean))


@pytest.mark.parametrize("rows,classes,label_dtype,ignore", [(300, 1000, I32, -100), (1024, 10, I64, 3), (65, 37, I32, -100)])
def test_cross_entropy_ignore_index_forward_and_gradient(ctx, oracle, rows, classes, label_dtype, ignore):
    # rows labelled with the ignore index give no loss and no gradient and are left out of the mean's
    # count (CpuLossReferenceKernel.java:196-218; gradient node list LossGradientRules.java:172-228,
    # executed node by node with integer SUB / EQ on the labels)
    rng = np.random.default_rng(rows + classes)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = rng.integers(0, classes, rows)
    labels[rng.random(rows) < 0.3] = ignore
    labels[0], labels[1] = ignore, (ignore + 1) % classes
    for reduction in ("mean", "sum", "none"):
        g = GraphBuilder()
        lv, tv = g.feed(F32, (rows, classes)), g.feed(label_dtype, (rows,))
        sv = g.feed(F32, (rows,) if reduction == "none" else ())
        g.publish(g.index_cross_entropy(lv, tv, reduction, ignore_index=ignore))
        g.publish(g.index_cross_entropy_backward(lv, tv, sv, reduction, ignore_index=ignore))
        plan = native.describe(g.build()).strip().split("\n")
        assert len(plan) == 1 and plan[0].startswith("cross_entropy") and "gradient" in plan[0]      # the chain is fused
        seed = rng.standard_normal(rows).astype(np.float32) if reduction == "none" else np.float32(1.0)
        loss, grad = run_image(ctx, g, [logits, labels, seed])
        # the same chain node by node (integer SCALAR_SUB / SUB / EQ on the labels): publishing the row
        # mask keeps it from being fused
        g2 = GraphBuilder()
        lv2, tv2 = g2.feed(F32, (rows, classes)), g2.feed(label_dtype, (rows,))
        sv2 = g2.feed(F32, (rows,) if reduction == "none" else ())
        g2.publish(g2.index_cross_entropy_backward(lv2, tv2, sv2, reduction, ignore_index=ignore))
        mask_node = next(n for n in g2.nodes if n.op == program.OPS["EQ"] and tuple(g2.values[n.outputs[0]].shape) == (rows,))
        g2.publish(g2.values[mask_node.outputs[0]])
        assert len(native.describe(g2.build()).strip().split("\n")) > 10
        grad2, mask = run_image(ctx, g2, [logits, labels, seed])
        assert np.array_equal(mask.astype(bool), labels == ignore)
        per_row, reduced = oracle.index_cross_entropy_ignore(logits, labels, ignore, reduction)
        if reduction == "none":
            active = labels != ignore
            assert np.all(loss[~active] == 0.0) and not np.any(np.signbit(loss[~active]))
            scale = np.abs(per_row) + np.abs(logits[np.arange(rows), np.clip(labels, 0, classes - 1)])
            assert np.all(np.abs(loss - per_row)[active] <= 4 * np.spacing(scale.astype(np.float32))[active])
        else:
            assert abs(float(loss) - float(reduced)) <= 4e-6 * abs(float(reduced))
        expect = oracle.index_cross_entropy_ignore_backward(logits, labels, ignore, seed, reduction)
        scale = np.abs(seed).max() if reduction == "none" else 1.0
        tol = 4 * np.spacing(np.abs(expect)) + np.float32(2.0 ** -24) * scale / (rows if reduction == "mean" else 1)
        assert np.all(np.abs(grad - expect) <= tol) and np.all(np.abs(grad2 - expect) <= tol)
        assert np.all(grad[labels == ignore] == 0.0) and np.all(grad2[labels == ignore] == 0.0)
        assert not np.any(np.signbit(grad[labels == ignore]))


def test_cross_entropy_ignore_index_edge_cases(ctx, oracle):
    # the ignore index is tested before the bounds: an ignored label far outside [0, classes) is fine,
    # another one out of bounds still fails; all rows ignored: MEAN is 0 / 0 = NaN, SUM is 0
    logits = np.zeros((4, 2), dtype=np.float32)
    for reduction, labels, expect in (("mean", [1, -100, 0, -100], np.float32(np.log(2.0))), ("sum", [-100] * 4, np.float32(0.0)),
                                      ("mean", [-100] * 4, np.float32(np.nan))):
        g = GraphBuilder()
        lv, tv = g.feed(F32, (4, 2)), g.feed(I64, (4,))
        g.publish(g.index_cross_entropy(lv, tv, reduction, ignore_index=-100))
        (loss,) = run_image(ctx, g, [logits, np.array(labels)])
        assert np.array_equal(np.float32(loss), expect, equal_nan=True)
        assert np.array_equal(oracle.index_cross_entropy_ignore(logits, labels, -100, reduction)[1], expect, equal_nan=True)
    g = GraphBuilder()
    lv, tv = g.feed(F32, (4, 2)), g.feed(I64, (4,))
    g.publish(g.index_cross_entropy(lv, tv, "mean", ignore_index=-100))
    with pytest.raises(native.NativeFailure) as failure:
        run_image(ctx, g, [logits, np.array([0, -100, 2, 1])])
    assert failure.value.status == 5


@pytest.mark.parametrize("rows,classes", [(300, 1000), (1024, 10), (65, 37)])
def test_dense_cross_entropy_forward_and_gradient(ctx, oracle, rows, classes):
    # dense target weights (CpuLossReferenceKernel.java:129-143); gradient node list
    # LossGradientRules.java:114-145 executed node by node; one row has only zero targets
    rng = np.random.default_rng(rows * classes)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    target = rng.random((rows, classes)).astype(np.float32)
    target[rng.random((rows, classes)) < 0.5] = 0.0
    target /= np.maximum(target.sum(axis=1, keepdims=True), 1e-6)
    target[3] = 0.0
    for reduction in ("mean", "sum", "none"):
        g = GraphBuilder()
        lv, tv = g.feed(F32, (rows, classes)), g.feed(F32, (rows, classes))
        sv = g.feed(F32, (rows,) if reduction == "none" else ())
        g.publish(g.dense_cross_entropy(lv, tv, reduction))
        g.publish(g.dense_cross_entropy_backward(lv, tv, sv, reduction))
        plan = native.describe(g.build()).strip().split("\n")
        assert len(plan) == 2 and plan[1].startswith("dense_cross_entropy_backward")         # the gradient chain is fused
        seed = rng.standard_normal(rows).astype(np.float32) if reduction == "none" else np.float32(1.0)
        loss, grad = run_image(ctx, g, [logits, target, seed])
        # the same chain node by node: publishing the empty-row mask keeps it from being fused
        g2 = GraphBuilder()
        lv2, tv2 = g2.feed(F32, (rows, classes)), g2.feed(F32, (rows, classes))
        sv2 = g2.feed(F32, (rows,) if reduction == "none" else ())
        g2.publish(g2.dense_cross_entropy_backward(lv2, tv2, sv2, reduction))
        mask_node = next(n for n in g2.nodes if n.op == program.OPS["EQ"] and tuple(g2.values[n.outputs[0]].shape) == (rows, 1))
        g2.publish(g2.values[mask_node.outputs[0]])
        assert len(native.describe(g2.build()).strip().split("\n")) > 10
        grad2, empty = run_image(ctx, g2, [logits, target, seed])
        assert np.array_equal(empty[:, 0].astype(bool), ~(target != 0).any(axis=1))
        per_row, reduced = oracle.dense_cross_entropy(logits, target, reduction)
        if reduction == "none":
            # stated tolerance: 4 units in the last place of sum |weight * (lse - x)| (the reference adds
            # the terms in binary32 order, the device in binary64 rounded once), plus the lse's own 4
            lse = np.log(np.exp(logits.astype(np.float64)).sum(axis=1, keepdims=True))
            bound = (np.abs(target * (lse - logits)).sum(axis=1) * (1 + classes * 2.0 ** -24)).astype(np.float32)
            extra = (np.abs(target).sum(axis=1) * np.spacing(np.abs(lse[:, 0]).astype(np.float32)) * 4).astype(np.float32)
            assert np.all(np.abs(loss - per_row) <= classes * np.spacing(bound) / 2 + extra)
            assert loss[3] == 0.0
        else:
            # the reference adds the rows in binary32 order (error up to rows * 2^-24 relative), the device in binary64
            assert abs(float(loss) - float(reduced)) <= 4e-6 * abs(float(reduced))
        expect = oracle.dense_cross_entropy_backward(logits, target, seed, reduction)
        scale = np.abs(seed).max() if reduction == "none" else 1.0
        tol = 4 * np.spacing(np.abs(expect)) + np.float32(2.0 ** -23) * scale / (rows if reduction == "mean" else 1)
        assert np.all(np.abs(grad - expect) <= tol) and np.all(np.abs(grad2 - expect) <= tol)
        assert np.all(grad[3] == 0.0) and np.all(grad2[3] == 0.0) and not np.any(np.signbit(grad[3]))


@pytest.mark.parametrize("cols", [128, 500, 1024])
def test_dense_cross_entropy_wide_rows_with_special_logits(ctx, oracle, cols):
    # rows wide enough for the register-cached kernel; rows whose logits hold +inf, -inf or NaN take the
    # careful routine and must propagate exactly as the reference's loops do (a -inf logit under a zero
    # weight is skipped, under a non-zero weight it gives +inf)
    rng = np.random.default_rng(cols)
    logits = (rng.standard_normal((24, cols)) * 2).astype(np.float32)
    target = rng.random((24, cols)).astype(np.float32)
    target[rng.random((24, cols)) < 0.5] = 0.0
    logits[1, 5] = np.inf
    logits[2, 7] = -np.inf; target[2, 7] = 0.0
    logits[3, 9] = -np.inf; target[3, 9] = 0.25
    logits[4, 11] = np.nan
    g = GraphBuilder()
    lv, tv = g.feed(F32, logits.shape), g.feed(F32, target.shape)
    g.publish(g.dense_cross_entropy(lv, tv, "none"))
    (loss,) = run_image(ctx, g, [logits, target])
    with np.errstate(invalid="ignore", over="ignore"):
        per_row, _ = oracle.dense_cross_entropy(logits, target, "none")
    assert np.array_equal(np.isnan(loss), np.isnan(per_row)) and np.isnan(per_row[1]) and np.isnan(per_row[4])
    assert loss[3] == np.inf and per_row[3] == np.inf and np.isfinite(loss[2])
    finite = np.isfinite(per_row)
    assert np.all(np.abs(loss[finite] - per_row[finite]) <= 2e-6 * np.abs(per_row[finite]))
    # the fused gradient kernel against the node list executed node by node (unfused by publishing the
    # empty-row mask): the same NaN rows, the same values elsewhere within the stated tolerance
    target[6] = 0.0
    grads = []
    for unfuse in (False, True):
        g = GraphBuilder()
        lv, tv, sv = g.feed(F32, logits.shape), g.feed(F32, target.shape), g.feed(F32, ())
        g.publish(g.dense_cross_entropy_backward(lv, tv, sv, "sum"))
        if unfuse:
            mask_node = next(n for n in g.nodes if n.op == program.OPS["EQ"] and tuple(g.values[n.outputs[0]].shape) == (24, 1))
            g.publish(g.values[mask_node.outputs[0]])
        assert (len(native.describe(g.build()).strip().split("\n")) == 1) == (not unfuse)
        grads.append(run_image(ctx, g, [logits, target, np.float32(0.5)])[0])
    fused, listed = grads
    assert np.array_equal(np.isnan(fused), np.isnan(listed)) and np.isnan(fused[1]).all() and np.isnan(fused[4]).all()
    assert np.all(fused[6] == 0.0) and np.all(listed[6] == 0.0)
    ok = ~np.isnan(listed)
    assert np.all(np.abs(fused[ok] - listed[ok]) <= 4 * np.spacing(np.abs(listed[ok])) + np.float32(2.0 ** -23) * 0.5 * np.abs(target).sum(axis=1).max())


def test_dense_cross_entropy_known_answer(ctx, oracle):
    # MetalNormalizationLossNativeTest.java:59-68: logits (0, 0), target (2, 0), MEAN -> 2 ln 2
    g = GraphBuilder()
    lv, tv = g.feed(F32, (1, 2)), g.feed(F32, (1, 2))
    g.publish(g.dense_cross_entropy(lv, tv, "mean"))
    (loss,) = run_image(ctx, g, [np.zeros((1, 2), dtype=np.float32), np.array([[2, 0]], dtype=np.float32)])
    assert np.float32(loss) == np.float32(2.0) * np.float32(np.log(2.0))


@pytest.mark.parametrize("rows,classes", [(300, 1000), (1024, 10)])
def test_cross_entropy_sum_and_none_gradients_are_fused(ctx, oracle, rows, classes):
    # the gradient chain with the cotangent restored for SUM (expand(seed)) and for NONE (one value per
    # row) is recognised like the MEAN form and runs in the same row kernel (LossGradientRules.java:239-252)
    rng = np.random.default_rng(rows + 1)
    logits = (rng.standard_normal((rows, classes)) * 2).astype(np.float32)
    labels = rng.integers(0, classes, rows).astype(np.int32)
    for reduction in ("sum", "none"):
        g = GraphBuilder()
        lv, tv = g.feed(F32, (rows, classes)), g.feed(I32, (rows,))
        sv = g.feed(F32, (rows,) if reduction == "none" else ())
        g.publish(g.index_cross_entropy(lv, tv, reduction))
        g.publish(g.index_cross_entropy_backward(lv, tv, sv, reduction))
        plan = native.describe(g.build()).strip().split("\n")
        assert len(plan) == 1 and plan[0].startswith("cross_entropy") and "gradient" in plan[0]
        seed = rng.standard_normal(rows).astype(np.float32) if reduction == "none" else np.float32(0.75)
        loss, grad = run_image(ctx, g, [logits, labels, seed])
        if reduction == "sum":
            expect = oracle.index_cross_entropy_backward(logits, labels, float(seed), count=1)
        else:
            expect = oracle.index_cross_entropy_ignore_backward(logits, labels, -1, seed, "none")
        scale = np.abs(seed).max()
        assert np.all(np.abs(grad - expect) <= 4 * np.spacing(np.abs(expect)) + np.float32(2.0 ** -24) * scale)
        per_row, _ = oracle.index_cross_entropy(logits, labels)
        if reduction == "none":
            lse_scale = np.abs(per_row) + np.abs(logits[np.arange(rows), labels])
            assert np.all(np.abs(loss - per_row) <= 4 * np.spacing(lse_scale.astype(np.float32)))


def test_cross_entropy_rejects_out_of_range_labels(ctx):
    g = GraphBuilder()
    lv, tv = g.feed(F32, (8, 5)), g.feed(I32, (8,))
    g.publish(g.index_cross_entropy(lv, tv))
    labels = np.zeros(8, dtype=np.int32)
    labels[3] = 5
    with pytest.raises(native.NativeFailure) as failure:
        run_image(ctx, g, [np.zeros((8, 5), dtype=np.float32), labels])
    assert failure.value.status == 5
    labels[3] = -1
    with pytest.raises(native.NativeFailure) as failure:
        run_image(ctx, g, [np.zeros((8, 5), dtype=np.float32), labels])
    assert failure.value.status == 5
    labels[3] = 4                                               # the context stays usable afterwards
    (loss,) = run_image(ctx, g, [np.zeros((8, 5), dtype=np.float32), labels])
    assert abs(float(loss) - math.log(5)) < 1e-6


def test_arg_max_is_bit_exact(ctx, oracle):
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((2049, 1000)) * 2).astype(np.float32)
    x[5, 17] = x[5, 900] = 50.0                                  # tie: first index
    x[6, 3] = np.nan
    x[6, 2] = np.inf
    x[7] = -0.0
    x[7, 500] = 0.0
    x[8] = -np.inf
    x[9, 10] = x[9, 11] = np.nan
    for data in (x, x[:, :10].copy(), x[:77, :33].copy()):
        g = GraphBuilder()
        v = g.feed(F32, data.shape)
        g.publish(g.arg_max(v, 1))
        (idx,) = run_image(ctx, g, [data])
        assert idx.dtype == np.int64 and np.array_equal(idx, oracle.argmax(data))


def test_column_sums_and_relu_backward(ctx, oracle):
    rng = np.random.default_rng(3)
    for m, n in ((1024, 128), (4097, 10), (513, 1000), (65, 1)):
        gmat = rng.standard_normal((m, n)).astype(np.float32)
        g = GraphBuilder()
        v = g.feed(F32, (m, n))
        g.publish(g.sum_to_shape(v, (n,)))
        (s,) = run_image(ctx, g, [gmat])
        assert ulp_distance(s, oracle.colsum_exact(gmat)).max() <= 1
    z = rng.standard_normal((300, 77)).astype(np.float32)
    z[0, :4] = [0.0, -0.0, np.nan, np.inf]
    up = rng.standard_normal((300, 77)).astype(np.float32)
    g = GraphBuilder()
    zv, uv = g.feed(F32, z.shape), g.feed(F32, z.shape)
    g.publish(g.relu_backward(zv, uv))
    (out,) = run_image(ctx, g, [z, up])
    assert np.array_equal(out.view(np.uint32), oracle.relu_backward(z, up).view(np.uint32))


def test_elementwise_nodes_round_once(ctx, oracle):
    rng = np.random.default_rng(4)
    a = rng.standard_normal((33, 17)).astype(np.float32)
    b = rng.standard_normal((17,)).astype(np.float32)
    g = GraphBuilder()
    av, bv = g.feed(F32, a.shape), g.feed(F32, b.shape)
    g.publish(g.add(av, bv)); g.publish(g.sub(av, bv)); g.publish(g.mul(av, bv)); g.publish(g.div(av, bv))
    g.publish(g.relu(av)); g.publish(g.scalar_mul(av, 2.5)); g.publish(g.gt(av, bv)); g.publish(g.exp(av))
    g.publish(g.sum(av, 1, True)); g.publish(g.permute(av, (1, 0))); g.publish(g.expand(bv, a.shape))
    add, sub, mul, div, relu, smul, gt, ex, ssum, perm, expd = run_image(ctx, g, [a, b])
    assert np.array_equal(add, a + b) and np.array_equal(sub, a - b) and np.array_equal(mul, a * b) and np.array_equal(div, a / b)
    assert np.array_equal(relu, oracle.relu(a)) and np.array_equal(smul, a * np.float32(2.5))
    assert np.array_equal(gt.astype(bool), a > b)
    assert ulp_distance(ex, np.exp(a.astype(np.float64)).astype(np.float32)).max() <= 1
    assert np.array_equal(ssum[:, 0], np.array([oracle.exact_sum(r) for r in a], dtype=np.float32))
    assert np.array_equal(perm, a.T) and np.array_equal(expd, np.broadcast_to(b, a.shape))
    labels = rng.integers(-2, 9, 50)
    g = GraphBuilder()
    lv = g.feed(I64, (50,))
    safe = g.scalar_min(g.scalar_max(lv, 0), 6)
    g.publish(safe); g.publish(g.one_hot(safe, 7))
    s, hot = run_image(ctx, g, [labels])
    assert np.array_equal(s, np.clip(labels, 0, 6)) and np.array_equal(hot.astype(bool), np.eye(7, dtype=bool)[np.clip(labels, 0, 6)])


def test_mse_matches_the_checker(ctx, oracle):
    rng = np.random.default_rng(6)
    p = rng.standard_normal((1024, 1)).astype(np.float32)
    t = rng.standard_normal((1024, 1)).astype(np.float32)
    g = GraphBuilder()
    pv, tv, sv = g.feed(F32, p.shape), g.feed(F32, p.shape), g.feed(F32, ())
    g.publish(g.mean_squared_error(pv, tv))
    g.publish(g.mean_squared_error_backward(pv, tv, sv))
    loss, grad = run_image(ctx, g, [p, t, np.float32(1.0)])
    assert np.float32(loss) == oracle.mse(p, t)                  # sequential sum, exact quotient: bit-identical
    assert np.array_equal(grad, oracle.mse_backward(p, t))


@pytest.mark.parametrize("shape", [(2048, 1000), (70001,), (300, 999)])
def test_mse_large_inputs_two_phase_reduction(ctx, oracle, shape):
    # above 65536 elements the squared differences are added in binary64 by many blocks and rounded once,
    # where the reference adds them in ascending binary32 order: the device result lies within a rounding
    # of the exact sum, the reference within its own sequential-sum error (count * 2^-25 relative at worst)
    rng = np.random.default_rng(len(shape) + shape[0])
    p = rng.standard_normal(shape).astype(np.float32)
    t = rng.standard_normal(shape).astype(np.float32)
    g = GraphBuilder()
    pv, tv = g.feed(F32, p.shape), g.feed(F32, p.shape)
    g.publish(g.mean_squared_error(pv, tv, "mean"))
    g.publish(g.mean_squared_error(pv, tv, "sum"))
    mean, total = run_image(ctx, g, [p, t])
    d = (p - t).astype(np.float32)
    exact = (d.astype(np.float64) ** 2).astype(np.float32).astype(np.float64).sum()      # each square rounded to binary32 first
    assert abs(float(total) - exact) <= 2.0 ** -23 * exact
    assert abs(float(mean) - exact / p.size) <= 2.0 ** -22 * exact / p.size
    assert abs(float(total) - float(oracle.squared_error(p, t, "sum"))) <= p.size * 2.0 ** -25 * exact
    assert abs(float(mean) - float(oracle.mse(p, t))) <= p.size * 2.0 ** -25 * exact / p.size


def test_mse_sum_and_none_reductions(ctx, oracle):
    # the other two reductions of the same reference kernel (CpuLossReferenceKernel.java:67-87) and the
    # cotangents the gradient rule restores for them (LossGradientRules.java:77-101): bit for bit
    rng = np.random.default_rng(16)
    p = rng.standard_normal((96, 7)).astype(np.float32)
    t = rng.standard_normal((96, 7)).astype(np.float32)
    up = rng.standard_normal((96, 7)).astype(np.float32)
    g = GraphBuilder()
    pv, tv, sv, uv = g.feed(F32, p.shape), g.feed(F32, p.shape), g.feed(F32, ()), g.feed(F32, p.shape)
    g.publish(g.mean_squared_error(pv, tv, "sum"))
    g.publish(g.mean_squared_error(pv, tv, "none"))
    g.publish(g.mean_squared_error_backward(pv, tv, sv, "sum"))
    g.publish(g.mean_squared_error_backward(pv, tv, uv, "none"))
    total, each, d_sum, d_none = run_image(ctx, g, [p, t, np.float32(0.75), up])
    assert np.float32(total) == oracle.squared_error(p, t, "sum")
    assert np.array_equal(each, oracle.squared_error(p, t, "none"))
    doubled = ((p - t).astype(np.float32) * np.float32(2.0)).astype(np.float32)
    assert np.array_equal(d_sum, (doubled * np.float32(0.75)).astype(np.float32))
    assert np.array_equal(d_none, (doubled * up).astype(np.float32))


def test_prefetch_overlaps_and_stays_ordered(ctx):
    # double-buffered feeding: while run i is enqueued, the operands of run i + 1 are copied on the
    # copy stream into the other buffer; a prefetch into a buffer waits for the run that still reads it,
    # and a run waits for the prefetch of its buffer.  Nothing is synchronised until the end.
    m, k, n = 256, 512, 384
    rng = np.random.default_rng(17)
    g = matmul_graph(m, k, n)
    exe = native.Executable(ctx, g.build())
    b_host = rng.integers(-3, 4, (k, n)).astype(np.float32)
    b_buf = ctx.upload(b_host)
    a_bufs = [ctx.buffer(m * k * 4), ctx.buffer(m * k * 4)]
    steps = 6
    hosts, outs = [], []
    for i in range(steps):
        pinned = native.PinnedArray((m, k), np.float32)
        pinned.array[...] = rng.integers(-3, 4, (m, k)).astype(np.float32)
        hosts.append(pinned)
        outs.append(ctx.buffer(m * n * 4))
    a_bufs[0].prefetch(hosts[0].pointer, hosts[0].nbytes)
    for i in range(steps):
        if i + 1 < steps:
            a_bufs[(i + 1) & 1].prefetch(hosts[i + 1].pointer, hosts[i + 1].nbytes)
        exe.enqueue([a_bufs[i & 1], b_buf], [outs[i]])
    exe.finish()
    for i in range(steps):
        want = (hosts[i].array.astype(np.int64) @ b_host.astype(np.int64)).astype(np.float32)
        assert np.array_equal(outs[i].download(np.float32, (m, n)), want), i
    # a plain upload after a prefetch of the same buffer lands after it
    a_bufs[0].prefetch(hosts[1].pointer, hosts[1].nbytes)
    a_bufs[0].upload(hosts[2].array)
    assert np.array_equal(a_bufs[0].download(np.float32, (m, k)), hosts[2].array)
    ctx.synchronize()
    exe.close()
    for h in hosts:
        h.close()
    for b in a_bufs + outs + [b_buf]:
        b.close()


@pytest.mark.parametrize("kind", ["tanh", "sigmoid", "silu", "gelu_tanh", "gelu", "erf"])
def test_tanh_and_sigmoid_nodes(ctx, oracle, kind):
    # binary64 function and one narrowing on both sides: identical except on the rare rounding tie
    # where the two binary64 libraries differ in the last place (stated bound: 1 ulp)
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(200000) * 4, rng.uniform(-110, 110, 50000),
                        [0.0, -0.0, np.inf, -np.inf, np.nan, 1e-30, -1e-30, 88.0, -88.0, 104.0, -104.0]]).astype(np.float32)
    g = GraphBuilder()
    v = g.feed(F32, x.shape)
    g.publish(getattr(g, kind)(v))
    (got,) = run_image(ctx, g, [x])
    want = getattr(oracle, kind)(x)
    finite = np.isfinite(want)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    if kind == "gelu":
        # 1 + erf(x / sqrt 2) cancels for x < 0 and is a multiple of 2^-53 on every side (the reference
        # forms it as 1 - erfc rounded to binary64): two units of that quantum times |x| / 2 are allowed
        # on top of the last place of the result
        slack = np.spacing(np.abs(want[finite])) + np.abs(x[finite]).astype(np.float64) * 2.0 ** -52
        assert np.all(np.abs(got[finite].astype(np.float64) - want[finite]) <= slack)
        assert (got[finite] == want[finite])[x[finite] > -3].mean() >= 0.9999
    else:
        assert ulp_distance(got[finite], want[finite]).max() <= 1
        assert (got[finite] == want[finite]).mean() >= 0.9999
    assert np.array_equal(np.signbit(got[finite]), np.signbit(want[finite]))


@pytest.mark.parametrize("kind", ["tanh", "sigmoid"])
def test_tanh_and_sigmoid_backward_chains_round_per_node(ctx, oracle, kind):
    rng = np.random.default_rng(4)
    y = (np.tanh(rng.standard_normal((64, 96))) if kind == "tanh" else rng.uniform(0, 1, (64, 96))).astype(np.float32)
    up = rng.standard_normal((64, 96)).astype(np.float32)
    g = GraphBuilder()
    yv, uv = g.feed(F32, y.shape), g.feed(F32, y.shape)
    g.publish(g.tanh_backward(yv, uv) if kind == "tanh" else g.sigmoid_backward(yv, uv))
    (got,) = run_image(ctx, g, [y, up])
    assert np.array_equal(got, oracle.activation_backward(kind, y, up))


@pytest.mark.parametrize("kind", ["silu", "gelu_tanh", "gelu"])
def test_silu_and_gelu_backward_chains_and_is_inf(ctx, oracle, kind):
    # silu: where(isInf(x), where(x > 0, g, 0), (g * s) * (1 + x * (1 - s))), s = SIGMOID(x); the tanh GELU
    # rule is the longer list of ElementwiseGradientRules.java:280-288.  Every node rounds once; the
    # device's sigmoid / tanh may differ from the checker's by 1 ulp on rare ties, so the chains are
    # compared at a few ulp of the result (plus a rounding of the upstream gradient where 1 - t * t
    # cancels) and exactly at the infinities
    rng = np.random.default_rng(6)
    x = np.concatenate([rng.standard_normal(6000) * 3, [np.inf, -np.inf, 0.0, -0.0, 50.0, -50.0]]).astype(np.float32).reshape(-1, 6)
    up = rng.standard_normal(x.shape).astype(np.float32)
    g = GraphBuilder()
    xv, uv = g.feed(F32, x.shape), g.feed(F32, x.shape)
    g.publish({"silu": g.silu_backward, "gelu_tanh": g.gelu_tanh_backward, "gelu": g.gelu_backward}[kind](xv, uv))
    g.publish(g.is_inf(xv))
    got, inf_mask = run_image(ctx, g, [x, up])
    assert np.array_equal(inf_mask.astype(bool), np.isinf(x))
    want = oracle.activation_backward(kind, None, up, x)
    assert np.array_equal(got[np.isinf(x)], want[np.isinf(x)])
    finite = np.isfinite(x)
    tol = 4 * np.spacing(np.abs(want[finite])) + np.float32(2.0 ** -22) * np.abs(up[finite])
    assert np.all(np.abs(got[finite] - want[finite]) <= tol)


def test_clamp_and_its_gradient_chain_are_bit_exact(ctx, oracle):
    # CLAMP = MIN(MAX(x, lo), hi) with Math.max / Math.min semantics (NaN propagates, -0 below +0), and
    # the gradient node list of ElementwiseGradientRules.clamp: inside the range the gradient passes, at
    # a bound half of it, outside nothing.  Only comparisons, selections and one exact halving: bit for bit.
    rng = np.random.default_rng(9)
    x = np.concatenate([rng.standard_normal(4000) * 2, [-1.0, 1.5, 0.0, -0.0, np.nan, np.inf, -np.inf, -1.0000001, 1.4999999]]).astype(np.float32)
    up = rng.standard_normal(x.shape).astype(np.float32)
    g = GraphBuilder()
    xv, uv = g.feed(F32, x.shape), g.feed(F32, x.shape)
    g.publish(g.clamp(xv, -1.0, 1.5))
    g.publish(g.clamp_backward(xv, uv, -1.0, 1.5))
    g.publish(g.clamp(xv, -0.0, 0.0))
    got, grad, zeros = run_image(ctx, g, [x, up])
    want = oracle.clamp(x, -1.0, 1.5)
    assert np.array_equal(got.view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)]) and np.array_equal(np.isnan(got), np.isnan(want))
    want_grad = oracle.clamp_backward(x, up, -1.0, 1.5)
    assert np.array_equal(grad, want_grad)
    assert grad[x == np.float32(-1.0)][0] == up[x == np.float32(-1.0)][0] * np.float32(0.5)
    # bounds [-0, +0]: negative inputs and -0 keep -0, positive inputs and +0 give +0 (Tensor.java:2328-2329)
    finite = ~np.isnan(x)
    assert np.array_equal(np.signbit(zeros[finite]), np.signbit(x[finite]))
    assert not zeros[finite].any()


# ---- buffers and error statuses -----------------------------------------------------------------
def test_buffers_canonical_bytes_and_errors(ctx):
    values = np.array([1.0, -2.5, 3.25e-3, 7e8], dtype=np.float32)
    buf = ctx.upload(values)
    big = buf.download_canonical(16, 4)
    assert big == values.astype(">f4").tobytes()
    buf.upload_canonical(np.array([5.0, 6.0], dtype=">f4").tobytes(), 4, offset=8)
    assert np.array_equal(buf.download(np.float32, (4,)), np.array([1.0, -2.5, 5.0, 6.0], dtype=np.float32))
    with pytest.raises(native.NativeFailure) as failure:
        buf.download(np.float32, (5,))
    assert failure.value.status == 5
    with pytest.raises(native.NativeFailure) as failure:
        buf.upload(values, offset=4)
    assert failure.value.status == 5
    g = matmul_graph(4, 4, 4)
    exe = native.Executable(ctx, g.build())
    a, b, c = ctx.buffer(64), ctx.buffer(64), ctx.buffer(64)
    small = ctx.buffer(8)
    for inputs, outputs, status in (([a], [c], 1), ([a, b], [small], 10), ([a, b], [a], 10), ([a, ctx], [c], 1)):
        with pytest.raises(native.NativeFailure) as failure:
            exe.run(inputs, outputs)
        assert failure.value.status == status
    exe.run([a, b], [c])
    assert exe.launch_count() == 1 and exe.last_timing_ms() >= 0.0
    exe.close()
    with pytest.raises(native.NativeFailure) as failure:
        native.Executable(ctx, b"not an image")
    assert failure.value.status == 9


# ---- optimizers ---------------------------------------------------------------------------------
def test_adam_is_bit_identical_to_the_checker(ctx, oracle):
    rng = np.random.default_rng(8)
    for kind, decoupled, wd in ((native.ADAM, False, 0.0), (native.ADAM, False, 0.01), (native.ADAMW, True, 0.01)):
        sizes = [70001, 513, 1]
        params = [rng.standard_normal(s).astype(np.float32) for s in sizes]
        bufs = [ctx.upload(p) for p in params]
        opt = native.Optimizer(ctx, kind, [1e-3, 0.9, 0.999, 1e-8, wd], bufs, sizes)
        m = [np.zeros(s, dtype=np.float32) for s in sizes]
        v = [np.zeros(s, dtype=np.float32) for s in sizes]
        for step in range(1, 4):
            grads = [(rng.standard_normal(s) * 10.0 ** rng.integers(-6, 2)).astype(np.float32) for s in sizes]
            gb = [ctx.upload(g) for g in grads]
            opt.step(gb)
            for i in range(len(sizes)):
                assert oracle.adam(params[i], grads[i], m[i], v[i], step, weight_decay=wd, decoupled=decoupled)
                assert np.array_equal(bufs[i].download(np.float32, (sizes[i],)).view(np.uint32), params[i].view(np.uint32))
                assert np.array_equal(opt.state(i, 0).view(np.uint32), m[i].view(np.uint32))
                assert np.array_equal(opt.state(i, 1).view(np.uint32), v[i].view(np.uint32))
            for b in gb:
                b.close()
        assert opt.steps() == 3
        opt.close()


@pytest.mark.parametrize("kind", ["adam", "sgd"])
def test_gradient_modes_match_the_checker(ctx, oracle, kind):
    # ACCUMULATE, ACCUMULATE, ACCUMULATE_AND_STEP, then RESET_AND_STEP after a dangling ACCUMULATE:
    # pending sums, parameters, moments and counters after every run, bit for bit
    rng = np.random.default_rng(23)
    shapes = [(37, 19), (19,), (5000,)]
    params = [rng.standard_normal(s).astype(np.float32) for s in shapes]
    bufs = [ctx.upload(p) for p in params]
    hyper = [1e-3, 0.9, 0.999, 1e-8, 0.0] if kind == "adam" else [0.05, 0.9, 0.0, 0.0, 0.0]
    opt = native.Optimizer(ctx, 1 if kind == "adam" else 0, hyper, bufs, [p.size for p in params])
    ref = [p.copy().reshape(-1) for p in params]
    m = [np.zeros(p.size, np.float32) for p in params]
    v = [np.zeros(p.size, np.float32) for p in params]
    acc = [np.zeros(p.size, np.float32) for p in params]
    steps = 0
    script = [native.Optimizer.ACCUMULATE, native.Optimizer.ACCUMULATE, native.Optimizer.ACCUMULATE_AND_STEP,
              native.Optimizer.ACCUMULATE, native.Optimizer.RESET_AND_STEP, native.Optimizer.ACCUMULATE_AND_STEP]
    runs = 0
    for mode in script:
        grads = [(rng.standard_normal(p.size) * 0.1).astype(np.float32) for p in params]
        gbufs = [ctx.upload(g) for g in grads]
        opt.run(mode, gbufs)
        for i, g in enumerate(grads):
            if mode == native.Optimizer.ACCUMULATE:
                assert oracle.accumulate(acc[i], g)
                continue
            used = g
            if mode == native.Optimizer.ACCUMULATE_AND_STEP:
                assert oracle.accumulate(acc[i], g)
                used = acc[i].copy()
            if kind == "adam":
                assert oracle.adam(ref[i], used, m[i], v[i], steps + 1)
            else:
                assert oracle.sgd(ref[i], used, m[i], lr=0.05, momentum=0.9, completed_steps=steps)
            acc[i][...] = 0.0
        if mode == native.Optimizer.ACCUMULATE:
            runs += 1
        else:
            steps += 1
            runs = 0
        assert opt.steps() == steps and opt.accumulated_runs() == runs
        for i, b in enumerate(bufs):
            assert np.array_equal(b.download(np.float32, (params[i].size,)), ref[i]), (mode, i)
            assert np.array_equal(opt.state(i, 0), m[i]) and np.array_equal(opt.state(i, 2), acc[i])
            if kind == "adam":
                assert np.array_equal(opt.state(i, 1), v[i])
        for b in gbufs:
            b.close()
    # snapshot bytes are the big-endian FLOAT32 elements TrainingState stores; restoring them round-trips
    opt.run(native.Optimizer.ACCUMULATE, [ctx.upload(np.full(p.size, 0.25, np.float32)) for p in params])
    blob = opt.state_canonical(2, 2)
    assert blob == np.full(params[2].size, 0.25, ">f4").tobytes()
    opt.zero_grad()
    assert opt.accumulated_runs() == 0 and not opt.state(2, 2).any()
    opt.restore_canonical(2, 2, blob)
    opt.set_progress(steps, 1)
    assert np.array_equal(opt.state(2, 2), np.full(params[2].size, 0.25, np.float32)) and opt.accumulated_runs() == 1
    opt.close()
    for b in bufs:
        b.close()


@pytest.mark.parametrize("decoupled", [False, True])
def test_gradient_mode_journey_of_the_reference(ctx, oracle, decoupled):
    # the protocol of AdamOptimizerTest.bothAlgorithmsFollowIndependentMultiStepOracleAndAllGradientModes
    # (modules/training/src/test/.../AdamOptimizerTest.java:32-66) on a FLOAT32 scalar: objective p * p,
    # Adam / AdamW(0.1, 0.5, 0.25, 0.01, 0.2); counters as asserted there, values against the checker
    hyper = dict(lr=0.1, beta1=0.5, beta2=0.25, eps=0.01, weight_decay=0.2, decoupled=decoupled)
    p_buf = ctx.upload(np.array([2.0], np.float32))
    opt = native.Optimizer(ctx, 2 if decoupled else 1, [0.1, 0.5, 0.25, 0.01, 0.2], [p_buf], [1])
    ref, m, v = np.array([2.0], np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32)

    def run(mode):
        g = ctx.upload(np.float32(2.0) * p_buf.download(np.float32, (1,)))      # d(p * p)/dp at the device's p
        opt.run(mode, [g])
        g.close()

    def check():
        assert np.array_equal(p_buf.download(np.float32, (1,)), ref)
        assert np.array_equal(opt.state(0, 0), m) and np.array_equal(opt.state(0, 1), v)

    run(native.Optimizer.RESET_AND_STEP)
    assert oracle.adam(ref, np.array([4.0], np.float32), m, v, 1, **hyper)
    check()
    current = np.float32(2.0) * ref.copy()
    run(native.Optimizer.ACCUMULATE)
    run(native.Optimizer.ACCUMULATE)
    assert opt.steps() == 1 and opt.accumulated_runs() == 2
    check()
    opt.zero_grad()
    assert opt.accumulated_runs() == 0
    run(native.Optimizer.ACCUMULATE)
    run(native.Optimizer.ACCUMULATE_AND_STEP)
    assert oracle.adam(ref, current + current, m, v, 2, **hyper)
    check()
    assert opt.steps() == 2 and opt.accumulated_runs() == 0
    grad = np.float32(2.0) * ref.copy()
    run(native.Optimizer.RESET_AND_STEP)
    assert oracle.adam(ref, grad, m, v, 3, **hyper)
    check()
    assert opt.steps() == 3
    opt.close()
    p_buf.close()


def test_adam_scales_before_dividing_and_reports_non_finite(ctx):
    gradient, rate = np.float32(1e19), 1e-30
    p = ctx.upload(np.array([1.0], dtype=np.float32))
    opt = native.Optimizer(ctx, native.ADAM, [rate, 0.5, 0.0, rate, 0.0], [p], [1])
    opt.step([ctx.upload(np.array([gradient], dtype=np.float32))])
    assert p.download(np.float32, (1,))[0] == np.float32(1.0)
    opt.step([ctx.upload(np.array([0.0], dtype=np.float32))])
    second = np.float32(0.5) * (np.float32(0.5) * gradient)
    update = (np.float32(rate) * (second / np.float32(0.75))) / np.float32(rate)
    assert p.download(np.float32, (1,))[0] == np.float32(1.0) - update
    with pytest.raises(native.NativeFailure) as failure:          # g*g overflows: the reference refuses the step
        opt.step([ctx.upload(np.array([1e30], dtype=np.float32))])
    assert failure.value.status == 11
    opt.close()


def test_sgd_variants_match_the_checker(ctx, oracle):
    rng = np.random.default_rng(9)
    for momentum, dampening, wd, nesterov in ((0.0, 0.0, 0.0, False), (0.9, 0.0, 0.0, False), (0.9, 0.1, 0.01, False), (0.8, 0.0, 0.0, True)):
        p = rng.standard_normal(5001).astype(np.float32)
        buf = ctx.upload(p)
        opt = native.Optimizer(ctx, native.SGD, [0.01, momentum, dampening, wd, 1.0 if nesterov else 0.0], [buf], [p.size])
        mom = np.zeros_like(p) if momentum else None
        for step in range(3):
            g = rng.standard_normal(p.size).astype(np.float32)
            opt.step([ctx.upload(g)])
            assert oracle.sgd(p, g, mom, 0.01, momentum, dampening, wd, nesterov, completed_steps=step)
            assert np.array_equal(buf.download(np.float32, p.shape).view(np.uint32), p.view(np.uint32))
        opt.close()


# ---- streaming kernels for products with a narrow extent -----------------------------------------
def test_narrow_head_kernels(ctx, oracle):
    rows, wide, classes = 8192, 512, 10                      # large enough for the automatic choice to pick them
    rng = np.random.default_rng(12)
    act = rng.uniform(0, 1, (rows, wide)).astype(np.float32)
    w = (rng.standard_normal((classes, wide)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(classes).astype(np.float32)
    dz = (rng.standard_normal((rows, classes)) * 1e-3).astype(np.float32)
    gate = rng.standard_normal((rows, wide)).astype(np.float32)
    g = GraphBuilder()
    av, wv, bv, dv, gv = g.feed(F32, act.shape), g.feed(F32, w.shape), g.feed(F32, bias.shape), g.feed(F32, dz.shape), g.feed(F32, gate.shape)
    wt, logits = g.linear(av, wv, bv)
    g.publish(logits)                                         # narrow result
    dx, dw, _ = g.linear_backward(av, wt, dv, need_dx=True, bias=False)
    g.publish(g.relu_backward(gv, dx))                        # narrow contraction with the gate folded in
    g.publish(dw)                                             # narrow weight gradient
    plan = native.describe(g.build())
    assert "narrow_out" in plan and "narrow_inner" in plan and "narrow_reduce" in plan
    out, dxg, dwg = run_image(ctx, g, [act, w, bias, dz, gate])
    ref = act.astype(np.float64) @ w.T.astype(np.float64) + bias
    bound = (wide + 2) * 2.0 ** -24 * (np.abs(act).astype(np.float64) @ np.abs(w.T).astype(np.float64) + np.abs(bias))
    assert np.all(np.abs(out - ref) <= bound)
    assert np.abs(out - ref).max() <= 64 * 2.0 ** -24 * np.abs(ref).max()
    sample = rng.choice(rows, 64, replace=False)
    expect = oracle.relu_backward(gate[sample], oracle.matmul_rows(dz, w, sample))
    assert np.array_equal(dxg[sample].view(np.uint32), expect.view(np.uint32))      # the reference's exact chain
    ref_dw = dz.T.astype(np.float64) @ act.astype(np.float64)
    assert np.abs(dwg - ref_dw).max() <= 2e-6 * np.abs(ref_dw).max()
    # integer operands: all three are exact
    acti = rng.integers(-3, 4, act.shape).astype(np.float32)
    wi = rng.integers(-3, 4, w.shape).astype(np.float32)
    dzi = rng.integers(-2, 3, dz.shape).astype(np.float32)
    out, dxg, dwg = run_image(ctx, g, [acti, wi, bias * 0, dzi, gate])
    assert np.array_equal(out, (acti.astype(np.int64) @ wi.T.astype(np.int64)).astype(np.float32))
    assert np.array_equal(dxg, (dzi.astype(np.int64) @ wi.astype(np.int64)).astype(np.float32) * (gate > 0))
    assert np.array_equal(dwg, (dzi.T.astype(np.int64) @ acti.astype(np.int64)).astype(np.float32))


# ---- the reference-held vectors of the gradient rules, on the device ------------------------------
class DeviceBackend:
    """The device behind the interface of golden_cases: every call is one program through the C ABI."""

    def __init__(self, ctx):
        self.ctx = ctx

    def softmax(self, x, log):
        g = GraphBuilder()
        v = g.feed(F32, x.shape)
        g.publish(g.log_softmax(v, 1) if log else g.softmax(v, 1))
        return run_image(self.ctx, g, [x])[0]

    def softmax_backward(self, y, upstream, log):
        g = GraphBuilder()
        yv, gv = g.feed(F32, y.shape), g.feed(F32, y.shape)
        g.publish(g.log_softmax_backward(yv, gv, 1) if log else g.softmax_backward(yv, gv, 1))
        return run_image(self.ctx, g, [y, upstream])[0]

    def softmax_with_backward(self, x, upstream, log):
        g = GraphBuilder()
        xv, gv = g.feed(F32, x.shape), g.feed(F32, x.shape)
        y = g.log_softmax(xv, 1) if log else g.softmax(xv, 1)
        g.publish(y)
        g.publish(g.log_softmax_backward(y, gv, 1) if log else g.softmax_backward(y, gv, 1))
        saved, dx = run_image(self.ctx, g, [x, upstream])
        return saved, dx

    @staticmethod
    def _label_type(dtype):
        return I32 if np.dtype(dtype) == np.int32 else I64

    def index_ce(self, logits, labels, reduction, ignore, label_dtype):
        g = GraphBuilder()
        lv, tv = g.feed(F32, logits.shape), g.feed(self._label_type(label_dtype), (logits.shape[0],))
        g.publish(g.index_cross_entropy(lv, tv, reduction, ignore))
        return run_image(self.ctx, g, [logits, np.asarray(labels, dtype=label_dtype)])[0]

    def index_ce_backward(self, logits, labels, seed, reduction, ignore, label_dtype):
        g = GraphBuilder()
        rows = logits.shape[0]
        lv, tv = g.feed(F32, logits.shape), g.feed(self._label_type(label_dtype), (rows,))
        sv = g.feed(F32, (rows,) if reduction == "none" else ())
        g.publish(g.index_cross_entropy_backward(lv, tv, sv, reduction, ignore))
        return run_image(self.ctx, g, [logits, np.asarray(labels, dtype=label_dtype), np.asarray(seed, dtype=np.float32)])[0]

    def dense_ce(self, logits, target, reduction):
        g = GraphBuilder()
        lv, tv = g.feed(F32, logits.shape), g.feed(F32, logits.shape)
        g.publish(g.dense_cross_entropy(lv, tv, reduction))
        return run_image(self.ctx, g, [logits, target])[0]

    def dense_ce_backward(self, logits, target, seed, reduction):
        g = GraphBuilder()
        rows = logits.shape[0]
        lv, tv = g.feed(F32, logits.shape), g.feed(F32, logits.shape)
        sv = g.feed(F32, (rows,) if reduction == "none" else ())
        g.publish(g.dense_cross_entropy_backward(lv, tv, sv, reduction))
        return run_image(self.ctx, g, [logits, target, np.asarray(seed, dtype=np.float32)])[0]

    def unary(self, name, x):
        g = GraphBuilder()
        v = g.feed(F32, x.shape)
        g.publish(g.erf(v) if name == "erf" else g.gelu(v))
        return run_image(self.ctx, g, [x])[0]


@pytest.mark.parametrize("check", golden_cases.ALL_CHECKS, ids=lambda f: f.__name__)
def test_reference_held_gradient_rule_vectors_on_the_device(ctx, check):
    # the same expectations the CPU checker is held to (tests/golden_cases.py): raw-bit equality wherever
    # the reference's own tests ask for it
    check(DeviceBackend(ctx))


# ---- activations other than ReLU in the GEMM epilogue ---------------------------------------------
@pytest.mark.parametrize("engine,m,k,n", [(2, 512, 256, 384), (2, 128, 96, 64), (2, 100, 70, 130), (1, 70, 33, 45)])
@pytest.mark.parametrize("activation", ["tanh", "sigmoid", "silu", "gelu_tanh", "gelu"])
def test_activation_epilogues_give_the_bits_of_the_separate_pass(ctx, oracle, activation, engine, m, k, n):
    # Y = act(X W^T + b) with the activation fused into the product (two-SM, one-SM and exact kernels):
    # (a) with the pre-activation published beside it, the activation is bit for bit what the element-wise
    # kernel makes of that pre-activation, and within the activation's own bound of the checker's value;
    # (b) without the pre-activation the product writes the same activation.
    rng = np.random.default_rng(m + k)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = rng.uniform(-0.3, 0.3, (n, k)).astype(np.float32)
    b = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    x[0, :4] = [np.inf, 1.0, 1.0, 1.0]                         # a row of non-finite pre-activations on the exact engine
    both = GraphBuilder()
    xv, wv, bv = both.feed(F32, (m, k)), both.feed(F32, (n, k)), both.feed(F32, (n,))
    _, z = both.linear(xv, wv, bv)
    both.publish(z)
    both.publish(both.activation(activation, z))
    assert f"act={ {'tanh': 'TANH', 'sigmoid': 'SIGMOID', 'silu': 'SILU', 'gelu_tanh': 'GELU_TANH_APPROXIMATION', 'gelu': 'GELU'}[activation]}" in native.describe(both.build())
    z_dev, y_dev = run_image(ctx, both, [x, w, b], engine=engine)
    alone = GraphBuilder()
    zv = alone.feed(F32, (m, n))
    alone.publish(alone.activation(activation, zv))
    (y_pass,) = run_image(ctx, alone, [z_dev])
    assert np.array_equal(y_dev.view(np.uint32), y_pass.view(np.uint32))
    want = {"tanh": oracle.tanh, "sigmoid": oracle.sigmoid, "silu": oracle.silu, "gelu_tanh": oracle.gelu_tanh, "gelu": oracle.gelu}[activation](z_dev)
    finite = np.isfinite(want)
    assert np.array_equal(np.isnan(y_dev), np.isnan(want))
    assert ulp_distance(y_dev[finite], want[finite]).max() <= 1 or np.abs(y_dev[finite] - want[finite]).max() <= 2 ** -52 * np.abs(z_dev[finite]).max() + 1e-45
    only = GraphBuilder()
    xv, wv, bv = only.feed(F32, (m, k)), only.feed(F32, (n, k)), only.feed(F32, (n,))
    _, z = only.linear(xv, wv, bv)
    only.publish(only.activation(activation, z))
    (y_only,) = run_image(ctx, only, [x, w, b], engine=engine)
    assert np.array_equal(y_only.view(np.uint32), y_dev.view(np.uint32))


@pytest.mark.parametrize("activation", ["tanh", "gelu"])
def test_tanh_and_gelu_networks_on_the_tensor_cores_follow_the_checker(ctx, oracle, activation):
    from synaptik_b200 import nn
    dims, batch = [256, 512, 384, 10], 512
    rng = np.random.default_rng(5)
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    labels = rng.integers(0, 10, batch)
    ctx.set_option("gemm_engine", 2)
    try:
        model = nn.Model(dims, ctx, seed=21, activation=activation)
        model.configure_training("ce", nn.Adam(1e-3))
        params = model.parameters()
        logits = model.compute(x)
        want = oracle.mlp_forward(x, params[0::2], params[1::2], activation)[-1]
        assert np.abs(logits - want).max() <= 2e-5 * np.abs(want).max()
        loss, grads = model.gradients(x, labels)
        ref_loss, ref_grads, _ = oracle.mlp_gradients(x, labels, params[0::2], params[1::2], "ce", activation=activation)
        assert abs(loss - float(ref_loss)) <= 1e-5 * abs(float(ref_loss))
        for got, ref in zip(grads, ref_grads):          # smooth activations: no gates to flip, so element-wise
            assert np.abs(got - ref).max() <= 5e-5 * np.abs(ref).max() + 1e-12
        model.close()
    finally:
        ctx.set_option("gemm_engine", 0)
