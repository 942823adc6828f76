"""16-bit storage (BFLOAT16 / FLOAT16) on a B200, through the C ABI: values travel as raw 16-bit patterns,
every node computes in FLOAT32 and narrows its result once (CpuScalarReferenceKernel.java:93-115,
CpuMatmulReferenceKernel.java:71-93).  The exact engine and the element-wise kernels are bit for bit the
checker; the tensor-core product (tcgen05 kind::f16, FP32 accumulation) adds its sums in another order, so
its narrowed results may land on the neighbouring 16-bit value where the FLOAT32 sums straddle a rounding
boundary."""
import numpy as np
import pytest

import golden_cases
from helpers import run_image
from synaptik_b200 import native, nn, program
from synaptik_b200.program import BF16, F16, I64, GraphBuilder

pytestmark = pytest.mark.gpu
DTYPES = {"bf16": BF16, "f16": F16}
OP_NAMES = {"tanh": "TANH", "sigmoid": "SIGMOID", "silu": "SILU", "gelu_tanh": "GELU_TANH_APPROXIMATION", "gelu": "GELU"}


@pytest.fixture(scope="module")
def ctx():
    c = native.Context(0)
    yield c
    c.close()


def run_bits(ctx, builder, feeds, engine=None):
    """helpers.run_image for programs whose values may be 16-bit: feeds and results as uint16 bit patterns."""
    return run_image(ctx, builder, feeds, engine=engine)


def linear_graph(kind, m, k, n, activation, keep_preactivation=False, bias=True):
    g = GraphBuilder()
    dt = DTYPES[kind]
    x, w = g.feed(dt, (m, k)), g.feed(dt, (n, k))
    b = g.feed(dt, (n,)) if bias else None
    _, z = g.linear(x, w, b)
    if keep_preactivation:
        g.publish(z)
    g.publish(g.activation(activation, z) if activation else z)
    return g


class DeviceLowBackend:
    def __init__(self, ctx):
        self.ctx = ctx

    def low_matmul(self, kind, a_bits, b_bits):
        g = GraphBuilder()
        dt = DTYPES[kind]
        # a transposed array is fed in its stored order and read through a PERMUTE view, as the reference's
        # private transposes are
        def operand(bits):
            if bits.flags["C_CONTIGUOUS"]:
                return g.feed(dt, bits.shape), np.ascontiguousarray(bits)
            stored = np.ascontiguousarray(bits.T)
            return g.permute(g.feed(dt, stored.shape), (1, 0)), stored
        av, a_feed = operand(a_bits)
        bv, b_feed = operand(b_bits)
        g.publish(g.matmul(av, bv))
        return run_bits(self.ctx, g, [a_feed, b_feed])[0]

    def low_unary(self, kind, name, bits):
        g = GraphBuilder()
        v = g.feed(DTYPES[kind], bits.shape)
        g.publish(g.activation(name, v))
        return run_bits(self.ctx, g, [bits])[0]


@pytest.mark.parametrize("check", golden_cases.LOW_CHECKS, ids=lambda f: f.__name__)
def test_reference_held_low_precision_vectors_on_the_device(ctx, check):
    check(DeviceLowBackend(ctx))


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("activation", [None, "relu", "tanh", "sigmoid", "silu", "gelu_tanh", "gelu"])
def test_exact_engine_linear_is_the_checker_bit_for_bit(ctx, oracle, kind, activation):
    rng = np.random.default_rng(7)
    for m, k, n in ((70, 33, 45), (128, 64, 96), (5, 1, 130)):
        x = oracle.low_encode(kind, rng.uniform(-1, 1, (m, k)).astype(np.float32))
        w = oracle.low_encode(kind, rng.uniform(-0.4, 0.4, (n, k)).astype(np.float32))
        b = oracle.low_encode(kind, rng.uniform(-0.5, 0.5, n).astype(np.float32))
        if m > 5:
            x[0, :3] = oracle.low_encode(kind, np.array([np.inf, -np.inf, np.nan], dtype=np.float32))
        z_ref, y_ref = oracle.low_linear(kind, x, w, b, activation)
        if activation:
            z_dev, y_dev = run_bits(ctx, linear_graph(kind, m, k, n, activation, keep_preactivation=True), [x, w, b], engine=1)
            assert np.array_equal(z_dev, z_ref), (m, k, n)
            assert np.array_equal(y_dev, y_ref), (m, k, n, activation)
        (y_only,) = run_bits(ctx, linear_graph(kind, m, k, n, activation), [x, w, b], engine=1)
        assert np.array_equal(y_only, y_ref)


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_element_wise_nodes_on_16_bit_storage(ctx, oracle, kind):
    rng = np.random.default_rng(3)
    a = oracle.low_encode(kind, (rng.standard_normal((37, 129)) * 4).astype(np.float32))
    b = oracle.low_encode(kind, (rng.standard_normal(129) * 2).astype(np.float32))
    fa, fb = oracle.low_decode(kind, a), oracle.low_decode(kind, b)[None, :]
    for name, fn in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("div", np.divide)):
        g = GraphBuilder()
        av, bv = g.feed(DTYPES[kind], a.shape), g.feed(DTYPES[kind], b.shape)
        g.publish(getattr(g, name)(av, bv))
        (got,) = run_bits(ctx, g, [a, b])
        with np.errstate(all="ignore"):
            assert np.array_equal(got, oracle.low_encode(kind, fn(fa, fb).astype(np.float32))), name
    for name in ("relu", "tanh", "sigmoid", "silu", "gelu_tanh", "gelu"):
        g = GraphBuilder()
        g.publish(g.activation(name, g.feed(DTYPES[kind], a.shape)))
        (got,) = run_bits(ctx, g, [a])
        want = oracle.low_encode(kind, oracle.low_activation(name, fa))
        # the binary64 elementary functions of device and host differ in rare last-place ties of the narrowing
        differing = got != want
        assert differing.mean() <= 2e-3, (name, differing.mean())
        assert np.all(np.abs(got[differing].astype(np.int32) - want[differing].astype(np.int32)) <= 1), name
    # a PERMUTE view made dense, and the row arg-max of 16-bit logits (first index among ties, NaN above +inf)
    g = GraphBuilder()
    g.publish(g.contiguous(g.permute(g.feed(DTYPES[kind], a.shape), (1, 0))))
    (got,) = run_bits(ctx, g, [a])
    assert np.array_equal(got, a.T)
    logits = oracle.low_encode(kind, rng.integers(-3, 4, (64, 10)).astype(np.float32))
    logits[5, 7] = oracle.low_encode(kind, np.array([np.nan], dtype=np.float32))[0]
    g = GraphBuilder()
    g.publish(g.arg_max(g.feed(DTYPES[kind], logits.shape), 1))
    (idx,) = run_bits(ctx, g, [logits])
    assert np.array_equal(idx, oracle.argmax(oracle.low_decode(kind, logits)))


def storage_ulps(kind, got_bits, want_bits):
    """Distance in units in the last place of the storage type (sign-magnitude aware)."""
    def ordered(bits):
        v = bits.astype(np.int32)
        return np.where(v & 0x8000, -(v & 0x7FFF), v)
    return np.abs(ordered(got_bits) - ordered(want_bits))


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("m,k,n", [(512, 256, 384), (300, 136, 200), (128, 4096, 64), (1024, 784, 10),
                                   (2600, 520, 1800)])     # the last: 88 tiles of 256 x 256, ragged on every side (two-SM kernel)
def test_tensor_core_product_on_16_bit_storage(ctx, oracle, kind, m, k, n):
    rng = np.random.default_rng(m + n)
    assert "tcgen05_f16" in native.describe(linear_graph(kind, m, k, n, "relu").build()) or m * n * k < 16 * 1024 * 1024
    # integer-valued operands: every product and sum is exact, so the result is exact whatever the order
    xi = oracle.low_encode(kind, rng.integers(-3, 4, (m, k)).astype(np.float32))
    wi = oracle.low_encode(kind, rng.integers(-2, 3, (n, k)).astype(np.float32))
    (got,) = run_bits(ctx, linear_graph(kind, m, k, n, None, bias=False), [xi, wi], engine=2)
    exact = oracle.low_decode(kind, xi).astype(np.float64) @ oracle.low_decode(kind, wi).astype(np.float64).T
    assert np.array_equal(got, oracle.low_encode(kind, exact.astype(np.float32)))
    # real-valued operands with bias and activation against the checker's sequential chain: the FP32 sums
    # differ by rounding, so a narrowed value may be the neighbouring 16-bit value
    x = oracle.low_encode(kind, rng.uniform(-1, 1, (m, k)).astype(np.float32))
    w = oracle.low_encode(kind, (rng.uniform(-1, 1, (n, k)) / np.sqrt(k)).astype(np.float32))
    b = oracle.low_encode(kind, rng.uniform(-0.5, 0.5, n).astype(np.float32))
    for activation in ("relu", "gelu"):
        z_dev, y_dev = run_bits(ctx, linear_graph(kind, m, k, n, activation, keep_preactivation=True), [x, w, b], engine=2)
        z_ref, y_ref = oracle.low_linear(kind, x, w, b, activation)
        # two FLOAT32 sums that differ by e narrow to values that differ by at most e plus one unit of the storage
        # type; e is the tensor-core bound of the FP32 products (one accumulator over up to 4096 steps truncates
        # by 0.2 * K units of 2^-24 of the sum of |a b|)
        fx, fw = oracle.low_decode(kind, x).astype(np.float64), oracle.low_decode(kind, w).astype(np.float64)
        e = (8.0 + 0.25 * k) * 2.0 ** -24 * (np.abs(fx) @ np.abs(fw).T)
        unit = 2.0 ** (-8 if kind == "bf16" else -11)
        dec = lambda bits: oracle.low_decode(kind, bits).astype(np.float64)
        # z = narrow(narrow(sum) + bias): a neighbouring value of the sum (neighbours are up to 2 * unit * |sum| apart,
        # |sum| <= |z| + |bias|) moves z by that much plus z's own narrowing
        z_slack = e + unit * (4 * np.maximum(np.abs(dec(z_dev)), np.abs(dec(z_ref))) + 2 * np.abs(dec(b))[None, :]) + 1e-30
        gap = np.abs(dec(z_dev) - dec(z_ref))
        worst = np.unravel_index(np.argmax(gap - z_slack), gap.shape)
        assert np.all(gap <= z_slack), (activation, worst, dec(z_dev)[worst], dec(z_ref)[worst], z_slack[worst], e[worst], dec(b)[worst[1]])
        # the activations' slopes are at most 1.13, and the activation's own narrowing adds one more unit
        assert np.all(np.abs(dec(y_dev) - dec(y_ref)) <= 1.2 * z_slack + unit * np.maximum(np.abs(dec(y_dev)), np.abs(dec(y_ref)))), activation
        assert (z_dev != z_ref).mean() <= 0.02 and (y_dev != y_ref).mean() <= 0.02, (activation, (z_dev != z_ref).mean())
        # without the second tensor the kernels write through shared memory and TMA stores: the same bits
        (y_only,) = run_bits(ctx, linear_graph(kind, m, k, n, activation), [x, w, b], engine=2)
        assert np.array_equal(y_only, y_dev), activation
        # the activation is applied to the device's own narrowed pre-activation exactly as the separate node would
        want_y = oracle.low_encode(kind, oracle.low_activation(activation, oracle.low_decode(kind, z_dev)))
        differing = y_dev != want_y
        assert differing.mean() <= 2e-3 and np.all(storage_ulps(kind, y_dev[differing], want_y[differing]) <= 1)


@pytest.mark.parametrize("kind", ["bf16", "f16"])
@pytest.mark.parametrize("m,k,n", [(300, 136, 200), (2600, 72, 1800)])
def test_tensor_core_product_carries_special_values(ctx, oracle, kind, m, k, n):
    """NaN, infinities, signed zeros and values that overflow the storage type take the same bits through the
    packed write-out (one tensor) as through the element-wise one (two tensors), and the checker's patterns."""
    rng = np.random.default_rng(k)
    x = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    w = (rng.uniform(-1, 1, (n, k)) / np.sqrt(k)).astype(np.float32)
    x[0, 3] = np.nan; x[1, 5] = np.inf; x[2, 7] = -np.inf; x[3, :] = 0.0; x[4, :] = -0.0
    if kind == "f16":
        x[5, :] = 6.0e4         # FLOAT32 sums far inside their range that narrow to infinity (BFLOAT16 has FLOAT32's range)
    w[7, :] = np.abs(w[7, :]); w[8, :] = -np.abs(w[8, :]); w[9, :] = 0.0
    b = rng.uniform(-0.5, 0.5, n).astype(np.float32); b[9] = -0.0; b[10] = np.nan
    xb, wb, bb = (oracle.low_encode(kind, a) for a in (x, w, b))
    for activation in (None, "relu", "tanh"):
        z_two, y_two = run_bits(ctx, linear_graph(kind, m, k, n, activation or "relu", keep_preactivation=True), [xb, wb, bb], engine=2)
        (y_one,) = run_bits(ctx, linear_graph(kind, m, k, n, activation), [xb, wb, bb], engine=2)
        assert np.array_equal(y_one, y_two if activation else z_two), activation
        _, y_ref = oracle.low_linear(kind, xb, wb, bb, activation)
        special = ~np.isfinite(oracle.low_decode(kind, y_ref))
        assert special[0].all() and special[:, 10].all()
        assert np.array_equal(y_one[special], y_ref[special]), activation
        if activation == "relu":        # Math.max(x, +0): -0 and negatives give +0
            assert np.all(y_one[oracle.low_decode(kind, z_two) <= 0] == 0)


@pytest.mark.parametrize("kind", ["bf16", "f16"])
def test_model_compute_on_16_bit_storage(ctx, oracle, kind):
    dims, batch = [784, 512, 256, 10], 300
    rng = np.random.default_rng(9)
    x = rng.uniform(0, 1, (batch, dims[0])).astype(np.float32)
    ctx.set_option("gemm_engine", 1)
    try:
        model = nn.Model(dims, ctx, seed=4, dtype=kind)
        params = model.parameters()
        biases = [rng.uniform(-0.1, 0.1, p.shape).astype(np.float32) for p in params[1::2]]
        model.load_parameters([a for pair in zip(params[0::2], biases) for a in pair])
        params = model.parameters()
        logits, idx = model.compute(x, arg_max=True)
    finally:
        ctx.set_option("gemm_engine", 0)
    enc = lambda a: oracle.low_encode(kind, a)
    want = oracle.low_mlp_forward(kind, enc(x), [enc(w) for w in params[0::2]], [enc(b) for b in params[1::2]])
    assert np.array_equal(enc(logits), want)                     # exact engine: bit for bit
    assert np.array_equal(idx, oracle.argmax(logits))
    # default engines (tensor cores for the wide layers): within one unit of the storage type per layer
    fast = nn.Model(dims, ctx, seed=4, dtype=kind)
    fast.load_parameters(params)
    logits_fast, idx_fast = fast.compute(x, arg_max=True)
    scale = np.abs(logits).max()
    assert np.abs(logits_fast - logits).max() <= (2.0 ** -6 if kind == "bf16" else 2.0 ** -9) * scale
    assert np.array_equal(idx_fast, oracle.argmax(logits_fast))
    with pytest.raises(ValueError):
        fast.configure_training("ce", nn.Adam())
    model.close(); fast.close()
