"""ctypes front-end of the CPU checker (``libsynaptik_oracle.so``).

Test infrastructure only: the test-suite, the smoke check and the benchmark's CPU-baseline leg
import this module; the product package never does.  Each function forwards to the C
restatement in ``synaptik_oracle.c`` (where the reference file:line each follows is cited) and
returns fresh numpy arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsynaptik_oracle.so")
_lib = None

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)


def build(force: bool = False) -> str:
    """Compile the checker with the Makefile beside it (gcc only) and return the library path."""
    sources = [os.path.join(_HERE, n) for n in ("synaptik_oracle.c", "cpu_baseline.c", "Makefile")]
    stale = force or not os.path.exists(_LIB_PATH) or any(
        os.path.getmtime(s) > os.path.getmtime(_LIB_PATH) for s in sources)
    if stale:
        subprocess.run(["make", "-s", "-C", _HERE, "-B", "libsynaptik_oracle.so"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.syn_oracle_exact_sum_f32.restype = ctypes.c_float
        _lib.syn_oracle_mse_f32.restype = ctypes.c_float
        _lib.syn_baseline_mlp_step.restype = ctypes.c_double
        _lib.syn_baseline_blas_name.restype = ctypes.c_char_p
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray, t=_f32p):
    return a.ctypes.data_as(t)


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Sequential-K FP32 product of two rank-2 arrays; arbitrary strides (views) are honoured."""
    assert a.dtype == np.float32 and b.dtype == np.float32 and a.ndim == 2 and b.ndim == 2
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = np.empty((m, n), dtype=np.float32)
    lib().syn_oracle_matmul_f32(
        ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k),
        _p(a), ctypes.c_int64(a.strides[0] // 4), ctypes.c_int64(a.strides[1] // 4),
        _p(b), ctypes.c_int64(b.strides[0] // 4), ctypes.c_int64(b.strides[1] // 4),
        _p(c), ctypes.c_int64(n), ctypes.c_int64(1))
    return c


def matmul_rows(a: np.ndarray, b: np.ndarray, rows) -> np.ndarray:
    """``matmul(a, b)[rows]`` without computing the other rows."""
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    m, k = a.shape
    _, n = b.shape
    c = np.empty((len(rows), n), dtype=np.float32)
    lib().syn_oracle_matmul_rows_f32(
        ctypes.c_int64(len(rows)), _p(rows, _i64p), ctypes.c_int64(n), ctypes.c_int64(k),
        _p(a), ctypes.c_int64(a.strides[0] // 4), ctypes.c_int64(a.strides[1] // 4),
        _p(b), ctypes.c_int64(b.strides[0] // 4), ctypes.c_int64(b.strides[1] // 4), _p(c))
    return c


def relu(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_relu_f32(ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def tanh(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(0, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def sigmoid(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(1, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def silu(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(2, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def clamp(x, lo: float, hi: float) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_clamp_f32(ctypes.c_int64(x.size), _p(x), ctypes.c_float(lo), ctypes.c_float(hi), _p(y))
    return y


def clamp_backward(x, upstream, lo: float, hi: float) -> np.ndarray:
    """ElementwiseGradientRules.clamp (:263-270): lowered = max(x, lo); upper = where(lowered < hi, g,
    where(lowered == hi, g * 0.5, 0)); where(x > lo, upper, where(x == lo, upper * 0.5, 0))."""
    x, g = _f32(x), _f32(upstream)
    lo32, hi32, half, zero = np.float32(lo), np.float32(hi), np.float32(0.5), np.float32(0.0)
    lowered = clamp(x, lo, np.inf)
    upper = np.where(lowered < hi32, g, np.where(lowered == hi32, g * half, zero)).astype(np.float32)
    return np.where(x > lo32, upper, np.where(x == lo32, upper * half, zero)).astype(np.float32)


def gelu_tanh(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(3, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def gelu(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(4, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def erf(x) -> np.ndarray:
    x = _f32(x)
    y = np.empty_like(x)
    lib().syn_oracle_activation_f32(5, ctypes.c_int64(x.size), _p(x), _p(y))
    return y


def _coefficient(bits: int) -> np.float32:
    return np.array([bits], dtype=np.uint32).view(np.float32)[0]


def activation_backward(kind: str, output, upstream, pre_activation=None) -> np.ndarray:
    """The reference's gradient node lists, one binary32 rounding per node
    (ElementwiseGradientRules.java:205-206,210,290-301): relu where(y > 0, g, 0); tanh g * (1 - y * y);
    sigmoid (g * y) * (1 - y); silu where(isInf(x), where(x > 0, g, 0), (g * s) * (1 + x * (1 - s)))
    with s = sigmoid(x) of the pre-activation x."""
    y, g = _f32(output), _f32(upstream)
    if kind == "relu":
        return relu_backward(y, g)
    one = np.float32(1.0)
    if kind == "gelu_tanh":
        # ElementwiseGradientRules.geluTanhApproximation (:280-288), FLOAT32 coefficients (:370-378)
        x = _f32(pre_activation)
        half, s2pi = _coefficient(0x3F000000), _coefficient(0x3F4C422A)
        cubic, cubic_d = _coefficient(0x3D372713), _coefficient(0x3E095D4F)
        with np.errstate(invalid="ignore", over="ignore"):
            squared = x * x
            u = (x + (squared * x) * cubic) * s2pi
            t = tanh(u)
            u_prime = (one + squared * cubic_d) * s2pi
            regular = g * ((one + t) * half + ((x * (one - t * t)) * u_prime) * half)
        return np.where(np.isinf(x), np.where(x > 0, g, np.float32(0.0)), regular).astype(np.float32)
    if kind == "gelu":
        # ElementwiseGradientRules.gelu (:272-278), FLOAT32 coefficients (:370-378)
        x = _f32(pre_activation)
        half, neg_half = _coefficient(0x3F000000), _coefficient(0xBF000000)
        inv_sqrt2, inv_sqrt_2pi = _coefficient(0x3F3504F3), _coefficient(0x3ECC422A)
        with np.errstate(invalid="ignore", over="ignore"):
            cdf = (one + erf(x * inv_sqrt2)) * half
            e = np.exp(((x * x) * neg_half).astype(np.float64)).astype(np.float32)
            regular = g * (cdf + (x * e) * inv_sqrt_2pi)
        return np.where(np.isinf(x), np.where(x > 0, g, np.float32(0.0)), regular).astype(np.float32)
    if kind == "silu":
        x = _f32(pre_activation)
        s = sigmoid(x)
        with np.errstate(invalid="ignore", over="ignore"):
            regular = ((g * s).astype(np.float32) * (one + (x * (one - s).astype(np.float32)).astype(np.float32)).astype(np.float32)).astype(np.float32)
        return np.where(np.isinf(x), np.where(x > 0, g, np.float32(0.0)), regular).astype(np.float32)
    if kind == "tanh":
        return (g * (one - (y * y).astype(np.float32)).astype(np.float32)).astype(np.float32)
    return ((g * y).astype(np.float32) * (one - y).astype(np.float32)).astype(np.float32)


def bias_act(u, bias, relu_flag: bool):
    """Returns (z, y): z = u + bias (row broadcast), y = relu(z) or z."""
    u = _f32(u)
    m, n = u.shape
    z = np.empty_like(u)
    y = np.empty_like(u)
    b = _f32(bias) if bias is not None else None
    lib().syn_oracle_bias_act_f32(ctypes.c_int64(m), ctypes.c_int64(n), _p(u),
                                  _p(b) if b is not None else None, int(relu_flag), _p(z), _p(y))
    return z, y


def linear(x, weight, bias, relu_flag: bool):
    """``Tensor.linear`` then optional ReLU: x[M,K] . weight[N,K]^T + bias -> (z, y)."""
    u = matmul(_f32(x), _f32(weight).T)
    return bias_act(u, bias, relu_flag)


def exact_sum(x) -> float:
    x = _f32(x).ravel()
    return float(lib().syn_oracle_exact_sum_f32(ctypes.c_int64(x.size), _p(x), ctypes.c_int64(1)))


def colsum_exact(g) -> np.ndarray:
    g = _f32(g)
    m, n = g.shape
    out = np.empty(n, dtype=np.float32)
    lib().syn_oracle_colsum_exact_f32(ctypes.c_int64(m), ctypes.c_int64(n), _p(g), _p(out))
    return out


def softmax(x) -> np.ndarray:
    x = _f32(x)
    rows, classes = x.shape
    out = np.empty_like(x)
    lib().syn_oracle_softmax_f32(ctypes.c_int64(rows), ctypes.c_int64(classes), _p(x), _p(out))
    return out


def log_softmax(x) -> np.ndarray:
    x = _f32(x)
    rows, classes = x.shape
    out = np.empty_like(x)
    lib().syn_oracle_log_softmax_f32(ctypes.c_int64(rows), ctypes.c_int64(classes), _p(x), _p(out))
    return out


def softmax_backward(output, upstream, log_kind: bool = False) -> np.ndarray:
    """Gradient node list of SOFTMAX / LOG_SOFTMAX (ReductionGradientRules.java:84-90), one binary32
    rounding per node, the row SUM exactly rounded (CpuExactSumEmitter.java:14-21)."""
    y, g = _f32(output), _f32(upstream)
    if log_kind:
        total = np.array([[exact_sum(row)] for row in g], dtype=np.float32)
        e = np.exp(y.astype(np.float64)).astype(np.float32)
        return (g - (e * total).astype(np.float32)).astype(np.float32)
    gy = (g * y).astype(np.float32)
    total = np.array([[exact_sum(row)] for row in gy], dtype=np.float32)
    return (y * (g - total).astype(np.float32)).astype(np.float32)


def index_cross_entropy(logits, labels):
    """Returns (per_row, mean).  Raises ValueError for an out-of-range label."""
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    rows, classes = logits.shape
    per_row = np.empty(rows, dtype=np.float32)
    mean = ctypes.c_float(0.0)
    status = lib().syn_oracle_index_ce_f32(ctypes.c_int64(rows), ctypes.c_int64(classes),
                                           _p(logits), _p(labels, _i64p), _p(per_row),
                                           ctypes.byref(mean))
    if status:
        raise ValueError("index target out of bounds")
    return per_row, np.float32(mean.value)


def index_cross_entropy_backward(logits, labels, seed: float = 1.0, count: int = 0) -> np.ndarray:
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    rows, classes = logits.shape
    out = np.empty_like(logits)
    lib().syn_oracle_index_ce_backward_f32(ctypes.c_int64(rows), ctypes.c_int64(classes),
                                           _p(logits), _p(labels, _i64p), ctypes.c_float(seed),
                                           ctypes.c_int64(count), _p(out))
    return out


_REDUCTIONS = {"none": 0, "mean": 1, "sum": 2}


def index_cross_entropy_ignore(logits, labels, ignore_index: int, reduction: str = "mean"):
    """Returns (per_row, reduced) under an ignore index; `reduced` is the mean over the rows that are
    not ignored, or the sum.  Raises ValueError for a label out of bounds that is not ignored."""
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    rows, classes = logits.shape
    per_row = np.empty(rows, dtype=np.float32)
    reduced = ctypes.c_float(0.0)
    status = lib().syn_oracle_index_ce_ignore_f32(ctypes.c_int64(rows), ctypes.c_int64(classes), _p(logits), _p(labels, _i64p),
                                                  ctypes.c_int64(ignore_index), ctypes.c_int(_REDUCTIONS[reduction]),
                                                  _p(per_row), ctypes.byref(reduced))
    if status:
        raise ValueError("index target out of bounds")
    return per_row, np.float32(reduced.value)


def dense_cross_entropy(logits, target, reduction: str = "mean"):
    """Returns (per_row, reduced) of the dense-target categorical cross entropy with logits."""
    logits, target = _f32(logits), _f32(target)
    rows, classes = logits.shape
    per_row = np.empty(rows, dtype=np.float32)
    reduced = ctypes.c_float(0.0)
    lib().syn_oracle_dense_ce_f32(ctypes.c_int64(rows), ctypes.c_int64(classes), _p(logits), _p(target),
                                  ctypes.c_int(_REDUCTIONS[reduction]), _p(per_row), ctypes.byref(reduced))
    return per_row, np.float32(reduced.value)


def _row_sums(x) -> np.ndarray:
    """Aggregate SUM over axis 1, kept: exactly rounded (CpuExactSumEmitter.java:14-21)."""
    return np.array([[exact_sum(row)] for row in _f32(x)], dtype=np.float32)


def _categorical_probabilities(logits) -> np.ndarray:
    """exp(x - MAX) / SUM(exp(x - MAX)), one binary32 rounding per node (LossGradientRules.java:239-243);
    finite logits only (the aggregate MAX is Math.max)."""
    x = _f32(logits)
    shifted = (x - x.max(axis=1, keepdims=True)).astype(np.float32)
    e = np.exp(shifted.astype(np.float64)).astype(np.float32)
    return (e / _row_sums(e)).astype(np.float32)


def _restored(seed, rows: int, reduction: str, count=None) -> np.ndarray:
    """The output cotangent on the sample domain, shape [rows, 1] (LossGradientRules.restore)."""
    if reduction == "none":
        return _f32(seed).reshape(rows, 1)
    scale = np.full((rows, 1), np.float32(seed), dtype=np.float32)
    if reduction == "mean":
        scale = (scale / np.float32(rows if count is None else count)).astype(np.float32)
    return scale


def index_cross_entropy_ignore_backward(logits, labels, ignore_index: int, seed=1.0, reduction: str = "mean") -> np.ndarray:
    """The node list of LossGradientRules.indexCategorical (:172-228) with an ignore index, node by
    node in binary32; finite logits only."""
    logits = _f32(logits)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    rows, classes = logits.shape
    ignored = (labels == ignore_index).reshape(rows, 1)
    active = np.float32(exact_sum(np.where(ignored, 0.0, 1.0).astype(np.float32)))
    scale = _restored(seed, rows, "none" if reduction == "none" else "sum")
    if reduction == "mean":
        scale = (scale / active).astype(np.float32)
    scale = np.where(ignored, np.float32(0.0), scale).astype(np.float32)
    safe_logits = np.where(ignored, np.float32(0.0), logits).astype(np.float32)
    hot = np.zeros_like(logits)
    hot[np.arange(rows), np.clip(labels, 0, classes - 1)] = 1.0
    raw = ((_categorical_probabilities(safe_logits) - hot).astype(np.float32) * scale).astype(np.float32)
    return np.where(ignored, np.float32(0.0), raw).astype(np.float32)


def dense_cross_entropy_backward(logits, target, seed=1.0, reduction: str = "mean") -> np.ndarray:
    """The logits cotangent of LossGradientRules.denseCategorical (:114-145), node by node in binary32;
    finite logits only."""
    logits, target = _f32(logits), _f32(target)
    rows, _ = logits.shape
    restored = _restored(seed, rows, reduction)
    membership = _row_sums(np.where(target == 0.0, 0.0, 1.0).astype(np.float32))
    empty = membership == 0.0
    p = _categorical_probabilities(np.where(empty, np.float32(0.0), logits).astype(np.float32))
    mass = _row_sums(target)
    scale = np.where(empty, np.float32(0.0), restored).astype(np.float32)
    raw = (((p * mass).astype(np.float32) - target).astype(np.float32) * scale).astype(np.float32)
    return np.where(empty, np.float32(0.0), raw).astype(np.float32)


def mse(prediction, target) -> np.float32:
    p, t = _f32(prediction).ravel(), _f32(target).ravel()
    return np.float32(lib().syn_oracle_mse_f32(ctypes.c_int64(p.size), _p(p), _p(t)))


def squared_error(prediction, target, reduction: str = "none"):
    """MEAN_SQUARED_ERROR with reduction NONE (per element) or SUM (CpuLossReferenceKernel.java:67-87)."""
    p, t = _f32(prediction), _f32(target)
    if reduction == "sum":
        lib().syn_oracle_squared_error_sum_f32.restype = ctypes.c_float
        return np.float32(lib().syn_oracle_squared_error_sum_f32(ctypes.c_int64(p.size), _p(p.ravel()), _p(t.ravel())))
    d = (p - t).astype(np.float32)
    return (d * d).astype(np.float32)


def mse_backward(prediction, target, seed: float = 1.0, count: int = 0) -> np.ndarray:
    p, t = _f32(prediction), _f32(target)
    out = np.empty_like(p)
    lib().syn_oracle_mse_backward_f32(ctypes.c_int64(p.size), _p(p), _p(t), ctypes.c_float(seed),
                                      ctypes.c_int64(count), _p(out))
    return out


def relu_backward(z, g) -> np.ndarray:
    z, g = _f32(z), _f32(g)
    out = np.empty_like(g)
    lib().syn_oracle_relu_backward_f32(ctypes.c_int64(z.size), _p(z), _p(g), _p(out))
    return out


def argmax(x) -> np.ndarray:
    x = _f32(x)
    rows, classes = x.shape
    out = np.empty(rows, dtype=np.int64)
    lib().syn_oracle_argmax_f32(ctypes.c_int64(rows), ctypes.c_int64(classes), _p(x), _p(out, _i64p))
    return out


def sgd(parameter, gradient, momentum_buffer=None, lr=0.01, momentum=0.0, dampening=0.0,
        weight_decay=0.0, nesterov=False, completed_steps=0):
    """In-place on float32 arrays; returns True when the update committed (all finite)."""
    assert parameter.dtype == np.float32 and parameter.flags.c_contiguous
    g = _f32(gradient)
    status = lib().syn_oracle_sgd_f32(
        ctypes.c_int64(parameter.size), _p(parameter), _p(g),
        _p(momentum_buffer) if momentum_buffer is not None else None,
        ctypes.c_double(lr), ctypes.c_double(momentum), ctypes.c_double(dampening),
        ctypes.c_double(weight_decay), int(nesterov), ctypes.c_int64(completed_steps))
    return status == 0


def accumulate(accumulated, gradient):
    """In-place pending gradient sum (GradientMode.ACCUMULATE); True when committed (all finite)."""
    assert accumulated.dtype == np.float32 and accumulated.flags.c_contiguous
    g = _f32(gradient)
    return lib().syn_oracle_accumulate_f32(ctypes.c_int64(accumulated.size), _p(accumulated), _p(g)) == 0


def adam(parameter, gradient, first, second, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8,
         weight_decay=0.0, decoupled=False):
    """In-place Adam/AdamW on float32 arrays; ``step`` counts from 1.  True when committed."""
    for a in (parameter, first, second):
        assert a.dtype == np.float32 and a.flags.c_contiguous
    g = _f32(gradient)
    status = lib().syn_oracle_adam_f32(
        ctypes.c_int64(parameter.size), _p(parameter), _p(g), _p(first), _p(second),
        ctypes.c_double(lr), ctypes.c_double(beta1), ctypes.c_double(beta2), ctypes.c_double(eps),
        ctypes.c_double(weight_decay), int(decoupled), ctypes.c_int64(step))
    return status == 0


# --------------------------------------------------------------------------------------------
# Composite: the training graph the backend is handed (forward, loss, backward), op by op.
# --------------------------------------------------------------------------------------------
def mlp_forward(x, weights, biases, activation: str = "relu", pre_activations=None):
    """Returns the list of post-activation values [a1..aL] (aL = logits, no activation); appends the
    pre-activations z1..zL to ``pre_activations`` when a list is given."""
    acts = []
    a = _f32(x)
    for index, (w, b) in enumerate(zip(weights, biases)):
        hidden_layer = index + 1 < len(weights)
        z, a = linear(a, w, b, relu_flag=hidden_layer and activation == "relu")
        if hidden_layer and activation != "relu":
            a = {"tanh": tanh, "sigmoid": sigmoid, "silu": silu, "gelu_tanh": gelu_tanh, "gelu": gelu}[activation](z)
        if pre_activations is not None:
            pre_activations.append(z)
        acts.append(a)
    return acts


def mlp_gradients(x, labels_or_target, weights, biases, loss: str = "ce", count: int = 0, hidden=None,
                  activation: str = "relu"):
    """Loss and gradients of an MLP, executing the reference's backward node lists in order.

    Returns (loss, [dW1, db1, dW2, db2, ...], logits).  ``loss`` is "ce" (index cross entropy,
    MEAN) or "mse" (MEAN).  ``count`` overrides the divisor of the loss gradient.  ``hidden``
    (the hidden activations a1..a(L-1)) replaces the checker's own forward values in the backward
    pass and in the last layer, so that a device's backward pass can be checked on the device's own
    ReLU gates (a pre-activation within rounding distance of zero may legitimately take the other
    branch on another implementation).
    """
    x = _f32(x)
    zs = []
    acts = mlp_forward(x, weights, biases, activation, zs)
    if hidden is not None:
        acts = [_f32(h) for h in hidden] + [linear(_f32(hidden[-1]), weights[-1], biases[-1], relu_flag=False)[1]]
    logits = acts[-1]
    if loss == "ce":
        _, value = index_cross_entropy(logits, labels_or_target)
        dz = index_cross_entropy_backward(logits, labels_or_target, 1.0, count)
    else:
        value = mse(logits, labels_or_target)
        dz = mse_backward(logits, _f32(labels_or_target).reshape(logits.shape), 1.0, count)
    grads = [None] * (2 * len(weights))
    for index in range(len(weights) - 1, -1, -1):
        a_prev = x if index == 0 else acts[index - 1]
        grads[2 * index + 1] = colsum_exact(dz)
        # dWt[K,N] = PERMUTE(a_prev)[K,M] . dz[M,N]; PERMUTE back gives dW[N,K]
        grads[2 * index] = np.ascontiguousarray(matmul(a_prev.T, dz).T)
        if index > 0:
            da = matmul(dz, _f32(weights[index]))
            # z > 0 <=> relu(z) > 0 for every binary32 value, so the stored activation serves
            dz = activation_backward(activation, a_prev, da, zs[index - 1])
    return value, grads, logits


# --------------------------------------------------------------------------------------------
# Timed CPU baseline (cpu_baseline.c)
# --------------------------------------------------------------------------------------------
def baseline_bind_openblas() -> str:
    """Binds an OpenBLAS the way the reference discovers one; returns the name used."""
    explicit = os.environ.get("SYNAPTIK_OPENBLAS", "")
    if not explicit:
        try:
            import glob
            import site
            for root in site.getsitepackages():
                found = sorted(glob.glob(os.path.join(root, "opencv_python_headless.libs",
                                                      "libopenblas*.so")))
                if found:
                    explicit = found[0]
                    break
        except Exception:
            explicit = ""
    if explicit:
        # the wheel-bundled OpenBLAS finds its Fortran runtime only when that is already loaded
        import glob
        folder = os.path.dirname(explicit)
        for pattern in ("libquadmath*.so*", "libgfortran*.so*"):
            for dep in sorted(glob.glob(os.path.join(folder, pattern))):
                try:
                    ctypes.CDLL(dep, mode=ctypes.RTLD_GLOBAL)
                except OSError:
                    pass
    lib().syn_baseline_bind_openblas(explicit.encode())
    return lib().syn_baseline_blas_name().decode()


def baseline_mlp_step(dims, x, labels, weights, biases, m1, m2, train=True, count_total=0,
                      adam_step=1, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, threads=1,
                      want_logits=False):
    """Runs one CPU MLP step in place on the given float32 arrays; returns (seconds, loss, logits)."""
    layers = len(dims) - 1
    rows = x.shape[0]
    lib().syn_baseline_set_threads(int(threads))
    dims_c = (ctypes.c_int * (layers + 1))(*dims)
    w_c = (_f32p * layers)(*[_p(w) for w in weights])
    b_c = (_f32p * layers)(*[_p(b) for b in biases])
    m1_c = (_f32p * (2 * layers))(*[_p(a) for a in m1]) if train else None
    m2_c = (_f32p * (2 * layers))(*[_p(a) for a in m2]) if train else None
    loss = ctypes.c_float(0.0)
    logits = np.empty((rows, dims[-1]), dtype=np.float32) if want_logits else None
    lab = np.ascontiguousarray(labels, dtype=np.int32) if labels is not None else None
    seconds = lib().syn_baseline_mlp_step(
        layers, dims_c, rows, _p(x), _p(lab, _i32p) if lab is not None else None, w_c, b_c,
        m1_c, m2_c, int(train), ctypes.c_int64(count_total or rows), ctypes.c_int64(adam_step),
        ctypes.c_double(lr), ctypes.c_double(beta1), ctypes.c_double(beta2), ctypes.c_double(eps),
        ctypes.byref(loss), _p(logits) if logits is not None else None)
    return seconds, np.float32(loss.value), logits


# --------------------------------------------------------------------------------------------
# 16-bit storage (BFLOAT16 / FLOAT16) with a FLOAT32 working type
# --------------------------------------------------------------------------------------------
# The reference keeps low-precision tensors as raw 16-bit patterns, widens every operand to FLOAT32,
# computes in FLOAT32 and narrows each NODE's result once, round to nearest even
# (CpuScalarReferenceKernel.java:93-115 lowFloat / lowBits, BFloat16Bits.java:17-29, Float16Bits =
# IEEE binary16).  Storage arrays here are uint16; `kind` is "bf16" or "f16".
def low_encode(kind: str, x) -> np.ndarray:
    """FLOAT32 -> storage bits.  BFLOAT16: NaN becomes 0x7FC0, otherwise round half to even on the
    discarded 16 bits (BFloat16Bits.fromFloat); FLOAT16: IEEE conversion (Float.floatToFloat16)."""
    x = _f32(x)
    if kind == "f16":
        with np.errstate(over="ignore"):
            out = x.astype(np.float16).view(np.uint16).copy()
        out[np.isnan(x)] = 0x7E00           # Float16Bits.CANONICAL_NAN
        return out
    bits = x.view(np.uint32)
    upper = (bits >> 16).astype(np.uint32)
    discarded = bits & np.uint32(0xFFFF)
    up = (discarded > 0x8000) | ((discarded == 0x8000) & ((upper & 1) == 1))
    upper = upper + up.astype(np.uint32)
    out = (upper & 0xFFFF).astype(np.uint16)
    out[np.isnan(x)] = 0x7FC0
    return out


def low_decode(kind: str, bits) -> np.ndarray:
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if kind == "f16":
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


def low_round(kind: str, x) -> np.ndarray:
    """A FLOAT32 working value as the storage type will hold it."""
    return low_decode(kind, low_encode(kind, x))


def low_activation(name: str, x) -> np.ndarray:
    """FLOAT32 working result of an activation on exactly decoded low inputs, before the one narrowing.
    SIGMOID, SILU and both GELUs are FLOAT32 composites (CpuScalarReferenceKernel.lowActivation, :1753-1775:
    every product, sum and quotient a binary32 rounding, the elementary function in binary64 and narrowed
    at once; -inf gives -0 except for SIGMOID); RELU and TANH take the binary64 function of the widened
    value and one narrowing (:1722-1742)."""
    x = _f32(x)
    one, half = np.float32(1.0), np.float32(0.5)
    with np.errstate(all="ignore"):
        if name == "relu":
            return relu(x)
        if name == "tanh":
            return tanh(x)
        if name in ("sigmoid", "silu"):
            e = np.exp(np.where(x >= 0, -x, x).astype(np.float64)).astype(np.float32)
            if name == "sigmoid":
                return (np.where(x >= 0, one, e) / (one + e)).astype(np.float32)
            y = (np.where(x >= 0, x, (x * e).astype(np.float32)) / (one + e)).astype(np.float32)
        elif name == "gelu":
            root = np.float32(np.sqrt(np.float64(np.float32(2.0))))
            inner = erf((x / root).astype(np.float32))
            y = ((half * x).astype(np.float32) * (one + inner).astype(np.float32)).astype(np.float32)
        elif name == "gelu_tanh":
            cube = ((x * x).astype(np.float32) * x).astype(np.float32)
            scale = np.float32(np.sqrt(np.float64(np.float32(2.0) / np.float32(np.pi))))
            argument = (scale * (x + (np.float32(0.044715) * cube).astype(np.float32)).astype(np.float32)).astype(np.float32)
            inner = np.tanh(argument.astype(np.float64)).astype(np.float32)
            y = ((half * x).astype(np.float32) * (one + inner).astype(np.float32)).astype(np.float32)
        else:
            raise ValueError(name)
        return np.where(np.isneginf(x), np.float32(-0.0), y).astype(np.float32)


def low_linear(kind: str, x_bits, w_bits, bias_bits, activation: str | None):
    """Tensor.linear on 16-bit storage, node by node: MATMUL as the sequential FLOAT32 chain over the
    widened operands with one narrowing of the sum (CpuMatmulReferenceKernel.java:71-93), ADD of the
    row-broadcast bias in FLOAT32 with one narrowing, then the activation with one narrowing.
    Returns the storage bits of (z, y)."""
    u = low_round(kind, matmul(low_decode(kind, x_bits), low_decode(kind, w_bits).T))
    z = low_round(kind, (u + low_decode(kind, bias_bits)[None, :]).astype(np.float32)) if bias_bits is not None else u
    y = low_round(kind, low_activation(activation, z)) if activation else z
    return low_encode(kind, z), low_encode(kind, y)


def low_mlp_forward(kind: str, x_bits, weights_bits, biases_bits, activation: str = "relu"):
    """Model.compute on 16-bit storage: the storage bits of the last layer's output."""
    a = x_bits
    for index, (w, b) in enumerate(zip(weights_bits, biases_bits)):
        z, y = low_linear(kind, a, w, b, activation if index + 1 < len(weights_bits) else None)
        a = y
    return a
