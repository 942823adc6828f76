"""Builds "SCU1" program images: the serialised form of one backend partition.

The Java partition finalizer would write exactly this from the CompiledNode list it is handed;
here a small expression builder plays that role for the tests, the benchmark and the Python
mirror of the model API.  One method per reference operation, named after the ``Tensor``
expression it stands for (modules/model/.../tensor/Tensor.java: matmul :1109, linear :1310,
relu :2695, softmax :4636, argMax :4373, categoricalCrossEntropyWithLogits :1218,
meanSquaredError :1150).  ``linear_backward`` / ``index_cross_entropy_backward`` /
``mean_squared_error_backward`` / ``relu_backward`` emit the node lists of the reference's
gradient rules (modules/compiler/.../LinearAlgebraGradientRules.java:97-104,
LossGradientRules.java:77-101,172-243, ElementwiseGradientRules.java:99-101,210) in that order,
so the image holds the same decomposed graph the compiler produces.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import List, Sequence

F32, I32, I64, BOOL, BF16, F16 = 1, 2, 3, 4, 5, 6
DTYPE_BYTES = {F32: 4, I32: 4, I64: 8, BOOL: 1, BF16: 2, F16: 2}
# BFLOAT16 / FLOAT16 are storage types (DataType.BFLOAT16 / FLOAT16): values travel as raw 16-bit patterns,
# every node widens its operands to FLOAT32, computes there and narrows its result once.  They are accepted
# by the views, MATMUL, ADD / SUB / MUL / DIV, the activations, CONTIGUOUS and ARG_MAX: the inference path.

STORAGE_DTYPES = {"f32": F32, "bf16": BF16, "f16": F16}


def to_storage(kind: str, array):
    """FLOAT32 values as the storage type holds them: the array itself for "f32", raw 16-bit patterns
    (uint16) for "bf16" (round to nearest even, NaN -> 0x7FC0: BFloat16Bits.fromFloat) and "f16" (IEEE
    binary16, NaN -> 0x7E00: Float16Bits.fromFloat)."""
    import numpy as np
    array = np.ascontiguousarray(array, dtype=np.float32)
    if kind == "f32":
        return array
    if kind == "f16":
        with np.errstate(over="ignore"):
            bits = array.astype(np.float16).view(np.uint16).copy()
        bits[np.isnan(array)] = 0x7E00
        return bits
    raw = array.view(np.uint32)
    upper = raw >> 16
    discarded = raw & np.uint32(0xFFFF)
    upper = upper + ((discarded > 0x8000) | ((discarded == 0x8000) & ((upper & 1) == 1))).astype(np.uint32)
    bits = (upper & 0xFFFF).astype(np.uint16)
    bits[np.isnan(array)] = 0x7FC0
    return bits


def from_storage(kind: str, bits):
    """The FLOAT32 values of raw storage patterns (exact)."""
    import numpy as np
    if kind == "f32":
        return np.ascontiguousarray(bits, dtype=np.float32)
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    if kind == "f16":
        return bits.view(np.float16).astype(np.float32)
    return (bits.astype(np.uint32) << 16).view(np.float32)


OPS = {
    "PERMUTE": 1, "MATMUL": 2, "ADD": 3, "SUB": 4, "MUL": 5, "DIV": 6, "SCALAR_MUL": 7, "SCALAR_MIN": 8,
    "SCALAR_MAX": 9, "RELU": 10, "EXP": 11, "GT": 12, "WHERE": 13, "EXPAND": 14, "EXPAND_DIMS": 15,
    "CONTIGUOUS": 16, "ONE_HOT": 17, "MAX": 18, "SUM": 19, "SUM_TO_SHAPE": 20, "SOFTMAX": 21,
    "INDEX_CROSS_ENTROPY": 22, "MEAN_SQUARED_ERROR": 23, "ARG_MAX": 24, "TANH": 25, "SIGMOID": 26, "SILU": 27, "IS_INF": 28, "GELU_TANH": 29, "CLAMP": 30, "LT": 31, "EQ": 32,
    "SCALAR_SUB": 33, "DENSE_CROSS_ENTROPY": 34, "GELU": 35, "ERF": 36,
}
ROLE_INTERMEDIATE, ROLE_FEED, ROLE_CONSTANT = 0, 1, 2
MASK64 = (1 << 64) - 1


def _f32_round(x: float) -> float:
    """The binary32 value nearest to x, as a Python float."""
    return struct.unpack("<f", struct.pack("<f", float(x)))[0]


def _f64_bits(x: float) -> int:
    return struct.unpack("<Q", struct.pack("<d", float(x)))[0]


@dataclass
class Value:
    index: int
    dtype: int
    shape: tuple
    role: int = ROLE_INTERMEDIATE
    constant_bits: int = 0
    strides: tuple | None = None

    @property
    def elements(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.elements * DTYPE_BYTES[self.dtype]


@dataclass
class _Node:
    op: int
    inputs: List[int]
    outputs: List[int]
    attrs: List[int] = field(default_factory=list)


def _broadcast(a: Sequence[int], b: Sequence[int]) -> tuple:
    r = max(len(a), len(b))
    a = (1,) * (r - len(a)) + tuple(a)
    b = (1,) * (r - len(b)) + tuple(b)
    out = []
    for x, y in zip(a, b):
        if x != y and x != 1 and y != 1:
            raise ValueError(f"shapes {a} and {b} do not broadcast")
        out.append(y if x == 1 else x)
    return tuple(out)


class GraphBuilder:
    def __init__(self):
        self.values: List[Value] = []
        self.nodes: List[_Node] = []
        self.feeds: List[int] = []
        self.publications: List[int] = []

    # ---- values ---------------------------------------------------------------------------
    def _value(self, dtype, shape, role=ROLE_INTERMEDIATE, bits=0, strides=None) -> Value:
        v = Value(len(self.values), dtype, tuple(int(d) for d in shape), role, bits, strides)
        self.values.append(v)
        return v

    def feed(self, dtype: int, shape: Sequence[int], strides: Sequence[int] | None = None) -> Value:
        v = self._value(dtype, shape, ROLE_FEED, 0, tuple(strides) if strides is not None else None)
        self.feeds.append(v.index)
        return v

    def constant(self, dtype: int, value) -> Value:
        bits = _f64_bits(value) if dtype == F32 else int(value) & MASK64
        return self._value(dtype, (), ROLE_CONSTANT, bits)

    def publish(self, value: Value) -> Value:
        self.publications.append(value.index)
        return value

    def _node(self, op: str, inputs: Sequence[Value], dtype: int, shape: Sequence[int], attrs: Sequence[int] = ()) -> Value:
        out = self._value(dtype, shape)
        self.nodes.append(_Node(OPS[op], [v.index for v in inputs], [out.index], [int(a) & MASK64 for a in attrs]))
        return out

    # ---- operations -----------------------------------------------------------------------
    def permute(self, x: Value, permutation: Sequence[int]) -> Value:
        return self._node("PERMUTE", [x], x.dtype, [x.shape[p] for p in permutation], permutation)

    def matmul(self, a: Value, b: Value) -> Value:
        """MATMUL over the last two dimensions; leading batch dimensions broadcast right-aligned
        (Tensor.java:1075-1096)."""
        if len(a.shape) < 2 or len(b.shape) < 2 or a.shape[-1] != b.shape[-2]:
            raise ValueError("MATMUL contraction extents differ")
        batch = _broadcast(tuple(a.shape[:-2]), tuple(b.shape[:-2]))
        return self._node("MATMUL", [a, b], a.dtype, tuple(batch) + (a.shape[-2], b.shape[-1]))

    def swap_last_two(self, x: Value) -> Value:
        """PERMUTE exchanging the final two axes (LinearAlgebraGradientRules.swapLastTwo)."""
        axes = list(range(len(x.shape)))
        axes[-2], axes[-1] = axes[-1], axes[-2]
        return self.permute(x, axes)

    def matmul_backward(self, a: Value, b: Value, upstream: Value):
        """MATMUL gradient rule for operands of rank two and above (LinearAlgebraGradientRules.java:97-104,
        normalize :121-131): g x swapLastTwo(b) and swapLastTwo(a) x g, each summed back over the batch
        dimensions its operand was broadcast along.  Returns (da, db)."""
        da = self.matmul(upstream, self.swap_last_two(b))
        db = self.matmul(self.swap_last_two(a), upstream)
        if tuple(da.shape) != tuple(a.shape):
            da = self.sum_to_shape(da, a.shape)
        if tuple(db.shape) != tuple(b.shape):
            db = self.sum_to_shape(db, b.shape)
        return da, db

    def _binary(self, op: str, a: Value, b: Value) -> Value:
        return self._node(op, [a, b], BOOL if op in ("GT", "LT", "EQ") else a.dtype, _broadcast(a.shape, b.shape))

    def add(self, a, b): return self._binary("ADD", a, b)
    def sub(self, a, b): return self._binary("SUB", a, b)
    def mul(self, a, b): return self._binary("MUL", a, b)
    def div(self, a, b): return self._binary("DIV", a, b)
    def gt(self, a, b): return self._binary("GT", a, b)
    def lt(self, a, b): return self._binary("LT", a, b)
    def eq(self, a, b): return self._binary("EQ", a, b)

    def clamp(self, x: Value, min_value: float, max_value: float) -> Value:
        """CLAMP: MIN(MAX(x, min), max) with FLOAT32 bounds (Tensor.java:2318-2345)."""
        return self._node("CLAMP", [x], F32, x.shape, [_f64_bits(_f32_round(min_value)), _f64_bits(_f32_round(max_value))])

    def clamp_backward(self, x: Value, upstream: Value, min_value: float, max_value: float) -> Value:
        """The node list of ElementwiseGradientRules.clamp (:263-270): the gradient passes inside the
        range, half of it at a bound, none outside."""
        zero = self.expand(self.constant(F32, 0.0), x.shape)
        lo = self.expand(self.constant(F32, _f32_round(min_value)), x.shape)
        hi = self.expand(self.constant(F32, _f32_round(max_value)), x.shape)
        lowered = self.scalar_max(x, _f32_round(min_value))
        upper = self.where(self.lt(lowered, hi), upstream, self.where(self.eq(lowered, hi), self.scalar_mul(upstream, 0.5), zero))
        return self.where(self.gt(x, lo), upper, self.where(self.eq(x, lo), self.scalar_mul(upper, 0.5), zero))

    def _scalar(self, op: str, x: Value, scalar) -> Value:
        bits = _f64_bits(scalar) if x.dtype == F32 else int(scalar)
        return self._node(op, [x], x.dtype, x.shape, [bits])

    def scalar_mul(self, x, s): return self._scalar("SCALAR_MUL", x, s)
    def scalar_min(self, x, s): return self._scalar("SCALAR_MIN", x, s)
    def scalar_max(self, x, s): return self._scalar("SCALAR_MAX", x, s)
    def scalar_sub(self, x, s): return self._scalar("SCALAR_SUB", x, s)
    def relu(self, x): return self._node("RELU", [x], x.dtype, x.shape)
    def exp(self, x): return self._node("EXP", [x], x.dtype, x.shape)
    def tanh(self, x): return self._node("TANH", [x], x.dtype, x.shape)
    def sigmoid(self, x): return self._node("SIGMOID", [x], x.dtype, x.shape)
    def silu(self, x): return self._node("SILU", [x], x.dtype, x.shape)
    def is_inf(self, x): return self._node("IS_INF", [x], BOOL, x.shape)
    def gelu_tanh(self, x): return self._node("GELU_TANH", [x], x.dtype, x.shape)
    def gelu(self, x): return self._node("GELU", [x], x.dtype, x.shape)
    def erf(self, x): return self._node("ERF", [x], x.dtype, x.shape)

    def activation(self, kind: str, x: Value) -> Value:
        return {"relu": self.relu, "tanh": self.tanh, "sigmoid": self.sigmoid, "silu": self.silu,
                "gelu_tanh": self.gelu_tanh, "gelu": self.gelu}[kind](x)

    def where(self, condition: Value, a: Value, b: Value) -> Value:
        return self._node("WHERE", [condition, a, b], F32, _broadcast(_broadcast(condition.shape, a.shape), b.shape))

    def expand(self, x: Value, shape: Sequence[int]) -> Value:
        return self._node("EXPAND", [x], x.dtype, shape)

    def expand_dims(self, x: Value, axis: int) -> Value:
        shape = list(x.shape)
        shape.insert(axis, 1)
        return self._node("EXPAND_DIMS", [x], x.dtype, shape, [axis])

    def contiguous(self, x): return self._node("CONTIGUOUS", [x], x.dtype, x.shape)

    def one_hot(self, indices: Value, depth: int) -> Value:
        return self._node("ONE_HOT", [indices], BOOL, tuple(indices.shape) + (depth,), [depth])

    def _reduce(self, op: str, x: Value, axis: int, keep: bool) -> Value:
        axis = axis % len(x.shape)
        shape = list(x.shape)
        if keep:
            shape[axis] = 1
        else:
            del shape[axis]
        return self._node(op, [x], F32, shape, [axis, int(keep)])

    def max(self, x, axis, keep_dimensions=False): return self._reduce("MAX", x, axis, keep_dimensions)
    def sum(self, x, axis, keep_dimensions=False): return self._reduce("SUM", x, axis, keep_dimensions)
    def sum_all(self, x): return self._node("SUM", [x], F32, (), [-1, 0])
    def sum_to_shape(self, x, shape): return self._node("SUM_TO_SHAPE", [x], F32, shape)
    def softmax(self, x, axis=-1): return self._node("SOFTMAX", [x], F32, x.shape, [axis % len(x.shape)])

    def log_softmax(self, x, axis=-1):
        """Tensor.logSoftmax (Tensor.java:4669): the SOFTMAX node with kind LOG_SOFTMAX."""
        return self._node("SOFTMAX", [x], F32, x.shape, [axis % len(x.shape), 1])

    def softmax_backward(self, output: Value, upstream: Value, axis: int = -1) -> Value:
        """y * (g - sum(g * y, axis, keep)) (ReductionGradientRules.java:84-90)."""
        return self.mul(output, self.sub(upstream, self.sum(self.mul(upstream, output), axis, True)))

    def log_softmax_backward(self, output: Value, upstream: Value, axis: int = -1) -> Value:
        """g - exp(y) * sum(g, axis, keep) (ReductionGradientRules.java:84-90)."""
        return self.sub(upstream, self.mul(self.exp(output), self.sum(upstream, axis, True)))

    def index_cross_entropy(self, logits: Value, labels: Value, reduction: str = "mean", ignore_index=None) -> Value:
        """INDEX_CATEGORICAL_CROSS_ENTROPY_WITH_LOGITS, class axis 1; reduction "mean", "sum" or "none"
        (one loss per row); rows labelled `ignore_index` contribute nothing and MEAN does not count them
        (TensorLossExpressions.java:301-403)."""
        shape = (logits.shape[0],) if reduction == "none" else ()
        attrs = [1, self.MSE_REDUCTIONS[reduction], 0 if ignore_index is None else 1, 0 if ignore_index is None else int(ignore_index)]
        return self._node("INDEX_CROSS_ENTROPY", [logits, labels], F32, shape, attrs)

    def dense_cross_entropy(self, logits: Value, target: Value, reduction: str = "mean") -> Value:
        """DENSE_CATEGORICAL_CROSS_ENTROPY_WITH_LOGITS with FLOAT32 target weights, class axis 1
        (TensorLossExpressions.java:204-221)."""
        shape = (logits.shape[0],) if reduction == "none" else ()
        return self._node("DENSE_CROSS_ENTROPY", [logits, target], F32, shape, [1, self.MSE_REDUCTIONS[reduction]])

    MSE_REDUCTIONS = {"none": 0, "mean": 1, "sum": 2}

    def mean_squared_error(self, prediction: Value, target: Value, reduction: str = "mean") -> Value:
        shape = prediction.shape if reduction == "none" else ()
        return self._node("MEAN_SQUARED_ERROR", [prediction, target], F32, shape, [self.MSE_REDUCTIONS[reduction]])

    def arg_max(self, x: Value, axis: int = 1, keep_dimensions: bool = False) -> Value:
        shape = list(x.shape)
        axis = axis % len(shape)
        if keep_dimensions:
            shape[axis] = 1
        else:
            del shape[axis]
        return self._node("ARG_MAX", [x], I64, shape, [axis, int(keep_dimensions)])

    # ---- composite expressions, as the reference builds them -----------------------------
    def linear(self, x: Value, weight: Value, bias: Value | None):
        """Tensor.linear: PERMUTE[1,0](W) -> MATMUL -> ADD(bias), no EXPAND for the bias
        (TensorLinearExpressions.java:74-76,142-144).  Returns (weight_view, pre_activation)."""
        wt = self.permute(weight, (1, 0))
        u = self.matmul(x, wt)
        return wt, (self.add(u, bias) if bias is not None else u)

    def linear_backward(self, x: Value, wt: Value, dz: Value, need_dx: bool, bias: bool = True):
        """ADD and MATMUL gradient rules.  Returns (dx or None, dW [N,K], db or None)."""
        db = self.sum_to_shape(dz, (dz.shape[1],)) if bias else None
        dx = self.matmul(dz, self.permute(wt, (1, 0))) if need_dx else None
        dwt = self.matmul(self.permute(x, (1, 0)), dz)
        dw = self.permute(dwt, (1, 0))
        return dx, dw, db

    def relu_backward(self, z: Value, upstream: Value) -> Value:
        """where(z > 0, g, 0) with EXPAND(0) and GT (ElementwiseGradientRules.java:210)."""
        zero = self.expand(self.constant(F32, 0.0), z.shape)
        return self.where(self.gt(z, zero), upstream, zero)

    def tanh_backward(self, output: Value, upstream: Value) -> Value:
        """g * (1 - y * y) with EXPAND(1) (ElementwiseGradientRules.java:206)."""
        one = self.expand(self.constant(F32, 1.0), output.shape)
        return self.mul(upstream, self.sub(one, self.mul(output, output)))

    def sigmoid_backward(self, output: Value, upstream: Value) -> Value:
        """(g * y) * (1 - y) with EXPAND(1) (ElementwiseGradientRules.java:205)."""
        one = self.expand(self.constant(F32, 1.0), output.shape)
        return self.mul(self.mul(upstream, output), self.sub(one, output))

    def silu_backward(self, x: Value, upstream: Value) -> Value:
        """where(isInf(x), where(x > 0, g, 0), (g * s) * (1 + x * (1 - s))) with s = SIGMOID(x)
        (ElementwiseGradientRules.java:290-301)."""
        one = self.expand(self.constant(F32, 1.0), x.shape)
        zero = self.expand(self.constant(F32, 0.0), x.shape)
        s = self.sigmoid(x)
        regular = self.mul(self.mul(upstream, s), self.add(one, self.mul(x, self.sub(one, s))))
        return self.where(self.is_inf(x), self.where(self.gt(x, zero), upstream, zero), regular)

    # FLOAT32 coefficients of the gradient rules (ElementwiseGradientRules.java:370-378, float32Bits column)
    _NEGATIVE_HALF, _INV_SQRT_2, _INV_SQRT_2_PI = 0xBF000000, 0x3F3504F3, 0x3ECC422A
    _HALF, _SQRT_2_OVER_PI = 0x3F000000, 0x3F4C422A
    _GELU_CUBIC, _GELU_CUBIC_DERIVATIVE = 0x3D372713, 0x3E095D4F

    def gelu_tanh_backward(self, x: Value, upstream: Value) -> Value:
        """The node list of ElementwiseGradientRules.geluTanhApproximation (:280-288): SCALAR_MUL by the
        FLOAT32 coefficients, TANH, and the infinity selection shared with SiLU."""
        f = lambda bits: struct.unpack("<f", struct.pack("<I", bits))[0]
        one = self.expand(self.constant(F32, 1.0), x.shape)
        zero = self.expand(self.constant(F32, 0.0), x.shape)
        squared = self.mul(x, x)
        u = self.scalar_mul(self.add(x, self.scalar_mul(self.mul(squared, x), f(self._GELU_CUBIC))), f(self._SQRT_2_OVER_PI))
        t = self.tanh(u)
        u_prime = self.scalar_mul(self.add(one, self.scalar_mul(squared, f(self._GELU_CUBIC_DERIVATIVE))), f(self._SQRT_2_OVER_PI))
        left = self.scalar_mul(self.add(one, t), f(self._HALF))
        right = self.scalar_mul(self.mul(self.mul(x, self.sub(one, self.mul(t, t))), u_prime), f(self._HALF))
        regular = self.mul(upstream, self.add(left, right))
        return self.where(self.is_inf(x), self.where(self.gt(x, zero), upstream, zero), regular)

    def gelu_backward(self, x: Value, upstream: Value) -> Value:
        """The node list of ElementwiseGradientRules.gelu (:272-278): g * (Phi(x) + x * phi(x)) with
        Phi = (1 + ERF(x / sqrt 2)) / 2 and phi = exp(-x^2 / 2) / sqrt(2 pi), every coefficient a
        SCALAR_MUL by its FLOAT32 bit pattern, and the infinity selection shared with SiLU."""
        f = lambda bits: struct.unpack("<f", struct.pack("<I", bits))[0]
        one = self.expand(self.constant(F32, 1.0), x.shape)
        zero = self.expand(self.constant(F32, 0.0), x.shape)
        cdf = self.scalar_mul(self.add(one, self.erf(self.scalar_mul(x, f(self._INV_SQRT_2)))), f(self._HALF))
        pdf_term = self.scalar_mul(self.mul(x, self.exp(self.scalar_mul(self.mul(x, x), f(self._NEGATIVE_HALF)))), f(self._INV_SQRT_2_PI))
        regular = self.mul(upstream, self.add(cdf, pdf_term))
        return self.where(self.is_inf(x), self.where(self.gt(x, zero), upstream, zero), regular)

    def activation_backward(self, kind: str, pre_activation: Value, output: Value, upstream: Value) -> Value:
        if kind == "gelu":
            return self.gelu_backward(pre_activation, upstream)
        if kind == "gelu_tanh":
            return self.gelu_tanh_backward(pre_activation, upstream)
        if kind == "relu":
            return self.relu_backward(pre_activation, upstream)
        if kind == "silu":
            return self.silu_backward(pre_activation, upstream)
        return self.tanh_backward(output, upstream) if kind == "tanh" else self.sigmoid_backward(output, upstream)

    def _loss_scale(self, seed: Value, rows: int) -> Value:
        ones = self.contiguous(self.expand(self.constant(F32, 1.0), (rows,)))
        count = self.sum_all(ones)
        return self.div(self.expand(seed, (rows,)), count)

    def _zeros(self, shape): return self.expand(self.constant(F32, 0.0), shape)
    def _ones(self, shape): return self.expand(self.constant(F32, 1.0), shape)

    def _restore(self, gradient: Value, rows: int, reduction: str) -> Value:
        """LossGradientRules.restore (:239-252): the reduced cotangent back on the sample domain."""
        if reduction == "none":
            return gradient
        return self._loss_scale(gradient, rows) if reduction == "mean" else self.expand(gradient, (rows,))

    def _categorical_probabilities(self, logits: Value) -> Value:
        """exp(x - MAX) / SUM(exp(x - MAX)) with aggregate MAX and SUM (LossGradientRules.java:239-243)."""
        e = self.exp(self.sub(logits, self.max(logits, 1, True)))
        return self.div(e, self.sum(e, 1, True))

    def index_cross_entropy_backward(self, logits: Value, labels: Value, seed: Value, reduction: str = "mean",
                                     ignore_index=None) -> Value:
        """The node list of LossGradientRules.indexCategorical (:172-228).  `seed` is the output
        cotangent: a scalar for "mean" / "sum", one value per row for "none"."""
        rows, classes = logits.shape
        if ignore_index is None:
            p = self._categorical_probabilities(logits)
        safe = self.scalar_min(self.scalar_max(labels, 0), classes - 1)
        hot = self.where(self.one_hot(safe, classes), self._ones(logits.shape), self._zeros(logits.shape))
        if ignore_index is None:
            scale = self.expand_dims(self._restore(seed, rows, reduction), 1)
            return self.mul(self.sub(p, hot), scale)
        delta = self.scalar_sub(labels, ignore_index)
        ignored = self.eq(delta, self.sub(delta, delta))
        scale = seed if tuple(seed.shape) == (rows,) else self.expand(seed, (rows,))
        if reduction == "mean":     # the rule builds `active` always; unused, the compiler's dead-code pass drops it
            active = self.where(ignored, self._zeros((rows,)), self._ones((rows,)))
            scale = self.div(scale, self.sum_all(active))
        scale = self.expand_dims(scale, 1)
        ignored_row = self.expand_dims(ignored, 1)
        safe_logits = self.where(ignored_row, self._zeros(logits.shape), logits)
        scale = self.where(ignored_row, self._zeros(scale.shape), scale)
        raw = self.mul(self.sub(self._categorical_probabilities(safe_logits), hot), scale)
        return self.where(ignored_row, self._zeros(logits.shape), raw)

    def dense_cross_entropy_backward(self, logits: Value, target: Value, seed: Value, reduction: str = "mean") -> Value:
        """The logits cotangent of LossGradientRules.denseCategorical (:114-145): (p * mass - target) *
        restored, with rows whose targets are all zero taken out."""
        rows, _ = logits.shape
        restored = self.expand_dims(self._restore(seed, rows, reduction), 1)
        zero_target = self.eq(target, self._zeros(target.shape))
        membership = self.sum(self.where(zero_target, self._zeros(target.shape), self._ones(target.shape)), 1, True)
        empty_row = self.eq(membership, self._zeros(membership.shape))
        probabilities = self._categorical_probabilities(self.where(empty_row, self._zeros(logits.shape), logits))
        mass = self.sum(target, 1, True)
        safe_scale = self.where(empty_row, self._zeros(restored.shape), restored)
        raw = self.mul(self.sub(self.mul(probabilities, mass), target), safe_scale)
        return self.where(empty_row, self._zeros(raw.shape), raw)

    def mean_squared_error_backward(self, prediction: Value, target: Value, seed: Value, reduction: str = "mean") -> Value:
        """((p - t) * 2) * restore(gradient) (LossGradientRules.java:77-101): MEAN restores the output
        cotangent as expand(seed) / count, SUM as expand(seed), NONE takes it element by element."""
        doubled = self.scalar_mul(self.sub(prediction, target), 2.0)
        if reduction == "none":
            return self.mul(doubled, seed)
        restored = self.expand(seed, prediction.shape)
        if reduction == "mean":
            ones = self.contiguous(self.expand(self.constant(F32, 1.0), prediction.shape))
            restored = self.div(restored, self.sum_all(ones))
        return self.mul(doubled, restored)

    # ---- serialisation --------------------------------------------------------------------
    def build(self) -> bytes:
        dims: List[int] = []
        strides: List[int] = []
        refs: List[int] = list(self.feeds) + list(self.publications)
        attrs: List[int] = []
        value_blob = b""
        for v in self.values:
            doff = len(dims)
            dims.extend(v.shape)
            soff = 0xFFFFFFFF
            if v.strides is not None:
                soff = len(strides)
                strides.extend(v.strides)
            value_blob += struct.pack("<IIIIQIIQ", v.dtype, len(v.shape), doff, soff, 0, v.role, 0, v.constant_bits & MASK64)
        node_blob = b""
        for n in self.nodes:
            io = len(refs)
            refs.extend(n.inputs)
            oo = len(refs)
            refs.extend(n.outputs)
            ao = len(attrs)
            attrs.extend(n.attrs)
            node_blob += struct.pack("<IIIIIIII", n.op, io, len(n.inputs), oo, len(n.outputs), ao, len(n.attrs), 0)
        body = (value_blob + node_blob + b"".join(struct.pack("<Q", d) for d in dims)
                + b"".join(struct.pack("<q", s) for s in strides) + b"".join(struct.pack("<I", r) for r in refs)
                + b"".join(struct.pack("<Q", a) for a in attrs))
        header = struct.pack("<16I", 0x31554353, 1, 64, 64 + len(body), len(self.values), len(self.nodes), len(dims),
                             len(strides), len(refs), len(attrs), len(self.feeds), len(self.publications), 0, 0, 0, 0)
        return header + body


@dataclass
class MlpGraph:
    image: bytes
    feeds: List[str]            # names in feed order: "x", "target", "seed", "w0", "b0", ...
    publications: List[str]     # "output" | "loss", "dw0", "db0", ...
    shapes: dict


def mlp_inference_graph(dims: Sequence[int], batch, arg_max: bool = False, bias: bool = True,
                        activation: str = "relu", dtype: int = F32) -> MlpGraph:
    """Model.compute of a Linear/activation stack (ModelBuilder.linear().relu() / .tanh() / .sigmoid()):
    feeds x then (w, b) per layer; publishes the last layer's output (and its row arg-max when asked).
    `batch` is the row count, or the tuple of leading dimensions of an input [batch.., features]
    (Linear applies to the last dimension, Tensor.java:1270-1365).  `dtype` is the storage type of input,
    parameters and output: FLOAT32, or BFLOAT16 / FLOAT16 (FLOAT32 working type, one narrowing per node)."""
    g = GraphBuilder()
    lead = tuple(batch) if isinstance(batch, (tuple, list)) else (int(batch),)
    if arg_max and len(lead) != 1:
        raise ValueError("row arg-max needs a [batch, features] input")
    batch = lead[0]
    x = g.feed(dtype, lead + (dims[0],))
    names, shapes = ["x"], {"x": lead + (dims[0],)}
    a = x
    params = []
    for l in range(len(dims) - 1):
        w = g.feed(dtype, (dims[l + 1], dims[l]))
        names.append(f"w{l}")
        shapes[f"w{l}"] = w.shape
        b = None
        if bias:
            b = g.feed(dtype, (dims[l + 1],))
            names.append(f"b{l}")
            shapes[f"b{l}"] = b.shape
        params.append((w, b))
    for l, (w, b) in enumerate(params):
        _, z = g.linear(a, w, b)
        a = g.activation(activation, z) if l + 2 < len(dims) else z
    g.publish(a)
    pubs = ["output"]
    shapes["output"] = a.shape
    if arg_max:
        g.publish(g.arg_max(a, 1))
        pubs.append("arg_max")
        shapes["arg_max"] = (batch,)
    return MlpGraph(g.build(), names, pubs, shapes)


def mlp_training_graph(dims: Sequence[int], batch: int, loss: str = "ce", label_dtype: int = I32, bias: bool = True,
                       publish_activations: bool = False, activation: str = "relu") -> MlpGraph:
    """The TRAINING_STEP graph TrainingSession compiles: forward, objective, and one gradient per
    parameter in trainingParameters() order (weight, bias per layer), published after the loss
    (TrainingSession.java:953-987).  Feeds: x, target, seed, then (w, b) per layer."""
    g = GraphBuilder()
    layers = len(dims) - 1
    x = g.feed(F32, (batch, dims[0]))
    target = g.feed(label_dtype, (batch,)) if loss == "ce" else g.feed(F32, (batch, dims[-1]))
    seed = g.feed(F32, ())
    names = ["x", "target", "seed"]
    shapes = {"x": x.shape, "target": target.shape, "seed": ()}
    params = []
    for l in range(layers):
        w = g.feed(F32, (dims[l + 1], dims[l]))
        names.append(f"w{l}")
        shapes[f"w{l}"] = w.shape
        b = None
        if bias:
            b = g.feed(F32, (dims[l + 1],))
            names.append(f"b{l}")
            shapes[f"b{l}"] = b.shape
        params.append((w, b))
    acts, zs, wts = [x], [], []
    a = x
    for l, (w, b) in enumerate(params):
        wt, z = g.linear(a, w, b)
        wts.append(wt)
        zs.append(z)
        a = g.activation(activation, z) if l + 1 < layers else z
        acts.append(a)
    if loss == "ce":
        objective = g.index_cross_entropy(a, target)
        dz = g.index_cross_entropy_backward(a, target, seed)
    else:
        objective = g.mean_squared_error(a, target)
        dz = g.mean_squared_error_backward(a, target, seed)
    g.publish(objective)
    grads = [None] * (2 * layers)
    for l in range(layers - 1, -1, -1):
        dx, dw, db = g.linear_backward(acts[l], wts[l], dz, need_dx=l > 0, bias=bias)
        grads[2 * l], grads[2 * l + 1] = dw, db
        if l > 0:
            dz = g.activation_backward(activation, zs[l - 1], acts[l], dx)
    pubs = ["loss"]
    shapes["loss"] = ()
    for l in range(layers):
        g.publish(grads[2 * l])
        pubs.append(f"dw{l}")
        shapes[f"dw{l}"] = grads[2 * l].shape
        if bias:
            g.publish(grads[2 * l + 1])
            pubs.append(f"db{l}")
            shapes[f"db{l}"] = grads[2 * l + 1].shape
    if publish_activations:          # hidden activations, for checks that need the device's own ReLU gates
        for l in range(1, layers):
            g.publish(acts[l])
            pubs.append(f"a{l}")
            shapes[f"a{l}"] = acts[l].shape
    return MlpGraph(g.build(), names, pubs, shapes)
