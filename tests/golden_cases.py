"""The reference-held vectors for the softmax / cross-entropy gradient rules and the activation
extremes (tests/golden/reference_known_answers.json, each entry citing the reference test that pins
it), written once as checks against a small backend interface, so that the CPU checker
(test_oracle_golden.py) and the device (test_gpu_parity.py) are held to the very same expectations.

A backend provides, on FLOAT32 arrays:
    softmax(x, log) -> y                                   rows along axis 1
    softmax_backward(y, g, log) -> dx
    softmax_with_backward(x, g, log) -> (y, dx)            one program: forward, then the rule on the saved y
    index_ce(logits, labels, reduction, ignore, label_dtype) -> objective (scalar, or per-row for "none")
    index_ce_backward(logits, labels, seed, reduction, ignore, label_dtype) -> dlogits
    dense_ce(logits, target, reduction) -> objective
    dense_ce_backward(logits, target, seed, reduction) -> dlogits
    unary(name, x) -> y                                    "erf" | "gelu"
`seed` is the upstream cotangent of the (reduced) loss: a scalar, or one value per row for "none".
"""
import json
import math
import os

import numpy as np

GOLDEN = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")))
F32_MAX = np.float32(3.4028234663852886e+38)


def vals(seq, shape=None) -> np.ndarray:
    a = np.array([float(v) if isinstance(v, str) else v for v in np.asarray(seq, dtype=object).ravel()], dtype=np.float32)
    return a.reshape(shape if shape is not None else np.asarray(seq, dtype=object).shape)


def bits(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def same_bits_or_nan(got, want) -> bool:
    got, want = np.asarray(got, dtype=np.float32), np.asarray(want, dtype=np.float32)
    nan = np.isnan(want)
    return bool(np.all(np.isnan(got[nan])) and np.array_equal(bits(got[~nan]), bits(want[~nan])))


def exact_row_sum(row) -> np.float32:
    """The exactly rounded FLOAT32 sum (the tests use BigDecimal, then floatValue())."""
    return np.float32(math.fsum(float(v) for v in row))


def recipe(y, g, log, sums=None) -> np.ndarray:
    """The FLOAT32 recipe of CpuSoftmaxBackwardConformanceTest.check: one rounding per operation."""
    y, g = np.asarray(y, dtype=np.float32), np.asarray(g, dtype=np.float32)
    out = np.empty_like(y)
    with np.errstate(all="ignore"):
        for r in range(y.shape[0]):
            if sums is not None:
                total = np.float32(sums[r])
            else:
                total = exact_row_sum(g[r]) if log else exact_row_sum((g[r] * y[r]).astype(np.float32))
            for c in range(y.shape[1]):
                if log:
                    e = np.float32(math.exp(float(y[r, c]))) if not math.isinf(float(y[r, c])) else np.float32(0.0 if y[r, c] < 0 else np.inf)
                    out[r, c] = np.float32(g[r, c] - np.float32(e * total))
                else:
                    out[r, c] = np.float32(y[r, c] * np.float32(g[r, c] - total))
    return out


def check_softmax_backward_recipe(b):
    case = GOLDEN["softmax_backward_recipe"]
    y = vals(case["y"], case["shape"])
    for g in case["g"]:
        g = vals(g, case["shape"])
        for log in (False, True):
            assert np.array_equal(bits(b.softmax_backward(y, g, log)), bits(recipe(y, g, log))), (log, g)


def check_softmax_backward_nonfinite(b):
    case = GOLDEN["softmax_backward_nonfinite"]
    y, g = vals(case["y"], case["shape"]), vals(case["g"], case["shape"])
    for log in (False, True):
        sums = vals(case["row_sums"]["log_softmax" if log else "softmax"])
        assert same_bits_or_nan(b.softmax_backward(y, g, log), recipe(y, g, log, sums)), log


def check_softmax_backward_through_forward(b):
    case = GOLDEN["softmax_backward_through_forward"]
    for run in case["runs"]:
        x, g = vals(run["x"], case["shape"]), vals(run["g"], case["shape"])
        for log in (False, True):
            saved, dx = b.softmax_with_backward(x, g, log)
            x64 = x.astype(np.float64)
            shifted = x64 - x64.max(axis=1, keepdims=True)
            denominator = np.exp(shifted).sum(axis=1, keepdims=True)
            want = shifted - np.log(denominator) if log else np.exp(shifted) / denominator
            assert np.abs(saved - want).max() <= case["forward_tol"]
            assert np.array_equal(bits(dx), bits(recipe(saved, g, log))), (log, run)


def check_softmax_tied_extremes(b):
    case = GOLDEN["softmax_tied_extremes"]
    x, g = vals(case["x"])[None, :], vals(case["upstream"])[None, :]
    for log in (False, True):
        key = "log_softmax" if log else "softmax"
        saved, dx = b.softmax_with_backward(x, g, log)
        assert np.isfinite(saved[0, 1]) and abs(float(saved[0, 1]) - case["objective"][key]) <= case["objective_tol"]
        assert np.array_equal(bits(dx[0]), bits(vals(case["gradient"][key]))), (key, dx)


def check_ce_finite_extremes(b):
    case = GOLDEN["ce_finite_extremes"]
    logits, want = vals(case["logits"]), vals(case["gradient"])
    for dtype in (np.int32, np.int64):
        labels = np.array(case["labels"], dtype=dtype)
        assert float(b.index_ce(logits, labels, "sum", case["ignore_index"], dtype)) == case["objective"]
        got = b.index_ce_backward(logits, labels, 1.0, "sum", case["ignore_index"], dtype)
        assert np.array_equal(got, want), got
    target = vals(case["dense_target"])
    assert float(b.dense_ce(logits, target, "sum")) == case["objective"]
    assert np.array_equal(b.dense_ce_backward(logits, target, 1.0, "sum"), want)
    case = GOLDEN["dense_ce_extreme_mass_two"]
    logits, target = vals(case["logits"]), vals(case["target"])
    assert float(b.dense_ce(logits, target, "sum")) == case["objective"]
    assert np.array_equal(b.dense_ce_backward(logits, target, 1.0, "sum"), vals(case["gradient"]))


def check_ce_mixed_infinity(b):
    case = GOLDEN["ce_mixed_infinity"]
    logits, target = vals(case["logits"]), vals(case["dense_target"])
    for reduction in ("none", "mean", "sum"):
        seed = np.ones(2, dtype=np.float32) if reduction == "none" else 1.0      # objective = loss.sum() for NONE
        for dtype in (np.int32, np.int64):
            labels = np.array(case["labels"], dtype=dtype)
            assert float(np.sum(b.index_ce(logits, labels, reduction, None, dtype))) == case["objective"], reduction
            assert np.all(b.index_ce_backward(logits, labels, seed, reduction, None, dtype) == 0.0), reduction
        assert float(np.sum(b.dense_ce(logits, target, reduction))) == case["objective"], reduction
        assert np.all(b.dense_ce_backward(logits, target, seed, reduction) == 0.0), reduction


def check_dense_ce_zero_rows(b):
    case = GOLDEN["dense_ce_zero_rows"]
    logits, target = vals(case["logits"]), vals(case["target"])
    for reduction in ("none", "mean", "sum"):
        seed = vals(case["seed"][reduction]) if reduction == "none" else float(case["seed"][reduction])
        got = b.dense_ce_backward(logits, target, seed, reduction)
        scale = case["scale"][reduction]
        assert np.all(got[:4] == 0.0), (reduction, got)
        assert got[4, 0] == np.float32(0.5 * scale) and got[4, 1] == np.float32(-0.5 * scale), (reduction, got)
        assert np.all(np.isfinite(b.dense_ce(logits, target, reduction))), reduction


def check_index_ce_ignored_rows(b):
    case = GOLDEN["index_ce_ignored_rows"]
    logits = vals(case["logits"])
    for dtype in (np.int32, np.int64):
        ignore = int(np.iinfo(dtype).min)
        for reduction in ("none", "mean", "sum"):
            for all_ignored in (False, True):
                labels = np.array([ignore, ignore, ignore, ignore if all_ignored else 0], dtype=dtype)
                seed = np.ones(4, dtype=np.float32) if reduction == "none" else 1.0
                got = b.index_ce_backward(logits, labels, seed, reduction, ignore, dtype)
                assert np.all(got[:3] == 0.0), (reduction, all_ignored, got)
                assert np.array_equal(got[3], np.array([0.0, 0.0] if all_ignored else [-0.5, 0.5], dtype=np.float32)), (reduction, all_ignored, got)
                value = float(np.sum(b.index_ce(logits, labels, reduction, ignore, dtype)))
                if all_ignored and reduction == "mean":
                    assert math.isnan(value)
                elif all_ignored:
                    assert value == 0.0
                else:
                    assert abs(value - float(np.float32(math.log(2)))) <= case["objective_tol"]


def check_ce_active_poison_rows(b):
    case = GOLDEN["ce_active_poison_rows"]
    for poison in case["poisons"]:
        logits = vals([[poison, case["logits_tail"]]])
        assert math.isnan(float(b.index_ce(logits, np.array([case["label"]], dtype=np.int64), "sum", None, np.int64)))
        assert np.all(np.isnan(b.index_ce_backward(logits, np.array([case["label"]], dtype=np.int64), 1.0, "sum", None, np.int64)))
        target = vals(case["dense_target"])
        assert math.isnan(float(b.dense_ce(logits, target, "sum")))
        assert np.all(np.isnan(b.dense_ce_backward(logits, target, 1.0, "sum")))


def check_erf_gelu_extremes(b):
    case = GOLDEN["erf_gelu_extremes"]
    x = vals(case["x"])
    for name in ("erf", "gelu"):
        assert same_bits_or_nan(b.unary(name, x), vals(case[name])), name


def check_softmax_finite_cases(b):
    case = GOLDEN["softmax_finite_cases"]
    for entry in case["cases"]:
        x = vals(entry["x"])[None, :]
        for log in (False, True):
            got, want = b.softmax(x, log)[0], vals(entry["log_softmax" if log else "softmax"])
            if entry.get("exact"):
                assert np.array_equal(got, want), (entry, log, got)
            else:
                assert np.abs(got - want).max() <= case["tol"], (entry, log, got)


ALL_CHECKS = [check_softmax_backward_recipe, check_softmax_backward_nonfinite, check_softmax_backward_through_forward,
              check_softmax_tied_extremes, check_ce_finite_extremes, check_ce_mixed_infinity, check_dense_ce_zero_rows,
              check_index_ce_ignored_rows, check_ce_active_poison_rows, check_erf_gelu_extremes, check_softmax_finite_cases]


# ---- 16-bit storage -------------------------------------------------------------------------------
# A backend additionally provides, on storage bit patterns (uint16) of kind "bf16" / "f16":
#     low_matmul(kind, a_bits [m,k] view, b_bits [k,n] view) -> bits [m,n]   (views may be transposed arrays)
#     low_unary(kind, name, bits) -> bits
def _encode(kind, x):
    """FLOAT32 -> storage bits, as BFloat16Bits.fromFloat / Float16Bits.fromFloat."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if kind == "f16":
        with np.errstate(over="ignore"):
            out = x.astype(np.float16).view(np.uint16).copy()
        out[np.isnan(x)] = 0x7E00
        return out
    raw = x.view(np.uint32)
    upper = raw >> 16
    discarded = raw & np.uint32(0xFFFF)
    upper = upper + ((discarded > 0x8000) | ((discarded == 0x8000) & ((upper & 1) == 1))).astype(np.uint32)
    out = (upper & 0xFFFF).astype(np.uint16)
    out[np.isnan(x)] = 0x7FC0
    return out


def _decode(kind, bits):
    bits = np.ascontiguousarray(bits, dtype=np.uint16)
    return bits.view(np.float16).astype(np.float32) if kind == "f16" else (bits.astype(np.uint32) << 16).view(np.float32)


def check_matmul_mod5_low_precision(b):
    case = GOLDEN["matmul_mod5_low_precision"]
    m, k, n = case["m"], case["k"], case["n"]
    for kind in ("bf16", "f16"):
        for right_transposed in (False, True):
            if right_transposed:        # left [m,k] row-major, right stored as [n,k]
                left = (np.arange(m * k) % 5 - 2).astype(np.float32).reshape(m, k)
                stored = (np.arange(n * k) % 5 - 2).astype(np.float32).reshape(n, k)
                a_bits, b_bits = _encode(kind, left), _encode(kind, stored).T
                want = left.astype(np.int64) @ stored.astype(np.int64).T
            else:                       # left stored as [k,m], right [k,n] row-major
                stored = (np.arange(k * m) % 5 - 2).astype(np.float32).reshape(k, m)
                right = (np.arange(k * n) % 5 - 2).astype(np.float32).reshape(k, n)
                a_bits, b_bits = _encode(kind, stored).T, _encode(kind, right)
                want = stored.astype(np.int64).T @ right.astype(np.int64)
            got = _decode(kind, b.low_matmul(kind, a_bits, b_bits))
            assert np.array_equal(got, want.astype(np.float32)), (kind, right_transposed)


def check_activation_low_extremes(b):
    case = GOLDEN["activation_low_extremes"]
    one, half = np.float32(1.0), np.float32(0.5)
    for kind in ("bf16", "f16"):
        x_bits = _encode(kind, vals(case["x"]))
        for name in case["kinds"]:
            want = []
            for f in _decode(kind, x_bits):
                f = np.float32(f)
                with np.errstate(all="ignore"):
                    if np.isnan(f):
                        r = np.float32(np.nan)
                    elif name == "gelu":
                        r = np.float32(np.copysign(0.0, f)) if f <= 0 else f
                    elif name == "gelu_tanh":
                        if np.isneginf(f):
                            r = np.float32(-0.0)
                        else:
                            cube = np.float32(np.float32(f * f) * f)
                            scale = np.float32(math.sqrt(float(np.float32(np.float32(2.0) / np.float32(math.pi)))))
                            inner = np.float32(scale * np.float32(f + np.float32(np.float32(0.044715) * cube)))
                            r = np.float32(np.float32(half * f) * np.float32(one + np.float32(math.tanh(float(inner)))))
                    elif name == "silu" and np.isneginf(f):
                        r = np.float32(-0.0)
                    else:
                        e = np.float32(math.exp(float(-f if f >= 0 else f))) if np.isfinite(f) else np.float32(0.0)
                        numerator = (one if f >= 0 else e) if name == "sigmoid" else (f if f >= 0 else np.float32(f * e))
                        r = np.float32(numerator / np.float32(one + e))
                want.append(r)
            want_bits = _encode(kind, np.array(want, dtype=np.float32))
            got_bits = b.low_unary(kind, name, x_bits)
            nan = np.isnan(_decode(kind, want_bits))
            assert np.all(np.isnan(_decode(kind, got_bits)[nan])) and np.array_equal(got_bits[~nan], want_bits[~nan]), (kind, name, got_bits, want_bits)


LOW_CHECKS = [check_matmul_mod5_low_precision, check_activation_low_extremes]
