/*
 * CPU restatement of the Synaptik CPU backend's arithmetic for the dense FP32 MLP path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is compared with; it is
 * never linked into, loaded by, or called from the product library.  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Every function restates one reference routine in plain scalar C, one IEEE binary32 rounding
 * per arithmetic operation (compile with -ffp-contract=off, no fast-math).  Citations give the
 * reference file (path inside the Synaptik project) and line range each function follows.
 *
 * Pinning: the Java reference cannot be built or executed in an image without a JDK, so this
 * restatement is pinned against the reference's own known-answer tests (see tests/golden/):
 * integer MATMUL results, softmax and log-softmax documented values, the dense-target and index
 * cross-entropy answers of the Metal native test, erf special values, the scalar SGD training trace,
 * the Adam multiply-before-divide overflow case and the double-precision Adam oracle of its unit
 * test; and, for the gradient rules, the vectors of the reference's softmax-backward conformance and
 * integration tests (the FLOAT32 recipe with its exactly rounded row sum, non-finite rows, tied
 * extremes, cross-entropy rows at the finite extremes, with infinities, without target mass and under
 * an ignore index), its ERF / GELU extremes and its finite softmax cases.  Parity unpinned (no FLOAT32
 * known answers in the reference's tests; pinned by special values and by the definition restated
 * here): TANH, SIGMOID, SILU, tanh GELU.
 * For arbitrary real-valued GEMM operands the reference's OpenBLAS route is itself unpinned
 * (any OpenBLAS version), so parity there is a stated tolerance, not bit equality.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define SYN_EXPORT __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------ */
/* MATMUL: modules/backend/cpu/.../internal/reference/CpuMatmulReferenceKernel.java:71-93      */
/* (FLOAT32 branch, NumericalForm.SEQUENTIAL chosen by CpuMatmulLowering.java:214,376):         */
/* per output cell sum = 0f; for k ascending: sum = sum + (a*b) with separate roundings;        */
/* K == 1 is a single product.  Operands are addressed through element strides so a PERMUTE     */
/* view (LayoutInference.java:112) costs nothing.                                               */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT void syn_oracle_matmul_f32(int64_t m, int64_t n, int64_t k,
        const float *a, int64_t a_ms, int64_t a_ks,
        const float *b, int64_t b_ks, int64_t b_ns,
        float *c, int64_t c_ms, int64_t c_ns) {
    for (int64_t i = 0; i < m; i++) {
        for (int64_t j = 0; j < n; j++) {
            const float *pa = a + i * a_ms;
            const float *pb = b + j * b_ns;
            float sum = 0.0f;
            if (k == 1) {
                sum = pa[0] * pb[0];
            } else {
                for (int64_t p = 0; p < k; p++) {
                    float prod = pa[p * a_ks] * pb[p * b_ks];
                    sum = sum + prod;
                }
            }
            c[i * c_ms + j * c_ns] = sum;
        }
    }
}

/* Same contraction for a subset of output rows (row_index[r] selects the logical row); used to
 * check very large products on sampled rows.  Output is dense [rows, n]. */
SYN_EXPORT void syn_oracle_matmul_rows_f32(int64_t rows, const int64_t *row_index, int64_t n,
        int64_t k, const float *a, int64_t a_ms, int64_t a_ks,
        const float *b, int64_t b_ks, int64_t b_ns, float *c) {
    for (int64_t r = 0; r < rows; r++) {
        const float *pa = a + row_index[r] * a_ms;
        for (int64_t j = 0; j < n; j++) {
            const float *pb = b + j * b_ns;
            float sum = 0.0f;
            if (k == 1) sum = pa[0] * pb[0];
            else for (int64_t p = 0; p < k; p++) { float prod = pa[p * a_ks] * pb[p * b_ks]; sum = sum + prod; }
            c[r * n + j] = sum;
        }
    }
}

/* RELU: UnaryElementwiseKind.java:184-192, emitted as Math.max(x, +0.0f)
 * (CpuScalarEmitter.java:329-335): negative, -0 and -inf give +0; NaN stays NaN. */
static inline float relu_value(float x) {
    if (x != x) return x;
    return x > 0.0f ? x : 0.0f;
}

SYN_EXPORT void syn_oracle_relu_f32(int64_t count, const float *x, float *y) {
    for (int64_t i = 0; i < count; i++) y[i] = relu_value(x[i]);
}

/* Broadcast bias ADD on rows followed by optional RELU: the MATMUL epilogue order
 * (CpuMatmulIr.java:92-101: ordered bias ADD then the terminal activation). */
SYN_EXPORT void syn_oracle_bias_act_f32(int64_t m, int64_t n, const float *u, const float *bias,
        int relu, float *z_out, float *y_out) {
    for (int64_t i = 0; i < m; i++) for (int64_t j = 0; j < n; j++) {
        float z = u[i * n + j] + (bias ? bias[j] : 0.0f);
        if (z_out) z_out[i * n + j] = z;
        if (y_out) y_out[i * n + j] = relu ? relu_value(z) : z;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* Exactly rounded summation: CpuExactSumEmitter.java:14-21 / CpuAggregateEmitter.java:17-19    */
/* (SUM, SUM_TO_SHAPE accumulate in an exact multi-limb accumulator and round once, RNE).       */
/* Fixed-point superaccumulator: bit 0 of the accumulator has weight 2^-149.                    */
/* ------------------------------------------------------------------------------------------ */
#define ACC_LIMBS 12   /* 12 x 32 bits = 384 bits: 277 value bits + > 64 bits of carry room */
typedef struct { int64_t limb[ACC_LIMBS]; int pending; int nan; int pinf; int ninf; } exact_acc;

static void acc_init(exact_acc *s) { memset(s, 0, sizeof *s); }

static void acc_normalize(exact_acc *s) {
    int64_t carry = 0;
    for (int i = 0; i < ACC_LIMBS; i++) {
        int64_t v = s->limb[i] + carry;
        int64_t low = v & 0xffffffffLL;
        carry = (v - low) >> 32;      /* arithmetic shift of an exact multiple of 2^32 */
        s->limb[i] = low;
    }
    /* the top limb keeps the sign through the final carry */
    s->limb[ACC_LIMBS - 1] += carry << 32;
    s->pending = 0;
}

static void acc_add(exact_acc *s, float x) {
    uint32_t bits; memcpy(&bits, &x, 4);
    uint32_t exponent = (bits >> 23) & 0xff;
    uint32_t fraction = bits & 0x7fffff;
    if (exponent == 0xff) {
        if (fraction) s->nan = 1; else if (bits >> 31) s->ninf = 1; else s->pinf = 1;
        return;
    }
    int64_t mant; int shift;
    if (exponent == 0) { mant = fraction; shift = 0; }
    else { mant = (int64_t)(fraction | 0x800000); shift = (int)exponent - 1; }
    if (mant == 0) return;
    if (bits >> 31) mant = -mant;
    int limb = shift >> 5, off = shift & 31;
    /* mant << off spans at most 24 + 31 = 55 bits: fits one int64 and lands on two limbs */
    int64_t wide = mant * ((int64_t)1 << off);
    int64_t low = wide & 0xffffffffLL;
    s->limb[limb] += low;
    s->limb[limb + 1] += (wide - low) >> 32;
    if (++s->pending >= (1 << 20)) acc_normalize(s);
}

static float acc_round(exact_acc *s) {
    if (s->nan || (s->pinf && s->ninf)) return NAN;
    if (s->pinf) return INFINITY;
    if (s->ninf) return -INFINITY;
    acc_normalize(s);
    int negative = s->limb[ACC_LIMBS - 1] < 0;
    uint32_t mag[ACC_LIMBS];
    if (negative) {   /* two's complement negate across limbs */
        int64_t carry = 1;
        for (int i = 0; i < ACC_LIMBS; i++) {
            int64_t v = ((~s->limb[i]) & 0xffffffffLL) + carry;
            mag[i] = (uint32_t)(v & 0xffffffffLL); carry = v >> 32;
        }
    } else for (int i = 0; i < ACC_LIMBS; i++) mag[i] = (uint32_t)(s->limb[i] & 0xffffffffLL);
    int top = -1;
    for (int i = ACC_LIMBS - 1; i >= 0 && top < 0; i--) if (mag[i]) {
        top = i * 32 + (31 - __builtin_clz(mag[i]));
    }
    if (top < 0) return 0.0f;     /* exact zero sum: +0 (RNE sum of exact zero) */
    /* value = mag * 2^-149; take the 24 leading bits, round to nearest even on the rest */
#define ACC_BIT(p) ((p) < 0 ? 0u : ((mag[(p) >> 5] >> ((p) & 31)) & 1u))
    uint64_t lead = 0;
    int lowbit = top - 23;        /* position of the last kept bit (may be negative: subnormal) */
    if (lowbit < 0) lowbit = 0;
    for (int p = top; p >= lowbit; p--) lead = (lead << 1) | ACC_BIT(p);
    int guard = lowbit > 0 ? (int)ACC_BIT(lowbit - 1) : 0;
    int sticky = 0;
    for (int p = lowbit - 2; p >= 0 && !sticky; p--) sticky |= (int)ACC_BIT(p);
#undef ACC_BIT
    if (guard && (sticky || (lead & 1))) lead++;
    double value = ldexp((double)lead, lowbit - 149);   /* exact: lead < 2^25 */
    float result = (float)value;                        /* exact or overflows to inf */
    return negative ? -result : result;
}

SYN_EXPORT float syn_oracle_exact_sum_f32(int64_t count, const float *x, int64_t stride) {
    exact_acc s; acc_init(&s);
    for (int64_t i = 0; i < count; i++) acc_add(&s, x[i * stride]);
    return acc_round(&s);
}

/* SUM_TO_SHAPE(g,[N]) for a row-broadcast bias (ElementwiseGradientRules.java:99-100,229-236):
 * db[n] = exactly rounded sum over rows of g[m,n]. */
SYN_EXPORT void syn_oracle_colsum_exact_f32(int64_t m, int64_t n, const float *g, float *out) {
    for (int64_t j = 0; j < n; j++) out[j] = syn_oracle_exact_sum_f32(m, g + j, n);
}

/* ------------------------------------------------------------------------------------------ */
/* SOFTMAX and LOG_SOFTMAX: CpuSoftmaxReferenceKernel.java:104-146 (evaluateFloat).             */
/* ------------------------------------------------------------------------------------------ */
static inline float java_max_f32(float a, float b) {   /* Math.max: NaN wins, +0 > -0 */
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? b : a;
    return a > b ? a : b;
}

/* log_kind 0: SOFTMAX, exp(x - max) / sum.  log_kind 1: LOG_SOFTMAX, (x - max) - (float)log(sum),
 * -inf beside a +inf (:114-123), never the logarithm of the rounded softmax. */
static void softmax_rows_f32(int log_kind, int64_t rows, int64_t classes, const float *x, float *out) {
    for (int64_t r = 0; r < rows; r++) {
        const float *v = x + r * classes; float *o = out + r * classes;
        float maximum = -INFINITY; int unshifted = 0;
        for (int64_t c = 0; c < classes; c++) {
            maximum = java_max_f32(maximum, v[c]);
            unshifted |= v[c] == -INFINITY;
        }
        if (maximum == INFINITY) {
            for (int64_t c = 0; c < classes; c++) o[c] = v[c] == INFINITY ? NAN : log_kind ? -INFINITY : 0.0f;
            continue;
        }
        if (unshifted && !(maximum != maximum)) maximum = 0.0f;
        float sum = 0.0f, compensation = 0.0f;
        for (int64_t c = 0; c < classes; c++) {
            float shifted = v[c] - maximum;
            float addend = (float)exp((double)shifted);
            if (unshifted) sum += addend;
            else {
                float adjusted = addend - compensation, temporary = sum + adjusted;
                compensation = (temporary - sum) - adjusted;
                sum = temporary;
            }
        }
        float logarithm = log_kind ? (float)log((double)sum) : 0.0f;
        for (int64_t c = 0; c < classes; c++) {
            float shifted = v[c] - maximum;
            o[c] = log_kind ? shifted - logarithm : (float)exp((double)shifted) / sum;
        }
    }
}

SYN_EXPORT void syn_oracle_softmax_f32(int64_t rows, int64_t classes, const float *x, float *out) {
    softmax_rows_f32(0, rows, classes, x, out);
}

SYN_EXPORT void syn_oracle_log_softmax_f32(int64_t rows, int64_t classes, const float *x, float *out) {
    softmax_rows_f32(1, rows, classes, x, out);
}

/* ------------------------------------------------------------------------------------------ */
/* Index categorical cross entropy with logits, forward:                                        */
/* CpuLossReferenceKernel.java:196-218 (indexCategoricalCrossEntropy), :261-265 (indexSlice),    */
/* :276-288 (logSumExp float): plain '>' maximum, plain sequential float sum, no compensation.   */
/* Returns 0 on success, 1 if a label is outside [0, classes) (the reference throws             */
/* IllegalArgumentException before any write).  per_row may be NULL.                            */
/* ------------------------------------------------------------------------------------------ */
static float log_sum_exp_f32(const float *v, int64_t classes) {
    float maximum = -INFINITY;
    for (int64_t c = 0; c < classes; c++) if (v[c] > maximum) maximum = v[c];
    float sum = 0.0f;
    for (int64_t c = 0; c < classes; c++) {
        float shifted = v[c] - maximum;
        sum += (float)exp((double)shifted);
    }
    return maximum + (float)log((double)sum);
}

SYN_EXPORT int syn_oracle_index_ce_f32(int64_t rows, int64_t classes, const float *logits,
        const int64_t *labels, float *per_row, float *mean_out) {
    for (int64_t r = 0; r < rows; r++) if (labels[r] < 0 || labels[r] >= classes) return 1;
    float sum = 0.0f;
    for (int64_t r = 0; r < rows; r++) {
        const float *v = logits + r * classes;
        float loss = log_sum_exp_f32(v, classes) - v[labels[r]];
        if (per_row) per_row[r] = loss;
        sum += loss;
    }
    if (mean_out) *mean_out = sum / (float)rows;
    return 0;
}

/* The same with an ignore index (CpuLossReferenceKernel.java:196-218,261-265): a row whose label
 * equals `ignore` is tested before the bounds and before its logits are read; NONE gives it 0,
 * SUM and MEAN skip it, and MEAN divides by the number of rows that are left (0 / 0 = NaN when none
 * is).  reduction: 0 NONE (per_row only), 1 MEAN, 2 SUM.  Returns 1 for a label out of bounds. */
SYN_EXPORT int syn_oracle_index_ce_ignore_f32(int64_t rows, int64_t classes, const float *logits,
        const int64_t *labels, int64_t ignore, int reduction, float *per_row, float *reduced_out) {
    for (int64_t r = 0; r < rows; r++) if (labels[r] != ignore && (labels[r] < 0 || labels[r] >= classes)) return 1;
    float sum = 0.0f;
    int64_t count = 0;
    for (int64_t r = 0; r < rows; r++) {
        const float *v = logits + r * classes;
        if (labels[r] == ignore) { if (per_row) per_row[r] = 0.0f; continue; }
        float loss = log_sum_exp_f32(v, classes) - v[labels[r]];
        if (per_row) per_row[r] = loss;
        sum += loss;
        count++;
    }
    if (reduced_out) *reduced_out = reduction == 1 ? sum / (float)count : sum;
    return 0;
}

/* Dense-target categorical cross entropy with logits, forward (CpuLossReferenceKernel.java:129-143,
 * denseSlice :251-259): per row lse = logSumExp, loss = ascending binary32 sum over the classes with a
 * non-zero weight of weight * (lse - logit); MEAN = sum / samples in binary32. */
SYN_EXPORT void syn_oracle_dense_ce_f32(int64_t rows, int64_t classes, const float *logits,
        const float *target, int reduction, float *per_row, float *reduced_out) {
    float sum = 0.0f;
    for (int64_t r = 0; r < rows; r++) {
        const float *v = logits + r * classes, *w = target + r * classes;
        float lse = log_sum_exp_f32(v, classes);
        float loss = 0.0f;
        for (int64_t c = 0; c < classes; c++) {
            float weight = w[c];
            if (weight != 0.0f) { float term = weight * (lse - v[c]); loss += term; }
        }
        if (per_row) per_row[r] = loss;
        sum += loss;
    }
    if (reduced_out) *reduced_out = reduction == 1 ? sum / (float)rows : sum;
}

/* ------------------------------------------------------------------------------------------ */
/* CE backward as the ordinary-node chain of LossGradientRules.java:172-228,239-243,254-267:     */
/* safe = min(max(label,0),C-1); hot = where(oneHot(safe),1,0); scale = expand(seed)/count with  */
/* count = exactly rounded SUM of ones (= rows); p = exp(x - MAX) / SUM(exp(x - MAX)) with MAX   */
/* and SUM aggregate nodes (SUM exactly rounded, no compensation); dlogits = (p - hot) * scale.  */
/* Each node rounds to binary32.  count_override > 0 replaces the row count (data-parallel       */
/* shards divide by the global batch).                                                          */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT void syn_oracle_index_ce_backward_f32(int64_t rows, int64_t classes,
        const float *logits, const int64_t *labels, float seed, int64_t count_override,
        float *dlogits) {
    float count = (float)(count_override > 0 ? count_override : rows);
    float scale = seed / count;
    float *e = (float *)malloc(sizeof(float) * (size_t)classes);
    for (int64_t r = 0; r < rows; r++) {
        const float *v = logits + r * classes; float *d = dlogits + r * classes;
        float maximum = v[0];                       /* aggregate MAX: NaN propagates */
        for (int64_t c = 1; c < classes; c++) maximum = java_max_f32(maximum, v[c]);
        for (int64_t c = 0; c < classes; c++) { float s = v[c] - maximum; e[c] = (float)exp((double)s); }
        float total = syn_oracle_exact_sum_f32(classes, e, 1);
        int64_t safe = labels[r] < 0 ? 0 : labels[r];
        if (safe > classes - 1) safe = classes - 1;
        for (int64_t c = 0; c < classes; c++) {
            float p = e[c] / total;
            float hot = c == safe ? 1.0f : 0.0f;
            float diff = p - hot;
            d[c] = diff * scale;
        }
    }
    free(e);
}

/* ------------------------------------------------------------------------------------------ */
/* MEAN_SQUARED_ERROR forward: CpuLossReferenceKernel.java:67-87; MEAN divides through           */
/* exactCountQuotient (:221-225): the exact rational sum/count rounded once.                     */
/* ------------------------------------------------------------------------------------------ */
static float exact_count_quotient(float value, int64_t count) {
    if (!isfinite(value) || value == 0.0f || count == 0) return value / (float)count;
    /* binary128 holds the 24-bit numerator and < 2^63 denominator quotient to 113 bits; the
       distance of a non-tie quotient from a binary32 tie is far above 2^-113 relative. */
    __float128 q = (__float128)value / (__float128)count;
    return (float)q;
}

SYN_EXPORT float syn_oracle_mse_f32(int64_t count, const float *prediction, const float *target) {
    float sum = 0.0f;
    for (int64_t i = 0; i < count; i++) {
        float difference = prediction[i] - target[i];
        sum += difference * difference;
    }
    return exact_count_quotient(sum, count);
}

/* The SUM reduction of the same kernel (CpuLossReferenceKernel.java:81-86): no quotient. */
SYN_EXPORT float syn_oracle_squared_error_sum_f32(int64_t count, const float *prediction, const float *target) {
    float sum = 0.0f;
    for (int64_t i = 0; i < count; i++) {
        float difference = prediction[i] - target[i];
        sum += difference * difference;
    }
    return sum;
}

/* MSE backward chain, LossGradientRules.java:77-101,254-267:
 * d = ((p - t) * 2) * (expand(seed) / count). */
SYN_EXPORT void syn_oracle_mse_backward_f32(int64_t count, const float *prediction,
        const float *target, float seed, int64_t count_override, float *dprediction) {
    float denominator = (float)(count_override > 0 ? count_override : count);
    float scale = seed / denominator;
    for (int64_t i = 0; i < count; i++) {
        float difference = prediction[i] - target[i];
        float doubled = difference * 2.0f;
        dprediction[i] = doubled * scale;
    }
}

/* RELU backward: ElementwiseGradientRules.java:210: where(z > 0, g, 0) on the pre-activation. */
SYN_EXPORT void syn_oracle_relu_backward_f32(int64_t count, const float *z, const float *g, float *out) {
    for (int64_t i = 0; i < count; i++) out[i] = z[i] > 0.0f ? g[i] : 0.0f;
}

/* ------------------------------------------------------------------------------------------ */
/* ARG_MAX, FIRST_INDEX ties: Tensor.java:4373-4412, CpuArgExtremaEmitter.java:268-318:          */
/* a NaN candidate replaces a non-NaN best (first NaN wins), a numeric candidate never replaces   */
/* a NaN best, larger value wins, equal values keep the first index except +0 replaces -0.        */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT void syn_oracle_argmax_f32(int64_t rows, int64_t classes, const float *x, int64_t *out) {
    for (int64_t r = 0; r < rows; r++) {
        const float *v = x + r * classes;
        int64_t best_index = 0; float best = v[0];
        for (int64_t c = 1; c < classes; c++) {
            float candidate = v[c];
            int update;
            if (candidate != candidate) update = !(best != best);
            else if (best != best) update = 0;
            else if (candidate > best) update = 1;
            else if (candidate != best) update = 0;
            else {
                uint32_t cb, bb; memcpy(&cb, &candidate, 4); memcpy(&bb, &best, 4);
                update = cb != bb && !(cb >> 31);
            }
            if (update) { best = candidate; best_index = c; }
        }
        out[r] = best_index;
    }
}

/* ------------------------------------------------------------------------------------------ */
/* SGD: TrainingParameter.java:622-672 (stageUpdate32).  Returns 0, or 1 when an intermediate    */
/* is non-finite (the reference throws ArithmeticException and leaves all state unchanged;       */
/* this restatement then also leaves the arrays unchanged).                                      */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT int syn_oracle_sgd_f32(int64_t count, float *parameter, const float *gradient,
        float *momentum_buffer, double learning_rate_d, double momentum_d, double dampening_d,
        double weight_decay_d, int nesterov, int64_t completed_steps) {
    float learning_rate = (float)learning_rate_d, momentum = (float)momentum_d;
    float dampening = (float)dampening_d, weight_decay = (float)weight_decay_d;
    float *np = (float *)malloc(sizeof(float) * (size_t)count);
    float *nb = momentum_buffer ? (float *)malloc(sizeof(float) * (size_t)count) : NULL;
    int bad = 0;
    for (int64_t i = 0; i < count && !bad; i++) {
        float p = parameter[i];
        float decay_term = weight_decay * p;
        float adjusted = gradient[i] + decay_term;
        float update = adjusted;
        if (momentum != 0.0f) {
            float updated_momentum;
            if (completed_steps == 0) updated_momentum = adjusted;
            else {
                float momentum_term = momentum * momentum_buffer[i];
                float dampened = (1.0f - dampening) * adjusted;
                updated_momentum = momentum_term + dampened;
            }
            nb[i] = updated_momentum;
            if (nesterov) { float look = momentum * updated_momentum; update = adjusted + look; }
            else update = updated_momentum;
            bad |= !isfinite(updated_momentum);
        } else if (nb) nb[i] = momentum_d != 0.0 ? 0.0f : momentum_buffer[i];
        float scaled = learning_rate * update;
        float candidate = p - scaled;
        np[i] = candidate;
        bad |= !isfinite(p) || !isfinite(decay_term) || !isfinite(adjusted) || !isfinite(update)
                || !isfinite(scaled) || !isfinite(candidate);
    }
    if (!bad) {
        memcpy(parameter, np, sizeof(float) * (size_t)count);
        if (nb) memcpy(momentum_buffer, nb, sizeof(float) * (size_t)count);
    }
    free(np); free(nb);
    return bad;
}

/* ------------------------------------------------------------------------------------------ */
/* Adam / AdamW: TrainingParameter.java:433-525 (stageAdaptive32, stageAdaptiveElement32) with    */
/* coefficients narrowed to binary32 first (AdaptiveCoefficients.java:33-58); bias corrections    */
/* 1f - (float)Math.pow(beta, step) evaluated in double on the narrowed beta; the update is       */
/* (lr * mhat) / (sqrt(vhat) + eps), multiply before divide (AdamOptimizerTest.java:136-162).     */
/* step = completed optimizer steps + 1.  Returns 0, or 1 on a non-finite intermediate (state     */
/* left unchanged, as the reference's staged transaction does).                                  */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT int syn_oracle_adam_f32(int64_t count, float *parameter, const float *gradient,
        float *first, float *second, double lr_d, double beta1_d, double beta2_d, double eps_d,
        double weight_decay_d, int decoupled, int64_t step) {
    float lr = (float)lr_d, b1 = (float)beta1_d, b2 = (float)beta2_d, eps = (float)eps_d;
    float decay = (float)weight_decay_d;
    float correction1 = 1.0f - (float)pow((double)b1, (double)step);
    float correction2 = 1.0f - (float)pow((double)b2, (double)step);
    if (!(correction1 > 0.0f) || !(correction2 > 0.0f) || !isfinite(correction1) || !isfinite(correction2)) return 1;
    float decay_factor = 1.0f;
    if (decoupled) { float decay_scale = lr * decay; decay_factor -= decay_scale; }
    float *np = (float *)malloc(sizeof(float) * (size_t)count);
    float *nm = (float *)malloc(sizeof(float) * (size_t)count);
    float *nv = (float *)malloc(sizeof(float) * (size_t)count);
    int bad = 0;
    for (int64_t i = 0; i < count && !bad; i++) {
        float p = parameter[i], g, base;
        if (decoupled) { base = p * decay_factor; g = gradient[i]; }
        else { float decay_term = decay * p; g = gradient[i] + decay_term; base = p; }
        float first_term = b1 * first[i];
        float first_gradient = (1.0f - b1) * g;
        float m = first_term + first_gradient;
        float squared = g * g;
        float second_term = b2 * second[i];
        float second_gradient = (1.0f - b2) * squared;
        float v = second_term + second_gradient;
        float corrected_first = m / correction1;
        float corrected_second = v / correction2;
        float root = (float)sqrt((double)corrected_second);
        float denominator = root + eps;
        float numerator = lr * corrected_first;
        float update = numerator / denominator;
        float candidate = base - update;
        np[i] = candidate; nm[i] = m; nv[i] = v;
        bad |= !isfinite(p) || !isfinite(base) || !isfinite(g) || !isfinite(first_term)
                || !isfinite(first_gradient) || !isfinite(m) || !isfinite(squared)
                || !isfinite(second_term) || !isfinite(second_gradient) || !isfinite(v)
                || !isfinite(corrected_first) || !isfinite(corrected_second) || !isfinite(root)
                || !(denominator > 0.0f) || !isfinite(denominator) || !isfinite(numerator)
                || !isfinite(update) || !isfinite(candidate);
    }
    if (!bad) {
        memcpy(parameter, np, sizeof(float) * (size_t)count);
        memcpy(first, nm, sizeof(float) * (size_t)count);
        memcpy(second, nv, sizeof(float) * (size_t)count);
    }
    free(np); free(nm); free(nv);
    return bad;
}

SYN_EXPORT uint32_t syn_oracle_version(void) { return 1; }

/* ------------------------------------------------------------------------------------------ */
/* Pending gradient sum of GradientMode.ACCUMULATE / ACCUMULATE_AND_STEP                        */
/* (modules/training/.../TrainingParameter.java:373-390, applied by TrainingSession.java:601-604): */
/* candidate[i] = accumulated[i] + gradient[i], one binary32 addition; every candidate must be   */
/* finite or nothing is committed.  Returns 0, or 1 with the sum left unchanged.                 */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT int syn_oracle_accumulate_f32(int64_t count, float *accumulated, const float *gradient) {
    for (int64_t i = 0; i < count; i++) {
        volatile float candidate = accumulated[i] + gradient[i];
        if (!isfinite(candidate)) return 1;
    }
    for (int64_t i = 0; i < count; i++) {
        volatile float candidate = accumulated[i] + gradient[i];
        accumulated[i] = candidate;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------ */
/* CLAMP (modules/model/.../tensor/Tensor.java:2318-2345): MIN(MAX(x, lo), hi) in that order with  */
/* Math.max / Math.min semantics: NaN propagates, -0 is below +0.                                */
/* ------------------------------------------------------------------------------------------ */
static float java_max_f(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? b : a;
    return a > b ? a : b;
}
static float java_min_f(float a, float b) {
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return signbit(a) ? a : b;
    return a < b ? a : b;
}
SYN_EXPORT void syn_oracle_clamp_f32(int64_t count, const float *x, float lo, float hi, float *y) {
    for (int64_t i = 0; i < count; i++) y[i] = java_min_f(java_max_f(x[i], lo), hi);
}

/* ------------------------------------------------------------------------------------------ */
/* Parity unpinned: the reference's tests hold no FLOAT32 known answers for the four functions    */
/* below; they are pinned by their special values and by this restatement of the definition only. */
/* TANH and SIGMOID on FLOAT32 (modules/backend/cpu/.../reference/CpuScalarReferenceKernel.java   */
/* :1729-1742): the value widened to double, StrictMath.tanh, or the two-branch sigmoid of        */
/* CpuScalarEmitter.java:429-439 (1 / (1 + exp(-x)) for x >= 0, exp(x) / (1 + exp(x)) below and   */
/* for NaN), then one narrowing to float.  glibc stands in for fdlibm as for exp and log.         */
/* SILU (CpuScalarReferenceKernel.java:1236-1241): -inf gives -0; x / (1 + exp(-x)) for x >= 0,    */
/* x * exp(x) / (1 + exp(x)) below and for NaN.                                                  */
/* Tanh GELU (:1224-1229): -inf gives -0; 0.5 x (1 + tanh(sqrt(2 / pi) (x + 0.044715 x^3))).      */
/* Exact GELU (CpuScalarEmitter.java:441-452): -inf gives -0; 0.5 x (1 + erf(x / sqrt 2)); ERF     */
/* (:353-366): erf of the widened value.  The reference's erf is a rational approximation accurate  */
/* to binary64 rounding (CpuScalarReferenceKernel.java:1254-1268: signed zero unchanged, +-1 from     */
/* |x| = 6 on, which is also what erf rounds to in binary64); the C library's erf stands in for it.  */
/* op: 0 = tanh, 1 = sigmoid, 2 = silu, 3 = tanh-approximated GELU, 4 = exact GELU, 5 = erf.        */
/* ------------------------------------------------------------------------------------------ */
SYN_EXPORT void syn_oracle_activation_f32(int op, int64_t count, const float *x, float *y) {
    for (int64_t i = 0; i < count; i++) {
        double v = (double)x[i];
        double r;
        if (op == 0) r = tanh(v);
        else if (op == 1) {
            if (v >= 0.0) r = 1.0 / (1.0 + exp(-v));
            else { double e = exp(v); r = e / (1.0 + e); }
        } else if (op == 2) {
            if (v == -INFINITY) r = -0.0;
            else if (v >= 0.0) r = v / (1.0 + exp(-v));
            else { double e = exp(v); r = v * e / (1.0 + e); }
        } else if (op == 4) {
            if (v == -INFINITY) r = -0.0;
            else r = 0.5 * v * (1.0 + erf(v / sqrt(2.0)));
        } else if (op == 5) {
            r = erf(v);
        } else {
            if (v == -INFINITY) r = -0.0;
            else { double cube = v * v * v; r = 0.5 * v * (1.0 + tanh(sqrt(2.0 / 3.14159265358979323846) * (v + 0.044715 * cube))); }
        }
        y[i] = (float)r;
    }
}
