// Launchers of the sm_100a kernels.  Every launcher enqueues on the given stream and returns the
// cudaError_t of the launch; none allocates or synchronises.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

#include "program.hpp"

namespace syn {
namespace kern {

// Bits of the device-side error word (one per context, checked after each run).
// ERR_COMM is written by the host, when it gives up on a collective, so that kernels queued behind it see a failure.
enum : int { ERR_LABEL_RANGE = 1, ERR_NON_FINITE = 2, ERR_WAIT_TIMEOUT = 4, ERR_COMM = 8 };

struct Index4 {                 // right-aligned rank-4 iteration space with per-operand element strides
    int64_t shape[4];
    int64_t sa[4], sb[4], sc[4];
};

// ---- generic node-by-node kernels (one binary32 rounding per operation) -----------------------
cudaError_t binary(cudaStream_t s, Op op, const float *a, const float *b, void *out, const Index4 &ix, int64_t total);
// SUB (wrapping) and EQ on INT32 / INT64 operands
cudaError_t binary_int(cudaStream_t s, Op op, DType dtype, const void *a, const void *b, void *out, const Index4 &ix, int64_t total);
cudaError_t scalar_op(cudaStream_t s, Op op, DType dtype, const void *a, void *out, uint64_t scalar_bits, int64_t total);
cudaError_t unary(cudaStream_t s, Op op, const float *a, void *out, int64_t total);      // IS_INF writes BOOL bytes
cudaError_t where(cudaStream_t s, const uint8_t *cond, const float *a, const float *b, float *out, const Index4 &ix, int64_t total);
cudaError_t one_hot(cudaStream_t s, DType index_type, const void *indices, uint8_t *out, int64_t count, int64_t depth);
cudaError_t copy_strided(cudaStream_t s, int element_bytes, const void *src, void *dst, const Index4 &ix, int64_t total);
cudaError_t row_reduce(cudaStream_t s, Op op, const float *x, float *out, int64_t rows, int64_t cols);
cudaError_t full_sum(cudaStream_t s, const float *x, const Index4 &ix, int64_t total, float *out);
cudaError_t argmax_rows(cudaStream_t s, const float *x, int64_t *out, int64_t rows, int64_t cols);
cudaError_t softmax_rows(cudaStream_t s, const float *x, float *out, int64_t rows, int64_t cols, bool log_kind);
// The gradient node lists of both kinds in one pass per row (ReductionGradientRules.java:84-90): y the stored
// forward result, g the upstream gradient, both dense [rows, cols].
cudaError_t softmax_backward_rows(cudaStream_t s, const float *y, const float *g, float *out, int64_t rows, int64_t cols, bool log_kind);
// Squared error (CpuLossReferenceKernel.java:67-87): reduction 0 = per-element (p - t)^2 into out[count],
// 1 = mean, 2 = sum into out[0]; up to 65536 elements the sum is the reference's sequential binary32 one.
// partials: mse_partial_count(count) doubles of scratch (0 for small inputs, which one thread adds in the
// reference's own order); without it large inputs are reduced by a single block.
int64_t mse_partial_count(int64_t count);
cudaError_t mse(cudaStream_t s, int reduction, const float *p, const float *t, int64_t count, float *out, double *partials = nullptr);

// ---- fused memory-bound kernels ----------------------------------------------------------------
// out = gate > 0 ? upstream : 0   (WHERE(GT(z,0), g, 0), ElementwiseGradientRules.java:210)
cudaError_t relu_backward(cudaStream_t s, const float *gate, const float *upstream, float *out, int64_t total);
// Column sums of a dense [rows, cols] matrix, accumulated in binary64 and rounded once.
// partials must hold colsum_partial_count(rows, cols) doubles.
int64_t colsum_partial_count(int64_t rows, int64_t cols);
// With plane_hi / plane_lo set (row pitch `pitch` floats, columns past `cols` already zero) the same pass
// also writes the hi / lo operand planes of g for the tensor-core products that read it; allowed when
// colsum_can_split(g, cols, pitch).
bool colsum_can_split(const float *g, int64_t cols, int64_t pitch);
cudaError_t colsum(cudaStream_t s, const float *g, int64_t rows, int64_t cols, double *partials, float *out,
                   float *plane_hi = nullptr, float *plane_lo = nullptr, int64_t pitch = 0);
// The same two column-sum kernels, with the partial sums kept in a fixed file-scope device array
// (kStaticColsumPartials doubles, 2 MiB, resident on every GPU that loads the library) so that the
// call performs no allocation at all.  `device` must be the current device.  Returns
// cudaErrorInvalidValue when colsum_partial_count(rows, cols) exceeds the array.
constexpr int64_t kStaticColsumPartials = 262144;
cudaError_t colsum_static(cudaStream_t s, int device, const float *g, int64_t rows, int64_t cols, float *out);
// Index cross entropy with logits: per-row loss into row_loss (rows floats of scratch), optional
// gradient (softmax - onehot) * (seed / rows), optional row arg-max, then the mean of row_loss
// into loss_out (optional).  Labels outside [0, cols) set ERR_LABEL_RANGE in *error_word.
// sum_only: loss_out receives the sum of the row losses instead of their mean (reduction SUM); for
// reduction NONE the caller passes its result as row_loss and no loss_out.
cudaError_t cross_entropy(cudaStream_t s, const float *logits, DType label_type, const void *labels,
                          const float *seed, int64_t rows, int64_t cols, float *row_loss, float *loss_out,
                          float *grad_out, int64_t *argmax_out, int *error_word, int sum_only = 0,
                          int has_ignore = 0, int64_t ignore = 0, int scale_mode = 0, float *active_scratch = nullptr);
// active_scratch: one float of device scratch, needed when a gradient with scale_mode 0 is asked for under
// an ignore index (it receives the number of rows that are not ignored, the MEAN rule's divisor).
// scale_mode: what each row of (softmax - onehot) is multiplied by: 0 seed / rows (the MEAN rule), 1 seed
// (SUM), 2 seed[row] (NONE: the cotangent comes one value per row).
// has_ignore: rows whose label equals `ignore` give zero loss and zero gradient, are exempt from the
// label range check and are left out of the MEAN's count (CpuLossReferenceKernel.java:196-218).

// Dense-target categorical cross entropy with logits, forward (CpuLossReferenceKernel.java:129-143):
// row_loss[r] = sum over classes with a non-zero weight of weight * (logsumexp(row) - logit); loss_out
// (when given) their mean, or their sum with sum_only.
cudaError_t dense_cross_entropy(cudaStream_t s, const float *logits, const float *target, int64_t rows, int64_t cols,
                                float *row_loss, float *loss_out, int sum_only);
// Its gradient with respect to the logits (LossGradientRules.java:131-145): (softmax * mass - target) *
// scale per row, zeros for a row without target mass; scale_mode as for cross_entropy.
cudaError_t dense_cross_entropy_backward(cudaStream_t s, const float *logits, const float *target, const float *seed, int64_t rows, int64_t cols,
                                         float *grad, int scale_mode);

// ---- optimizers -----------------------------------------------------------------------------
// A step is a transaction, like the reference's stage / validate / commit (TrainingSession.java:1151-1171,
// TrainingParameter.java:391-409): the kernels read the current parameter, moments and pending sum and
// write CANDIDATES into a second set of arrays (p_out, m_out, v_out); nothing the step reads is
// overwritten.  The host makes the candidate set current by exchanging pointers and exchanges them back
// when the step turns out to have failed.  Every optimizer kernel first looks at the context's error
// word: when an earlier launch has already reported a failure (a label outside its range, a bounded wait
// that ran out, a non-finite intermediate of an earlier step) it writes nothing at all.  A kernel that
// skips or fails records its sequence number in *failed_sequence (atomic minimum), so the host knows the
// first step that did not take place.
// acc: pending gradient sum of the tensor (TrainingParameter.java:373-390), used per `gradient_mode`:
// 0 the step uses g, 2 the step uses acc + g.  The step kernels never write acc; clear_pending zeroes it
// afterwards, and only when the error word is still clear.
struct TensorSlot { const float *p; const float *g; const float *m; const float *v; int64_t count; float *acc; float *p_out, *m_out, *v_out; };
struct SgdArgs { float lr, momentum, dampening, weight_decay; int nesterov, first_step, has_buffer, zero_buffer; int gradient_mode; int sequence; int *failed_sequence; };
struct AdamArgs { float lr, b1, b2, eps, decay, correction1, correction2, decay_factor; int decoupled; int gradient_mode; int sequence; int *failed_sequence; };
cudaError_t sgd_step(cudaStream_t s, const TensorSlot *slots, int slot_count, const SgdArgs &args, int *error_word);
cudaError_t adam_step(cudaStream_t s, const TensorSlot *slots, int slot_count, const AdamArgs &args, int *error_word);
// acc = 0 for every tensor unless the error word is set (one launch, after the step kernel).
cudaError_t clear_pending(cudaStream_t s, const TensorSlot *slots, int slot_count, int *error_word);
// acc = acc + g for every tensor (GradientMode.ACCUMULATE) in two launches: the first only looks for a
// non-finite sum (ERR_NON_FINITE, *failed_sequence), the second adds unless the error word is set.
cudaError_t accumulate_gradients(cudaStream_t s, const TensorSlot *slots, int slot_count, int sequence, int *failed_sequence, int *error_word);
// One block whose only work is a bounded wait on a barrier that nothing signals: the wait gives up after
// limit_ns and the kernel sets ERR_WAIT_TIMEOUT and returns normally.  It runs the same wait routine as
// the tensor-core GEMMs, whose limit is fixed at two seconds.
cudaError_t wait_probe(cudaStream_t s, uint64_t limit_ns, int *error_word);
// `blocks` blocks that each hold one SM (all of its shared memory) for `hold_ns`, then end by themselves.
cudaError_t occupy(cudaStream_t s, int blocks, uint64_t hold_ns);

// ---- GEMM -------------------------------------------------------------------------------------
struct GemmEpilogue {
    const float *bias = nullptr;        // [n], added to every row
    int act = 0;                        // activation applied to z: 0 none, else the wire code of RELU, TANH, SIGMOID,
                                        // SILU, GELU_TANH or GELU (the CPU backend's epilogue vocabulary, CpuMatmulIr.java:96-101)
    const float *gate = nullptr;        // dense [m,n]: out = gate > 0 ? z : 0
    float *second = nullptr;            // dense [m,n]: when set, `out` receives z and `second` act(z)
    // tensor-core kernel only: also write the hi/lo operand planes of the result (the activation when
    // act is set) for later GEMMs, [m, plane_ld]
    float *plane_hi = nullptr, *plane_lo = nullptr; int64_t plane_ld = 0;
};
// Exact CUDA-core product: every output cell is the reference's ascending-k chain of separately
// rounded multiply and add (CpuMatmulReferenceKernel.java:71-93), operands and result strided.
cudaError_t gemm_exact(cudaStream_t s, int64_t m, int64_t n, int64_t k,
                       const float *a, int64_t a_ms, int64_t a_ks, const float *b, int64_t b_ks, int64_t b_ns,
                       float *c, int64_t c_ms, int64_t c_ns, const GemmEpilogue &ep);

// Streaming kernels for products with one extent of at most 16 (kernels_skinny.cu).  The
// *_supported predicates are pure host functions used by the lowering.
//   narrow_out    C[m, n<=16] = A[m,k] (row-major, lda) . W[n,k]^T (rows ldw) (+ bias, ReLU)
//   narrow_inner  C[m, n] (row-major, ldc) = A[m, k<=16] . B[k, n] (row-major, ldb), optional gate; exact chain
//   narrow_reduce D[i, j<=16] = sum_r S[r, i] * T[r, j]  (S rows lds, i contiguous), two-phase, fixed order
bool narrow_out_supported(int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldw);
cudaError_t gemm_narrow_out(cudaStream_t s, int sm_count, int64_t m, int64_t n, int64_t k, const float *a, int64_t lda,
                            const float *w, int64_t ldw, const float *bias, int relu, float *c, int64_t c_ms, int64_t c_ns);
bool narrow_inner_supported(int64_t m, int64_t n, int64_t k, int64_t ldb, int64_t ldc);
cudaError_t gemm_narrow_inner(cudaStream_t s, int64_t m, int64_t n, int64_t k, const float *a, int64_t lda,
                              const float *b, int64_t ldb, const float *gate, float *c, int64_t ldc);
bool narrow_reduce_supported(int64_t wide, int64_t n, int64_t depth, int64_t lds);
int64_t narrow_reduce_partial_floats(int64_t wide, int64_t n, int64_t depth);
cudaError_t gemm_narrow_reduce(cudaStream_t s, int64_t wide, int64_t n, int64_t depth, const float *src, int64_t lds,
                               const float *t, int64_t ldt, float *partial, float *out, int64_t stride_wide, int64_t stride_narrow);

// Tensor-core path.  split_planes writes hi = tf32(x) and lo = tf32(x - hi) of a row-major
// [rows, cols] matrix (row stride rs, unit column stride) into two [rows, pitch] planes whose padding
// columns are zero.  A GEMM operand with `extent` rows (m or n) and contraction length k is given
// either as K-major planes [extent, padded_k(k)] or, when the operand's storage is contiguous along
// its rows instead, as MN-major planes [k, padded_k(extent)]; the kernel reads both forms directly,
// so no operand is ever transposed in memory.  The product is D[m,n] = sum_k P[m,k] * Q[n,k].
int64_t padded_k(int64_t k);
// Row pitch (floats) of a plane with k_padded columns: a pitch that is a multiple of 2 KB gets one more
// 128-byte line so that the rows of a tile do not all fall on the same L2 sets.
int64_t plane_pitch(int64_t k_padded);
cudaError_t split_planes(cudaStream_t s, const float *src, int64_t rows, int64_t cols, int64_t rs,
                         float *hi, float *lo, int64_t pitch);
struct TcOperand { const float *hi = nullptr, *lo = nullptr; int64_t pitch = 0; int mn_major = 0; };
struct TensorCoreGemm;       // opaque: tensor maps and launch geometry prepared once per plan step
// mode: bit 0 = FP32 promotion of partial sums, bit 1 = two-SM tiles where the shape fills them,
// bit 2 = the launch will have no epilogue work (bias, gate, activation, second output, planes), so the
// contraction may be split into slices whose partial products are added by a second kernel; such a
// GEMM needs tc_gemm_workspace_floats(g) floats of scratch at launch.  Bits 8-15: k-blocks (of 32 contraction
// steps) per tensor-memory partial sum of the promoted kernels, 0 = the default (16, or 8 from K = 8192 on).
TensorCoreGemm *tc_gemm_prepare(const TcOperand &p, const TcOperand &q, int64_t m, int64_t n, int64_t k,
                                int sm_count, int mode, int *status);
void tc_gemm_release(TensorCoreGemm *g);
int64_t tc_gemm_workspace_floats(const TensorCoreGemm *g);
int tc_gemm_launches(const TensorCoreGemm *g);
// The product's write-out goes through shared memory and TMA stores (two-SM kernel, unsliced, 16-byte rows)
// when its result arrays are 16-byte aligned: further arrays written from the epilogue are then cheap.
bool tc_gemm_staged_shape(const TensorCoreGemm *g);
// A two-SM product, not cut into slices, whose tiles are at most one per SM pair: it cannot rebalance when
// another kernel holds some of the SMs.
bool tc_gemm_single_wave(const TensorCoreGemm *g);
// unit_counter (optional, two-SM products only): a device int that is zero when the kernel starts; the
// pairs then take their tiles from it one by one instead of by a fixed assignment.
cudaError_t tc_gemm_launch(cudaStream_t s, const TensorCoreGemm *g, float *d, int64_t ldd, const GemmEpilogue &ep, float *workspace,
                           int *unit_counter, int *error_word);

// ---- 16-bit storage (BFLOAT16 = kind 1, FLOAT16 = kind 2), FLOAT32 working type ---------------------
// Every node narrows its result once (round to nearest even); a fused MATMUL -> ADD(bias) -> activation
// narrows after each of the three, as the separate nodes would.  Buffers hold raw 16-bit patterns.
// Exact product: the reference's ascending-k FLOAT32 chain over the widened operands, any strides.
cudaError_t gemm_exact_low(cudaStream_t s, int kind, int64_t m, int64_t n, int64_t k, const void *a, int64_t a_ms, int64_t a_ks,
                           const void *b, int64_t b_ks, int64_t b_ns, void *c, int64_t c_ms, int64_t c_ns,
                           const void *bias, int act, void *second);
// Tensor-core product C[m, n] = A[m, k] . W[n, k]^T on K-major operands (rows lda / ldw elements apart,
// multiples of 8; 16-byte aligned bases), result rows ldc apart; bias [n], activation wire code, optional
// second output as for the FP32 epilogue.  chunk_steps: contraction steps per tensor-memory partial sum
// (0 = default).  The tensor maps are encoded from the pointers on every launch.
bool low_gemm_supported(int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldw, int64_t ldc);
cudaError_t low_gemm_launch(cudaStream_t s, int kind, int sm_count, int64_t m, int64_t n, int64_t k, const void *a, int64_t lda,
                            const void *w, int64_t ldw, void *c, int64_t ldc, const void *bias, int act, void *second,
                            int chunk_steps, int *error_word);
// Element-wise nodes and the row arg-max on 16-bit storage.
cudaError_t binary_low(cudaStream_t s, int kind, Op op, const void *a, const void *b, void *out, const Index4 &ix, int64_t total);
cudaError_t unary_low(cudaStream_t s, int kind, Op op, const void *a, void *out, int64_t total);
cudaError_t argmax_rows_low(cudaStream_t s, int kind, const void *x, int64_t *out, int64_t rows, int64_t cols);

}  // namespace kern
}  // namespace syn
