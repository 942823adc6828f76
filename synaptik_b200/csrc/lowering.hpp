// Lowering of a decoded program to a list of fused launch steps.  Host-only: no CUDA types.
//
// The partition is pattern-matched structurally (never by node position, because the reference's
// exact graph optimisations may fold constants or merge duplicates,
// docs/explanation/packages/execution.md:398-406):
//   * MATMUL -> ADD(row-broadcast bias) -> RELU | TANH | SIGMOID | SILU | GELU_TANH | GELU
//                                                         one GEMM with a bias/activation epilogue
//     (the anchor-epilogue fusion the Metal backend recognises,
//     modules/backend/metal/.../MetalAnchorEpilogueRecognizer.java:70-147); the pre-activation is
//     not stored when its only other readers are GT(z, 0) predicates, which then read the stored
//     activation instead (z > 0 <=> relu(z) > 0 for every binary32 value, NaN and signed zero
//     included)
//   * WHERE(GT(z, 0), g, 0)                                  ReLU backward, folded into the epilogue
//     of the MATMUL that produces g when g has no other reader
//   * the decomposed index-cross-entropy gradient chain of
//     modules/compiler/.../LossGradientRules.java:172-228 together with the forward loss node
//     on the same logits                                     one row kernel (loss, gradient)
//   * PERMUTE / EXPAND / EXPAND_DIMS                         views, no launch
//   * MATMUL whose only reader is a published PERMUTE        written transposed, no copy
// Everything else becomes one launch per node with one binary32 rounding per operation, which is
// exactly the reference's node-by-node arithmetic.
#pragma once
#include <string>
#include <vector>

#include "program.hpp"

namespace syn {

enum class SlotKind : int { FEED = 0, PUBLICATION = 1, SCRATCH = 2, CONSTANT = 3 };

struct View {
    SlotKind slot = SlotKind::SCRATCH;
    int index = -1;                 // feed / publication / scratch / constant index
    int64_t offset = 0;             // in elements
    std::vector<int64_t> shape, strides;
    DType dtype = DType::F32;
    bool dense() const;
};

enum class StepKind : int {
    GEMM, BINARY, SCALAR, UNARY, WHERE, ONE_HOT, COPY, ROW_REDUCE, FULL_SUM, COLSUM, SOFTMAX,
    CROSS_ENTROPY, MSE, ARG_MAX, RELU_BACKWARD, DENSE_CROSS_ENTROPY, DENSE_CE_BACKWARD, SOFTMAX_BACKWARD
};
const char *step_name(StepKind k);

enum class GemmEngine : int { EXACT_SIMT = 0, TENSOR_CORE = 1, NARROW_OUT = 2, NARROW_INNER = 3, NARROW_REDUCE = 4 };
const char *engine_name(GemmEngine e);

struct Step {
    StepKind kind = StepKind::BINARY;
    Op op = Op::ADD;                // BINARY / SCALAR / UNARY / ROW_REDUCE flavour
    int a = -1, b = -1, c = -1;     // input value ids (meaning per kind, see lowering.cpp)
    int out = -1, out2 = -1, out3 = -1;   // output value ids
    int bias = -1, mask = -1;       // GEMM epilogue operands
    bool relu = false;
    int act = 0;                    // GEMM epilogue activation other than ReLU: the wire code of TANH, SIGMOID, SILU, GELU_TANH or GELU
    int64_t m = 0, n = 0, k = 0;    // GEMM extents, or rows / cols of row kernels
    uint64_t scalar_bits = 0;       // SCALAR operand, ONE_HOT depth, loss reduction
    bool batch_contraction = false; // GEMM: a and b are dense [batch.., rows, x] tensors contracted over batch * rows
    int scale_mode = 0;             // CROSS_ENTROPY gradient: 0 seed / rows (MEAN), 1 seed (SUM), 2 seed[row] (NONE)
    bool has_ignore = false;        // CROSS_ENTROPY: rows labelled `ignore` are skipped
    int64_t ignore = 0;
    GemmEngine engine = GemmEngine::EXACT_SIMT;
    int publication_ready = -1;     // >= 0: this step completes that publication (for comm overlap)
    std::vector<int> ready_publications;
    std::vector<int> nodes;         // program nodes this step covers
};

struct Plan {
    std::vector<View> views;                 // one per program value
    std::vector<Step> steps;
    std::vector<int64_t> scratch_bytes;      // per scratch slot
    std::vector<int> constant_values;        // program value id per constant slot
};

struct LoweringOptions {
    int gemm_engine = 0;        // 0 automatic, 1 always exact CUDA-core kernel, 2 tensor cores when the shape allows
};

// Shape test for the tensor-core path: extents the tcgen05 kernel's tiles divide into and
// operand views that the split pass can read (unit stride along one axis).
bool tensor_core_eligible(int64_t m, int64_t n, int64_t k);
// Automatic engine choice: tensor cores only where the product is large enough to matter.
bool tensor_core_preferred(int64_t m, int64_t n, int64_t k);

Status lower_program(const Program &g, const LoweringOptions &options, Plan &plan, std::string &message);
std::string describe_plan(const Program &g, const Plan &plan);

}  // namespace syn
