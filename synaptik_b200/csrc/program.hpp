// Program image ("SCU1") and the in-memory graph it decodes to.  Host-only: no CUDA types.
//
// The image is this backend's private, little-endian description of one backend partition, in
// the spirit of the Metal library's "SM22" image (modules/backend/metal/macos-arm64/README.md,
// "ABI version 7": header, value descriptors, node descriptors, dimension / stride / reference /
// attribute pools).  The Java partition finalizer would serialise the CompiledNode list it is
// handed (modules/prepare/.../BackendPartitionFinalizer.java:20-45) into it unchanged: one node
// per reference operation, PERMUTE / EXPAND as view-producing nodes, splat scalar constants as
// constant values (PrepareContext constants).
//
// Layout (all integers little-endian):
//   header          16 x u32 : magic 'SCU1' (0x31554353), schema 1, header bytes 64, total bytes,
//                              value count, node count, dimension count, stride count,
//                              reference count, attribute count, feed count, publication count,
//                              4 reserved zero words
//   values          value_count x 40 bytes : u32 dtype, u32 rank, u32 dimension offset,
//                              u32 stride offset (0xffffffff = dense row-major), u64 storage offset
//                              in elements, u32 role (0 intermediate, 1 feed, 2 splat constant),
//                              u32 reserved, u64 constant bits (binary64 for F32, int64 otherwise)
//   nodes           node_count x 32 bytes : u32 operation, u32 input reference offset, u32 input
//                              count, u32 output reference offset, u32 output count, u32 attribute
//                              offset, u32 attribute count, u32 reserved
//   dimensions      dimension_count x u64
//   strides         stride_count x i64 (element strides)
//   references      reference_count x u32 : feed values, then publication values, then the
//                              per-node input / output lists
//   attributes      attribute_count x u64
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace syn {

enum Status : int32_t {
    OK = 0, INVALID_ARGUMENT = 1, NO_DEVICE = 2, NO_STREAM = 3, ALLOCATION_FAILED = 4,
    RANGE_OUT_OF_BOUNDS = 5, COPY_FAILED = 6, INTERNAL_ERROR = 7, UNSUPPORTED_SHAPE = 8,
    GRAPH_COMPILATION_FAILED = 9, INCOMPATIBLE_RESOURCE = 10, EXECUTION_FAILED = 11,
    KERNEL_COMPILATION_FAILED = 12, UNSUPPORTED_OPERATION = 13, TIMEOUT = 14, COMM_FAILED = 15
};

// BF16 / F16 are storage types (DataType.BFLOAT16 / FLOAT16 of the reference): raw 16-bit patterns in memory,
// a FLOAT32 working type inside every node, one narrowing (round to nearest even; BFLOAT16 NaN -> 0x7FC0,
// BFloat16Bits.java:17-29) of each node's result (CpuScalarReferenceKernel.java:93-115).
enum class DType : uint32_t { F32 = 1, I32 = 2, I64 = 3, BOOL = 4, BF16 = 5, F16 = 6 };
inline int dtype_bytes(DType t) { return t == DType::F32 || t == DType::I32 ? 4 : t == DType::I64 ? 8 : (t == DType::BF16 || t == DType::F16) ? 2 : 1; }
inline bool dtype_low(DType t) { return t == DType::BF16 || t == DType::F16; }
inline bool dtype_floating(DType t) { return t == DType::F32 || dtype_low(t); }

// Operation wire codes: one per reference operation kind on the dense-MLP path
// (modules/model/.../tensor/Tensor.java expression builders; node lists in
// modules/compiler/.../LossGradientRules.java:77-101,172-243, ElementwiseGradientRules.java:99-101,210,
// LinearAlgebraGradientRules.java:97-104).
enum class Op : uint32_t {
    PERMUTE = 1, MATMUL = 2, ADD = 3, SUB = 4, MUL = 5, DIV = 6, SCALAR_MUL = 7, SCALAR_MIN = 8,
    SCALAR_MAX = 9, RELU = 10, EXP = 11, GT = 12, WHERE = 13, EXPAND = 14, EXPAND_DIMS = 15,
    CONTIGUOUS = 16, ONE_HOT = 17, MAX = 18, SUM = 19, SUM_TO_SHAPE = 20, SOFTMAX = 21,
    INDEX_CROSS_ENTROPY = 22, MEAN_SQUARED_ERROR = 23, ARG_MAX = 24, TANH = 25, SIGMOID = 26, SILU = 27, IS_INF = 28, GELU_TANH = 29, CLAMP = 30, LT = 31, EQ = 32,
    SCALAR_SUB = 33, DENSE_CROSS_ENTROPY = 34, GELU = 35, ERF = 36
};
const char *op_name(Op op);

enum class Role : uint32_t { INTERMEDIATE = 0, FEED = 1, CONSTANT = 2 };

struct Value {
    DType dtype = DType::F32;
    std::vector<int64_t> shape;
    std::vector<int64_t> strides;      // element strides; dense row-major when the image gave none
    int64_t offset = 0;
    Role role = Role::INTERMEDIATE;
    uint64_t constant_bits = 0;
    int producer = -1;                 // node index, -1 for feeds and constants
    std::vector<int> consumers;        // node indices
    int publication = -1;              // index among publications, -1 if not published
    int feed = -1;
    int64_t elements() const { int64_t n = 1; for (auto d : shape) n *= d; return n; }
    double constant_f64() const;
    int64_t constant_i64() const { return (int64_t)constant_bits; }
    bool is_dense() const;
};

struct Node {
    Op op = Op::ADD;
    std::vector<int> inputs, outputs;
    std::vector<uint64_t> attrs;
    int64_t attr_i(size_t i, int64_t fallback = 0) const { return i < attrs.size() ? (int64_t)attrs[i] : fallback; }
    double attr_f(size_t i) const;
};

struct Program {
    std::vector<Value> values;
    std::vector<Node> nodes;
    std::vector<int> feeds, publications;
};

std::vector<int64_t> dense_strides(const std::vector<int64_t> &shape);

// Decodes and validates an image: bounds of every section, reference ranges, topological order
// (a node reads only feeds, constants and outputs of earlier nodes), one producer per value,
// operation arity, dtypes and shape agreement of every node.  Returns OK,
// GRAPH_COMPILATION_FAILED (malformed), UNSUPPORTED_OPERATION (unknown wire code or a dtype /
// rank outside capability) or UNSUPPORTED_SHAPE, with a message for diagnostics.
Status parse_program(const uint8_t *bytes, uint32_t size, Program &out, std::string &message);

}  // namespace syn
