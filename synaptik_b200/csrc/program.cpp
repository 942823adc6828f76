// Decoder and validator of the "SCU1" program image (layout in program.hpp).
#include "program.hpp"

#include <algorithm>
#include <cstring>
#include <sstream>

namespace syn {

const char *op_name(Op op) {
    switch (op) {
        case Op::PERMUTE: return "PERMUTE"; case Op::MATMUL: return "MATMUL"; case Op::ADD: return "ADD";
        case Op::SUB: return "SUB"; case Op::MUL: return "MUL"; case Op::DIV: return "DIV";
        case Op::SCALAR_MUL: return "SCALAR_MUL"; case Op::SCALAR_MIN: return "SCALAR_MIN";
        case Op::SCALAR_MAX: return "SCALAR_MAX"; case Op::RELU: return "RELU"; case Op::EXP: return "EXP";
        case Op::GT: return "GT"; case Op::WHERE: return "WHERE"; case Op::EXPAND: return "EXPAND";
        case Op::EXPAND_DIMS: return "EXPAND_DIMS"; case Op::CONTIGUOUS: return "CONTIGUOUS";
        case Op::ONE_HOT: return "ONE_HOT"; case Op::MAX: return "MAX"; case Op::SUM: return "SUM";
        case Op::SUM_TO_SHAPE: return "SUM_TO_SHAPE"; case Op::SOFTMAX: return "SOFTMAX";
        case Op::INDEX_CROSS_ENTROPY: return "INDEX_CATEGORICAL_CROSS_ENTROPY_WITH_LOGITS";
        case Op::MEAN_SQUARED_ERROR: return "MEAN_SQUARED_ERROR"; case Op::ARG_MAX: return "ARG_MAX";
        case Op::TANH: return "TANH"; case Op::SIGMOID: return "SIGMOID"; case Op::SILU: return "SILU";
        case Op::IS_INF: return "IS_INF"; case Op::GELU_TANH: return "GELU_TANH_APPROXIMATION";
        case Op::CLAMP: return "CLAMP"; case Op::LT: return "LT"; case Op::EQ: return "EQ";
        case Op::SCALAR_SUB: return "SCALAR_SUB"; case Op::GELU: return "GELU"; case Op::ERF: return "ERF";
        case Op::DENSE_CROSS_ENTROPY: return "DENSE_CATEGORICAL_CROSS_ENTROPY_WITH_LOGITS";
    }
    return "?";
}

double Value::constant_f64() const { double d; std::memcpy(&d, &constant_bits, 8); return d; }
double Node::attr_f(size_t i) const { double d = 0; if (i < attrs.size()) std::memcpy(&d, &attrs[i], 8); return d; }

std::vector<int64_t> dense_strides(const std::vector<int64_t> &shape) {
    std::vector<int64_t> s(shape.size());
    int64_t run = 1;
    for (int i = (int)shape.size() - 1; i >= 0; i--) { s[i] = run; run *= shape[i]; }
    return s;
}

bool Value::is_dense() const {
    auto d = dense_strides(shape);
    for (size_t i = 0; i < shape.size(); i++) if (shape[i] != 1 && strides[i] != d[i]) return false;
    return true;
}

namespace {

struct Reader {
    const uint8_t *p; uint32_t size;
    uint32_t u32(uint64_t off) const { uint32_t v; std::memcpy(&v, p + off, 4); return v; }
    uint64_t u64(uint64_t off) const { uint64_t v; std::memcpy(&v, p + off, 8); return v; }
};

bool broadcastable(const std::vector<int64_t> &a, const std::vector<int64_t> &b, std::vector<int64_t> &out) {
    size_t r = a.size() > b.size() ? a.size() : b.size();
    out.assign(r, 1);
    for (size_t i = 0; i < r; i++) {
        int64_t da = i < r - a.size() ? 1 : a[i - (r - a.size())];
        int64_t db = i < r - b.size() ? 1 : b[i - (r - b.size())];
        if (da != db && da != 1 && db != 1) return false;
        out[i] = da == 1 ? db : da;
    }
    return true;
}

bool expands_to(const std::vector<int64_t> &from, const std::vector<int64_t> &to) {
    if (from.size() > to.size()) return false;
    for (size_t i = 0; i < from.size(); i++) {
        int64_t d = from[from.size() - 1 - i], t = to[to.size() - 1 - i];
        if (d != t && d != 1) return false;
    }
    return true;
}

#define FAIL(status, text) do { std::ostringstream os_; os_ << text; message = os_.str(); return status; } while (0)

Status check_node(const Program &g, int index, std::string &message) {
    const Node &n = g.nodes[index];
    auto in = [&](size_t i) -> const Value & { return g.values[n.inputs[i]]; };
    auto out = [&](size_t i) -> const Value & { return g.values[n.outputs[i]]; };
    auto need = [&](size_t ins, size_t outs) { return n.inputs.size() == ins && n.outputs.size() == outs; };
    const char *name = op_name(n.op);
    std::vector<int64_t> shape;
    switch (n.op) {
        case Op::PERMUTE: {
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            size_t r = in(0).shape.size();
            if (n.attrs.size() != r || out(0).shape.size() != r) FAIL(GRAPH_COMPILATION_FAILED, name << ": permutation rank");
            std::vector<bool> seen(r, false);
            for (size_t i = 0; i < r; i++) {
                uint64_t a = n.attrs[i];
                if (a >= r || seen[a]) FAIL(GRAPH_COMPILATION_FAILED, name << ": not a permutation");
                seen[a] = true;
                if (out(0).shape[i] != in(0).shape[a]) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            }
            if (out(0).dtype != in(0).dtype) FAIL(GRAPH_COMPILATION_FAILED, name << ": dtype");
            return OK;
        }
        case Op::MATMUL:
            if (!need(2, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (!dtype_floating(in(0).dtype) || in(1).dtype != in(0).dtype || out(0).dtype != in(0).dtype)
                FAIL(UNSUPPORTED_OPERATION, name << ": operands and result of one floating type (FLOAT32, BFLOAT16, FLOAT16)");
            if (dtype_low(in(0).dtype) && (in(0).shape.size() != 2 || in(1).shape.size() != 2))
                FAIL(UNSUPPORTED_OPERATION, name << ": 16-bit operands only of rank 2");
            if (in(0).shape.size() == 2 && in(1).shape.size() == 2) {
                if (out(0).shape.size() != 2 || in(0).shape[1] != in(1).shape[0] || out(0).shape[0] != in(0).shape[0] || out(0).shape[1] != in(1).shape[1])
                    FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            } else {
                // leading batch dimensions broadcast right-aligned (Tensor.java:1075-1096)
                const size_t ra = in(0).shape.size(), rb = in(1).shape.size();
                if (ra < 2 || rb < 2 || ra > 4 || rb > 4) FAIL(UNSUPPORTED_SHAPE, name << ": operand rank outside 2..4");
                std::vector<int64_t> batch_a(in(0).shape.begin(), in(0).shape.end() - 2), batch_b(in(1).shape.begin(), in(1).shape.end() - 2);
                if (!broadcastable(batch_a, batch_b, shape)) FAIL(GRAPH_COMPILATION_FAILED, name << ": batch dimensions do not broadcast");
                shape.push_back(in(0).shape[ra - 2]); shape.push_back(in(1).shape[rb - 1]);
                if (in(0).shape[ra - 1] != in(1).shape[rb - 2] || shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            }
            if (in(0).shape.back() < 1) FAIL(UNSUPPORTED_SHAPE, name << ": empty contraction");
            if (out(0).elements() < 1) FAIL(UNSUPPORTED_SHAPE, name << ": empty result");
            return OK;
        case Op::ADD: case Op::SUB: case Op::MUL: case Op::DIV: case Op::GT: case Op::LT: case Op::EQ:
            if (!need(2, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != in(1).dtype) FAIL(GRAPH_COMPILATION_FAILED, name << ": operand dtypes differ");
            // integer operands (labels against an ignore index) only for SUB and EQ
            // 16-bit storage for the four arithmetic nodes (FLOAT32 working type, one narrowing)
            if (in(0).dtype != DType::F32 && !((in(0).dtype == DType::I32 || in(0).dtype == DType::I64) && (n.op == Op::SUB || n.op == Op::EQ))
                && !(dtype_low(in(0).dtype) && (n.op == Op::ADD || n.op == Op::SUB || n.op == Op::MUL || n.op == Op::DIV)))
                FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32 operands (SUB and EQ also INT32 / INT64; ADD, SUB, MUL, DIV also BFLOAT16 / FLOAT16)");
            if (out(0).dtype != ((n.op == Op::GT || n.op == Op::LT || n.op == Op::EQ) ? DType::BOOL : in(0).dtype)) FAIL(GRAPH_COMPILATION_FAILED, name << ": result dtype");
            if (!broadcastable(in(0).shape, in(1).shape, shape) || shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": broadcast shape");
            if (shape.size() > 4) FAIL(UNSUPPORTED_SHAPE, name << ": rank above 4");
            return OK;
        case Op::SCALAR_MUL: case Op::SCALAR_MIN: case Op::SCALAR_MAX: case Op::SCALAR_SUB:
            if (!need(1, 1) || n.attrs.size() != 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != out(0).dtype || in(0).shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape or dtype");
            if (in(0).dtype == DType::BOOL || (n.op == Op::SCALAR_MUL && in(0).dtype != DType::F32)) FAIL(UNSUPPORTED_OPERATION, name << ": dtype");
            return OK;
        case Op::CLAMP:
            if (!need(1, 1) || n.attrs.size() != 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            if (in(0).shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        case Op::IS_INF:
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            if (out(0).dtype != DType::BOOL || in(0).shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": result");
            return OK;
        case Op::RELU: case Op::EXP: case Op::TANH: case Op::SIGMOID: case Op::SILU: case Op::GELU_TANH: case Op::GELU: case Op::ERF:
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (out(0).dtype != in(0).dtype) FAIL(GRAPH_COMPILATION_FAILED, name << ": dtype");
            if (in(0).dtype != DType::F32 && !(dtype_low(in(0).dtype) && n.op != Op::EXP && n.op != Op::ERF))
                FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32 (the activations also BFLOAT16 / FLOAT16)");
            if (in(0).shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        case Op::WHERE: {
            if (!need(3, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::BOOL || in(1).dtype != DType::F32 || in(2).dtype != DType::F32 || out(0).dtype != DType::F32)
                FAIL(UNSUPPORTED_OPERATION, name << ": needs BOOL, FLOAT32, FLOAT32");
            std::vector<int64_t> partial;
            if (!broadcastable(in(0).shape, in(1).shape, partial) || !broadcastable(partial, in(2).shape, shape) || shape != out(0).shape)
                FAIL(GRAPH_COMPILATION_FAILED, name << ": broadcast shape");
            if (shape.size() > 4) FAIL(UNSUPPORTED_SHAPE, name << ": rank above 4");
            return OK;
        }
        case Op::EXPAND:
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != out(0).dtype || !expands_to(in(0).shape, out(0).shape)) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape or dtype");
            return OK;
        case Op::EXPAND_DIMS: {
            if (!need(1, 1) || n.attrs.size() != 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            shape = in(0).shape;
            if (n.attrs[0] > shape.size()) FAIL(GRAPH_COMPILATION_FAILED, name << ": axis");
            shape.insert(shape.begin() + (long)n.attrs[0], 1);
            if (shape != out(0).shape || in(0).dtype != out(0).dtype) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape or dtype");
            return OK;
        }
        case Op::CONTIGUOUS:
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != out(0).dtype || in(0).shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape or dtype");
            return OK;
        case Op::ONE_HOT:
            if (!need(1, 1) || n.attrs.size() != 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if ((in(0).dtype != DType::I32 && in(0).dtype != DType::I64) || out(0).dtype != DType::BOOL) FAIL(UNSUPPORTED_OPERATION, name << ": needs integer indices and a BOOL result");
            shape = in(0).shape; shape.push_back((int64_t)n.attrs[0]);
            if (shape != out(0).shape || (int64_t)n.attrs[0] < 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        case Op::MAX: case Op::SUM: {
            if (!need(1, 1) || n.attrs.size() != 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            int64_t axis = (int64_t)n.attrs[0];
            if (axis == -1) {                       // complete reduction to a scalar
                if (n.op != Op::SUM) FAIL(UNSUPPORTED_OPERATION, name << ": complete reduction only for SUM");
                if (out(0).elements() != 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
                return OK;
            }
            if (axis < 0 || axis >= (int64_t)in(0).shape.size()) FAIL(GRAPH_COMPILATION_FAILED, name << ": axis");
            if (axis != (int64_t)in(0).shape.size() - 1) FAIL(UNSUPPORTED_SHAPE, name << ": only the last axis");
            shape = in(0).shape;
            if (n.attrs[1]) shape[axis] = 1; else shape.erase(shape.begin() + axis);
            if (shape != out(0).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            if (in(0).shape[axis] < 1) FAIL(UNSUPPORTED_SHAPE, name << ": empty axis");
            return OK;
        }
        case Op::SUM_TO_SHAPE:
            if (!need(1, 1)) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            // the broadcast-reversing reduction over leading dimensions: the result's dimensions are the
            // input's trailing ones (leading result dimensions of 1 allowed), e.g. [M,N] -> [N] for a
            // row-broadcast bias, [B,T,N] -> [N], [B,K,N] -> [K,N]
            {
                std::vector<int64_t> target = out(0).shape;
                while (target.size() > 1 && target.front() == 1) target.erase(target.begin());
                const std::vector<int64_t> &src = in(0).shape;
                if (target.empty() || target.size() >= src.size() || !std::equal(target.begin(), target.end(), src.end() - (long)target.size()))
                    FAIL(UNSUPPORTED_SHAPE, name << ": only sums over leading dimensions");
            }
            return OK;
        case Op::SOFTMAX:
            // attributes: axis, then optionally the kind of the family (0 SOFTMAX, 1 LOG_SOFTMAX)
            if (!need(1, 1) || n.attrs.size() < 1 || n.attrs.size() > 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (n.attr_i(1) != 0 && n.attr_i(1) != 1) FAIL(UNSUPPORTED_OPERATION, name << ": unknown kind");
            if (in(0).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            if (in(0).shape != out(0).shape || in(0).shape.empty()) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            if ((int64_t)n.attrs[0] != (int64_t)in(0).shape.size() - 1) FAIL(UNSUPPORTED_SHAPE, name << ": only the last axis");
            return OK;
        case Op::INDEX_CROSS_ENTROPY:
            if (!need(2, 1) || n.attrs.size() < 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || (in(1).dtype != DType::I32 && in(1).dtype != DType::I64) || out(0).dtype != DType::F32)
                FAIL(UNSUPPORTED_OPERATION, name << ": needs FLOAT32 logits and INT32/INT64 targets");
            if (in(0).shape.size() != 2 || in(1).shape.size() != 1 || in(1).shape[0] != in(0).shape[0] || (int64_t)n.attrs[0] != 1)
                FAIL(UNSUPPORTED_SHAPE, name << ": only [rows, classes] logits with class axis 1");
            // attributes: class axis, reduction (0 NONE = one loss per row, 1 MEAN, 2 SUM), has-ignore-index, ignore index
            if (n.attrs[1] > 2 || n.attr_i(2) < 0 || n.attr_i(2) > 1) FAIL(UNSUPPORTED_OPERATION, name << ": unknown reduction or ignore flag");
            if (n.attrs[1] == 0 ? (out(0).shape.size() != 1 || out(0).shape[0] != in(0).shape[0]) : out(0).elements() != 1)
                FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        case Op::DENSE_CROSS_ENTROPY:
            // attributes: class axis, reduction (0 NONE = one loss per row, 1 MEAN, 2 SUM)
            if (!need(2, 1) || n.attrs.size() < 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || in(1).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            if (in(0).shape.size() != 2 || in(1).shape != in(0).shape || (int64_t)n.attrs[0] != 1)
                FAIL(UNSUPPORTED_SHAPE, name << ": only [rows, classes] logits and targets with class axis 1");
            if (in(0).shape[0] < 1 || in(0).shape[1] < 1) FAIL(UNSUPPORTED_SHAPE, name << ": empty extent");
            if (n.attrs[1] > 2) FAIL(UNSUPPORTED_OPERATION, name << ": unknown reduction");
            if (n.attrs[1] == 0 ? (out(0).shape.size() != 1 || out(0).shape[0] != in(0).shape[0]) : out(0).elements() != 1)
                FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        case Op::MEAN_SQUARED_ERROR:
            if (!need(2, 1) || n.attrs.size() < 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (in(0).dtype != DType::F32 || in(1).dtype != DType::F32 || out(0).dtype != DType::F32) FAIL(UNSUPPORTED_OPERATION, name << ": only FLOAT32");
            // reduction: 0 NONE (per-element result), 1 MEAN, 2 SUM
            if (n.attrs[0] > 2) FAIL(UNSUPPORTED_OPERATION, name << ": unknown reduction");
            if (in(0).shape != in(1).shape) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            if (n.attrs[0] == 0 ? out(0).shape != in(0).shape : out(0).elements() != 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": result shape");
            return OK;
        case Op::ARG_MAX: {
            if (!need(1, 1) || n.attrs.size() != 2) FAIL(GRAPH_COMPILATION_FAILED, name << ": arity");
            if (!dtype_floating(in(0).dtype) || out(0).dtype != DType::I64) FAIL(UNSUPPORTED_OPERATION, name << ": needs a floating input and an INT64 result");
            int64_t axis = (int64_t)n.attrs[0];
            if (in(0).shape.size() != 2 || axis != 1) FAIL(UNSUPPORTED_SHAPE, name << ": only [rows, classes] with axis 1");
            if (in(0).shape[1] < 1) FAIL(GRAPH_COMPILATION_FAILED, name << ": empty axis");
            if (out(0).elements() != in(0).shape[0]) FAIL(GRAPH_COMPILATION_FAILED, name << ": shape");
            return OK;
        }
    }
    FAIL(UNSUPPORTED_OPERATION, "unknown operation wire code " << (uint32_t)n.op);
}

}  // namespace

Status parse_program(const uint8_t *bytes, uint32_t size, Program &g, std::string &message) {
    if (!bytes || size < 64) FAIL(GRAPH_COMPILATION_FAILED, "image shorter than its header");
    Reader r{bytes, size};
    if (r.u32(0) != 0x31554353u) FAIL(GRAPH_COMPILATION_FAILED, "bad magic");
    if (r.u32(4) != 1) FAIL(GRAPH_COMPILATION_FAILED, "unsupported schema " << r.u32(4));
    if (r.u32(8) != 64 || r.u32(12) != size) FAIL(GRAPH_COMPILATION_FAILED, "header or total byte count disagrees");
    uint64_t nv = r.u32(16), nn = r.u32(20), nd = r.u32(24), ns = r.u32(28), nr = r.u32(32), na = r.u32(36);
    uint64_t nf = r.u32(40), np = r.u32(44);
    for (int w = 12; w < 16; w++) if (r.u32(4 * w)) FAIL(GRAPH_COMPILATION_FAILED, "reserved header word is not zero");
    uint64_t off_v = 64, off_n = off_v + nv * 40, off_d = off_n + nn * 32, off_s = off_d + nd * 8;
    uint64_t off_r = off_s + ns * 8, off_a = off_r + nr * 4, end = off_a + na * 8;
    if (end != size) FAIL(GRAPH_COMPILATION_FAILED, "section sizes do not add up to the image size");
    if (nf + np > nr) FAIL(GRAPH_COMPILATION_FAILED, "feed/publication lists exceed the reference pool");
    if (nv == 0 || nv > (1u << 20) || nn > (1u << 20)) FAIL(GRAPH_COMPILATION_FAILED, "value or node count out of range");

    g = Program();
    g.values.resize(nv);
    for (uint64_t i = 0; i < nv; i++) {
        uint64_t o = off_v + i * 40;
        Value &v = g.values[i];
        uint32_t dt = r.u32(o), rank = r.u32(o + 4), doff = r.u32(o + 8), soff = r.u32(o + 12);
        if (dt < 1 || dt > 6) FAIL(UNSUPPORTED_OPERATION, "value " << i << ": data type code " << dt);
        if (rank > 8) FAIL(UNSUPPORTED_SHAPE, "value " << i << ": rank above 8");
        if ((uint64_t)doff + rank > nd) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << ": dimensions out of range");
        v.dtype = (DType)dt;
        int64_t total = 1;
        for (uint32_t a = 0; a < rank; a++) {
            uint64_t d = r.u64(off_d + ((uint64_t)doff + a) * 8);
            if (d > (1ull << 40)) FAIL(UNSUPPORTED_SHAPE, "value " << i << ": extent too large");
            v.shape.push_back((int64_t)d);
            total *= (int64_t)d;
            if (total > (1ll << 46)) FAIL(UNSUPPORTED_SHAPE, "value " << i << ": too many elements");
        }
        if (soff == 0xffffffffu) v.strides = dense_strides(v.shape);
        else {
            if ((uint64_t)soff + rank > ns) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << ": strides out of range");
            for (uint32_t a = 0; a < rank; a++) {
                int64_t s = (int64_t)r.u64(off_s + ((uint64_t)soff + a) * 8);
                if (s < 0) FAIL(UNSUPPORTED_SHAPE, "value " << i << ": negative stride");
                v.strides.push_back(s);
            }
        }
        v.offset = (int64_t)r.u64(o + 16);
        if (v.offset < 0) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << ": storage offset");
        uint32_t role = r.u32(o + 24);
        if (role > 2) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << ": role");
        v.role = (Role)role;
        v.constant_bits = r.u64(o + 32);
        if (v.role == Role::CONSTANT && v.elements() != 1) FAIL(UNSUPPORTED_SHAPE, "value " << i << ": only splat scalar constants");
        if (v.role == Role::CONSTANT && dtype_low(v.dtype)) FAIL(UNSUPPORTED_OPERATION, "value " << i << ": 16-bit constants");
        if (v.role != Role::FEED && (soff != 0xffffffffu && v.role == Role::CONSTANT)) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << ": constant with strides");
    }
    auto ref = [&](uint64_t index) { return r.u32(off_r + index * 4); };
    for (uint64_t i = 0; i < nf; i++) {
        uint32_t v = ref(i);
        if (v >= nv || g.values[v].role != Role::FEED || g.values[v].feed >= 0) FAIL(GRAPH_COMPILATION_FAILED, "feed " << i << " is not a distinct feed value");
        g.values[v].feed = (int)i;
        g.feeds.push_back((int)v);
    }
    for (uint64_t i = 0; i < nv; i++) if (g.values[i].role == Role::FEED && g.values[i].feed < 0) FAIL(GRAPH_COMPILATION_FAILED, "feed value " << i << " is not listed");
    g.nodes.resize(nn);
    std::vector<char> defined(nv, 0);
    for (uint64_t i = 0; i < nv; i++) defined[i] = g.values[i].role != Role::INTERMEDIATE;
    for (uint64_t i = 0; i < nn; i++) {
        uint64_t o = off_n + i * 32;
        Node &n = g.nodes[i];
        n.op = (Op)r.u32(o);
        uint64_t io = r.u32(o + 4), ic = r.u32(o + 8), oo = r.u32(o + 12), oc = r.u32(o + 16), ao = r.u32(o + 20), ac = r.u32(o + 24);
        if (io + ic > nr || oo + oc > nr || ao + ac > na || ic > 8 || oc > 4) FAIL(GRAPH_COMPILATION_FAILED, "node " << i << ": list out of range");
        for (uint64_t k = 0; k < ic; k++) {
            uint32_t v = ref(io + k);
            if (v >= nv || !defined[v]) FAIL(GRAPH_COMPILATION_FAILED, "node " << i << ": input " << k << " is not defined before use");
            n.inputs.push_back((int)v);
            g.values[v].consumers.push_back((int)i);
        }
        for (uint64_t k = 0; k < oc; k++) {
            uint32_t v = ref(oo + k);
            if (v >= nv || defined[v]) FAIL(GRAPH_COMPILATION_FAILED, "node " << i << ": output " << k << " already has a producer");
            defined[v] = 1;
            g.values[v].producer = (int)i;
            n.outputs.push_back((int)v);
        }
        for (uint64_t k = 0; k < ac; k++) n.attrs.push_back(r.u64(off_a + (ao + k) * 8));
        Status s = check_node(g, (int)i, message);
        if (s != OK) { message = "node " + std::to_string(i) + ": " + message; return s; }
    }
    for (uint64_t i = 0; i < nv; i++) if (!defined[i]) FAIL(GRAPH_COMPILATION_FAILED, "value " << i << " has no producer");
    for (uint64_t i = 0; i < np; i++) {
        uint32_t v = ref(nf + i);
        if (v >= nv) FAIL(GRAPH_COMPILATION_FAILED, "publication " << i << " out of range");
        if (g.values[v].publication >= 0) FAIL(GRAPH_COMPILATION_FAILED, "value published twice");
        g.values[v].publication = (int)i;
        g.publications.push_back((int)v);
    }
    if (np == 0) FAIL(GRAPH_COMPILATION_FAILED, "no publication");
    return OK;
}

}  // namespace syn
