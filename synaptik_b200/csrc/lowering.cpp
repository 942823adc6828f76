// Pattern matching and layout assignment: Program -> Plan (see lowering.hpp for the rules).
//
// Step operand meaning per kind:
//   GEMM           a = left [m,k] view, b = right [k,n] view, bias = [n] or -1, mask = value whose
//                  sign gates the result (ReLU backward) or -1, out = result (pre-activation, or the
//                  activation when relu and the pre-activation is not needed), out2 = activation
//                  when both are stored
//   BINARY         a, b -> out (op = ADD/SUB/MUL/DIV/GT), right-aligned broadcasting by strides
//   SCALAR         a -> out (op = SCALAR_MUL/MIN/MAX, scalar_bits)
//   UNARY          a -> out (op = RELU/EXP/TANH/SIGMOID/SILU/GELU_TANH/GELU/ERF, or IS_INF with a BOOL result)
//   WHERE          a = condition, b, c -> out
//   ONE_HOT        a -> out (scalar_bits = depth)
//   COPY           a (any view) -> out (dense)
//   ROW_REDUCE     a [m,n] -> out [m] (op = MAX or SUM over the last axis)
//   FULL_SUM       a -> out scalar
//   COLSUM         a [m,n] -> out [n]
//   SOFTMAX        a [m,n] -> out
//   CROSS_ENTROPY  a = logits [m,n], b = labels [m], c = seed scalar or -1 -> out = mean loss or -1,
//                  out2 = gradient wrt logits or -1, out3 = row arg-max (INT64) or -1
//   MSE            a, b -> out scalar
//   ARG_MAX        a [m,n] -> out [m] INT64
//   RELU_BACKWARD  a = gate source, b = upstream gradient -> out
#include "lowering.hpp"
#include "kernels.hpp"

#include <algorithm>
#include <cstring>
#include <map>
#include <set>
#include <sstream>

namespace syn {

bool View::dense() const {
    auto d = dense_strides(shape);
    for (size_t i = 0; i < shape.size(); i++) if (shape[i] != 1 && strides[i] != d[i]) return false;
    return true;
}

const char *step_name(StepKind k) {
    switch (k) {
        case StepKind::GEMM: return "gemm"; case StepKind::BINARY: return "binary"; case StepKind::SCALAR: return "scalar";
        case StepKind::UNARY: return "unary"; case StepKind::WHERE: return "where"; case StepKind::ONE_HOT: return "one_hot";
        case StepKind::COPY: return "copy"; case StepKind::ROW_REDUCE: return "row_reduce"; case StepKind::FULL_SUM: return "full_sum";
        case StepKind::COLSUM: return "colsum"; case StepKind::SOFTMAX: return "softmax"; case StepKind::CROSS_ENTROPY: return "cross_entropy"; case StepKind::DENSE_CROSS_ENTROPY: return "dense_cross_entropy"; case StepKind::DENSE_CE_BACKWARD: return "dense_cross_entropy_backward"; case StepKind::SOFTMAX_BACKWARD: return "softmax_backward";
        case StepKind::MSE: return "mse"; case StepKind::ARG_MAX: return "arg_max"; case StepKind::RELU_BACKWARD: return "relu_backward";
    }
    return "?";
}

const char *engine_name(GemmEngine e) {
    switch (e) {
        case GemmEngine::EXACT_SIMT: return "exact_simt"; case GemmEngine::TENSOR_CORE: return "tcgen05_3xtf32";
        case GemmEngine::NARROW_OUT: return "narrow_out"; case GemmEngine::NARROW_INNER: return "narrow_inner";
        case GemmEngine::NARROW_REDUCE: return "narrow_reduce";
    }
    return "?";
}

bool tensor_core_eligible(int64_t m, int64_t n, int64_t k) { return m >= 64 && n >= 64 && k >= 8; }
bool tensor_core_preferred(int64_t m, int64_t n, int64_t k) {
    return tensor_core_eligible(m, n, k) && m >= 128 && k >= 32 && (double)m * (double)n * (double)k >= 64.0 * 1024 * 1024;
}

namespace {

struct Matcher {
    Program &g;
    explicit Matcher(Program &p) : g(p) {}
    const Node *producer(int v, Op op) const {
        int p = g.values[v].producer;
        return p >= 0 && g.nodes[p].op == op ? &g.nodes[p] : nullptr;
    }
    int producer_index(int v) const { return g.values[v].producer; }
    // Follows view-only nodes down to a splat constant; returns the constant's value id or -1.
    int splat_source(int v) const {
        for (int guard = 0; guard < 16; guard++) {
            const Value &val = g.values[v];
            if (val.role == Role::CONSTANT) return v;
            int p = val.producer;
            if (p < 0) return -1;
            Op op = g.nodes[p].op;
            if (op != Op::EXPAND && op != Op::EXPAND_DIMS && op != Op::CONTIGUOUS) return -1;
            v = g.nodes[p].inputs[0];
        }
        return -1;
    }
    bool is_splat(int v, double x) const {
        int c = splat_source(v);
        if (c < 0) return false;
        const Value &val = g.values[c];
        return val.dtype == DType::F32 ? val.constant_f64() == x : (double)val.constant_i64() == x;
    }
    bool only_consumer(int v, int node) const {
        const Value &val = g.values[v];
        return val.publication < 0 && val.consumers.size() == 1 && val.consumers[0] == node;
    }
    // The output cotangent restored on the sample domain (LossGradientRules.restore, :239-252), as the loss
    // gradient chains hold it under their EXPAND_DIMS: DIV(EXPAND(seed), divisor) for MEAN (scale_mode 0;
    // `divisor_ok` checks the divisor and claims its nodes), EXPAND(seed) for SUM (1), or the [rows]
    // cotangent itself for NONE (2).  Claims the nodes it walks through; false when no form fits.
    template <typename DivisorOk>
    bool restored_cotangent(int scale, int64_t rows, std::set<int> &nodes, int &seed, int &scale_mode, DivisorOk divisor_ok) const {
        if (const Node *sdiv = producer(scale, Op::DIV)) {
            nodes.insert(producer_index(scale));
            seed = sdiv->inputs[0];
            if (const Node *ex = producer(seed, Op::EXPAND)) { nodes.insert(producer_index(seed)); seed = ex->inputs[0]; }
            if (g.values[seed].elements() != 1 || g.values[seed].dtype != DType::F32) return false;
            scale_mode = 0;
            return divisor_ok(sdiv->inputs[1]);
        }
        if (const Node *ex = producer(scale, Op::EXPAND)) {
            if (g.values[ex->inputs[0]].elements() != 1 || g.values[ex->inputs[0]].dtype != DType::F32 || splat_source(scale) >= 0) return false;
            nodes.insert(producer_index(scale));
            seed = ex->inputs[0];
            scale_mode = 1;
            return true;
        }
        const Value &sv = g.values[scale];
        if (sv.dtype != DType::F32 || sv.shape.size() != 1 || sv.shape[0] != rows || sv.role == Role::CONSTANT) return false;
        if (sv.role == Role::FEED ? !sv.is_dense() : (sv.producer < 0 || g.nodes[sv.producer].op == Op::PERMUTE || g.nodes[sv.producer].op == Op::EXPAND
                                                      || g.nodes[sv.producer].op == Op::EXPAND_DIMS)) return false;
        seed = scale;
        scale_mode = 2;
        return true;
    }
    // The divisor of the plain MEAN form: the splat constant `rows`, or SUM over `rows` ones.
    bool row_count(int count, int64_t rows, std::set<int> &nodes) const {
        if (is_splat(count, (double)rows)) return true;
        const Node *csum = producer(count, Op::SUM);
        if (!csum || csum->attr_i(0) != -1 || !is_splat(csum->inputs[0], 1.0) || g.values[csum->inputs[0]].elements() != rows) return false;
        nodes.insert(producer_index(count));
        return true;
    }
    // Every value produced inside a matched chain (other than by `final_node`) must stay inside it.  View-only
    // nodes over constants cost nothing and may be shared, so they are not claimed.  Returns the claimed
    // nodes in `claimed` and whether the chain is closed.
    bool claim_closed_chain(const std::set<int> &nodes, int final_node, std::set<int> &claimed) const {
        claimed.clear();
        for (int n : nodes) {
            const Node &node = g.nodes[n];
            const bool view_of_constant = (node.op == Op::EXPAND || node.op == Op::EXPAND_DIMS || node.op == Op::CONTIGUOUS)
                                          && splat_source(node.outputs[0]) >= 0;
            if (!view_of_constant) claimed.insert(n);
        }
        for (int n : claimed) {
            if (n == final_node) continue;
            for (int v : g.nodes[n].outputs) {
                if (g.values[v].publication >= 0) return false;
                for (int c : g.values[v].consumers) if (!nodes.count(c)) return false;
            }
        }
        return true;
    }
};

struct LinearGroup {          // MATMUL [-> ADD bias] [-> RELU] [-> gate by WHERE(GT(.,0),.,0)]
    int matmul = -1, add = -1, relu = -1, where = -1, gt = -1;
    int act = 0;                  // wire code of a fused activation other than ReLU (its node is `relu`)
    int bias = -1, mask = -1;
    int out = -1, out2 = -1;
    int emit_at = -1;
};

struct CrossEntropyGroup {
    int logits = -1, labels = -1, seed = -1, loss = -1, grad = -1, argmax = -1;
    int reduction = 1;                      // of the forward loss node: 0 NONE, 1 MEAN, 2 SUM
    bool has_ignore = false;                // of the forward loss node
    int64_t ignore = 0;
    int scale_mode = 0;                     // of the gradient chain: 0 seed / rows, 1 seed, 2 seed[row]
    bool chain_ignore = false;              // the gradient chain is the ignore-index form (rows left = rows not ignored)
    std::set<int> nodes;
    int emit_at = -1;
};

bool match_ce_backward(Matcher &mt, int mul_index, CrossEntropyGroup &ce) {
    Program &g = mt.g;
    const Node &mul = g.nodes[mul_index];
    if (mul.op != Op::MUL) return false;
    for (int order = 0; order < 2; order++) {
        int lhs = mul.inputs[order], rhs = mul.inputs[1 - order];
        const Node *sub = mt.producer(lhs, Op::SUB);
        if (!sub) continue;
        std::set<int> extra;
        auto through_expand = [&](int v) {      // explicit broadcast nodes are optional in the chain
            while (const Node *ex = mt.producer(v, Op::EXPAND)) { extra.insert(mt.producer_index(v)); v = ex->inputs[0]; }
            return v;
        };
        int p = sub->inputs[0], hot = through_expand(sub->inputs[1]);
        const Node *div = mt.producer(p, Op::DIV);
        if (!div) continue;
        int e = div->inputs[0], s = through_expand(div->inputs[1]);
        const Node *expn = mt.producer(e, Op::EXP);
        const Node *sumn = mt.producer(s, Op::SUM);
        if (!expn || !sumn || sumn->inputs[0] != e || sumn->attr_i(0) != 1 || !sumn->attr_i(1)) continue;
        const Node *shift = mt.producer(expn->inputs[0], Op::SUB);
        if (!shift) continue;
        int logits = shift->inputs[0], mx = through_expand(shift->inputs[1]);
        const Node *maxn = mt.producer(mx, Op::MAX);
        if (!maxn || maxn->inputs[0] != logits || maxn->attr_i(0) != 1 || !maxn->attr_i(1)) continue;
        if (g.values[logits].shape.size() != 2) continue;
        int64_t rows = g.values[logits].shape[0], classes = g.values[logits].shape[1];
        const Node *where = mt.producer(hot, Op::WHERE);
        if (!where || !mt.is_splat(where->inputs[1], 1.0) || !mt.is_splat(where->inputs[2], 0.0)) continue;
        const Node *onehot = mt.producer(where->inputs[0], Op::ONE_HOT);
        if (!onehot || onehot->attr_i(0) != classes) continue;
        int labels = onehot->inputs[0];
        std::set<int> nodes = {mul_index, mt.producer_index(lhs), mt.producer_index(p), mt.producer_index(e),
                               mt.producer_index(s), mt.producer_index(expn->inputs[0]), mt.producer_index(mx),
                               mt.producer_index(hot), mt.producer_index(where->inputs[0])};
        nodes.insert(extra.begin(), extra.end());
        if (const Node *smin = mt.producer(labels, Op::SCALAR_MIN)) {
            const Node *smax = mt.producer(smin->inputs[0], Op::SCALAR_MAX);
            if (smin->attr_i(0) != classes - 1 || !smax || smax->attr_i(0) != 0) continue;
            nodes.insert(mt.producer_index(labels));
            nodes.insert(mt.producer_index(smin->inputs[0]));
            labels = smax->inputs[0];
        }
        if (g.values[labels].shape.size() != 1 || g.values[labels].shape[0] != rows) continue;
        // rhs: [EXPAND] <- EXPAND_DIMS(axis 1) <- the restored cotangent (LossGradientRules.restore):
        // DIV(EXPAND(seed), count) for MEAN, EXPAND(seed) for SUM, the [rows] cotangent itself for NONE
        int scale = rhs;
        if (const Node *ex = mt.producer(scale, Op::EXPAND)) { nodes.insert(mt.producer_index(scale)); scale = ex->inputs[0]; }
        const Node *ed = mt.producer(scale, Op::EXPAND_DIMS);
        if (!ed || ed->attr_i(0) != 1) continue;
        nodes.insert(mt.producer_index(scale));
        scale = ed->inputs[0];
        int seed = -1, scale_mode = 0;
        if (!mt.restored_cotangent(scale, rows, nodes, seed, scale_mode, [&](int count) { return mt.row_count(count, rows, nodes); })) continue;
        std::set<int> claimed;
        if (!mt.claim_closed_chain(nodes, mul_index, claimed)) continue;
        ce.logits = logits; ce.labels = labels; ce.seed = seed; ce.grad = mul.outputs[0]; ce.scale_mode = scale_mode;
        ce.nodes = claimed;
        return true;
    }
    return false;
}

// The same gradient under an ignore index (LossGradientRules.java:203-226): rows whose label equals the
// ignore value are taken out three times over (their logits replaced by zeros, their scale by zero, their
// result by zero), and the MEAN form divides the cotangent by the number of rows that are left.
//   WHERE(ignoredRow, 0, MUL(SUB(p(WHERE(ignoredRow, 0, logits)), hot), WHERE(ignoredRow, 0, EXPAND_DIMS(scale))))
//   ignoredRow = EXPAND_DIMS(ignored), ignored = EQ(delta, SUB(delta, delta)), delta = SCALAR_SUB(labels, ignore)
//   scale = DIV(expand(seed), SUM(WHERE(ignored, 0, 1))) | expand(seed) | the [rows] cotangent
bool match_ce_ignore_backward(Matcher &mt, int where_index, CrossEntropyGroup &ce) {
    Program &g = mt.g;
    const Node &fin = g.nodes[where_index];
    if (fin.op != Op::WHERE || !mt.is_splat(fin.inputs[1], 0.0)) return false;
    const int ignored_row = fin.inputs[0];
    const Node *ird = mt.producer(ignored_row, Op::EXPAND_DIMS);
    if (!ird || ird->attr_i(0) != 1) return false;
    const int ignored = ird->inputs[0];
    const Node *eq = mt.producer(ignored, Op::EQ);
    if (!eq) return false;
    const int delta = eq->inputs[0];
    const Node *zero = mt.producer(eq->inputs[1], Op::SUB);
    const Node *ssub = mt.producer(delta, Op::SCALAR_SUB);
    if (!zero || zero->inputs[0] != delta || zero->inputs[1] != delta || !ssub) return false;
    const int labels = ssub->inputs[0];
    if (g.values[labels].dtype != DType::I32 && g.values[labels].dtype != DType::I64) return false;
    const Node *mul = mt.producer(fin.inputs[2], Op::MUL);
    if (!mul) return false;
    for (int order = 0; order < 2; order++) {
        const int lhs = mul->inputs[order], rhs = mul->inputs[1 - order];
        const Node *sub = mt.producer(lhs, Op::SUB);
        if (!sub) continue;
        const int p = sub->inputs[0], hot = sub->inputs[1];
        const Node *div = mt.producer(p, Op::DIV);
        if (!div) continue;
        const int e = div->inputs[0], s = div->inputs[1];
        const Node *expn = mt.producer(e, Op::EXP);
        const Node *sumn = mt.producer(s, Op::SUM);
        if (!expn || !sumn || sumn->inputs[0] != e || sumn->attr_i(0) != 1 || !sumn->attr_i(1)) continue;
        const Node *shift = mt.producer(expn->inputs[0], Op::SUB);
        if (!shift) continue;
        const int safe_logits = shift->inputs[0], mx = shift->inputs[1];
        const Node *maxn = mt.producer(mx, Op::MAX);
        if (!maxn || maxn->inputs[0] != safe_logits || maxn->attr_i(0) != 1 || !maxn->attr_i(1)) continue;
        const Node *wl = mt.producer(safe_logits, Op::WHERE);
        if (!wl || wl->inputs[0] != ignored_row || !mt.is_splat(wl->inputs[1], 0.0)) continue;
        const int logits = wl->inputs[2];
        if (g.values[logits].shape.size() != 2 || g.values[logits].dtype != DType::F32) continue;
        const int64_t rows = g.values[logits].shape[0], classes = g.values[logits].shape[1];
        if (g.values[labels].shape.size() != 1 || g.values[labels].shape[0] != rows) continue;
        const Node *where_hot = mt.producer(hot, Op::WHERE);
        if (!where_hot || !mt.is_splat(where_hot->inputs[1], 1.0) || !mt.is_splat(where_hot->inputs[2], 0.0)) continue;
        const Node *onehot = mt.producer(where_hot->inputs[0], Op::ONE_HOT);
        if (!onehot || onehot->attr_i(0) != classes) continue;
        const Node *smin = mt.producer(onehot->inputs[0], Op::SCALAR_MIN);
        const Node *smax = smin ? mt.producer(smin->inputs[0], Op::SCALAR_MAX) : nullptr;
        if (!smin || !smax || smin->attr_i(0) != classes - 1 || smax->attr_i(0) != 0 || smax->inputs[0] != labels) continue;
        const Node *ws = mt.producer(rhs, Op::WHERE);
        if (!ws || ws->inputs[0] != ignored_row || !mt.is_splat(ws->inputs[1], 0.0)) continue;
        const int scale1 = ws->inputs[2];
        const Node *ed = mt.producer(scale1, Op::EXPAND_DIMS);
        if (!ed || ed->attr_i(0) != 1) continue;
        const int scale0 = ed->inputs[0];
        std::set<int> nodes = {where_index, mt.producer_index(fin.inputs[2]), mt.producer_index(lhs), mt.producer_index(p), mt.producer_index(e),
                               mt.producer_index(s), mt.producer_index(expn->inputs[0]), mt.producer_index(mx), mt.producer_index(safe_logits),
                               mt.producer_index(hot), mt.producer_index(where_hot->inputs[0]), mt.producer_index(onehot->inputs[0]),
                               mt.producer_index(smin->inputs[0]), mt.producer_index(rhs), mt.producer_index(scale1),
                               mt.producer_index(ignored_row), mt.producer_index(ignored), mt.producer_index(eq->inputs[1]), mt.producer_index(delta)};
        int seed = -1, scale_mode = 0;
        auto rows_left = [&](int count) {       // SUM over WHERE(ignored, 0, 1): the rows that are not ignored
            const Node *csum = mt.producer(count, Op::SUM);
            if (!csum || csum->attr_i(0) != -1) return false;
            const Node *wa = mt.producer(csum->inputs[0], Op::WHERE);
            if (!wa || wa->inputs[0] != ignored || !mt.is_splat(wa->inputs[1], 0.0) || !mt.is_splat(wa->inputs[2], 1.0)) return false;
            nodes.insert(mt.producer_index(count));
            nodes.insert(mt.producer_index(csum->inputs[0]));
            return true;
        };
        if (!mt.restored_cotangent(scale0, rows, nodes, seed, scale_mode, rows_left)) continue;
        std::set<int> claimed;
        if (!mt.claim_closed_chain(nodes, where_index, claimed)) continue;
        ce.logits = logits; ce.labels = labels; ce.seed = seed; ce.grad = fin.outputs[0]; ce.scale_mode = scale_mode;
        ce.chain_ignore = true; ce.ignore = ssub->attr_i(0);
        ce.nodes = claimed;
        return true;
    }
    return false;
}

// Logits cotangent of the dense-target loss (LossGradientRules.java:131-145):
//   WHERE(emptyRow, 0, MUL(SUB(MUL(p(WHERE(emptyRow, 0, logits)), SUM(target)), target), WHERE(emptyRow, 0, restored)))
//   emptyRow = EQ(SUM(WHERE(EQ(target, 0), 0, 1)), 0), restored = EXPAND_DIMS(the cotangent on the sample domain)
struct DenseCrossEntropyGroup { int logits = -1, target = -1, seed = -1, grad = -1, scale_mode = 0; std::set<int> nodes; };

bool match_dense_ce_backward(Matcher &mt, int where_index, DenseCrossEntropyGroup &dg) {
    Program &g = mt.g;
    const Node &fin = g.nodes[where_index];
    if (fin.op != Op::WHERE || !mt.is_splat(fin.inputs[1], 0.0)) return false;
    const int empty_row = fin.inputs[0];
    const Node *eq_empty = mt.producer(empty_row, Op::EQ);
    if (!eq_empty || !mt.is_splat(eq_empty->inputs[1], 0.0)) return false;
    const int membership = eq_empty->inputs[0];
    const Node *msum = mt.producer(membership, Op::SUM);
    if (!msum || msum->attr_i(0) != 1 || !msum->attr_i(1)) return false;
    const Node *member = mt.producer(msum->inputs[0], Op::WHERE);
    if (!member || !mt.is_splat(member->inputs[1], 0.0) || !mt.is_splat(member->inputs[2], 1.0)) return false;
    const Node *eq_zero = mt.producer(member->inputs[0], Op::EQ);
    if (!eq_zero || !mt.is_splat(eq_zero->inputs[1], 0.0)) return false;
    const int target = eq_zero->inputs[0];
    const Node *mul = mt.producer(fin.inputs[2], Op::MUL);
    if (!mul) return false;
    for (int order = 0; order < 2; order++) {
        const int lhs = mul->inputs[order], rhs = mul->inputs[1 - order];
        const Node *sub = mt.producer(lhs, Op::SUB);
        if (!sub || sub->inputs[1] != target) continue;
        const Node *pm = mt.producer(sub->inputs[0], Op::MUL);
        if (!pm) continue;
        int p = -1, mass = -1;
        for (int o = 0; o < 2 && p < 0; o++) {
            const Node *ms = mt.producer(pm->inputs[1 - o], Op::SUM);
            if (ms && ms->inputs[0] == target && ms->attr_i(0) == 1 && ms->attr_i(1) && mt.producer(pm->inputs[o], Op::DIV)) { p = pm->inputs[o]; mass = pm->inputs[1 - o]; }
        }
        if (p < 0) continue;
        const Node *div = mt.producer(p, Op::DIV);
        const int e = div->inputs[0], s = div->inputs[1];
        const Node *expn = mt.producer(e, Op::EXP);
        const Node *sumn = mt.producer(s, Op::SUM);
        if (!expn || !sumn || sumn->inputs[0] != e || sumn->attr_i(0) != 1 || !sumn->attr_i(1)) continue;
        const Node *shift = mt.producer(expn->inputs[0], Op::SUB);
        if (!shift) continue;
        const int safe_logits = shift->inputs[0], mx = shift->inputs[1];
        const Node *maxn = mt.producer(mx, Op::MAX);
        if (!maxn || maxn->inputs[0] != safe_logits || maxn->attr_i(0) != 1 || !maxn->attr_i(1)) continue;
        const Node *wl = mt.producer(safe_logits, Op::WHERE);
        if (!wl || wl->inputs[0] != empty_row || !mt.is_splat(wl->inputs[1], 0.0)) continue;
        const int logits = wl->inputs[2];
        if (g.values[logits].shape.size() != 2 || g.values[logits].dtype != DType::F32 || g.values[target].shape != g.values[logits].shape) continue;
        const int64_t rows = g.values[logits].shape[0];
        const Node *ws = mt.producer(rhs, Op::WHERE);
        if (!ws || ws->inputs[0] != empty_row || !mt.is_splat(ws->inputs[1], 0.0)) continue;
        const Node *ed = mt.producer(ws->inputs[2], Op::EXPAND_DIMS);
        if (!ed || ed->attr_i(0) != 1) continue;
        const int scale0 = ed->inputs[0];
        std::set<int> nodes = {where_index, mt.producer_index(fin.inputs[2]), mt.producer_index(lhs), mt.producer_index(sub->inputs[0]), mt.producer_index(p),
                               mt.producer_index(mass), mt.producer_index(e), mt.producer_index(s), mt.producer_index(expn->inputs[0]), mt.producer_index(mx),
                               mt.producer_index(safe_logits), mt.producer_index(rhs), mt.producer_index(ws->inputs[2]), mt.producer_index(empty_row),
                               mt.producer_index(membership), mt.producer_index(msum->inputs[0]), mt.producer_index(member->inputs[0])};
        int seed = -1, scale_mode = 0;
        if (!mt.restored_cotangent(scale0, rows, nodes, seed, scale_mode, [&](int count) { return mt.row_count(count, rows, nodes); })) continue;
        std::set<int> claimed;
        if (!mt.claim_closed_chain(nodes, where_index, claimed)) continue;
        dg.logits = logits; dg.target = target; dg.seed = seed; dg.grad = fin.outputs[0]; dg.scale_mode = scale_mode;
        dg.nodes = claimed;
        return true;
    }
    return false;
}

}  // namespace

Status lower_program(const Program &source, const LoweringOptions &options, Plan &plan, std::string &message) {
    Program g = source;     // GT predicates may be re-pointed at stored activations
    Matcher mt(g);
    const int node_count = (int)g.nodes.size();
    std::vector<int> covered(node_count, 0);
    std::map<int, std::vector<Step>> emit_at;

    // Nodes nothing observes (no output is published or read by a node that is itself observed) are
    // never launched: marked covered before any pattern looks at them.  The reference's compiler removes
    // such nodes itself; a hand-written image may still hold them.
    {
        std::vector<char> observed(node_count, 0);
        for (int i = node_count - 1; i >= 0; i--) {
            for (int v : g.nodes[i].outputs) {
                if (g.values[v].publication >= 0) observed[i] = 1;
                for (int c : g.values[v].consumers) if (observed[c]) observed[i] = 1;
            }
            if (!observed[i]) covered[i] = 1;
        }
    }

    auto choose_engine = [&](int64_t m, int64_t n, int64_t k) {
        bool tc = options.gemm_engine == 1 ? false : options.gemm_engine == 2 ? tensor_core_eligible(m, n, k) : tensor_core_preferred(m, n, k);
        return tc ? GemmEngine::TENSOR_CORE : GemmEngine::EXACT_SIMT;
    };

    // ---- linear groups ---------------------------------------------------------------------
    std::vector<LinearGroup> linear;
    std::map<int, int> group_of_matmul_output;      // result value -> group index
    for (int i = 0; i < node_count; i++) {
        const Node &mm = g.nodes[i];
        if (mm.op != Op::MATMUL || covered[i]) continue;
        // A left operand with batch dimensions joins a group when it is stored dense (a dense feed or a
        // value some kernel materialises), so that [batch.., rows, k] reads as [batch * rows, k] over the
        // shared rank-2 right operand: Linear on [batch, time, features] keeps its fused epilogue.  Other
        // batched products are lowered per slice further down.
        if (g.values[mm.inputs[1]].shape.size() != 2) continue;
        if (g.values[mm.inputs[0]].shape.size() != 2) {
            const Value &left = g.values[mm.inputs[0]];
            bool stored_dense = left.role == Role::FEED ? left.is_dense() : false;
            if (left.role == Role::INTERMEDIATE && left.producer >= 0) {
                Op producer = g.nodes[left.producer].op;
                stored_dense = producer != Op::PERMUTE && producer != Op::EXPAND && producer != Op::EXPAND_DIMS && producer != Op::CONTIGUOUS;
            }
            if (!stored_dense) continue;
        }
        LinearGroup lg;
        lg.matmul = i;
        lg.emit_at = i;
        int z = mm.outputs[0];
        int64_t n = g.values[z].shape.back();
        if (g.values[z].publication < 0 && g.values[z].consumers.size() == 1) {
            int c = g.values[z].consumers[0];
            const Node &add = g.nodes[c];
            if (add.op == Op::ADD && g.values[add.outputs[0]].shape == g.values[z].shape) {
                int other = add.inputs[0] == z ? add.inputs[1] : add.inputs[0];
                const Value &bv = g.values[other];
                bool row_bias = other != z && bv.elements() == n && !bv.shape.empty() && bv.shape.back() == n
                                && bv.dtype == g.values[z].dtype && (bv.role != Role::INTERMEDIATE ? true : bv.producer < i);
                if (row_bias && (add.inputs[0] == z || add.inputs[1] == z)) {
                    lg.add = c; lg.bias = other; lg.emit_at = c;
                    z = add.outputs[0];
                }
            }
        }
        lg.out = z;
        // activation
        int relu_node = -1;
        for (int c : g.values[z].consumers) if (g.nodes[c].op == Op::RELU) { relu_node = c; break; }
        if (relu_node >= 0) {
            int y = g.nodes[relu_node].outputs[0];
            bool z_needed = g.values[z].publication >= 0;
            std::vector<int> predicates;
            for (int c : g.values[z].consumers) {
                if (c == relu_node) continue;
                const Node &u = g.nodes[c];
                if (u.op == Op::GT && u.inputs[0] == z && mt.is_splat(u.inputs[1], 0.0)) predicates.push_back(c);
                else z_needed = true;
            }
            lg.relu = relu_node;
            if (!z_needed) {
                for (int c : predicates) {
                    g.nodes[c].inputs[0] = y;
                    g.values[y].consumers.push_back(c);
                }
                g.values[z].consumers.assign(1, relu_node);
                lg.out = y;
            } else {
                lg.out2 = y;
            }
        } else {
            // the other activations of the CPU backend's epilogue vocabulary (CpuMatmulIr.java:96-101): the
            // first such reader of z joins the product; z itself is stored as well when anything else reads
            // it (the SILU / GELU gradient rules do) or it is published
            for (int c : g.values[z].consumers) {
                const Op op = g.nodes[c].op;
                if (covered[c] || (op != Op::TANH && op != Op::SIGMOID && op != Op::SILU && op != Op::GELU_TANH && op != Op::GELU)) continue;
                lg.relu = c; lg.act = (int)op;
                const int y = g.nodes[c].outputs[0];
                if (g.values[z].publication < 0 && g.values[z].consumers.size() == 1) lg.out = y;
                else lg.out2 = y;
                break;
            }
        }
        if (lg.add < 0 && lg.relu < 0) group_of_matmul_output[mm.outputs[0]] = (int)linear.size();
        linear.push_back(lg);
    }

    // ---- weight gradient of a Linear over batch dimensions -------------------------------------
    // SUM_TO_SHAPE(MATMUL(swapLastTwo(X), G), [k, n]) with X [batch.., rows, k] and G [batch.., rows, n]
    // both stored dense is one product X^T G contracted over batch * rows.  The per-slice products and
    // their sum over the batch are an unobservable single-use intermediate, so only the order of the
    // additions changes; taken where the joined product runs on the tensor cores (the exact engine keeps
    // the reference's per-slice chains).
    auto stored_dense = [&](int v) {
        const Value &val = g.values[v];
        if (val.role == Role::FEED) return val.is_dense();
        if (val.role != Role::INTERMEDIATE || val.producer < 0) return false;
        Op producer = g.nodes[val.producer].op;
        return producer != Op::PERMUTE && producer != Op::EXPAND && producer != Op::EXPAND_DIMS && producer != Op::CONTIGUOUS;
    };
    for (int i = 0; i < node_count; i++) {
        const Node &sum = g.nodes[i];
        if (sum.op != Op::SUM_TO_SHAPE || covered[i]) continue;
        const Node *mm = mt.producer(sum.inputs[0], Op::MATMUL);
        if (!mm || !mt.only_consumer(sum.inputs[0], i)) continue;
        const Node *swap = mt.producer(mm->inputs[0], Op::PERMUTE);
        if (!swap) continue;
        const int x = swap->inputs[0], up = mm->inputs[1];
        const std::vector<int64_t> &xs = g.values[x].shape, &us = g.values[up].shape;
        const size_t r = xs.size();
        if (r < 3 || us.size() != r || !stored_dense(x) || !stored_dense(up)) continue;
        bool last_two = true;
        for (size_t d = 0; d < r; d++) last_two &= swap->attr_i(d) == (int64_t)(d == r - 2 ? r - 1 : d == r - 1 ? r - 2 : d);
        if (!last_two || !std::equal(xs.begin(), xs.end() - 1, us.begin())) continue;
        if (g.values[sum.outputs[0]].elements() != xs.back() * us.back()) continue;      // all batch dimensions are summed
        const int64_t contraction = g.values[x].elements() / xs.back();
        if (choose_engine(xs.back(), us.back(), contraction) != GemmEngine::TENSOR_CORE) continue;
        Step st;
        st.kind = StepKind::GEMM; st.batch_contraction = true;
        st.a = x; st.b = up; st.out = sum.outputs[0];
        st.m = xs.back(); st.n = us.back(); st.k = contraction;
        st.engine = GemmEngine::TENSOR_CORE;
        st.nodes = {mt.producer_index(sum.inputs[0]), i};
        covered[i] = 1; covered[mt.producer_index(sum.inputs[0])] = 1;
        if (mt.only_consumer(mm->inputs[0], mt.producer_index(sum.inputs[0]))) { covered[mt.producer_index(mm->inputs[0])] = 1; st.nodes.push_back(mt.producer_index(mm->inputs[0])); }
        emit_at[i].push_back(st);
    }

    // ---- ReLU backward: WHERE(GT(z, 0), g, 0) ----------------------------------------------
    std::vector<Step> relu_backward_steps;
    for (int i = 0; i < node_count; i++) {
        const Node &w = g.nodes[i];
        if (w.op != Op::WHERE || covered[i] || !mt.is_splat(w.inputs[2], 0.0)) continue;
        const Node *gt = mt.producer(w.inputs[0], Op::GT);
        if (!gt || !mt.is_splat(gt->inputs[1], 0.0)) continue;
        int gate = gt->inputs[0], upstream = w.inputs[1], result = w.outputs[0];
        if (g.values[gate].shape != g.values[result].shape || g.values[upstream].shape != g.values[result].shape) continue;
        int gt_index = mt.producer_index(w.inputs[0]);
        bool own_gt = mt.only_consumer(w.inputs[0], i);
        // fold into the producing GEMM when the upstream gradient has no other reader
        auto it = group_of_matmul_output.find(upstream);
        if (it != group_of_matmul_output.end() && mt.only_consumer(upstream, i)) {
            LinearGroup &lg = linear[it->second];
            if (lg.add < 0 && lg.relu < 0 && lg.where < 0 && g.values[gate].producer < i) {
                lg.where = i; lg.mask = gate; lg.out = result; lg.emit_at = i;
                if (own_gt) lg.gt = gt_index;
                continue;
            }
        }
        Step st;
        st.kind = StepKind::RELU_BACKWARD; st.a = gate; st.b = upstream; st.out = result;
        st.nodes = {i};
        covered[i] = 1;
        if (own_gt) { covered[gt_index] = 1; st.nodes.push_back(gt_index); }
        emit_at[i].push_back(st);
    }

    for (const LinearGroup &lg : linear) {
        const Node &mm = g.nodes[lg.matmul];
        Step st;
        st.kind = StepKind::GEMM;
        st.a = mm.inputs[0]; st.b = mm.inputs[1];
        st.k = g.values[st.a].shape.back(); st.m = g.values[st.a].elements() / st.k; st.n = g.values[st.b].shape[1];
        st.bias = lg.bias; st.mask = lg.mask; st.relu = lg.relu >= 0 && lg.act == 0; st.act = lg.act;
        st.out = lg.out; st.out2 = lg.out2;
        st.engine = choose_engine(st.m, st.n, st.k);
        for (int n : {lg.matmul, lg.add, lg.relu, lg.where, lg.gt}) if (n >= 0) { covered[n] = 1; st.nodes.push_back(n); }
        emit_at[lg.emit_at].push_back(st);
    }

    // ---- cross entropy ---------------------------------------------------------------------
    std::vector<CrossEntropyGroup> ces;
    for (int i = 0; i < node_count; i++) {
        if (covered[i] || g.nodes[i].op != Op::MUL) continue;
        CrossEntropyGroup ce;
        if (!match_ce_backward(mt, i, ce)) continue;
        bool clash = false;
        for (int n : ce.nodes) clash |= covered[n] != 0;
        if (clash) continue;
        ces.push_back(ce);
        for (int n : ce.nodes) covered[n] = 1;
    }
    for (int i = 0; i < node_count; i++) {
        if (covered[i] || g.nodes[i].op != Op::WHERE) continue;
        CrossEntropyGroup ce;
        if (!match_ce_ignore_backward(mt, i, ce)) continue;
        bool clash = false;
        for (int n : ce.nodes) clash |= covered[n] != 0;
        if (clash) continue;
        ce.has_ignore = true;
        ces.push_back(ce);
        for (int n : ce.nodes) covered[n] = 1;
    }
    // ---- SOFTMAX / LOG_SOFTMAX gradient node lists (ReductionGradientRules.java:84-90) --------------
    //   MUL(y, SUB(g, SUM(MUL(g, y), last axis, keep)))   and   SUB(g, MUL(EXP(y), SUM(g, last axis, keep)))
    for (int i = 0; i < node_count; i++) {
        if (covered[i]) continue;
        const Node &top = g.nodes[i];
        int y = -1, up = -1;
        bool log_kind = false;
        std::set<int> nodes = {i};
        auto row_sum_of = [&](int v, int of) -> const Node * {        // SUM over the last axis, kept, of value `of`
            const Node *sn = mt.producer(v, Op::SUM);
            const size_t r = g.values[of].shape.size();
            return sn && sn->inputs[0] == of && r == 2 && sn->attr_i(0) == 1 && sn->attr_i(1) ? sn : nullptr;
        };
        if (top.op == Op::MUL) {
            for (int order = 0; order < 2 && y < 0; order++) {
                const int yy = top.inputs[order];
                const Node *sub = mt.producer(top.inputs[1 - order], Op::SUB);
                if (!sub) continue;
                const Node *sn = mt.producer(sub->inputs[1], Op::SUM);
                if (!sn) continue;
                const Node *gy = mt.producer(sn->inputs[0], Op::MUL);
                if (!gy || !row_sum_of(sub->inputs[1], sn->inputs[0])) continue;
                const int gg = sub->inputs[0];
                if (!((gy->inputs[0] == gg && gy->inputs[1] == yy) || (gy->inputs[0] == yy && gy->inputs[1] == gg))) continue;
                y = yy; up = gg;
                nodes.insert(mt.producer_index(top.inputs[1 - order])); nodes.insert(mt.producer_index(sub->inputs[1])); nodes.insert(mt.producer_index(sn->inputs[0]));
            }
        } else if (top.op == Op::SUB) {
            const Node *em = mt.producer(top.inputs[1], Op::MUL);
            if (em) for (int order = 0; order < 2 && y < 0; order++) {
                const Node *ex = mt.producer(em->inputs[order], Op::EXP);
                if (!ex || !row_sum_of(em->inputs[1 - order], top.inputs[0])) continue;
                y = ex->inputs[0]; up = top.inputs[0]; log_kind = true;
                nodes.insert(mt.producer_index(top.inputs[1])); nodes.insert(mt.producer_index(em->inputs[order])); nodes.insert(mt.producer_index(em->inputs[1 - order]));
            }
        }
        if (y < 0) continue;
        const Value &yv = g.values[y], &uv = g.values[up];
        if (yv.shape.size() != 2 || uv.shape != yv.shape || g.values[top.outputs[0]].shape != yv.shape || yv.dtype != DType::F32 || uv.dtype != DType::F32) continue;
        bool ok = true;
        for (int n : nodes) {
            ok &= !covered[n];
            if (n == i) continue;
            for (int v : g.nodes[n].outputs) {
                if (g.values[v].publication >= 0) ok = false;
                for (int c : g.values[v].consumers) if (!nodes.count(c)) ok = false;
            }
        }
        const int first = *nodes.begin();
        if (!ok || g.values[y].producer >= first || g.values[up].producer >= first) continue;
        for (int n : nodes) covered[n] = 1;
        Step st;
        st.kind = StepKind::SOFTMAX_BACKWARD;
        st.a = y; st.b = up; st.out = top.outputs[0];
        st.m = yv.shape[0]; st.n = yv.shape[1];
        st.scalar_bits = log_kind ? 1 : 0;
        st.nodes.assign(nodes.begin(), nodes.end());
        emit_at[first].push_back(st);
    }

    for (int i = 0; i < node_count; i++) {
        if (covered[i] || g.nodes[i].op != Op::WHERE) continue;
        DenseCrossEntropyGroup dg;
        if (!match_dense_ce_backward(mt, i, dg)) continue;
        bool clash = false;
        for (int n : dg.nodes) clash |= covered[n] != 0;
        int first = *dg.nodes.begin();
        auto before = [&](int v) { return g.values[v].producer < first; };
        if (clash || !before(dg.logits) || !before(dg.target) || !before(dg.seed)) continue;
        for (int n : dg.nodes) covered[n] = 1;
        Step st;
        st.kind = StepKind::DENSE_CE_BACKWARD;
        st.a = dg.logits; st.b = dg.target; st.c = dg.seed; st.out = dg.grad;
        st.m = g.values[dg.logits].shape[0]; st.n = g.values[dg.logits].shape[1];
        st.scale_mode = dg.scale_mode;
        st.nodes.assign(dg.nodes.begin(), dg.nodes.end());
        emit_at[first].push_back(st);
    }
    for (int i = 0; i < node_count; i++) {
        const Node &n = g.nodes[i];
        if (n.op != Op::INDEX_CROSS_ENTROPY || covered[i]) continue;
        CrossEntropyGroup *host = nullptr;
        // a loss node joins the gradient chain over the same logits and labels with the same ignore index (or none)
        for (auto &ce : ces) if (ce.loss < 0 && ce.logits == n.inputs[0] && ce.labels == n.inputs[1]
                                 && ce.chain_ignore == (n.attr_i(2) != 0) && (!ce.chain_ignore || ce.ignore == n.attr_i(3))) { host = &ce; break; }
        if (!host) { ces.emplace_back(); host = &ces.back(); host->logits = n.inputs[0]; host->labels = n.inputs[1]; }
        host->loss = n.outputs[0];
        host->reduction = (int)n.attrs[1];
        host->has_ignore = n.attr_i(2) != 0; host->ignore = n.attr_i(3);
        host->nodes.insert(i);
        covered[i] = 1;
    }
    // a row ARG_MAX over the same logits rides in the same pass (the row is already in registers)
    for (int i = 0; i < node_count; i++) {
        const Node &n = g.nodes[i];
        if (n.op != Op::ARG_MAX || covered[i]) continue;
        for (auto &ce : ces) if (ce.argmax < 0 && ce.logits == n.inputs[0] && i > *ce.nodes.begin()) {
            ce.argmax = n.outputs[0];
            ce.nodes.insert(i);
            covered[i] = 1;
            break;
        }
    }
    for (auto &ce : ces) {
        int first = *ce.nodes.begin();
        auto defined_before = [&](int v) { return v < 0 || g.values[v].producer < first; };
        if (!defined_before(ce.logits) || !defined_before(ce.labels) || !defined_before(ce.seed)) {
            message = "cross-entropy inputs are produced after the loss chain starts";
            return GRAPH_COMPILATION_FAILED;
        }
        Step st;
        st.kind = StepKind::CROSS_ENTROPY;
        st.a = ce.logits; st.b = ce.labels; st.c = ce.seed; st.out = ce.loss; st.out2 = ce.grad; st.out3 = ce.argmax;
        st.m = g.values[ce.logits].shape[0]; st.n = g.values[ce.logits].shape[1];
        st.scalar_bits = (uint64_t)ce.reduction;
        st.has_ignore = ce.has_ignore; st.ignore = ce.ignore; st.scale_mode = ce.scale_mode;
        st.nodes.assign(ce.nodes.begin(), ce.nodes.end());
        emit_at[first].push_back(st);
    }

    // ---- dead nodes: whatever no launch, view or publication still reads (e.g. the ones tensor
    // that only the fused loss chain counted) is dropped ----------------------------------------
    {
        std::vector<char> needed(g.values.size(), 0);
        for (int v : g.publications) needed[v] = 1;
        for (auto &entry : emit_at) for (const Step &st : entry.second)
            for (int v : {st.a, st.b, st.c, st.bias, st.mask}) if (v >= 0) needed[v] = 1;
        for (int i = node_count - 1; i >= 0; i--) {
            if (covered[i]) continue;
            bool live = false;
            for (int v : g.nodes[i].outputs) live |= needed[v] != 0;
            if (!live) { covered[i] = 1; continue; }
            for (int v : g.nodes[i].inputs) needed[v] = 1;
        }
    }

    // ---- layout assignment and per-node steps ------------------------------------------------
    plan = Plan();
    plan.views.resize(g.values.size());
    std::vector<char> assigned(g.values.size(), 0);
    auto new_scratch = [&](const Value &v) {
        plan.scratch_bytes.push_back(std::max<int64_t>(v.elements(), 1) * dtype_bytes(v.dtype));
        return (int)plan.scratch_bytes.size() - 1;
    };
    for (size_t i = 0; i < g.values.size(); i++) {
        const Value &v = g.values[i];
        View &w = plan.views[i];
        w.shape = v.shape; w.dtype = v.dtype;
        if (v.role == Role::FEED) { w.slot = SlotKind::FEED; w.index = v.feed; w.offset = v.offset; w.strides = v.strides; assigned[i] = 1; }
        else if (v.role == Role::CONSTANT) {
            w.slot = SlotKind::CONSTANT; w.index = (int)plan.constant_values.size(); w.strides.assign(v.shape.size(), 0);
            plan.constant_values.push_back((int)i); assigned[i] = 1;
        }
    }
    // a MATMUL read only by a published PERMUTE writes straight into that publication, transposed
    std::map<int, int> transposed_into;     // value -> publication index
    for (int i = 0; i < node_count; i++) {
        const Node &pn = g.nodes[i];
        if (pn.op != Op::PERMUTE || g.values[pn.outputs[0]].publication < 0) continue;
        int v = pn.inputs[0];
        if (g.values[v].shape.size() == 2 && pn.attr_i(0) == 1 && pn.attr_i(1) == 0 && mt.only_consumer(v, i)
            && g.values[v].producer >= 0 && g.nodes[g.values[v].producer].op == Op::MATMUL)
            transposed_into[v] = g.values[pn.outputs[0]].publication;
    }
    auto assign_output = [&](int v) {
        if (assigned[v]) return;
        const Value &val = g.values[v];
        View &w = plan.views[v];
        auto t = transposed_into.find(v);
        if (t != transposed_into.end()) {
            w.slot = SlotKind::PUBLICATION; w.index = t->second; w.offset = 0;
            w.strides = {1, val.shape[0]};
        } else if (val.publication >= 0) {
            w.slot = SlotKind::PUBLICATION; w.index = val.publication; w.offset = 0; w.strides = dense_strides(val.shape);
        } else {
            w.slot = SlotKind::SCRATCH; w.index = new_scratch(val); w.offset = 0; w.strides = dense_strides(val.shape);
        }
        assigned[v] = 1;
    };
    std::vector<char> published_done(g.publications.size(), 0);
    auto finish_step = [&](Step st) {
        for (int v : {st.out, st.out2, st.out3}) if (v >= 0) {
            const View &w = plan.views[v];
            if (w.slot == SlotKind::PUBLICATION) { st.ready_publications.push_back(w.index); published_done[w.index] = 1; }
        }
        plan.steps.push_back(st);
    };
    auto dense_input = [&](int v) -> int {     // row kernels need dense operands; copy a view when they are not
        if (plan.views[v].dense()) return v;
        message = "non-dense operand of a row kernel";
        return -1;
    };

    // engine and operand checks of one GEMM step whose views are assigned
    auto prepare_gemm = [&](Step &st) -> Status {
        {
            {
                const View &c = plan.views[st.out];
                bool transposed = c.strides.size() == 2 && c.strides[0] == 1 && c.shape[0] != 1 && c.strides[1] != 1;
                if (transposed && (st.bias >= 0 || st.mask >= 0 || st.relu || st.act)) { message = "transposed GEMM result with an epilogue"; return UNSUPPORTED_SHAPE; }
                const View &a = plan.views[st.a], &b = plan.views[st.b];
                bool a_ok = a.strides[0] == 1 || a.strides[1] == 1 || a.shape[0] == 1 || a.shape[1] == 1;
                bool b_ok = b.strides[0] == 1 || b.strides[1] == 1 || b.shape[0] == 1 || b.shape[1] == 1;
                if (!a_ok || !b_ok) st.engine = GemmEngine::EXACT_SIMT;
                if (dtype_low(a.dtype)) {
                    // 16-bit storage: the tensor-core kernel reads K-major operands straight from the tensors
                    // (x [m, k] and W [n, k] as Linear stores them) and writes a row-major result; anything
                    // else takes the exact kernel.  No narrow engines, no gate.
                    const bool direct = a.strides[1] == 1 && b.strides[0] == 1 && (c.strides[1] == 1 || c.shape[1] == 1) && !transposed && st.mask < 0
                                        && a.offset % 8 == 0 && b.offset % 8 == 0
                                        && kern::low_gemm_supported(st.m, st.n, st.k, a.strides[0], b.strides[1], c.strides[0]);
                    if (st.engine == GemmEngine::TENSOR_CORE && !direct) st.engine = GemmEngine::EXACT_SIMT;
                    // narrow products too (the 10-class head): a 64-wide tile wastes tensor work, not time
                    if (st.engine == GemmEngine::EXACT_SIMT && direct && options.gemm_engine != 1
                        && (double)st.m * (double)st.n * (double)st.k >= 16.0 * 1024 * 1024) st.engine = GemmEngine::TENSOR_CORE;
                    if (st.bias >= 0 && !plan.views[st.bias].dense()) { message = "strided bias"; return UNSUPPORTED_SHAPE; }
                    return OK;
                }
                // large products with one extent of at most 16 stream through the narrow kernels
                if (options.gemm_engine != 1 && st.engine == GemmEngine::EXACT_SIMT && st.out2 < 0
                    && (double)st.m * (double)st.n * (double)st.k >= 16.0 * 1024 * 1024) {
                    const bool c_rows = c.strides[1] == 1 || c.shape[1] == 1;
                    if (st.n <= 16 && st.mask < 0 && !st.act && a.strides[1] == 1 && b.strides[0] == 1
                        && kern::narrow_out_supported(st.m, st.n, st.k, a.strides[0], b.strides[1]))
                        st.engine = GemmEngine::NARROW_OUT;
                    else if (st.k <= 16 && st.bias < 0 && !st.relu && !st.act && a.strides[1] == 1 && b.strides[1] == 1 && c_rows && !transposed
                             && kern::narrow_inner_supported(st.m, st.n, st.k, b.strides[0], c.strides[0]))
                        st.engine = GemmEngine::NARROW_INNER;
                    else if (st.n <= 16 && st.bias < 0 && !st.relu && !st.act && st.mask < 0 && a.strides[0] == 1 && b.strides[1] == 1
                             && kern::narrow_reduce_supported(st.m, st.n, st.k, a.strides[1]))
                        st.engine = GemmEngine::NARROW_REDUCE;
                }
                if (st.bias >= 0 && !plan.views[st.bias].dense()) { message = "strided bias"; return UNSUPPORTED_SHAPE; }
                if (st.mask >= 0 && !plan.views[st.mask].dense()) { message = "strided gate"; return UNSUPPORTED_SHAPE; }
            }
        }
        return OK;
    };

    for (int i = 0; i < node_count; i++) {
        auto pending = emit_at.find(i);
        if (pending != emit_at.end()) for (Step st : pending->second) {
            for (int v : {st.out, st.out2, st.out3}) if (v >= 0) assign_output(v);
            if (st.kind == StepKind::GEMM) {
                if (st.batch_contraction) {
                    // X^T G over batch * rows: X read as [k, batch * rows] (contraction along its rows), G
                    // as [batch * rows, n], the result as [k, n]
                    for (int *v : {&st.a, &st.b, &st.out}) {
                        View w = plan.views[*v];
                        if (!w.dense()) { message = "batch contraction over a strided tensor"; return UNSUPPORTED_SHAPE; }
                        const int64_t cols = v == &st.out ? st.n : w.shape.back();
                        int64_t count = 1; for (auto d : w.shape) count *= d;
                        if (v == &st.a) { w.shape = {cols, count / cols}; w.strides = {1, cols}; }
                        else { w.shape = {count / cols, cols}; w.strides = {cols, 1}; }
                        plan.views.push_back(w);
                        *v = (int)plan.views.size() - 1;
                    }
                } else if (plan.views[st.a].shape.size() > 2) {
                    // grouped product over a left operand with batch dimensions: every tensor of the step
                    // is dense, so each reads as a matrix of batch * rows rows
                    for (int *v : {&st.a, &st.out, &st.out2, &st.mask}) {
                        if (*v < 0) continue;
                        View w = plan.views[*v];
                        if (!w.dense()) { message = "batched product over a strided tensor inside a fused group"; return UNSUPPORTED_SHAPE; }
                        const int64_t cols = w.shape.back();
                        int64_t count = 1; for (auto d : w.shape) count *= d;
                        w.shape = {count / cols, cols}; w.strides = {cols, 1};
                        plan.views.push_back(w);
                        *v = (int)plan.views.size() - 1;
                    }
                }
                Status gs = prepare_gemm(st);
                if (gs != OK) return gs;
            } else if (st.kind == StepKind::CROSS_ENTROPY) {
                if (dense_input(st.a) < 0 || dense_input(st.b) < 0) return UNSUPPORTED_SHAPE;
            } else if (st.kind == StepKind::SOFTMAX_BACKWARD) {
                if (dense_input(st.a) < 0 || dense_input(st.b) < 0) return UNSUPPORTED_SHAPE;
            } else if (st.kind == StepKind::DENSE_CE_BACKWARD) {
                if (dense_input(st.a) < 0 || dense_input(st.b) < 0 || dense_input(st.c) < 0) return UNSUPPORTED_SHAPE;
            } else if (st.kind == StepKind::RELU_BACKWARD) {
                if (dense_input(st.a) < 0 || dense_input(st.b) < 0) return UNSUPPORTED_SHAPE;
            }
            finish_step(st);
        }
        if (covered[i]) continue;
        const Node &n = g.nodes[i];
        int in0 = n.inputs.empty() ? -1 : n.inputs[0];
        int out0 = n.outputs[0];
        const Value &ov = g.values[out0];
        Step st;
        st.nodes = {i};
        st.op = n.op;
        switch (n.op) {
            case Op::PERMUTE: case Op::EXPAND: case Op::EXPAND_DIMS: case Op::CONTIGUOUS: {
                const View &src = plan.views[in0];
                View w;
                w.slot = src.slot; w.index = src.index; w.offset = src.offset; w.dtype = src.dtype; w.shape = ov.shape;
                size_t r = ov.shape.size();
                w.strides.assign(r, 0);
                if (n.op == Op::PERMUTE) for (size_t d = 0; d < r; d++) w.strides[d] = src.strides[n.attrs[d]];
                else if (n.op == Op::EXPAND) {
                    size_t lead = r - src.shape.size();
                    for (size_t d = 0; d < src.shape.size(); d++) w.strides[lead + d] = src.shape[d] == 1 && ov.shape[lead + d] != 1 ? 0 : src.strides[d];
                } else if (n.op == Op::EXPAND_DIMS) {
                    size_t axis = (size_t)n.attrs[0];
                    for (size_t d = 0, s = 0; d < r; d++) w.strides[d] = d == axis ? 0 : src.strides[s++];
                } else w.strides = src.strides;
                bool needs_copy = n.op == Op::CONTIGUOUS && !w.dense();
                if (!needs_copy && ov.publication < 0) { plan.views[out0] = w; assigned[out0] = 1; break; }
                if (!needs_copy && ov.publication >= 0 && w.slot == SlotKind::PUBLICATION && w.index == ov.publication && w.dense() && w.offset == 0) {
                    plan.views[out0] = w; assigned[out0] = 1; break;     // already written in place, transposed
                }
                // materialise: register the view under a private value id, then copy it out
                plan.views.push_back(w);
                assign_output(out0);
                st.kind = StepKind::COPY; st.a = (int)plan.views.size() - 1; st.out = out0;
                finish_step(st);
                break;
            }
            case Op::MATMUL: {
                // Operands with leading batch dimensions (Tensor.java:1075-1096).  A left operand whose
                // batch and row dimensions collapse into one row dimension over a right operand shared by
                // the whole batch (Linear applied to [batch, time, features]) is one product; anything
                // else is one product per batch slice, each over views of the operands.
                assign_output(out0);
                const View va = plan.views[n.inputs[0]], vb = plan.views[n.inputs[1]], vo = plan.views[out0];
                const size_t r = vo.shape.size(), nb = r - 2;
                auto aligned_batch_strides = [&](const View &v) {     // stride per result batch dimension, 0 where broadcast
                    std::vector<int64_t> s(nb, 0);
                    const size_t own = v.shape.size() - 2;
                    for (size_t d = 0; d < own; d++) s[nb - own + d] = v.shape[d] == 1 ? 0 : v.strides[d];
                    return s;
                };
                const std::vector<int64_t> sa = aligned_batch_strides(va), sb = aligned_batch_strides(vb), so = aligned_batch_strides(vo);
                const int64_t M = vo.shape[r - 2], N = vo.shape[r - 1], K = va.shape.back();
                int64_t batches = 1;
                for (size_t d = 0; d < nb; d++) batches *= vo.shape[d];
                auto rows_collapse = [&](const View &v, const std::vector<int64_t> &bs) {   // [batch.., M, X] reads as [batches * M, X]
                    int64_t expect = v.strides[v.shape.size() - 2] * M;
                    for (size_t d = nb; d-- > 0;) { if (vo.shape[d] != 1 && bs[d] != expect) return false; expect *= vo.shape[d]; }
                    return true;
                };
                bool shared_right = true;
                for (size_t d = 0; d < nb; d++) shared_right &= sb[d] == 0 || vo.shape[d] == 1;
                auto slice = [&](const View &v, int64_t offset, int64_t rows) {
                    View w;
                    w.slot = v.slot; w.index = v.index; w.dtype = v.dtype; w.offset = v.offset + offset;
                    w.shape = {rows, v.shape.back()};
                    w.strides = {v.strides[v.shape.size() - 2], v.strides.back()};
                    plan.views.push_back(w);
                    return (int)plan.views.size() - 1;
                };
                auto emit = [&](int64_t oa, int64_t ob, int64_t oo, int64_t rows) -> Status {
                    Step gs = st;
                    gs.kind = StepKind::GEMM;
                    gs.a = slice(va, oa, rows); gs.b = slice(vb, ob, K); gs.out = slice(vo, oo, rows);
                    gs.m = rows; gs.n = N; gs.k = K;
                    gs.engine = choose_engine(gs.m, gs.n, gs.k);
                    Status status = prepare_gemm(gs);
                    if (status != OK) return status;
                    plan.steps.push_back(gs);
                    return OK;
                };
                if (shared_right && rows_collapse(va, sa) && rows_collapse(vo, so)) {
                    Status status = emit(0, 0, 0, batches * M);
                    if (status != OK) return status;
                } else {
                    if (batches > 4096) { message = "more than 4096 batch slices"; return UNSUPPORTED_SHAPE; }
                    std::vector<int64_t> index(nb, 0);
                    for (int64_t bi = 0; bi < batches; bi++) {
                        int64_t oa = 0, ob = 0, oo = 0;
                        for (size_t d = 0; d < nb; d++) { oa += index[d] * sa[d]; ob += index[d] * sb[d]; oo += index[d] * so[d]; }
                        Status status = emit(oa, ob, oo, M);
                        if (status != OK) return status;
                        for (size_t d = nb; d-- > 0;) { if (++index[d] < vo.shape[d]) break; index[d] = 0; }
                    }
                }
                // the last slice completes the result
                if (vo.slot == SlotKind::PUBLICATION) { plan.steps.back().ready_publications.push_back(vo.index); published_done[vo.index] = 1; }
                break;
            }
            case Op::ADD: case Op::SUB: case Op::MUL: case Op::DIV: case Op::GT: case Op::LT: case Op::EQ:
                assign_output(out0);
                st.kind = StepKind::BINARY; st.a = n.inputs[0]; st.b = n.inputs[1]; st.out = out0;
                finish_step(st);
                break;
            case Op::SCALAR_MUL: case Op::SCALAR_MIN: case Op::SCALAR_MAX: case Op::SCALAR_SUB:
                assign_output(out0);
                st.kind = StepKind::SCALAR; st.a = in0; st.out = out0; st.scalar_bits = n.attrs[0];
                finish_step(st);
                break;
            case Op::CLAMP: {
                // MIN(MAX(input, minValue), maxValue), exactly in that order (Tensor.java:2318-2345):
                // the lower bound into the result, then the upper bound in place
                assign_output(out0);
                Step lower = st;
                lower.kind = StepKind::SCALAR; lower.op = Op::SCALAR_MAX; lower.a = in0; lower.out = out0; lower.scalar_bits = n.attrs[0];
                finish_step(lower);
                st.kind = StepKind::SCALAR; st.op = Op::SCALAR_MIN; st.a = out0; st.out = out0; st.scalar_bits = n.attrs[1];
                finish_step(st);
                break;
            }
            case Op::RELU: case Op::EXP: case Op::TANH: case Op::SIGMOID: case Op::SILU: case Op::IS_INF: case Op::GELU_TANH:
            case Op::GELU: case Op::ERF:
                assign_output(out0);
                st.kind = StepKind::UNARY; st.a = in0; st.out = out0;
                finish_step(st);
                break;
            case Op::WHERE:
                assign_output(out0);
                st.kind = StepKind::WHERE; st.a = n.inputs[0]; st.b = n.inputs[1]; st.c = n.inputs[2]; st.out = out0;
                finish_step(st);
                break;
            case Op::ONE_HOT:
                if (dense_input(in0) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::ONE_HOT; st.a = in0; st.out = out0; st.scalar_bits = n.attrs[0];
                st.m = g.values[in0].elements(); st.n = (int64_t)n.attrs[0];
                finish_step(st);
                break;
            case Op::MAX: case Op::SUM: {
                assign_output(out0);
                st.a = in0; st.out = out0;
                if ((int64_t)n.attrs[0] == -1) {
                    st.kind = StepKind::FULL_SUM; st.m = g.values[in0].elements();
                } else {
                    if (dense_input(in0) < 0) return UNSUPPORTED_SHAPE;
                    st.kind = StepKind::ROW_REDUCE; st.n = g.values[in0].shape.back(); st.m = g.values[in0].elements() / std::max<int64_t>(st.n, 1);
                }
                finish_step(st);
                break;
            }
            case Op::SUM_TO_SHAPE:
                if (dense_input(in0) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::COLSUM; st.a = in0; st.out = out0;
                st.n = ov.elements(); st.m = g.values[in0].elements() / std::max<int64_t>(st.n, 1);     // leading dimensions are summed
                finish_step(st);
                break;
            case Op::SOFTMAX:
                if (dense_input(in0) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::SOFTMAX; st.a = in0; st.out = out0;
                st.n = g.values[in0].shape.back(); st.m = g.values[in0].elements() / std::max<int64_t>(st.n, 1);
                st.scalar_bits = n.attr_i(1);           // kind: 0 SOFTMAX, 1 LOG_SOFTMAX
                finish_step(st);
                break;
            case Op::INDEX_CROSS_ENTROPY: message = "internal: loss not grouped"; return INTERNAL_ERROR;
            case Op::DENSE_CROSS_ENTROPY:
                if (dense_input(n.inputs[0]) < 0 || dense_input(n.inputs[1]) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::DENSE_CROSS_ENTROPY; st.a = n.inputs[0]; st.b = n.inputs[1]; st.out = out0;
                st.m = g.values[n.inputs[0]].shape[0]; st.n = g.values[n.inputs[0]].shape[1];
                st.scalar_bits = n.attrs[1];            // reduction: 0 NONE, 1 MEAN, 2 SUM
                finish_step(st);
                break;
            case Op::MEAN_SQUARED_ERROR:
                if (dense_input(n.inputs[0]) < 0 || dense_input(n.inputs[1]) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::MSE; st.a = n.inputs[0]; st.b = n.inputs[1]; st.out = out0; st.m = g.values[n.inputs[0]].elements();
                st.scalar_bits = n.attrs[0];            // reduction: 0 NONE, 1 MEAN, 2 SUM
                finish_step(st);
                break;
            case Op::ARG_MAX:
                if (dense_input(in0) < 0) return UNSUPPORTED_SHAPE;
                assign_output(out0);
                st.kind = StepKind::ARG_MAX; st.a = in0; st.out = out0; st.m = g.values[in0].shape[0]; st.n = g.values[in0].shape[1];
                finish_step(st);
                break;
        }
    }
    // publications that are views of something else (a feed, a shared intermediate) are copied out
    for (size_t j = 0; j < g.publications.size(); j++) {
        if (published_done[j]) continue;
        int v = g.publications[j];
        const View &w = plan.views[v];
        if (!assigned[v]) { message = "publication was never produced"; return INTERNAL_ERROR; }
        View target;
        target.slot = SlotKind::PUBLICATION; target.index = (int)j; target.offset = 0; target.dtype = w.dtype;
        target.shape = w.shape; target.strides = dense_strides(w.shape);
        plan.views.push_back(target);
        Step st;
        st.kind = StepKind::COPY; st.a = v; st.out = (int)plan.views.size() - 1;
        st.ready_publications.push_back((int)j);
        plan.steps.push_back(st);
    }
    return OK;
}

std::string describe_plan(const Program &g, const Plan &plan) {
    std::ostringstream os;
    for (const Step &st : plan.steps) {
        os << step_name(st.kind);
        if (st.kind == StepKind::GEMM) {
            const DType operand_type = plan.views[st.a].dtype;
            os << " engine=" << (dtype_low(operand_type) && st.engine == GemmEngine::TENSOR_CORE ? "tcgen05_f16" : engine_name(st.engine))
               << " m=" << st.m << " n=" << st.n << " k=" << st.k;
            if (operand_type == DType::BF16) os << " bf16";
            if (operand_type == DType::F16) os << " f16";
            if (st.bias >= 0) os << " bias";
            if (st.relu) os << " relu";
            if (st.act) os << " act=" << op_name((Op)st.act);
            if (st.out2 >= 0) os << " keep_preactivation";
            if (st.mask >= 0) os << " relu_gate";
            const View &c = plan.views[st.out];
            if (c.strides.size() == 2 && c.strides[0] == 1 && c.shape[0] != 1 && c.strides[1] != 1) os << " transposed_result";
        } else if (st.kind == StepKind::BINARY || st.kind == StepKind::SCALAR || st.kind == StepKind::UNARY || st.kind == StepKind::ROW_REDUCE) {
            os << " op=" << op_name(st.op);
        } else if (st.kind == StepKind::CROSS_ENTROPY) {
            os << " rows=" << st.m << " classes=" << st.n << (st.out >= 0 ? " loss" : "") << (st.out2 >= 0 ? " gradient" : "") << (st.out3 >= 0 ? " arg_max" : "");
        }
        if (st.kind != StepKind::GEMM && st.kind != StepKind::CROSS_ENTROPY && st.m) os << " m=" << st.m << " n=" << st.n;
        os << " nodes=[";
        for (size_t i = 0; i < st.nodes.size(); i++) os << (i ? "," : "") << op_name(g.nodes[st.nodes[i]].op);
        os << "]";
        if (!st.ready_publications.empty()) {
            os << " publishes=[";
            for (size_t i = 0; i < st.ready_publications.size(); i++) os << (i ? "," : "") << st.ready_publications[i];
            os << "]";
        }
        os << "\n";
    }
    return os.str();
}

}  // namespace syn
