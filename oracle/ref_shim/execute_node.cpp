// Stand-in for the one reference translation unit that cannot be built here:
// src/cpu/kernels.cpp needs Eigen 3.4.0 (cmake/Dependencies.cmake:12-28), which
// is neither vendored nor installed. It provides minicompiler::cpu::execute_node
// with the reference's signature (src/cpu/kernels.hpp) so that the reference's own
// constant-folding pass links. Arithmetic: each op is evaluated in double and
// rounded to float once, which is what the reference's own test oracle does
// (tests/test_util.cpp:87-159) and lies within the few-ulp envelope the reference
// documents for Eigen (include/minicompiler/passes/constant_folding.hpp:20-24).
// TEST INFRASTRUCTURE ONLY.
#include "cpu/kernels.hpp"

#include "minicompiler/ops.hpp"

#include <cmath>

namespace minicompiler::cpu {
namespace {

double unary_d(OpKind op, double x) {
    switch (op) {
        case OpKind::Neg: return -x;
        case OpKind::Exp: return std::exp(x);
        case OpKind::Log: return std::log(x);
        case OpKind::Sqrt: return std::sqrt(x);
        case OpKind::Relu: return x > 0.0 ? x : 0.0;
        case OpKind::Sigmoid: return 1.0 / (1.0 + std::exp(-x));
        case OpKind::Tanh: return std::tanh(x);
        default: return 0.0;
    }
}

double binary_d(OpKind op, double a, double b) {
    switch (op) {
        case OpKind::Add: return a + b;
        case OpKind::Sub: return a - b;
        case OpKind::Mul: return a * b;
        case OpKind::Div: return a / b;
        default: return 0.0;
    }
}

std::int64_t offset_of(std::size_t i, const Shape& out, const std::vector<std::int64_t>& strides) {
    std::int64_t off = 0;
    for (std::size_t d = out.size(); d-- > 0;) {
        off += static_cast<std::int64_t>(i % static_cast<std::size_t>(out[d])) * strides[d];
        i /= static_cast<std::size_t>(out[d]);
    }
    return off;
}

}  // namespace

void execute_node(const Node& node, const std::vector<const float*>& operands, const std::vector<Shape>& operand_shapes,
                  float* out, std::vector<float>& scratch) {
    (void)scratch;
    const Shape& oshape = node.type.shape;
    const std::size_t count = node.type.num_elements();
    if (node.op == OpKind::MatMul) {
        const std::int64_t m = operand_shapes[0][0], k = operand_shapes[0][1], n = operand_shapes[1][1];
        for (std::int64_t r = 0; r < m; ++r) {
            for (std::int64_t c = 0; c < n; ++c) {
                double acc = 0.0;
                for (std::int64_t t = 0; t < k; ++t) acc += static_cast<double>(operands[0][r * k + t]) * operands[1][t * n + c];
                out[r * n + c] = static_cast<float>(acc);
            }
        }
        return;
    }
    std::vector<std::vector<std::int64_t>> strides;
    for (const Shape& s : operand_shapes) strides.push_back(broadcast_strides(s, oshape));
    if (node.op == OpKind::FusedElementwise) {
        const FusedProgram& p = *node.fused;
        std::vector<double> regs(p.instrs.size());
        for (std::size_t e = 0; e < count; ++e) {
            for (std::size_t r = 0; r < p.instrs.size(); ++r) {
                const FusedInstr& ins = p.instrs[r];
                double x = 0.0;
                switch (ins.kind) {
                    case FusedInstr::Kind::Load: x = operands[ins.a][offset_of(e, oshape, strides[ins.a])]; break;
                    case FusedInstr::Kind::Immediate: x = ins.immediate; break;
                    case FusedInstr::Kind::Unary: x = unary_d(ins.op, regs[ins.a]); break;
                    case FusedInstr::Kind::Binary: x = binary_d(ins.op, regs[ins.a], regs[ins.b]); break;
                }
                regs[r] = static_cast<float>(x);
            }
            out[e] = static_cast<float>(regs.back());
        }
        return;
    }
    for (std::size_t e = 0; e < count; ++e) {
        const double a = operands[0][offset_of(e, oshape, strides[0])];
        out[e] = static_cast<float>(is_unary_elementwise(node.op)
                                        ? unary_d(node.op, a)
                                        : binary_d(node.op, a, operands[1][offset_of(e, oshape, strides[1])]));
    }
}

}  // namespace minicompiler::cpu
