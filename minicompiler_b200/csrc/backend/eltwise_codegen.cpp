#include "backend/eltwise_codegen.hpp"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <sstream>

namespace minicompiler::cuda {

std::string float_bits_literal(float v) {
    std::uint32_t bits = 0;
    std::memcpy(&bits, &v, sizeof bits);
    char text[40];
    std::snprintf(text, sizeof text, "__uint_as_float(0x%08xu)", static_cast<unsigned>(bits));
    return text;
}

std::string op_expression(OpKind op, const std::string& a, const std::string& b) {
    switch (op) {
        case OpKind::Neg: return "-" + a;
        case OpKind::Exp: return "expf(" + a + ")";
        case OpKind::Log: return "logf(" + a + ")";
        case OpKind::Sqrt: return "sqrtf(" + a + ")";
        case OpKind::Relu: return "fmaxf(" + a + ", 0.0f)";
        case OpKind::Sigmoid: return "1.0f / (1.0f + expf(-" + a + "))";
        case OpKind::Tanh: return "tanhf(" + a + ")";
        case OpKind::Add: return a + " + " + b;
        case OpKind::Sub: return a + " - " + b;
        case OpKind::Mul: return a + " * " + b;
        case OpKind::Div: return a + " / " + b;
        default: return "0.0f /* unsupported op */";
    }
}

Access classify_access(const Shape& in, const Shape& out) {
    Access acc;
    const std::size_t in_count = num_elements(in);
    if (in_count == 1) {
        acc.kind = AccessKind::Scalar;
        return acc;
    }
    if (in_count == num_elements(out)) return acc;  // broadcastable and as large: identical layout
    std::size_t skip = 0;
    while (skip < in.size() && in[skip] == 1) ++skip;
    const std::size_t tail = in.size() - skip;
    if (tail <= out.size() && std::equal(in.begin() + static_cast<std::ptrdiff_t>(skip), in.end(),
                                         out.end() - static_cast<std::ptrdiff_t>(tail))) {
        acc.kind = AccessKind::Periodic;
        acc.period = in_count;
        return acc;
    }
    acc.kind = AccessKind::General;
    acc.strides = broadcast_strides(in, out);
    return acc;
}

namespace {

std::string u32(std::uint64_t v) { return std::to_string(v) + "u"; }

// sum over dims d < dims_used of coord_d * multiplier[d], where coord_d = (i / divisor[d]) % out[d]
// (no `% out[0]`: the outermost coordinate never wraps; no `/ 1`, no `* 1`).
std::string broadcast_index(const Shape& out, std::size_t dims_used, const std::vector<std::uint64_t>& divisor,
                            const std::vector<std::uint64_t>& multiplier) {
    std::string expr;
    for (std::size_t d = 0; d < dims_used; ++d) {
        if (multiplier[d] == 0) continue;
        std::string coord = divisor[d] == 1 ? std::string("i") : "(i / " + u32(divisor[d]) + ")";
        if (d > 0) coord = "(" + coord + " % " + u32(static_cast<std::uint64_t>(out[d])) + ")";
        if (multiplier[d] != 1) coord += " * " + u32(multiplier[d]);
        expr += (expr.empty() ? "" : " + ") + coord;
    }
    return expr.empty() ? std::string("0u") : expr;
}

}  // namespace

ElementwiseKernel generate_elementwise_kernel(const FusedProgram& program, const std::vector<Shape>& input_shapes,
                                              const Shape& out_shape, const ElementwiseOptions& options) {
    const std::size_t num_inputs = input_shapes.size();
    std::vector<Access> access;
    for (const Shape& s : input_shapes) access.push_back(classify_access(s, out_shape));

    const std::size_t total = num_elements(out_shape);
    const std::size_t rank = out_shape.size();
    const std::uint64_t last_extent = out_shape.empty() ? 1 : static_cast<std::uint64_t>(out_shape.back());
    const bool want_half = options.write_half != HalfKind::None;
    const std::uint64_t half_row_pitch =
        want_half && options.half_pitch > 0 ? static_cast<std::uint64_t>(options.half_pitch) : last_extent;
    const bool half_dense = half_row_pitch == last_extent;

    // 128-bit accesses need every group of 4 consecutive output elements to map, per input, to either 4
    // consecutive aligned elements or one element.
    bool vectorized = options.allow_vectorize && total % 4 == 0;
    for (const Access& a : access) {
        if (a.kind == AccessKind::Periodic && a.period % 4 != 0) vectorized = false;
        if (a.kind == AccessKind::General && last_extent % 4 != 0) vectorized = false;
    }
    if (want_half && !half_dense && (last_extent % 4 != 0 || half_row_pitch % 4 != 0)) vectorized = false;

    const unsigned unroll = std::max(1u, options.unroll);
    const unsigned tile = kElementwiseBlock * unroll;  // items per block per trip
    const std::size_t last = program.instrs.size() - 1;
    const char* half_name = options.write_half == HalfKind::Bf16 ? "bf16" : "f16";

    // Inputs the program actually reads, and whether each is read once per element or once per kernel.
    std::vector<bool> used(num_inputs, false);
    for (const FusedInstr& ins : program.instrs) {
        if (ins.kind == FusedInstr::Kind::Load) used[static_cast<std::size_t>(ins.a)] = true;
    }
    auto streamed = [&](std::size_t k) { return used[k] && access[k].kind != AccessKind::Scalar; };

    std::ostringstream os;
    os << "// Generated by minicompiler-b200: " << program.num_ops() << " elementwise op(s), "
       << (vectorized ? "128-bit accesses, " : "32-bit accesses, ") << unroll << " per thread per trip.\n";

    // The straight-line program for one element.
    os << "static __device__ __forceinline__ float mc_eval(";
    {
        const char* sep = "";
        for (std::size_t k = 0; k < num_inputs; ++k) {
            if (!used[k]) continue;
            os << sep << "const float x" << k;
            sep = ", ";
        }
    }
    os << ")\n{\n";
    for (std::size_t r = 0; r < program.instrs.size(); ++r) {
        const FusedInstr& ins = program.instrs[r];
        os << "\tconst float r" << r << " = ";
        switch (ins.kind) {
            case FusedInstr::Kind::Load: os << "x" << ins.a << ";\n"; break;
            case FusedInstr::Kind::Immediate: {
                char note[40];
                std::snprintf(note, sizeof note, "%.9g", static_cast<double>(ins.immediate));
                os << float_bits_literal(ins.immediate) << ";  // " << note << "\n";
                break;
            }
            case FusedInstr::Kind::Unary: os << op_expression(ins.op, "r" + std::to_string(ins.a), "") << ";\n"; break;
            case FusedInstr::Kind::Binary:
                os << op_expression(ins.op, "r" + std::to_string(ins.a), "r" + std::to_string(ins.b)) << ";\n";
                break;
        }
    }
    os << "\treturn r" << last << ";\n}\n\n";

    os << "extern \"C\" __global__ void __launch_bounds__(" << kElementwiseBlock << ")\n" << kElementwiseKernelName << "(";
    {
        const char* sep = "";
        if (options.write_f32) {
            os << "float* __restrict__ out";
            sep = ", ";
        }
        if (want_half) {
            os << sep << "unsigned short* __restrict__ out16";
            sep = ", ";
        }
        for (std::size_t k = 0; k < num_inputs; ++k) {
            os << sep << "const float* __restrict__ in" << k;
            sep = ", ";
        }
        os << sep << "unsigned n)\n{\n";
    }

    // One-element inputs are read once, before the loop.
    for (std::size_t k = 0; k < num_inputs; ++k) {
        if (used[k] && access[k].kind == AccessKind::Scalar) os << "\tconst float s" << k << " = in" << k << "[0];\n";
    }

    const std::string ld_stream = options.streaming_hints ? "__ldcs" : "__ldg";
    // mc_eval(...) for one lane ("" for the 32-bit path, ".x" ... for the 128-bit path).
    auto eval_call = [&](const std::string& lane) {
        std::string call = "mc_eval(";
        const char* sep = "";
        for (std::size_t k = 0; k < num_inputs; ++k) {
            if (!used[k]) continue;
            call += sep;
            call += access[k].kind == AccessKind::Scalar ? "s" + std::to_string(k) : "v" + std::to_string(k) + "[u]" + lane;
            sep = ", ";
        }
        return call + ")";
    };

    if (vectorized) {
        const std::uint64_t row_groups = last_extent / 4;
        for (std::size_t k = 0; k < num_inputs; ++k) {
            if (streamed(k)) os << "\tconst float4* __restrict__ q" << k << " = reinterpret_cast<const float4*>(in" << k << ");\n";
        }
        if (options.write_f32) os << "\tfloat4* __restrict__ qo = reinterpret_cast<float4*>(out);\n";
        if (want_half) os << "\tuint2* __restrict__ qh = reinterpret_cast<uint2*>(out16);\n";

        // The expression that loads input k's 4 values for group index i.
        auto vector_load = [&](std::size_t k) -> std::string {
            const Access& a = access[k];
            const std::string q = "q" + std::to_string(k);
            if (a.kind == AccessKind::Contiguous) return ld_stream + "(" + q + " + i)";
            if (a.kind == AccessKind::Periodic) return "__ldg(" + q + " + (i % " + u32(a.period / 4) + "))";
            // General: the 4 elements of a group share every coordinate but the last.
            std::vector<std::uint64_t> divisor(rank, 1), multiplier(rank, 0);
            std::uint64_t span = row_groups;
            for (std::size_t d = rank - 1; d-- > 0;) {
                divisor[d] = span;
                span *= static_cast<std::uint64_t>(out_shape[d]);
            }
            const bool walks_row = a.strides[rank - 1] != 0;
            for (std::size_t d = 0; d + 1 < rank; ++d) {
                const auto s = static_cast<std::uint64_t>(a.strides[d]);
                multiplier[d] = walks_row ? s / 4 : s;
            }
            const std::string rows = broadcast_index(out_shape, rank - 1, divisor, multiplier);
            if (walks_row) return "__ldg(" + q + " + (" + rows + " + (i % " + u32(row_groups) + ")))";
            return "mc_splat(__ldg(in" + std::to_string(k) + " + (" + rows + ")))";
        };

        os << "\tconst unsigned trip = gridDim.x * " << u32(tile) << ";\n";
        os << "\tfor (unsigned base = blockIdx.x * " << u32(tile) << " + threadIdx.x; base < n; base += trip) {\n";
        // A trip that lies wholly inside the tensor runs without per-access bounds checks.
        os << "\t\tconst bool whole = base + " << u32(static_cast<std::uint64_t>(unroll - 1) * kElementwiseBlock) << " < n;\n";
        for (std::size_t k = 0; k < num_inputs; ++k) {
            if (streamed(k)) os << "\t\tfloat4 v" << k << "[" << unroll << "];\n";
        }
        // All loads of the trip are issued before any arithmetic.
        os << "#pragma unroll\n\t\tfor (unsigned u = 0; u < " << unroll << "u; ++u) {\n";
        os << "\t\t\tconst unsigned i = base + u * " << u32(kElementwiseBlock) << ";\n";
        os << "\t\t\tif (!whole && i >= n) continue;\n";
        for (std::size_t k = 0; k < num_inputs; ++k) {
            if (streamed(k)) os << "\t\t\tv" << k << "[u] = " << vector_load(k) << ";\n";
        }
        os << "\t\t}\n";
        os << "#pragma unroll\n\t\tfor (unsigned u = 0; u < " << unroll << "u; ++u) {\n";
        os << "\t\t\tconst unsigned i = base + u * " << u32(kElementwiseBlock) << ";\n";
        os << "\t\t\tif (!whole && i >= n) continue;\n";
        os << "\t\t\tfloat4 o;\n";
        for (const char* lane : {".x", ".y", ".z", ".w"}) os << "\t\t\to" << lane << " = " << eval_call(lane) << ";\n";
        if (options.write_f32) {
            os << (options.streaming_hints ? "\t\t\t__stcs(qo + i, o);\n" : "\t\t\tqo[i] = o;\n");
        }
        if (want_half) {
            os << "\t\t\tuint2 h;\n";
            os << "\t\t\tasm(\"cvt.rn." << half_name << "x2.f32 %0, %1, %2;\" : \"=r\"(h.x) : \"f\"(o.y), \"f\"(o.x));\n";
            os << "\t\t\tasm(\"cvt.rn." << half_name << "x2.f32 %0, %1, %2;\" : \"=r\"(h.y) : \"f\"(o.w), \"f\"(o.z));\n";
            if (half_dense) {
                os << "\t\t\tqh[i] = h;\n";
            } else {
                os << "\t\t\tqh[(i / " << u32(row_groups) << ") * " << u32(half_row_pitch / 4) << " + (i % " << u32(row_groups)
                   << ")] = h;\n";
            }
        }
        os << "\t\t}\n\t}\n}\n";

        std::string source = os.str();
        if (source.find("mc_splat(") != std::string::npos) {
            source = "static __device__ __forceinline__ float4 mc_splat(float v) { return make_float4(v, v, v, v); }\n" + source;
        }
        return {std::move(source), true, unroll, options.write_f32, want_half};
    }

    // 32-bit path: one element per item, still `unroll` items in flight per thread.
    auto scalar_load = [&](std::size_t k) -> std::string {
        const Access& a = access[k];
        const std::string p = "in" + std::to_string(k);
        if (a.kind == AccessKind::Contiguous) return ld_stream + "(" + p + " + i)";
        if (a.kind == AccessKind::Periodic) return "__ldg(" + p + " + (i % " + u32(a.period) + "))";
        std::vector<std::uint64_t> divisor(rank, 1), multiplier(rank, 0);
        std::uint64_t span = 1;
        for (std::size_t d = rank; d-- > 0;) {
            divisor[d] = span;
            span *= static_cast<std::uint64_t>(out_shape[d]);
            multiplier[d] = static_cast<std::uint64_t>(a.strides[d]);
        }
        return "__ldg(" + p + " + (" + broadcast_index(out_shape, rank, divisor, multiplier) + "))";
    };

    os << "\tconst unsigned trip = gridDim.x * " << u32(tile) << ";\n";
    os << "\tfor (unsigned base = blockIdx.x * " << u32(tile) << " + threadIdx.x; base < n; base += trip) {\n";
    for (std::size_t k = 0; k < num_inputs; ++k) {
        if (streamed(k)) os << "\t\tfloat v" << k << "[" << unroll << "];\n";
    }
    os << "#pragma unroll\n\t\tfor (unsigned u = 0; u < " << unroll << "u; ++u) {\n";
    os << "\t\t\tconst unsigned i = base + u * " << u32(kElementwiseBlock) << ";\n";
    os << "\t\t\tif (i >= n) continue;\n";
    for (std::size_t k = 0; k < num_inputs; ++k) {
        if (streamed(k)) os << "\t\t\tv" << k << "[u] = " << scalar_load(k) << ";\n";
    }
    os << "\t\t}\n";
    os << "#pragma unroll\n\t\tfor (unsigned u = 0; u < " << unroll << "u; ++u) {\n";
    os << "\t\t\tconst unsigned i = base + u * " << u32(kElementwiseBlock) << ";\n";
    os << "\t\t\tif (i >= n) continue;\n";
    os << "\t\t\tconst float o = " << eval_call("") << ";\n";
    if (options.write_f32) os << "\t\t\tout[i] = o;\n";
    if (want_half) {
        os << "\t\t\tunsigned short h;\n";
        os << "\t\t\tasm(\"cvt.rn." << half_name << ".f32 %0, %1;\" : \"=h\"(h) : \"f\"(o));\n";
        if (half_dense) {
            os << "\t\t\tout16[i] = h;\n";
        } else {
            os << "\t\t\tout16[(i / " << u32(last_extent) << ") * " << u32(half_row_pitch) << " + (i % " << u32(last_extent)
               << ")] = h;\n";
        }
    }
    os << "\t\t}\n\t}\n}\n";
    return {os.str(), false, unroll, options.write_f32, want_half};
}

}  // namespace minicompiler::cuda
