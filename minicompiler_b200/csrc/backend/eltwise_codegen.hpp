#pragma once
// CUDA C++ source generator for one elementwise / fused node, aimed at B200.
// It replaces the reference's generator (src/cuda/codegen.{hpp,cpp}) behind the
// same contract: a kernel named mc_elementwise taking (out, in0, in1, ..., n)
// that evaluates a FusedProgram per output element, with shapes known at
// compile time so that all broadcast index math has constant divisors,
// one-element inputs and immediates hoisted out of the loop, and immediates
// spelled as exact bit patterns.
//
// What is different from the reference's output:
//   * every thread keeps `unroll` independent 128-bit loads in flight per input
//     before it computes (HBM3e needs several MB in flight), and walks the
//     tensor in block-contiguous, fully coalesced tiles;
//   * the 128-bit path also covers general broadcasts (a [M,1] column, a
//     [B,1,N] slab ...) whenever the output's last extent is a multiple of 4,
//     not just suffix-shaped operands;
//   * streamed operands use evict-first loads/stores, re-used (broadcast)
//     operands go through the read-only path;
//   * a kernel can also emit a bf16/fp16 copy of its result, so that a
//     tensor-core matmul downstream reads 16-bit operands without a cast pass.
//
// This file has no CUDA dependency; it is exercised on hosts without a GPU.

#include "core/ir.hpp"

#include <string>
#include <vector>

namespace minicompiler::cuda {

inline constexpr const char* kElementwiseKernelName = "mc_elementwise";
inline constexpr unsigned kElementwiseBlock = 256;  // matches __launch_bounds__ in the generated source

enum class HalfKind : int { None = 0, Bf16 = 1, F16 = 2 };

struct ElementwiseOptions {
    bool allow_vectorize = true;
    unsigned unroll = 4;               // accesses in flight per thread per input
    bool write_f32 = true;             // emit the float result
    HalfKind write_half = HalfKind::None;  // also (or only) emit a 16-bit copy
    std::int64_t half_pitch = 0;       // row pitch of the 16-bit copy in elements; 0 = dense
    bool streaming_hints = true;
};

struct ElementwiseKernel {
    std::string source;
    bool vectorized = false;  // n counts groups of 4 elements
    unsigned unroll = 1;      // items (groups or elements) per thread per trip
    // Kernel parameter order: [float* out] [uint16* out16] in0 in1 ... unsigned n
    bool has_f32_out = true;
    bool has_half_out = false;
};

// How one input is addressed relative to the output (same classes as the
// reference generator, src/cuda/codegen.cpp:41-82).
enum class AccessKind { Contiguous, Scalar, Periodic, General };
struct Access {
    AccessKind kind = AccessKind::Contiguous;
    std::size_t period = 0;                 // Periodic: elements per repetition
    std::vector<std::int64_t> strides;      // General: per output dim, 0 where broadcast
};
Access classify_access(const Shape& in, const Shape& out);

ElementwiseKernel generate_elementwise_kernel(const FusedProgram& program, const std::vector<Shape>& input_shapes,
                                              const Shape& out_shape, const ElementwiseOptions& options = {});

// `v` as a CUDA expression with its exact bits: "__uint_as_float(0x3f000000u)".
std::string float_bits_literal(float v);
// The C expression of `op` applied to operand expressions `a` (and `b`).
std::string op_expression(OpKind op, const std::string& a, const std::string& b);

}  // namespace minicompiler::cuda
