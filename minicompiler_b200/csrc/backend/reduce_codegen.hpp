#pragma once
// CUDA C++ source generator for a row reduction (row_sum / row_max) with an elementwise prologue.
//
// The reference has no reduction op (README.md:561-562 names reductions with warp-shuffle kernels as future
// work); this generator follows the conventions of the elementwise one (src/cuda/codegen.cpp:97-182 in the
// reference, eltwise_codegen.cpp here): shapes are compile-time constants, one-element inputs are read once,
// immediates are exact bit patterns, the per-element program is a straight-line `mc_eval`.
//
// Kernel contract: `mc_row_reduce(float* out, in0, in1, ..., unsigned rows)`. The program is evaluated for every
// element of the pre-reduction shape `in_shape` (its inputs broadcast against that shape), and the values of each
// row of the last dimension are combined: per thread in increasing column order, then across the lanes of a warp
// by an xor-shuffle tree, then (rows of 1024 elements or more, one 256-thread block per row) across the 8 warps
// in warp order. The order is fixed, so results do not depend on scheduling. Sums are FP32 (the definition of the
// op is the double-precision sum rounded once; the kernel is within n*2^-24 * sum|x| of it); maxima are exact.

#include "core/ir.hpp"

#include <string>
#include <vector>

namespace minicompiler::cuda {

inline constexpr const char* kRowReduceKernelName = "mc_row_reduce";
inline constexpr unsigned kRowReduceBlock = 256;

struct RowReduceKernel {
    std::string source;
    unsigned threads_per_row = 32;  // 32: eight rows per block, one warp each; 256: one row per block
    unsigned rows_per_block = 8;
};

RowReduceKernel generate_row_reduce_kernel(OpKind reduce_op, const FusedProgram& program,
                                           const std::vector<Shape>& input_shapes, const Shape& in_shape);

}  // namespace minicompiler::cuda
