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
// by an xor-shuffle tree, then (rows of more than 1024 elements, one block per row) across the block's warps in
// warp order. The order is fixed, so results do not depend on scheduling. Sums are FP32 (the definition of the
// op is the double-precision sum rounded once; the kernel is within n*2^-24 * sum|x| of it); maxima are exact.

#include "core/ir.hpp"

#include <string>
#include <vector>

namespace minicompiler::cuda {

inline constexpr const char* kRowReduceKernelName = "mc_row_reduce";
inline constexpr unsigned kRowReduceBlock = 256;

// How a row is shared out, for both kernels of this file. Up to 1024 elements a warp takes a row (8 rows per
// 256-thread block; at 1024 columns 32 elements per lane and no block-wide barrier: 18.4 against 20.6 us for softmax
// f32[8192,1024]). Up to 8192 elements a 256-thread block takes it. Wider rows, up to 65536 elements, are cut into
// 2, 4 or 8 chunks of at most 8192 columns, one 256-thread CTA each, and those CTAs form a thread-block cluster: every
// CTA reduces its chunk, the per-CTA results are exchanged through distributed shared memory and combined in rank
// order by every CTA (the same fixed order in both kernels). Several small CTAs per SM overlap their loads, arithmetic
// and stores where one 1024-thread block per SM cannot. Beyond 65536 a single 256-thread block loops over the row.
inline unsigned row_cluster(std::int64_t width) {
    return width <= 8192 ? 1u : width <= 16384 ? 2u : width <= 32768 ? 4u : width <= 65536 ? 8u : 1u;
}
inline unsigned row_threads(std::int64_t width) { return width <= 1024 ? 32u : 256u; }
inline unsigned row_block(std::int64_t width) { (void)width; return 256u; }
// Columns per CTA of the cluster: whole trips of 256 threads.
inline std::int64_t row_chunk(std::int64_t width) {
    const std::int64_t c = row_cluster(width);
    return c == 1 ? width : ((width + c - 1) / c + 255) / 256 * 256;
}

struct RowReduceKernel {
    std::string source;
    unsigned threads_per_row = 32;  // row_threads(width)
    unsigned rows_per_block = 8;
    unsigned block = kRowReduceBlock;  // threads per block to launch with
    unsigned cluster = 1;              // CTAs per row (the kernel carries __cluster_dims__(cluster, 1, 1))
};

RowReduceKernel generate_row_reduce_kernel(OpKind reduce_op, const FusedProgram& program,
                                           const std::vector<Shape>& input_shapes, const Shape& in_shape);

}  // namespace minicompiler::cuda

// ---------------------------------------------------------------- whole rows in one kernel
//
// A run of steps that all work on rows of one shape [.., N] - elementwise steps on the full shape, row reductions,
// elementwise steps on the reduced [.., 1] values - is generated as ONE kernel: a 256-thread block (a warp, for rows
// of up to 1024 elements; a cluster of 2, 4 or 8 blocks for rows wider than 8192) owns a row, keeps every full-shaped
// value in registers (at most 32 elements per thread), gets reduced values by a block (warp, cluster) reduction and
// runs the steps in their original order, so x is read once and y written once (softmax, LayerNorm: two tensor passes
// instead of four). The reduction order is exactly that of `mc_row_reduce` for the same row length, so a fused run
// gives the bits of the separate kernels.

namespace minicompiler::cuda {

inline constexpr const char* kRowFusedKernelName = "mc_row_fused";
inline constexpr std::int64_t kRowFusedMinWidth = 2;     // rows of up to 1024 elements take one warp, as in mc_row_reduce
inline constexpr std::int64_t kRowFusedMaxWidth = 65536;  // 8 CTAs of 8192 columns: at most 32 registers per full-shaped value and thread

struct RowOperand {
    enum class Kind { Full, PerRow, RowVector, Scalar };
    Kind kind = Kind::Full;
    int external = -1;  // index into the kernel's external pointers, or
    int value = -1;     // the `result` number of an earlier part
};

struct RowPart {
    bool is_reduce = false;
    OpKind reduce_op = OpKind::RowSum;
    FusedProgram program;              // over `operands`
    std::vector<RowOperand> operands;
    int result = 0;                    // value number this part defines
    bool result_is_full = true;        // false: one value per row (a reduction, or elementwise on reduced values)
    int output = -1;                   // index into the kernel's output pointers when the value is written
    std::string name;                  // for the comment line
};

// Kernel parameters: out0, out1, ..., ex0, ex1, ..., unsigned rows.
std::string generate_row_fused_kernel(const std::vector<RowPart>& parts, const std::vector<RowOperand::Kind>& externals,
                                      int num_outputs, std::int64_t width);

}  // namespace minicompiler::cuda
