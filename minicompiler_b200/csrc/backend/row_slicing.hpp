#pragma once
// Row slicing of a compiled graph: which values can be cut along their leading
// dimension so that every slice of rows is an independent run of the same graph.
//
// It serves run() on pinned host memory. The reference copies all inputs in,
// runs, and copies all outputs out (src/cuda/cuda_backend.cpp:154-196); when the
// graph is row-independent the three phases of consecutive row slices can overlap
// instead, on both copy engines and the SMs at once. Unlike the multi-GPU
// partitioner (partition.hpp), which re-parses the source text at two batch sizes,
// this works on the optimized Graph alone, because an executable no longer has the
// text: it is a dataflow analysis over the ops, sound whatever the author meant the
// leading dimension to be.

#include "core/ir.hpp"

#include <cstdint>
#include <vector>

namespace minicompiler::cuda {

struct RowSlicing {
    bool ok = false;
    std::int64_t rows = 0;       // the leading extent that is cut
    std::vector<char> carries;   // per node: 1 when the value is cut along its leading dimension
};

// Finds the largest set of graph inputs with a common leading extent such that cutting them (and every value
// computed from them) by rows leaves each op separable: elementwise ops with aligned leading dimensions, matmuls
// whose left operand is cut and whose right operand is not, row reductions over a trailing dimension. Every
// graph output must be a computed, cut value. ok = false when no such set exists.
RowSlicing analyze_row_slicing(const Graph& graph);

// The same graph with the leading extent of every cut value replaced by `rows` (node ids are preserved).
Result<Graph> with_leading_extent(const Graph& graph, const RowSlicing& slicing, std::int64_t rows);

}  // namespace minicompiler::cuda
