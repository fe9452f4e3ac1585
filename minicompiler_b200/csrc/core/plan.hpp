#pragma once
// Lifetime-based buffer planning. Steps run in order; a value is live from the
// step that defines it to the last step that reads it (graph outputs to the
// end), and values whose lifetimes do not overlap share a buffer. Placement
// policy is the reference's (src/runtime/memory_plan.cpp:12-70): best fit among
// the free buffers, else grow the largest free one, else open a new one; a
// step's output is placed before its operands are released, so no step writes
// a buffer it still reads; a value nobody reads is released at once.
//
// plan_memory() is the reference's node-level entry point. plan_pool() is the
// same policy over an arbitrary step list, which the GPU backend uses after
// lowering (a lowered step can define two copies of a value, and a matmul whose
// consumer was folded into its epilogue defines nothing of its own).

#include "core/ir.hpp"

#include <cstddef>
#include <cstdint>
#include <vector>

namespace minicompiler {

struct PlanOptions {
    bool pool_outputs = true;  // false: graph outputs live in caller memory
};

struct MemoryPlan {
    static constexpr std::int32_t kNotPooled = -1;

    std::vector<std::int32_t> buffer_of;    // per node
    std::vector<std::size_t> buffer_bytes;  // per buffer
    std::vector<NodeId> last_use;           // per node: last reader, num_nodes() for outputs, kNoNode if unread
    std::size_t bytes_without_reuse = 0;
    std::size_t bytes_with_reuse() const;
};

MemoryPlan plan_memory(const Graph& graph, const PlanOptions& options = {});

struct PoolValue {
    std::size_t bytes = 0;
    bool pooled = true;     // false: lives elsewhere (inputs, constants)
    bool live_out = false;  // stays live past the last step
};

struct PoolStep {
    std::vector<std::int32_t> defines;  // value indices
    std::vector<std::int32_t> reads;    // value indices
};

struct PoolPlan {
    static constexpr std::int32_t kNotPooled = -1;
    std::vector<std::int32_t> buffer_of;  // per value
    std::vector<std::size_t> buffer_bytes;
    std::size_t bytes_without_reuse = 0;
    std::size_t bytes_with_reuse() const;
};

PoolPlan plan_pool(const std::vector<PoolValue>& values, const std::vector<PoolStep>& steps);

}  // namespace minicompiler
