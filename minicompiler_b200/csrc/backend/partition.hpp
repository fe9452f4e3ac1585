#pragma once
// Batch-dimension partitioning of a graph over the GPUs of one box. The reference
// has no multi-GPU path; this is the new partitioner. Every op of the IR is
// row-independent in the leading dimension (elementwise ops act per element and
// `matmul x[B,K], w[K,N]` is independent per row of x), so a graph whose batch
// dim appears only as the leading extent of activations can be cut into row
// shards with no exchange between layers: each rank compiles the same graph file
// with the batch dim overridden to its share (the reference's own dim override,
// src/parser.cpp:214-227) and constants, whose seeds do not depend on the batch,
// are identical on every rank.

#include "core/mcg.hpp"

#include <cstdint>
#include <string>
#include <vector>

namespace minicompiler {

struct ShardPlan {
    std::map<std::string, std::int64_t> dims;  // dim overrides for this rank
    std::int64_t batch = 0;                    // the unsharded extent
    std::int64_t rows = 0;                     // this rank's share
    std::int64_t row_offset = 0;               // first row of the share
    std::vector<bool> input_is_sharded;        // per graph input
    std::vector<bool> output_is_sharded;       // per graph output
};

// Checks that `text` can be sharded along dim `batch_dim` and returns rank `rank`'s plan.
// Rejected: a batch extent that is not a multiple of `world_size`; a tensor carrying the
// batch dim anywhere but as its leading extent; a constant or a matmul right-hand side
// that carries it; a graph that no longer type-checks with the smaller batch.
Result<ShardPlan> plan_batch_shard(std::string_view text, const std::map<std::string, std::int64_t>& dims,
                                   const std::string& batch_dim, int rank, int world_size);

}  // namespace minicompiler
