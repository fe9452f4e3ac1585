#pragma once
// The kept pass pipeline: dne -> fold -> dne -> fuse -> dne. Each pass builds a
// new graph and the driver re-verifies it, as in the reference
// (include/minicompiler/passes/*.hpp, src/passes/*.cpp).

#include "core/ir.hpp"

#include <cstddef>
#include <functional>
#include <string>
#include <string_view>
#include <vector>

namespace minicompiler {

struct PassReport {
    std::string pass;
    GraphStats before;
    GraphStats after;
    std::string summary;
};

// Drops every node no output depends on; graph inputs always stay
// (src/passes/dead_node_elimination.cpp:7-42).
Result<Graph> eliminate_dead_nodes(const Graph& graph, PassReport* report = nullptr);

struct ConstantFoldingOptions {
    std::size_t max_elements = std::size_t{1} << 22;  // larger results stay runtime work
};

// A compute node whose operands are all constants becomes a constant, computed
// on the host at compile time (src/passes/constant_folding.cpp:10-51).
Result<Graph> fold_constants(const Graph& graph, PassReport* report = nullptr,
                             const ConstantFoldingOptions& options = {});

// Groups of same-shape elementwise nodes whose values never leave the group
// (src/passes/operator_fusion.cpp:10-51). Members ascending, root last.
std::vector<std::vector<NodeId>> find_fusion_groups(const Graph& graph);
// Each group becomes one FusedElementwise node at the root's position.
Result<Graph> fuse_elementwise(const Graph& graph, PassReport* report = nullptr);

using PassFn = Result<Graph> (*)(const Graph&, PassReport*);
struct PassInfo {
    const char* name;
    const char* description;
    PassFn run;
};

const std::vector<PassInfo>& registered_passes();
const std::vector<std::string>& default_pipeline();
// "default", "none"/"" or a comma list of dne|fold|fuse.
Result<std::vector<std::string>> parse_pipeline(std::string_view spec);

using PassObserver = std::function<void(std::size_t stage, const std::string& pass, const Graph& graph)>;
Result<Graph> run_pipeline(const Graph& graph, const std::vector<std::string>& passes,
                           std::vector<PassReport>* reports = nullptr, const PassObserver& observer = {});

// Host evaluation of one compute node on row-major float buffers, used only by
// constant folding. Float arithmetic with every op rounded to float; libm for
// the transcendental ops.
void evaluate_node_on_host(const Node& node, const std::vector<const float*>& operands,
                           const std::vector<Shape>& operand_shapes, float* out);

}  // namespace minicompiler
