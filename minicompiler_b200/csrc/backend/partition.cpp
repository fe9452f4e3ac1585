#include "backend/partition.hpp"

namespace minicompiler {

Result<ShardPlan> plan_batch_shard(std::string_view text, const std::map<std::string, std::int64_t>& dims,
                                   const std::string& batch_dim, int rank, int world_size) {
    if (world_size < 1 || rank < 0 || rank >= world_size) {
        return Error{"rank " + std::to_string(rank) + " is outside a world of " + std::to_string(world_size)};
    }
    std::map<std::string, std::int64_t> resolved;
    ParseOptions whole_options;
    whole_options.dims = dims;
    whole_options.resolved_dims = &resolved;
    MC_ASSIGN(whole, parse_graph(text, whole_options));
    const auto found = resolved.find(batch_dim);
    if (found == resolved.end()) return Error{"the graph declares no dim '" + batch_dim + "'"};
    const std::int64_t batch = found->second;
    if (batch % world_size != 0) {
        return Error{"dim '" + batch_dim + "' = " + std::to_string(batch) + " does not divide over " +
                     std::to_string(world_size) + " devices"};
    }

    ShardPlan plan;
    plan.dims = dims;
    plan.batch = batch;
    plan.rows = batch / world_size;
    plan.row_offset = plan.rows * rank;
    plan.dims[batch_dim] = plan.rows;
    if (world_size == 1) {
        plan.input_is_sharded.assign(whole.inputs().size(), false);
        plan.output_is_sharded.assign(whole.outputs().size(), false);
        return plan;
    }

    // Compare the graph at the full batch and at a different batch: every value whose type moved carries
    // the batch dim. (With a one-row share the two could coincide only if batch == 1, excluded above.)
    ParseOptions part_options;
    part_options.dims = plan.dims;
    Result<Graph> part = parse_graph(text, part_options);
    if (!part.ok()) return Error{"the graph does not type-check with '" + batch_dim + "' sharded: " + part.error().message};
    if (part->num_nodes() != whole.num_nodes()) return Error{"the graph changes structure with the batch size"};

    std::vector<bool> carries(whole.num_nodes(), false);
    for (std::size_t i = 0; i < whole.num_nodes(); ++i) {
        const Node& a = whole.node(static_cast<NodeId>(i));
        const Node& b = part->node(static_cast<NodeId>(i));
        if (a.type.shape == b.type.shape) continue;
        const std::string what = "'" + a.name + "' : " + to_string(a.type);
        bool leading_only = a.type.rank() == b.type.rank() && a.type.rank() >= 1 && a.type.shape[0] == batch &&
                            b.type.shape[0] == plan.rows;
        for (std::size_t d = 1; leading_only && d < a.type.rank(); ++d) leading_only = a.type.shape[d] == b.type.shape[d];
        if (!leading_only) return Error{what + " carries dim '" + batch_dim + "' other than as its leading extent"};
        if (a.op == OpKind::Constant) return Error{"constant " + what + " carries dim '" + batch_dim + "'"};
        carries[i] = true;
    }
    for (std::size_t i = 0; i < whole.num_nodes(); ++i) {
        const Node& n = whole.node(static_cast<NodeId>(i));
        if (n.op == OpKind::MatMul && carries[static_cast<std::size_t>(n.inputs[1])]) {
            return Error{"matmul '" + n.name + "' has a right-hand side that carries dim '" + batch_dim +
                         "': its rows would need an exchange between devices"};
        }
        if (is_row_reduce(n.op) && carries[static_cast<std::size_t>(n.inputs[0])] && whole.node(n.inputs[0]).type.rank() < 2) {
            return Error{std::string(op_name(n.op)) + " '" + n.name + "' reduces over dim '" + batch_dim +
                         "': its partial results would need an exchange between devices"};
        }
        // A batch-carrying operand broadcast against a same-extent non-batch operand would silently change meaning.
        if (is_binary_elementwise(n.op) && carries[i]) {
            for (NodeId in : n.inputs) {
                const Node& operand = whole.node(in);
                if (!carries[static_cast<std::size_t>(in)] && operand.type.rank() == n.type.rank() &&
                    operand.type.rank() >= 1 && operand.type.shape[0] == batch && batch != 1) {
                    return Error{"'" + operand.name + "' has leading extent " + std::to_string(batch) +
                                 " but does not carry dim '" + batch_dim + "'"};
                }
            }
        }
    }
    for (NodeId in : whole.inputs()) plan.input_is_sharded.push_back(carries[static_cast<std::size_t>(in)]);
    for (NodeId o : whole.outputs()) plan.output_is_sharded.push_back(carries[static_cast<std::size_t>(o)]);
    return plan;
}

}  // namespace minicompiler
