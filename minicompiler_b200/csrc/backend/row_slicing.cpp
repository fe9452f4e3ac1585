#include "backend/row_slicing.hpp"

namespace minicompiler::cuda {

namespace {

// Propagates "is cut by rows" from the chosen inputs; false when some op would mix rows.
bool propagate(const Graph& graph, std::int64_t rows, std::vector<char>* carries) {
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const Node& n = graph.node(static_cast<NodeId>(i));
        if (!is_compute(n.op)) continue;
        char& mine = (*carries)[i];
        mine = 0;
        if (n.op == OpKind::MatMul) {
            if ((*carries)[static_cast<std::size_t>(n.inputs[1])]) return false;  // rows of the right operand are summed over
            mine = (*carries)[static_cast<std::size_t>(n.inputs[0])];
            continue;
        }
        if (is_row_reduce(n.op)) {
            const char in = (*carries)[static_cast<std::size_t>(n.inputs[0])];
            if (in && graph.node(n.inputs[0]).type.rank() < 2) return false;  // it would reduce over the cut dimension
            mine = in;
            continue;
        }
        // Elementwise (single op or fused program): operands broadcast against the result's shape from the right.
        bool any = false;
        for (NodeId in : n.inputs) any = any || (*carries)[static_cast<std::size_t>(in)];
        if (!any) continue;
        const std::size_t rank = n.type.rank();
        if (rank == 0 || n.type.shape[0] != rows) return false;
        for (NodeId in : n.inputs) {
            const TensorType& t = graph.node(in).type;
            if ((*carries)[static_cast<std::size_t>(in)]) {
                if (t.rank() != rank) return false;  // its leading dimension is not the result's leading dimension
            } else if (t.rank() == rank && t.shape[0] != 1) {
                return false;  // a full-height operand that is not cut: each slice would need its own rows of it
            }
        }
        mine = 1;
    }
    return true;
}

}  // namespace

RowSlicing analyze_row_slicing(const Graph& graph) {
    RowSlicing best;
    std::int64_t rows = 0;
    for (NodeId in : graph.inputs()) {
        const TensorType& t = graph.node(in).type;
        if (t.rank() >= 2 && t.shape[0] > 1) {
            rows = t.shape[0];
            break;
        }
    }
    if (rows == 0) return best;
    std::vector<NodeId> candidates;
    for (NodeId in : graph.inputs()) {
        const TensorType& t = graph.node(in).type;
        if (t.rank() >= 1 && t.shape[0] == rows) candidates.push_back(in);
    }
    if (candidates.empty() || candidates.size() > 10) return best;
    int best_count = 0;
    for (unsigned mask = 1; mask < (1u << candidates.size()); ++mask) {
        const int count = __builtin_popcount(mask);
        if (count <= best_count) continue;
        std::vector<char> carries(graph.num_nodes(), 0);
        for (std::size_t c = 0; c < candidates.size(); ++c) {
            if (mask & (1u << c)) carries[static_cast<std::size_t>(candidates[c])] = 1;
        }
        if (!propagate(graph, rows, &carries)) continue;
        bool outputs_cut = !graph.outputs().empty();
        for (NodeId o : graph.outputs()) {
            outputs_cut = outputs_cut && carries[static_cast<std::size_t>(o)] && is_compute(graph.node(o).op);
        }
        if (!outputs_cut) continue;
        best.ok = true;
        best.rows = rows;
        best.carries = std::move(carries);
        best_count = count;
    }
    return best;
}

Result<Graph> with_leading_extent(const Graph& graph, const RowSlicing& slicing, std::int64_t rows) {
    Graph out(graph.name());
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const Node& n = graph.node(static_cast<NodeId>(i));
        TensorType type = n.type;
        if (slicing.carries[i]) type.shape[0] = rows;
        Result<NodeId> id = Error{"unreachable"};
        switch (n.op) {
            case OpKind::Input: id = out.add_input(n.name, type); break;
            case OpKind::Constant: id = out.add_constant(n.name, type, n.constant); break;
            case OpKind::FusedElementwise: id = out.add_fused(n.inputs, n.fused, type, n.name); break;
            default: id = out.add_op(n.op, n.inputs, n.name); break;
        }
        if (!id.ok()) return id.error();
        if (*id != static_cast<NodeId>(i) || out.node(*id).type.shape != type.shape) {
            return Error{"'" + n.name + "' does not keep its place or shape when the leading extent changes"};
        }
    }
    for (NodeId o : graph.outputs()) MC_TRY(out.add_output(o));
    return out;
}

}  // namespace minicompiler::cuda
