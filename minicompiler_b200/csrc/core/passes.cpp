// dne / fold / fuse and the pipeline driver. Semantics follow the reference's
// src/passes/{dead_node_elimination,constant_folding,operator_fusion,pipeline}.cpp;
// its tests pin the fusion groups, folded values and stage counts.

#include "core/passes.hpp"

#include <algorithm>
#include <cmath>
#include <map>
#include <queue>

namespace minicompiler {

namespace {

void report_pass(PassReport* report, const char* pass, const Graph& before, const Graph& after, std::string summary) {
    if (report == nullptr) return;
    report->pass = pass;
    report->before = compute_stats(before);
    report->after = compute_stats(after);
    report->summary = std::move(summary);
}

// Copies the graph's output list through an old-id -> new-id map.
Status carry_outputs(const Graph& from, const std::vector<NodeId>& new_id, Graph& to) {
    for (NodeId out : from.outputs()) MC_TRY(to.add_output(new_id[static_cast<std::size_t>(out)]));
    return Status();
}

std::vector<NodeId> mapped(const std::vector<NodeId>& ids, const std::vector<NodeId>& new_id) {
    std::vector<NodeId> out;
    out.reserve(ids.size());
    for (NodeId id : ids) out.push_back(new_id[static_cast<std::size_t>(id)]);
    return out;
}

}  // namespace

// -------------------------------------------------------------------- dne

Result<Graph> eliminate_dead_nodes(const Graph& graph, PassReport* report) {
    const std::size_t count = graph.num_nodes();
    std::vector<char> needed(count, 0);
    for (NodeId out : graph.outputs()) needed[static_cast<std::size_t>(out)] = 1;
    // Users come after producers, so one sweep from the back reaches everything.
    for (std::size_t i = count; i-- > 0;) {
        if (!needed[i]) continue;
        for (NodeId in : graph.node(static_cast<NodeId>(i)).inputs) needed[static_cast<std::size_t>(in)] = 1;
    }
    for (NodeId in : graph.inputs()) needed[static_cast<std::size_t>(in)] = 1;  // calling convention

    Graph kept(graph.name());
    std::vector<NodeId> new_id(count, kNoNode);
    std::size_t dropped = 0;
    for (std::size_t i = 0; i < count; ++i) {
        if (!needed[i]) {
            ++dropped;
            continue;
        }
        const Node& n = graph.node(static_cast<NodeId>(i));
        MC_ASSIGN(id, kept.copy_node(n, mapped(n.inputs, new_id)));
        new_id[i] = id;
    }
    MC_TRY(carry_outputs(graph, new_id, kept));
    report_pass(report, "dne", graph, kept, "removed " + std::to_string(dropped) + " dead node(s)");
    return kept;
}

// ------------------------------------------------------------------- fold

namespace {

float host_unary(OpKind op, float x) {
    switch (op) {
        case OpKind::Neg: return -x;
        case OpKind::Exp: return std::exp(x);
        case OpKind::Log: return std::log(x);
        case OpKind::Sqrt: return std::sqrt(x);
        case OpKind::Relu: return x > 0.0f ? x : 0.0f;
        case OpKind::Sigmoid: return 1.0f / (1.0f + std::exp(-x));
        case OpKind::Tanh: return std::tanh(x);
        default: return 0.0f;
    }
}

float host_binary(OpKind op, float a, float b) {
    switch (op) {
        case OpKind::Add: return a + b;
        case OpKind::Sub: return a - b;
        case OpKind::Mul: return a * b;
        case OpKind::Div: return a / b;
        default: return 0.0f;
    }
}

// Linear output index -> element offset of an operand read with broadcast strides.
std::int64_t operand_offset(std::size_t linear, const Shape& out, const std::vector<std::int64_t>& strides) {
    std::int64_t off = 0;
    for (std::size_t d = out.size(); d-- > 0;) {
        const auto extent = static_cast<std::size_t>(out[d]);
        off += static_cast<std::int64_t>(linear % extent) * strides[d];
        linear /= extent;
    }
    return off;
}

}  // namespace

void evaluate_node_on_host(const Node& node, const std::vector<const float*>& operands,
                           const std::vector<Shape>& operand_shapes, float* out) {
    const Shape& oshape = node.type.shape;
    const std::size_t count = node.type.num_elements();
    if (node.op == OpKind::MatMul) {
        const std::int64_t m = operand_shapes[0][0], k = operand_shapes[0][1], n = operand_shapes[1][1];
        for (std::int64_t r = 0; r < m; ++r) {
            for (std::int64_t c = 0; c < n; ++c) {
                float acc = 0.0f;
                for (std::int64_t t = 0; t < k; ++t) acc += operands[0][r * k + t] * operands[1][t * n + c];
                out[r * n + c] = acc;
            }
        }
        return;
    }
    if (is_row_reduce(node.op)) {
        // One result per row of the operand's last dimension; sums accumulate in double and round once.
        const std::int64_t width = operand_shapes[0].back();
        for (std::size_t r = 0; r < count; ++r) {
            const float* row = operands[0] + static_cast<std::int64_t>(r) * width;
            if (node.op == OpKind::RowSum) {
                double acc = 0.0;
                for (std::int64_t c = 0; c < width; ++c) acc += static_cast<double>(row[c]);
                out[r] = static_cast<float>(acc);
            } else {
                float best = row[0];
                for (std::int64_t c = 1; c < width; ++c) best = row[c] > best ? row[c] : best;
                out[r] = best;
            }
        }
        return;
    }
    std::vector<std::vector<std::int64_t>> strides;
    for (const Shape& s : operand_shapes) strides.push_back(broadcast_strides(s, oshape));
    if (node.op == OpKind::FusedElementwise) {
        const FusedProgram& program = *node.fused;
        std::vector<float> regs(program.instrs.size());
        for (std::size_t e = 0; e < count; ++e) {
            for (std::size_t r = 0; r < program.instrs.size(); ++r) {
                const FusedInstr& ins = program.instrs[r];
                switch (ins.kind) {
                    case FusedInstr::Kind::Load:
                        regs[r] = operands[static_cast<std::size_t>(ins.a)]
                                          [operand_offset(e, oshape, strides[static_cast<std::size_t>(ins.a)])];
                        break;
                    case FusedInstr::Kind::Immediate: regs[r] = ins.immediate; break;
                    case FusedInstr::Kind::Unary: regs[r] = host_unary(ins.op, regs[static_cast<std::size_t>(ins.a)]); break;
                    case FusedInstr::Kind::Binary:
                        regs[r] = host_binary(ins.op, regs[static_cast<std::size_t>(ins.a)],
                                              regs[static_cast<std::size_t>(ins.b)]);
                        break;
                }
            }
            out[e] = regs.back();
        }
        return;
    }
    for (std::size_t e = 0; e < count; ++e) {
        const float a = operands[0][operand_offset(e, oshape, strides[0])];
        out[e] = is_unary_elementwise(node.op)
                     ? host_unary(node.op, a)
                     : host_binary(node.op, a, operands[1][operand_offset(e, oshape, strides[1])]);
    }
}

Result<Graph> fold_constants(const Graph& graph, PassReport* report, const ConstantFoldingOptions& options) {
    Graph folded(graph.name());
    std::vector<NodeId> new_id(graph.num_nodes(), kNoNode);
    std::size_t hits = 0;
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const Node& n = graph.node(static_cast<NodeId>(i));
        std::vector<NodeId> ins = mapped(n.inputs, new_id);
        bool foldable = is_compute(n.op) && !ins.empty() && n.type.num_elements() <= options.max_elements;
        for (NodeId in : ins) foldable = foldable && folded.node(in).op == OpKind::Constant;
        if (foldable) {
            std::vector<const float*> data;
            std::vector<Shape> shapes;
            for (NodeId in : ins) {
                data.push_back(folded.node(in).constant->data());
                shapes.push_back(folded.node(in).type.shape);
            }
            std::vector<float> values(n.type.num_elements());
            evaluate_node_on_host(n, data, shapes, values.data());
            MC_ASSIGN(id, folded.add_constant(n.name, n.type, std::move(values)));
            new_id[i] = id;
            ++hits;
        } else {
            MC_ASSIGN(id, folded.copy_node(n, std::move(ins)));
            new_id[i] = id;
        }
    }
    MC_TRY(carry_outputs(graph, new_id, folded));
    report_pass(report, "fold", graph, folded, "folded " + std::to_string(hits) + " node(s) into constants");
    return folded;
}

// ------------------------------------------------------------------- fuse

std::vector<std::vector<NodeId>> find_fusion_groups(const Graph& graph) {
    const std::size_t count = graph.num_nodes();
    const std::vector<std::vector<NodeId>> users = graph.compute_users();
    std::vector<std::int32_t> owner(count, -1);
    std::vector<std::vector<NodeId>> groups;  // in order of discovery: roots descending

    for (std::size_t i = count; i-- > 0;) {
        const auto root = static_cast<NodeId>(i);
        const Node& root_node = graph.node(root);
        if (owner[i] != -1 || !is_elementwise(root_node.op)) continue;

        const auto gid = static_cast<std::int32_t>(groups.size());
        owner[i] = gid;
        std::vector<NodeId> members{root};
        // Producers are examined from the highest id down, so by the time one
        // is looked at every user that could have joined has been decided.
        std::priority_queue<NodeId> frontier;
        for (NodeId in : root_node.inputs) frontier.push(in);
        while (!frontier.empty()) {
            const NodeId p = frontier.top();
            frontier.pop();
            const auto pi = static_cast<std::size_t>(p);
            if (owner[pi] != -1) continue;
            const Node& pn = graph.node(p);
            const bool joins = is_elementwise(pn.op) && pn.type.shape == root_node.type.shape &&
                               !graph.is_output(p) &&
                               std::all_of(users[pi].begin(), users[pi].end(),
                                           [&](NodeId u) { return owner[static_cast<std::size_t>(u)] == gid; });
            if (!joins) continue;
            owner[pi] = gid;
            members.push_back(p);
            for (NodeId in : pn.inputs) frontier.push(in);
        }
        std::sort(members.begin(), members.end());
        groups.push_back(std::move(members));
    }

    std::vector<std::vector<NodeId>> result;
    for (auto g = groups.rbegin(); g != groups.rend(); ++g) {
        if (g->size() >= 2) result.push_back(std::move(*g));
    }
    return result;
}

namespace {

// Builds the straight-line program of one group. External operands are loaded
// once each, in first-use order; one-element constants become immediates.
struct GroupLowering {
    const Graph& graph;
    const std::vector<NodeId>& new_id;
    std::shared_ptr<FusedProgram> program = std::make_shared<FusedProgram>();
    std::vector<NodeId> externals;  // ids in the graph being built
    std::map<NodeId, std::int32_t> reg_of;

    std::int32_t define(NodeId id, FusedInstr ins) {
        program->instrs.push_back(ins);
        const auto reg = static_cast<std::int32_t>(program->instrs.size()) - 1;
        reg_of[id] = reg;
        return reg;
    }

    std::int32_t reg_for(NodeId id) {
        const auto hit = reg_of.find(id);
        if (hit != reg_of.end()) return hit->second;
        const Node& n = graph.node(id);
        if (n.op == OpKind::Constant && n.type.num_elements() == 1) return define(id, FusedInstr::imm(n.constant->at(0)));
        externals.push_back(new_id[static_cast<std::size_t>(id)]);
        return define(id, FusedInstr::load(static_cast<std::int32_t>(externals.size()) - 1));
    }

    void lower(NodeId id) {
        const Node& n = graph.node(id);
        const std::int32_t lhs = reg_for(n.inputs[0]);
        if (is_unary_elementwise(n.op)) {
            define(id, FusedInstr::unary(n.op, lhs));
        } else {
            const std::int32_t rhs = reg_for(n.inputs[1]);  // strictly after lhs: keeps register order fixed
            define(id, FusedInstr::binary(n.op, lhs, rhs));
        }
        program->source_nodes.push_back(n.name);
    }
};

}  // namespace

Result<Graph> fuse_elementwise(const Graph& graph, PassReport* report) {
    const std::vector<std::vector<NodeId>> groups = find_fusion_groups(graph);
    std::vector<std::int32_t> group_of(graph.num_nodes(), -1);
    for (std::size_t g = 0; g < groups.size(); ++g) {
        for (NodeId m : groups[g]) group_of[static_cast<std::size_t>(m)] = static_cast<std::int32_t>(g);
    }

    Graph fused(graph.name());
    std::vector<NodeId> new_id(graph.num_nodes(), kNoNode);
    std::size_t ops_fused = 0;
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const auto id = static_cast<NodeId>(i);
        const Node& n = graph.node(id);
        if (group_of[i] < 0) {
            MC_ASSIGN(copied, fused.copy_node(n, mapped(n.inputs, new_id)));
            new_id[i] = copied;
            continue;
        }
        const std::vector<NodeId>& members = groups[static_cast<std::size_t>(group_of[i])];
        if (id != members.back()) continue;  // the whole group is emitted where its root stood
        GroupLowering lowering{graph, new_id, std::make_shared<FusedProgram>(), {}, {}};
        for (NodeId m : members) lowering.lower(m);
        MC_ASSIGN(node_id, fused.add_fused(lowering.externals, lowering.program, n.type, n.name));
        new_id[i] = node_id;
        ops_fused += members.size();
    }
    MC_TRY(carry_outputs(graph, new_id, fused));
    report_pass(report, "fuse", graph, fused,
                "fused " + std::to_string(ops_fused) + " op(s) into " + std::to_string(groups.size()) + " kernel(s)");
    return fused;
}

// --------------------------------------------------------------- pipeline

const std::vector<PassInfo>& registered_passes() {
    static const std::vector<PassInfo> table = {
        {"dne", "dead-node elimination: remove nodes no output depends on", &eliminate_dead_nodes},
        {"fold", "constant folding: evaluate nodes whose operands are all constants",
         [](const Graph& g, PassReport* r) { return fold_constants(g, r); }},
        {"fuse", "operator fusion: merge groups of elementwise ops into single kernels", &fuse_elementwise},
    };
    return table;
}

const std::vector<std::string>& default_pipeline() {
    static const std::vector<std::string> order = {"dne", "fold", "dne", "fuse", "dne"};
    return order;
}

namespace {

const PassInfo* lookup_pass(std::string_view name) {
    for (const PassInfo& p : registered_passes()) {
        if (name == p.name) return &p;
    }
    return nullptr;
}

}  // namespace

Result<std::vector<std::string>> parse_pipeline(std::string_view spec) {
    if (spec == "default") return default_pipeline();
    if (spec.empty() || spec == "none") return std::vector<std::string>{};
    std::vector<std::string> names;
    std::size_t from = 0;
    for (;;) {
        std::size_t to = spec.find(',', from);
        if (to == std::string_view::npos) to = spec.size();
        const std::string_view name = spec.substr(from, to - from);
        if (lookup_pass(name) == nullptr) {
            std::string known;
            for (const PassInfo& p : registered_passes()) known += (known.empty() ? "" : ", ") + std::string(p.name);
            return Error{"unknown pass '" + std::string(name) + "' (passes: " + known + ")"};
        }
        names.emplace_back(name);
        if (to == spec.size()) break;
        from = to + 1;
    }
    return names;
}

Result<Graph> run_pipeline(const Graph& graph, const std::vector<std::string>& passes, std::vector<PassReport>* reports,
                           const PassObserver& observer) {
    Status st = graph.verify();
    if (!st.ok()) return Error{"input graph is invalid: " + st.message()};
    Graph current = graph;
    if (observer) observer(0, "input", current);
    for (std::size_t i = 0; i < passes.size(); ++i) {
        const PassInfo* pass = lookup_pass(passes[i]);
        if (pass == nullptr) return Error{"unknown pass '" + passes[i] + "'"};
        PassReport report;
        Result<Graph> next = pass->run(current, &report);
        if (!next.ok()) return Error{"pass '" + passes[i] + "' failed: " + next.error().message};
        st = next->verify();
        if (!st.ok()) return Error{"pass '" + passes[i] + "' produced an invalid graph: " + st.message()};
        current = std::move(next).value();
        if (reports != nullptr) reports->push_back(std::move(report));
        if (observer) observer(i + 1, passes[i], current);
    }
    return current;
}

}  // namespace minicompiler
