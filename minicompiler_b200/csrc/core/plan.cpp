#include "core/plan.hpp"

#include <algorithm>
#include <numeric>

namespace minicompiler {

std::size_t MemoryPlan::bytes_with_reuse() const {
    return std::accumulate(buffer_bytes.begin(), buffer_bytes.end(), std::size_t{0});
}

std::size_t PoolPlan::bytes_with_reuse() const {
    return std::accumulate(buffer_bytes.begin(), buffer_bytes.end(), std::size_t{0});
}

PoolPlan plan_pool(const std::vector<PoolValue>& values, const std::vector<PoolStep>& steps) {
    constexpr std::int32_t kNever = -1;
    const auto end_of_time = static_cast<std::int32_t>(steps.size());
    PoolPlan plan;
    plan.buffer_of.assign(values.size(), PoolPlan::kNotPooled);

    std::vector<std::int32_t> final_read(values.size(), kNever);
    for (std::size_t s = 0; s < steps.size(); ++s) {
        for (std::int32_t v : steps[s].reads) final_read[static_cast<std::size_t>(v)] = static_cast<std::int32_t>(s);
    }
    for (std::size_t v = 0; v < values.size(); ++v) {
        if (values[v].live_out) final_read[v] = end_of_time;
    }

    std::vector<std::int32_t> idle;  // buffers holding no live value, in release order
    for (std::size_t s = 0; s < steps.size(); ++s) {
        const PoolStep& step = steps[s];
        for (std::int32_t v : step.defines) {
            const PoolValue& value = values[static_cast<std::size_t>(v)];
            if (!value.pooled) continue;
            plan.bytes_without_reuse += value.bytes;

            auto pick = idle.end();
            for (auto it = idle.begin(); it != idle.end(); ++it) {  // smallest buffer that is large enough
                const std::size_t have = plan.buffer_bytes[static_cast<std::size_t>(*it)];
                if (have < value.bytes) continue;
                if (pick == idle.end() || have < plan.buffer_bytes[static_cast<std::size_t>(*pick)]) pick = it;
            }
            if (pick == idle.end() && !idle.empty()) {  // none fits: enlarge the biggest idle one
                pick = std::max_element(idle.begin(), idle.end(), [&](std::int32_t a, std::int32_t b) {
                    return plan.buffer_bytes[static_cast<std::size_t>(a)] < plan.buffer_bytes[static_cast<std::size_t>(b)];
                });
                plan.buffer_bytes[static_cast<std::size_t>(*pick)] = value.bytes;
            }
            if (pick != idle.end()) {
                plan.buffer_of[static_cast<std::size_t>(v)] = *pick;
                idle.erase(pick);
            } else {
                plan.buffer_of[static_cast<std::size_t>(v)] = static_cast<std::int32_t>(plan.buffer_bytes.size());
                plan.buffer_bytes.push_back(value.bytes);
            }
        }
        // Operands are released only now, after the outputs have their buffers.
        for (std::size_t k = 0; k < step.reads.size(); ++k) {
            const std::int32_t v = step.reads[k];
            const bool seen_before = std::find(step.reads.begin(), step.reads.begin() + static_cast<std::ptrdiff_t>(k), v) !=
                                     step.reads.begin() + static_cast<std::ptrdiff_t>(k);
            if (seen_before) continue;
            const auto vi = static_cast<std::size_t>(v);
            if (plan.buffer_of[vi] != PoolPlan::kNotPooled && final_read[vi] == static_cast<std::int32_t>(s)) {
                idle.push_back(plan.buffer_of[vi]);
            }
        }
        for (std::int32_t v : step.defines) {
            const auto vi = static_cast<std::size_t>(v);
            if (plan.buffer_of[vi] != PoolPlan::kNotPooled && final_read[vi] == kNever) idle.push_back(plan.buffer_of[vi]);
        }
    }
    return plan;
}

MemoryPlan plan_memory(const Graph& graph, const PlanOptions& options) {
    const std::size_t count = graph.num_nodes();
    MemoryPlan plan;
    plan.last_use.assign(count, kNoNode);
    for (std::size_t i = 0; i < count; ++i) {
        for (NodeId in : graph.node(static_cast<NodeId>(i)).inputs) {
            plan.last_use[static_cast<std::size_t>(in)] = static_cast<NodeId>(i);
        }
    }
    for (NodeId out : graph.outputs()) plan.last_use[static_cast<std::size_t>(out)] = static_cast<NodeId>(count);

    // One value per node; one step per compute node.
    std::vector<PoolValue> values(count);
    std::vector<PoolStep> steps;
    for (std::size_t i = 0; i < count; ++i) {
        const auto id = static_cast<NodeId>(i);
        const Node& n = graph.node(id);
        values[i].bytes = n.type.size_bytes();
        values[i].pooled = is_compute(n.op) && (options.pool_outputs || !graph.is_output(id));
        values[i].live_out = graph.is_output(id);
        if (!is_compute(n.op)) continue;
        PoolStep step;
        step.defines.push_back(id);
        step.reads.assign(n.inputs.begin(), n.inputs.end());
        steps.push_back(std::move(step));
    }
    PoolPlan pool = plan_pool(values, steps);
    plan.buffer_of = std::move(pool.buffer_of);
    plan.buffer_bytes = std::move(pool.buffer_bytes);
    plan.bytes_without_reuse = pool.bytes_without_reuse;
    return plan;
}

}  // namespace minicompiler
