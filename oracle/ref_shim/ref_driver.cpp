// C-ABI driver over the reference's own host code, compiled from the sources under
// the read-only reference checkout (parser, IR, passes, planner, elementwise code
// generator, and its tests' double-precision evaluator and random-graph generator).
// It exists so that tests can compare this repository's host logic and its CPU
// oracle with what the reference itself computes on the same inputs.
// TEST INFRASTRUCTURE ONLY: the product never links or loads this.
#include "cuda/codegen.hpp"
#include "minicompiler/parser.hpp"
#include "minicompiler/passes/operator_fusion.hpp"
#include "minicompiler/passes/pipeline.hpp"
#include "minicompiler/random.hpp"
#include "minicompiler/runtime/host_tensor.hpp"
#include "minicompiler/runtime/memory_plan.hpp"
#include "test_util.hpp"

#include <cstdio>
#include <cstring>
#include <sstream>
#include <string>

using namespace minicompiler;

namespace {

thread_local std::string g_text;

struct RefGraph {
    Graph graph;
    std::vector<std::size_t> stage_nodes;
    std::vector<std::size_t> stage_compute;
};

int give(const std::string& text, char* out, int size) {
    if (out != nullptr && size > 0) std::snprintf(out, static_cast<std::size_t>(size), "%s", text.c_str());
    return static_cast<int>(text.size());
}

ParseOptions dims_of(const char* dims) {
    ParseOptions options;
    std::stringstream list(dims ? dims : "");
    for (std::string item; std::getline(list, item, ',');) {
        const std::size_t eq = item.find('=');
        if (eq != std::string::npos) options.dims[item.substr(0, eq)] = std::atoll(item.c_str() + eq + 1);
    }
    return options;
}

RefGraph* optimize(Result<Graph> parsed, const char* passes, char* error, int error_size) {
    if (!parsed.ok()) {
        give(parsed.error().message, error, error_size);
        return nullptr;
    }
    Result<std::vector<std::string>> pipeline = parse_pipeline(passes ? passes : "default");
    if (!pipeline.ok()) {
        give(pipeline.error().message, error, error_size);
        return nullptr;
    }
    auto ref = new RefGraph();
    Result<Graph> done = run_pipeline(parsed.value(), pipeline.value(), nullptr,
                                      [&](std::size_t, const std::string&, const Graph& g) {
                                          const GraphStats s = compute_stats(g);
                                          ref->stage_nodes.push_back(s.nodes);
                                          ref->stage_compute.push_back(s.compute_nodes);
                                      });
    if (!done.ok()) {
        give(done.error().message, error, error_size);
        delete ref;
        return nullptr;
    }
    ref->graph = std::move(done).value();
    return ref;
}

// A graph as parseable .mcg text (constants as literal lists; %.9g round-trips a float).
std::string to_mcg(const Graph& g) {
    std::ostringstream os;
    os << "graph " << g.name() << "\n";
    auto shape_text = [](const Shape& s) {
        std::string t = "f32[";
        for (std::size_t i = 0; i < s.size(); ++i) t += (i ? ", " : "") + std::to_string(s[i]);
        return t + "]";
    };
    for (std::size_t i = 0; i < g.num_nodes(); ++i) {
        const Node& n = g.node(static_cast<NodeId>(i));
        if (n.op == OpKind::Input) {
            os << "input " << n.name << " : " << shape_text(n.type.shape) << "\n";
        } else if (n.op == OpKind::Constant) {
            os << "const " << n.name << " : " << shape_text(n.type.shape) << " = [";
            for (std::size_t k = 0; k < n.constant->size(); ++k) {
                char buf[32];
                std::snprintf(buf, sizeof buf, "%.9g", static_cast<double>((*n.constant)[k]));
                os << (k ? ", " : "") << buf;
            }
            os << "]\n";
        } else {
            os << n.name << " = " << op_name(n.op);
            for (std::size_t k = 0; k < n.inputs.size(); ++k) os << (k ? ", " : " ") << g.node(n.inputs[k]).name;
            os << "\n";
        }
    }
    os << "output";
    for (std::size_t k = 0; k < g.outputs().size(); ++k) os << (k ? ", " : " ") << g.node(g.outputs()[k]).name;
    os << "\n";
    return os.str();
}

}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void* ref_open_file(const char* path, const char* dims, const char* passes, char* error, int error_size) {
    return optimize(parse_graph_file(path, dims_of(dims)), passes, error, error_size);
}

REF_API void* ref_open_text(const char* text, const char* dims, const char* passes, char* error, int error_size) {
    return optimize(parse_graph(text, dims_of(dims)), passes, error, error_size);
}

REF_API void ref_close(void* g) { delete static_cast<RefGraph*>(g); }

REF_API int ref_print(const void* g, char* out, int size) { return give(print_graph(static_cast<const RefGraph*>(g)->graph), out, size); }

REF_API int ref_stage_counts(const void* g, char* out, int size) {
    const auto* ref = static_cast<const RefGraph*>(g);
    std::string text;
    for (std::size_t i = 0; i < ref->stage_nodes.size(); ++i) {
        text += (i ? " " : "") + std::to_string(ref->stage_nodes[i]) + "," + std::to_string(ref->stage_compute[i]);
    }
    return give(text, out, size);
}

REF_API int ref_plan(const void* g, int pool_outputs, char* out, int size) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    PlanOptions options;
    options.pool_outputs = pool_outputs != 0;
    const MemoryPlan plan = plan_memory(graph, options);
    std::ostringstream os;
    os << "{\"buffer_of\": [";
    for (std::size_t i = 0; i < plan.buffer_of.size(); ++i) os << (i ? ", " : "") << plan.buffer_of[i];
    os << "], \"buffer_bytes\": [";
    for (std::size_t i = 0; i < plan.buffer_bytes.size(); ++i) os << (i ? ", " : "") << plan.buffer_bytes[i];
    os << "], \"last_use\": [";
    for (std::size_t i = 0; i < plan.last_use.size(); ++i) os << (i ? ", " : "") << plan.last_use[i];
    os << "], \"bytes_without_reuse\": " << plan.bytes_without_reuse << ", \"bytes_with_reuse\": " << plan.bytes_with_reuse()
       << "}";
    return give(os.str(), out, size);
}

REF_API int ref_fusion_groups(const void* g, char* out, int size) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    std::string text;
    for (const std::vector<NodeId>& group : find_fusion_groups(graph)) {
        std::string line;
        for (NodeId m : group) line += (line.empty() ? "" : " ") + graph.node(m).name;
        text += line + "\n";
    }
    return give(text, out, size);
}

// The reference generator's output for every elementwise / fused node ("mcc --emit-cuda").
REF_API int ref_emit_cuda(const void* g, char* out, int size) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    std::string text;
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const Node& n = graph.node(static_cast<NodeId>(i));
        if (!is_elementwise(n.op) && n.op != OpKind::FusedElementwise) continue;
        std::vector<Shape> shapes;
        for (NodeId in : n.inputs) shapes.push_back(graph.node(in).type.shape);
        const FusedProgram program = n.op == OpKind::FusedElementwise ? *n.fused : cuda::single_op_program(n.op);
        text += cuda::generate_elementwise_kernel(program, shapes, n.type.shape).source + "\n";
    }
    return give(text, out, size);
}

REF_API int ref_num_inputs(const void* g) { return static_cast<int>(static_cast<const RefGraph*>(g)->graph.inputs().size()); }
REF_API int ref_num_outputs(const void* g) { return static_cast<int>(static_cast<const RefGraph*>(g)->graph.outputs().size()); }
REF_API long long ref_input_elements(const void* g, int k) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    return static_cast<long long>(graph.node(graph.inputs()[static_cast<std::size_t>(k)]).type.num_elements());
}
REF_API long long ref_output_elements(const void* g, int k) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    return static_cast<long long>(graph.node(graph.outputs()[static_cast<std::size_t>(k)]).type.num_elements());
}

// The reference's double-precision evaluator (tests/test_util.cpp:87-159) on caller inputs.
REF_API int ref_evaluate(const void* g, const float* const* inputs, float* const* outputs) {
    const Graph& graph = static_cast<const RefGraph*>(g)->graph;
    std::vector<HostTensor> in;
    for (std::size_t k = 0; k < graph.inputs().size(); ++k) {
        const TensorType& type = graph.node(graph.inputs()[k]).type;
        in.emplace_back(type, std::vector<float>(inputs[k], inputs[k] + type.num_elements()));
    }
    const std::vector<HostTensor> out = testutil::evaluate_reference(graph, in);
    for (std::size_t k = 0; k < out.size(); ++k) std::memcpy(outputs[k], out[k].data.data(), out[k].data.size() * sizeof(float));
    return 0;
}

// The reference's random-graph generator (tests/test_util.cpp:177-341), as .mcg text.
REF_API int ref_random_graph(unsigned long long seed, int num_ops, int allow_matmul, char* out, int size) {
    testutil::RandomGraphOptions options;
    options.num_ops = num_ops;
    options.allow_matmul = allow_matmul != 0;
    return give(to_mcg(testutil::make_random_graph(seed, options)), out, size);
}

REF_API void ref_uniform_values(float* out, long long count, unsigned long long seed, float lo, float hi) {
    fill_uniform(out, static_cast<std::size_t>(count), seed, lo, hi);
}
