// The C ABI: the `mc_*` calls with the reference's contract (bench/capi.cpp:62-235)
// in front of the B200 backend, and the host-only `mcb_*` introspection calls.

#include "minicompiler_b200.h"

#include "backend/b200_backend.hpp"
#include "backend/partition.hpp"
#include "backend/row_slicing.hpp"
#include "core/passes.hpp"
#include "core/plan.hpp"
#include "minicompiler_b200_device.h"

#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <memory>
#include <sstream>
#include <mutex>
#include <set>
#include <string>
#include <vector>

using namespace minicompiler;

namespace {

thread_local std::string g_error;

struct Compiled {
    Graph graph;
    std::unique_ptr<Executable> exe;
    cuda::CudaExecutable* gpu = nullptr;
    std::vector<const float*> inputs;
    std::vector<float*> outputs;
};

struct OpenGraph {
    Graph graph;
    std::vector<PassReport> reports;
};

void put(char* out, int size, const std::string& text) {
    if (out != nullptr && size > 0) std::snprintf(out, static_cast<std::size_t>(size), "%s", text.c_str());
}

int put_len(char* out, int size, const std::string& text) {
    put(out, size, text);
    return static_cast<int>(text.size());
}

void* reject(char* error, int error_size, const std::string& message) {
    g_error = message;
    put(error, error_size, message);
    return nullptr;
}

int failed(const Status& st) {
    if (st.ok()) return 0;
    g_error = st.message();
    return 1;
}

// "M=64,N=4096" -> map. The message for a malformed item is the reference's.
Status parse_dims(const char* dims, std::map<std::string, std::int64_t>* out) {
    std::stringstream list(dims != nullptr ? dims : "");
    for (std::string item; std::getline(list, item, ',');) {
        const std::size_t eq = item.find('=');
        char* end = nullptr;
        errno = 0;
        const long long value = eq == std::string::npos ? 0 : std::strtoll(item.c_str() + eq + 1, &end, 10);
        if (eq == std::string::npos || *end != '\0' || errno == ERANGE) {
            return Error{"bad dim '" + item + "', expected NAME=VALUE"};
        }
        (*out)[item.substr(0, eq)] = value;
    }
    return Status();
}

Status parse_options(const char* text, cuda::CudaOptions* options) {
    std::stringstream list(text != nullptr ? text : "");
    for (std::string item; std::getline(list, item, ',');) {
        if (item.empty()) continue;
        const std::size_t eq = item.find('=');
        if (eq == std::string::npos) return Error{"bad option '" + item + "', expected KEY=VALUE"};
        const std::string key = item.substr(0, eq);
        const std::string value = item.substr(eq + 1);
        if (key == "matmul") {
            MC_ASSIGN(kernel, cuda::matmul_kernel_from_name(value));
            options->matmul = kernel;
        } else if (key == "b_layout") {
            if (value == "auto") {
                options->b_layout = cuda::BLayout::Auto;
            } else if (value == "kn") {
                options->b_layout = cuda::BLayout::RowMajorKN;
            } else if (value == "transposed") {
                options->b_layout = cuda::BLayout::Transposed;
            } else {
                return Error{"unknown b_layout '" + value + "' (auto, kn, transposed)"};
            }
        } else {
            char* end = nullptr;
            const long number = std::strtol(value.c_str(), &end, 10);
            if (value.empty() || *end != '\0') return Error{"option '" + key + "' needs an integer, got '" + value + "'"};
            if (key == "device") {
                options->device = static_cast<int>(number);
            } else if (key == "vectorize") {
                options->vectorize = number != 0;
            } else if (key == "fuse_epilogue") {
                options->fuse_epilogue = number != 0;
            } else if (key == "unroll") {
                if (number < 1 || number > 16) return Error{"unroll must be between 1 and 16"};
                options->eltwise_unroll = static_cast<unsigned>(number);
            } else if (key == "streaming") {
                options->streaming_hints = number != 0;
            } else if (key == "gemm_variant") {
                options->gemm_variant = static_cast<int>(number);
            } else if (key == "host_io_slices") {
                options->host_io_slices = static_cast<int>(number);
            } else if (key == "host_io_row_slices") {
                options->host_io_row_slices = static_cast<int>(number);
            } else if (key == "balance_splits") {
                options->balance_splits = number != 0;
            } else if (key == "fuse_rows") {
                options->fuse_rows = number != 0;
            } else if (key == "rematerialize") {
                options->rematerialize = number != 0;
            } else if (key == "host_io") {
                options->host_io = static_cast<int>(number);
            } else if (key == "graph") {
                options->replay_graph = number != 0;
            } else if (key == "fmad") {
                options->eltwise_fmad = number != 0;
            } else if (key == "blocks_per_sm") {
                options->eltwise_blocks_per_sm = static_cast<int>(number);
            } else {
                return Error{"unknown option '" + key +
                             "' (device, matmul, vectorize, fuse_epilogue, b_layout, unroll, streaming, gemm_variant, fmad, blocks_per_sm, graph, host_io, host_io_slices, host_io_row_slices, rematerialize, fuse_rows, balance_splits)"};
            }
        }
    }
    return Status();
}

Result<Graph> load_and_optimize(const char* path, const char* text, const char* dims, const char* passes,
                                std::vector<PassReport>* reports) {
    ParseOptions options;
    MC_TRY(parse_dims(dims, &options.dims));
    Result<Graph> graph = text != nullptr ? parse_graph(text, options) : parse_graph_file(path != nullptr ? path : "", options);
    if (!graph.ok()) return graph.error();
    MC_ASSIGN(pipeline, parse_pipeline(passes != nullptr ? passes : "default"));
    return run_pipeline(graph.value(), pipeline, reports);
}

void* compile_common(const char* path, const char* text, const char* dims, const char* passes,
                     const cuda::CudaOptions& options, char* error, int error_size) {
    Result<Graph> optimized = load_and_optimize(path, text, dims, passes, nullptr);
    if (!optimized.ok()) return reject(error, error_size, optimized.error().message);
    Result<std::unique_ptr<Backend>> backend = cuda::make_cuda_backend(options);
    if (!backend.ok()) return reject(error, error_size, backend.error().message);
    Result<std::unique_ptr<Executable>> exe = (*backend)->compile(optimized.value());
    if (!exe.ok()) return reject(error, error_size, exe.error().message);
    auto compiled = std::make_unique<Compiled>();
    compiled->graph = std::move(optimized).value();
    compiled->exe = std::move(exe).value();
    compiled->gpu = dynamic_cast<cuda::CudaExecutable*>(compiled->exe.get());
    return compiled.release();
}

Compiled* as_compiled(void* handle) { return static_cast<Compiled*>(handle); }
const Compiled* as_compiled(const void* handle) { return static_cast<const Compiled*>(handle); }

std::string json_escape(const std::string& s) {
    std::string out;
    for (char c : s) {
        if (c == '"' || c == '\\') {
            out += '\\';
            out += c;
        } else if (c == '\n') {
            out += "\\n";
        } else {
            out += c;
        }
    }
    return out;
}

std::string stats_json(const GraphStats& s) {
    std::ostringstream os;
    os << "{\"nodes\": " << s.nodes << ", \"inputs\": " << s.inputs << ", \"constants\": " << s.constants
       << ", \"compute_nodes\": " << s.compute_nodes << ", \"fused_nodes\": " << s.fused_nodes
       << ", \"elementwise_ops\": " << s.elementwise_ops << ", \"matmuls\": " << s.matmuls << "}";
    return os.str();
}

}  // namespace

extern "C" {

const char* mc_last_error(void) { return g_error.c_str(); }

void* mc_compile(const char* graph_path, const char* dims, const char* passes, const char* backend, char* error,
                 int error_size) {
    const std::string name = backend != nullptr ? backend : "cuda";
    if (name != "cuda") {
        Result<std::unique_ptr<Backend>> chosen = create_backend(name);  // yields the right message
        return reject(error, error_size, chosen.ok() ? "unsupported backend" : chosen.error().message);
    }
    return compile_common(graph_path, nullptr, dims, passes, cuda::CudaOptions{}, error, error_size);
}

void* mc_compile_ex(const char* graph_path, const char* graph_text, const char* dims, const char* passes,
                    const char* options, char* error, int error_size) {
    cuda::CudaOptions parsed;
    Status st = parse_options(options, &parsed);
    if (!st.ok()) return reject(error, error_size, st.message());
    return compile_common(graph_path, graph_text, dims, passes, parsed, error, error_size);
}

int mc_num_inputs(const void* handle) { return static_cast<int>(as_compiled(handle)->graph.inputs().size()); }
int mc_num_outputs(const void* handle) { return static_cast<int>(as_compiled(handle)->graph.outputs().size()); }

long long mc_output_elements(const void* handle, int k) {
    const Graph& g = as_compiled(handle)->graph;
    return static_cast<long long>(g.node(g.outputs()[static_cast<std::size_t>(k)]).type.num_elements());
}

long long mc_input_elements(const void* handle, int k) {
    const Graph& g = as_compiled(handle)->graph;
    return static_cast<long long>(g.node(g.inputs()[static_cast<std::size_t>(k)]).type.num_elements());
}

int mc_run(void* handle, const float* const* inputs, float* const* outputs) {
    Compiled* c = as_compiled(handle);
    c->inputs.assign(inputs, inputs + c->graph.inputs().size());
    c->outputs.assign(outputs, outputs + c->graph.outputs().size());
    return failed(c->exe->run_buffers(c->inputs, c->outputs));
}

int mc_upload(void* handle, const float* const* inputs) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr) return 1;
    c->inputs.assign(inputs, inputs + c->graph.inputs().size());
    if (int rc = failed(c->gpu->upload_inputs(c->inputs))) return rc;
    return failed(c->gpu->synchronize());
}

int mc_enqueue(void* handle, void* stream) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? failed(c->gpu->enqueue(stream)) : 1;
}

int mc_download(void* handle, float* const* outputs) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr) return 1;
    c->outputs.assign(outputs, outputs + c->graph.outputs().size());
    return failed(c->gpu->download_outputs(c->outputs));
}

int mc_synchronize(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? failed(c->gpu->synchronize()) : 1;
}

int mc_kernel_launches(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? static_cast<int>(c->gpu->kernel_launches()) : -1;
}

int mc_matmul_kernels(void* handle, char* out, int size) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr) return 1;
    std::string names;
    for (cuda::MatmulKernel k : c->gpu->matmul_kernels()) {
        if (!names.empty()) names += ",";
        names += cuda::matmul_kernel_name(k);
    }
    put(out, size, names);
    return 0;
}

double mc_gpu_sm_clock_mhz(void) { return cuda::current_sm_clock_mhz(0); }

int mc_gpu_device_json(const double* clocks, int n, char* out, int size) {
    Result<cuda::DeviceInfo> device = cuda::query_device(0);
    if (!device.ok()) return 1;
    const cuda::DeviceInfo& d = device.value();
    std::vector<double> samples(clocks, clocks + (clocks != nullptr ? n : 0));
    double lo = 0, hi = 0, mean = 0;
    if (!samples.empty()) {
        lo = hi = samples[0];
        for (double s : samples) {
            lo = std::min(lo, s);
            hi = std::max(hi, s);
            mean += s;
        }
        mean /= static_cast<double>(samples.size());
    }
    const double clock_for_peak = mean > 0 ? mean : (d.max_sm_clock_mhz > 0 ? d.max_sm_clock_mhz : d.sm_clock_mhz);
    std::ostringstream os;
    os << "{\"name\": \"" << json_escape(d.name) << "\", \"compute_capability\": \"" << d.cc_major << "." << d.cc_minor
       << "\", \"sm_count\": " << d.sm_count << ", \"fp32_lanes_per_sm\": " << d.fp32_lanes_per_sm
       << ", \"sm_clock_mhz\": " << d.sm_clock_mhz << ", \"max_sm_clock_mhz\": " << d.max_sm_clock_mhz
       << ", \"mem_clock_mhz\": " << d.mem_clock_mhz << ", \"bus_width_bits\": " << d.bus_width_bits
       << ", \"total_memory\": " << d.total_memory << ", \"runtime_version\": " << d.runtime_version
       << ", \"driver_version\": " << d.driver_version << ", \"peak_bandwidth_gbs\": " << d.peak_bandwidth_gbs()
       << ", \"peak_fp32_gflops\": " << d.peak_fp32_gflops(clock_for_peak) << ", \"sm_clock_samples\": {\"count\": "
       << samples.size() << ", \"min\": " << lo << ", \"max\": " << hi << ", \"mean\": " << mean << "}}";
    const std::string text = os.str();
    if (static_cast<int>(text.size()) >= size) return 2;
    put(out, size, text);
    return 0;
}

void mc_release(void* handle) { delete as_compiled(handle); }

int mc_constants_region(void* handle, void** device_ptr, size_t* bytes) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr) return 1;
    c->gpu->constants_region(device_ptr, bytes);
    return 0;
}

int mc_status_word_ptr(void* handle, void** device_ptr) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr || device_ptr == nullptr) return 1;
    *device_ptr = c->gpu->status_word_address();
    return 0;
}

int mcb_in_place_pointers_ok(const void* const* pointers, int count, int any_vectorized) {
    std::vector<const void*> list(pointers, pointers + (count > 0 ? count : 0));
    return minicompiler::cuda::in_place_pointers_ok(any_vectorized != 0, list) ? 1 : 0;
}

int mc_replicate_constants(void* handle, void* comm, int root) {
    Compiled* c = as_compiled(handle);
    if (c == nullptr || c->gpu == nullptr) {
        g_error = "mc_replicate_constants: not a GPU executable";
        return 1;
    }
    return failed(c->gpu->replicate_constants(comm, root));
}

int mc_gather_output(void* handle, int k, void* comm, void* device_dst) {
    Compiled* c = as_compiled(handle);
    if (c == nullptr || c->gpu == nullptr || k < 0) {
        g_error = "mc_gather_output: not a GPU executable, or a negative output index";
        return 1;
    }
    return failed(c->gpu->gather_output(static_cast<std::size_t>(k), comm, device_dst));
}

int mc_row_slices(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? static_cast<int>(c->gpu->row_slices()) : 0;
}

int mc_refresh_constants(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? failed(c->gpu->refresh_constants()) : 1;
}

int mc_input_device_ptr(void* handle, int k, void** device_ptr, size_t* elements) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr || k < 0 || static_cast<std::size_t>(k) >= c->graph.inputs().size()) return 1;
    c->gpu->input_buffer(static_cast<std::size_t>(k), device_ptr, elements);
    return 0;
}

int mc_output_device_ptr(void* handle, int k, void** device_ptr, size_t* elements) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr || k < 0 || static_cast<std::size_t>(k) >= c->graph.outputs().size()) return 1;
    c->gpu->output_buffer(static_cast<std::size_t>(k), device_ptr, elements);
    return 0;
}

long long mc_intermediate_bytes(void* handle) { return static_cast<long long>(as_compiled(handle)->exe->intermediate_bytes()); }

long long mc_arena_bytes(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? static_cast<long long>(c->gpu->arena_bytes()) : -1;
}

double mc_jit_compile_ms(void* handle) {
    Compiled* c = as_compiled(handle);
    return c->gpu != nullptr ? c->gpu->jit_compile_ms() : 0.0;
}

int mc_kernel_sources(void* handle, char* out, int size) {
    Compiled* c = as_compiled(handle);
    if (c->gpu == nullptr) return -1;
    std::string all;
    for (const std::string& s : c->gpu->kernel_sources()) all += (all.empty() ? "" : "\n// ----\n") + s;
    return put_len(out, size, all);
}

int mc_shard_dims(const char* graph_path, const char* dims, const char* batch_dim, int rank, int world_size, char* out_dims,
                  int out_size, long long* row_offset, long long* rows) {
    std::map<std::string, std::int64_t> parsed;
    if (int rc = failed(parse_dims(dims, &parsed))) return rc;
    std::ifstream file(graph_path != nullptr ? graph_path : "", std::ios::binary);
    if (!file) {
        g_error = std::string("cannot open '") + (graph_path != nullptr ? graph_path : "") + "'";
        return 1;
    }
    std::ostringstream text;
    text << file.rdbuf();
    Result<ShardPlan> plan = plan_batch_shard(text.str(), parsed, batch_dim != nullptr ? batch_dim : "", rank, world_size);
    if (!plan.ok()) {
        g_error = plan.error().message;
        return 1;
    }
    std::string joined;
    for (const auto& kv : plan->dims) joined += (joined.empty() ? "" : ",") + kv.first + "=" + std::to_string(kv.second);
    if (static_cast<int>(joined.size()) >= out_size) {
        g_error = "dims buffer too small";
        return 2;
    }
    put(out_dims, out_size, joined);
    if (row_offset != nullptr) *row_offset = plan->row_offset;
    if (rows != nullptr) *rows = plan->rows;
    return 0;
}

// ------------------------------------------------------------ introspection

void* mcb_graph_open(const char* path, const char* text, const char* dims, const char* passes, char* error, int error_size) {
    auto open = std::make_unique<OpenGraph>();
    Result<Graph> g = load_and_optimize(path, text, dims, passes, &open->reports);
    if (!g.ok()) return reject(error, error_size, g.error().message);
    open->graph = std::move(g).value();
    return open.release();
}

void mcb_graph_close(void* graph) { delete static_cast<OpenGraph*>(graph); }

int mcb_graph_print(const void* graph, char* out, int size) {
    return put_len(out, size, print_graph(static_cast<const OpenGraph*>(graph)->graph));
}

int mcb_graph_num_nodes(const void* graph) {
    return static_cast<int>(static_cast<const OpenGraph*>(graph)->graph.num_nodes());
}

int mcb_graph_stats_json(const void* graph, char* out, int size) {
    const auto* open = static_cast<const OpenGraph*>(graph);
    std::ostringstream os;
    os << "{\"final\": " << stats_json(compute_stats(open->graph)) << ", \"passes\": [";
    for (std::size_t i = 0; i < open->reports.size(); ++i) {
        const PassReport& r = open->reports[i];
        os << (i ? ", " : "") << "{\"pass\": \"" << r.pass << "\", \"summary\": \"" << json_escape(r.summary)
           << "\", \"before\": " << stats_json(r.before) << ", \"after\": " << stats_json(r.after) << "}";
    }
    os << "]}";
    return put_len(out, size, os.str());
}

int mcb_graph_plan_json(const void* graph, int pool_outputs, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    const MemoryPlan plan = plan_memory(g, PlanOptions{pool_outputs != 0});
    std::ostringstream os;
    os << "{\"buffer_of\": [";
    for (std::size_t i = 0; i < plan.buffer_of.size(); ++i) os << (i ? ", " : "") << plan.buffer_of[i];
    os << "], \"buffer_bytes\": [";
    for (std::size_t i = 0; i < plan.buffer_bytes.size(); ++i) os << (i ? ", " : "") << plan.buffer_bytes[i];
    os << "], \"last_use\": [";
    for (std::size_t i = 0; i < plan.last_use.size(); ++i) os << (i ? ", " : "") << plan.last_use[i];
    os << "], \"bytes_without_reuse\": " << plan.bytes_without_reuse << ", \"bytes_with_reuse\": " << plan.bytes_with_reuse()
       << "}";
    return put_len(out, size, os.str());
}

int mcb_graph_fusion_groups(const void* graph, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    std::string text;
    for (const std::vector<NodeId>& group : find_fusion_groups(g)) {
        std::string line;
        for (NodeId m : group) line += (line.empty() ? "" : " ") + g.node(m).name;
        text += line + "\n";
    }
    return put_len(out, size, text);
}

int mcb_graph_row_slicing(const void* graph, long long slice_rows, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    const cuda::RowSlicing slicing = cuda::analyze_row_slicing(g);
    if (!slicing.ok) return put_len(out, size, "none");
    std::string text = "rows=" + std::to_string(slicing.rows) + " cut=";
    bool first = true;
    for (std::size_t i = 0; i < g.num_nodes(); ++i) {
        if (!slicing.carries[i]) continue;
        text += (first ? "" : ",") + g.node(static_cast<NodeId>(i)).name;
        first = false;
    }
    if (slice_rows > 0) {
        Result<Graph> sliced = cuda::with_leading_extent(g, slicing, slice_rows);
        if (!sliced.ok()) {
            g_error = sliced.error().message;
            return -1;
        }
        text += "\n" + print_graph(*sliced);
    }
    return put_len(out, size, text);
}

int mcb_graph_emit_cuda(const void* graph, const char* options, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    cuda::CudaOptions parsed;
    if (failed(parse_options(options, &parsed))) return -1;
    std::string text;
    for (std::size_t i = 0; i < g.num_nodes(); ++i) {
        const Node& n = g.node(static_cast<NodeId>(i));
        if (is_row_reduce(n.op)) {  // the node on its own: identity prologue
            FusedProgram identity;
            identity.instrs.push_back(FusedInstr::load(0));
            const Shape& in_shape = g.node(n.inputs[0]).type.shape;
            text += "// node %" + std::to_string(i) + " '" + n.name + "' : " + to_string(n.type) + "\n";
            text += cuda::generate_row_reduce_kernel(n.op, identity, {in_shape}, in_shape).source + "\n";
            continue;
        }
        if (!is_elementwise(n.op) && n.op != OpKind::FusedElementwise) continue;
        std::vector<Shape> shapes;
        for (NodeId in : n.inputs) shapes.push_back(g.node(in).type.shape);
        cuda::ElementwiseOptions eo;
        eo.allow_vectorize = parsed.vectorize;
        eo.unroll = parsed.eltwise_unroll;
        eo.streaming_hints = parsed.streaming_hints;
        const FusedProgram program = n.op == OpKind::FusedElementwise ? *n.fused : single_op_program(n.op);
        text += "// node %" + std::to_string(i) + " '" + n.name + "' : " + to_string(n.type) + "\n";
        text += cuda::generate_elementwise_kernel(program, shapes, n.type.shape, eo).source + "\n";
    }
    return put_len(out, size, text);
}

int mcb_graph_launch_plan(const void* graph, const char* options, int sm_count, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    cuda::CudaOptions parsed;
    if (failed(parse_options(options, &parsed))) return -1;
    Result<cuda::LoweredGraph> lowered = cuda::lower_graph(g, parsed, sm_count);
    if (!lowered.ok()) {
        g_error = lowered.error().message;
        return -1;
    }
    std::ostringstream os;
    os << cuda::describe(g, lowered.value());
    os << "launches=" << lowered->kernel_launches << " intermediate_bytes=" << lowered->pool.bytes_with_reuse()
       << " workspace_bytes=" << lowered->workspace_bytes << "\n";
    return put_len(out, size, os.str());
}

long long mcb_graph_constant(const void* graph, const char* name, float* out, long long capacity) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    const std::optional<NodeId> id = g.find(name != nullptr ? name : "");
    if (!id || g.node(*id).op != OpKind::Constant) return -1;
    const std::vector<float>& v = *g.node(*id).constant;
    const auto n = static_cast<long long>(v.size());
    if (out != nullptr) std::memcpy(out, v.data(), static_cast<std::size_t>(std::min(n, capacity)) * sizeof(float));
    return n;
}

int mcd_jit_compile_only(const char* source, const char* options, size_t* cubin_bytes);

namespace {

// The text generated for one step of a launch plan: the kernel of an elementwise, reduction or row-fused step, the
// epilogue plus kernel family of a matmul with a fused consumer; empty for a matmul that runs a built-in kernel.
std::string step_source(const Graph& g, const cuda::CudaOptions& parsed, const cuda::Step& step) {
    std::vector<Shape> shapes;
    for (NodeId in : step.inputs) shapes.push_back(g.node(in).type.shape);
    switch (step.kind) {
        case cuda::Step::Kind::Elementwise: {
            cuda::ElementwiseOptions eo;
            eo.allow_vectorize = parsed.vectorize;
            eo.unroll = parsed.eltwise_unroll;
            eo.write_f32 = step.write_f32;
            eo.write_half = step.write_half;
            eo.streaming_hints = parsed.streaming_hints;
            const TensorType& type = g.node(step.result).type;
            if (step.write_half != cuda::HalfKind::None && type.shape.size() == 2) eo.half_pitch = cuda::half_pitch(type.shape[1]);
            return cuda::generate_elementwise_kernel(step.program, shapes, type.shape, eo).source;
        }
        case cuda::Step::Kind::RowFused:
            return cuda::generate_row_fused_kernel(step.row_parts, step.row_externals, static_cast<int>(step.row_outputs.size()),
                                                   step.reduce_shape.back());
        case cuda::Step::Kind::Reduce:
            return cuda::generate_row_reduce_kernel(step.reduce_op, step.program, shapes, step.reduce_shape).source;
        case cuda::Step::Kind::Matmul:
            if (!step.has_epilogue) return {};
            return cuda::generate_epilogue_source(g, step) + mcd_gemm_source(step.launches > 1 ? -1 : static_cast<int>(step.arith));
    }
    return {};
}

}  // namespace

int mcb_graph_check_kernels(const void* graph, const char* options, int sm_count) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    cuda::CudaOptions parsed;
    if (failed(parse_options(options, &parsed))) return 1;
    Result<cuda::LoweredGraph> lowered = cuda::lower_graph(g, parsed, sm_count);
    if (!lowered.ok()) {
        g_error = lowered.error().message;
        return 1;
    }
    // Every distinct text is compiled once. Of a tensor-core kernel family, which holds ten entry points, one
    // entry point of each body (one CTA per tile, SM pair, SM pair with two tiles) is compiled, as at run time.
    static std::set<std::string> seen;  // texts that compiled, for the life of the process
    static std::mutex seen_mutex;
    auto compile_once = [&](const std::string& text) -> bool {
        {
            std::lock_guard<std::mutex> lock(seen_mutex);
            if (seen.count(text) != 0) return true;
        }
        if (mcd_jit_compile_only(text.c_str(), "--fmad=false", nullptr) != 0) {
            g_error = mcd_last_error();
            return false;
        }
        std::lock_guard<std::mutex> lock(seen_mutex);
        seen.insert(text);
        return true;
    };
    for (const cuda::Step& step : lowered->steps) {
        const std::string source = step_source(g, parsed, step);
        if (source.empty()) continue;
        if (step.kind == cuda::Step::Kind::Matmul && step.splits == 1 && step.arith != cuda::Arith::F32) {
            const bool tf32 = step.arith == cuda::Arith::Tf32;
            for (const char* entry : {tf32 ? "mc_gemm_tc_tf32_bk" : "mc_gemm_tc_h16_bmn", tf32 ? "mc_gemm_tc2_tf32_bk" : "mc_gemm_tc2_h16_bk",
                                      tf32 ? "mc_gemm_tc2w_tf32_bk" : "mc_gemm_tc2w_h16_bmn"}) {
                if (!compile_once(std::string("#define MC_SINGLE_ENTRY 1\n#define MC_ONLY_") + entry + " 1\n" + source)) return 1;
            }
            continue;
        }
        if (!compile_once(source)) return 1;
    }
    return 0;
}

int mcb_graph_plan_sources(const void* graph, const char* options, int sm_count, char* out, int size) {
    const Graph& g = static_cast<const OpenGraph*>(graph)->graph;
    cuda::CudaOptions parsed;
    if (failed(parse_options(options, &parsed))) return -1;
    Result<cuda::LoweredGraph> lowered = cuda::lower_graph(g, parsed, sm_count);
    if (!lowered.ok()) {
        g_error = lowered.error().message;
        return -1;
    }
    std::string text;
    for (std::size_t i = 0; i < lowered->steps.size(); ++i) {
        const cuda::Step& step = lowered->steps[i];
        if (step.kind == cuda::Step::Kind::Matmul) {
            if (step.has_epilogue) {
                text += "// step " + std::to_string(i) + ": epilogue of matmul '" + g.node(step.matmul).name + "' computing '" +
                        g.node(step.result).name + "'\n" + cuda::generate_epilogue_source(g, step) + "\n";
            }
            continue;
        }
        text += "// step " + std::to_string(i) + "\n" + step_source(g, parsed, step) + "\n";
    }
    return put_len(out, size, text);
}

void mcb_uniform_values(float* out, long long count, unsigned long long seed, float lo, float hi) {
    fill_uniform(out, static_cast<std::size_t>(count), seed, lo, hi);
}

int mcb_split_k_splits(int m, int n, int k, int sm_count, int blocks_per_sm) {
    return cuda::split_k_splits(m, n, k, sm_count, blocks_per_sm);
}

int mcb_balanced_fp32_splits(int m, int n, int k, int sm_count) { return cuda::balanced_fp32_splits(m, n, k, sm_count); }

int mcb_tensor_core_splits(int m, int n, int k, int sm_count, int elem_bytes) {
    return cuda::tensor_core_splits(m, n, k, sm_count, elem_bytes);
}

int mcb_tensor_core_tile_n(int m, int n, int k, int sm_count, int elem_bytes) {
    return cuda::tensor_core_tile_n(m, n, k, sm_count, elem_bytes);
}

const char* mcb_resolve_matmul_kernel(const char* kernel_name, int m, int n, int k, int sm_count) {
    Result<cuda::MatmulKernel> kernel = cuda::matmul_kernel_from_name(kernel_name != nullptr ? kernel_name : "");
    if (!kernel.ok()) {
        g_error = kernel.error().message;
        return nullptr;
    }
    return cuda::matmul_kernel_name(cuda::resolve_matmul_kernel(kernel.value(), m, n, k, sm_count));
}

}  // extern "C"
