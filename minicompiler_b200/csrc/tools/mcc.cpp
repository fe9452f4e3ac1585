// mcc: command-line driver with the reference's flags (tools/mcc.cpp:27-51) in front of
// the B200 backend. `--emit-cuda`, `--print`, `--stats` and the listings need no GPU;
// `--run` and `--bench` need a B200. `--backend` defaults to cuda here, because this
// build has no CPU execution path. Additions: `--matmul NAME`, `--option KEY=VALUE`,
// `--print-plan`.

#include "backend/b200_backend.hpp"
#include "core/mcg.hpp"
#include "core/passes.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

using namespace minicompiler;

namespace {

constexpr const char* kUsage = R"(usage: mcc GRAPH.mcg [options]

compile:
  --dim NAME=VALUE      override a dim declared in the graph (repeatable)
  --passes LIST         "default" (dne,fold,dne,fuse,dne), "none", or a
                        comma-separated list of: dne, fold, fuse
  --print               print the optimized graph
  --emit-cuda           print the CUDA source generated for each elementwise or fused
                        node (needs no GPU)
  --stats               print node counts after each pass
  --print-plan          print the launch plan (kernels, epilogue folding, splits)
  --matmul NAME         matmul kernel: auto, split_k, tensor_core_tf32, tensor_core_bf16,
                        tensor_core_f16, ... (default auto)

run:
  --backend NAME        cuda (default; this build has no cpu backend)
  --run                 run once on seeded random inputs; print output checksums
  --seed N              input seed (default 1)
  --dump-outputs FILE   write the outputs as raw float32, concatenated
  --bench               time repeated runs and print JSON
  --warmup N            untimed runs before timing (default 10)
  --reps N              timed runs (default 50)

info:
  --list-backends       print the backends compiled into this build
  --list-passes         print the available passes
)";

struct Options {
    std::string graph_path;
    ParseOptions parse;
    std::string passes = "default";
    bool print = false, emit_cuda = false, stats = false, print_plan = false;
    std::string backend = "cuda";
    cuda::CudaOptions cuda;
    bool run = false;
    std::uint64_t seed = 1;
    std::string dump_outputs;
    bool bench = false;
    int warmup = 10;
    int reps = 50;
};

int fail(const std::string& message) {
    std::cerr << "mcc: " << message << "\n";
    return 1;
}

bool to_int(const std::string& s, long long* out) {
    char* end = nullptr;
    errno = 0;
    const long long v = std::strtoll(s.c_str(), &end, 10);
    if (s.empty() || end != s.c_str() + s.size() || errno == ERANGE) return false;
    *out = v;
    return true;
}

std::string stats_line(const GraphStats& s) {
    return std::to_string(s.nodes) + " nodes, " + std::to_string(s.compute_nodes) + " compute (" +
           std::to_string(s.elementwise_ops) + " elementwise ops, " + std::to_string(s.matmuls) + " matmul, " +
           std::to_string(s.fused_nodes) + " fused kernels)";
}

}  // namespace

int main(int argc, char** argv) {
    Options opt;
    std::vector<std::string> args(argv + 1, argv + argc);
    for (std::size_t i = 0; i < args.size(); ++i) {
        const std::string& a = args[i];
        auto value = [&](std::string* out) {
            if (i + 1 >= args.size()) return false;
            *out = args[++i];
            return true;
        };
        std::string v;
        long long n = 0;
        if (a == "--help" || a == "-h") {
            std::cout << kUsage;
            return 0;
        } else if (a == "--list-backends") {
            for (const std::string& b : available_backends()) std::cout << b << "\n";
            return 0;
        } else if (a == "--list-passes") {
            for (const PassInfo& p : registered_passes()) std::cout << p.name << "  " << p.description << "\n";
            return 0;
        } else if (a == "--dim") {
            if (!value(&v)) return fail("--dim needs NAME=VALUE");
            const std::size_t eq = v.find('=');
            if (eq == std::string::npos || !to_int(v.substr(eq + 1), &n)) return fail("bad --dim '" + v + "', expected NAME=VALUE");
            opt.parse.dims[v.substr(0, eq)] = n;
        } else if (a == "--passes") {
            if (!value(&opt.passes)) return fail("--passes needs a list");
        } else if (a == "--print") {
            opt.print = true;
        } else if (a == "--emit-cuda") {
            opt.emit_cuda = true;
        } else if (a == "--stats") {
            opt.stats = true;
        } else if (a == "--print-plan") {
            opt.print_plan = true;
        } else if (a == "--matmul") {
            if (!value(&v)) return fail("--matmul needs a kernel name");
            Result<cuda::MatmulKernel> k = cuda::matmul_kernel_from_name(v);
            if (!k.ok()) return fail(k.error().message);
            opt.cuda.matmul = k.value();
        } else if (a == "--no-epilogue-fusion") {
            opt.cuda.fuse_epilogue = false;
        } else if (a == "--backend") {
            if (!value(&opt.backend)) return fail("--backend needs a name");
        } else if (a == "--run") {
            opt.run = true;
        } else if (a == "--seed") {
            if (!value(&v) || !to_int(v, &n) || n < 0) return fail("--seed needs a non-negative integer");
            opt.seed = static_cast<std::uint64_t>(n);
        } else if (a == "--dump-outputs") {
            if (!value(&opt.dump_outputs)) return fail("--dump-outputs needs a file");
        } else if (a == "--bench") {
            opt.bench = true;
        } else if (a == "--warmup") {
            if (!value(&v) || !to_int(v, &n) || n < 0) return fail("--warmup needs a non-negative integer");
            opt.warmup = static_cast<int>(n);
        } else if (a == "--reps") {
            if (!value(&v) || !to_int(v, &n) || n < 1) return fail("--reps needs a positive integer");
            opt.reps = static_cast<int>(n);
        } else if (a == "--dump-dot") {
            return fail("--dump-dot is not part of this build (graph visualisation is out of scope)");
        } else if (!a.empty() && a[0] == '-') {
            return fail("unknown option '" + a + "'\n" + kUsage);
        } else if (opt.graph_path.empty()) {
            opt.graph_path = a;
        } else {
            return fail("more than one graph file given");
        }
    }
    if (opt.graph_path.empty()) {
        std::cerr << kUsage;
        return 1;
    }

    Result<Graph> parsed = parse_graph_file(opt.graph_path, opt.parse);
    if (!parsed.ok()) return fail(parsed.error().message);
    Result<std::vector<std::string>> pipeline = parse_pipeline(opt.passes);
    if (!pipeline.ok()) return fail(pipeline.error().message);
    std::vector<PassReport> reports;
    const GraphStats before = compute_stats(parsed.value());
    Result<Graph> optimized = run_pipeline(parsed.value(), pipeline.value(), &reports);
    if (!optimized.ok()) return fail(optimized.error().message);
    const Graph& graph = optimized.value();

    if (opt.stats) {
        std::cout << "input: " << stats_line(before) << "\n";
        for (const PassReport& r : reports) std::cout << r.pass << ": " << stats_line(r.after) << "  [" << r.summary << "]\n";
    }
    if (opt.print) std::cout << print_graph(graph);
    if (opt.emit_cuda) {
        for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
            const Node& n = graph.node(static_cast<NodeId>(i));
            if (is_row_reduce(n.op)) {  // the node on its own: identity prologue
                FusedProgram identity;
                identity.instrs.push_back(FusedInstr::load(0));
                const Shape& in_shape = graph.node(n.inputs[0]).type.shape;
                std::cout << "// node %" << i << " '" << n.name << "' : " << to_string(n.type) << "\n"
                          << cuda::generate_row_reduce_kernel(n.op, identity, {in_shape}, in_shape).source << "\n";
                continue;
            }
            if (!is_elementwise(n.op) && n.op != OpKind::FusedElementwise) continue;
            std::vector<Shape> shapes;
            for (NodeId in : n.inputs) shapes.push_back(graph.node(in).type.shape);
            const FusedProgram program = n.op == OpKind::FusedElementwise ? *n.fused : single_op_program(n.op);
            cuda::ElementwiseOptions eo;
            eo.allow_vectorize = opt.cuda.vectorize;
            std::cout << "// node %" << i << " '" << n.name << "' : " << to_string(n.type) << "\n"
                      << cuda::generate_elementwise_kernel(program, shapes, n.type.shape, eo).source << "\n";
        }
    }
    if (opt.print_plan) {
        Result<cuda::LoweredGraph> lowered = cuda::lower_graph(graph, opt.cuda, 148);
        if (!lowered.ok()) return fail(lowered.error().message);
        std::cout << cuda::describe(graph, lowered.value());
    }
    if (!opt.run && !opt.bench && opt.dump_outputs.empty()) return 0;

    if (opt.backend != "cuda") {
        Result<std::unique_ptr<Backend>> b = create_backend(opt.backend);
        return fail(b.ok() ? "unsupported backend" : b.error().message);
    }
    Result<std::unique_ptr<Backend>> backend = cuda::make_cuda_backend(opt.cuda);
    if (!backend.ok()) return fail(backend.error().message);
    Result<std::unique_ptr<Executable>> exe = (*backend)->compile(graph);
    if (!exe.ok()) return fail(exe.error().message);

    const std::vector<HostTensor> inputs = make_random_inputs(graph, opt.seed);
    std::vector<HostTensor> outputs;
    Status st = (*exe)->run(inputs, outputs);
    if (!st.ok()) return fail(st.message());

    if (opt.run) {
        for (std::size_t k = 0; k < outputs.size(); ++k) {
            double sum = 0.0, abs_sum = 0.0;
            for (float v : outputs[k].data) {
                sum += v;
                abs_sum += std::fabs(v);
            }
            std::printf("%s : %s  sum %.9g  abs-sum %.9g\n", graph.node(graph.outputs()[k]).name.c_str(),
                        to_string(outputs[k].type).c_str(), sum, abs_sum);
        }
    }
    if (!opt.dump_outputs.empty()) {
        std::ofstream out(opt.dump_outputs, std::ios::binary);
        if (!out) return fail("cannot write '" + opt.dump_outputs + "'");
        for (const HostTensor& t : outputs) {
            out.write(reinterpret_cast<const char*>(t.data.data()), static_cast<std::streamsize>(t.data.size() * sizeof(float)));
        }
    }
    if (opt.bench) {
        // Wall clock around run(), copies included, as the reference's --bench does (tools/mcc.cpp:242-258).
        for (int i = 0; i < opt.warmup; ++i) {
            st = (*exe)->run(inputs, outputs);
            if (!st.ok()) return fail(st.message());
        }
        std::vector<double> ms;
        for (int i = 0; i < opt.reps; ++i) {
            const auto t0 = std::chrono::steady_clock::now();
            st = (*exe)->run(inputs, outputs);
            const auto t1 = std::chrono::steady_clock::now();
            if (!st.ok()) return fail(st.message());
            ms.push_back(std::chrono::duration<double, std::milli>(t1 - t0).count());
        }
        std::sort(ms.begin(), ms.end());
        auto pct = [&](double p) { return ms[static_cast<std::size_t>(p * static_cast<double>(ms.size() - 1) + 0.5)]; };
        double mean = 0.0;
        for (double v : ms) mean += v;
        mean /= static_cast<double>(ms.size());
        const GraphStats s = compute_stats(graph);
        std::printf("{\"graph\": \"%s\", \"backend\": \"cuda\", \"passes\": \"%s\", \"warmup\": %d, \"reps\": %d, "
                    "\"ms\": {\"median\": %.6f, \"min\": %.6f, \"p10\": %.6f, \"p90\": %.6f, \"mean\": %.6f}, "
                    "\"stats\": {\"nodes\": %zu, \"compute_nodes\": %zu, \"elementwise_ops\": %zu, \"matmuls\": %zu, "
                    "\"fused_nodes\": %zu}, \"intermediate_bytes\": %zu}\n",
                    graph.name().c_str(), opt.passes.c_str(), opt.warmup, opt.reps, pct(0.5), ms.front(), pct(0.1), pct(0.9),
                    mean, s.nodes, s.compute_nodes, s.elementwise_ops, s.matmuls, s.fused_nodes, (*exe)->intermediate_bytes());
    }
    return 0;
}
