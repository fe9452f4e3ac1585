#pragma once
// Reader and printer for the .mcg text format, and the seeded generator that
// fills `uniform(...)` constants and benchmark inputs. The grammar, the dim
// override rule and every diagnostic follow the reference
// (include/minicompiler/parser.hpp:13-38, src/parser.cpp, src/random.cpp:6-26).
//
//   graph mlp                                    optional, before any node
//   dim B = 64                                   named extent, overridable
//   input x : f32[B, 256]
//   const w : f32[256, 512] = uniform(seed=1, lo=-0.05, hi=0.05)
//   const b : f32[512] = 0.1                     splat
//   const v : f32[3] = [1, 2, 3]                 row-major literal
//   h = matmul x, w
//   output y, h

#include "core/ir.hpp"

#include <cstdint>
#include <map>
#include <string>
#include <string_view>
#include <vector>

namespace minicompiler {

struct ParseOptions {
    std::map<std::string, std::int64_t> dims;  // replaces the value of `dim NAME = ...`
    // When set, receives the value every declared dim ended up with.
    std::map<std::string, std::int64_t>* resolved_dims = nullptr;
};

Result<Graph> parse_graph(std::string_view text, const ParseOptions& options = {});
Result<Graph> parse_graph_file(const std::string& path, const ParseOptions& options = {});

std::string print_graph(const Graph& graph);
std::string describe_constant(const Node& constant);  // "0.5", "[1, 2, 3]", "<4096 values>"

// splitmix64 stream -> 24-bit mantissa u in [0,1) -> lo + (hi-lo)*u, with the
// multiply and the add rounded separately (never one FMA).
void fill_uniform(float* out, std::size_t count, std::uint64_t seed, float lo, float hi);
std::vector<float> uniform_values(std::size_t count, std::uint64_t seed, float lo, float hi);

// A tensor in host memory.
struct HostTensor {
    TensorType type;
    std::vector<float> data;

    HostTensor() = default;
    explicit HostTensor(TensorType t) : type(std::move(t)), data(type.num_elements()) {}
    HostTensor(TensorType t, std::vector<float> values) : type(std::move(t)), data(std::move(values)) {}
};

// Input k of the graph gets uniform_values(n, seed + k, lo, hi)
// (reference src/runtime/host_tensor.cpp:7-14).
std::vector<HostTensor> make_random_inputs(const Graph& graph, std::uint64_t seed, float lo = -1.0f, float hi = 1.0f);

}  // namespace minicompiler
