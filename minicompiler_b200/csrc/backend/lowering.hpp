#pragma once
// Graph -> launch plan for B200. Pure host logic with no CUDA dependency, so it
// is exercised on machines without a GPU.
//
// It keeps the reference's matmul-kernel vocabulary and selection rules
// (include/minicompiler/cuda/cuda_backend.hpp:20-56, src/cuda/cuda_backend.cpp:14-49,
// src/cuda/matmul_kernels.cu:352-383) and adds what the reference lists as future
// work: an elementwise / fused node whose only matmul-shaped operand is a matmul
// result with no other user is folded into that matmul's epilogue, so the product
// never goes to memory in FP32 and one launch disappears.

#include "backend/eltwise_codegen.hpp"
#include "backend/reduce_codegen.hpp"
#include "core/ir.hpp"
#include "core/plan.hpp"

#include <array>
#include <cstddef>
#include <string>
#include <vector>

namespace minicompiler::cuda {

// Names kept from the reference. On B200 the seven FP32 names all run the one
// FP32 SIMT kernel (SplitK forces the split rule, Auto applies it when the output
// cannot fill the GPU); the TensorCore* names run the tcgen05 kernels.
enum class MatmulKernel {
    Auto,
    Naive,
    Tiled,
    RegisterTiled128,
    RegisterTiled64,
    Vectorized,
    DoubleBuffered,
    SplitK,
    TensorCoreTf32,
    TensorCoreBf16,
    TensorCoreF16,
};

const char* matmul_kernel_name(MatmulKernel kernel);
Result<MatmulKernel> matmul_kernel_from_name(const std::string& name);
bool is_tensor_core(MatmulKernel kernel);
bool uses_split_k(MatmulKernel kernel);

// The reference's split rule, from the count of 128x128 output tiles
// (src/cuda/matmul_kernels.cu:352-367); its tests pin known answers for 30 SMs.
int split_k_splits(int m, int n, int k, int sm_count, int blocks_per_sm = 2);
// Beyond the reference's rule, for `auto` on B200: a problem whose 128x128 tiles cover the SMs but share out badly
// (256 tiles on 148 SMs: two on most, one on the rest, 0.86 of the time useful) is split along K when finer work
// items share out evenly and the reduction costs less than that gains (2048^3: 4 splits, 398 -> 349 us measured).
// Returns the split count, 1 to leave the problem whole.
int balanced_fp32_splits(int m, int n, int k, int sm_count);
// The rule for the tcgen05 kernels: 128x256 tiles, one persistent CTA per SM.
int tensor_core_splits(int m, int n, int k, int sm_count, int elem_bytes);
// Columns per tile of the one-CTA tcgen05 kernel for this problem: 256, or 128 / 64 for problems that neither fill
// the SMs with 128 x 256 tiles nor are worth a K split (operand traffic of the narrow tiling at most this many bytes).
constexpr std::int64_t kNarrowTileTrafficLimit = 128LL << 20;
int tensor_core_tile_n(int m, int n, int k, int sm_count, int elem_bytes);
// Whether a tensor-core matmul split `splits` ways adds its partial tiles inside thread-block clusters (one launch,
// no workspace): asked for with gemm_variant bit 64, for 2, 4 or 8 effective K splits of 256-column tiles (off by
// default: it measured no faster than the second launch it saves). The device layer
// applies the same rule when it launches (tc_cluster_reduce in gemm_launch.cu; a host test compares the two).
bool tensor_core_cluster_reduce(int k, int elem_bytes, int splits, int tile_n, int gemm_variant);
MatmulKernel resolve_matmul_kernel(MatmulKernel kernel, int m, int n, int k, int sm_count);
int matmul_splits(MatmulKernel kernel, int m, int n, int k, int sm_count);
std::size_t matmul_workspace_bytes(MatmulKernel kernel, int m, int n, int splits);

// How the B operand of a tensor-core matmul is laid out for the kernel.
enum class BLayout : int {
    Auto = 0,       // as stored by the graph ([k,n] row-major, an "MN-major" operand)
    RowMajorKN = 1, // same, forced
    Transposed = 2, // a [n,k] copy ("K-major"); free for constants, one pass for inputs
};

struct CudaOptions {
    int device = 0;
    MatmulKernel matmul = MatmulKernel::Auto;
    bool vectorize = true;
    // Additions (trailing, defaulted): not part of the reference's struct.
    bool fuse_epilogue = true;
    BLayout b_layout = BLayout::Auto;
    unsigned eltwise_unroll = 4;
    bool streaming_hints = true;
    int gemm_variant = 0;
    bool replay_graph = true;       // record the launch list once and replay it as a CUDA graph (2+ launches)
    // run() on pinned caller memory for graphs that only stream: 0 = always copy in / run / copy out;
    // 1 = slices pipelined over both copy engines when the graph allows it, else kernels on host memory in place;
    // 2 = kernels on host memory in place only.
    int host_io = 1;
    bool eltwise_fmad = false;      // let the compiler contract a*b+c in generated kernels (not bit-exact vs the CPU)
    // Grid of the generated kernels. 0 (default): one block per tile of the tensor (per row, or 8 rows, for the row
    // kernels) - on B200 the 512 MiB GELU pass streams at 6.32 TB/s this way. n > 0: one wave of n looping blocks per
    // SM instead (4 was the best of those at 5.94 TB/s; 3 gives 5.43, 5 gives 5.46, 8 gives 5.36).
    int eltwise_blocks_per_sm = 0;
    int host_io_slices = 10;    // slices of the pipelined run() on pinned host memory (host_io = 1), streaming graphs
    int host_io_row_slices = 16;  // same for row-independent graphs with matmuls or row kernels (0 turns that path off)
    bool fuse_rows = true;      // runs of steps on rows of one shape become one kernel (reduce_codegen.hpp)
    bool rematerialize = true;  // recompute cheap elementwise values read by a row reduction in each reader
    bool balance_splits = true; // `auto`: split K of FP32 matmuls whose whole tiles share out badly over the SMs
};

enum class Arith : int { F32 = 0, Tf32 = 1, Bf16 = 2, F16 = 3 };  // same numbering as MCD_GEMM_*

// The forms a value can be held in on the device.
enum Rep : int { kRepF32 = 0, kRepHalf = 1, kRepHalfT = 2, kRepF32T = 3, kNumReps = 4 };

struct EpilogueOperand {
    enum class Kind { Scalar, Row, Column, Full };
    NodeId node = kNoNode;
    Kind kind = Kind::Full;
};

struct Step {
    enum class Kind { Elementwise, Matmul, Reduce, RowFused };
    Kind kind = Kind::Elementwise;
    NodeId result = kNoNode;  // the node whose value this step defines

    // Elementwise: `program` over `inputs`. Matmul with a folded consumer: `program` is the
    // consumer's program, loads of `matmul` read the accumulator, other loads read `operands`.
    // Reduce: `program` over `inputs` is evaluated per element of `reduce_shape` (the identity program,
    // or the program of an elementwise producer that only this reduction reads) and each row of the last
    // dimension is combined with `reduce_op`.
    FusedProgram program;
    std::vector<NodeId> inputs;

    OpKind reduce_op = OpKind::RowSum;
    Shape reduce_shape;
    // RowFused: a run of Elementwise / Reduce steps on rows of `reduce_shape`, generated as one kernel
    // (reduce_codegen.hpp). `inputs` are the values it reads from memory, `row_outputs` the values it writes
    // (`result` is the first of them); values used only inside the run never exist in memory.
    std::vector<RowPart> row_parts;
    std::vector<RowOperand::Kind> row_externals;  // per entry of `inputs`
    std::vector<NodeId> row_outputs;

    NodeId matmul = kNoNode;
    NodeId lhs = kNoNode;
    NodeId rhs = kNoNode;
    int m = 0, n = 0, k = 0;
    MatmulKernel kernel = MatmulKernel::DoubleBuffered;  // what matmul_kernels() reports
    Arith arith = Arith::F32;
    int splits = 1;
    int tile_n = 256;  // tensor-core kernels: columns per tile (tensor_core_tile_n)
    bool rhs_transposed = false;
    bool has_epilogue = false;
    std::vector<EpilogueOperand> operands;  // indexed by the program's load numbers (entry for the matmul unused)
    std::vector<int> load_is_accumulator;   // per program input: 1 when it is the matmul result

    bool write_f32 = true;
    HalfKind write_half = HalfKind::None;
    int launches = 1;
};

// A copy made right after a step (or right after upload, for inputs): f32 -> another Rep.
struct Recast {
    NodeId node = kNoNode;
    Rep to = kRepHalf;
};

struct LoweredGraph {
    std::vector<Step> steps;
    std::vector<std::vector<Recast>> after_step;  // per step
    std::vector<Recast> after_upload;             // for graph inputs
    std::vector<Recast> at_compile;               // for constants
    // needs[node][rep]: that form of the value is read by some step (or is a graph output).
    std::vector<std::array<bool, kNumReps>> needs;
    HalfKind half_kind = HalfKind::None;
    std::size_t kernel_launches = 0;

    // Buffer plan over (node, rep) values: index node * kNumReps + rep.
    std::vector<PoolValue> pool_values;
    std::vector<PoolStep> pool_steps;
    PoolPlan pool;
    std::size_t workspace_bytes = 0;  // one split-K workspace shared by all steps
};

// Row pitch (in elements) of the 16-bit copy of a rank-2 tensor with `cols` columns:
// padded so that every row starts on a 16-byte boundary, as TMA requires.
inline std::int64_t half_pitch(std::int64_t cols) { return (cols + 7) / 8 * 8; }
std::size_t rep_bytes(const TensorType& type, Rep rep);

// pool_outputs = false keeps the FP32 form of every graph output out of the buffer pool (the executable then gives
// each output a region of its own): needed when row slices of one run overlap, so that a later slice's
// intermediates cannot land on an earlier slice's output rows that are still being copied out.
Result<LoweredGraph> lower_graph(const Graph& graph, const CudaOptions& options, int sm_count, bool pool_outputs = true);

// The `mc_epilogue` device function for a matmul step with a folded consumer
// (the text that goes in front of mcd_gemm_source()).
std::string generate_epilogue_source(const Graph& graph, const Step& step);

// One line per step, for tests and `mcc --print-plan`.
std::string describe(const Graph& graph, const LoweredGraph& lowered);

}  // namespace minicompiler::cuda
