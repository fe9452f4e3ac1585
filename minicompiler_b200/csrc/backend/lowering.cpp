#include "backend/lowering.hpp"

#include <algorithm>
#include <cmath>
#include <array>
#include <cstdio>
#include <sstream>

namespace minicompiler::cuda {

// ------------------------------------------------------- kernel vocabulary

namespace {

constexpr MatmulKernel kAllKernels[] = {
    MatmulKernel::Auto,           MatmulKernel::Naive,          MatmulKernel::Tiled,
    MatmulKernel::RegisterTiled128, MatmulKernel::RegisterTiled64, MatmulKernel::Vectorized,
    MatmulKernel::DoubleBuffered, MatmulKernel::SplitK,         MatmulKernel::TensorCoreTf32,
    MatmulKernel::TensorCoreBf16, MatmulKernel::TensorCoreF16,
};

}  // namespace

const char* matmul_kernel_name(MatmulKernel kernel) {
    switch (kernel) {
        case MatmulKernel::Auto: return "auto";
        case MatmulKernel::Naive: return "naive";
        case MatmulKernel::Tiled: return "tiled";
        case MatmulKernel::RegisterTiled128: return "register_tiled_128";
        case MatmulKernel::RegisterTiled64: return "register_tiled_64";
        case MatmulKernel::Vectorized: return "vectorized";
        case MatmulKernel::DoubleBuffered: return "double_buffered";
        case MatmulKernel::SplitK: return "split_k";
        case MatmulKernel::TensorCoreTf32: return "tensor_core_tf32";
        case MatmulKernel::TensorCoreBf16: return "tensor_core_bf16";
        case MatmulKernel::TensorCoreF16: return "tensor_core_f16";
    }
    return "?";
}

Result<MatmulKernel> matmul_kernel_from_name(const std::string& name) {
    std::string known;
    for (MatmulKernel k : kAllKernels) {
        if (name == matmul_kernel_name(k)) return k;
        known += (known.empty() ? "" : ", ") + std::string(matmul_kernel_name(k));
    }
    return Error{"unknown matmul kernel '" + name + "' (" + known + ")"};
}

bool is_tensor_core(MatmulKernel kernel) {
    return kernel == MatmulKernel::TensorCoreTf32 || kernel == MatmulKernel::TensorCoreBf16 ||
           kernel == MatmulKernel::TensorCoreF16;
}

bool uses_split_k(MatmulKernel kernel) { return kernel == MatmulKernel::SplitK || is_tensor_core(kernel); }

int split_k_splits(int m, int n, int k, int sm_count, int blocks_per_sm) {
    const std::int64_t tiles = ((static_cast<std::int64_t>(m) + 127) / 128) * ((static_cast<std::int64_t>(n) + 127) / 128);
    const std::int64_t sms = sm_count;
    if (5 * tiles >= 4 * sms) return 1;  // the output alone covers 80% of the SMs
    // Up to half the SMs' worth of tiles: aim for one block per SM. Between half and 80%: two per SM
    // where an SM holds two blocks, otherwise still one.
    std::int64_t splits = (2 * tiles <= sms || blocks_per_sm < 2) ? sms / tiles : 2 * sms / tiles;
    splits = std::min<std::int64_t>(splits, k / 64);  // no split shorter than 64 along K
    return static_cast<int>(std::max<std::int64_t>(splits, 1));
}

namespace {

struct TensorCoreTiling {
    int tile_n;
    int splits;
};

TensorCoreTiling tensor_core_tiling(int m, int n, int k, int sm_count, int elem_bytes, bool narrow_single_row = true) {
    const std::int64_t rows = (static_cast<std::int64_t>(m) + 127) / 128;
    const std::int64_t sms = sm_count;
    const std::int64_t wide_tiles = rows * ((static_cast<std::int64_t>(n) + 255) / 256);
    if (5 * wide_tiles >= 4 * sms) return {256, 1};
    // A problem too small to fill the SMs with 128 x 256 tiles: narrower tiles in one launch beat a K split plus
    // its reduction pass as long as the extra operand traffic stays small (every tile re-reads its 128 rows of A).
    const std::int64_t block_k = 128 / elem_bytes;
    const std::int64_t k_blocks = (k + block_k - 1) / block_k;
    for (int width : {128, 64}) {
        const std::int64_t tiles = rows * ((static_cast<std::int64_t>(n) + width - 1) / width);
        const std::int64_t traffic = tiles * k_blocks * (128 * 128 + width * 128);
        if (5 * tiles >= 4 * sms || width == 64) {
            if (traffic <= kNarrowTileTrafficLimit && 2 * tiles >= sms) return {width, 1};
            break;
        }
    }
    // Split K, at least 4 K blocks per work item.
    const std::int64_t wide_splits = std::max<std::int64_t>(1, std::min<std::int64_t>(sms / wide_tiles, k_blocks / 4));
    // A single row of tiles (up to 128 rows of A) that would be cut 4 or more ways: 128-column tiles need half the K
    // slices for the same number of work items, so half the partial sums are written and added up again, and with
    // fewer than 128 rows the ring stages only the rows there are and is deep enough for the narrower B tiles
    // (128 x 8192 x 8192: 40.0 against 44.0 us; 64 rows: 37.9 against 40.0; 16 and 32 rows: the same 38 us).
    if (narrow_single_row && rows == 1 && wide_splits >= 4) {
        const std::int64_t tiles = (static_cast<std::int64_t>(n) + 127) / 128;
        const std::int64_t splits = std::max<std::int64_t>(1, std::min<std::int64_t>(sms / tiles, k_blocks / 4));
        if (splits >= 2) return {128, static_cast<int>(splits)};
    }
    return {256, static_cast<int>(wide_splits)};
}

}  // namespace

int tensor_core_tile_n(int m, int n, int k, int sm_count, int elem_bytes) {
    return tensor_core_tiling(m, n, k, sm_count, elem_bytes).tile_n;
}

int tensor_core_splits(int m, int n, int k, int sm_count, int elem_bytes) {
    return tensor_core_tiling(m, n, k, sm_count, elem_bytes).splits;
}

int balanced_fp32_splits(int m, int n, int k, int sm_count) {
    const std::int64_t tiles = ((static_cast<std::int64_t>(m) + 127) / 128) * ((static_cast<std::int64_t>(n) + 127) / 128);
    // Work is shared out in whole blocks: with `items` equal blocks an SM gets ceil(items / SMs) of them at worst.
    auto efficiency = [&](std::int64_t items) {
        const double per_sm = static_cast<double>(items) / sm_count;
        return per_sm / std::ceil(per_sm);
    };
    const double unsplit = efficiency(tiles);
    if (unsplit >= 0.9) return 1;
    // Seconds: the matmul at the kernel's measured rate, and the reduction that a split adds (it reads `splits`
    // partial results and writes one, plus a launch).
    const double main_s = 2.0 * m * n * static_cast<double>(k) / 50e12 / unsplit;
    int best = 1;
    double best_gain = 0.03;
    for (int splits : {2, 3, 4, 6, 8}) {
        if (k / splits < 256) break;
        const double reduce_s = (splits + 1) * 4.0 * m * n / 5e12 + 4e-6;
        const double total_s = main_s * unsplit / efficiency(tiles * splits) + reduce_s;
        const double gain = main_s / total_s - 1.0;
        if (gain > best_gain) {
            best_gain = gain;
            best = splits;
        }
    }
    return best;
}

bool tensor_core_cluster_reduce(int k, int elem_bytes, int splits, int tile_n, int gemm_variant) {
    if ((gemm_variant & 64) == 0 || (tile_n != 0 && tile_n != 256)) return false;
    const int block_k = 128 / elem_bytes;
    const int k_blocks = (k + block_k - 1) / block_k;
    const int asked = std::max(1, std::min(splits, k_blocks));
    const int per = (k_blocks + asked - 1) / asked;
    const int effective = (k_blocks + per - 1) / per;
    return effective == 2 || effective == 4 || effective == 8;
}

MatmulKernel resolve_matmul_kernel(MatmulKernel kernel, int m, int n, int k, int sm_count) {
    if (kernel != MatmulKernel::Auto) return kernel;
    return split_k_splits(m, n, k, sm_count) > 1 ? MatmulKernel::SplitK : MatmulKernel::DoubleBuffered;
}

int matmul_splits(MatmulKernel kernel, int m, int n, int k, int sm_count) {
    if (kernel == MatmulKernel::SplitK) return split_k_splits(m, n, k, sm_count);
    if (kernel == MatmulKernel::TensorCoreTf32) return tensor_core_splits(m, n, k, sm_count, 4);
    if (is_tensor_core(kernel)) return tensor_core_splits(m, n, k, sm_count, 2);
    return 1;
}

std::size_t matmul_workspace_bytes(MatmulKernel kernel, int m, int n, int splits) {
    if (!uses_split_k(kernel) || splits <= 1) return 0;
    return static_cast<std::size_t>(splits) * static_cast<std::size_t>(m) * static_cast<std::size_t>(n) * sizeof(float);
}

std::size_t rep_bytes(const TensorType& type, Rep rep) {
    if (rep == kRepF32) return type.size_bytes();
    // The other forms exist only for rank-2 matmul operands.
    const std::int64_t rows = type.shape.size() == 2 ? type.shape[0] : 1;
    const std::int64_t cols = type.shape.size() == 2 ? type.shape[1] : static_cast<std::int64_t>(type.num_elements());
    switch (rep) {
        case kRepHalf: return static_cast<std::size_t>(rows * half_pitch(cols)) * 2;
        case kRepHalfT: return static_cast<std::size_t>(cols * half_pitch(rows)) * 2;
        case kRepF32T: return static_cast<std::size_t>(cols * ((rows + 3) / 4 * 4)) * 4;
        default: return type.size_bytes();
    }
}

// ---------------------------------------------------------------- lowering

namespace {

// Can `operand` be read from inside a matmul epilogue over an [m,n] result?
bool classify_epilogue_operand(const Shape& operand, const Shape& out, EpilogueOperand::Kind* kind) {
    const Access a = classify_access(operand, out);
    switch (a.kind) {
        case AccessKind::Scalar: *kind = EpilogueOperand::Kind::Scalar; return true;
        case AccessKind::Contiguous: *kind = EpilogueOperand::Kind::Full; return true;
        case AccessKind::Periodic:
            if (a.period != static_cast<std::size_t>(out[1])) return false;
            *kind = EpilogueOperand::Kind::Row;
            return true;
        case AccessKind::General:
            if (a.strides.size() == 2 && a.strides[0] == 1 && a.strides[1] == 0) {
                *kind = EpilogueOperand::Kind::Column;
                return true;
            }
            return false;
    }
    return false;
}

// `user` reads value `value`, which `producer` computes: returns the program that evaluates the producer's
// instructions in place of those loads, over the user's other inputs followed by the producer's inputs it did not
// already read. Per element it performs the same operations in the same order as the two programs did.
void inline_producer(Step* user, NodeId value, const Step& producer) {
    std::vector<NodeId> inputs;
    for (NodeId in : user->inputs) {
        if (in != value && std::find(inputs.begin(), inputs.end(), in) == inputs.end()) inputs.push_back(in);
    }
    for (NodeId in : producer.inputs) {
        if (std::find(inputs.begin(), inputs.end(), in) == inputs.end()) inputs.push_back(in);
    }
    auto slot_of = [&](NodeId in) {
        return static_cast<std::int32_t>(std::find(inputs.begin(), inputs.end(), in) - inputs.begin());
    };
    FusedProgram merged;
    merged.source_nodes = producer.program.source_nodes;
    merged.source_nodes.insert(merged.source_nodes.end(), user->program.source_nodes.begin(), user->program.source_nodes.end());
    std::vector<std::int32_t> reg_of_producer(producer.program.instrs.size());
    for (std::size_t r = 0; r < producer.program.instrs.size(); ++r) {
        FusedInstr ins = producer.program.instrs[r];
        if (ins.kind == FusedInstr::Kind::Load) {
            ins.a = slot_of(producer.inputs[static_cast<std::size_t>(ins.a)]);
        } else if (ins.kind != FusedInstr::Kind::Immediate) {
            ins.a = reg_of_producer[static_cast<std::size_t>(ins.a)];
            if (ins.kind == FusedInstr::Kind::Binary) ins.b = reg_of_producer[static_cast<std::size_t>(ins.b)];
        }
        reg_of_producer[r] = static_cast<std::int32_t>(merged.instrs.size());
        merged.instrs.push_back(ins);
    }
    const std::int32_t produced = reg_of_producer.back();
    std::vector<std::int32_t> reg_of_user(user->program.instrs.size());
    for (std::size_t r = 0; r < user->program.instrs.size(); ++r) {
        FusedInstr ins = user->program.instrs[r];
        if (ins.kind == FusedInstr::Kind::Load) {
            const NodeId in = user->inputs[static_cast<std::size_t>(ins.a)];
            if (in == value) {
                reg_of_user[r] = produced;
                continue;
            }
            ins.a = slot_of(in);
        } else if (ins.kind != FusedInstr::Kind::Immediate) {
            ins.a = reg_of_user[static_cast<std::size_t>(ins.a)];
            if (ins.kind == FusedInstr::Kind::Binary) ins.b = reg_of_user[static_cast<std::size_t>(ins.b)];
        }
        reg_of_user[r] = static_cast<std::int32_t>(merged.instrs.size());
        merged.instrs.push_back(ins);
    }
    if (reg_of_user.back() != static_cast<std::int32_t>(merged.instrs.size()) - 1) {
        // The user's result is the produced value itself: the result must be the last instruction.
        merged.instrs.push_back(merged.instrs[static_cast<std::size_t>(reg_of_user.back())]);
    }
    user->program = std::move(merged);
    user->inputs = std::move(inputs);
}

// How a value of shape `operand` that lives in memory is read by a step working on rows of `rows_shape`
// (`over_full`: the step computes one value per element, otherwise one per row).
bool classify_row_operand(const Shape& operand, const Shape& rows_shape, bool over_full, RowOperand::Kind* kind) {
    if (num_elements(operand) == 1) {
        *kind = RowOperand::Kind::Scalar;
        return true;
    }
    Shape reduced = rows_shape;
    reduced.back() = 1;
    if (operand == reduced) {
        *kind = RowOperand::Kind::PerRow;
        return true;
    }
    if (!over_full) return false;
    if (operand == rows_shape) {
        *kind = RowOperand::Kind::Full;
        return true;
    }
    if (operand.size() <= rows_shape.size() && operand.back() == rows_shape.back() &&
        num_elements(operand) == static_cast<std::size_t>(rows_shape.back())) {
        *kind = RowOperand::Kind::RowVector;
        return true;
    }
    return false;
}

// Runs of consecutive steps that all work on rows of one shape and contain a row reduction become one RowFused
// step (see reduce_codegen.hpp). Steps keep their order inside the kernel, values read by nothing outside the run
// are never written.
void fuse_row_runs(const Graph& graph, std::vector<Step>* steps) {
    auto reads = [](const Step& s, NodeId v) {
        return s.lhs == v || s.rhs == v || std::find(s.inputs.begin(), s.inputs.end(), v) != s.inputs.end();
    };
    for (std::size_t r = 0; r < steps->size(); ++r) {
        if ((*steps)[r].kind != Step::Kind::Reduce) continue;
        const Shape rows_shape = (*steps)[r].reduce_shape;
        const std::int64_t width = rows_shape.back();
        if (width < kRowFusedMinWidth || width > kRowFusedMaxWidth) continue;
        Shape reduced = rows_shape;
        reduced.back() = 1;
        // Whether a step can join, given the results of the steps already in the run (which it may read freely).
        auto joins = [&](const Step& s, const std::vector<NodeId>& inside) {
            bool over_full = true;
            if (s.kind == Step::Kind::Reduce) {
                if (s.reduce_shape != rows_shape) return false;
            } else if (s.kind == Step::Kind::Elementwise) {
                const Shape& shape = graph.node(s.result).type.shape;
                if (shape != rows_shape && shape != reduced) return false;
                over_full = shape == rows_shape;
            } else {
                return false;
            }
            for (NodeId in : s.inputs) {
                if (std::find(inside.begin(), inside.end(), in) != inside.end()) continue;
                RowOperand::Kind kind;
                if (!classify_row_operand(graph.node(in).type.shape, rows_shape, over_full, &kind)) return false;
            }
            return true;
        };
        std::size_t lo = r, hi = r;
        std::vector<NodeId> inside{(*steps)[r].result};
        if (!joins((*steps)[r], {})) continue;
        // Later steps may read what the run has produced; earlier steps are taken while every step already in the
        // run stays readable (their results only replace memory operands of the same shapes).
        while (hi + 1 < steps->size() && joins((*steps)[hi + 1], inside)) inside.push_back((*steps)[++hi].result);
        while (lo > 0 && joins((*steps)[lo - 1], {})) inside.push_back((*steps)[--lo].result);
        if (hi == lo) continue;

        Step fused;
        fused.kind = Step::Kind::RowFused;
        fused.reduce_shape = rows_shape;
        std::vector<NodeId> produced;  // value number = position
        std::size_t full_values = 0;
        bool ok = true;
        for (std::size_t i = lo; i <= hi && ok; ++i) {
            const Step& s = (*steps)[i];
            RowPart part;
            part.is_reduce = s.kind == Step::Kind::Reduce;
            part.reduce_op = s.reduce_op;
            part.program = s.program;
            part.result = static_cast<int>(produced.size());
            part.result_is_full = !part.is_reduce && graph.node(s.result).type.shape == rows_shape;
            part.name = graph.node(s.result).name;
            const bool over_full = part.is_reduce || part.result_is_full;
            for (NodeId in : s.inputs) {
                RowOperand operand;
                const auto made = std::find(produced.begin(), produced.end(), in);
                if (made != produced.end()) {
                    operand.value = static_cast<int>(made - produced.begin());
                    operand.kind = fused.row_parts[static_cast<std::size_t>(operand.value)].result_is_full ? RowOperand::Kind::Full
                                                                                                           : RowOperand::Kind::PerRow;
                    if (operand.kind == RowOperand::Kind::Full && !over_full) ok = false;
                } else {
                    ok = ok && classify_row_operand(graph.node(in).type.shape, rows_shape, over_full, &operand.kind);
                    auto seen = std::find(fused.inputs.begin(), fused.inputs.end(), in);
                    if (seen == fused.inputs.end()) {
                        fused.inputs.push_back(in);
                        fused.row_externals.push_back(operand.kind);
                        if (operand.kind == RowOperand::Kind::Full) ++full_values;
                        seen = fused.inputs.end() - 1;
                    }
                    operand.external = static_cast<int>(seen - fused.inputs.begin());
                    if (fused.row_externals[static_cast<std::size_t>(operand.external)] != operand.kind) ok = false;
                }
                part.operands.push_back(operand);
            }
            if (part.result_is_full) ++full_values;
            bool leaves = graph.is_output(s.result);
            for (std::size_t u = 0; u < steps->size() && !leaves; ++u) {
                if ((u < lo || u > hi) && reads((*steps)[u], s.result)) leaves = true;
            }
            if (leaves) {
                part.output = static_cast<int>(fused.row_outputs.size());
                fused.row_outputs.push_back(s.result);
            }
            produced.push_back(s.result);
            fused.row_parts.push_back(std::move(part));
        }
        // Every full-shaped value costs width / 256 registers per thread while it is live.
        const std::size_t per_thread = static_cast<std::size_t>((row_chunk(width) + row_threads(width) - 1) / row_threads(width));
        if (!ok || fused.row_outputs.empty() || full_values * per_thread > 160) continue;
        fused.result = fused.row_outputs[0];
        steps->erase(steps->begin() + static_cast<std::ptrdiff_t>(lo), steps->begin() + static_cast<std::ptrdiff_t>(hi) + 1);
        steps->insert(steps->begin() + static_cast<std::ptrdiff_t>(lo), std::move(fused));
        r = lo;
    }
}

// The shape a step evaluates its program over.
const Shape& evaluation_shape(const Graph& graph, const Step& s) {
    return s.kind == Step::Kind::Reduce ? s.reduce_shape : graph.node(s.result).type.shape;
}

// An elementwise value that a row reduction reads, together with other elementwise or reduction steps of the same
// shape, is recomputed by each of them instead of being written once and read back: the readers already stream
// tensors of that size, so this removes one write and one read pass (softmax: exp(x - max); LayerNorm: x - mean).
// Only cheap producers qualify, and only when every reader can take them.
void rematerialize_for_reductions(const Graph& graph, std::vector<Step>* steps) {
    constexpr std::size_t kMaxProducerOps = 16;
    constexpr std::size_t kMaxInputs = 8;
    for (std::size_t pi = 0; pi < steps->size();) {
        const Step& producer = (*steps)[pi];
        const NodeId value = producer.result;
        bool candidate = producer.kind == Step::Kind::Elementwise && !graph.is_output(value) &&
                         producer.program.num_ops() <= kMaxProducerOps;
        std::vector<std::size_t> readers;
        bool feeds_reduction = false;
        for (std::size_t ui = 0; candidate && ui < steps->size(); ++ui) {
            const Step& user = (*steps)[ui];
            if (user.kind == Step::Kind::Matmul || user.kind == Step::Kind::RowFused) {
                const bool reads = user.lhs == value || user.rhs == value ||
                                   std::find(user.inputs.begin(), user.inputs.end(), value) != user.inputs.end();
                if (reads) candidate = false;
                continue;
            }
            if (std::find(user.inputs.begin(), user.inputs.end(), value) == user.inputs.end()) continue;
            if (evaluation_shape(graph, user) != graph.node(value).type.shape) candidate = false;
            std::size_t merged_inputs = producer.inputs.size();
            for (NodeId in : user.inputs) {
                if (in != value && std::find(producer.inputs.begin(), producer.inputs.end(), in) == producer.inputs.end()) ++merged_inputs;
            }
            if (merged_inputs > kMaxInputs) candidate = false;
            feeds_reduction = feeds_reduction || user.kind == Step::Kind::Reduce;
            readers.push_back(ui);
        }
        if (!candidate || !feeds_reduction || readers.size() < 2) {
            ++pi;
            continue;
        }
        const Step copy = producer;
        for (std::size_t ui : readers) inline_producer(&(*steps)[ui], value, copy);
        steps->erase(steps->begin() + static_cast<std::ptrdiff_t>(pi));
    }
}

}  // namespace

Result<LoweredGraph> lower_graph(const Graph& graph, const CudaOptions& options, int sm_count, bool pool_outputs) {
    const std::size_t count = graph.num_nodes();
    const std::vector<std::vector<NodeId>> users = graph.compute_users();
    LoweredGraph out;
    out.needs.assign(count, {false, false, false, false});
    if (options.matmul == MatmulKernel::TensorCoreBf16) out.half_kind = HalfKind::Bf16;
    if (options.matmul == MatmulKernel::TensorCoreF16) out.half_kind = HalfKind::F16;
    const bool rhs_transposed = options.b_layout == BLayout::Transposed;

    // Which matmul is folded into which consumer.
    std::vector<NodeId> folded_into(count, kNoNode);  // matmul -> consumer
    std::vector<NodeId> carries(count, kNoNode);      // consumer -> matmul
    if (options.fuse_epilogue) {
        for (std::size_t i = 0; i < count; ++i) {
            const auto h = static_cast<NodeId>(i);
            const Node& hn = graph.node(h);
            if (hn.op != OpKind::MatMul || graph.is_output(h) || users[i].size() != 1) continue;
            const NodeId u = users[i][0];
            const Node& un = graph.node(u);
            const bool elementwise_like = is_elementwise(un.op) || un.op == OpKind::FusedElementwise;
            if (!elementwise_like || un.type.shape != hn.type.shape || carries[static_cast<std::size_t>(u)] != kNoNode) continue;
            bool ok = true;
            std::size_t extra = 0;
            for (NodeId in : un.inputs) {
                if (in == h) continue;
                EpilogueOperand::Kind kind;
                if (graph.node(in).op == OpKind::MatMul && folded_into[static_cast<std::size_t>(in)] == u) ok = false;
                if (!classify_epilogue_operand(graph.node(in).type.shape, un.type.shape, &kind)) ok = false;
                ++extra;
            }
            if (!ok || extra > 6) continue;
            folded_into[i] = u;
            carries[static_cast<std::size_t>(u)] = h;
        }
    }

    auto make_matmul_step = [&](NodeId h) {
        const Node& hn = graph.node(h);
        const Shape& a = graph.node(hn.inputs[0]).type.shape;
        Step s;
        s.kind = Step::Kind::Matmul;
        s.matmul = h;
        s.result = h;
        s.lhs = hn.inputs[0];
        s.rhs = hn.inputs[1];
        s.m = static_cast<int>(a[0]);
        s.k = static_cast<int>(a[1]);
        s.n = static_cast<int>(hn.type.shape[1]);
        MatmulKernel kernel = resolve_matmul_kernel(options.matmul, s.m, s.n, s.k, sm_count);
        // TF32 reads the FP32 tensors in place through TMA, which needs 16-byte row pitches.
        if (kernel == MatmulKernel::TensorCoreTf32 && (s.k % 4 != 0 || s.n % 4 != 0)) {
            kernel = resolve_matmul_kernel(MatmulKernel::Auto, s.m, s.n, s.k, sm_count);
        }
        // `auto` on a problem the reference's rule leaves whole: split K after all when whole tiles would leave SMs
        // idle for a good part of the launch and finer work items share out evenly.
        int balanced = 1;
        if (options.matmul == MatmulKernel::Auto && kernel == MatmulKernel::DoubleBuffered && options.balance_splits) {
            balanced = balanced_fp32_splits(s.m, s.n, s.k, sm_count);
            if (balanced > 1) kernel = MatmulKernel::SplitK;
        }
        s.kernel = kernel;
        s.arith = kernel == MatmulKernel::TensorCoreTf32   ? Arith::Tf32
                  : kernel == MatmulKernel::TensorCoreBf16 ? Arith::Bf16
                  : kernel == MatmulKernel::TensorCoreF16  ? Arith::F16
                                                           : Arith::F32;
        s.splits = balanced > 1 ? balanced : matmul_splits(kernel, s.m, s.n, s.k, sm_count);
        if (is_tensor_core(kernel)) {
            // The slices of a tile can only meet inside clusters (variant bit 64) with 256-column tiles.
            const TensorCoreTiling tiling = tensor_core_tiling(s.m, s.n, s.k, sm_count, kernel == MatmulKernel::TensorCoreTf32 ? 4 : 2,
                                                               (options.gemm_variant & 64) == 0);
            s.tile_n = tiling.tile_n;
            s.splits = tiling.splits;
        }
        // TF32 always takes the [n,k] copy of B: with 32-bit elements the MN-major shared-memory form did not
        // yield correct products on B200, while the K-major form does. 16-bit operands work in both forms.
        s.rhs_transposed = is_tensor_core(kernel) && (rhs_transposed || kernel == MatmulKernel::TensorCoreTf32);
        s.launches = s.splits > 1 ? 2 : 1;
        if (is_tensor_core(kernel) && s.splits > 1 &&
            tensor_core_cluster_reduce(s.k, kernel == MatmulKernel::TensorCoreTf32 ? 4 : 2, s.splits, s.tile_n, options.gemm_variant)) {
            s.launches = 1;  // the K slices of a tile meet inside a thread-block cluster: no second launch, no workspace
        }
        return s;
    };

    // An elementwise producer that only a row reduction reads is evaluated inside the reduction kernel and never
    // written out.
    std::vector<NodeId> absorbed_by(count, kNoNode);  // producer -> reduction
    for (std::size_t i = 0; i < count; ++i) {
        const Node& rn = graph.node(static_cast<NodeId>(i));
        if (!is_row_reduce(rn.op)) continue;
        const NodeId p = rn.inputs[0];
        const Node& pn = graph.node(p);
        const auto pi = static_cast<std::size_t>(p);
        const bool elementwise_like = is_elementwise(pn.op) || pn.op == OpKind::FusedElementwise;
        if (elementwise_like && !graph.is_output(p) && users[pi].size() == 1 && carries[pi] == kNoNode) {
            absorbed_by[pi] = static_cast<NodeId>(i);
        }
    }

    std::vector<std::int32_t> step_of(count, -1);
    for (std::size_t i = 0; i < count; ++i) {
        const auto id = static_cast<NodeId>(i);
        const Node& n = graph.node(id);
        if (!is_compute(n.op)) continue;
        if (absorbed_by[i] != kNoNode) continue;  // evaluated inside its reduction
        if (is_row_reduce(n.op)) {
            Step s;
            s.kind = Step::Kind::Reduce;
            s.result = id;
            s.reduce_op = n.op;
            const NodeId p = n.inputs[0];
            const Node& pn = graph.node(p);
            s.reduce_shape = pn.type.shape;
            if (absorbed_by[static_cast<std::size_t>(p)] == id) {
                s.program = pn.op == OpKind::FusedElementwise ? *pn.fused : single_op_program(pn.op);
                s.inputs = pn.inputs;
            } else {
                s.program.instrs.push_back(FusedInstr::load(0));
                s.inputs = {p};
            }
            out.steps.push_back(std::move(s));
        } else if (n.op == OpKind::MatMul) {
            if (folded_into[i] != kNoNode) continue;  // emitted with its consumer
            out.steps.push_back(make_matmul_step(id));
        } else if (carries[i] != kNoNode) {
            Step s = make_matmul_step(carries[i]);
            s.result = id;
            s.has_epilogue = true;
            s.program = n.op == OpKind::FusedElementwise ? *n.fused : single_op_program(n.op);
            s.inputs = n.inputs;
            for (NodeId in : n.inputs) {
                EpilogueOperand operand;
                operand.node = in;
                const bool is_acc = in == carries[i];
                s.load_is_accumulator.push_back(is_acc ? 1 : 0);
                if (!is_acc) classify_epilogue_operand(graph.node(in).type.shape, n.type.shape, &operand.kind);
                s.operands.push_back(operand);
            }
            out.steps.push_back(std::move(s));
        } else {
            Step s;
            s.kind = Step::Kind::Elementwise;
            s.result = id;
            s.program = n.op == OpKind::FusedElementwise ? *n.fused : single_op_program(n.op);
            s.inputs = n.inputs;
            out.steps.push_back(std::move(s));
        }
    }
    if (options.fuse_rows) fuse_row_runs(graph, &out.steps);
    if (options.rematerialize) rematerialize_for_reductions(graph, &out.steps);
    std::vector<bool> f32_only(count, false);  // values whose producing kernel writes FP32 and nothing else
    for (std::size_t i = 0; i < out.steps.size(); ++i) {
        const Step& s = out.steps[i];
        step_of[static_cast<std::size_t>(s.result)] = static_cast<std::int32_t>(i);
        if (s.kind == Step::Kind::Reduce) f32_only[static_cast<std::size_t>(s.result)] = true;
        for (NodeId w : s.row_outputs) {
            step_of[static_cast<std::size_t>(w)] = static_cast<std::int32_t>(i);
            f32_only[static_cast<std::size_t>(w)] = true;
        }
    }

    // What form each value is read in.
    auto need = [&](NodeId v, Rep rep) { out.needs[static_cast<std::size_t>(v)][rep] = true; };
    for (const Step& s : out.steps) {
        if (s.kind != Step::Kind::Matmul) {
            for (NodeId in : s.inputs) need(in, kRepF32);
            continue;
        }
        const bool half = s.arith == Arith::Bf16 || s.arith == Arith::F16;
        need(s.lhs, half ? kRepHalf : kRepF32);
        if (half) {
            need(s.rhs, s.rhs_transposed ? kRepHalfT : kRepHalf);
        } else {
            need(s.rhs, s.rhs_transposed ? kRepF32T : kRepF32);
        }
        if (s.has_epilogue) {
            for (std::size_t k = 0; k < s.inputs.size(); ++k) {
                if (!s.load_is_accumulator[k]) need(s.inputs[k], kRepF32);
            }
        }
    }
    for (NodeId o : graph.outputs()) need(o, kRepF32);

    // Derived forms that no kernel writes directly come from the FP32 form by a recast.
    out.after_step.resize(out.steps.size());
    for (std::size_t i = 0; i < count; ++i) {
        const auto id = static_cast<NodeId>(i);
        const Node& n = graph.node(id);
        auto& needs = out.needs[i];
        if (is_compute(n.op)) {
            if (step_of[i] < 0) continue;  // a folded matmul or an absorbed producer has no value of its own
            for (Rep rep : {kRepHalf, kRepHalfT, kRepF32T}) {
                if (!needs[rep]) continue;
                if (rep == kRepHalf && !f32_only[i]) continue;  // written by the producing kernel itself
                needs[kRepF32] = true;
                out.after_step[static_cast<std::size_t>(step_of[i])].push_back({id, rep});
            }
            if (!needs[kRepF32] && !needs[kRepHalf]) needs[kRepF32] = true;  // a dead node still runs and writes
        } else {
            for (Rep rep : {kRepHalf, kRepHalfT, kRepF32T}) {
                if (!needs[rep]) continue;
                if (n.op == OpKind::Input) {
                    out.after_upload.push_back({id, rep});
                } else {
                    out.at_compile.push_back({id, rep});
                }
            }
            needs[kRepF32] = true;  // inputs and constants always land in FP32 first
        }
    }
    for (Step& s : out.steps) {
        const auto& needs = out.needs[static_cast<std::size_t>(s.result)];
        s.write_f32 = needs[kRepF32];
        s.write_half = needs[kRepHalf] && !f32_only[static_cast<std::size_t>(s.result)] ? out.half_kind : HalfKind::None;
    }

    // Launch count and the shared split-K workspace.
    for (std::size_t i = 0; i < out.steps.size(); ++i) {
        const Step& s = out.steps[i];
        out.kernel_launches += static_cast<std::size_t>(s.launches) + out.after_step[i].size();
        if (s.kind == Step::Kind::Matmul && s.splits > 1 && s.launches > 1) {
            out.workspace_bytes = std::max(out.workspace_bytes, static_cast<std::size_t>(s.splits) * s.m * s.n * sizeof(float));
        }
    }

    // Buffer plan over the forms of every computed value.
    out.pool_values.assign(count * kNumReps, PoolValue{});
    for (std::size_t i = 0; i < count; ++i) {
        const Node& n = graph.node(static_cast<NodeId>(i));
        for (int rep = 0; rep < kNumReps; ++rep) {
            PoolValue& v = out.pool_values[i * kNumReps + static_cast<std::size_t>(rep)];
            v.bytes = rep_bytes(n.type, static_cast<Rep>(rep));
            v.live_out = rep == kRepF32 && graph.is_output(static_cast<NodeId>(i));
            v.pooled = is_compute(n.op) && out.needs[i][static_cast<std::size_t>(rep)] && (pool_outputs || !v.live_out);
        }
    }
    auto value_index = [](NodeId node, Rep rep) { return static_cast<std::int32_t>(node) * kNumReps + rep; };
    for (std::size_t i = 0; i < out.steps.size(); ++i) {
        const Step& s = out.steps[i];
        PoolStep ps;
        std::vector<NodeId> defined = s.row_outputs;
        if (defined.empty()) defined.push_back(s.result);
        for (NodeId d : defined) {
            for (int rep = 0; rep < kNumReps; ++rep) {
                if (out.needs[static_cast<std::size_t>(d)][static_cast<std::size_t>(rep)]) {
                    ps.defines.push_back(value_index(d, static_cast<Rep>(rep)));
                }
            }
        }
        if (s.kind != Step::Kind::Matmul) {
            for (NodeId in : s.inputs) ps.reads.push_back(value_index(in, kRepF32));
        } else {
            const bool half = s.arith == Arith::Bf16 || s.arith == Arith::F16;
            ps.reads.push_back(value_index(s.lhs, half ? kRepHalf : kRepF32));
            ps.reads.push_back(value_index(s.rhs, half ? (s.rhs_transposed ? kRepHalfT : kRepHalf)
                                                       : (s.rhs_transposed ? kRepF32T : kRepF32)));
            for (std::size_t k = 0; k < s.inputs.size(); ++k) {
                if (!s.load_is_accumulator[k]) ps.reads.push_back(value_index(s.inputs[k], kRepF32));
            }
        }
        out.pool_steps.push_back(std::move(ps));
    }
    out.pool = plan_pool(out.pool_values, out.pool_steps);

    return out;
}

// ---------------------------------------------------------------- epilogue

std::string generate_epilogue_source(const Graph& graph, const Step& step) {
    std::ostringstream os;
    // No node names in the text: layers that differ only in their operands (the 8 layers of an MLP stack) then
    // generate the same source and share one compiled kernel in the device layer's cache.
    os << "// Generated by minicompiler-b200: matmul epilogue of " << step.program.num_ops() << " elementwise op(s).\n";
    (void)graph;
    os << "#define MC_EPILOGUE_DEFINED 1\n";
    os << "struct McEpilogueArgs {\n    const float* p[6];\n};\n";
    // Program input k -> slot in McEpilogueArgs::p (accumulator loads take none).
    std::vector<int> slot(step.inputs.size(), -1);
    std::vector<std::size_t> input_of_slot;
    for (std::size_t k = 0; k < step.inputs.size(); ++k) {
        if (step.load_is_accumulator[k]) continue;
        slot[k] = static_cast<int>(input_of_slot.size());
        input_of_slot.push_back(k);
    }
    const std::size_t slots = input_of_slot.size();

    // The straight-line program on values: the accumulator and one value per extra operand.
    os << "__device__ __forceinline__ float mc_epi_eval(float acc";
    for (std::size_t s = 0; s < slots; ++s) os << ", float x" << s;
    os << ") {\n    (void)acc;\n";
    for (std::size_t r = 0; r < step.program.instrs.size(); ++r) {
        const FusedInstr& ins = step.program.instrs[r];
        os << "    const float r" << r << " = ";
        switch (ins.kind) {
            case FusedInstr::Kind::Load: {
                const auto k = static_cast<std::size_t>(ins.a);
                if (step.load_is_accumulator[k]) {
                    os << "acc";
                } else {
                    os << "x" << slot[k];
                }
                break;
            }
            case FusedInstr::Kind::Immediate: {
                char note[40];
                std::snprintf(note, sizeof note, "%.9g", static_cast<double>(ins.immediate));
                os << float_bits_literal(ins.immediate) << ";  // " << note << "\n";
                continue;
            }
            case FusedInstr::Kind::Unary: os << op_expression(ins.op, "r" + std::to_string(ins.a), ""); break;
            case FusedInstr::Kind::Binary:
                os << op_expression(ins.op, "r" + std::to_string(ins.a), "r" + std::to_string(ins.b));
                break;
        }
        os << ";\n";
    }
    os << "    return r" << step.program.instrs.size() - 1 << ";\n}\n";

    auto kind_of = [&](std::size_t s) { return step.operands[input_of_slot[s]].kind; };
    auto scalar_address = [&](std::size_t s, const std::string& row, const std::string& col) {
        const std::string p = "e.p[" + std::to_string(s) + "]";
        switch (kind_of(s)) {
            case EpilogueOperand::Kind::Scalar: return p;
            case EpilogueOperand::Kind::Row: return p + " + " + col;
            case EpilogueOperand::Kind::Column: return p + " + " + row;
            case EpilogueOperand::Kind::Full: return p + " + ((unsigned long long)" + row + " * " + std::to_string(step.n) + "ull + " + col + ")";
        }
        return p;
    };

    // One element.
    os << "__device__ __forceinline__ float mc_epilogue(float acc, unsigned row, unsigned col, const McEpilogueArgs& e) {\n";
    os << "    (void)row;\n    (void)col;\n    (void)e;\n";
    os << "    return mc_epi_eval(acc";
    for (std::size_t s = 0; s < slots; ++s) os << ", __ldg(" << scalar_address(s, "row", "col") << ")";
    os << ");\n}\n";

    // 32 consecutive columns of one row, all in range, col0 a multiple of 32: row and full operands come
    // in as 128-bit loads (the operand bases are 256-byte aligned; a full operand needs n % 4 == 0).
    const bool wide_full = step.n % 4 == 0;
    os << "#define MC_EPILOGUE32_DEFINED 1\n";
    os << "__device__ __forceinline__ void mc_epilogue32(float (&f)[32], unsigned row, unsigned col0, const McEpilogueArgs& e) {\n";
    os << "    (void)row;\n    (void)col0;\n    (void)e;\n";
    for (std::size_t s = 0; s < slots; ++s) {
        if (kind_of(s) == EpilogueOperand::Kind::Scalar || kind_of(s) == EpilogueOperand::Kind::Column) {
            os << "    const float s" << s << " = __ldg(" << scalar_address(s, "row", "col0") << ");\n";
        }
    }
    os << "#pragma unroll\n    for (int q = 0; q < 8; ++q) {\n";
    for (std::size_t s = 0; s < slots; ++s) {
        const bool wide = kind_of(s) == EpilogueOperand::Kind::Row || (kind_of(s) == EpilogueOperand::Kind::Full && wide_full);
        if (wide) {
            os << "        const float4 v" << s << " = __ldg(reinterpret_cast<const float4*>(" << scalar_address(s, "row", "col0")
               << ") + q);\n";
        } else if (kind_of(s) == EpilogueOperand::Kind::Full) {
            os << "        const float* u" << s << " = " << scalar_address(s, "row", "col0") << " + 4 * q;\n";
            os << "        const float4 v" << s << " = make_float4(__ldg(u" << s << "), __ldg(u" << s << " + 1), __ldg(u" << s
               << " + 2), __ldg(u" << s << " + 3));\n";
        }
    }
    for (const char* lane : {"x", "y", "z", "w"}) {
        const int j = lane[0] == 'x' ? 0 : lane[0] == 'y' ? 1 : lane[0] == 'z' ? 2 : 3;
        os << "        f[4 * q + " << j << "] = mc_epi_eval(f[4 * q + " << j << "]";
        for (std::size_t s = 0; s < slots; ++s) {
            if (kind_of(s) == EpilogueOperand::Kind::Scalar || kind_of(s) == EpilogueOperand::Kind::Column) {
                os << ", s" << s;
            } else {
                os << ", v" << s << "." << lane;
            }
        }
        os << ");\n";
    }
    os << "    }\n}\n";
    return os.str();
}

std::string describe(const Graph& graph, const LoweredGraph& lowered) {
    std::ostringstream os;
    for (std::size_t i = 0; i < lowered.steps.size(); ++i) {
        const Step& s = lowered.steps[i];
        os << i << ": ";
        if (s.kind == Step::Kind::Elementwise) {
            os << "elementwise " << graph.node(s.result).name << " ops=" << s.program.num_ops();
        } else if (s.kind == Step::Kind::RowFused) {
            os << "row_fused";
            for (const RowPart& part : s.row_parts) os << " " << part.name << (part.output >= 0 ? "*" : "");
            os << " rows of " << s.reduce_shape.back() << " reads=" << s.inputs.size() << " writes=" << s.row_outputs.size();
        } else if (s.kind == Step::Kind::Reduce) {
            os << op_name(s.reduce_op) << " " << graph.node(s.result).name << " rows of " << s.reduce_shape.back()
               << " prologue_ops=" << s.program.num_ops();
        } else {
            os << "matmul " << graph.node(s.matmul).name << " " << s.m << "x" << s.n << "x" << s.k << " kernel="
               << matmul_kernel_name(s.kernel) << " splits=" << s.splits;
            if (s.tile_n != 256) os << " tile_n=" << s.tile_n;
            if (s.rhs_transposed) os << " rhs=transposed";
            if (s.has_epilogue) os << " epilogue=" << graph.node(s.result).name << "(" << s.program.num_ops() << " ops)";
        }
        os << " out=" << (s.write_f32 ? "f32" : "") << (s.write_f32 && s.write_half != HalfKind::None ? "+" : "")
           << (s.write_half == HalfKind::Bf16 ? "bf16" : s.write_half == HalfKind::F16 ? "f16" : "");
        os << " launches=" << s.launches << "\n";
        for (const Recast& rc : lowered.after_step[i]) {
            os << "   recast " << graph.node(rc.node).name << " -> rep " << static_cast<int>(rc.to) << "\n";
        }
    }
    return os.str();
}

}  // namespace minicompiler::cuda
