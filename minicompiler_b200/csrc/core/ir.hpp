#pragma once
// The SSA DAG that the GPU backend consumes. It keeps the reference's IR
// contract (include/minicompiler/{tensor,ops,graph,fused_program}.hpp): nodes
// sit in a vector, operands refer to strictly earlier nodes, so node order is
// both a topological order and the execution order; only f32 tensors exist;
// binary elementwise ops broadcast NumPy-style; matmul is rank-2 x rank-2.

#include "core/status.hpp"

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <optional>
#include <string>
#include <string_view>
#include <vector>

namespace minicompiler {

// ---------------------------------------------------------------- tensors

enum class DType : std::uint8_t { Float32, Float64, Int32, Int64, Bool };

std::size_t dtype_size_bytes(DType dt);
const char* dtype_name(DType dt);

using Shape = std::vector<std::int64_t>;

// Tensors are indexed with 32-bit element indices on the device, so no tensor
// may hold more than 2^31 - 1 elements (reference tensor.hpp:45-47).
inline constexpr std::size_t kMaxElements = (std::size_t{1} << 31) - 1;

// Element count, or nullopt when a dimension is < 1 or the product would pass
// kMaxElements. Untrusted shapes go through this before anything is sized.
std::optional<std::size_t> checked_num_elements(const Shape& shape);
std::size_t num_elements(const Shape& shape);

struct TensorType {
    Shape shape;
    DType dtype = DType::Float32;

    TensorType() = default;
    explicit TensorType(Shape s, DType d = DType::Float32) : shape(std::move(s)), dtype(d) {}

    std::size_t rank() const { return shape.size(); }
    std::size_t num_elements() const { return minicompiler::num_elements(shape); }
    std::size_t size_bytes() const { return num_elements() * dtype_size_bytes(dtype); }
    bool operator==(const TensorType& o) const { return dtype == o.dtype && shape == o.shape; }
    bool operator!=(const TensorType& o) const { return !(*this == o); }
};

std::string to_string(const Shape& shape);      // "[4,8]", scalar "[]"
std::string to_string(const TensorType& type);  // "f32[4,8]"

// -------------------------------------------------------------------- ops

enum class OpKind : std::uint8_t {
    Input,
    Constant,
    Neg,
    Exp,
    Log,
    Sqrt,
    Relu,
    Sigmoid,
    Tanh,
    Add,
    Sub,
    Mul,
    Div,
    MatMul,
    FusedElementwise,
    // Row reductions (an extension; the reference's IR has none, README.md:561-562): the last dimension of the
    // operand collapses to extent 1, every other extent is kept, so the result broadcasts back against the operand.
    // row_sum is defined as the sum accumulated in double and rounded once; row_max as the largest element (the
    // operand is assumed free of NaN).
    RowSum,
    RowMax,
};

const char* op_name(OpKind op);
// Only the twelve mnemonics a graph file may spell after `name =`.
std::optional<OpKind> op_from_name(std::string_view name);
bool is_unary_elementwise(OpKind op);
bool is_binary_elementwise(OpKind op);
inline bool is_elementwise(OpKind op) { return is_unary_elementwise(op) || is_binary_elementwise(op); }
inline bool is_row_reduce(OpKind op) { return op == OpKind::RowSum || op == OpKind::RowMax; }
inline bool is_compute(OpKind op) { return op != OpKind::Input && op != OpKind::Constant; }
int op_arity(OpKind op);  // -1 for FusedElementwise

Result<Shape> broadcast_shapes(const Shape& a, const Shape& b);
// Per output dimension, the element stride to read `in` with (0 where it is broadcast).
std::vector<std::int64_t> broadcast_strides(const Shape& in, const Shape& out);
Result<TensorType> infer_result_type(OpKind op, const std::vector<TensorType>& operands);

// --------------------------------------------------------- fused programs

// One straight-line instruction of a fused elementwise kernel; each defines
// one float "register" and operands name earlier registers.
struct FusedInstr {
    enum class Kind : std::uint8_t { Load, Immediate, Unary, Binary };

    Kind kind = Kind::Load;
    OpKind op = OpKind::Input;
    std::int32_t a = -1;
    std::int32_t b = -1;
    float immediate = 0.0f;

    static FusedInstr load(std::int32_t input) { return {Kind::Load, OpKind::Input, input, -1, 0.0f}; }
    static FusedInstr imm(float v) { return {Kind::Immediate, OpKind::Constant, -1, -1, v}; }
    static FusedInstr unary(OpKind op, std::int32_t x) { return {Kind::Unary, op, x, -1, 0.0f}; }
    static FusedInstr binary(OpKind op, std::int32_t x, std::int32_t y) { return {Kind::Binary, op, x, y, 0.0f}; }
};

struct FusedProgram {
    std::vector<FusedInstr> instrs;         // the last one is the result
    std::vector<std::string> source_nodes;  // names of the graph nodes it replaced
    std::size_t num_ops() const;            // Unary + Binary instructions
};

Status validate(const FusedProgram& program, std::size_t num_inputs);
std::string to_string(const FusedProgram& program);  // "r2 = mul r0, r1" per line
// load operands, apply `op`: how an unfused elementwise node is run.
FusedProgram single_op_program(OpKind op);

// ------------------------------------------------------------------ graph

using NodeId = std::int32_t;
inline constexpr NodeId kNoNode = -1;

struct Node {
    OpKind op = OpKind::Input;
    std::string name;
    std::vector<NodeId> inputs;
    TensorType type;
    std::shared_ptr<const std::vector<float>> constant;  // Constant nodes
    std::shared_ptr<const FusedProgram> fused;           // FusedElementwise nodes
};

class Graph {
public:
    explicit Graph(std::string name = "graph") : name_(std::move(name)) {}

    const std::string& name() const { return name_; }

    Result<NodeId> add_input(std::string name, TensorType type);
    Result<NodeId> add_constant(std::string name, TensorType type, std::vector<float> values);
    Result<NodeId> add_constant(std::string name, TensorType type, std::shared_ptr<const std::vector<float>> values);
    Result<NodeId> add_op(OpKind op, std::vector<NodeId> inputs, std::string name = {});
    Result<NodeId> add_fused(std::vector<NodeId> inputs, std::shared_ptr<const FusedProgram> program, TensorType type,
                             std::string name = {});
    Status add_output(NodeId id);
    // Same kind, name and payload as `proto`, new operands (how passes rebuild graphs).
    Result<NodeId> copy_node(const Node& proto, std::vector<NodeId> inputs);

    std::size_t num_nodes() const { return nodes_.size(); }
    const Node& node(NodeId id) const { return nodes_[static_cast<std::size_t>(id)]; }
    const std::vector<Node>& nodes() const { return nodes_; }
    const std::vector<NodeId>& inputs() const { return inputs_; }
    const std::vector<NodeId>& outputs() const { return outputs_; }
    bool is_output(NodeId id) const;
    std::optional<NodeId> find(std::string_view name) const;
    // users[v]: the nodes reading v, each once, ascending.
    std::vector<std::vector<NodeId>> compute_users() const;
    Status verify() const;

private:
    NodeId push(Node n);
    Status operands_exist(const std::vector<NodeId>& ids) const;

    std::string name_;
    std::vector<Node> nodes_;
    std::vector<NodeId> inputs_;
    std::vector<NodeId> outputs_;
};

struct GraphStats {
    std::size_t nodes = 0;
    std::size_t inputs = 0;
    std::size_t constants = 0;
    std::size_t compute_nodes = 0;
    std::size_t fused_nodes = 0;
    std::size_t elementwise_ops = 0;
    std::size_t matmuls = 0;
    std::size_t reductions = 0;
    std::map<std::string, std::size_t> op_counts;
};

GraphStats compute_stats(const Graph& graph);

}  // namespace minicompiler
