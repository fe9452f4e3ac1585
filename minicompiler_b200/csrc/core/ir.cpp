// IR semantics follow the reference's src/{graph,ops,fused_program}.cpp: the
// same invariants are enforced and the same diagnostics are produced, since
// the reference's tests treat those messages as part of the contract.

#include "core/ir.hpp"

#include <algorithm>
#include <sstream>

namespace minicompiler {

// ---------------------------------------------------------------- tensors

std::size_t dtype_size_bytes(DType dt) {
    switch (dt) {
        case DType::Float32:
        case DType::Int32: return 4;
        case DType::Float64:
        case DType::Int64: return 8;
        case DType::Bool: return 1;
    }
    return 0;
}

const char* dtype_name(DType dt) {
    switch (dt) {
        case DType::Float32: return "f32";
        case DType::Float64: return "f64";
        case DType::Int32: return "i32";
        case DType::Int64: return "i64";
        case DType::Bool: return "bool";
    }
    return "?";
}

std::optional<std::size_t> checked_num_elements(const Shape& shape) {
    std::size_t total = 1;
    for (std::int64_t extent : shape) {
        if (extent < 1) return std::nullopt;
        const auto e = static_cast<std::size_t>(extent);
        if (total > kMaxElements / e) return std::nullopt;
        total *= e;
    }
    return total;
}

std::size_t num_elements(const Shape& shape) {
    std::size_t total = 1;
    for (std::int64_t extent : shape) total *= static_cast<std::size_t>(extent);
    return total;
}

std::string to_string(const Shape& shape) {
    std::string text = "[";
    const char* sep = "";
    for (std::int64_t extent : shape) {
        text += sep;
        text += std::to_string(extent);
        sep = ",";
    }
    return text + "]";
}

std::string to_string(const TensorType& type) { return dtype_name(type.dtype) + to_string(type.shape); }

// -------------------------------------------------------------------- ops

namespace {

struct OpRow {
    OpKind op;
    const char* name;
    int arity;      // -1: varies
    bool writable;  // may appear as `name = op ...` in a graph file
};

constexpr OpRow kOps[] = {
    {OpKind::Input, "input", 0, false},     {OpKind::Constant, "const", 0, false},
    {OpKind::Neg, "neg", 1, true},          {OpKind::Exp, "exp", 1, true},
    {OpKind::Log, "log", 1, true},          {OpKind::Sqrt, "sqrt", 1, true},
    {OpKind::Relu, "relu", 1, true},        {OpKind::Sigmoid, "sigmoid", 1, true},
    {OpKind::Tanh, "tanh", 1, true},        {OpKind::Add, "add", 2, true},
    {OpKind::Sub, "sub", 2, true},          {OpKind::Mul, "mul", 2, true},
    {OpKind::Div, "div", 2, true},          {OpKind::MatMul, "matmul", 2, true},
    {OpKind::FusedElementwise, "fused", -1, false},
    {OpKind::RowSum, "row_sum", 1, true},   {OpKind::RowMax, "row_max", 1, true},
};

const OpRow* row_of(OpKind op) {
    for (const OpRow& r : kOps) {
        if (r.op == op) return &r;
    }
    return nullptr;
}

}  // namespace

const char* op_name(OpKind op) {
    const OpRow* r = row_of(op);
    return r ? r->name : "?";
}

std::optional<OpKind> op_from_name(std::string_view name) {
    for (const OpRow& r : kOps) {
        if (r.writable && name == r.name) return r.op;
    }
    return std::nullopt;
}

bool is_unary_elementwise(OpKind op) { return op >= OpKind::Neg && op <= OpKind::Tanh; }
bool is_binary_elementwise(OpKind op) { return op >= OpKind::Add && op <= OpKind::Div; }

int op_arity(OpKind op) {
    const OpRow* r = row_of(op);
    return r ? r->arity : -1;
}

Result<Shape> broadcast_shapes(const Shape& a, const Shape& b) {
    const std::size_t rank = std::max(a.size(), b.size());
    Shape out(rank, 1);
    for (std::size_t back = 1; back <= rank; ++back) {  // walk from the last dimension
        const std::int64_t ea = back <= a.size() ? a[a.size() - back] : 1;
        const std::int64_t eb = back <= b.size() ? b[b.size() - back] : 1;
        if (ea != eb && ea != 1 && eb != 1) {
            return Error{"cannot broadcast " + to_string(a) + " with " + to_string(b)};
        }
        out[rank - back] = ea == 1 ? eb : ea;
    }
    return out;
}

std::vector<std::int64_t> broadcast_strides(const Shape& in, const Shape& out) {
    std::vector<std::int64_t> strides(out.size(), 0);
    std::int64_t running = 1;
    for (std::size_t back = 1; back <= in.size(); ++back) {
        const std::int64_t extent = in[in.size() - back];
        if (extent != 1) strides[out.size() - back] = running;
        running *= extent;
    }
    return strides;
}

Result<TensorType> infer_result_type(OpKind op, const std::vector<TensorType>& operands) {
    const int arity = op_arity(op);
    if (arity <= 0) return Error{std::string("'") + op_name(op) + "' has no inferred result type"};
    if (operands.size() != static_cast<std::size_t>(arity)) {
        return Error{std::string(op_name(op)) + " expects " + std::to_string(arity) + " operand(s), got " +
                     std::to_string(operands.size())};
    }
    for (const TensorType& t : operands) {
        if (t.dtype != DType::Float32) {
            return Error{std::string(op_name(op)) + ": only f32 is supported, got " + to_string(t)};
        }
    }
    if (is_unary_elementwise(op)) return operands[0];
    if (is_row_reduce(op)) {
        Shape shape = operands[0].shape;
        if (shape.empty()) return Error{std::string(op_name(op)) + " expects an operand of rank 1 or more, got " + to_string(shape)};
        shape.back() = 1;
        return TensorType(std::move(shape));
    }
    if (is_binary_elementwise(op)) {
        Result<Shape> shape = broadcast_shapes(operands[0].shape, operands[1].shape);
        if (!shape.ok()) return Error{std::string(op_name(op)) + ": " + shape.error().message};
        return TensorType(std::move(shape).value());
    }
    const Shape& lhs = operands[0].shape;
    const Shape& rhs = operands[1].shape;
    if (lhs.size() != 2 || rhs.size() != 2) {
        return Error{"matmul expects rank-2 operands, got " + to_string(lhs) + " and " + to_string(rhs)};
    }
    if (lhs[1] != rhs[0]) {
        return Error{"matmul inner dimensions differ: " + to_string(lhs) + " x " + to_string(rhs)};
    }
    return TensorType(Shape{lhs[0], rhs[1]});
}

// --------------------------------------------------------- fused programs

std::size_t FusedProgram::num_ops() const {
    return static_cast<std::size_t>(std::count_if(instrs.begin(), instrs.end(), [](const FusedInstr& i) {
        return i.kind == FusedInstr::Kind::Unary || i.kind == FusedInstr::Kind::Binary;
    }));
}

Status validate(const FusedProgram& program, std::size_t num_inputs) {
    if (program.instrs.empty()) return Error{"fused program is empty"};
    for (std::size_t r = 0; r < program.instrs.size(); ++r) {
        const FusedInstr& ins = program.instrs[r];
        const std::string where = "fused instruction r" + std::to_string(r) + ": ";
        const auto defined = [r](std::int32_t reg) { return reg >= 0 && static_cast<std::size_t>(reg) < r; };
        if (ins.kind == FusedInstr::Kind::Load) {
            if (ins.a < 0 || static_cast<std::size_t>(ins.a) >= num_inputs) {
                return Error{where + "loads input " + std::to_string(ins.a) + " of " + std::to_string(num_inputs)};
            }
        } else if (ins.kind == FusedInstr::Kind::Unary) {
            if (!is_unary_elementwise(ins.op)) {
                return Error{where + op_name(ins.op) + " is not a unary elementwise op"};
            }
            if (!defined(ins.a)) return Error{where + "operand must be an earlier instruction"};
        } else if (ins.kind == FusedInstr::Kind::Binary) {
            if (!is_binary_elementwise(ins.op)) {
                return Error{where + op_name(ins.op) + " is not a binary elementwise op"};
            }
            if (!defined(ins.a) || !defined(ins.b)) return Error{where + "operands must be earlier instructions"};
        }
    }
    return Status();
}

std::string to_string(const FusedProgram& program) {
    std::ostringstream os;
    for (std::size_t r = 0; r < program.instrs.size(); ++r) {
        const FusedInstr& ins = program.instrs[r];
        os << "r" << r << " = ";
        switch (ins.kind) {
            case FusedInstr::Kind::Load: os << "load in" << ins.a; break;
            case FusedInstr::Kind::Immediate: os << "imm " << ins.immediate; break;
            case FusedInstr::Kind::Unary: os << op_name(ins.op) << " r" << ins.a; break;
            case FusedInstr::Kind::Binary: os << op_name(ins.op) << " r" << ins.a << ", r" << ins.b; break;
        }
        os << "\n";
    }
    return os.str();
}

FusedProgram single_op_program(OpKind op) {
    FusedProgram p;
    p.instrs.push_back(FusedInstr::load(0));
    if (is_unary_elementwise(op)) {
        p.instrs.push_back(FusedInstr::unary(op, 0));
    } else {
        p.instrs.push_back(FusedInstr::load(1));
        p.instrs.push_back(FusedInstr::binary(op, 0, 1));
    }
    p.source_nodes.push_back(op_name(op));
    return p;
}

// ------------------------------------------------------------------ graph

namespace {

Status type_is_usable(const TensorType& type, const std::string& what) {
    if (type.dtype != DType::Float32) return Error{what + ": only f32 is supported, got " + to_string(type)};
    for (std::int64_t extent : type.shape) {
        if (extent < 1) return Error{what + ": dimensions must be >= 1, got " + to_string(type)};
    }
    if (!checked_num_elements(type.shape)) {
        return Error{what + ": " + to_string(type) + " has more than 2^31 - 1 elements"};
    }
    return Status();
}

Status fused_is_usable(const FusedProgram& program, const std::vector<TensorType>& operands, const TensorType& type,
                       const std::string& what) {
    Status st = validate(program, operands.size());
    if (!st.ok()) return Error{what + ": " + st.message()};
    for (const TensorType& t : operands) {
        Result<Shape> joined = broadcast_shapes(t.shape, type.shape);
        if (!joined.ok() || joined.value() != type.shape) {
            return Error{what + ": input " + to_string(t) + " does not broadcast to " + to_string(type)};
        }
    }
    return Status();
}

}  // namespace

NodeId Graph::push(Node n) {
    const auto id = static_cast<NodeId>(nodes_.size());
    if (n.name.empty()) n.name = std::string(op_name(n.op)) + "_" + std::to_string(id);
    nodes_.push_back(std::move(n));
    return id;
}

Status Graph::operands_exist(const std::vector<NodeId>& ids) const {
    for (NodeId id : ids) {
        if (id < 0 || static_cast<std::size_t>(id) >= nodes_.size()) {
            return Error{"operand %" + std::to_string(id) + " does not exist"};
        }
    }
    return Status();
}

Result<NodeId> Graph::add_input(std::string name, TensorType type) {
    MC_TRY(type_is_usable(type, "input '" + name + "'"));
    Node n;
    n.op = OpKind::Input;
    n.name = std::move(name);
    n.type = std::move(type);
    const NodeId id = push(std::move(n));
    inputs_.push_back(id);
    return id;
}

Result<NodeId> Graph::add_constant(std::string name, TensorType type, std::vector<float> values) {
    return add_constant(std::move(name), std::move(type),
                        std::make_shared<const std::vector<float>>(std::move(values)));
}

Result<NodeId> Graph::add_constant(std::string name, TensorType type,
                                   std::shared_ptr<const std::vector<float>> values) {
    const std::string what = "constant '" + name + "'";
    MC_TRY(type_is_usable(type, what));
    const std::size_t have = values ? values->size() : 0;
    if (!values || have != type.num_elements()) {
        return Error{what + ": expected " + std::to_string(type.num_elements()) + " values for " + to_string(type) +
                     ", got " + std::to_string(have)};
    }
    Node n;
    n.op = OpKind::Constant;
    n.name = std::move(name);
    n.type = std::move(type);
    n.constant = std::move(values);
    return push(std::move(n));
}

Result<NodeId> Graph::add_op(OpKind op, std::vector<NodeId> inputs, std::string name) {
    if (!is_elementwise(op) && op != OpKind::MatMul && !is_row_reduce(op)) {
        return Error{std::string("add_op cannot create '") + op_name(op) + "' nodes"};
    }
    MC_TRY(operands_exist(inputs));
    std::vector<TensorType> operand_types;
    for (NodeId in : inputs) operand_types.push_back(node(in).type);
    const std::string label = name.empty() ? std::string(op_name(op)) : name;
    Result<TensorType> type = infer_result_type(op, operand_types);
    if (!type.ok()) return Error{label + ": " + type.error().message};
    MC_TRY(type_is_usable(type.value(), label));  // a broadcast or matmul result can outgrow its operands
    Node n;
    n.op = op;
    n.name = std::move(name);
    n.inputs = std::move(inputs);
    n.type = std::move(type).value();
    return push(std::move(n));
}

Result<NodeId> Graph::add_fused(std::vector<NodeId> inputs, std::shared_ptr<const FusedProgram> program,
                                TensorType type, std::string name) {
    const std::string what = "fused node '" + name + "'";
    if (!program) return Error{what + ": missing program"};
    MC_TRY(operands_exist(inputs));
    MC_TRY(type_is_usable(type, what));
    std::vector<TensorType> operand_types;
    for (NodeId in : inputs) operand_types.push_back(node(in).type);
    MC_TRY(fused_is_usable(*program, operand_types, type, what));
    Node n;
    n.op = OpKind::FusedElementwise;
    n.name = std::move(name);
    n.inputs = std::move(inputs);
    n.type = std::move(type);
    n.fused = std::move(program);
    return push(std::move(n));
}

Status Graph::add_output(NodeId id) {
    MC_TRY(operands_exist({id}));
    if (is_output(id)) return Error{"'" + node(id).name + "' is already an output"};
    outputs_.push_back(id);
    return Status();
}

Result<NodeId> Graph::copy_node(const Node& proto, std::vector<NodeId> inputs) {
    if (proto.op == OpKind::Input) return add_input(proto.name, proto.type);
    if (proto.op == OpKind::Constant) return add_constant(proto.name, proto.type, proto.constant);
    if (proto.op == OpKind::FusedElementwise) return add_fused(std::move(inputs), proto.fused, proto.type, proto.name);
    return add_op(proto.op, std::move(inputs), proto.name);
}

bool Graph::is_output(NodeId id) const { return std::find(outputs_.begin(), outputs_.end(), id) != outputs_.end(); }

std::optional<NodeId> Graph::find(std::string_view name) const {
    for (std::size_t i = 0; i < nodes_.size(); ++i) {
        if (nodes_[i].name == name) return static_cast<NodeId>(i);
    }
    return std::nullopt;
}

std::vector<std::vector<NodeId>> Graph::compute_users() const {
    std::vector<std::vector<NodeId>> users(nodes_.size());
    for (std::size_t i = 0; i < nodes_.size(); ++i) {
        const auto user = static_cast<NodeId>(i);
        for (NodeId in : nodes_[i].inputs) {
            auto& list = users[static_cast<std::size_t>(in)];
            if (list.empty() || list.back() != user) list.push_back(user);  // x*x is one user of x
        }
    }
    return users;
}

Status Graph::verify() const {
    std::size_t seen_inputs = 0;
    for (std::size_t i = 0; i < nodes_.size(); ++i) {
        const Node& n = nodes_[i];
        const std::string what = "node %" + std::to_string(i) + " '" + n.name + "'";
        for (NodeId in : n.inputs) {
            if (in < 0 || static_cast<std::size_t>(in) >= i) {
                return Error{what + ": operand %" + std::to_string(in) + " does not precede it"};
            }
        }
        const int arity = op_arity(n.op);
        if (arity >= 0 && n.inputs.size() != static_cast<std::size_t>(arity)) {
            return Error{what + ": " + op_name(n.op) + " has " + std::to_string(n.inputs.size()) + " operands"};
        }
        std::vector<TensorType> operand_types;
        for (NodeId in : n.inputs) operand_types.push_back(node(in).type);

        if (n.op == OpKind::Input) {
            ++seen_inputs;
            if (std::find(inputs_.begin(), inputs_.end(), static_cast<NodeId>(i)) == inputs_.end()) {
                return Error{what + ": input node missing from the input list"};
            }
            MC_TRY(type_is_usable(n.type, what));
        } else if (n.op == OpKind::Constant) {
            MC_TRY(type_is_usable(n.type, what));
            if (!n.constant || n.constant->size() != n.type.num_elements()) {
                return Error{what + ": constant payload does not match " + to_string(n.type)};
            }
        } else if (n.op == OpKind::FusedElementwise) {
            if (!n.fused) return Error{what + ": missing fused program"};
            MC_TRY(fused_is_usable(*n.fused, operand_types, n.type, what));
        } else {
            MC_TRY(type_is_usable(n.type, what));
            Result<TensorType> expect = infer_result_type(n.op, operand_types);
            if (!expect.ok()) return Error{what + ": " + expect.error().message};
            if (expect.value() != n.type) {
                return Error{what + ": type " + to_string(n.type) + " should be " + to_string(expect.value())};
            }
        }
    }
    if (seen_inputs != inputs_.size()) return Error{"input list does not match the input nodes"};
    for (NodeId in : inputs_) {
        if (in < 0 || static_cast<std::size_t>(in) >= nodes_.size() || node(in).op != OpKind::Input) {
            return Error{"input list refers to a non-input node"};
        }
    }
    if (outputs_.empty()) return Error{"graph has no outputs"};
    for (std::size_t k = 0; k < outputs_.size(); ++k) {
        const NodeId out = outputs_[k];
        if (out < 0 || static_cast<std::size_t>(out) >= nodes_.size()) return Error{"output refers to a missing node"};
        if (std::find(outputs_.begin(), outputs_.begin() + static_cast<std::ptrdiff_t>(k), out) !=
            outputs_.begin() + static_cast<std::ptrdiff_t>(k)) {
            return Error{"'" + node(out).name + "' is listed as an output twice"};
        }
    }
    return Status();
}

GraphStats compute_stats(const Graph& graph) {
    GraphStats s;
    s.nodes = graph.num_nodes();
    for (const Node& n : graph.nodes()) {
        if (n.op == OpKind::Input) {
            ++s.inputs;
        } else if (n.op == OpKind::Constant) {
            ++s.constants;
        } else {
            ++s.compute_nodes;
            ++s.op_counts[op_name(n.op)];
            if (n.op == OpKind::FusedElementwise) {
                ++s.fused_nodes;
                s.elementwise_ops += n.fused->num_ops();
            } else if (n.op == OpKind::MatMul) {
                ++s.matmuls;
            } else if (is_row_reduce(n.op)) {
                ++s.reductions;
            } else {
                ++s.elementwise_ops;
            }
        }
    }
    return s;
}

}  // namespace minicompiler
