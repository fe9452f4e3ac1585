// .mcg reader/printer and the seeded uniform generator. Behaviour (grammar,
// override rules, message texts) follows the reference's src/parser.cpp and
// src/random.cpp; the reference's tests/test_parser.cpp pins the messages.

#include "core/mcg.hpp"

#include <cctype>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>
#include <unordered_map>

namespace minicompiler {

// -------------------------------------------------------------- generator

namespace {

inline std::uint64_t next_splitmix64(std::uint64_t& s) {
    s += 0x9E3779B97F4A7C15ULL;
    std::uint64_t z = s;
    z ^= z >> 30;
    z *= 0xBF58476D1CE4E5B9ULL;
    z ^= z >> 27;
    z *= 0x94D049BB133111EBULL;
    z ^= z >> 31;
    return z;
}

}  // namespace

void fill_uniform(float* out, std::size_t count, std::uint64_t seed, float lo, float hi) {
    std::uint64_t state = seed;
    const float span = hi - lo;
    for (std::size_t i = 0; i < count; ++i) {
        // Top 24 bits as an exact float in [0, 1).
        const float u = static_cast<float>(next_splitmix64(state) >> 40) * (1.0f / 16777216.0f);
        // The product is rounded to float before the add; a fused multiply-add
        // would change the last bit against the published golden values.
        volatile float scaled = span * u;
        out[i] = lo + scaled;
    }
}

std::vector<float> uniform_values(std::size_t count, std::uint64_t seed, float lo, float hi) {
    std::vector<float> v(count);
    fill_uniform(v.data(), count, seed, lo, hi);
    return v;
}

std::vector<HostTensor> make_random_inputs(const Graph& graph, std::uint64_t seed, float lo, float hi) {
    std::vector<HostTensor> tensors;
    std::uint64_t k = 0;
    for (NodeId id : graph.inputs()) {
        const TensorType& type = graph.node(id).type;
        tensors.emplace_back(type, uniform_values(type.num_elements(), seed + k, lo, hi));
        ++k;
    }
    return tensors;
}

// ----------------------------------------------------------------- reader

namespace {

enum class Tok { Word, Number, Symbol };

struct Lexeme {
    Tok kind;
    std::string text;
};

bool word_start(char c) { return std::isalpha(static_cast<unsigned char>(c)) || c == '_'; }
bool word_part(char c) { return std::isalnum(static_cast<unsigned char>(c)) || c == '_'; }
bool digit(char c) { return std::isdigit(static_cast<unsigned char>(c)) != 0; }

// One line -> lexemes. '#' opens a comment.
Result<std::vector<Lexeme>> scan_line(std::string_view line) {
    std::vector<Lexeme> out;
    std::size_t at = 0;
    const std::size_t end = line.size();
    while (at < end) {
        const char c = line[at];
        if (std::isspace(static_cast<unsigned char>(c))) {
            ++at;
        } else if (c == '#') {
            break;
        } else if (word_start(c)) {
            std::size_t stop = at + 1;
            while (stop < end && word_part(line[stop])) ++stop;
            out.push_back({Tok::Word, std::string(line.substr(at, stop - at))});
            at = stop;
        } else if (digit(c) || c == '.' ||
                   ((c == '+' || c == '-') && at + 1 < end && (digit(line[at + 1]) || line[at + 1] == '.'))) {
            std::size_t stop = at + 1;
            for (;;) {
                if (stop < end && (digit(line[stop]) || line[stop] == '.')) {
                    ++stop;
                } else if (stop < end && (line[stop] == 'e' || line[stop] == 'E')) {
                    ++stop;
                    if (stop < end && (line[stop] == '+' || line[stop] == '-')) ++stop;
                } else {
                    break;
                }
            }
            out.push_back({Tok::Number, std::string(line.substr(at, stop - at))});
            at = stop;
        } else if (std::strchr(":=,[]()", c) != nullptr) {
            out.push_back({Tok::Symbol, std::string(1, c)});
            ++at;
        } else {
            return Error{std::string("unexpected character '") + c + "'"};
        }
    }
    return out;
}

// Reads one statement's lexemes left to right.
class Reader {
public:
    explicit Reader(std::vector<Lexeme> lexemes) : lex_(std::move(lexemes)) {}

    bool done() const { return at_ >= lex_.size(); }
    const Lexeme& head() const { return lex_[at_]; }
    bool head_is(Tok kind) const { return !done() && head().kind == kind; }

    bool take_symbol(char c) {
        if (!head_is(Tok::Symbol) || head().text[0] != c) return false;
        ++at_;
        return true;
    }
    Status need_symbol(char c) {
        if (take_symbol(c)) return Status();
        return Error{std::string("expected '") + c + "' " + seen()};
    }
    Result<std::string> word(const char* what) {
        if (!head_is(Tok::Word)) return Error{std::string("expected ") + what + " " + seen()};
        return lex_[at_++].text;
    }
    Result<double> real(const char* what) {
        if (!head_is(Tok::Number)) return Error{std::string("expected ") + what + " " + seen()};
        const std::string& text = lex_[at_++].text;
        char* stop = nullptr;
        errno = 0;
        const double v = std::strtod(text.c_str(), &stop);
        if (stop != text.c_str() + text.size() || errno == ERANGE) return Error{"bad number '" + text + "'"};
        return v;
    }
    Result<std::int64_t> whole(const char* what) {
        if (!head_is(Tok::Number)) return Error{std::string("expected ") + what + " " + seen()};
        const std::string& text = lex_[at_++].text;
        char* stop = nullptr;
        errno = 0;
        const long long v = std::strtoll(text.c_str(), &stop, 10);
        if (stop != text.c_str() + text.size() || errno == ERANGE) {
            return Error{"expected an integer, got '" + text + "'"};
        }
        return static_cast<std::int64_t>(v);
    }
    std::string seen() const { return done() ? "at end of line" : "but found '" + head().text + "'"; }

private:
    std::vector<Lexeme> lex_;
    std::size_t at_ = 0;
};

class McgReader {
public:
    explicit McgReader(const ParseOptions& options) : options_(options) {}

    Result<Graph> read(std::string_view text) {
        std::size_t line_no = 0;
        std::size_t from = 0;
        for (;;) {
            std::size_t to = text.find('\n', from);
            const bool last = to == std::string_view::npos;
            if (last) to = text.size();
            std::string_view line = text.substr(from, to - from);
            if (!line.empty() && line.back() == '\r') line.remove_suffix(1);
            ++line_no;

            Result<std::vector<Lexeme>> lexemes = scan_line(line);
            Status st = lexemes.status();
            if (st.ok() && !lexemes->empty()) {
                Reader r(std::move(lexemes).value());
                st = statement(r);
            }
            if (!st.ok()) return Error{"line " + std::to_string(line_no) + ": " + st.message()};
            if (last || to == text.size()) break;
            from = to + 1;
        }
        for (const auto& kv : options_.dims) {
            if (dims_.find(kv.first) == dims_.end()) return Error{"the graph declares no dim '" + kv.first + "'"};
        }
        if (graph_.outputs().empty()) return Error{"the graph declares no outputs"};
        MC_TRY(graph_.verify());
        if (options_.resolved_dims != nullptr) *options_.resolved_dims = dims_;
        return std::move(graph_);
    }

private:
    Status statement(Reader& r) {
        MC_ASSIGN(keyword, r.word("a statement"));
        Status st;
        if (keyword == "graph") {
            st = graph_stmt(r);
        } else if (keyword == "dim") {
            st = dim_stmt(r);
        } else if (keyword == "input") {
            st = input_stmt(r);
        } else if (keyword == "const") {
            st = const_stmt(r);
        } else if (keyword == "output") {
            st = output_stmt(r);
        } else {
            st = op_stmt(r, keyword);
        }
        MC_TRY(st);
        if (!r.done()) return Error{"unexpected '" + r.head().text + "'"};
        return Status();
    }

    Status graph_stmt(Reader& r) {
        MC_ASSIGN(name, r.word("a graph name"));
        if (graph_.num_nodes() > 0) return Error{"'graph' must come before any node"};
        graph_ = Graph(name);
        return Status();
    }

    Status dim_stmt(Reader& r) {
        MC_ASSIGN(name, r.word("a dim name"));
        MC_TRY(r.need_symbol('='));
        MC_ASSIGN(written, r.whole("a dim value"));
        if (dims_.count(name) != 0) return Error{"dim '" + name + "' is declared twice"};
        const auto forced = options_.dims.find(name);
        const std::int64_t extent = forced == options_.dims.end() ? written : forced->second;
        if (extent < 1) return Error{"dim '" + name + "' must be >= 1, got " + std::to_string(extent)};
        dims_[name] = extent;
        return Status();
    }

    Status input_stmt(Reader& r) {
        MC_ASSIGN(name, r.word("an input name"));
        MC_TRY(r.need_symbol(':'));
        MC_ASSIGN(type, tensor_type(r));
        return bind(name, graph_.add_input(name, std::move(type)));
    }

    Status const_stmt(Reader& r) {
        MC_ASSIGN(name, r.word("a constant name"));
        MC_TRY(r.need_symbol(':'));
        MC_ASSIGN(type, tensor_type(r));
        MC_TRY(r.need_symbol('='));
        MC_ASSIGN(values, initializer(r, type));
        return bind(name, graph_.add_constant(name, std::move(type), std::move(values)));
    }

    Status output_stmt(Reader& r) {
        do {
            MC_ASSIGN(name, r.word("an output name"));
            MC_ASSIGN(id, resolve(name));
            MC_TRY(graph_.add_output(id));
        } while (r.take_symbol(','));
        return Status();
    }

    Status op_stmt(Reader& r, const std::string& name) {
        if (!r.take_symbol('=')) return Error{"unknown statement '" + name + "'"};
        MC_ASSIGN(mnemonic, r.word("an op name"));
        const std::optional<OpKind> op = op_from_name(mnemonic);
        if (!op) return Error{"unknown op '" + mnemonic + "'"};
        std::vector<NodeId> operands;
        do {
            MC_ASSIGN(operand, r.word("an operand"));
            MC_ASSIGN(id, resolve(operand));
            operands.push_back(id);
        } while (r.take_symbol(','));
        return bind(name, graph_.add_op(*op, std::move(operands), name));
    }

    Result<TensorType> tensor_type(Reader& r) {
        MC_ASSIGN(elem, r.word("an element type"));
        if (elem != "f32") return Error{"unsupported element type '" + elem + "' (only f32)"};
        MC_TRY(r.need_symbol('['));
        Shape shape;
        if (r.take_symbol(']')) return TensorType(shape);
        do {
            if (r.head_is(Tok::Word)) {
                const std::string dim = r.word("a dim").value();
                const auto known = dims_.find(dim);
                if (known == dims_.end()) return Error{"unknown dim '" + dim + "'"};
                shape.push_back(known->second);
            } else {
                MC_ASSIGN(extent, r.whole("a dimension"));
                shape.push_back(extent);
            }
        } while (r.take_symbol(','));
        MC_TRY(r.need_symbol(']'));
        // Rejected here, before an initializer could try to allocate the values.
        if (!checked_num_elements(shape)) {
            return Error{"invalid shape " + to_string(shape) +
                         ": dimensions must be >= 1 and the total at most 2^31 - 1 elements"};
        }
        return TensorType(shape);
    }

    Result<std::vector<float>> initializer(Reader& r, const TensorType& type) {
        const std::size_t count = type.num_elements();
        if (r.head_is(Tok::Number)) {
            MC_ASSIGN(v, r.real("a value"));
            return std::vector<float>(count, static_cast<float>(v));
        }
        if (r.take_symbol('[')) {
            std::vector<float> values;
            do {
                MC_ASSIGN(v, r.real("a value"));
                values.push_back(static_cast<float>(v));
            } while (r.take_symbol(','));
            MC_TRY(r.need_symbol(']'));
            if (values.size() != count) {
                return Error{"expected " + std::to_string(count) + " values for " + to_string(type) + ", got " +
                             std::to_string(values.size())};
            }
            return values;
        }
        MC_ASSIGN(fn, r.word("a value, [values] or uniform(...)"));
        if (fn != "uniform") return Error{"unknown initializer '" + fn + "'"};
        MC_TRY(r.need_symbol('('));
        std::optional<std::uint64_t> seed;  // stays an integer: a double would drop bits above 2^53
        std::map<std::string, double> bounds;
        do {
            MC_ASSIGN(key, r.word("seed, lo or hi"));
            if (key != "seed" && key != "lo" && key != "hi") {
                return Error{"uniform() takes seed, lo and hi, not '" + key + "'"};
            }
            MC_TRY(r.need_symbol('='));
            if (key == "seed") {
                MC_ASSIGN(s, r.whole("a seed"));
                if (s < 0) return Error{"seed must be >= 0"};
                seed = static_cast<std::uint64_t>(s);
            } else {
                MC_ASSIGN(v, r.real("a bound"));
                bounds[key] = v;
            }
        } while (r.take_symbol(','));
        MC_TRY(r.need_symbol(')'));
        if (!seed || bounds.size() != 2) return Error{"uniform() needs seed, lo and hi"};
        const auto lo = static_cast<float>(bounds["lo"]);
        const auto hi = static_cast<float>(bounds["hi"]);
        if (!(lo < hi)) return Error{"uniform() needs lo < hi"};
        return uniform_values(count, *seed, lo, hi);
    }

    Result<NodeId> resolve(const std::string& name) const {
        const auto hit = names_.find(name);
        if (hit == names_.end()) return Error{"unknown value '" + name + "'"};
        return hit->second;
    }

    Status bind(const std::string& name, Result<NodeId> id) {
        if (!id.ok()) return id.error();
        if (!names_.emplace(name, id.value()).second) return Error{"'" + name + "' is defined twice"};
        return Status();
    }

    const ParseOptions& options_;
    Graph graph_;
    std::map<std::string, std::int64_t> dims_;
    std::unordered_map<std::string, NodeId> names_;
};

}  // namespace

Result<Graph> parse_graph(std::string_view text, const ParseOptions& options) { return McgReader(options).read(text); }

Result<Graph> parse_graph_file(const std::string& path, const ParseOptions& options) {
    std::ifstream file(path, std::ios::binary);
    if (!file) return Error{"cannot open '" + path + "'"};
    std::ostringstream text;
    text << file.rdbuf();
    Result<Graph> g = parse_graph(text.str(), options);
    if (!g.ok()) return Error{path + ": " + g.error().message};
    return g;
}

// ---------------------------------------------------------------- printer

std::string describe_constant(const Node& constant) {
    const std::vector<float>& v = *constant.constant;
    std::ostringstream os;
    if (v.size() == 1) {
        os << v[0];
    } else if (v.size() <= 4) {
        os << "[";
        for (std::size_t i = 0; i < v.size(); ++i) os << (i == 0 ? "" : ", ") << v[i];
        os << "]";
    } else {
        os << "<" << v.size() << " values>";
    }
    return os.str();
}

std::string print_graph(const Graph& graph) {
    std::ostringstream os;
    os << "graph " << graph.name() << "\n";
    for (std::size_t i = 0; i < graph.num_nodes(); ++i) {
        const auto id = static_cast<NodeId>(i);
        const Node& n = graph.node(id);
        os << "  %" << id << " " << n.name << " = ";
        if (n.op == OpKind::Constant) {
            os << "const " << describe_constant(n);
        } else {
            os << op_name(n.op);
            const char* sep = " %";
            for (NodeId in : n.inputs) {
                os << sep << in;
                sep = ", %";
            }
        }
        os << " : " << to_string(n.type);
        if (graph.is_output(id)) os << "  (output)";
        os << "\n";
        if (n.op == OpKind::FusedElementwise) {
            std::istringstream body(to_string(*n.fused));
            for (std::string line; std::getline(body, line);) os << "        " << line << "\n";
        }
    }
    return os.str();
}

}  // namespace minicompiler
