#include "backend/b200_backend.hpp"

#include "backend/row_slicing.hpp"

#include "minicompiler_b200_device.h"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>

namespace minicompiler {

std::vector<std::string> available_backends() { return {"cuda"}; }

Result<std::unique_ptr<Backend>> create_backend(std::string_view name) {
    if (name == "cuda") return cuda::make_cuda_backend();
    if (name == "cpu") {
        return Error{"this library replaces the CUDA backend only and has no CPU execution path (available: cuda)"};
    }
    return Error{"unknown backend '" + std::string(name) + "' (available: cuda)"};
}

namespace cuda {

namespace {

Status device_error(const char* what) { return Error{std::string(what) + ": " + mcd_last_error()}; }

#define MCD_TRY(call)                                  \
    do {                                               \
        if ((call) != 0) return device_error(#call);   \
    } while (0)

constexpr std::size_t kAlign = 256;
std::size_t align_up(std::size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct Launch {
    enum class Kind { Elementwise, Matmul, Recast } kind = Kind::Elementwise;
    // Elementwise: an NVRTC-compiled kernel; params = [out] [out16] in... n
    void* function = nullptr;
    unsigned grid = 0;
    unsigned block = kElementwiseBlock;
    unsigned count = 0;
    std::vector<void*> pointers;
    std::vector<char> advances;  // per pointer: 1 when it walks the tensor element by element (output, same-size inputs)
    bool vectorized = false;
    std::vector<void*> params;
    // Matmul
    mcd_gemm_args gemm{};
    MatmulKernel reported = MatmulKernel::DoubleBuffered;
    // Recast: FP32 form -> another form
    const float* src = nullptr;
    void* dst = nullptr;
    long long rows = 0, cols = 0, src_pitch = 0, dst_pitch = 0;
    int transpose = 0;
    int half_kind = 0;  // 0: FP32 transpose
    // Row slicing: bytes by which each pointer moves per row of the cut dimension (0: the tensor is not cut).
    // Elementwise kinds: one entry per `pointers` slot. Matmul: a, c, c16, then the epilogue inputs. Recast: src, dst.
    std::vector<std::size_t> row_bytes;
};

using LaunchList = std::vector<std::unique_ptr<Launch>>;

class B200Executable final : public CudaExecutable {
public:
    static Result<std::unique_ptr<B200Executable>> create(const Graph& graph, const CudaOptions& options) {
        std::unique_ptr<B200Executable> exe(new B200Executable(graph, options));
        Status st = exe->init();
        if (!st.ok()) return st.error();
        return exe;
    }

    ~B200Executable() override {
        if (arena_ != nullptr || stream_ != nullptr) mcd_set_device(options_.device);
        if (replay_ != nullptr) mcd_graph_destroy(replay_);
        for (void* f : jit_functions_) mcd_jit_release(f);
        for (void* e : slice_in_) mcd_event_destroy(e);
        for (void* e : slice_done_) mcd_event_destroy(e);
        if (copy_in_ != nullptr) mcd_stream_destroy(copy_in_);
        if (copy_out_ != nullptr) mcd_stream_destroy(copy_out_);
        if (stream_ != nullptr) mcd_stream_destroy(stream_);
        if (arena_ != nullptr) mcd_free(arena_);
    }

    Status run(const std::vector<HostTensor>& inputs, std::vector<HostTensor>& outputs) override {
        if (static_cast<const void*>(&inputs) == static_cast<const void*>(&outputs)) {
            return Error{"run() needs separate input and output vectors"};
        }
        if (inputs.size() != graph_.inputs().size()) {
            return Error{"expected " + std::to_string(graph_.inputs().size()) + " inputs, got " +
                         std::to_string(inputs.size())};
        }
        std::vector<const float*> in;
        for (std::size_t k = 0; k < inputs.size(); ++k) {
            const Node& node = graph_.node(graph_.inputs()[k]);
            if (inputs[k].type != node.type || inputs[k].data.size() != node.type.num_elements()) {
                return Error{"input '" + node.name + "' should be " + to_string(node.type) + ", got " +
                             to_string(inputs[k].type)};
            }
            in.push_back(inputs[k].data.data());
        }
        outputs.resize(graph_.outputs().size());
        std::vector<float*> out;
        for (std::size_t k = 0; k < outputs.size(); ++k) {
            const TensorType& type = graph_.node(graph_.outputs()[k]).type;
            outputs[k].type = type;
            outputs[k].data.resize(type.num_elements());
            out.push_back(outputs[k].data.data());
        }
        return run_buffers(in, out);
    }

    Status run_buffers(const std::vector<const float*>& inputs, const std::vector<float*>& outputs) override {
        if (inputs.size() != graph_.inputs().size() || outputs.size() != graph_.outputs().size()) {
            return Error{"expected " + std::to_string(graph_.inputs().size()) + " input and " +
                         std::to_string(graph_.outputs().size()) + " output buffers"};
        }
        bool done = false;
        MC_TRY(run_in_row_slices(inputs, outputs, &done));
        if (done) return Status();
        MC_TRY(run_on_host_memory(inputs, outputs, &done));
        if (done) return Status();
        MC_TRY(upload_inputs(inputs));
        MC_TRY(enqueue(nullptr));
        return download_outputs(outputs);
    }

    std::size_t intermediate_bytes() const override { return lowered_.pool.bytes_with_reuse() + unpooled_output_bytes_; }

    Status upload_inputs(const std::vector<const float*>& host_inputs) override {
        if (host_inputs.size() != graph_.inputs().size()) return Error{"wrong number of inputs"};
        MCD_TRY(mcd_set_device(options_.device));
        for (std::size_t k = 0; k < host_inputs.size(); ++k) {
            const NodeId id = graph_.inputs()[k];
            MCD_TRY(mcd_copy_h2d(address(id, kRepF32), host_inputs[k], graph_.node(id).type.size_bytes(), stream_));
        }
        for (const Launch& l : upload_recasts_) MC_TRY(issue(l, stream_));
        // Kernels may be enqueued on another stream, which would not wait for these copies.
        MCD_TRY(mcd_stream_synchronize(stream_));
        return Status();
    }

    Status enqueue(void* stream) override {
        // One process may drive several GPUs: launches (and the tensor maps and per-device kernel set-up behind a
        // matmul) belong to this executable's device whatever the calling thread used last.
        MCD_TRY(mcd_set_device(options_.device));
        void* s = stream != nullptr ? stream : stream_;
        if (replay_ != nullptr) {
            MCD_TRY(mcd_graph_launch(replay_, s));
            return Status();
        }
        for (const std::unique_ptr<Launch>& l : launches_) MC_TRY(issue(*l, s));
        return Status();
    }

    Status synchronize() override {
        MCD_TRY(mcd_set_device(options_.device));
        MCD_TRY(mcd_device_synchronize());
        return check_status_word();
    }

    Status download_outputs(const std::vector<float*>& host_outputs) override {
        if (host_outputs.size() != graph_.outputs().size()) return Error{"wrong number of outputs"};
        MCD_TRY(mcd_set_device(options_.device));
        MCD_TRY(mcd_device_synchronize());  // kernels may sit on a caller's stream
        MC_TRY(check_status_word());
        for (std::size_t k = 0; k < host_outputs.size(); ++k) {
            const NodeId id = graph_.outputs()[k];
            MCD_TRY(mcd_copy_d2h(host_outputs[k], address(id, kRepF32), graph_.node(id).type.size_bytes(), stream_));
        }
        MCD_TRY(mcd_stream_synchronize(stream_));
        return Status();
    }

    std::size_t kernel_launches() const override { return lowered_.kernel_launches; }
    std::vector<std::string> kernel_sources() const override { return sources_; }
    std::vector<MatmulKernel> matmul_kernels() const override {
        std::vector<MatmulKernel> kernels;
        for (const std::unique_ptr<Launch>& l : launches_) {
            if (l->kind == Launch::Kind::Matmul) kernels.push_back(l->reported);
        }
        return kernels;
    }
    double jit_compile_ms() const override { return jit_ms_; }

    void constants_region(void** ptr, std::size_t* bytes) const override {
        *ptr = arena_;
        *bytes = constants_bytes_;
    }

    Status refresh_constants() override {
        MCD_TRY(mcd_set_device(options_.device));
        for (const Launch& l : constant_recasts_) MC_TRY(issue(l, stream_));
        MCD_TRY(mcd_stream_synchronize(stream_));
        return Status();
    }

    void* status_word_address() const override { return uses_status_ ? status_word() : nullptr; }

    Status replicate_constants(void* comm, int root) override {
        MCD_TRY(mcd_set_device(options_.device));
        if (constants_bytes_ == 0) return Status();
        MCD_TRY(mcd_nccl_broadcast(comm, arena_, constants_bytes_, root, stream_));
        MCD_TRY(mcd_nccl_wait(comm, stream_));
        return refresh_constants();
    }

    Status gather_output(std::size_t k, void* comm, void* device_dst) override {
        if (k >= graph_.outputs().size()) return Error{"no output " + std::to_string(k)};
        MCD_TRY(mcd_set_device(options_.device));
        MCD_TRY(mcd_device_synchronize());  // the kernels may sit on a caller's stream
        MC_TRY(check_status_word());
        const NodeId id = graph_.outputs()[k];
        MCD_TRY(mcd_nccl_all_gather(comm, address(id, kRepF32), device_dst, graph_.node(id).type.size_bytes(), stream_));
        MCD_TRY(mcd_nccl_wait(comm, stream_));
        return Status();
    }

    std::size_t row_slices() const override { return slice_rows_ > 0 ? static_cast<std::size_t>(slicing_.rows / slice_rows_) : 0; }
    std::size_t arena_bytes() const override { return arena_bytes_; }
    std::string plan_description() const override { return describe(graph_, lowered_); }

    void output_buffer(std::size_t k, void** ptr, std::size_t* elements) const override {
        const NodeId id = graph_.outputs()[k];
        *ptr = address(id, kRepF32);
        *elements = graph_.node(id).type.num_elements();
    }
    void input_buffer(std::size_t k, void** ptr, std::size_t* elements) const override {
        const NodeId id = graph_.inputs()[k];
        *ptr = address(id, kRepF32);
        *elements = graph_.node(id).type.num_elements();
    }

private:
    B200Executable(const Graph& graph, const CudaOptions& options) : graph_(graph), options_(options) {}

    // run() in row slices, three stages deep, for row-independent graphs on pinned caller memory: while slice i is
    // computed, slice i+1 comes in on one copy engine and slice i-1 goes out on the other. Every slice runs the
    // launches of the slice-sized plan with its pointers moved down by the slice's first row; slices follow one
    // another on the compute stream, so intermediates of different slices never coexist, and outputs live outside
    // the buffer pool, so a later slice cannot touch rows that are still being copied out. Sets *done when it ran.
    Status run_in_row_slices(const std::vector<const float*>& inputs, const std::vector<float*>& outputs, bool* done) {
        *done = false;
        if (slice_rows_ == 0) return Status();
        for (const float* p : inputs) {
            void* alias = nullptr;
            if (mcd_host_device_pointer(p, &alias) != 0) return Status();  // pageable memory: copies would not overlap
        }
        for (float* p : outputs) {
            void* alias = nullptr;
            if (mcd_host_device_pointer(p, &alias) != 0) return Status();
        }
        MCD_TRY(mcd_set_device(options_.device));
        const std::size_t slices = slice_in_.size();
        for (std::size_t c = 0; c < slices; ++c) {
            const std::size_t first_row = c * static_cast<std::size_t>(slice_rows_);
            for (std::size_t k = 0; k < inputs.size(); ++k) {
                const NodeId id = graph_.inputs()[k];
                const std::size_t per_row = row_bytes(graph_, id, kRepF32);
                if (per_row > 0) {
                    MCD_TRY(mcd_copy_h2d(address(id, kRepF32) + first_row * per_row,
                                         reinterpret_cast<const char*>(inputs[k]) + first_row * per_row,
                                         static_cast<std::size_t>(slice_rows_) * per_row, copy_in_));
                } else if (c == 0) {
                    MCD_TRY(mcd_copy_h2d(address(id, kRepF32), inputs[k], graph_.node(id).type.size_bytes(), copy_in_));
                }
            }
            MCD_TRY(mcd_event_record(slice_in_[c], copy_in_));
            MCD_TRY(mcd_stream_wait_event(stream_, slice_in_[c]));
            if (c == 0) {
                // 16-bit / transposed forms of inputs that are not cut are made once, from the whole tensor.
                for (const Launch& l : upload_recasts_) {
                    if (l.row_bytes[0] == 0) MC_TRY(issue(l, stream_));
                }
            }
            for (const Launch& l : slice_upload_recasts_) {
                if (l.row_bytes[0] != 0) MC_TRY(issue_at_row(l, first_row, stream_));
            }
            for (const std::unique_ptr<Launch>& l : slice_launches_) MC_TRY(issue_at_row(*l, first_row, stream_));
            MCD_TRY(mcd_event_record(slice_done_[c], stream_));
            MCD_TRY(mcd_stream_wait_event(copy_out_, slice_done_[c]));
            for (std::size_t k = 0; k < outputs.size(); ++k) {
                const NodeId id = graph_.outputs()[k];
                const std::size_t per_row = row_bytes(graph_, id, kRepF32);
                MCD_TRY(mcd_copy_d2h(reinterpret_cast<char*>(outputs[k]) + first_row * per_row,
                                     address(id, kRepF32) + first_row * per_row, static_cast<std::size_t>(slice_rows_) * per_row,
                                     copy_out_));
            }
        }
        MCD_TRY(mcd_stream_synchronize(copy_out_));
        MCD_TRY(mcd_stream_synchronize(stream_));
        MC_TRY(check_status_word());
        *done = true;
        return Status();
    }

    // One launch of the slice-sized plan, with every pointer into a cut tensor moved down to `first_row`.
    Status issue_at_row(const Launch& l, std::size_t first_row, void* stream) const {
        auto moved = [&](const void* p, std::size_t per_row) {
            return p == nullptr ? nullptr : const_cast<char*>(static_cast<const char*>(p)) + first_row * per_row;
        };
        switch (l.kind) {
            case Launch::Kind::Elementwise: {
                std::vector<void*> pointers(l.pointers.size());
                for (std::size_t i = 0; i < pointers.size(); ++i) pointers[i] = moved(l.pointers[i], l.row_bytes[i]);
                std::vector<void*> params;
                for (void*& p : pointers) params.push_back(&p);
                unsigned count = l.count;
                params.push_back(&count);
                MCD_TRY(mcd_launch(l.function, l.grid, 1, 1, l.block, 0, stream, params.data()));
                return Status();
            }
            case Launch::Kind::Matmul: {
                mcd_gemm_args g = l.gemm;
                g.a = moved(g.a, l.row_bytes[0]);
                g.c = static_cast<float*>(static_cast<void*>(moved(g.c, l.row_bytes[1])));
                g.c16 = moved(g.c16, l.row_bytes[2]);
                for (int i = 0; i < g.num_epilogue_inputs; ++i) {
                    g.epilogue_inputs[i] = static_cast<const float*>(static_cast<const void*>(
                        moved(g.epilogue_inputs[i], l.row_bytes[3 + static_cast<std::size_t>(i)])));
                }
                MCD_TRY(mcd_gemm(&g, stream));
                return Status();
            }
            case Launch::Kind::Recast: {
                Launch at = l;
                at.src = static_cast<const float*>(static_cast<const void*>(moved(l.src, l.row_bytes[0])));
                at.dst = moved(l.dst, l.row_bytes[1]);
                return issue(at, stream);
            }
        }
        return Status();
    }

    // run() without staging copies, for graphs that only stream: when every step is a generated elementwise
    // kernel, every graph input is read by exactly one of them and every output is written by one and read by
    // none, and the caller's buffers are pinned host memory the GPU can address, the kernels read the inputs
    // and write the outputs in place over PCIe. Both directions then move at once and each byte crosses the bus
    // once, instead of copy-in, compute, copy-out one after the other. Sets *done when it ran.
    Status run_on_host_memory(const std::vector<const float*>& inputs, const std::vector<float*>& outputs, bool* done) {
        *done = false;
        if (!streams_only_) return Status();
        std::vector<void*> in_alias(inputs.size()), out_alias(outputs.size());
        for (std::size_t k = 0; k < inputs.size(); ++k) {
            if (mcd_host_device_pointer(inputs[k], &in_alias[k]) != 0) return Status();
        }
        for (std::size_t k = 0; k < outputs.size(); ++k) {
            if (mcd_host_device_pointer(outputs[k], &out_alias[k]) != 0) return Status();
        }
        // The generated kernels move 128 bits per access when they are vectorised, which the arena's 256-byte
        // alignment guarantees but a caller's buffer (a view into a pinned allocation, say) may not: such a
        // call takes the staged path, whose copies have no alignment requirement.
        bool any_vectorized = false;
        for (const std::unique_ptr<Launch>& l : launches_) any_vectorized = any_vectorized || l->vectorized;
        std::vector<const void*> touched(in_alias.begin(), in_alias.end());
        touched.insert(touched.end(), out_alias.begin(), out_alias.end());
        if (pipeline_elements_ == 0 && !in_place_pointers_ok(any_vectorized, touched)) return Status();
        MCD_TRY(mcd_set_device(options_.device));
        if (pipeline_elements_ > 0) {
            MC_TRY(run_pipelined(inputs, outputs));
            *done = true;
            return Status();
        }
        for (const std::unique_ptr<Launch>& l : launches_) {
            std::vector<void*> pointers = l->pointers;
            for (void*& ptr : pointers) {
                for (std::size_t k = 0; k < inputs.size(); ++k) {
                    if (ptr == address(graph_.inputs()[k], kRepF32)) ptr = in_alias[k];
                }
                for (std::size_t k = 0; k < outputs.size(); ++k) {
                    if (ptr == address(graph_.outputs()[k], kRepF32)) ptr = out_alias[k];
                }
            }
            std::vector<void*> params;
            for (void*& ptr : pointers) params.push_back(&ptr);
            unsigned count = l->count;
            params.push_back(&count);
            MCD_TRY(mcd_launch(l->function, l->grid, 1, 1, kElementwiseBlock, 0, stream_, params.data()));
        }
        MCD_TRY(mcd_stream_synchronize(stream_));
        *done = true;
        return Status();
    }

    // The streaming graph in slices of rows, three stages deep: while slice i is computed, slice i+1 comes in
    // on one copy engine and slice i-1 goes out on the other, so both directions of the bus stay busy.
    // Applies when every tensor the kernels walk has the same element count (pipeline_elements_).
    Status run_pipelined(const std::vector<const float*>& inputs, const std::vector<float*>& outputs) {
        const std::size_t total = pipeline_elements_;
        const std::size_t slices = pipeline_slices();
        const std::size_t per = ((total + slices - 1) / slices + 1023) / 1024 * 1024;  // whole 128-bit groups, whole periods
        // Equal slices, except that the first and the last are cut further (1/4, 1/4, 1/2 and back): the bus is idle in
        // one direction while the first slice comes in and while the last goes out, so those are kept short.
        std::vector<std::size_t> counts;
        for (std::size_t first = 0; first < total; first += per) {
            const std::size_t n = std::min(per, total - first);
            const std::size_t quarter = n / 4 / 1024 * 1024;
            const bool head = first == 0, tail = first + per >= total;
            if (quarter == 0 || (!head && !tail) || (head && tail)) {
                counts.push_back(n);
            } else if (head) {
                counts.insert(counts.end(), {quarter, quarter, n - 2 * quarter});
            } else {
                counts.insert(counts.end(), {n - 2 * quarter, quarter, quarter});
            }
        }
        std::size_t first = 0;
        for (std::size_t c = 0; c < counts.size(); first += counts[c], ++c) {
            const std::size_t count = counts[c];
            for (std::size_t k = 0; k < inputs.size(); ++k) {
                const NodeId id = graph_.inputs()[k];
                const std::size_t n = graph_.node(id).type.num_elements();
                if (n == total) {
                    MCD_TRY(mcd_copy_h2d(address(id, kRepF32) + first * 4, inputs[k] + first, count * 4, copy_in_));
                } else if (c == 0) {
                    MCD_TRY(mcd_copy_h2d(address(id, kRepF32), inputs[k], n * 4, copy_in_));
                }
            }
            MCD_TRY(mcd_event_record(slice_in_[c], copy_in_));
            MCD_TRY(mcd_stream_wait_event(stream_, slice_in_[c]));
            for (const std::unique_ptr<Launch>& l : launches_) {
                std::vector<void*> pointers = l->pointers;
                for (std::size_t i = 0; i < pointers.size(); ++i) {
                    if (l->advances[i]) pointers[i] = static_cast<char*>(pointers[i]) + first * 4;
                }
                std::vector<void*> params;
                for (void*& ptr : pointers) params.push_back(&ptr);
                unsigned n = static_cast<unsigned>(l->vectorized ? count / 4 : count);
                params.push_back(&n);
                const std::size_t per_block = static_cast<std::size_t>(kElementwiseBlock) * options_.eltwise_unroll;
                const unsigned grid = static_cast<unsigned>(std::max<std::size_t>(1, std::min<std::size_t>(l->grid, (n + per_block - 1) / per_block)));
                MCD_TRY(mcd_launch(l->function, grid, 1, 1, kElementwiseBlock, 0, stream_, params.data()));
            }
            MCD_TRY(mcd_event_record(slice_done_[c], stream_));
            MCD_TRY(mcd_stream_wait_event(copy_out_, slice_done_[c]));
            for (std::size_t k = 0; k < outputs.size(); ++k) {
                const NodeId id = graph_.outputs()[k];
                MCD_TRY(mcd_copy_d2h(outputs[k] + first, address(id, kRepF32) + first * 4, count * 4, copy_out_));
            }
        }
        MCD_TRY(mcd_stream_synchronize(copy_out_));
        MCD_TRY(mcd_stream_synchronize(stream_));
        return Status();
    }

    // Element count shared by every walked tensor when the graph can run in row slices, else 0.
    std::size_t pipeline_elements() const {
        if (!streams_only_ || options_.host_io != 1) return 0;
        std::size_t total = 0;
        for (const std::unique_ptr<Launch>& l : launches_) {
            const std::size_t n = static_cast<std::size_t>(l->count) * (l->vectorized ? 4 : 1);
            if (total == 0) total = n;
            if (n != total || (l->vectorized ? n % 4 != 0 : false)) return 0;
        }
        // Operands that repeat (bias rows) must repeat whole within a slice: slices are multiples of 1024 elements.
        // Anything whose index depends on the position in the whole tensor (a [M,1] column, say) rules slicing out.
        for (const Step& s : lowered_.steps) {
            const Shape& out_shape = graph_.node(s.result).type.shape;
            for (NodeId in : s.inputs) {
                const Access a = classify_access(graph_.node(in).type.shape, out_shape);
                if (a.kind == AccessKind::General) return 0;
                if (a.kind == AccessKind::Periodic && (a.period > 1024 || 1024 % a.period != 0)) return 0;
            }
        }
        return total >= (std::size_t{1} << 22) ? total : 0;  // below 16 MiB a slice is too small to be worth a stage
    }

    // Whether run_on_host_memory applies to this graph at all (decided once, at compile time).
    bool graph_only_streams() const {
        if (options_.host_io == 0) return false;
        std::vector<int> reads(graph_.num_nodes(), 0);
        for (const Step& s : lowered_.steps) {
            if (s.kind != Step::Kind::Elementwise) return false;
            if (s.write_half != HalfKind::None) return false;
            std::vector<NodeId> seen;
            for (NodeId in : s.inputs) {
                if (std::find(seen.begin(), seen.end(), in) != seen.end()) continue;
                seen.push_back(in);
                ++reads[static_cast<std::size_t>(in)];
                // A broadcast operand would cross the bus once per repetition: only same-size or one-element inputs.
                const std::size_t count = graph_.node(in).type.num_elements();
                if (graph_.node(in).op == OpKind::Input && count != 1 &&
                    count != graph_.node(s.result).type.num_elements()) {
                    return false;
                }
            }
        }
        for (const std::vector<Recast>& after : lowered_.after_step) {
            if (!after.empty()) return false;
        }
        for (NodeId in : graph_.inputs()) {
            if (reads[static_cast<std::size_t>(in)] != 1 || graph_.is_output(in)) return false;
        }
        for (NodeId out : graph_.outputs()) {
            if (!is_compute(graph_.node(out).op) || reads[static_cast<std::size_t>(out)] != 0) return false;
        }
        return !lowered_.steps.empty();
    }

    char* address(NodeId id, Rep rep) const {
        const std::size_t slot = static_cast<std::size_t>(id) * kNumReps + static_cast<std::size_t>(rep);
        return offset_[slot] == kNoOffset ? nullptr : static_cast<char*>(arena_) + offset_[slot];
    }

    Status check_status_word() {
        if (!uses_status_) return Status();
        unsigned word = 0;
        MCD_TRY(mcd_copy_d2h(&word, status_word(), sizeof word, stream_));
        MCD_TRY(mcd_stream_synchronize(stream_));
        if (word != 0) {
            MCD_TRY(mcd_memset(status_word(), 0, sizeof word, stream_));
            return Error{"a matmul kernel gave up a bounded wait (status 0x" + to_hex(word) +
                         "): results of this run are incomplete"};
        }
        return Status();
    }

    static std::string to_hex(unsigned v) {
        char text[16];
        std::snprintf(text, sizeof text, "%x", v);
        return text;
    }

    unsigned* status_word() const { return reinterpret_cast<unsigned*>(static_cast<char*>(arena_) + status_offset_); }

    Status issue(const Launch& l, void* stream) const {
        switch (l.kind) {
            case Launch::Kind::Elementwise:
                MCD_TRY(mcd_launch(l.function, l.grid, 1, 1, l.block, 0, stream, const_cast<void**>(l.params.data())));
                return Status();
            case Launch::Kind::Matmul: MCD_TRY(mcd_gemm(&l.gemm, stream)); return Status();
            case Launch::Kind::Recast:
                if (l.half_kind == 0) {
                    MCD_TRY(mcd_transpose_f32(l.src, static_cast<float*>(l.dst), l.rows, l.cols, l.src_pitch, l.dst_pitch, stream));
                } else {
                    MCD_TRY(mcd_cast_f32_to_half(l.half_kind, l.src, l.dst, l.rows, l.cols, l.src_pitch, l.dst_pitch,
                                                 l.transpose, stream));
                }
                return Status();
        }
        return Status();
    }

    Launch make_recast(const Graph& graph, const Recast& rc) const {
        const TensorType& type = graph.node(rc.node).type;
        Launch l;
        l.kind = Launch::Kind::Recast;
        l.src = reinterpret_cast<const float*>(address(rc.node, kRepF32));
        l.dst = address(rc.node, rc.to);
        l.rows = type.shape[0];
        l.cols = type.shape[1];
        l.src_pitch = l.cols;
        const int half = lowered_.half_kind == HalfKind::Bf16 ? MCD_HALF_BF16 : MCD_HALF_F16;
        switch (rc.to) {
            case kRepHalf:
                l.half_kind = half;
                l.dst_pitch = half_pitch(l.cols);
                break;
            case kRepHalfT:
                l.half_kind = half;
                l.transpose = 1;
                l.dst_pitch = half_pitch(l.rows);
                break;
            default:  // kRepF32T
                l.half_kind = 0;
                l.transpose = 1;
                l.dst_pitch = (l.rows + 3) / 4 * 4;
                break;
        }
        l.row_bytes = {row_bytes(graph, rc.node, kRepF32), row_bytes(graph, rc.node, rc.to)};
        return l;
    }

    // Bytes between consecutive rows of the cut dimension in form `rep` of `node`; 0 when the value is not cut.
    std::size_t row_bytes(const Graph& graph, NodeId node, Rep rep) const {
        if (!slicing_.ok || !slicing_.carries[static_cast<std::size_t>(node)]) return 0;
        const TensorType& type = graph.node(node).type;
        const std::size_t per_row = type.num_elements() / static_cast<std::size_t>(type.shape[0]);
        switch (rep) {
            case kRepF32: return per_row * sizeof(float);
            case kRepHalf: return (type.rank() == 2 ? static_cast<std::size_t>(half_pitch(type.shape[1])) : per_row) * 2;
            default: return 0;  // transposed forms are never cut (their rows are the other dimension)
        }
    }

    Status init() {
        Result<DeviceInfo> device = query_device(options_.device);
        if (!device.ok()) return device.error();
        device_ = std::move(device).value();
        if (device_.cc_major != 10) {
            return Error{"this backend is built for sm_100a (B200) only; device " + std::to_string(options_.device) + " is " +
                         device_.name + " (compute capability " + std::to_string(device_.cc_major) + "." +
                         std::to_string(device_.cc_minor) + ")"};
        }
        MCD_TRY(mcd_set_device(options_.device));
        MCD_TRY(mcd_stream_create(&stream_));

        // Row slicing for run() on pinned memory is decided first: it changes where outputs live.
        MC_TRY(plan_row_slices());
        MC_ASSIGN(lowered, lower_graph(graph_, options_, device_.sm_count, /*pool_outputs=*/slice_rows_ == 0));
        lowered_ = std::move(lowered);
        if (slice_rows_ > 0) {
            MC_TRY(lower_row_slices());
            if (slice_rows_ == 0) {  // the slice-sized graph lowers differently: outputs go back into the pool
                MC_ASSIGN(again, lower_graph(graph_, options_, device_.sm_count, true));
                lowered_ = std::move(again);
            }
        }

        // ---- arena layout: constants | inputs | outputs kept out of the pool | pooled buffers | split-K workspace | status word
        const std::size_t count = graph_.num_nodes();
        offset_.assign(count * kNumReps, kNoOffset);
        std::size_t cursor = 0;
        auto place_leaves = [&](OpKind kind) {
            for (std::size_t i = 0; i < count; ++i) {
                const Node& n = graph_.node(static_cast<NodeId>(i));
                if (n.op != kind) continue;
                for (int rep = 0; rep < kNumReps; ++rep) {
                    if (!lowered_.needs[i][static_cast<std::size_t>(rep)]) continue;
                    offset_[i * kNumReps + static_cast<std::size_t>(rep)] = cursor;
                    cursor += align_up(rep_bytes(n.type, static_cast<Rep>(rep)));
                }
            }
        };
        place_leaves(OpKind::Constant);
        constants_bytes_ = cursor;
        place_leaves(OpKind::Input);
        unpooled_output_bytes_ = 0;
        for (std::size_t v = 0; v < lowered_.pool_values.size(); ++v) {
            const PoolValue& value = lowered_.pool_values[v];
            if (value.pooled || !value.live_out || !is_compute(graph_.node(static_cast<NodeId>(v / kNumReps)).op)) continue;
            offset_[v] = cursor;
            cursor += align_up(value.bytes);
            unpooled_output_bytes_ += value.bytes;
        }
        std::vector<std::size_t> buffer_offset(lowered_.pool.buffer_bytes.size());
        for (std::size_t b = 0; b < buffer_offset.size(); ++b) {
            buffer_offset[b] = cursor;
            cursor += align_up(std::max<std::size_t>(lowered_.pool.buffer_bytes[b], sizeof(float)));
        }
        for (std::size_t v = 0; v < lowered_.pool.buffer_of.size(); ++v) {
            const std::int32_t b = lowered_.pool.buffer_of[v];
            if (b != PoolPlan::kNotPooled) offset_[v] = buffer_offset[static_cast<std::size_t>(b)];
        }
        const std::size_t workspace_bytes = std::max(lowered_.workspace_bytes, slice_rows_ > 0 ? slice_lowered_.workspace_bytes : 0);
        const std::size_t workspace_offset = cursor;
        cursor += align_up(workspace_bytes);
        status_offset_ = cursor;
        cursor += kAlign;
        arena_bytes_ = cursor;
        MCD_TRY(mcd_malloc(&arena_, arena_bytes_));
        MCD_TRY(mcd_memset(status_word(), 0, kAlign, stream_));
        float* workspace = workspace_bytes > 0 ? reinterpret_cast<float*>(static_cast<char*>(arena_) + workspace_offset) : nullptr;

        // ---- constants: uploaded once, derived forms made once
        for (std::size_t i = 0; i < count; ++i) {
            const Node& n = graph_.node(static_cast<NodeId>(i));
            if (n.op != OpKind::Constant) continue;
            MCD_TRY(mcd_copy_h2d(address(static_cast<NodeId>(i), kRepF32), n.constant->data(), n.type.size_bytes(), stream_));
        }
        for (const Recast& rc : lowered_.at_compile) constant_recasts_.push_back(make_recast(graph_, rc));
        for (const Recast& rc : lowered_.after_upload) upload_recasts_.push_back(make_recast(graph_, rc));
        for (const Launch& l : constant_recasts_) MC_TRY(issue(l, stream_));
        MCD_TRY(mcd_stream_synchronize(stream_));

        // ---- launches
        MC_TRY(build_launches(graph_, lowered_, workspace, launches_));
        if (slice_rows_ > 0) {
            MC_TRY(build_launches(slice_graph_, slice_lowered_, workspace, slice_launches_));
            for (const Recast& rc : slice_lowered_.after_upload) slice_upload_recasts_.push_back(make_recast(slice_graph_, rc));
            MCD_TRY(mcd_stream_create(&copy_in_));
            MCD_TRY(mcd_stream_create(&copy_out_));
            const std::size_t slices = static_cast<std::size_t>(slicing_.rows / slice_rows_);
            slice_in_.assign(slices, nullptr);
            slice_done_.assign(slices, nullptr);
            for (std::size_t c = 0; c < slices; ++c) {
                MCD_TRY(mcd_event_create(&slice_in_[c]));
                MCD_TRY(mcd_event_create(&slice_done_[c]));
            }
        }
        // Every buffer address is fixed for the life of the executable, so the launch list can be recorded
        // once and replayed: one graph launch per enqueue instead of one driver call (and, for tensor-core
        // matmuls, two tensor-map encodings) per kernel. The list runs once for real first, so that one-time
        // kernel set-up does not happen inside the recording.
        streams_only_ = slice_rows_ == 0 && graph_only_streams();
        pipeline_elements_ = pipeline_elements();
        if (pipeline_elements_ > 0) {
            MCD_TRY(mcd_stream_create(&copy_in_));
            MCD_TRY(mcd_stream_create(&copy_out_));
            slice_in_.assign(pipeline_slices() + 4, nullptr);  // the first and the last slice are cut in three
            slice_done_.assign(pipeline_slices() + 4, nullptr);
            for (std::size_t c = 0; c < slice_in_.size(); ++c) {
                MCD_TRY(mcd_event_create(&slice_in_[c]));
                MCD_TRY(mcd_event_create(&slice_done_[c]));
            }
        }
        if (options_.replay_graph && launches_.size() >= 2) {
            for (const std::unique_ptr<Launch>& l : launches_) MC_TRY(issue(*l, stream_));
            MCD_TRY(mcd_stream_synchronize(stream_));
            MCD_TRY(mcd_graph_begin_capture(stream_));
            Status recorded;
            for (const std::unique_ptr<Launch>& l : launches_) {
                recorded = issue(*l, stream_);
                if (!recorded.ok()) break;
            }
            void* graph = nullptr;
            const int rc = mcd_graph_end_capture(stream_, &graph);
            if (!recorded.ok()) return recorded;
            if (rc != 0) return device_error("mcd_graph_end_capture");
            replay_ = graph;
            MCD_TRY(mcd_memset(status_word(), 0, kAlign, stream_));
            MCD_TRY(mcd_stream_synchronize(stream_));
        }
        return Status();
    }

    Status build_launches(const Graph& graph, const LoweredGraph& lowered, float* workspace, LaunchList& list) {
        for (std::size_t i = 0; i < lowered.steps.size(); ++i) {
            const Step& step = lowered.steps[i];
            if (step.kind == Step::Kind::Elementwise) {
                MC_TRY(add_elementwise(graph, step, list));
            } else if (step.kind == Step::Kind::RowFused) {
                MC_TRY(add_row_fused(graph, step, list));
            } else if (step.kind == Step::Kind::Reduce) {
                MC_TRY(add_reduce(graph, step, list));
            } else {
                MC_TRY(add_matmul(graph, step, workspace, list));
            }
            for (const Recast& rc : lowered.after_step[i]) list.push_back(std::make_unique<Launch>(make_recast(graph, rc)));
        }
        return Status();
    }

    // Decides whether run() on pinned memory works in row slices, and how many rows a slice has (slice_rows_;
    // 0 = no). Worth it for graphs that are not one streaming elementwise launch (those have a path of their
    // own), whose rows are independent, and that move enough bytes over the bus for the overlap to pay.
    Status plan_row_slices() {
        slice_rows_ = 0;
        if (options_.host_io != 1 || options_.host_io_row_slices < 2) return Status();
        bool has_heavy_node = false;
        for (const Node& n : graph_.nodes()) has_heavy_node = has_heavy_node || n.op == OpKind::MatMul || is_row_reduce(n.op);
        if (!has_heavy_node) return Status();
        slicing_ = analyze_row_slicing(graph_);
        if (!slicing_.ok) return Status();
        std::size_t moved = 0;
        for (NodeId in : graph_.inputs()) moved += graph_.node(in).type.size_bytes();
        for (NodeId out : graph_.outputs()) moved += graph_.node(out).type.size_bytes();
        if (moved < kMinSlicedBytes) {
            slicing_ = RowSlicing{};
            return Status();
        }
        // The largest slice count up to the requested one that divides the rows into multiples of 128 (whole tiles)
        // and leaves every slice at least 16 MiB to move: smaller copies cost more at the stream hand-offs than
        // shorter ends save.
        const std::int64_t most = std::min<std::int64_t>(options_.host_io_row_slices, static_cast<std::int64_t>(moved / kMinSliceBytes));
        for (std::int64_t slices = most; slices >= 2; --slices) {
            if (slicing_.rows % slices == 0 && (slicing_.rows / slices) % 128 == 0) {
                slice_rows_ = slicing_.rows / slices;
                break;
            }
        }
        if (slice_rows_ == 0) slicing_ = RowSlicing{};
        return Status();
    }

    // Lowers the graph at the slice's row count and checks that it is the same plan as the full one: same steps in
    // the same order defining the same forms, so that the slice's launches can use the full plan's addresses.
    // K splits are taken from the full plan, so a slice adds every output's products in the same order as the
    // unsliced run (results are bit-identical). Anything else turns slicing off (slice_rows_ = 0).
    Status lower_row_slices() {
        auto give_up = [&] {
            slice_rows_ = 0;
            slicing_ = RowSlicing{};
            return Status();
        };
        Result<Graph> sliced = with_leading_extent(graph_, slicing_, slice_rows_);
        if (!sliced.ok()) return give_up();
        Result<LoweredGraph> lowered = lower_graph(*sliced, options_, device_.sm_count, false);
        if (!lowered.ok()) return give_up();
        if (lowered->steps.size() != lowered_.steps.size() || lowered->needs != lowered_.needs) return give_up();
        for (std::size_t i = 0; i < lowered_.steps.size(); ++i) {
            Step& mine = lowered->steps[i];
            const Step& full = lowered_.steps[i];
            if (mine.kind != full.kind || mine.result != full.result || mine.inputs != full.inputs ||
                mine.write_f32 != full.write_f32 || mine.write_half != full.write_half ||
                mine.has_epilogue != full.has_epilogue || mine.row_outputs != full.row_outputs ||
                lowered->after_step[i].size() != lowered_.after_step[i].size()) {
                return give_up();
            }
            if (mine.kind == Step::Kind::Matmul) {
                mine.splits = full.splits;
                mine.launches = full.launches;
                if (mine.splits > 1) {
                    lowered->workspace_bytes = std::max(
                        lowered->workspace_bytes, static_cast<std::size_t>(mine.splits) * mine.m * mine.n * sizeof(float));
                }
            }
        }
        // Forms of cut values that a slice cannot address by rows.
        for (std::size_t i = 0; i < graph_.num_nodes(); ++i) {
            if (slicing_.carries[i] && (lowered_.needs[i][kRepHalfT] || lowered_.needs[i][kRepF32T])) return give_up();
        }
        slice_graph_ = std::move(sliced).value();
        slice_lowered_ = std::move(lowered).value();
        return Status();
    }

    Status add_elementwise(const Graph& graph, const Step& step, LaunchList& list) {
        const Node& node = graph.node(step.result);
        std::vector<Shape> shapes;
        for (NodeId in : step.inputs) shapes.push_back(graph.node(in).type.shape);
        ElementwiseOptions eo;
        eo.allow_vectorize = options_.vectorize;
        eo.unroll = options_.eltwise_unroll;
        eo.write_f32 = step.write_f32;
        eo.write_half = step.write_half;
        eo.streaming_hints = options_.streaming_hints;
        if (step.write_half != HalfKind::None && node.type.shape.size() == 2) eo.half_pitch = half_pitch(node.type.shape[1]);
        const ElementwiseKernel kernel = generate_elementwise_kernel(step.program, shapes, node.type.shape, eo);

        auto launch = std::make_unique<Launch>();
        launch->kind = Launch::Kind::Elementwise;
        double ms = 0.0;
        if (mcd_jit_kernel(options_.device, kernel.source.c_str(), kElementwiseKernelName, options_.eltwise_fmad ? "--fmad=true" : "--fmad=false", &launch->function,
                           &ms) != 0) {
            return Error{std::string("compiling the kernel of '") + node.name + "' failed: " + mcd_last_error()};
        }
        jit_ms_ += ms;
        jit_functions_.push_back(launch->function);
        sources_.push_back(kernel.source);

        const std::size_t n = node.type.num_elements();
        launch->count = static_cast<unsigned>(kernel.vectorized ? n / 4 : n);
        int blocks_per_sm = 0;
        MCD_TRY(mcd_jit_occupancy(launch->function, static_cast<int>(kElementwiseBlock), 0, &blocks_per_sm));
        if (options_.eltwise_blocks_per_sm > 0) blocks_per_sm = std::min(blocks_per_sm, options_.eltwise_blocks_per_sm);
        // By default one block per tile of the tensor (measured on B200: 6.32 against 5.94 TB/s for one wave of
        // resident blocks that loop); a positive blocks_per_sm asks for the looping form with that many blocks per SM.
        const std::size_t per_block = static_cast<std::size_t>(kElementwiseBlock) * kernel.unroll;
        const std::size_t wanted = (launch->count + per_block - 1) / per_block;
        std::size_t resident = std::max<std::size_t>(1, static_cast<std::size_t>(blocks_per_sm) * device_.sm_count);
        if (options_.eltwise_blocks_per_sm <= 0) resident = wanted;
        launch->grid = static_cast<unsigned>(std::max<std::size_t>(1, std::min(wanted, resident)));
        launch->vectorized = kernel.vectorized;
        if (kernel.has_f32_out) {
            launch->pointers.push_back(address(step.result, kRepF32));
            launch->advances.push_back(1);
            launch->row_bytes.push_back(row_bytes(graph, step.result, kRepF32));
        }
        if (kernel.has_half_out) {
            launch->pointers.push_back(address(step.result, kRepHalf));
            launch->advances.push_back(1);
            launch->row_bytes.push_back(row_bytes(graph, step.result, kRepHalf));
        }
        for (NodeId in : step.inputs) {
            launch->pointers.push_back(address(in, kRepF32));
            launch->advances.push_back(graph.node(in).type.num_elements() == n ? 1 : 0);
            launch->row_bytes.push_back(row_bytes(graph, in, kRepF32));
        }
        for (void*& p : launch->pointers) launch->params.push_back(&p);
        launch->params.push_back(&launch->count);
        list.push_back(std::move(launch));
        return Status();
    }

    // A row reduction with its elementwise prologue: one generated kernel, a warp or a block per row.
    Status add_reduce(const Graph& graph, const Step& step, LaunchList& list) {
        const Node& node = graph.node(step.result);
        std::vector<Shape> shapes;
        for (NodeId in : step.inputs) shapes.push_back(graph.node(in).type.shape);
        const RowReduceKernel kernel = generate_row_reduce_kernel(step.reduce_op, step.program, shapes, step.reduce_shape);

        auto launch = std::make_unique<Launch>();
        launch->kind = Launch::Kind::Elementwise;
        double ms = 0.0;
        if (mcd_jit_kernel(options_.device, kernel.source.c_str(), kRowReduceKernelName, "--fmad=false", &launch->function, &ms) != 0) {
            return Error{std::string("compiling the kernel of '") + node.name + "' failed: " + mcd_last_error()};
        }
        jit_ms_ += ms;
        jit_functions_.push_back(launch->function);
        sources_.push_back(kernel.source);

        const std::size_t rows = node.type.num_elements();
        launch->count = static_cast<unsigned>(rows);
        launch->block = kernel.block;
        int blocks_per_sm = 0;
        MCD_TRY(mcd_jit_occupancy(launch->function, static_cast<int>(kernel.block), 0, &blocks_per_sm));
        // One block (one cluster of blocks, for rows wider than 8192) per row; the grid is a whole number of clusters.
        const std::size_t wanted = (rows + kernel.rows_per_block - 1) / kernel.rows_per_block * kernel.cluster;
        std::size_t resident = std::max<std::size_t>(1, static_cast<std::size_t>(blocks_per_sm) * device_.sm_count);
        if (options_.eltwise_blocks_per_sm <= 0) resident = wanted;
        resident = std::max<std::size_t>(kernel.cluster, resident / kernel.cluster * kernel.cluster);
        launch->grid = static_cast<unsigned>(std::max<std::size_t>(1, std::min(wanted, resident)));
        launch->pointers.push_back(address(step.result, kRepF32));
        launch->advances.push_back(0);
        launch->row_bytes.push_back(row_bytes(graph, step.result, kRepF32));
        for (NodeId in : step.inputs) {
            launch->pointers.push_back(address(in, kRepF32));
            launch->advances.push_back(0);
            launch->row_bytes.push_back(row_bytes(graph, in, kRepF32));
        }
        for (void*& p : launch->pointers) launch->params.push_back(&p);
        launch->params.push_back(&launch->count);
        list.push_back(std::move(launch));
        return Status();
    }

    // A run of steps on rows of one shape as one kernel, a block per row.
    Status add_row_fused(const Graph& graph, const Step& step, LaunchList& list) {
        const std::string source = generate_row_fused_kernel(step.row_parts, step.row_externals,
                                                             static_cast<int>(step.row_outputs.size()), step.reduce_shape.back());
        auto launch = std::make_unique<Launch>();
        launch->kind = Launch::Kind::Elementwise;
        double ms = 0.0;
        if (mcd_jit_kernel(options_.device, source.c_str(), kRowFusedKernelName, "--fmad=false", &launch->function, &ms) != 0) {
            return Error{std::string("compiling the row kernel of '") + graph.node(step.result).name + "' failed: " + mcd_last_error()};
        }
        jit_ms_ += ms;
        jit_functions_.push_back(launch->function);
        sources_.push_back(source);
        const std::size_t rows = num_elements(step.reduce_shape) / static_cast<std::size_t>(step.reduce_shape.back());
        launch->count = static_cast<unsigned>(rows);
        launch->block = row_block(step.reduce_shape.back());
        int blocks_per_sm = 0;
        MCD_TRY(mcd_jit_occupancy(launch->function, static_cast<int>(launch->block), 0, &blocks_per_sm));
        std::size_t resident = std::max<std::size_t>(1, static_cast<std::size_t>(blocks_per_sm) * device_.sm_count);
        const std::size_t rows_per_block = launch->block / row_threads(step.reduce_shape.back());
        const std::size_t cluster = row_cluster(step.reduce_shape.back());
        const std::size_t wanted = (rows + rows_per_block - 1) / rows_per_block * cluster;
        if (options_.eltwise_blocks_per_sm <= 0) resident = wanted;
        resident = std::max<std::size_t>(cluster, resident / cluster * cluster);
        launch->grid = static_cast<unsigned>(std::max<std::size_t>(1, std::min(wanted, resident)));
        for (NodeId w : step.row_outputs) {
            launch->pointers.push_back(address(w, kRepF32));
            launch->advances.push_back(0);
            launch->row_bytes.push_back(row_bytes(graph, w, kRepF32));
        }
        for (NodeId in : step.inputs) {
            launch->pointers.push_back(address(in, kRepF32));
            launch->advances.push_back(0);
            launch->row_bytes.push_back(row_bytes(graph, in, kRepF32));
        }
        for (void*& p : launch->pointers) launch->params.push_back(&p);
        launch->params.push_back(&launch->count);
        list.push_back(std::move(launch));
        return Status();
    }

    Status add_matmul(const Graph& graph, const Step& step, float* workspace, LaunchList& list) {
        auto launch = std::make_unique<Launch>();
        launch->kind = Launch::Kind::Matmul;
        launch->reported = step.kernel;
        mcd_gemm_args& g = launch->gemm;
        std::memset(&g, 0, sizeof g);
        g.arith = static_cast<int>(step.arith);
        g.m = step.m;
        g.n = step.n;
        g.k = step.k;
        const bool half = step.arith == Arith::Bf16 || step.arith == Arith::F16;
        if (is_tensor_core(step.kernel) && mcd_tensor_core_supported(options_.device, g.arith) == 0) {
            return Error{std::string("matmul kernel '") + matmul_kernel_name(step.kernel) + "' does not run on " + device_.name +
                         ": the tcgen05 kernels need compute capability 10.x"};
        }
        g.a = address(step.lhs, half ? kRepHalf : kRepF32);
        g.lda = half ? half_pitch(step.k) : step.k;
        if (step.rhs_transposed) {
            g.b = address(step.rhs, half ? kRepHalfT : kRepF32T);
            g.ldb = half ? half_pitch(step.k) : (step.k + 3) / 4 * 4;
            g.b_transposed = 1;
        } else {
            g.b = address(step.rhs, half ? kRepHalf : kRepF32);
            g.ldb = half ? half_pitch(step.n) : step.n;
        }
        g.c = step.write_f32 ? reinterpret_cast<float*>(address(step.result, kRepF32)) : nullptr;
        g.ldc = step.n;
        if (step.write_half != HalfKind::None) {
            g.c16 = address(step.result, kRepHalf);
            g.c16_kind = step.write_half == HalfKind::Bf16 ? MCD_HALF_BF16 : MCD_HALF_F16;
            g.ldc16 = half_pitch(step.n);
        }
        std::vector<std::size_t> epilogue_row_bytes;
        launch->row_bytes = {row_bytes(graph, step.lhs, half ? kRepHalf : kRepF32),
                             step.write_f32 ? row_bytes(graph, step.result, kRepF32) : 0,
                             step.write_half != HalfKind::None ? row_bytes(graph, step.result, kRepHalf) : 0};
        g.splits = step.splits;
        g.tile_n = step.tile_n;
        g.workspace = step.splits > 1 ? workspace : nullptr;
        g.variant = options_.gemm_variant;
        // Kernels fed by TMA wait on mbarriers; a wait that gives up reports through this word.
        g.status = status_word();
        uses_status_ = true;
        if (step.has_epilogue) {
            g.has_epilogue = 1;
            int slot = 0;
            for (std::size_t k = 0; k < step.inputs.size(); ++k) {
                if (step.load_is_accumulator[k]) continue;
                g.epilogue_inputs[slot++] = reinterpret_cast<const float*>(address(step.inputs[k], kRepF32));
                epilogue_row_bytes.push_back(row_bytes(graph, step.inputs[k], kRepF32));
            }
            g.num_epilogue_inputs = slot;
            const std::string epilogue = generate_epilogue_source(graph, step);
            sources_.push_back(epilogue);
            double ms = 0.0;
            if (mcd_gemm_launches(&g) > 1) {
                // K is split: the main kernel writes raw partial sums, the reduction applies the epilogue.
                const std::string source = epilogue + mcd_gemm_source(-1);
                if (mcd_jit_kernel(options_.device, source.c_str(), mcd_gemm_entry_point(nullptr), "--fmad=false",
                                   &g.reduce_function, &ms) != 0) {
                    return Error{std::string("compiling the epilogue of '") + graph.node(step.result).name +
                                 "' failed: " + mcd_last_error()};
                }
                jit_functions_.push_back(g.reduce_function);
            } else {
                // Only the entry point this launch uses is compiled out of the kernel family's text.
                const std::string entry = mcd_gemm_entry_point(&g);
                const std::string source =
                    "#define MC_SINGLE_ENTRY 1\n#define MC_ONLY_" + entry + " 1\n" + epilogue + mcd_gemm_source(g.arith);
                if (mcd_jit_kernel(options_.device, source.c_str(), entry.c_str(), "--fmad=false", &g.function,
                                   &ms) != 0) {
                    return Error{std::string("compiling the epilogue of '") + graph.node(step.result).name +
                                 "' failed: " + mcd_last_error()};
                }
                jit_functions_.push_back(g.function);
                const std::size_t smem = mcd_gemm_dynamic_smem(g.arith);
                if (smem > 0) MCD_TRY(mcd_jit_set_dynamic_smem(g.function, smem));
            }
            jit_ms_ += ms;
        }
        launch->row_bytes.insert(launch->row_bytes.end(), epilogue_row_bytes.begin(), epilogue_row_bytes.end());
        list.push_back(std::move(launch));
        return Status();
    }

    static constexpr std::size_t kNoOffset = static_cast<std::size_t>(-1);

    Graph graph_;
    CudaOptions options_;
    DeviceInfo device_;
    LoweredGraph lowered_;
    void* stream_ = nullptr;
    void* arena_ = nullptr;
    void* replay_ = nullptr;
    bool streams_only_ = false;
    std::size_t pipeline_slices() const {
        return static_cast<std::size_t>(std::min(256, std::max(2, options_.host_io_slices)));
    }
    std::size_t pipeline_elements_ = 0;
    void* copy_in_ = nullptr;
    void* copy_out_ = nullptr;
    std::vector<void*> slice_in_;
    std::vector<void*> slice_done_;
    std::size_t arena_bytes_ = 0;
    std::size_t constants_bytes_ = 0;
    std::size_t status_offset_ = 0;
    bool uses_status_ = false;
    std::vector<std::size_t> offset_;  // per (node, rep): byte offset in the arena
    LaunchList launches_;
    // Row slicing of run() on pinned memory: the analysis, the rows per slice (0 = off), the graph and plan at
    // that row count, and its launches, which use the full plan's addresses and are moved row-wise per slice.
    static constexpr std::size_t kMinSlicedBytes = std::size_t{32} << 20;
    static constexpr std::size_t kMinSliceBytes = std::size_t{16} << 20;
    RowSlicing slicing_;
    std::int64_t slice_rows_ = 0;
    Graph slice_graph_;
    LoweredGraph slice_lowered_;
    LaunchList slice_launches_;
    std::vector<Launch> slice_upload_recasts_;
    std::size_t unpooled_output_bytes_ = 0;
    std::vector<Launch> upload_recasts_;
    std::vector<Launch> constant_recasts_;
    std::vector<std::string> sources_;
    std::vector<void*> jit_functions_;  // one reference each in the device layer's kernel cache
    double jit_ms_ = 0.0;
};

class B200Backend final : public Backend {
public:
    explicit B200Backend(const CudaOptions& options) : options_(options) {}
    const char* name() const override { return "cuda"; }
    Result<std::unique_ptr<Executable>> compile(const Graph& graph) override {
        Result<std::unique_ptr<CudaExecutable>> exe = compile_for_cuda(graph, options_);
        if (!exe.ok()) return exe.error();
        return std::unique_ptr<Executable>(std::move(exe).value());
    }

private:
    CudaOptions options_;
};

}  // namespace

Result<DeviceInfo> query_device(int device) {
    mcd_device_info raw;
    if (mcd_query_device(device, &raw) != 0) return Error{mcd_last_error()};
    DeviceInfo info;
    info.name = raw.name;
    info.cc_major = raw.cc_major;
    info.cc_minor = raw.cc_minor;
    info.sm_count = raw.sm_count;
    info.fp32_lanes_per_sm = raw.fp32_lanes_per_sm;
    info.sm_clock_mhz = raw.sm_clock_mhz;
    info.max_sm_clock_mhz = raw.max_sm_clock_mhz;
    info.mem_clock_mhz = raw.mem_clock_mhz;
    info.bus_width_bits = raw.bus_width_bits;
    info.total_memory = raw.total_memory;
    info.runtime_version = raw.runtime_version;
    info.driver_version = raw.driver_version;
    return info;
}

double current_sm_clock_mhz(int device) { return mcd_current_sm_clock_mhz(device); }

bool in_place_pointers_ok(bool any_vectorized, const std::vector<const void*>& pointers) {
    if (!any_vectorized) return true;
    for (const void* p : pointers) {
        if (reinterpret_cast<std::uintptr_t>(p) % 16 != 0) return false;
    }
    return true;
}

Result<std::unique_ptr<CudaExecutable>> compile_for_cuda(const Graph& graph, const CudaOptions& options) {
    MC_TRY(graph.verify());
    Result<std::unique_ptr<B200Executable>> exe = B200Executable::create(graph, options);
    if (!exe.ok()) return exe.error();
    return std::unique_ptr<CudaExecutable>(std::move(exe).value());
}

Result<std::unique_ptr<Backend>> make_cuda_backend(const CudaOptions& options) {
    Result<DeviceInfo> device = query_device(options.device);
    if (!device.ok()) return Error{"no usable CUDA device: " + device.error().message};
    return std::unique_ptr<Backend>(std::make_unique<B200Backend>(options));
}

}  // namespace cuda
}  // namespace minicompiler
