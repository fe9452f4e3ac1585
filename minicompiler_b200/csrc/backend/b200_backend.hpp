#pragma once
// The runtime API in front of the B200 backend: Backend / Executable /
// CudaExecutable / compile_for_cuda / make_cuda_backend / query_device, with the
// reference's names, argument meaning and error behaviour
// (include/minicompiler/runtime/backend.hpp:18-49,
// include/minicompiler/cuda/cuda_backend.hpp:51-107). Behind it nothing is
// shared with the reference: values live in one device arena laid out from the
// memory plan, kernels come from the sm_100a device layer, and every CUDA call
// goes through the C-ABI in minicompiler_b200_device.h.

#include "backend/lowering.hpp"
#include "core/ir.hpp"
#include "core/mcg.hpp"

#include <cstddef>
#include <memory>
#include <string>
#include <string_view>
#include <vector>

namespace minicompiler {

class Executable {
public:
    virtual ~Executable() = default;
    // `inputs` follow Graph::inputs(); `outputs` is resized to Graph::outputs() and must be a
    // different vector.
    virtual Status run(const std::vector<HostTensor>& inputs, std::vector<HostTensor>& outputs) = 0;
    // Caller-owned host memory, graph order.
    virtual Status run_buffers(const std::vector<const float*>& inputs, const std::vector<float*>& outputs) = 0;
    virtual std::size_t intermediate_bytes() const = 0;
};

class Backend {
public:
    virtual ~Backend() = default;
    virtual const char* name() const = 0;
    virtual Result<std::unique_ptr<Executable>> compile(const Graph& graph) = 0;
};

// This library is the GPU backend only: {"cuda"}.
std::vector<std::string> available_backends();
Result<std::unique_ptr<Backend>> create_backend(std::string_view name);

namespace cuda {

struct DeviceInfo {
    std::string name;
    int cc_major = 0;
    int cc_minor = 0;
    int sm_count = 0;
    int fp32_lanes_per_sm = 0;
    double sm_clock_mhz = 0;
    double max_sm_clock_mhz = 0;
    double mem_clock_mhz = 0;
    int bus_width_bits = 0;
    std::size_t total_memory = 0;
    int runtime_version = 0;
    int driver_version = 0;

    double peak_bandwidth_gbs() const { return 2.0 * mem_clock_mhz * 1e6 * bus_width_bits / 8.0 / 1e9; }
    double peak_fp32_gflops(double clock_mhz) const { return 2.0 * sm_count * fp32_lanes_per_sm * clock_mhz * 1e6 / 1e9; }
};

Result<DeviceInfo> query_device(int device = 0);
double current_sm_clock_mhz(int device = 0);

class CudaExecutable : public Executable {
public:
    // Returns once the inputs are on the device (and any 16-bit copies of them are made).
    virtual Status upload_inputs(const std::vector<const float*>& host_inputs) = 0;
    // Launches every kernel in order on `stream` (cudaStream_t; nullptr = the executable's own
    // stream). No copies, no synchronization.
    virtual Status enqueue(void* stream = nullptr) = 0;
    virtual Status synchronize() = 0;
    // Waits for the device, then copies the outputs out.
    virtual Status download_outputs(const std::vector<float*>& host_outputs) = 0;

    virtual std::size_t kernel_launches() const = 0;
    virtual std::vector<std::string> kernel_sources() const = 0;
    virtual std::vector<MatmulKernel> matmul_kernels() const = 0;
    virtual double jit_compile_ms() const = 0;

    // Additions for multi-GPU replication and introspection.
    // The packed constants (FP32 and derived forms) as one device range.
    virtual void constants_region(void** ptr, std::size_t* bytes) const = 0;
    // Re-derives the 16-bit / transposed forms of the constants from their FP32 form
    // (after the region was overwritten, e.g. by a broadcast).
    virtual Status refresh_constants() = 0;
    // Device address of the word into which a tensor-core kernel that gives up a bounded wait ORs its code
    // (nullptr when no launch of this executable can wait). synchronize() / download_outputs() read and clear it.
    virtual void* status_word_address() const = 0;
    // Row slices run() on pinned host memory is cut into (0: it copies in, runs and copies out, or streams).
    virtual std::size_t row_slices() const = 0;
    // Multi-GPU (one process per GPU, `comm` from mcd_nccl_init): one broadcast makes `root`'s packed constants
    // everybody's and the derived forms are rebuilt; an all-gather assembles output k of all ranks (each holding
    // its rows) in `device_dst`, world_size times the output's size. Both return when the data is in place.
    virtual Status replicate_constants(void* comm, int root) = 0;
    virtual Status gather_output(std::size_t k, void* comm, void* device_dst) = 0;
    virtual std::size_t arena_bytes() const = 0;
    virtual std::string plan_description() const = 0;
    // Device address and element count of output k's FP32 buffer.
    virtual void output_buffer(std::size_t k, void** ptr, std::size_t* elements) const = 0;
    virtual void input_buffer(std::size_t k, void** ptr, std::size_t* elements) const = 0;
};

// Whether kernels may read and write these caller buffers in place: a vectorised kernel moves 128 bits per
// access, so every buffer must then start on a 16-byte boundary (a pinned allocation does; a view into one need not).
bool in_place_pointers_ok(bool any_vectorized, const std::vector<const void*>& pointers);

Result<std::unique_ptr<CudaExecutable>> compile_for_cuda(const Graph& graph, const CudaOptions& options = {});
Result<std::unique_ptr<Backend>> make_cuda_backend(const CudaOptions& options = {});

}  // namespace cuda
}  // namespace minicompiler
