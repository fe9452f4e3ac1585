// Device layer, part 1: device query, memory, streams, events and run-time
// compilation. The CUDA runtime is linked statically; the driver API is reached
// through cudaGetDriverEntryPoint and NVRTC / NVML through dlopen, so the
// library loads (and its host-side half works) on machines without a GPU driver.

#include "minicompiler_b200_device.h"

#include "device/driver_api.hpp"

#include <cuda.h>
#include <cuda_runtime_api.h>
#include <dlfcn.h>
#include <nvrtc.h>
#include <nvtx3/nvToolsExt.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

namespace mcd {

thread_local std::string g_last_error;
std::atomic<unsigned long long> g_launches{0};

int fail(const std::string& message) {
    g_last_error = message;
    return 1;
}

int check_rt(cudaError_t err, const char* what) {
    if (err == cudaSuccess) return 0;
    return fail(std::string(what) + ": " + cudaGetErrorString(err));
}

int check_drv(CUresult err, const char* what) {
    if (err == CUDA_SUCCESS) return 0;
    const char* text = nullptr;
    const DriverApi* api = driver_api();
    if (api != nullptr && api->GetErrorString != nullptr) api->GetErrorString(err, &text);
    return fail(std::string(what) + ": " + (text != nullptr ? text : "CUDA driver error " + std::to_string(static_cast<int>(err))));
}

// ------------------------------------------------------------ driver API

namespace {

template <typename Fn>
bool resolve(const char* symbol, Fn& slot) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint(symbol, &fn, cudaEnableDefault, &status) != cudaSuccess || fn == nullptr ||
        status != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return false;
    }
    slot = reinterpret_cast<Fn>(fn);
    return true;
}

}  // namespace

const DriverApi* driver_api() {
    static DriverApi api;
    static std::once_flag once;
    static bool usable = false;
    std::call_once(once, [] {
        bool ok = true;
        ok = resolve("cuGetErrorString", api.GetErrorString) && ok;
        ok = resolve("cuModuleLoadData", api.ModuleLoadData) && ok;
        ok = resolve("cuModuleGetFunction", api.ModuleGetFunction) && ok;
        ok = resolve("cuModuleUnload", api.ModuleUnload) && ok;
        ok = resolve("cuLaunchKernel", api.LaunchKernel) && ok;
        ok = resolve("cuLaunchKernelEx", api.LaunchKernelEx) && ok;
        ok = resolve("cuFuncSetAttribute", api.FuncSetAttribute) && ok;
        ok = resolve("cuOccupancyMaxActiveBlocksPerMultiprocessor", api.OccupancyMaxActiveBlocksPerMultiprocessor) && ok;
        ok = resolve("cuTensorMapEncodeTiled", api.TensorMapEncodeTiled) && ok;
        usable = ok;
    });
    return usable ? &api : nullptr;
}

// ------------------------------------------------------------------ NVRTC

namespace {

struct NvrtcApi {
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*);
    nvrtcResult (*DestroyProgram)(nvrtcProgram*);
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*);
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*);
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*);
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*);
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*);
    const char* (*GetErrorString)(nvrtcResult);
};

const NvrtcApi* nvrtc_api(std::string* why) {
    static NvrtcApi api;
    static std::once_flag once;
    static bool usable = false;
    static std::string reason;
    std::call_once(once, [] {
        void* lib = nullptr;
        for (const char* name : {"libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"}) {
            lib = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (lib != nullptr) break;
        }
        if (lib == nullptr) {
            reason = std::string("cannot load libnvrtc.so.12: ") + dlerror();
            return;
        }
        bool ok = true;
        auto sym = [&](const char* name, auto& slot) {
            void* p = dlsym(lib, name);
            if (p == nullptr) ok = false;
            slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(p);
        };
        sym("nvrtcCreateProgram", api.CreateProgram);
        sym("nvrtcDestroyProgram", api.DestroyProgram);
        sym("nvrtcCompileProgram", api.CompileProgram);
        sym("nvrtcGetCUBINSize", api.GetCUBINSize);
        sym("nvrtcGetCUBIN", api.GetCUBIN);
        sym("nvrtcGetProgramLogSize", api.GetProgramLogSize);
        sym("nvrtcGetProgramLog", api.GetProgramLog);
        sym("nvrtcGetErrorString", api.GetErrorString);
        usable = ok;
        if (!ok) reason = "libnvrtc.so.12 lacks an expected entry point";
    });
    if (!usable && why != nullptr) *why = reason;
    return usable ? &api : nullptr;
}

}  // namespace

// Source -> sm_100a cubin. Needs no GPU, so generated kernels are compile-checked on any host.
int compile_to_cubin(const char* source, const char* options, std::vector<char>* cubin, std::string* log) {
    std::string why;
    const NvrtcApi* rtc = nvrtc_api(&why);
    if (rtc == nullptr) return fail(why);
    nvrtcProgram program = nullptr;
    nvrtcResult rc = rtc->CreateProgram(&program, source, "mc_kernel.cu", 0, nullptr, nullptr);
    if (rc != NVRTC_SUCCESS) return fail(std::string("nvrtcCreateProgram: ") + rtc->GetErrorString(rc));

    std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo"};
    if (options != nullptr) {
        const char* at = options;
        while (*at != '\0') {
            while (*at == ' ') ++at;
            const char* stop = at;
            while (*stop != '\0' && *stop != ' ') ++stop;
            if (stop > at) opts.emplace_back(at, stop);
            at = stop;
        }
    }
    std::vector<const char*> argv;
    for (const std::string& o : opts) argv.push_back(o.c_str());
    rc = rtc->CompileProgram(program, static_cast<int>(argv.size()), argv.data());
    if (rc != NVRTC_SUCCESS) {
        std::string text;
        size_t log_size = 0;
        if (rtc->GetProgramLogSize(program, &log_size) == NVRTC_SUCCESS && log_size > 1) {
            text.resize(log_size);
            rtc->GetProgramLog(program, text.data());
        }
        rtc->DestroyProgram(&program);
        if (log != nullptr) *log = text;
        return fail(std::string("nvrtcCompileProgram: ") + rtc->GetErrorString(rc) + "\n" + text + "\n--- source ---\n" + source);
    }
    size_t size = 0;
    rc = rtc->GetCUBINSize(program, &size);
    if (rc == NVRTC_SUCCESS) {
        cubin->resize(size);
        rc = rtc->GetCUBIN(program, cubin->data());
    }
    rtc->DestroyProgram(&program);
    if (rc != NVRTC_SUCCESS) return fail(std::string("nvrtcGetCUBIN: ") + rtc->GetErrorString(rc));
    return 0;
}

}  // namespace mcd

using namespace mcd;

extern "C" {

const char* mcd_last_error(void) { return g_last_error.c_str(); }

unsigned long long mcd_launch_count(void) { return g_launches.load(); }

int mcd_device_count(int* count) {
    *count = 0;
    return check_rt(cudaGetDeviceCount(count), "cudaGetDeviceCount");
}

namespace {

// FP32 lanes per SM by compute capability (CUDA programming guide, arithmetic throughput table).
int fp32_lanes(int major, int minor) {
    if (major >= 9) return 128;
    if (major == 8) return minor == 0 ? 64 : 128;
    if (major == 7) return 64;
    if (major == 6) return minor == 0 ? 64 : 128;
    return 128;
}

struct Nvml {
    int (*Init)() = nullptr;
    int (*DeviceGetHandleByIndex)(unsigned, void**) = nullptr;
    int (*DeviceGetMaxClockInfo)(void*, int, unsigned*) = nullptr;
    int (*DeviceGetClockInfo)(void*, int, unsigned*) = nullptr;
    bool ready = false;
};

Nvml& nvml() {
    static Nvml n;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
        if (lib == nullptr) return;
        n.Init = reinterpret_cast<int (*)()>(dlsym(lib, "nvmlInit_v2"));
        n.DeviceGetHandleByIndex = reinterpret_cast<int (*)(unsigned, void**)>(dlsym(lib, "nvmlDeviceGetHandleByIndex_v2"));
        n.DeviceGetMaxClockInfo = reinterpret_cast<int (*)(void*, int, unsigned*)>(dlsym(lib, "nvmlDeviceGetMaxClockInfo"));
        n.DeviceGetClockInfo = reinterpret_cast<int (*)(void*, int, unsigned*)>(dlsym(lib, "nvmlDeviceGetClockInfo"));
        n.ready = n.Init && n.DeviceGetHandleByIndex && n.DeviceGetMaxClockInfo && n.DeviceGetClockInfo && n.Init() == 0;
    });
    return n;
}

constexpr int kNvmlClockSm = 1;  // NVML_CLOCK_SM

}  // namespace

int mcd_query_device(int device, mcd_device_info* out) {
    std::memset(out, 0, sizeof *out);
    int count = 0;
    if (int rc = check_rt(cudaGetDeviceCount(&count), "cudaGetDeviceCount")) return rc;
    if (device < 0 || device >= count) {
        return fail("device " + std::to_string(device) + " does not exist (" + std::to_string(count) + " visible)");
    }
    cudaDeviceProp prop;
    if (int rc = check_rt(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties")) return rc;
    std::snprintf(out->name, sizeof out->name, "%.127s", prop.name);
    out->cc_major = prop.major;
    out->cc_minor = prop.minor;
    out->sm_count = prop.multiProcessorCount;
    out->fp32_lanes_per_sm = fp32_lanes(prop.major, prop.minor);
    int khz = 0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device) == cudaSuccess) out->sm_clock_mhz = khz / 1000.0;
    if (cudaDeviceGetAttribute(&khz, cudaDevAttrMemoryClockRate, device) == cudaSuccess) out->mem_clock_mhz = khz / 1000.0;
    cudaDeviceGetAttribute(&out->bus_width_bits, cudaDevAttrGlobalMemoryBusWidth, device);
    cudaDeviceGetAttribute(&out->max_smem_per_block_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
    out->total_memory = prop.totalGlobalMem;
    cudaRuntimeGetVersion(&out->runtime_version);
    cudaDriverGetVersion(&out->driver_version);
    cudaGetLastError();
    Nvml& n = nvml();
    void* handle = nullptr;
    unsigned mhz = 0;
    if (n.ready && n.DeviceGetHandleByIndex(static_cast<unsigned>(device), &handle) == 0 &&
        n.DeviceGetMaxClockInfo(handle, kNvmlClockSm, &mhz) == 0) {
        out->max_sm_clock_mhz = mhz;
    }
    return 0;
}

double mcd_current_sm_clock_mhz(int device) {
    Nvml& n = nvml();
    void* handle = nullptr;
    unsigned mhz = 0;
    if (n.ready && n.DeviceGetHandleByIndex(static_cast<unsigned>(device), &handle) == 0 &&
        n.DeviceGetClockInfo(handle, kNvmlClockSm, &mhz) == 0) {
        return mhz;
    }
    return 0.0;
}

int mcd_set_device(int device) { return check_rt(cudaSetDevice(device), "cudaSetDevice"); }

int mcd_malloc(void** ptr, size_t bytes) {
    *ptr = nullptr;
    return check_rt(cudaMalloc(ptr, bytes == 0 ? 16 : bytes), "cudaMalloc");
}
int mcd_free(void* ptr) { return ptr == nullptr ? 0 : check_rt(cudaFree(ptr), "cudaFree"); }
int mcd_memset(void* ptr, int byte, size_t bytes, void* stream) {
    return check_rt(cudaMemsetAsync(ptr, byte, bytes, static_cast<cudaStream_t>(stream)), "cudaMemsetAsync");
}
int mcd_copy_h2d(void* dst, const void* src, size_t bytes, void* stream) {
    return check_rt(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)),
                    "cudaMemcpyAsync(host to device)");
}
int mcd_copy_d2h(void* dst, const void* src, size_t bytes, void* stream) {
    return check_rt(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)),
                    "cudaMemcpyAsync(device to host)");
}
int mcd_copy_d2d(void* dst, const void* src, size_t bytes, void* stream) {
    return check_rt(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)),
                    "cudaMemcpyAsync(device to device)");
}
int mcd_host_device_pointer(const void* host, void** device_alias) {
    *device_alias = nullptr;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, host) != cudaSuccess) {
        cudaGetLastError();
        return fail("mcd_host_device_pointer: not a CUDA-visible address");
    }
    if (attr.type != cudaMemoryTypeHost || attr.devicePointer == nullptr) {
        return fail("mcd_host_device_pointer: the memory is not pinned and mapped");
    }
    *device_alias = attr.devicePointer;
    return 0;
}
int mcd_host_register(void* ptr, size_t bytes) {
    return check_rt(cudaHostRegister(ptr, bytes, cudaHostRegisterDefault), "cudaHostRegister");
}
int mcd_host_unregister(void* ptr) { return check_rt(cudaHostUnregister(ptr), "cudaHostUnregister"); }
int mcd_stream_create(void** stream) {
    cudaStream_t s = nullptr;
    const int rc = check_rt(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreateWithFlags");
    *stream = s;
    return rc;
}
int mcd_stream_destroy(void* stream) {
    return stream == nullptr ? 0 : check_rt(cudaStreamDestroy(static_cast<cudaStream_t>(stream)), "cudaStreamDestroy");
}
int mcd_stream_synchronize(void* stream) {
    return check_rt(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "cudaStreamSynchronize");
}
int mcd_device_synchronize(void) { return check_rt(cudaDeviceSynchronize(), "cudaDeviceSynchronize"); }
int mcd_event_create(void** event) {
    cudaEvent_t e = nullptr;
    const int rc = check_rt(cudaEventCreate(&e), "cudaEventCreate");
    *event = e;
    return rc;
}
int mcd_event_destroy(void* event) {
    return event == nullptr ? 0 : check_rt(cudaEventDestroy(static_cast<cudaEvent_t>(event)), "cudaEventDestroy");
}
int mcd_stream_wait_event(void* stream, void* event) {
    return check_rt(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0), "cudaStreamWaitEvent");
}
int mcd_event_record(void* event, void* stream) {
    return check_rt(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)), "cudaEventRecord");
}
int mcd_event_record_external(void* event, void* stream) {
    return check_rt(cudaEventRecordWithFlags(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream), cudaEventRecordExternal),
                    "cudaEventRecordWithFlags(external)");
}
int mcd_range_push(const char* label) {
    nvtxRangePushA(label != nullptr ? label : "");
    return 0;
}
int mcd_range_pop(void) {
    nvtxRangePop();
    return 0;
}
int mcd_event_elapsed_ms(void* start, void* stop, float* ms) {
    if (int rc = check_rt(cudaEventSynchronize(static_cast<cudaEvent_t>(stop)), "cudaEventSynchronize")) return rc;
    return check_rt(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)),
                    "cudaEventElapsedTime");
}

// ------------------------------------------------------------------- JIT
//
// Modules are cached process-wide. The key is (device, options, entry point, 64-bit hash and length of the
// source), so the table does not keep the source texts. Every mcd_jit_kernel call takes a reference that
// mcd_jit_release gives back; a module nobody holds stays loaded as long as at most kJitIdleLimit such
// modules exist (a graph compiled again shortly after its executable was destroyed costs nothing), beyond
// that the least recently used idle module is unloaded. NVRTC runs outside the lock, so threads compiling
// different kernels (or for different devices) do not wait for one another.

namespace {

struct JitKey {
    int device;
    std::string options;
    std::string entry;
    unsigned long long hash;
    std::size_t length;
    bool operator<(const JitKey& o) const {
        return std::tie(device, hash, length, entry, options) < std::tie(o.device, o.hash, o.length, o.entry, o.options);
    }
};

struct JitEntry {
    CUmodule module = nullptr;
    CUfunction function = nullptr;
    long refs = 0;
    unsigned long long last_use = 0;
};

constexpr std::size_t kJitIdleLimit = 128;

std::mutex g_jit_mutex;
std::map<JitKey, JitEntry> g_jit_cache;
std::map<void*, JitKey> g_jit_by_function;
unsigned long long g_jit_clock = 0;

unsigned long long fnv1a64(const char* text, std::size_t n) {
    unsigned long long h = 1469598103934665603ull;
    for (std::size_t i = 0; i < n; ++i) {
        h ^= static_cast<unsigned char>(text[i]);
        h *= 1099511628211ull;
    }
    return h;
}

void unload_on(int device, CUmodule module) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr || module == nullptr) return;
    int current = -1;
    cudaGetDevice(&current);
    if (current != device) cudaSetDevice(device);
    drv->ModuleUnload(module);
    if (current != device && current >= 0) cudaSetDevice(current);
}

// Called with the lock held: unloads least-recently-used idle modules beyond the limit.
void evict_idle_locked() {
    for (;;) {
        std::size_t idle = 0;
        auto oldest = g_jit_cache.end();
        for (auto it = g_jit_cache.begin(); it != g_jit_cache.end(); ++it) {
            if (it->second.refs > 0) continue;
            ++idle;
            if (oldest == g_jit_cache.end() || it->second.last_use < oldest->second.last_use) oldest = it;
        }
        if (idle <= kJitIdleLimit || oldest == g_jit_cache.end()) return;
        unload_on(oldest->first.device, oldest->second.module);
        g_jit_by_function.erase(oldest->second.function);
        g_jit_cache.erase(oldest);
    }
}

}  // namespace

int mcd_jit_kernel(int device, const char* source, const char* kernel_name, const char* options, void** function,
                   double* compile_ms) {
    *function = nullptr;
    if (compile_ms != nullptr) *compile_ms = 0.0;
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable (no driver on this machine?)");
    const std::size_t length = std::strlen(source);
    const JitKey key{device, std::string(options != nullptr ? options : ""), std::string(kernel_name), fnv1a64(source, length),
                     length};
    {
        std::lock_guard<std::mutex> lock(g_jit_mutex);
        const auto hit = g_jit_cache.find(key);
        if (hit != g_jit_cache.end()) {
            ++hit->second.refs;
            hit->second.last_use = ++g_jit_clock;
            *function = hit->second.function;
            return 0;
        }
    }
    int current = -1;
    if (int rc = check_rt(cudaGetDevice(&current), "cudaGetDevice")) return rc;
    if (current != device) {
        if (int rc = check_rt(cudaSetDevice(device), "cudaSetDevice")) return rc;
    }
    if (int rc = check_rt(cudaFree(nullptr), "cudaFree(nullptr)")) return rc;  // make the primary context current

    const auto t0 = std::chrono::steady_clock::now();
    std::vector<char> cubin;
    int rc = compile_to_cubin(source, options, &cubin, nullptr);
    JitEntry entry;
    if (rc == 0) rc = check_drv(drv->ModuleLoadData(&entry.module, cubin.data()), "cuModuleLoadData");
    if (rc == 0) rc = check_drv(drv->ModuleGetFunction(&entry.function, entry.module, kernel_name), "cuModuleGetFunction");
    const auto t1 = std::chrono::steady_clock::now();
    if (rc != 0 && entry.module != nullptr) drv->ModuleUnload(entry.module);
    if (current != device) cudaSetDevice(current);
    if (rc != 0) return rc;
    if (compile_ms != nullptr) *compile_ms = std::chrono::duration<double, std::milli>(t1 - t0).count();

    std::lock_guard<std::mutex> lock(g_jit_mutex);
    const auto raced = g_jit_cache.find(key);
    if (raced != g_jit_cache.end()) {
        // Another thread compiled the same kernel meanwhile: keep its module, drop ours.
        unload_on(device, entry.module);
        ++raced->second.refs;
        raced->second.last_use = ++g_jit_clock;
        *function = raced->second.function;
        return 0;
    }
    entry.refs = 1;
    entry.last_use = ++g_jit_clock;
    g_jit_by_function.emplace(entry.function, key);
    g_jit_cache.emplace(key, entry);
    *function = entry.function;
    evict_idle_locked();
    return 0;
}

int mcd_jit_release(void* function) {
    if (function == nullptr) return 0;
    std::lock_guard<std::mutex> lock(g_jit_mutex);
    const auto key = g_jit_by_function.find(function);
    if (key == g_jit_by_function.end()) return fail("mcd_jit_release: not a kernel of mcd_jit_kernel (or released too often)");
    const auto entry = g_jit_cache.find(key->second);
    if (entry == g_jit_cache.end() || entry->second.refs <= 0) return fail("mcd_jit_release: released more often than obtained");
    --entry->second.refs;
    evict_idle_locked();
    return 0;
}

int mcd_jit_cache_stats(long long* modules, long long* idle) {
    std::lock_guard<std::mutex> lock(g_jit_mutex);
    long long n = 0, unused = 0;
    for (const auto& kv : g_jit_cache) {
        ++n;
        if (kv.second.refs == 0) ++unused;
    }
    if (modules != nullptr) *modules = n;
    if (idle != nullptr) *idle = unused;
    return 0;
}

int mcd_jit_occupancy(void* function, int block_threads, size_t dynamic_smem, int* blocks_per_sm) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    return check_drv(drv->OccupancyMaxActiveBlocksPerMultiprocessor(blocks_per_sm, static_cast<CUfunction>(function),
                                                                    block_threads, dynamic_smem),
                     "cuOccupancyMaxActiveBlocksPerMultiprocessor");
}

int mcd_jit_set_dynamic_smem(void* function, size_t bytes) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    return check_drv(drv->FuncSetAttribute(static_cast<CUfunction>(function), CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                           static_cast<int>(bytes)),
                     "cuFuncSetAttribute(max dynamic shared memory)");
}

int mcd_launch(void* function, unsigned grid_x, unsigned grid_y, unsigned grid_z, unsigned block_x, size_t dynamic_smem,
               void* stream, void** params) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return check_drv(drv->LaunchKernel(static_cast<CUfunction>(function), grid_x, grid_y, grid_z, block_x, 1, 1,
                                       static_cast<unsigned>(dynamic_smem), static_cast<CUstream>(stream), params, nullptr),
                     "cuLaunchKernel");
}

int mcd_launch_cluster(void* function, unsigned grid_x, unsigned cluster_x, unsigned block_x, size_t dynamic_smem, void* stream,
                       void** params) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    if (cluster_x == 0 || grid_x % cluster_x != 0) return fail("mcd_launch_cluster: the grid is not a whole number of clusters");
    CUlaunchAttribute attribute;
    attribute.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attribute.value.clusterDim.x = cluster_x;
    attribute.value.clusterDim.y = 1;
    attribute.value.clusterDim.z = 1;
    CUlaunchConfig config;
    std::memset(&config, 0, sizeof config);
    config.gridDimX = grid_x;
    config.gridDimY = 1;
    config.gridDimZ = 1;
    config.blockDimX = block_x;
    config.blockDimY = 1;
    config.blockDimZ = 1;
    config.sharedMemBytes = static_cast<unsigned>(dynamic_smem);
    config.hStream = static_cast<CUstream>(stream);
    config.attrs = &attribute;
    config.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return check_drv(drv->LaunchKernelEx(&config, static_cast<CUfunction>(function), params, nullptr), "cuLaunchKernelEx");
}

int mcd_launch_dependent(void* function, unsigned grid_x, unsigned block_x, size_t dynamic_smem, void* stream, void** params) {
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    CUlaunchAttribute attribute;
    attribute.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attribute.value.programmaticStreamSerializationAllowed = 1;
    CUlaunchConfig config;
    std::memset(&config, 0, sizeof config);
    config.gridDimX = grid_x;
    config.gridDimY = 1;
    config.gridDimZ = 1;
    config.blockDimX = block_x;
    config.blockDimY = 1;
    config.blockDimZ = 1;
    config.sharedMemBytes = static_cast<unsigned>(dynamic_smem);
    config.hStream = static_cast<CUstream>(stream);
    config.attrs = &attribute;
    config.numAttrs = 1;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return check_drv(drv->LaunchKernelEx(&config, static_cast<CUfunction>(function), params, nullptr), "cuLaunchKernelEx");
}

// ------------------------------------------------------------ graph replay

namespace {
struct GraphExec {
    cudaGraphExec_t exec = nullptr;
    unsigned long long kernels = 0;
};
thread_local unsigned long long g_capture_start = 0;
}  // namespace

int mcd_graph_begin_capture(void* stream) {
    g_capture_start = g_launches.load();
    return check_rt(cudaStreamBeginCapture(static_cast<cudaStream_t>(stream), cudaStreamCaptureModeThreadLocal),
                    "cudaStreamBeginCapture");
}

int mcd_graph_end_capture(void* stream, void** graph_exec) {
    *graph_exec = nullptr;
    cudaGraph_t graph = nullptr;
    if (int rc = check_rt(cudaStreamEndCapture(static_cast<cudaStream_t>(stream), &graph), "cudaStreamEndCapture")) return rc;
    auto* ge = new GraphExec();
    ge->kernels = g_launches.load() - g_capture_start;
    g_launches.store(g_capture_start);  // recorded, not run
    const int rc = check_rt(cudaGraphInstantiate(&ge->exec, graph, 0), "cudaGraphInstantiate");
    cudaGraphDestroy(graph);
    if (rc != 0) {
        delete ge;
        return rc;
    }
    *graph_exec = ge;
    return 0;
}

int mcd_graph_launch(void* graph_exec, void* stream) {
    auto* ge = static_cast<GraphExec*>(graph_exec);
    g_launches.fetch_add(ge->kernels, std::memory_order_relaxed);
    return check_rt(cudaGraphLaunch(ge->exec, static_cast<cudaStream_t>(stream)), "cudaGraphLaunch");
}

int mcd_graph_destroy(void* graph_exec) {
    auto* ge = static_cast<GraphExec*>(graph_exec);
    if (ge == nullptr) return 0;
    const int rc = check_rt(cudaGraphExecDestroy(ge->exec), "cudaGraphExecDestroy");
    delete ge;
    return rc;
}

// Compile-only entry point (no GPU needed): used by tests and `mcc --emit-cuda --check`.
MCD_API int mcd_jit_compile_only(const char* source, const char* options, size_t* cubin_bytes) {
    std::vector<char> cubin;
    const int rc = compile_to_cubin(source, options, &cubin, nullptr);
    if (cubin_bytes != nullptr) *cubin_bytes = cubin.size();
    return rc;
}

}  // extern "C"
