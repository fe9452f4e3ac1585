// mcd_gemm_f32_split_no_alloc: the FP32 split-K matmul for callers that must not
// allocate device memory.
//
// Who that is: a process that gave all of HBM to its own pool at start-up and has
// nothing left for cudaMalloc to hand out; and code on a latency-critical path, where
// the implicit device-wide synchronisation of cudaMalloc / cudaFree is not acceptable.
// Such callers cannot use the split-K path of mcd_gemm, because that one expects the
// caller to bring a workspace of splits*m*n floats for the partial sums.
//
// Here the partial sums live in a fixed array that is part of the library image. CUDA
// loads the module that owns it lazily, so a GPU starts to hold its
// MCD_NO_ALLOC_SCRATCH_BYTES on the FIRST call made on it (that call may allocate and
// synchronise inside the driver, so it belongs at start-up, before the caller's pool
// takes the rest of HBM and before any stream capture; a tiny splits = 1 problem will
// do) and keeps them until the process exits. The kernels are the very same source as the regular path (the .cuh files are
// included a second time under other entry-point names), so results are bit-identical
// to mcd_gemm with the same split count.

#include "minicompiler_b200_device.h"

#include "device/driver_api.hpp"

#include <cuda_runtime.h>

#include <atomic>
#include <mutex>
#include <string>

// Same kernel text as gemm_launch.cu, under names of their own (one definition per image).
#define mc_gemm_f32_vec mc_na_gemm_f32_vec
#define mc_gemm_f32_any mc_na_gemm_f32_any
#define mc_gemm_f32_body mc_na_gemm_f32_body
#define mc_splitk_reduce mc_na_splitk_reduce
#define MC_F32_NO_TMA_KERNEL 1  // this image keeps the register-staged kernels only
#include "kernels/epilogue.cuh"
#include "kernels/gemm_f32_simt.cuh"
#include "kernels/splitk_reduce.cuh"

namespace mcd {
extern std::atomic<unsigned long long> g_launches;
}

namespace {

// The scratch itself. In host code this name is only a handle for the runtime (it is not a
// device address): the address the kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float mc_na_scratch[MCD_NO_ALLOC_SCRATCH_BYTES / sizeof(float)];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
float* g_scratch_address[kMaxDevices] = {nullptr};

// Once per device, with that device current: resolve the device address of the array.
int scratch_for_current_device(float** out) {
    int device = 0;
    if (int rc = mcd::check_rt(cudaGetDevice(&device), "cudaGetDevice")) return rc;
    if (device < 0 || device >= kMaxDevices) return mcd::fail("mcd_gemm_f32_split_no_alloc: device ordinal out of range");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
        void* address = nullptr;
        if (int rc = mcd::check_rt(cudaGetSymbolAddress(&address, mc_na_scratch), "cudaGetSymbolAddress(scratch)")) return rc;
        g_scratch_address[device] = static_cast<float*>(address);
    }
    *out = g_scratch_address[device];
    return 0;
}

bool aligned16(const void* p) { return (reinterpret_cast<unsigned long long>(p) & 15ull) == 0; }

}  // namespace

extern "C" int mcd_gemm_f32_split_no_alloc(const float* a, const float* b, float* c, int m, int n, int k, int splits,
                                           void* stream) {
    if (a == nullptr || b == nullptr || c == nullptr) return mcd::fail("mcd_gemm_f32_split_no_alloc: null operand");
    if (m <= 0 || n <= 0 || k <= 0) return mcd::fail("mcd_gemm_f32_split_no_alloc: empty problem");
    // Same split arithmetic as the regular FP32 path: whole K steps per slice, no empty slice.
    int want = splits < 1 ? 1 : splits;
    const int k_per_split = ((k + want - 1) / want + MC_F32_BK - 1) / MC_F32_BK * MC_F32_BK;
    const int depth = (k + k_per_split - 1) / k_per_split;
    const unsigned long long need = static_cast<unsigned long long>(depth) * static_cast<unsigned long long>(m) *
                                    static_cast<unsigned long long>(n) * sizeof(float);
    if (depth > 1 && need > MCD_NO_ALLOC_SCRATCH_BYTES) {
        return mcd::fail("mcd_gemm_f32_split_no_alloc: " + std::to_string(depth) + " slices of " + std::to_string(m) + "x" +
                         std::to_string(n) + " partial sums need " + std::to_string(need) + " bytes of scratch, the built-in array holds " +
                         std::to_string(static_cast<unsigned long long>(MCD_NO_ALLOC_SCRATCH_BYTES)) +
                         " (use fewer splits, or mcd_gemm with a workspace of your own)");
    }
    float* scratch = nullptr;
    if (int rc = scratch_for_current_device(&scratch)) return rc;

    auto s = static_cast<cudaStream_t>(stream);
    const bool vec = aligned16(a) && aligned16(b) && aligned16(c) && k % 4 == 0 && n % 4 == 0;
    const dim3 grid((n + MC_F32_BN - 1) / MC_F32_BN, (m + MC_F32_BM - 1) / MC_F32_BM, depth);
    McEpilogueArgs epi;
    for (int i = 0; i < 6; ++i) epi.p[i] = nullptr;
    // Every partial sum of every slice is written before the reduction reads it, so nothing in
    // the scratch has to start at zero; what the previous call left there is simply overwritten.
    if (vec) {
        mc_na_gemm_f32_vec<<<grid, 256, 0, s>>>(a, b, c, nullptr, 0, m, n, k, k, n, n, 0, k_per_split, scratch, epi);
    } else {
        mc_na_gemm_f32_any<<<grid, 256, 0, s>>>(a, b, c, nullptr, 0, m, n, k, k, n, n, 0, k_per_split, scratch, epi);
    }
    mcd::g_launches.fetch_add(1, std::memory_order_relaxed);
    if (int rc = mcd::check_rt(cudaGetLastError(), "mc_na_gemm_f32")) return rc;
    if (depth == 1) return 0;

    const long long count = static_cast<long long>(m) * n;
    const long long items = (n % 4 == 0) ? count / 4 : count;
    long long blocks = (items + 255) / 256;
    if (blocks > 8 * 148) blocks = 8 * 148;
    if (blocks < 1) blocks = 1;
    mc_na_splitk_reduce<<<static_cast<unsigned>(blocks), 256, 0, s>>>(scratch, c, nullptr, 0, m, n, n, 0, depth, epi);
    mcd::g_launches.fetch_add(1, std::memory_order_relaxed);
    return mcd::check_rt(cudaGetLastError(), "mc_na_splitk_reduce");
}
