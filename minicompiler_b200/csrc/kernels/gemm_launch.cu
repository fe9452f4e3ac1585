// Device layer, part 2: the ahead-of-time compiled kernels (identity epilogue)
// and the host launchers behind mcd_gemm / mcd_cast_f32_to_half / mcd_transpose_f32.
// The kernel bodies live in the .cuh files next to this one; the very same text
// is embedded in the library (mcd_gemm_source) so that a fused epilogue can be
// compiled in front of it at run time.

#include "minicompiler_b200_device.h"

#include "device/driver_api.hpp"
#include "device/per_device.hpp"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>

#include "kernels/epilogue.cuh"
#include "kernels/async_copy.cuh"
#include "kernels/gemm_f32_simt.cuh"
#include "kernels/gemm_tcgen05.cuh"
#include "kernels/gemm_tcgen05_2cta.cuh"
#include "kernels/splitk_reduce.cuh"

namespace mcd {
extern std::atomic<unsigned long long> g_launches;
extern const char* const kSourceEpilogue;
extern const char* const kSourceAsyncCopy;
extern const char* const kSourceGemmF32;
extern const char* const kSourceGemmTc;
extern const char* const kSourceGemmTc2;
extern const char* const kSourceSplitkReduce;
}  // namespace mcd

using namespace mcd;

// --------------------------------------------------------------- cast kernels

namespace {

// One 32x32 tile per block through shared memory, so both the read and the
// (possibly transposed) write are coalesced.
template <typename Out, bool kTranspose>
__global__ void __launch_bounds__(256) mc_cast_tile(const float* __restrict__ src, Out* __restrict__ dst, long long rows,
                                                    long long cols, long long src_pitch, long long dst_pitch, int kind) {
    __shared__ float tile[32][33];
    const long long tiles_c = (cols + 31) / 32;
    const long long tiles_r = (rows + 31) / 32;
    const int tx = threadIdx.x & 31;
    const int ty = threadIdx.x >> 5;  // 0..7
    for (long long t = blockIdx.x; t < tiles_r * tiles_c; t += gridDim.x) {
        const long long r0 = (t / tiles_c) * 32;
        const long long c0 = (t % tiles_c) * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long r = r0 + ty + 8 * i;
            const long long c = c0 + tx;
            tile[ty + 8 * i][tx] = (r < rows && c < cols) ? src[r * src_pitch + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (kTranspose) {
                const long long c = c0 + ty + 8 * i;  // becomes the row of dst
                const long long r = r0 + tx;
                if (c < cols && r < rows) {
                    const float v = tile[tx][ty + 8 * i];
                    if constexpr (sizeof(Out) == 2) {
                        dst[c * dst_pitch + r] = mc_to_half(v, kind);
                    } else {
                        dst[c * dst_pitch + r] = v;
                    }
                }
            } else {
                const long long r = r0 + ty + 8 * i;
                const long long c = c0 + tx;
                if (r < rows && c < cols) {
                    const float v = tile[ty + 8 * i][tx];
                    if constexpr (sizeof(Out) == 2) {
                        dst[r * dst_pitch + c] = mc_to_half(v, kind);
                    } else {
                        dst[r * dst_pitch + c] = v;
                    }
                }
            }
        }
        __syncthreads();
    }
}

// Dense, 8-aligned rows: 8 floats in, one 16-byte store out per thread-iteration.
__global__ void __launch_bounds__(256) mc_cast_rows_vec8(const float* __restrict__ src, unsigned short* __restrict__ dst,
                                                         long long rows, long long cols, long long src_pitch,
                                                         long long dst_pitch, int kind) {
    const long long groups_per_row = cols >> 3;
    const long long groups = rows * groups_per_row;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups; g += (long long)gridDim.x * blockDim.x) {
        const long long r = g / groups_per_row;
        const long long c = (g % groups_per_row) << 3;
        const float4 lo = __ldcs(reinterpret_cast<const float4*>(src + r * src_pitch + c));
        const float4 hi = __ldcs(reinterpret_cast<const float4*>(src + r * src_pitch + c + 4));
        uint4 pack;
        pack.x = mc_to_half2(lo.x, lo.y, kind);
        pack.y = mc_to_half2(lo.z, lo.w, kind);
        pack.z = mc_to_half2(hi.x, hi.y, kind);
        pack.w = mc_to_half2(hi.z, hi.w, kind);
        *reinterpret_cast<uint4*>(dst + r * dst_pitch + c) = pack;
    }
}

int sm_count_of_current_device() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    return sms;
}

int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return dev;
}

int launched(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return check_rt(cudaGetLastError(), what);
}

}  // namespace

extern "C" int mcd_cast_f32_to_half(int half_kind, const float* src, void* dst, long long rows, long long cols,
                                    long long src_pitch, long long dst_pitch, int transpose, void* stream) {
    if (half_kind != MCD_HALF_BF16 && half_kind != MCD_HALF_F16) return fail("mcd_cast_f32_to_half: unknown 16-bit format");
    if (rows <= 0 || cols <= 0) return 0;
    auto s = static_cast<cudaStream_t>(stream);
    auto* out = static_cast<unsigned short*>(dst);
    const int sms = sm_count_of_current_device();
    const bool vec = !transpose && cols % 8 == 0 && src_pitch % 4 == 0 && dst_pitch % 8 == 0 &&
                     (reinterpret_cast<std::uintptr_t>(src) & 15) == 0 && (reinterpret_cast<std::uintptr_t>(dst) & 15) == 0;
    if (vec) {
        const long long groups = rows * (cols / 8);
        const unsigned grid = static_cast<unsigned>(std::min<long long>((groups + 255) / 256, 8LL * sms));
        mc_cast_rows_vec8<<<grid, 256, 0, s>>>(src, out, rows, cols, src_pitch, dst_pitch, half_kind);
        return launched("mc_cast_rows_vec8");
    }
    const long long tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    const unsigned grid = static_cast<unsigned>(std::min<long long>(tiles, 16LL * sms));
    if (transpose) {
        mc_cast_tile<unsigned short, true><<<grid, 256, 0, s>>>(src, out, rows, cols, src_pitch, dst_pitch, half_kind);
    } else {
        mc_cast_tile<unsigned short, false><<<grid, 256, 0, s>>>(src, out, rows, cols, src_pitch, dst_pitch, half_kind);
    }
    return launched("mc_cast_tile");
}

extern "C" int mcd_transpose_f32(const float* src, float* dst, long long rows, long long cols, long long src_pitch,
                                 long long dst_pitch, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const long long tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    const unsigned grid = static_cast<unsigned>(std::min<long long>(tiles, 16LL * sm_count_of_current_device()));
    mc_cast_tile<float, true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst, rows, cols, src_pitch, dst_pitch, 0);
    return launched("mc_cast_tile<float>");
}

// ------------------------------------------------------------------ matmuls

namespace {

McEpilogueArgs epilogue_args(const mcd_gemm_args* a) {
    McEpilogueArgs e;
    for (int i = 0; i < 6; ++i) e.p[i] = i < a->num_epilogue_inputs ? a->epilogue_inputs[i] : nullptr;
    return e;
}

bool aligned16(const void* p) { return (reinterpret_cast<std::uintptr_t>(p) & 15) == 0; }

int reduce_splits(const mcd_gemm_args* a, int splits, cudaStream_t s) {
    McEpilogueArgs epi = epilogue_args(a);
    const long long count = static_cast<long long>(a->m) * a->n;
    const long long items = (a->n % 4 == 0) ? count / 4 : count;
    const unsigned grid = static_cast<unsigned>(
        std::max<long long>(1, std::min<long long>((items + 255) / 256, 8LL * sm_count_of_current_device())));
    const float* ws = a->workspace;
    float* c = a->c;
    auto* c16 = static_cast<unsigned short*>(a->c16);
    int kind = a->c16_kind, m = a->m, n = a->n;
    long long ldc = a->ldc, ldc16 = a->ldc16;
    // A programmatic dependent of the matmul launched just before it: its blocks take their places while the matmul
    // drains and wait (griddepcontrol.wait) until the partial sums are complete. Variant bit 2048: a plain launch.
    const bool dependent = (a->variant & 2048) == 0;
    if (a->reduce_function != nullptr) {
        void* params[] = {&ws, &c, &c16, &kind, &m, &n, &ldc, &ldc16, &splits, &epi};
        if (dependent) return mcd_launch_dependent(a->reduce_function, grid, 256, 0, s, params);
        return mcd_launch(a->reduce_function, grid, 1, 1, 256, 0, s, params);
    }
    if (dependent) {
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute.val.programmaticStreamSerializationAllowed = 1;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(grid, 1, 1);
        config.blockDim = dim3(256, 1, 1);
        config.stream = s;
        config.attrs = &attribute;
        config.numAttrs = 1;
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return check_rt(cudaLaunchKernelEx(&config, mc_splitk_reduce, ws, c, c16, kind, m, n, ldc, ldc16, splits, epi),
                        "cudaLaunchKernelEx(mc_splitk_reduce, dependent)");
    }
    mc_splitk_reduce<<<grid, 256, 0, s>>>(ws, c, c16, kind, m, n, ldc, ldc16, splits, epi);
    return launched("mc_splitk_reduce");
}

unsigned instruction_descriptor(int arith, bool b_is_k_major) {
    // c_format F32 (1) at bit 4; a/b formats at bits 7 and 10 (F16 0, BF16 1, TF32 2);
    // b_major at bit 16 (1 = MN-major); N >> 3 at bit 17; M >> 4 at bit 24.
    const unsigned fmt = arith == MCD_GEMM_F16 ? 0u : arith == MCD_GEMM_BF16 ? 1u : 2u;
    unsigned d = 0;
    d |= 1u << 4;
    d |= fmt << 7;
    d |= fmt << 10;
    d |= (b_is_k_major ? 0u : 1u) << 16;
    d |= static_cast<unsigned>(MC_TC_BN >> 3) << 17;
    d |= static_cast<unsigned>(MC_TC_BM >> 4) << 24;
    return d;
}

// cuTensorMapEncodeTiled is a pure function of its arguments, and an executable launches the same matmuls on the same
// arena addresses over and over: the encoded maps are kept, so a launch outside a replayed graph pays two look-ups
// instead of two driver calls (several microseconds, which shows on problems of 15 us).
struct MapKey {
    const void* base;
    unsigned long long inner, outer, pitch;
    unsigned box_inner, box_outer;
    int type, elem_bytes, swizzle;
    bool operator<(const MapKey& o) const {
        return std::tie(base, inner, outer, pitch, box_inner, box_outer, type, elem_bytes, swizzle) <
               std::tie(o.base, o.inner, o.outer, o.pitch, o.box_inner, o.box_outer, o.type, o.elem_bytes, o.swizzle);
    }
};
std::mutex g_map_mutex;
std::map<MapKey, CUtensorMap> g_map_cache;
std::atomic<unsigned long long> g_map_encodes{0};

int encode_map(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, unsigned long long inner,
               unsigned long long outer, unsigned long long pitch_elems, unsigned box_inner, unsigned box_outer,
               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    const MapKey key{base, inner, outer, pitch_elems, box_inner, box_outer, static_cast<int>(type), elem_bytes,
                     static_cast<int>(swizzle)};
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        const auto hit = g_map_cache.find(key);
        if (hit != g_map_cache.end()) {
            *map = hit->second;
            return 0;
        }
    }
    const DriverApi* drv = driver_api();
    if (drv == nullptr) return fail("the CUDA driver API is unavailable");
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {pitch_elems * static_cast<unsigned long long>(elem_bytes)};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t elem_strides[2] = {1, 1};
    if (int rc = check_drv(drv->TensorMapEncodeTiled(map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
                                                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE),
                           "cuTensorMapEncodeTiled")) {
        return rc;
    }
    g_map_encodes.fetch_add(1, std::memory_order_relaxed);
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_map_cache.size() >= 4096) g_map_cache.clear();  // a bound, not a policy: maps are cheap to make again
    g_map_cache.emplace(key, *map);
    return 0;
}

int f32_splits(const mcd_gemm_args* a, int* k_per_split) {
    int splits = std::max(1, a->splits);
    *k_per_split = ((a->k + splits - 1) / splits + MC_F32_BK - 1) / MC_F32_BK * MC_F32_BK;
    return (a->k + *k_per_split - 1) / *k_per_split;
}

// Whether the FP32 launch uses the TMA-fed kernel: operands a tensor map can describe (16-byte aligned bases, row
// pitches that are multiples of 4 floats), aligned outputs, and at least 512 of K per block - below that the ring's
// start-up costs more than it saves (256 x 2048 x 512 split 4 ways: 27.2 against 25.7 us; 4096^3: 55.7 against
// 52.0 TFLOP/s). Variant bit 512 keeps the register-staged kernel, bit 1024 takes the TMA-fed one whatever K is.
bool f32_uses_tma(const mcd_gemm_args* a) {
    if ((a->variant & 512) != 0) return false;
    int k_per_split = 0;
    const int splits = f32_splits(a, &k_per_split);
    if (k_per_split < 512 && (a->variant & 1024) == 0) return false;
    return aligned16(a->a) && aligned16(a->b) && (a->c == nullptr || aligned16(a->c)) && a->lda % 4 == 0 && a->ldb % 4 == 0 &&
           (splits == 1 || aligned16(a->workspace));
}

int gemm_f32(const mcd_gemm_args* a, cudaStream_t s) {
    if (a->b_transposed) return fail("mcd_gemm: the FP32 kernel reads B as [k,n]");
    int k_per_split = 0;
    const int splits = f32_splits(a, &k_per_split);
    if (splits > 1 && a->workspace == nullptr) return fail("mcd_gemm: a split matmul needs a workspace");
    const bool vec = aligned16(a->a) && aligned16(a->b) && (a->c == nullptr || aligned16(a->c)) && a->lda % 4 == 0 &&
                     a->ldb % 4 == 0 && (splits == 1 || aligned16(a->workspace));
    const dim3 grid((a->n + MC_F32_BN - 1) / MC_F32_BN, (a->m + MC_F32_BM - 1) / MC_F32_BM, splits);
    McEpilogueArgs epi = epilogue_args(a);
    const auto* pa = static_cast<const float*>(a->a);
    const auto* pb = static_cast<const float*>(a->b);
    float* pc = a->c;
    auto* pc16 = static_cast<unsigned short*>(a->c16);
    int kind = a->c16_kind, m = a->m, n = a->n, k = a->k;
    long long lda = a->lda, ldb = a->ldb, ldc = a->ldc, ldc16 = a->ldc16;
    float* ws = a->workspace;
    unsigned* status = a->status;
    if (f32_uses_tma(a)) {
        McTensorMap map_a, map_b;
        if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_a), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->a, a->k, a->m, a->lda,
                                MC_F32_BK, MC_F32_BM, CU_TENSOR_MAP_SWIZZLE_NONE)) {
            return rc;
        }
        if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_b), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->b, a->n, a->k, a->ldb,
                                MC_F32_BN, MC_F32_BK, CU_TENSOR_MAP_SWIZZLE_NONE)) {
            return rc;
        }
        if (a->function != nullptr && splits == 1) {
            void* params[] = {&map_a, &map_b, &pc, &pc16, &kind, &m, &n, &k, &ldc, &ldc16, &k_per_split, &ws, &status, &epi};
            return mcd_launch(a->function, grid.x, grid.y, grid.z, 256, MC_F32_TMA_SMEM_BYTES, s, params);
        }
        static PerDeviceOnce configured;
        const int device = current_device();
        if (configured.first_use(device)) {
            if (int rc = check_rt(cudaFuncSetAttribute(mc_gemm_f32_tma, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_F32_TMA_SMEM_BYTES),
                                  "cudaFuncSetAttribute(max dynamic shared memory)")) {
                configured.forget(device);
                return rc;
            }
        }
        mc_gemm_f32_tma<<<grid, 256, MC_F32_TMA_SMEM_BYTES, s>>>(map_a, map_b, pc, pc16, kind, m, n, k, ldc, ldc16, k_per_split, ws, status, epi);
        if (int rc = launched("mc_gemm_f32_tma")) return rc;
        if (splits > 1) return reduce_splits(a, splits, s);
        return 0;
    }
    if (a->function != nullptr && splits == 1) {
        // `function` is the entry point mcd_gemm_entry_point named for these arguments.
        void* params[] = {&pa, &pb, &pc, &pc16, &kind, &m, &n, &k, &lda, &ldb, &ldc, &ldc16, &k_per_split, &ws, &epi};
        return mcd_launch(a->function, grid.x, grid.y, grid.z, 256, 0, s, params);
    }
    if (vec) {
        mc_gemm_f32_vec<<<grid, 256, 0, s>>>(pa, pb, pc, pc16, kind, m, n, k, lda, ldb, ldc, ldc16, k_per_split, ws, epi);
    } else {
        mc_gemm_f32_any<<<grid, 256, 0, s>>>(pa, pb, pc, pc16, kind, m, n, k, lda, ldb, ldc, ldc16, k_per_split, ws, epi);
    }
    if (int rc = launched("mc_gemm_f32")) return rc;
    if (splits > 1) return reduce_splits(a, splits, s);
    return 0;
}

// K blocks and effective K splits of a tensor-core launch.
int tc_splits(const mcd_gemm_args* a) {
    const int block_k = a->arith == MCD_GEMM_TF32 ? 32 : 64;
    const int k_blocks = (a->k + block_k - 1) / block_k;
    int splits = std::max(1, std::min(a->splits, k_blocks));
    const int per = (k_blocks + splits - 1) / splits;
    return (k_blocks + per - 1) / per;
}

// Whether a split tensor-core launch adds its partial tiles inside thread-block clusters (one launch, no workspace):
// asked for with variant bit 64, for 2, 4 or 8 effective K splits of 256-column tiles. Off by default: measured on
// B200 it is no faster than the workspace and the second launch it saves (16 x 8192 x 8192 split 4 ways: 40.4 against
// 39.9 us; 128 x 8192 x 8192: 51.2 against 46.1 us; 1024 x 1024 x 65536: 122.9 against 117.8 us) - the two hand-shakes
// between the CTAs of a cluster cost about 3 us and the exchange through distributed shared memory the rest. The
// lowering mirrors this rule (tensor_core_cluster_reduce in lowering.cpp) to count launches and size the workspace.
bool tc_cluster_reduce(const mcd_gemm_args* a) {
    if (a->arith == MCD_GEMM_F32 || (a->variant & 64) == 0) return false;
    if (a->tile_n != 0 && a->tile_n != MC_TC_BN) return false;
    const int splits = tc_splits(a);
    return splits == 2 || splits == 4 || splits == 8;
}

// Whether the launch goes to the SM-pair kernel: unsplit problems with at least half a wave of 256 x 256 pair
// tiles (2048^3: 64 tiles on 74 pairs, 739 against 653 TFLOP/s); variant bit 8 forces it for any unsplit problem,
// bit 4 turns it off.
bool tc_uses_pairs(const mcd_gemm_args* a) {
    if (a->arith == MCD_GEMM_F32 || tc_splits(a) != 1 || (a->variant & 4) != 0) return false;
    if (a->tile_n != 0 && a->tile_n != MC_TC_BN) return false;
    if (a->arith == MCD_GEMM_TF32 && a->b_transposed == 0) return false;
    if ((a->variant & 8) != 0) return true;
    const long long tiles_m = (a->m + MC_TC_BM - 1) / MC_TC_BM;
    if (tiles_m % 2 != 0 && tiles_m < 9) return false;  // the odd row block's partner would idle
    const long long items = ((tiles_m + 1) / 2) * ((a->n + MC_TC_BN - 1) / MC_TC_BN);
    return 2 * items >= sm_count_of_current_device() / 2;  // from half a wave of pair tiles upwards
}

// Whether the SM-pair kernel takes two 256-column tiles per work item.
// That form saves a quarter of the operand traffic per flop, but the epilogue of an item's second tile is not
// overlapped with MMAs as well as in the one-tile form. Measured: without a fused epilogue it wins from 32 K blocks
// and one wave of items upwards; with one, only from 128 K blocks and two waves. Variant bit 16 forces it, bit 32
// turns it off.
bool tc_pair_wide(const mcd_gemm_args* a) {
    if ((a->variant & 32) != 0) return false;
    if ((a->variant & 16) != 0) return true;
    const int block_k = a->arith == MCD_GEMM_TF32 ? 32 : 64;
    const long long k_blocks = (a->k + block_k - 1) / block_k;
    const long long tiles_m = (a->m + MC_TC_BM - 1) / MC_TC_BM;
    const long long tiles_n = (a->n + MC_TC_BN - 1) / MC_TC_BN;
    const long long wide_tiles = ((tiles_m + 1) / 2) * ((tiles_n + 1) / 2);
    const long long clusters = sm_count_of_current_device() / 2;
    const bool fused = a->has_epilogue != 0;
    return fused ? (k_blocks >= 128 && wide_tiles >= 2 * clusters) : (k_blocks >= 32 && wide_tiles >= clusters);
}

int gemm_tc(const mcd_gemm_args* a, cudaStream_t s) {
    const bool tf32 = a->arith == MCD_GEMM_TF32;
    const int elem = tf32 ? 4 : 2;
    const int block_k = 128 / elem;
    const bool b_k_major = a->b_transposed != 0;
    if (!aligned16(a->a) || !aligned16(a->b) || (a->lda * elem) % 16 != 0 || (a->ldb * elem) % 16 != 0) {
        return fail("mcd_gemm: tensor-core operands need 16-byte aligned bases and row pitches");
    }
    if (tf32 && !b_k_major) return fail("mcd_gemm: TF32 reads B as a [n,k] copy only (set b_transposed)");
    const int tile_n = a->tile_n == 0 ? MC_TC_BN : a->tile_n;
    if (tile_n != 64 && tile_n != 128 && tile_n != MC_TC_BN) return fail("mcd_gemm: tile_n must be 0, 64, 128 or 256");
    const int k_blocks = (a->k + block_k - 1) / block_k;
    int splits = std::max(1, std::min(a->splits, k_blocks));
    const int per = (k_blocks + splits - 1) / splits;
    splits = (k_blocks + per - 1) / per;
    const bool cluster = tc_cluster_reduce(a);
    if (splits > 1 && !cluster && a->workspace == nullptr) return fail("mcd_gemm: a split matmul needs a workspace");

    CUtensorMapDataType type = tf32 ? ((a->variant & 1) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_TFLOAT32)
                               : a->arith == MCD_GEMM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                           : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    McTensorMap map_a, map_b;
    static_assert(sizeof(McTensorMap) == sizeof(CUtensorMap), "tensor map size");
    const bool pairs = tc_uses_pairs(a);
    // The one-CTA kernel stages only the rows a problem of fewer than 128 rows has (in whole groups of 8), and cuts
    // its ring out of the same shared memory: as many stages as fit, leaving room behind the last one for the 128
    // rows an MMA reads from wherever its A tile starts.
    const int a_rows = (!pairs && a->m < MC_TC_BM) ? (a->m + 7) / 8 * 8 : MC_TC_BM;
    if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_a), type, elem, a->a, a->k, a->m, a->lda, block_k,
                            static_cast<unsigned>(a_rows))) {
        return rc;
    }
    if (b_k_major) {
        // A CTA of the pair kernel keeps 128 of the tile's 256 columns.
        if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_b), type, elem, a->b, a->k, a->n, a->ldb, block_k,
                                pairs ? MC_TC_BN / 2 : tile_n)) {
            return rc;
        }
    } else {
        if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_b), type, elem, a->b, a->n, a->k, a->ldb, 128 / elem, block_k)) {
            return rc;
        }
    }

    McTcParams p;
    p.c = a->c;
    p.c16 = static_cast<unsigned short*>(a->c16);
    p.workspace = a->workspace;
    p.status = a->status;
    p.ldc = a->ldc;
    p.ldc16 = a->ldc16;
    p.c16_kind = a->c16_kind;
    p.m = a->m;
    p.n = a->n;
    p.k = a->k;
    p.idesc = instruction_descriptor(a->arith, b_k_major);
    p.idesc = (p.idesc & ~(0x3Fu << 17)) | (static_cast<unsigned>(tile_n >> 3) << 17);
    p.tile_n = tile_n;
    p.k_blocks_per_split = per;
    p.splits = splits;
    p.wide = 0;
    p.cluster_reduce = cluster ? splits : 0;
    p.staged = (a->variant & 128) == 0 ? 1 : 0;
    p.a_rows = a_rows;
    {
        const int stage_bytes = (a_rows + tile_n) * 128;
        const int room = MC_TC_STAGES * MC_TC_STAGE_BYTES - (MC_TC_BM - a_rows) * 128;
        p.stages = std::max(2, std::min(MC_TC_MAX_STAGES, room / stage_bytes));
    }
    // Tiles that do not fill the last wave of CTAs are cut in two when both halves of all of them fit in one wave.
    const int sms = sm_count_of_current_device();
    const int all_tiles = ((a->m + MC_TC_BM - 1) / MC_TC_BM) * ((a->n + tile_n - 1) / tile_n);
    const int tail = all_tiles % sms;
    p.half_tiles = (splits == 1 && tile_n == MC_TC_BN && (a->variant & 2) == 0 && tail > 0 && 2 * tail <= sms) ? tail : 0;
    McEpilogueArgs epi = epilogue_args(a);

    if (pairs) {
        p.idesc = (p.idesc & ~(0x1Fu << 24)) | (static_cast<unsigned>(2 * MC_TC_BM >> 4) << 24);  // M = 256 over the pair
        const int tiles_m = (a->m + MC_TC_BM - 1) / MC_TC_BM;
        const int tiles_n = (a->n + MC_TC_BN - 1) / MC_TC_BN;
        p.wide = tc_pair_wide(a) ? 1 : 0;
        const int pair_tiles = ((tiles_m + 1) / 2) * (p.wide ? (tiles_n + 1) / 2 : tiles_n);
        const int clusters = sms / 2;
        const int pair_tail = pair_tiles % clusters;
        p.half_tiles = ((a->variant & 2) == 0 && pair_tail > 0 && 2 * pair_tail <= clusters) ? pair_tail : 0;
        const int items = pair_tiles + p.half_tiles;
        const unsigned pair_grid = 2u * static_cast<unsigned>(std::max(1, std::min(items, clusters)));
        // Outputs leave as TMA stores of 32 x 32 boxes out of each warp's staging buffer (128-byte rows of FP32 with the
        // 128-byte swizzle, 64-byte rows of 16-bit values with the 64-byte swizzle) when a tensor map can describe them:
        // 16-byte aligned bases and row pitches. Otherwise the kernel stores directly from registers.
        McTensorMap map_c, map_c16;
        std::memset(&map_c, 0, sizeof(map_c));
        std::memset(&map_c16, 0, sizeof(map_c16));
        const bool c_ok = a->c == nullptr || (aligned16(a->c) && a->ldc % 4 == 0);
        const bool c16_ok = a->c16 == nullptr || (aligned16(a->c16) && a->ldc16 % 8 == 0);
        if (p.staged != 0 && c_ok && c16_ok) {
            if (a->c != nullptr) {
                if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_c), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->c, a->n, a->m,
                                        a->ldc, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
                    return rc;
                }
            }
            if (a->c16 != nullptr) {
                if (int rc = encode_map(reinterpret_cast<CUtensorMap*>(&map_c16), CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, a->c16, a->n,
                                        a->m, a->ldc16, 32, 32, CU_TENSOR_MAP_SWIZZLE_64B)) {
                    return rc;
                }
            }
        } else {
            p.staged = 0;
        }
        // The pair kernels are launched as programmatic dependents of whatever precedes them in the stream: their CTAs
        // may start on SMs the previous grid has left (it says so early if it is one of these kernels; any other kernel
        // does by ending) and wait for that grid to complete before they touch global memory. Variant bit 32768: plain.
        const bool dependent = (a->variant & 32768) == 0;
        if (a->function != nullptr) {
            void* params[] = {&map_a, &map_b, &map_c, &map_c16, &p, &epi};
            if (dependent) return mcd_launch_dependent(a->function, pair_grid, MC_TC_THREADS, MC_TC2_SMEM_BYTES, s, params);
            return mcd_launch(a->function, pair_grid, 1, 1, MC_TC_THREADS, MC_TC2_SMEM_BYTES, s, params);
        }
        using PairKernel = void (*)(const McTensorMap, const McTensorMap, const McTensorMap, const McTensorMap, const McTcParams,
                                    const McEpilogueArgs);
        PairKernel kernel = p.wide ? (tf32 ? mc_gemm_tc2w_tf32_bk : (b_k_major ? mc_gemm_tc2w_h16_bk : mc_gemm_tc2w_h16_bmn))
                                   : (tf32 ? mc_gemm_tc2_tf32_bk : (b_k_major ? mc_gemm_tc2_h16_bk : mc_gemm_tc2_h16_bmn));
        // The opt-in to more than 48 KB of dynamic shared memory is kept per device.
        static PerDeviceOnce pair_configured;
        const int device = current_device();
        if (pair_configured.first_use(device)) {
            for (PairKernel kfn : {mc_gemm_tc2_tf32_bk, mc_gemm_tc2_h16_bk, mc_gemm_tc2_h16_bmn, mc_gemm_tc2w_tf32_bk,
                                   mc_gemm_tc2w_h16_bk, mc_gemm_tc2w_h16_bmn}) {
                if (int rc = check_rt(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_TC2_SMEM_BYTES),
                                      "cudaFuncSetAttribute(max dynamic shared memory)")) {
                    pair_configured.forget(device);
                    return rc;
                }
            }
        }
        if (dependent) {
            cudaLaunchAttribute attribute;
            attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attribute.val.programmaticStreamSerializationAllowed = 1;
            cudaLaunchConfig_t config = {};
            config.gridDim = dim3(pair_grid, 1, 1);
            config.blockDim = dim3(MC_TC_THREADS, 1, 1);
            config.dynamicSmemBytes = MC_TC2_SMEM_BYTES;
            config.stream = s;
            config.attrs = &attribute;
            config.numAttrs = 1;
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return check_rt(cudaLaunchKernelEx(&config, kernel, map_a, map_b, map_c, map_c16, p, epi),
                            "cudaLaunchKernelEx(mc_gemm_tc2, dependent)");
        }
        kernel<<<pair_grid, MC_TC_THREADS, MC_TC2_SMEM_BYTES, s>>>(map_a, map_b, map_c, map_c16, p, epi);
        return launched("mc_gemm_tc2");
    }

    const int tiles = (all_tiles + p.half_tiles) * splits;
    const unsigned grid = static_cast<unsigned>(std::max(1, std::min(tiles, sms)));

    if (a->function != nullptr && cluster) {
        // One CTA per (tile, K slice); the slices of a tile are consecutive block indices, hence one cluster.
        void* params[] = {&map_a, &map_b, &p, &epi};
        return mcd_launch_cluster(a->function, static_cast<unsigned>(tiles), static_cast<unsigned>(splits), MC_TC_THREADS,
                                  MC_TC_SMEM_BYTES, s, params);
    }
    if (a->function != nullptr && splits == 1) {
        void* params[] = {&map_a, &map_b, &p, &epi};
        return mcd_launch(a->function, grid, 1, 1, MC_TC_THREADS, MC_TC_SMEM_BYTES, s, params);
    }
    using Kernel = void (*)(const McTensorMap, const McTensorMap, const McTcParams, const McEpilogueArgs);
    Kernel kernel = tf32 ? (b_k_major ? mc_gemm_tc_tf32_bk : mc_gemm_tc_tf32_bmn)
                         : (b_k_major ? mc_gemm_tc_h16_bk : mc_gemm_tc_h16_bmn);
    static PerDeviceOnce configured;
    const int device = current_device();
    if (configured.first_use(device)) {
        for (Kernel kfn : {mc_gemm_tc_tf32_bk, mc_gemm_tc_tf32_bmn, mc_gemm_tc_h16_bk, mc_gemm_tc_h16_bmn}) {
            if (int rc = check_rt(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_TC_SMEM_BYTES),
                                  "cudaFuncSetAttribute(max dynamic shared memory)")) {
                configured.forget(device);
                return rc;
            }
        }
    }
    if (cluster) {
        cudaLaunchAttribute attribute;
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = static_cast<unsigned>(splits);
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(static_cast<unsigned>(tiles), 1, 1);
        config.blockDim = dim3(MC_TC_THREADS, 1, 1);
        config.dynamicSmemBytes = MC_TC_SMEM_BYTES;
        config.stream = s;
        config.attrs = &attribute;
        config.numAttrs = 1;
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return check_rt(cudaLaunchKernelEx(&config, kernel, map_a, map_b, p, epi), "cudaLaunchKernelEx(mc_gemm_tc, cluster)");
    }
    kernel<<<grid, MC_TC_THREADS, MC_TC_SMEM_BYTES, s>>>(map_a, map_b, p, epi);
    if (int rc = launched("mc_gemm_tc")) return rc;
    if (splits > 1) return reduce_splits(a, splits, s);
    return 0;
}

}  // namespace

extern "C" int mcd_gemm(const mcd_gemm_args* args, void* stream) {
    if (args == nullptr) return fail("mcd_gemm: null arguments");
    if (args->m <= 0 || args->n <= 0 || args->k <= 0) return fail("mcd_gemm: empty problem");
    if (args->c == nullptr && args->c16 == nullptr) return fail("mcd_gemm: no output buffer");
    if (args->num_epilogue_inputs < 0 || args->num_epilogue_inputs > MCD_MAX_EPILOGUE_INPUTS) {
        return fail("mcd_gemm: too many epilogue inputs");
    }
    auto s = static_cast<cudaStream_t>(stream);
    switch (args->arith) {
        case MCD_GEMM_F32: return gemm_f32(args, s);
        case MCD_GEMM_TF32:
        case MCD_GEMM_BF16:
        case MCD_GEMM_F16: return gemm_tc(args, s);
        default: return fail("mcd_gemm: unknown arithmetic");
    }
}

extern "C" int mcd_gemm_launches(const mcd_gemm_args* a) {
    if (a->arith == MCD_GEMM_F32) {
        int k_per_split = 0;
        return f32_splits(a, &k_per_split) > 1 ? 2 : 1;
    }
    if (tc_cluster_reduce(a)) return 1;
    return tc_splits(a) > 1 ? 2 : 1;
}

extern "C" const char* mcd_gemm_source(int arith) {
    static const std::string f32 = std::string(kSourceEpilogue) + kSourceAsyncCopy + kSourceGemmF32;
    static const std::string tc = std::string(kSourceEpilogue) + kSourceAsyncCopy + kSourceGemmTc + kSourceGemmTc2;
    static const std::string reduce = std::string(kSourceEpilogue) + kSourceSplitkReduce;
    if (arith == MCD_GEMM_F32) return f32.c_str();
    if (arith < 0) return reduce.c_str();
    return tc.c_str();
}

extern "C" const char* mcd_gemm_entry_point(const mcd_gemm_args* a) {
    if (a == nullptr) return "mc_splitk_reduce";
    if (a->arith == MCD_GEMM_F32) {
        const bool vec = aligned16(a->a) && aligned16(a->b) && (a->c == nullptr || aligned16(a->c)) && a->lda % 4 == 0 &&
                         a->ldb % 4 == 0;
        if (f32_uses_tma(a)) return "mc_gemm_f32_tma";
        return vec ? "mc_gemm_f32_vec" : "mc_gemm_f32_any";
    }
    if (tc_uses_pairs(a)) {
        if (tc_pair_wide(a)) {
            if (a->arith == MCD_GEMM_TF32) return "mc_gemm_tc2w_tf32_bk";
            return a->b_transposed ? "mc_gemm_tc2w_h16_bk" : "mc_gemm_tc2w_h16_bmn";
        }
        if (a->arith == MCD_GEMM_TF32) return "mc_gemm_tc2_tf32_bk";
        return a->b_transposed ? "mc_gemm_tc2_h16_bk" : "mc_gemm_tc2_h16_bmn";
    }
    if (a->arith == MCD_GEMM_TF32) return a->b_transposed ? "mc_gemm_tc_tf32_bk" : "mc_gemm_tc_tf32_bmn";
    return a->b_transposed ? "mc_gemm_tc_h16_bk" : "mc_gemm_tc_h16_bmn";
}

extern "C" size_t mcd_gemm_dynamic_smem(int arith) {
    static_assert(MC_TC2_SMEM_BYTES >= MC_TC_SMEM_BYTES, "the pair kernels set the limit of both tensor-core families");
    static_assert(MC_TC2_SMEM_BYTES + 64 <= 227 * 1024, "dynamic plus static shared memory of the pair kernel");
    if (arith == MCD_GEMM_F32) return MC_F32_TMA_SMEM_BYTES;  // the TMA-fed kernel's ring; harmless for the others
    return (arith == MCD_GEMM_TF32 || arith == MCD_GEMM_BF16 || arith == MCD_GEMM_F16) ? MC_TC2_SMEM_BYTES : 0;
}

extern "C" int mcd_gemm_max_active_clusters(int arith, int b_transposed, int cluster_size, int* clusters) {
    using Kernel = void (*)(const McTensorMap, const McTensorMap, const McTcParams, const McEpilogueArgs);
    const bool tf32 = arith == MCD_GEMM_TF32;
    Kernel kernel = tf32 ? (b_transposed ? mc_gemm_tc_tf32_bk : mc_gemm_tc_tf32_bmn) : (b_transposed ? mc_gemm_tc_h16_bk : mc_gemm_tc_h16_bmn);
    if (int rc = check_rt(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, MC_TC_SMEM_BYTES),
                          "cudaFuncSetAttribute(max dynamic shared memory)")) {
        return rc;
    }
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeClusterDimension;
    attribute.val.clusterDim.x = static_cast<unsigned>(cluster_size);
    attribute.val.clusterDim.y = 1;
    attribute.val.clusterDim.z = 1;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(cluster_size) * 64, 1, 1);
    config.blockDim = dim3(MC_TC_THREADS, 1, 1);
    config.dynamicSmemBytes = MC_TC_SMEM_BYTES;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return check_rt(cudaOccupancyMaxActiveClusters(clusters, kernel, &config), "cudaOccupancyMaxActiveClusters");
}

extern "C" int mcd_per_device_once_probe(const int* devices, int count, int* first) {
    PerDeviceOnce flag;
    for (int i = 0; i < count; ++i) first[i] = flag.first_use(devices[i]) ? 1 : 0;
    return 0;
}

extern "C" int mcd_tensor_core_supported(int device, int arith) {
    (void)arith;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return major == 10 ? 1 : 0;
}
