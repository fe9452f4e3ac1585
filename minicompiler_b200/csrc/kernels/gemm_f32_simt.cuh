// FP32 SIMT matmul, the exact path: C[m,n] = epilogue(A[m,k] * B[k,n]) with FP32
// FMA accumulation, any m, n, k. It stands where the reference's FP32 ladder and
// its split-K variant stood (src/cuda/matmul_kernels.cu:244-288, :292-315).
//
// One 256-thread block owns a 128x128 tile of C and walks K in steps of 16.
// A is staged transposed (k-major) so that both operands are read from shared
// memory as 128-bit vectors; each thread keeps an 8x8 block of accumulators laid
// out as 2x2 quads of 4x4, and the next K step's global loads are in registers
// while the current one is multiplied. With gridDim.z > 1 each z-slice covers
// `k_per_split` of K and writes raw partial sums to `workspace[z][m][n]`; the
// reduction kernel adds them in slice order and applies the epilogue, so the
// result never depends on block scheduling.

#define MC_F32_BM 128
#define MC_F32_BN 128
#define MC_F32_BK 16
#define MC_F32_APITCH 132

// Two IEEE FP32 fused multiply-adds in one instruction (sm_100: fma.rn.f32x2 on register pairs). Each half is
// rounded exactly like fmaf, so results are bit-identical to the scalar form; what changes is that a warp issues
// half as many FMA instructions, which leaves issue slots for the shared-memory loads beside them.
__device__ __forceinline__ unsigned long long mc_pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void mc_unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void mc_fma2(unsigned long long& acc, unsigned long long a, unsigned long long b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// The thread's 8x8 block of finished sums: epilogue and stores (or raw partial sums when K is split).
template <bool kVec>
__device__ __forceinline__ void mc_gemm_f32_finish(const float (&acc)[8][8], int m0, int n0, int ty, int tx, float* __restrict__ C,
                                                   unsigned short* __restrict__ C16, int c16_kind, int M, int N, long long ldc,
                                                   long long ldc16, float* __restrict__ workspace, const McEpilogueArgs& epi) {
    const bool partial = gridDim.z > 1;
    float* dst = partial ? workspace + (long long)blockIdx.z * M * N : C;
    const long long ld = partial ? (long long)N : ldc;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int row = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (row >= M) continue;
#pragma unroll
        for (int jh = 0; jh < 2; ++jh) {
            const int col = n0 + jh * 64 + tx * 4;
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                v[j] = acc[i][jh * 4 + j];
                if (!partial && col + j < N) v[j] = mc_epilogue(v[j], (unsigned)row, (unsigned)(col + j), epi);
            }
            if (dst != nullptr) {
                float* out = dst + (long long)row * ld + col;
                if (kVec && col + 3 < N && (ld & 3) == 0) {
                    *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (col + j < N) out[j] = v[j];
                    }
                }
            }
            if (!partial && C16 != nullptr) {
                unsigned short* out16 = C16 + (long long)row * ldc16 + col;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (col + j < N) out16[j] = mc_to_half(v[j], c16_kind);
                }
            }
        }
    }
}

template <bool kVec>
__device__ __forceinline__ void mc_gemm_f32_body(const float* __restrict__ A, const float* __restrict__ B,
                                                 float* __restrict__ C, unsigned short* __restrict__ C16, int c16_kind,
                                                 int M, int N, int K, long long lda, long long ldb, long long ldc,
                                                 long long ldc16, int k_per_split, float* __restrict__ workspace,
                                                 const McEpilogueArgs& epi) {
    __shared__ __align__(16) float As[2][MC_F32_BK][MC_F32_APITCH];
    __shared__ __align__(16) float Bs[2][MC_F32_BK][MC_F32_BN];

    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * MC_F32_BM;
    const int n0 = blockIdx.x * MC_F32_BN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    // With K split, the reduction kernel that follows may take its places while this grid drains (it waits for this
    // grid to complete before it reads the partial sums).
    if (gridDim.z > 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // Global -> register staging coordinates.
    // 0..63 (and +64). The two upper k-groups of a lane quad take the row 8 further on, so that the transposed
    // stores of a warp (k-groups 16 banks apart at pitch 132) fall on 32 different banks.
    const int a_row = (tid >> 2) ^ ((tid & 2) << 2);
    const int a_k = (tid & 3) << 2;    // 0,4,8,12
    const int b_k = tid >> 5;          // 0..7 (and +8)
    const int b_n = (tid & 31) << 2;   // 0..124

    float4 a_stage[2];
    float4 b_stage[2];

    auto fetch = [&](int k0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = m0 + a_row + h * 64;
            const int kk = k0 + a_k;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < M) {
                const float* src = A + (long long)row * lda + kk;
                if (kVec && kk + 3 < k_end) {
                    v = *reinterpret_cast<const float4*>(src);
                } else {
                    if (kk + 0 < k_end) v.x = src[0];
                    if (kk + 1 < k_end) v.y = src[1];
                    if (kk + 2 < k_end) v.z = src[2];
                    if (kk + 3 < k_end) v.w = src[3];
                }
            }
            a_stage[h] = v;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int kk = k0 + b_k + h * 8;
            const int col = n0 + b_n;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (kk < k_end) {
                const float* src = B + (long long)kk * ldb + col;
                if (kVec && col + 3 < N) {
                    v = *reinterpret_cast<const float4*>(src);
                } else {
                    if (col + 0 < N) v.x = src[0];
                    if (col + 1 < N) v.y = src[1];
                    if (col + 2 < N) v.z = src[2];
                    if (col + 3 < N) v.w = src[3];
                }
            }
            b_stage[h] = v;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = a_row + h * 64;
            As[buf][a_k + 0][row] = a_stage[h].x;
            As[buf][a_k + 1][row] = a_stage[h].y;
            As[buf][a_k + 2][row] = a_stage[h].z;
            As[buf][a_k + 3][row] = a_stage[h].w;
            *reinterpret_cast<float4*>(&Bs[buf][b_k + h * 8][b_n]) = b_stage[h];
        }
    };

    const int ty = tid >> 4;  // 0..15 -> rows ty*4 and 64 + ty*4
    const int tx = tid & 15;  // 0..15 -> cols tx*4 and 64 + tx*4
    // acc2[i][p] holds columns 2p and 2p+1 of row i of the thread's 8x8 block.
    unsigned long long acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int p = 0; p < 4; ++p) acc2[i][p] = 0ull;  // two +0.0f
    }

    const int steps = (k_end - k_begin + MC_F32_BK - 1) / MC_F32_BK;
    if (steps > 0) {
        fetch(k_begin);
        stash(0);
    }
    __syncthreads();
    for (int s = 0; s < steps; ++s) {
        const int buf = s & 1;
        if (s + 1 < steps) fetch(k_begin + (s + 1) * MC_F32_BK);
#pragma unroll
        for (int kk = 0; kk < MC_F32_BK; ++kk) {
            const float4 a_lo = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 4]);
            const float4 a_hi = *reinterpret_cast<const float4*>(&As[buf][kk][64 + ty * 4]);
            const float4 b_lo = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
            const float4 b_hi = *reinterpret_cast<const float4*>(&Bs[buf][kk][64 + tx * 4]);
            const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
            const unsigned long long b2[4] = {mc_pack2(b_lo.x, b_lo.y), mc_pack2(b_lo.z, b_lo.w), mc_pack2(b_hi.x, b_hi.y),
                                              mc_pack2(b_hi.z, b_hi.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned long long a2 = mc_pack2(a[i], a[i]);
#pragma unroll
                for (int p = 0; p < 4; ++p) mc_fma2(acc2[i][p], a2, b2[p]);
            }
        }
        if (s + 1 < steps) stash(buf ^ 1);
        __syncthreads();
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int p = 0; p < 4; ++p) mc_unpack2(acc2[i][p], acc[i][2 * p], acc[i][2 * p + 1]);
    }

    mc_gemm_f32_finish<kVec>(acc, m0, n0, ty, tx, C, C16, c16_kind, M, N, ldc, ldc16, workspace, epi);
}

// kVec: A, B, C (and the workspace) are 16-byte aligned and lda, ldb are multiples of 4.
extern "C" __global__ void __launch_bounds__(256, 2)
mc_gemm_f32_vec(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                unsigned short* __restrict__ C16, int c16_kind, int M, int N, int K, long long lda, long long ldb,
                long long ldc, long long ldc16, int k_per_split, float* __restrict__ workspace, McEpilogueArgs epi) {
    mc_gemm_f32_body<true>(A, B, C, C16, c16_kind, M, N, K, lda, ldb, ldc, ldc16, k_per_split, workspace, epi);
}

extern "C" __global__ void __launch_bounds__(256, 2)
mc_gemm_f32_any(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                unsigned short* __restrict__ C16, int c16_kind, int M, int N, int K, long long lda, long long ldb,
                long long ldc, long long ldc16, int k_per_split, float* __restrict__ workspace, McEpilogueArgs epi) {
    mc_gemm_f32_body<false>(A, B, C, C16, c16_kind, M, N, K, lda, ldb, ldc, ldc16, k_per_split, workspace, epi);
}

#ifndef MC_F32_NO_TMA_KERNEL
// The same tile and the same arithmetic, fed by TMA: when A and B can be described by tensor maps (16-byte aligned,
// row pitches multiples of 4 floats) one elected thread keeps a 4-stage ring of 128 x 16 A tiles and 16 x 128 B tiles
// filled with cp.async.bulk.tensor (no multicast; TMA zero-fills the ragged edges of M, N and K, so the main loop has
// no bounds checks), stages change hands through mbarriers, and the FMA warps neither stage operands through
// registers nor meet at a block-wide barrier per K step. A stays row-major in shared memory (k contiguous): a thread
// reads four K values of a row with one 128-bit load. Every output is accumulated over K in the same order as in the
// register-staged kernel, so the two agree bit for bit. Waits are bounded like those of the tensor-core kernels.
#define MC_F32_STAGES 4
#define MC_F32_A_BYTES (MC_F32_BM * MC_F32_BK * 4)
#define MC_F32_B_BYTES (MC_F32_BK * MC_F32_BN * 4)
#define MC_F32_STAGE_BYTES (MC_F32_A_BYTES + MC_F32_B_BYTES)
#define MC_F32_TMA_SMEM_BYTES (MC_F32_STAGES * MC_F32_STAGE_BYTES + 128)
#define MC_F32_ERR_WAIT 0x20u

extern "C" __global__ void __launch_bounds__(256, 2)
mc_gemm_f32_tma(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b, float* __restrict__ C,
                unsigned short* __restrict__ C16, int c16_kind, int M, int N, int K, long long ldc, long long ldc16,
                int k_per_split, float* __restrict__ workspace, unsigned* status, McEpilogueArgs epi) {
    extern __shared__ unsigned char mc_f32_smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * MC_F32_STAGES];
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;
    const unsigned ring = (mc_smem_addr(mc_f32_smem_raw) + 127u) & ~127u;
    const unsigned bar_full = mc_smem_addr(bars);
    const unsigned bar_empty = bar_full + 8 * MC_F32_STAGES;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int m0 = blockIdx.y * MC_F32_BM;
    const int n0 = blockIdx.x * MC_F32_BN;
    const int k_begin = blockIdx.z * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    const int steps = (k_end - k_begin + MC_F32_BK - 1) / MC_F32_BK;
    if (gridDim.z > 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (tid == 0) {
        abort_flag_storage = 0;
        for (int s = 0; s < MC_F32_STAGES; ++s) {
            mc_mbar_init(bar_full + 8 * s, 1);
            mc_mbar_init(bar_empty + 8 * s, 8);  // one arrival per warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    auto fill = [&](int step) {  // thread 0 only
        const int stage = step % MC_F32_STAGES;
        const unsigned full = bar_full + 8 * stage;
        const unsigned dst = ring + stage * MC_F32_STAGE_BYTES;
        const int k0 = k_begin + step * MC_F32_BK;
        mc_mbar_expect_tx(full, MC_F32_STAGE_BYTES);
        mc_tma_load_2d(dst, &map_a, full, k0, m0);
        mc_tma_load_2d(dst + MC_F32_A_BYTES, &map_b, full, n0, k0);
    };
    int issued = 0;
    if (tid == 0) {
        for (; issued < steps && issued < MC_F32_STAGES; ++issued) fill(issued);
    }

    const int ty = tid >> 4;  // 0..15 -> rows ty*4 and 64 + ty*4
    const int tx = tid & 15;  // 0..15 -> cols tx*4 and 64 + tx*4
    unsigned long long acc2[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int p = 0; p < 4; ++p) acc2[i][p] = 0ull;
    }

    bool ok = true;
    int s = 0;
    for (; s < steps; ++s) {
        const int stage = s % MC_F32_STAGES;
        const unsigned phase = (unsigned)(s / MC_F32_STAGES) & 1u;
        // The stage that every warp released one step ago is refilled now: by then the wait is all but over.
        if (tid == 0 && s >= 1 && issued < steps) {
            const int freed = (s - 1) % MC_F32_STAGES;
            if (mc_mbar_wait(bar_empty + 8 * freed, (unsigned)((s - 1) / MC_F32_STAGES) & 1u, abort_flag, status, MC_F32_ERR_WAIT)) {
                fill(issued);
                ++issued;
            }
        }
        ok = mc_mbar_wait(bar_full + 8 * stage, phase, abort_flag, status, MC_F32_ERR_WAIT);
        ok = __all_sync(0xffffffffu, ok);  // a warp leaves the loop as one
        if (!ok) break;
        const unsigned a_base = ring + stage * MC_F32_STAGE_BYTES;
        const float* As = static_cast<const float*>(__cvta_shared_to_generic(a_base));                    // [128][16]
        const float* Bs = static_cast<const float*>(__cvta_shared_to_generic(a_base + MC_F32_A_BYTES));   // [16][128]
#pragma unroll
        for (int k4 = 0; k4 < MC_F32_BK; k4 += 4) {
            float4 a4[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int row = (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
                a4[i] = *reinterpret_cast<const float4*>(As + row * MC_F32_BK + k4);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 b_lo = *reinterpret_cast<const float4*>(Bs + (k4 + kk) * MC_F32_BN + tx * 4);
                const float4 b_hi = *reinterpret_cast<const float4*>(Bs + (k4 + kk) * MC_F32_BN + 64 + tx * 4);
                const unsigned long long b2[4] = {mc_pack2(b_lo.x, b_lo.y), mc_pack2(b_lo.z, b_lo.w), mc_pack2(b_hi.x, b_hi.y),
                                                  mc_pack2(b_hi.z, b_hi.w)};
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float a = kk == 0 ? a4[i].x : kk == 1 ? a4[i].y : kk == 2 ? a4[i].z : a4[i].w;
                    const unsigned long long a2 = mc_pack2(a, a);
#pragma unroll
                    for (int p = 0; p < 4; ++p) mc_fma2(acc2[i][p], a2, b2[p]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mc_mbar_arrive(bar_empty + 8 * stage);
    }
    __syncthreads();  // every warp is past the loop, finished or given up
    if (*abort_flag != 0) {
        // Copies still in flight must land before this block's shared memory is released.
        if (tid == 0) {
            for (int step = s; step < issued; ++step) {
                const unsigned long long t0 = mc_globaltimer();
                while (!mc_mbar_try_wait(bar_full + 8 * (step % MC_F32_STAGES), (unsigned)(step / MC_F32_STAGES) & 1u)) {
                    if (mc_globaltimer() - t0 > MC_WAIT_NS / 4) break;
                }
            }
        }
        return;
    }

    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
#pragma unroll
        for (int p = 0; p < 4; ++p) mc_unpack2(acc2[i][p], acc[i][2 * p], acc[i][2 * p + 1]);
    }
    mc_gemm_f32_finish<true>(acc, m0, n0, ty, tx, C, C16, c16_kind, M, N, ldc, ldc16, workspace, epi);
}
#endif  // MC_F32_NO_TMA_KERNEL
