// Tensor-core matmul for sm_100a: C[m,n] = epilogue(A[m,k] * B[k,n]) with BF16,
// FP16 or TF32 multiplicands and FP32 accumulation. It stands where the
// reference's WMMA kernel stood (src/cuda/matmul_tensor_core.cu:96-222) and is
// built on the Blackwell execution model instead:
//
//   * one persistent CTA per SM walks (m-block, n-block, k-split) work items in
//     an order that keeps a wave of CTAs on a near-square patch of C, so A and B
//     tiles are shared through L2;
//   * warp 0 (one lane) is the TMA producer: per K block it brings a 128 x 128B
//     A tile and a 256-column B tile into 128B-swizzled shared memory through a
//     4-stage mbarrier ring (TMA zero-fills the ragged edges of M, N and K);
//   * warp 1 (one lane) issues tcgen05.mma (128 x 256 x 16 for 16-bit operands,
//     128 x 256 x 8 for TF32) from shared-memory descriptors into a TMEM
//     accumulator and releases each stage with tcgen05.commit;
//   * warps 2-9 drain the accumulator with tcgen05.ld (each warp owns 32 TMEM
//     lanes = 32 rows and one half of the columns), apply the fused epilogue and store C as FP32 and/or as a
//     16-bit copy for a downstream tensor-core matmul. TMEM holds two 256-column
//     accumulators, so the epilogue of one tile overlaps the main loop of the next.
//
// B is read either as stored by the graph ([k,n] row-major: "MN-major" operand,
// mc_gemm_tc_*_bmn) or from a [n,k] copy ("K-major", mc_gemm_tc_*_bk).
//
// Split K without a workspace (p.cluster_reduce = S in {2, 4, 8}): the S work items of a tile form a thread-block
// cluster, one K slice each. When every CTA of the cluster has finished its MMAs, each sends the S-th part of its
// partial tile that a peer owns into that peer's shared memory (distributed shared memory, st.shared::cluster,
// in the space the operand ring no longer needs); every CTA then adds the S partial sums of its columns in slice
// order, applies the epilogue and stores them. The partial sums never touch global memory, there is no second
// launch, and the order of the additions is that of the separate reduction kernel (bit-identical results).
//
// Every wait is bounded: a wait that exceeds MC_TC_WAIT_NS of wall time records
// MC_TC_ERR_* in *status, raises a CTA-wide abort flag and every role leaves its
// loop; the CTA then waits (bounded) for its TMA copies in flight, frees its
// TMEM and returns.

#define MC_TC_BM 128
#define MC_TC_BN 256
#define MC_TC_STAGES 4
#define MC_TC_EPILOGUE_WARPS 8
#define MC_TC_THREADS (64 + 32 * MC_TC_EPILOGUE_WARPS)
#define MC_TC_A_BYTES (MC_TC_BM * 128)
#define MC_TC_B_BYTES (MC_TC_BN * 128)
#define MC_TC_STAGE_BYTES (MC_TC_A_BYTES + MC_TC_B_BYTES)
#define MC_TC_MAX_STAGES 24  // the ring of the one-CTA kernel is cut at run time out of the same 4 x 48 KB (McTcParams.stages)
#define MC_TC_BARRIER_BYTES 512
#define MC_TC_SMEM_BYTES (MC_TC_STAGES * MC_TC_STAGE_BYTES + 1024 + MC_TC_BARRIER_BYTES)
#define MC_TC_WAIT_NS MC_WAIT_NS
#define MC_TC_RASTER 16

#define MC_TC_ERR_PRODUCER 0x1u
#define MC_TC_ERR_MMA 0x2u
#define MC_TC_ERR_EPILOGUE 0x4u
#define MC_TC_ERR_DRAIN 0x8u
#define MC_TC_ERR_CLUSTER 0x10u

struct McTcParams {
    float* c;
    unsigned short* c16;
    float* workspace;
    unsigned* status;
    long long ldc;
    long long ldc16;
    int c16_kind;
    int m, n, k;
    unsigned idesc;
    int k_blocks_per_split;  // K blocks (of 128 bytes) per work item
    int splits;
    int half_tiles;  // the last `half_tiles` tiles are each issued as two 128-column work items (splits == 1 only)
    int wide;        // SM-pair kernel only: two 256-column tiles per work item
    int staged;      // SM-pair kernel only: outputs leave through shared memory as whole row segments
    int tile_n;      // one-CTA kernel only: columns per tile, 256 (default), 128 or 64; narrow tiles let a small
                     // problem fill the SMs in one launch instead of splitting K (idesc carries the same N)
    int cluster_reduce;  // one-CTA kernel only: 0, or the K splits of a tile are the CTAs of a cluster of this size,
                         // which add their partial tiles through distributed shared memory (one work item per CTA)
    int stages;  // one-CTA kernel only: depth of the operand ring, 2 .. MC_TC_MAX_STAGES
    int a_rows;  // one-CTA kernel only: rows of A staged per K block (the box of A's tensor map), a multiple of 8 up to 128.
                 // A problem of fewer than 128 rows stages only its own rows: a stage shrinks to a_rows * 128 bytes of A
                 // plus tile_n * 128 bytes of B and the ring grows deeper by as much. The MMA still spans 128 rows; the
                 // rows past a_rows are whatever follows in shared memory and land in accumulator lanes nobody reads.
};

__device__ __forceinline__ unsigned mc_cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// The shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ unsigned mc_mapa(unsigned addr, unsigned rank) {
    unsigned out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}

__device__ __forceinline__ void mc_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mc_mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Arrive with release semantics at cluster scope: shared-memory writes to the barrier's CTA made before it (by
// threads ordered before the arriving one) are visible to a waiter that acquires at cluster scope.
__device__ __forceinline__ void mc_mbar_arrive_release_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// A non-blocking test: try_wait may put the thread to sleep until the phase completes or a system-chosen time limit
// passes, and an arrival from another CTA of the cluster did not end that sleep early (each such wait then cost
// several microseconds); the waits on cluster barriers therefore poll.
__device__ __forceinline__ bool mc_mbar_try_wait_cluster(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// mc_mbar_wait for a barrier that CTAs of the cluster arrive on.
__device__ __forceinline__ bool mc_mbar_wait_cluster(unsigned bar, unsigned parity, volatile int* abort_flag, unsigned* status,
                                                     unsigned err_code) {
    if (mc_mbar_try_wait_cluster(bar, parity)) return true;
    const unsigned long long t0 = mc_globaltimer();
    unsigned spins = 0;
    while (!mc_mbar_try_wait_cluster(bar, parity)) {
        if ((++spins & 255u) == 0u) {
            if (*abort_flag != 0) return false;
            if (mc_globaltimer() - t0 > MC_TC_WAIT_NS) {
                if (status != nullptr) atomicOr(status, err_code);
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void mc_st_cluster_v4(unsigned cluster_addr, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ float mc_ld_shared_f32(unsigned addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void mc_umma(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b,
                                        unsigned idesc, unsigned accumulate, bool tf32) {
    if (tf32) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

__device__ __forceinline__ void mc_umma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mc_tmem_load32(unsigned taddr, unsigned (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}

// Shared-memory operand descriptor, 128-byte swizzle (layout type 2, descriptor version 1).
__device__ __forceinline__ unsigned long long mc_smem_desc(unsigned addr, unsigned leading_bytes, unsigned stride_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((addr & 0x3FFFFu) >> 4);
    d |= (unsigned long long)((leading_bytes >> 4) & 0x3FFFu) << 16;
    d |= (unsigned long long)((stride_bytes >> 4) & 0x3FFFu) << 32;
    d |= 1ull << 46;
    d |= 2ull << 61;
    return d;
}

// Work item -> (m block, n block, k split, column half), rastered in bands of MC_TC_RASTER m-blocks.
// When the tiles do not fill the last wave of CTAs, the tiles of that wave are cut into two 128-column
// halves (half = 0 / 1, otherwise -1), so that twice as many SMs share the tail.
__device__ __forceinline__ void mc_tc_decode(int item, int tiles_m, int tiles_n, int splits, int half_tiles, int& mb, int& nb,
                                             int& split, int& half) {
    split = item % splits;
    int tile = item / splits;
    half = -1;
    const int whole = tiles_m * tiles_n - half_tiles;
    if (half_tiles > 0 && tile >= whole) {
        half = (tile - whole) & 1;
        tile = whole + ((tile - whole) >> 1);
    }
    const int band_tiles = MC_TC_RASTER * tiles_n;
    const int band = tile / band_tiles;
    const int first_m = band * MC_TC_RASTER;
    const int band_rows = min(MC_TC_RASTER, tiles_m - first_m);
    const int within = tile - band * band_tiles;
    mb = first_m + within % band_rows;
    nb = within / band_rows;
}

template <int kElemBytes, bool kBIsKMajor>
__device__ __forceinline__ void mc_gemm_tc_body(const McTensorMap& map_a, const McTensorMap& map_b, const McTcParams& p,
                                                const McEpilogueArgs& epi) {
    constexpr int kBlockK = 128 / kElemBytes;    // elements per K block (one 128-byte swizzle row)
    constexpr int kMmaK = 32 / kElemBytes;       // elements per tcgen05.mma
    constexpr int kMmasPerBlock = kBlockK / kMmaK;  // 4
    constexpr int kAtomN = 128 / kElemBytes;     // MN-major B: columns per 128-byte atom
    constexpr bool kTf32 = kElemBytes == 4;

    extern __shared__ unsigned char mc_tc_smem_raw[];
    const unsigned raw = mc_smem_addr(mc_tc_smem_raw);
    const unsigned tiles_base = (raw + 1023u) & ~1023u;  // 128B swizzle wants 1024-byte aligned tiles
    const unsigned bars_base = tiles_base + MC_TC_STAGES * MC_TC_STAGE_BYTES;
    // barrier slots (8 bytes each): full[MAX_STAGES], empty[MAX_STAGES], tmem_full[2], tmem_empty[2]
    const unsigned bar_full = bars_base;
    const unsigned bar_empty = bars_base + 8 * MC_TC_MAX_STAGES;
    const unsigned bar_tmem_full = bars_base + 16 * MC_TC_MAX_STAGES;
    const int stages = p.stages;
    const unsigned a_bytes = (unsigned)p.a_rows * 128u;
    const unsigned stage_bytes = a_bytes + (unsigned)p.tile_n * 128u;
    const unsigned bar_tmem_empty = bar_tmem_full + 16;
    // cluster reduction: peers_done (every CTA of the cluster has finished its MMAs), data_ready (every epilogue warp
    // of every CTA has delivered its partial sums)
    const unsigned bar_peers_done = bar_tmem_empty + 16;
    const unsigned bar_data_ready = bar_peers_done + 8;
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // When K is split, the reduction kernel that follows is launched as a programmatic dependent: once every CTA of
    // this grid has passed this point its blocks may take their places (they wait for this grid to complete before
    // they read anything), which hides its launch latency behind the main loop.
    if (p.splits > 1) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int tiles_m = (p.m + MC_TC_BM - 1) / MC_TC_BM;
    const int bn = p.tile_n;  // columns per tile; accumulators stay MC_TC_BN TMEM columns apart
    const int tiles_n = (p.n + bn - 1) / bn;
    const int k_blocks = (p.k + kBlockK - 1) / kBlockK;
    const int items = (tiles_m * tiles_n + p.half_tiles) * p.splits;

    if (threadIdx.x == 0) {
        abort_flag_storage = 0;
        for (int s = 0; s < stages; ++s) {
            mc_mbar_init(bar_full + 8 * s, 1);
            mc_mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mc_mbar_init(bar_tmem_full + 8 * a, 1);
            mc_mbar_init(bar_tmem_empty + 8 * a, MC_TC_EPILOGUE_WARPS);  // one arrival per epilogue warp
        }
        if (p.cluster_reduce > 1) {
            mc_mbar_init(bar_peers_done, (unsigned)p.cluster_reduce);
            mc_mbar_init(bar_data_ready, (unsigned)(p.cluster_reduce * MC_TC_EPILOGUE_WARPS));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mc_smem_addr(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;
    if (p.cluster_reduce > 1) mc_cluster_sync();  // every CTA's barriers exist before a peer arrives on them

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            int issued = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < items; item += gridDim.x) {
                int mb, nb, split, half;
                mc_tc_decode(item, tiles_m, tiles_n, p.splits, p.half_tiles, mb, nb, split, half);
                const int kb_begin = split * p.k_blocks_per_split;
                const int kb_end = min(k_blocks, kb_begin + p.k_blocks_per_split);
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = mc_mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, MC_TC_ERR_PRODUCER);
                    if (!ok) break;
                    const unsigned full = bar_full + 8 * stage;
                    const unsigned a_dst = tiles_base + stage * stage_bytes;
                    const unsigned b_dst = a_dst + a_bytes;
                    mc_mbar_expect_tx(full, stage_bytes);
                    mc_tma_load_2d(a_dst, &map_a, full, kb * kBlockK, mb * MC_TC_BM);
                    if (kBIsKMajor) {
                        mc_tma_load_2d(b_dst, &map_b, full, kb * kBlockK, nb * bn);  // the map's box holds bn rows
                    } else {
#pragma unroll
                        for (int j = 0; j < MC_TC_BN / kAtomN; ++j) {
                            if (j * kAtomN >= bn) break;
                            mc_tma_load_2d(b_dst + j * (kBlockK * 128), &map_b, full, nb * bn + j * kAtomN,
                                           kb * kBlockK);
                        }
                    }
                    ++issued;
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) {
                // Give the copies still in flight time to land before shared memory is released:
                // the most recently issued min(issued, STAGES) stages each complete their `full` barrier.
                int s = stage;
                unsigned ph = phase;
                const int pending = min(issued, stages);
                for (int i = 0; i < pending; ++i) {
                    if (s == 0) {
                        s = stages;
                        ph ^= 1u;
                    }
                    --s;
                    const unsigned long long t0 = mc_globaltimer();
                    while (!mc_mbar_try_wait(bar_full + 8 * s, ph)) {
                        if (mc_globaltimer() - t0 > MC_TC_WAIT_NS / 4) {
                            if (p.status != nullptr) atomicOr(p.status, MC_TC_ERR_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            int acc = 0;
            unsigned acc_phase = 0;
            bool ok = true;
            for (int item = blockIdx.x; ok && item < items; item += gridDim.x) {
                int mb, nb, split, half;
                mc_tc_decode(item, tiles_m, tiles_n, p.splits, p.half_tiles, mb, nb, split, half);
                const int kb_begin = split * p.k_blocks_per_split;
                const int kb_end = min(k_blocks, kb_begin + p.k_blocks_per_split);
                ok = mc_mbar_wait(bar_tmem_empty + 8 * acc, acc_phase ^ 1u, abort_flag, p.status, MC_TC_ERR_MMA);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned tmem_d = tmem_base + (unsigned)(acc * MC_TC_BN);
                // N field of the instruction descriptor (bits 17-22, N >> 3): 128 for a half tile.
                const unsigned idesc = half < 0 ? p.idesc : ((p.idesc & ~(0x3Fu << 17)) | ((unsigned)(MC_TC_BN / 2 >> 3) << 17));
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    ok = mc_mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, MC_TC_ERR_MMA);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_src = tiles_base + stage * stage_bytes;
                    const unsigned b_src = a_src + a_bytes;
                    // K-major operand: rows of 128 bytes, 8-row groups 1024 bytes apart; a K step is 32 bytes.
                    const unsigned long long desc_a = mc_smem_desc(a_src, 16, 1024);
                    // MN-major B: 128-byte atoms of columns, each holding kBlockK rows; 8-row groups 1024 bytes
                    // apart, atoms kBlockK*128 bytes apart; a K step is kMmaK rows.
                    // A half tile reads its 128 columns out of the same staged 256-column tile: 128 rows further
                    // on in the K-major form, two column atoms further on in the MN-major form, 16 KB either way.
                    const unsigned b_half = half == 1 ? (unsigned)(MC_TC_B_BYTES / 2) : 0u;
                    const unsigned long long desc_b = kBIsKMajor ? mc_smem_desc(b_src + b_half, 16, 1024)
                                                                 : mc_smem_desc(b_src + b_half, kBlockK * 128, 1024);
                    const unsigned b_step = kBIsKMajor ? 2u : (unsigned)(kMmaK * 128) >> 4;
#pragma unroll
                    for (int ks = 0; ks < kMmasPerBlock; ++ks) {
                        mc_umma(tmem_d, desc_a + (unsigned long long)(2 * ks), desc_b + (unsigned long long)(b_step * ks),
                                idesc, (kb > kb_begin || ks > 0) ? 1u : 0u, kTf32);
                    }
                    mc_umma_commit(bar_empty + 8 * stage);  // the stage is free once these MMAs have read it
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                mc_umma_commit(bar_tmem_full + 8 * acc);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;  // the TMEM lanes this warp may touch: [32*quarter, +32)
        // Two warps share each lane quarter and take one half of the tile's columns each.
        const int kColsPerWarp = bn / (MC_TC_EPILOGUE_WARPS / 4);
        const int col_begin = ((warp - 2) >> 2) * kColsPerWarp;
        int acc = 0;
        unsigned acc_phase = 0;
        bool ok = true;
        const bool partial = p.splits > 1;
        if (p.cluster_reduce > 1) {
            // ---- K slices of one tile as a cluster: partial tiles meet in distributed shared memory
            const int S = p.cluster_reduce;
            const unsigned my_rank = mc_cluster_ctarank();
            int mb, nb, split, half;
            mc_tc_decode((int)blockIdx.x, tiles_m, tiles_n, p.splits, 0, mb, nb, split, half);
            const int cw = bn / S;        // columns of the tile each CTA finishes
            const int pitch = cw + 4;     // floats per row of a received slot (the pad spreads rows over the banks)
            const unsigned recv_base = tiles_base;  // slot r (from rank r): [128 rows][pitch] floats, in the operand ring's space
            ok = mc_mbar_wait(bar_tmem_full, 0u, abort_flag, p.status, MC_TC_ERR_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // This CTA's MMAs are complete, so its ring is free: tell every CTA of the cluster, then wait for all.
                if (warp == 2 && lane == 0) {
                    for (int r = 0; r < S; ++r) mc_mbar_arrive_release_cluster(mc_mapa(bar_peers_done, (unsigned)r));
                }
                ok = mc_mbar_wait_cluster(bar_peers_done, 0u, abort_flag, p.status, MC_TC_ERR_CLUSTER);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                const int row_in_tile = quarter * 32 + lane;
                const bool row_valid = mb * MC_TC_BM + row_in_tile < p.m;
                for (int chunk = 0; chunk < kColsPerWarp / 32; ++chunk) {
                    const int col = col_begin + chunk * 32;  // within the tile
                    if (nb * bn + col >= p.n) break;         // warp-uniform: nobody reads these columns
                    unsigned v[32];
                    mc_tmem_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)col, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (row_valid) {
                        const int owner = col / cw;
                        const unsigned local = recv_base + (unsigned)((((int)my_rank * MC_TC_BM + row_in_tile) * pitch + col % cw) * 4);
                        const unsigned remote = mc_mapa(local, (unsigned)owner);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) mc_st_cluster_v4(remote + 4u * j, v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
                asm volatile("fence.acq_rel.cluster;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    for (int r = 0; r < S; ++r) mc_mbar_arrive_release_cluster(mc_mapa(bar_data_ready, (unsigned)r));
                }
                ok = mc_mbar_wait_cluster(bar_data_ready, 0u, abort_flag, p.status, MC_TC_ERR_CLUSTER);
                ok = __all_sync(0xffffffffu, ok);
            }
            if (ok) {
                // Columns [my_rank * cw, +cw) of the tile. Rows go round the 8 warps (so a problem of 16 rows still uses
                // all of them), lanes along the columns; a row's S x cw/32 values are requested together, then the
                // slices are added in index order.
                const float* recv = static_cast<const float*>(__cvta_shared_to_generic(recv_base));
                const int rows_here = min(MC_TC_BM, p.m - mb * MC_TC_BM);
                const int per_lane = cw / 32;  // 1, 2 or 4 columns per lane
                for (int r = warp - 2; r < rows_here; r += MC_TC_EPILOGUE_WARPS) {
                    const int row = mb * MC_TC_BM + r;
                    float part[8][4];
#pragma unroll
                    for (int z = 0; z < 8; ++z) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            part[z][j] = (z < S && j < per_lane) ? recv[(z * MC_TC_BM + r) * pitch + lane + 32 * j] : 0.0f;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (j >= per_lane) break;
                        const int colg = nb * bn + (int)my_rank * cw + lane + 32 * j;
                        if (colg >= p.n) continue;
                        float sum = part[0][j];
#pragma unroll
                        for (int z = 1; z < 8; ++z) {
                            if (z < S) sum += part[z][j];
                        }
                        sum = mc_epilogue(sum, (unsigned)row, (unsigned)colg, epi);
                        if (p.c != nullptr) p.c[(long long)row * p.ldc + colg] = sum;
                        if (p.c16 != nullptr) p.c16[(long long)row * p.ldc16 + colg] = mc_to_half(sum, p.c16_kind);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        } else
        for (int item = blockIdx.x; ok && item < items; item += gridDim.x) {
            int mb, nb, split, half;
            mc_tc_decode(item, tiles_m, tiles_n, p.splits, p.half_tiles, mb, nb, split, half);
            ok = mc_mbar_wait(bar_tmem_full + 8 * acc, acc_phase, abort_flag, p.status, MC_TC_ERR_EPILOGUE);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = mb * MC_TC_BM + quarter * 32 + lane;
            const int n0 = nb * bn;
            float* dst = partial ? p.workspace + (long long)split * p.m * p.n : p.c;
            const long long ld = partial ? (long long)p.n : p.ldc;
            const bool vec4 = (ld & 3) == 0 && (((unsigned long long)dst) & 15) == 0;
            const bool vec16 = (p.ldc16 & 7) == 0 && (((unsigned long long)p.c16) & 15) == 0;
            // A whole tile: this warp's half of 256 columns. A half tile: this warp's half of its 128 columns,
            // which sit in accumulator columns 0..127.
            const int warp_cols = half < 0 ? kColsPerWarp : kColsPerWarp / 2;
            const int acc_col_begin = half < 0 ? col_begin : col_begin / 2;
            const int tile_col_begin = half < 0 ? col_begin : half * (MC_TC_BN / 2) + col_begin / 2;
            for (int chunk = 0; chunk < warp_cols / 32; ++chunk) {
                const int col0 = n0 + tile_col_begin + chunk * 32;
                if (col0 >= p.n) break;  // warp-uniform
                unsigned v[32];
                mc_tmem_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(acc * MC_TC_BN + acc_col_begin + chunk * 32), v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < p.m) {
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                    if (!partial) {
                        if (col0 + 32 <= p.n) {
                            mc_epilogue32(f, (unsigned)row, (unsigned)col0, epi);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < p.n) f[j] = mc_epilogue(f[j], (unsigned)row, (unsigned)(col0 + j), epi);
                            }
                        }
                    }
                    if (dst != nullptr) {
                        float* out = dst + (long long)row * ld + col0;
                        if (vec4 && col0 + 32 <= p.n) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                *reinterpret_cast<float4*>(out + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < p.n) out[j] = f[j];
                            }
                        }
                    }
                    if (!partial && p.c16 != nullptr) {
                        unsigned short* out16 = p.c16 + (long long)row * p.ldc16 + col0;
                        if (vec16 && col0 + 32 <= p.n) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 pack;
                                pack.x = mc_to_half2(f[j + 0], f[j + 1], p.c16_kind);
                                pack.y = mc_to_half2(f[j + 2], f[j + 3], p.c16_kind);
                                pack.z = mc_to_half2(f[j + 4], f[j + 5], p.c16_kind);
                                pack.w = mc_to_half2(f[j + 6], f[j + 7], p.c16_kind);
                                *reinterpret_cast<uint4*>(out16 + j) = pack;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < p.n) out16[j] = mc_to_half(f[j], p.c16_kind);
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mc_mbar_arrive(bar_tmem_empty + 8 * acc);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
        }
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    // No CTA of a cluster lets go of its shared memory while a peer may still write to it or arrive on its barriers.
    if (p.cluster_reduce > 1) mc_cluster_sync();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc_h16_bmn)
extern "C" __global__ void __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc_h16_bmn(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                   const McTcParams p, const McEpilogueArgs epi) {
    mc_gemm_tc_body<2, false>(map_a, map_b, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc_h16_bk)
extern "C" __global__ void __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc_h16_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                  const McTcParams p, const McEpilogueArgs epi) {
    mc_gemm_tc_body<2, true>(map_a, map_b, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc_tf32_bmn)
extern "C" __global__ void __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc_tf32_bmn(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                    const McTcParams p, const McEpilogueArgs epi) {
    mc_gemm_tc_body<4, false>(map_a, map_b, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc_tf32_bk)
extern "C" __global__ void __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc_tf32_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                   const McTcParams p, const McEpilogueArgs epi) {
    mc_gemm_tc_body<4, true>(map_a, map_b, p, epi);
}
#endif
