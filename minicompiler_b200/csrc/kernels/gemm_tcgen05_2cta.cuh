// Tensor-core matmul on SM pairs: the same contract as gemm_tcgen05.cuh, for problems large enough
// to fill the GPU without splitting K. Two CTAs of a cluster (an SM pair) own one 256 x 256 tile of C:
// each stages its own 128 rows of A and its own 128 columns of B, and the leader CTA issues
// tcgen05.mma.cta_group::2 (256 x 256 x 16), which reads A and B from both CTAs' shared memory and
// accumulates each CTA's 128 rows into that CTA's TMEM. Per K block a CTA therefore loads 32 KB instead
// of 48 KB for the same arithmetic, the ring holds 6 stages instead of 4, and shared-memory read traffic
// per MMA halves.
//
// Protocol (all barriers live at the same shared-memory offsets in both CTAs):
//   full[s]       leader's only. Armed by the leader's producer with the bytes of BOTH CTAs; the TMA loads of
//                 both CTAs complete on it (no multicast: every CTA loads only what it keeps).
//   empty[s]      one per CTA; the leader's tcgen05.commit (cta_group::2, cluster mask 0b11) arrives on both.
//   tmem_full[a]  one per CTA; same commit form once a tile's last MMA is issued.
//   tmem_empty[a] leader's only; the 8 epilogue warps of each CTA arrive on it remotely (16 arrivals).
// Waits are bounded exactly as in the one-CTA kernel; before it returns, every thread of the pair passes a
// cluster barrier, so neither CTA's shared memory or TMEM goes away under its peer.
//
// This text follows gemm_tcgen05.cuh in the same translation unit and uses its helpers.

#define MC_TC2_STAGES 6
#define MC_TC2_WIDE_STAGES 4
#define MC_TC2_A_BYTES (MC_TC_BM * 128)
#define MC_TC2_B_BYTES (128 * 128)
#define MC_TC2_STAGE_BYTES (MC_TC2_A_BYTES + MC_TC2_B_BYTES)
#define MC_TC2_STAGING_PER_WARP 4096
#define MC_TC2_BARRIER_BYTES 1024  // keeps the staging buffers behind the barriers 1024-byte aligned (128-byte swizzle)
#define MC_TC2_SMEM_BYTES \
    (MC_TC2_STAGES * MC_TC2_STAGE_BYTES + 1024 + MC_TC2_BARRIER_BYTES + MC_TC_EPILOGUE_WARPS * MC_TC2_STAGING_PER_WARP)

// TMA load whose completion is counted on a barrier that may sit in the peer CTA of the pair.
__device__ __forceinline__ void mc_tma_load_2d_pair(unsigned smem_dst, const McTensorMap* map, unsigned bar_cluster_addr, int c0,
                                                    int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"((unsigned long long)map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
        : "memory");
}

// TMA store of one box from shared memory; completion is tracked in the issuing thread's bulk groups. Rows and
// columns of the box that lie outside the tensor are not written.
__device__ __forceinline__ void mc_tma_store_2d(const McTensorMap* map, unsigned smem_src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"((unsigned long long)map),
                 "r"(smem_src), "r"(c0), "r"(c1)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Until the bulk stores this thread has issued have read their shared-memory source.
__device__ __forceinline__ void mc_tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

// The same, but the most recent store may still be reading: enough to reuse the buffer of the store before it.
__device__ __forceinline__ void mc_tma_store_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }

// Shared-memory writes of this thread become visible to the TMA unit.
__device__ __forceinline__ void mc_fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mc_st_shared_v4u(unsigned addr, unsigned a, unsigned b, unsigned c, unsigned d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void mc_st_shared_v4(unsigned addr, float a, float b, float c, float d) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__device__ __forceinline__ void mc_umma_pair(unsigned tmem_d, unsigned long long desc_a, unsigned long long desc_b, unsigned idesc,
                                             unsigned accumulate, bool tf32) {
    if (tf32) {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
            "}\n" ::"r"(tmem_d),
            "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Arrives (once the MMAs issued so far have completed) on the barrier at the same offset in both CTAs.
__device__ __forceinline__ void mc_umma_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                 "h"((unsigned short)3)
                 : "memory");
}

template <int kElemBytes, bool kBIsKMajor, bool kWide>
__device__ __forceinline__ void mc_gemm_tc2_body(const McTensorMap& map_a, const McTensorMap& map_b, const McTensorMap& map_c,
                                                 const McTensorMap& map_c16, const McTcParams& p, const McEpilogueArgs& epi) {
    constexpr int kBlockK = 128 / kElemBytes;
    constexpr int kMmaK = 32 / kElemBytes;
    constexpr int kMmasPerBlock = kBlockK / kMmaK;
    constexpr int kAtomN = 128 / kElemBytes;
    constexpr bool kTf32 = kElemBytes == 4;

    // Two shapes of work item share this body. Normal: one 256 x 256 tile per item, the two TMEM regions used
    // in turn so that the epilogue of one item overlaps the MMAs of the next; 32 KB stages, 6 deep. Wide
    // (p.wide): two 256 x 256 tiles side by side per item, one per TMEM region, fed by the same A rows - a CTA
    // then loads 48 KB per K block for twice the arithmetic; 48 KB stages, 4 deep.
    constexpr bool wide = kWide;
    constexpr int stages = kWide ? MC_TC2_WIDE_STAGES : MC_TC2_STAGES;
    constexpr unsigned stage_bytes = kWide ? (unsigned)(MC_TC2_A_BYTES + 2 * MC_TC2_B_BYTES) : (unsigned)MC_TC2_STAGE_BYTES;
    constexpr int kMaxSub = kWide ? 2 : 1;

    extern __shared__ unsigned char mc_tc_smem_raw[];
    const unsigned raw = mc_smem_addr(mc_tc_smem_raw);
    const unsigned tiles_base = (raw + 1023u) & ~1023u;
    const unsigned bars_base = tiles_base + MC_TC2_STAGES * MC_TC2_STAGE_BYTES;
    const unsigned bar_full = bars_base;
    const unsigned bar_empty = bars_base + 8 * MC_TC2_STAGES;
    const unsigned bar_tmem_full = bars_base + 16 * MC_TC2_STAGES;
    const unsigned bar_tmem_empty = bar_tmem_full + 16;
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag_storage;
    volatile int* abort_flag = &abort_flag_storage;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // The launch behind this one may take its place as soon as SMs fall free (a kernel launched as a programmatic
    // dependent, e.g. the next layer of a stack): its CTAs set themselves up while the last tiles of this grid finish.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const unsigned rank = mc_cluster_ctarank();
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;

    const int tiles_m = (p.m + MC_TC_BM - 1) / MC_TC_BM;
    const int pairs_m = (tiles_m + 1) / 2;
    const int tiles_n = (p.n + MC_TC_BN - 1) / MC_TC_BN;
    const int k_blocks = (p.k + kBlockK - 1) / kBlockK;
    const int cols_n = wide ? (tiles_n + 1) / 2 : tiles_n;  // column tiles of this mode
    // The last `half_tiles` tiles are issued as two items each, so that a short last wave spreads over twice as
    // many SM pairs: a normal tile as its two 128-column halves, a wide tile as its two 256-column tiles.
    const int whole = pairs_m * cols_n - p.half_tiles;
    const int items = whole + 2 * p.half_tiles;

    if (threadIdx.x == 0) {
        abort_flag_storage = 0;
        for (int s = 0; s < MC_TC2_STAGES; ++s) {
            mc_mbar_init(bar_full + 8 * s, 1);
            mc_mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mc_mbar_init(bar_tmem_full + 8 * a, 1);
            mc_mbar_init(bar_tmem_empty + 8 * a, 2 * MC_TC_EPILOGUE_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(mc_smem_addr(&tmem_base_slot)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    mc_cluster_sync();  // both CTAs' barriers are initialised before either signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_base = tmem_base_slot;
    // Launched as a programmatic dependent, this grid may have started before the one in front of it was done: nothing
    // is read from or written to global memory before that grid has completed and its writes are visible (a no-op for
    // a plain launch). Barriers, TMEM and the tensor maps in the parameters are set up by then.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // Work item -> row pair `mp`, first 256-column block `nb`, number of 256-column tiles `nsub` (0: nothing to
    // do), and `half` = 0 / 1 when the item is a 128-column half of a normal tile (-1 otherwise).
    auto decode = [&](int item, int& mp, int& nb, int& nsub, int& half) {
        // bands of 16 row pairs: against 8, +0.7 % at 8192^3 and +0.9 % at 4096^3 (alternating runs on one box), no
        // difference at 16384^3 or on the 8-column-tile layers of the MLP stack; 4 and 32 are slower
        constexpr int kBand = MC_TC_RASTER;
        int part = -1;
        int tile = item;
        if (item >= whole) {
            part = (item - whole) & 1;
            tile = whole + ((item - whole) >> 1);
        }
        const int band_tiles = kBand * cols_n;
        const int band = tile / band_tiles;
        const int first = band * kBand;
        const int band_rows = min(kBand, pairs_m - first);
        const int within = tile - band * band_tiles;
        mp = first + within % band_rows;
        const int col = within / band_rows;
        half = -1;
        if (wide) {
            nb = part < 0 ? 2 * col : 2 * col + part;
            nsub = part < 0 ? min(2, tiles_n - nb) : (nb < tiles_n ? 1 : 0);
        } else {
            nb = col;
            nsub = 1;
            half = part;
        }
    };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            unsigned phase = 0;
            int issued = 0;
            bool ok = true;
            for (int item = cluster_id; ok && item < items; item += num_clusters) {
                int mp, nb, nsub, half;
                decode(item, mp, nb, nsub, half);
                if (nsub == 0) continue;
                const int row0 = (2 * mp + (int)rank) * MC_TC_BM;
                // A whole tile: this CTA's 128 of the 256 columns. A half tile: its 64 of the half's 128 columns,
                // fetched with the same 128-column copies (the upper 64 are not used).
                const int col_first = nb * MC_TC_BN + (half < 0 ? (int)rank * 128 : half * 128 + (int)rank * 64);
                const unsigned bytes = (unsigned)(MC_TC2_A_BYTES + nsub * MC_TC2_B_BYTES);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    ok = mc_mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status, MC_TC_ERR_PRODUCER);
                    if (!ok) break;
                    const unsigned full_local = bar_full + 8 * stage;
                    const unsigned full_leader = mc_mapa(full_local, 0);
                    const unsigned a_dst = tiles_base + stage * stage_bytes;
                    if (leader) mc_mbar_expect_tx(full_local, 2 * bytes);
                    mc_tma_load_2d_pair(a_dst, &map_a, full_leader, kb * kBlockK, row0);
#pragma unroll
                    for (int s = 0; s < kMaxSub; ++s) {
                        if (s >= nsub) break;
                        const unsigned b_dst = a_dst + MC_TC2_A_BYTES + s * MC_TC2_B_BYTES;
                        const int col0 = col_first + s * MC_TC_BN;
                        if (kBIsKMajor) {
                            mc_tma_load_2d_pair(b_dst, &map_b, full_leader, kb * kBlockK, col0);
                        } else {
#pragma unroll
                            for (int j = 0; j < 128 / kAtomN; ++j) {
                                mc_tma_load_2d_pair(b_dst + j * (kBlockK * 128), &map_b, full_leader, col0 + j * kAtomN, kb * kBlockK);
                            }
                        }
                    }
                    ++issued;
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok && leader) {
                // Let the copies in flight land before shared memory is released (the leader's barriers see both CTAs').
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
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            int stage = 0;
            unsigned phase = 0;
            int acc = 0;              // normal mode: the TMEM region of this item
            unsigned empty_phase = 0;  // bit r: parity of region r's tmem_empty barrier
            bool ok = true;
            for (int item = cluster_id; ok && item < items; item += num_clusters) {
                int mp, nb, nsub, half;
                decode(item, mp, nb, nsub, half);
                if (nsub == 0) continue;
                const int region0 = wide ? 0 : acc;
                ok = mc_mbar_wait(bar_tmem_empty + 8 * region0, ((empty_phase >> region0) & 1u) ^ 1u, abort_flag, p.status,
                                  MC_TC_ERR_MMA);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // N field of the instruction descriptor (bits 17-22, N >> 3): 128 for a half tile.
                const unsigned idesc = half < 0 ? p.idesc : ((p.idesc & ~(0x3Fu << 17)) | ((unsigned)(MC_TC_BN / 2 >> 3) << 17));
                const unsigned b_step = kBIsKMajor ? 2u : (unsigned)(kMmaK * 128) >> 4;
                auto issue = [&](int st, int s, bool first_block) {
                    const unsigned a_src = tiles_base + st * stage_bytes;
                    const unsigned b_src = a_src + MC_TC2_A_BYTES + s * MC_TC2_B_BYTES;
                    const unsigned tmem_d = tmem_base + (unsigned)((region0 + s) * MC_TC_BN);
                    const unsigned long long desc_a = mc_smem_desc(a_src, 16, 1024);
                    const unsigned long long desc_b =
                        kBIsKMajor ? mc_smem_desc(b_src, 16, 1024) : mc_smem_desc(b_src, kBlockK * 128, 1024);
#pragma unroll
                    for (int ks = 0; ks < kMmasPerBlock; ++ks) {
                        mc_umma_pair(tmem_d, desc_a + (unsigned long long)(2 * ks), desc_b + (unsigned long long)(b_step * ks), idesc,
                                     (!first_block || ks > 0) ? 1u : 0u, kTf32);
                    }
                };
                int kb = 0;
                if (kWide && nsub == 2) {
                    // The second region may still be draining: start on the first with as many K blocks as the ring
                    // holds, then catch the second region up on the same blocks and release them.
                    const int head = min(stages, k_blocks);
                    int st = stage;
                    unsigned ph = phase;
                    for (int i = 0; i < head; ++i) {
                        ok = mc_mbar_wait(bar_full + 8 * st, ph, abort_flag, p.status, MC_TC_ERR_MMA);
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        issue(st, 0, i == 0);
                        if (++st == stages) {
                            st = 0;
                            ph ^= 1u;
                        }
                    }
                    if (!ok) break;
                    ok = mc_mbar_wait(bar_tmem_empty + 8 * 1, ((empty_phase >> 1) & 1u) ^ 1u, abort_flag, p.status, MC_TC_ERR_MMA);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    for (int i = 0; i < head; ++i) {
                        issue(stage, 1, i == 0);
                        mc_umma_commit_pair(bar_empty + 8 * stage);
                        if (++stage == stages) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                    kb = head;
                }
                for (; kb < k_blocks; ++kb) {
                    ok = mc_mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, MC_TC_ERR_MMA);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                    for (int s = 0; s < kMaxSub; ++s) {
                        if (s < nsub) issue(stage, s, kb == 0);
                    }
                    mc_umma_commit_pair(bar_empty + 8 * stage);
                    if (++stage == stages) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (!ok) break;
                for (int s = 0; s < nsub; ++s) {
                    mc_umma_commit_pair(bar_tmem_full + 8 * (region0 + s));
                    empty_phase ^= 1u << (region0 + s);
                }
                acc ^= 1;
            }
        }
    } else {
        // ------------------------------------------------ epilogue (both CTAs, own 128 rows each)
        const int quarter = warp & 3;
        constexpr int kColsPerWarp = MC_TC_BN / (MC_TC_EPILOGUE_WARPS / 4);
        const int col_begin = ((warp - 2) >> 2) * kColsPerWarp;
        const bool vec4 = (p.ldc & 3) == 0 && (((unsigned long long)p.c) & 15) == 0;
        const bool vec16 = (p.ldc16 & 7) == 0 && (((unsigned long long)p.c16) & 15) == 0;
        // Staged stores need the aligned fast paths of both outputs; anything else takes the direct per-row stores.
        const bool staged = p.staged != 0 && (p.c == nullptr || vec4) && (p.c16 == nullptr || vec16);
        const unsigned stage_base = bars_base + MC_TC2_BARRIER_BYTES + (unsigned)(warp - 2) * MC_TC2_STAGING_PER_WARP;
        int acc = 0;
        unsigned full_phase = 0;  // bit r: parity of region r's tmem_full barrier
        unsigned buffer_turn = 0;  // which half of the staging buffer the next 2 KB box goes through
        bool ok = true;
        for (int item = cluster_id; ok && item < items; item += num_clusters) {
            int mp, nb, nsub, half;
            decode(item, mp, nb, nsub, half);
            if (nsub == 0) continue;
            const int region0 = wide ? 0 : acc;
            const int row_base = (2 * mp + (int)rank) * MC_TC_BM + quarter * 32;
            const int row = row_base + lane;
            // A whole tile: this warp's half of 256 columns. A half tile: this warp's half of its 128 columns,
            // which sit in accumulator columns 0..127.
            const int warp_cols = half < 0 ? kColsPerWarp : kColsPerWarp / 2;
            const int acc_col_begin = half < 0 ? col_begin : col_begin / 2;
            const int tile_col_begin = half < 0 ? col_begin : half * (MC_TC_BN / 2) + col_begin / 2;
            for (int s = 0; s < nsub; ++s) {
                const int r = region0 + s;
                ok = mc_mbar_wait(bar_tmem_full + 8 * r, (full_phase >> r) & 1u, abort_flag, p.status, MC_TC_ERR_EPILOGUE);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const int n0 = (nb + s) * MC_TC_BN;
                // The warp reads its slice of the region 32 columns at a time and finishes each piece (arithmetic,
                // staging, hand-over to the TMA unit) before it asks for the next: 32 live accumulator registers instead
                // of 128. TMEM reads were measured to cost the running MMAs nothing. The region goes back to the MMA
                // issuer when the last piece is in registers.
                int last_chunk = -1;
#pragma unroll
                for (int chunk = 0; chunk < kColsPerWarp / 32; ++chunk) {
                    if (chunk * 32 < warp_cols) last_chunk = chunk;
                }
#pragma unroll
                for (int chunk = 0; chunk < kColsPerWarp / 32; ++chunk) {
                    if (chunk * 32 >= warp_cols) continue;  // warp-uniform
                    unsigned v[32];
                    mc_tmem_load32(tmem_base + ((unsigned)(quarter * 32) << 16) + (unsigned)(r * MC_TC_BN + acc_col_begin + chunk * 32), v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (chunk == last_chunk) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) mc_mbar_arrive_cluster(mc_mapa(bar_tmem_empty + 8 * r, 0));
                    }
                    const int col0 = n0 + tile_col_begin + chunk * 32;
                    if (col0 >= p.n) continue;  // warp-uniform
                    float f[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
                    const bool whole_chunk = col0 + 32 <= p.n;
                    if (row < p.m) {
                        if (whole_chunk) {
                            mc_epilogue32(f, (unsigned)row, (unsigned)col0, epi);
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < p.n) f[j] = mc_epilogue(f[j], (unsigned)row, (unsigned)(col0 + j), epi);
                            }
                        }
                    }
                    if (staged) {
                        // The 32 x 32 block is written to this warp's staging buffer in the layout a swizzled TMA box
                        // has (16-byte pieces XOR-ed with the row number: no bank conflicts) and leaves as ONE TMA store:
                        // the data never passes through the load/store unit again. Plain vector stores from the
                        // 8 warps were measured to hold up the MMAs of the next tile by 1.5 us per 256 x 256 tile (the
                        // same kernel with the stores left out, or with the TMEM reads alone, ran at the MMA rate).
                        // TMA writes only the part of the box that lies inside the tensor, so ragged edges need no care.
                        if (p.c != nullptr) {
                            // 128-byte rows of FP32 through the whole buffer, one box at a time (two boxes of 16 columns
                            // taking turns in its halves measured no faster: 8192^3 1536 against 1538 TFLOP/s on one box)
                            if (lane == 0) mc_tma_store_wait_read();  // the previous box has left the buffer
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                mc_st_shared_v4(stage_base + lane * 128 + ((j ^ (lane & 7)) << 4), f[4 * j], f[4 * j + 1], f[4 * j + 2],
                                                f[4 * j + 3]);
                            }
                            mc_fence_async_shared();
                            __syncwarp();
                            if (lane == 0) {
                                mc_tma_store_2d(&map_c, stage_base, col0, row_base);
                                if (p.c16 != nullptr) mc_tma_store_wait_read();  // the 16-bit form goes through the same buffer next
                            }
                            __syncwarp();
                        }
                        if (p.c16 != nullptr) {
                            // 64-byte rows, 16-byte pieces XOR-ed with bits 1-2 of the row number (the 64-byte swizzle);
                            // the 2 KB box takes turns with the one before it in the two halves of the buffer
                            const unsigned half_buf = stage_base + (unsigned)(buffer_turn & 1) * 2048u;
                            if (lane == 0) mc_tma_store_wait_read_but_one();
                            __syncwarp();
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                mc_st_shared_v4u(half_buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4),
                                                 mc_to_half2(f[8 * j + 0], f[8 * j + 1], p.c16_kind),
                                                 mc_to_half2(f[8 * j + 2], f[8 * j + 3], p.c16_kind),
                                                 mc_to_half2(f[8 * j + 4], f[8 * j + 5], p.c16_kind),
                                                 mc_to_half2(f[8 * j + 6], f[8 * j + 7], p.c16_kind));
                            }
                            mc_fence_async_shared();
                            __syncwarp();
                            if (lane == 0) mc_tma_store_2d(&map_c16, half_buf, col0, row_base);
                            ++buffer_turn;
                        }
                    } else if (row < p.m) {
                        if (p.c != nullptr) {
                            float* out = p.c + (long long)row * p.ldc + col0;
                            if (vec4 && whole_chunk) {
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
                        if (p.c16 != nullptr) {
                            unsigned short* out16 = p.c16 + (long long)row * p.ldc16 + col0;
                            if (vec16 && whole_chunk) {
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
                full_phase ^= 1u << r;
            }
            acc ^= 1;
        }
        // Every store this warp issued has read its source before the CTA gives up its shared memory (the writes
        // themselves complete with the grid, as for any other store).
        if (lane == 0) mc_tma_store_wait_read();
    }

    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    mc_cluster_sync();  // neither CTA lets go of its shared memory or TMEM while the peer may still touch them
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2_h16_bmn)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2_h16_bmn(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                    const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                    const McEpilogueArgs epi) {
    mc_gemm_tc2_body<2, false, false>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2_h16_bk)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2_h16_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                   const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                   const McEpilogueArgs epi) {
    mc_gemm_tc2_body<2, true, false>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2_tf32_bk)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2_tf32_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                    const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                    const McEpilogueArgs epi) {
    mc_gemm_tc2_body<4, true, false>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2w_h16_bmn)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2w_h16_bmn(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                     const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                     const McEpilogueArgs epi) {
    mc_gemm_tc2_body<2, false, true>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2w_h16_bk)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2w_h16_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                    const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                    const McEpilogueArgs epi) {
    mc_gemm_tc2_body<2, true, true>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif

#if !defined(MC_SINGLE_ENTRY) || defined(MC_ONLY_mc_gemm_tc2w_tf32_bk)
extern "C" __global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MC_TC_THREADS, 1)
mc_gemm_tc2w_tf32_bk(const __grid_constant__ McTensorMap map_a, const __grid_constant__ McTensorMap map_b,
                     const __grid_constant__ McTensorMap map_c, const __grid_constant__ McTensorMap map_c16, const McTcParams p,
                     const McEpilogueArgs epi) {
    mc_gemm_tc2_body<4, true, true>(map_a, map_b, map_c, map_c16, p, epi);
}
#endif
