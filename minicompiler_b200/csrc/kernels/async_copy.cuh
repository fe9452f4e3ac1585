// Asynchronous-copy plumbing shared by the GEMM kernel sources: tensor maps, mbarriers with bounded waits, and the
// tiled TMA load (no multicast). Like the other kernel texts it is compiled ahead of time into the library and at run
// time by NVRTC in front of a kernel family, so it holds no #include lines.

#ifndef MC_ASYNC_COPY_DEFINED
#define MC_ASYNC_COPY_DEFINED

#define MC_WAIT_NS 2000000000ull  // a wait gives up after this much wall time

struct __align__(64) McTensorMap {
    unsigned long long opaque[16];
};

__device__ __forceinline__ unsigned mc_smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long mc_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mc_mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mc_mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mc_mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mc_mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait. Returns false when it gave up (or when another role already did).
__device__ __forceinline__ bool mc_mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag, unsigned* status,
                                             unsigned err_code) {
    if (mc_mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = mc_globaltimer();
    unsigned spins = 0;
    while (!mc_mbar_try_wait(bar, parity)) {
        if ((++spins & 255u) == 0u) {
            if (*abort_flag != 0) return false;
            if (mc_globaltimer() - t0 > MC_WAIT_NS) {
                if (status != nullptr) atomicOr(status, err_code);
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}


__device__ __forceinline__ void mc_tma_load_2d(unsigned smem_dst, const McTensorMap* map, unsigned bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_dst), "l"((unsigned long long)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

#endif  // MC_ASYNC_COPY_DEFINED
