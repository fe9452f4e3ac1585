// Split-K reduction: C = epilogue(sum over slices of workspace[z][m][n]), slices
// added in index order for every element (the determinism the reference promises,
// src/cuda/matmul_kernels.cu:290-315), with the fused epilogue applied once the
// sum is complete and the optional 16-bit copy written in the same pass.

extern "C" __global__ void __launch_bounds__(256)
mc_splitk_reduce(const float* __restrict__ workspace, float* __restrict__ C, unsigned short* __restrict__ C16,
                 int c16_kind, int M, int N, long long ldc, long long ldc16, int splits, McEpilogueArgs epi) {
    // Launched as a programmatic dependent of the matmul that wrote the partial sums: its blocks may already be
    // resident while that grid drains, and wait here until it has completed and its writes are visible.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const long long slice = (long long)M * N;
    const bool vec = (N & 3) == 0 && (ldc & 3) == 0 && ((unsigned long long)C & 15) == 0 &&
                     ((unsigned long long)workspace & 15) == 0;
    if (vec) {
        const long long groups = slice >> 2;
        const int row_groups = N >> 2;
        for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < groups;
             g += (long long)gridDim.x * blockDim.x) {
            float4 sum = __ldcs(reinterpret_cast<const float4*>(workspace) + g);
            for (int z = 1; z < splits; ++z) {
                const float4 part = __ldcs(reinterpret_cast<const float4*>(workspace + z * slice) + g);
                sum.x += part.x;
                sum.y += part.y;
                sum.z += part.z;
                sum.w += part.w;
            }
            const unsigned row = (unsigned)(g / row_groups);
            const unsigned col = (unsigned)(g % row_groups) << 2;
            sum.x = mc_epilogue(sum.x, row, col + 0, epi);
            sum.y = mc_epilogue(sum.y, row, col + 1, epi);
            sum.z = mc_epilogue(sum.z, row, col + 2, epi);
            sum.w = mc_epilogue(sum.w, row, col + 3, epi);
            if (C != nullptr) *reinterpret_cast<float4*>(C + (long long)row * ldc + col) = sum;
            if (C16 != nullptr) {
                unsigned short* out16 = C16 + (long long)row * ldc16 + col;
                out16[0] = mc_to_half(sum.x, c16_kind);
                out16[1] = mc_to_half(sum.y, c16_kind);
                out16[2] = mc_to_half(sum.z, c16_kind);
                out16[3] = mc_to_half(sum.w, c16_kind);
            }
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < slice; i += (long long)gridDim.x * blockDim.x) {
        float sum = workspace[i];
        for (int z = 1; z < splits; ++z) sum += workspace[z * slice + i];
        const unsigned row = (unsigned)(i / N);
        const unsigned col = (unsigned)(i % N);
        sum = mc_epilogue(sum, row, col, epi);
        if (C != nullptr) C[(long long)row * ldc + col] = sum;
        if (C16 != nullptr) C16[(long long)row * ldc16 + col] = mc_to_half(sum, c16_kind);
    }
}
