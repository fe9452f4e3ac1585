// Shared prelude of every GEMM-family kernel source. The text is compiled twice:
// ahead of time (identity epilogue) into the library, and at run time by NVRTC
// with a generated `mc_epilogue` in front of it when a fused elementwise group
// is folded into a matmul. It must therefore stay free of #include lines and of
// anything NVRTC does not predefine.

#ifndef MC_EPILOGUE_DEFINED
#define MC_EPILOGUE_DEFINED 0
struct McEpilogueArgs {
    const float* p[6];
};
// acc: the finished dot product for output element (row, col).
__device__ __forceinline__ float mc_epilogue(float acc, unsigned row, unsigned col, const McEpilogueArgs& e) {
    (void)row;
    (void)col;
    (void)e;
    return acc;
}
#endif

#ifndef MC_EPILOGUE32_DEFINED
#define MC_EPILOGUE32_DEFINED 0
// The epilogue over 32 consecutive in-range columns of one row (col0 a multiple of 32); a generated
// one fetches row and full-shape operands with 128-bit loads instead of one load per element.
__device__ __forceinline__ void mc_epilogue32(float (&f)[32], unsigned row, unsigned col0, const McEpilogueArgs& e) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = mc_epilogue(f[j], row, col0 + j, e);
}
#endif

#ifndef MC_HALF_HELPERS
#define MC_HALF_HELPERS
// Round-to-nearest-even conversions to the 16-bit operand formats (kind 1 = bf16, 2 = fp16).
__device__ __forceinline__ unsigned short mc_to_half(float v, int kind) {
    unsigned short h;
    if (kind == 1) {
        asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(h) : "f"(v));
    } else {
        asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(v));
    }
    return h;
}
__device__ __forceinline__ unsigned mc_to_half2(float lo, float hi, int kind) {
    unsigned d;
    if (kind == 1) {
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    } else {
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    }
    return d;
}
#endif
