/* Plain-C restatement of the reference's CPU kernels, for the timed CPU baseline.
 *
 * TEST / BENCH INFRASTRUCTURE, NOT PRODUCT: only bench.py's cpu_baseline and
 * `--impl reference` legs and tests/ call this, through oracle/cpu_baseline.py.
 *
 * What it follows:
 *  - oracle_fused: the reference evaluates a fused program 512 elements at a time,
 *    every instruction running over one block before the next block starts, with one
 *    block buffer per instruction (src/cpu/kernels.cpp:199-262, kFusedBlock in
 *    src/cpu/kernels.hpp:15-18); inputs are read in place (same layout), as one scalar,
 *    or as a row that repeats every `period` elements (load_block, :111-141).
 *    Arithmetic per op as apply_unary / apply_binary (:20-43): one float operation per
 *    element, sigmoid = 1/(1+exp(-x)), relu = max(x,0).
 *  - oracle_sgemm: C[m,n] = A[m,k] B[k,n], row-major float32 (matmul, :192-197).
 * The reference gets its vector math and its GEMM from Eigen 3.4.0, single-threaded;
 * here libm supplies exp/log/tanh and the GEMM is a cache-blocked loop nest, and both
 * take a thread count (rows / blocks are independent) so that a run can use every host
 * core. It is a port, not the reference's binary: bench.py labels it "port".
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_BLOCK 512

enum { ORACLE_LOAD = 0, ORACLE_IMM = 1, ORACLE_UNARY = 2, ORACLE_BINARY = 3 };
enum { OP_NEG = 0, OP_EXP, OP_LOG, OP_SQRT, OP_RELU, OP_SIGMOID, OP_TANH, OP_ADD, OP_SUB, OP_MUL, OP_DIV };
enum { IN_CONTIGUOUS = 0, IN_SCALAR = 1, IN_PERIODIC = 2 };

typedef struct oracle_instr {
    int kind;
    int op;
    int a;
    int b;
    float imm;
} oracle_instr;

static void unary_block(int op, const float* x, float* y, int len) {
    int j;
    switch (op) {
        case OP_NEG: for (j = 0; j < len; ++j) y[j] = -x[j]; break;
        case OP_EXP: for (j = 0; j < len; ++j) y[j] = expf(x[j]); break;
        case OP_LOG: for (j = 0; j < len; ++j) y[j] = logf(x[j]); break;
        case OP_SQRT: for (j = 0; j < len; ++j) y[j] = sqrtf(x[j]); break;
        case OP_RELU: for (j = 0; j < len; ++j) y[j] = x[j] > 0.0f ? x[j] : 0.0f; break;
        case OP_SIGMOID: for (j = 0; j < len; ++j) y[j] = 1.0f / (1.0f + expf(-x[j])); break;
        case OP_TANH: for (j = 0; j < len; ++j) y[j] = tanhf(x[j]); break;
        default: break;
    }
}

static void binary_block(int op, const float* a, const float* b, float* y, int len) {
    int j;
    switch (op) {
        case OP_ADD: for (j = 0; j < len; ++j) y[j] = a[j] + b[j]; break;
        case OP_SUB: for (j = 0; j < len; ++j) y[j] = a[j] - b[j]; break;
        case OP_MUL: for (j = 0; j < len; ++j) y[j] = a[j] * b[j]; break;
        case OP_DIV: for (j = 0; j < len; ++j) y[j] = a[j] / b[j]; break;
        default: break;
    }
}

/* Evaluates `prog` for n output elements. outs[r] (may be NULL) receives register r for every
 * element; the last register normally has an output. Returns 0, or 1 on a bad argument. */
__attribute__((visibility("default")))
int oracle_fused(const oracle_instr* prog, int n_instr, const float* const* inputs, const int* in_kind,
                 const long long* in_period, int n_inputs, float* const* outs, long long n, int threads) {
    if (n_instr <= 0 || n_instr > 256) return 1;
    (void)n_inputs;
    const long long blocks = (n + ORACLE_BLOCK - 1) / ORACLE_BLOCK;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel num_threads(threads)
#endif
    {
        float* scratch = (float*)malloc((size_t)n_instr * ORACLE_BLOCK * sizeof(float));
        long long blk;
#ifdef _OPENMP
#pragma omp for schedule(static)
#endif
        for (blk = 0; blk < blocks; ++blk) {
            const long long start = blk * ORACLE_BLOCK;
            const int len = (int)((n - start) < ORACLE_BLOCK ? (n - start) : ORACLE_BLOCK);
            int r, j;
            for (r = 0; r < n_instr; ++r) {
                const oracle_instr* ins = &prog[r];
                float* dst = scratch + (size_t)r * ORACLE_BLOCK;
                if (ins->kind == ORACLE_LOAD) {
                    const float* in = inputs[ins->a];
                    if (in_kind[ins->a] == IN_CONTIGUOUS) {
                        memcpy(dst, in + start, (size_t)len * sizeof(float));
                    } else if (in_kind[ins->a] == IN_SCALAR) {
                        for (j = 0; j < len; ++j) dst[j] = in[0];
                    } else {
                        const long long period = in_period[ins->a];
                        long long pos = start % period;
                        for (j = 0; j < len; ++j) {
                            dst[j] = in[pos];
                            if (++pos == period) pos = 0;
                        }
                    }
                } else if (ins->kind == ORACLE_IMM) {
                    for (j = 0; j < len; ++j) dst[j] = ins->imm;
                } else if (ins->kind == ORACLE_UNARY) {
                    unary_block(ins->op, scratch + (size_t)ins->a * ORACLE_BLOCK, dst, len);
                } else {
                    binary_block(ins->op, scratch + (size_t)ins->a * ORACLE_BLOCK, scratch + (size_t)ins->b * ORACLE_BLOCK, dst, len);
                }
                if (outs[r] != NULL) memcpy(outs[r] + start, dst, (size_t)len * sizeof(float));
            }
        }
        free(scratch);
    }
    return 0;
}

/* Row-major C = A B in float32; k is walked in panels so that a panel of B stays in cache. */
__attribute__((visibility("default")))
void oracle_sgemm(const float* a, const float* b, float* c, long long m, long long k, long long n, int threads) {
    const long long KB = 256, NB = 512, MB = 4;
    const long long row_blocks = (m + MB - 1) / MB;
    long long ib;
#ifdef _OPENMP
    if (threads < 1) threads = 1;
#pragma omp parallel for schedule(static) num_threads(threads)
#endif
    for (ib = 0; ib < row_blocks; ++ib) {
        const long long i0 = ib * MB;
        const long long rows = (m - i0) < MB ? (m - i0) : MB;
        long long j0, k0, kk, j, r;
        for (r = 0; r < rows; ++r) memset(c + (i0 + r) * n, 0, (size_t)n * sizeof(float));
        for (j0 = 0; j0 < n; j0 += NB) {
            const long long j1 = j0 + NB < n ? j0 + NB : n;
            for (k0 = 0; k0 < k; k0 += KB) {
                const long long k1 = k0 + KB < k ? k0 + KB : k;
                if (rows == MB) {
                    float* c0 = c + (i0 + 0) * n;
                    float* c1 = c + (i0 + 1) * n;
                    float* c2 = c + (i0 + 2) * n;
                    float* c3 = c + (i0 + 3) * n;
                    for (kk = k0; kk < k1; ++kk) {
                        const float a0 = a[(i0 + 0) * k + kk], a1 = a[(i0 + 1) * k + kk];
                        const float a2 = a[(i0 + 2) * k + kk], a3 = a[(i0 + 3) * k + kk];
                        const float* brow = b + kk * n;
                        for (j = j0; j < j1; ++j) {
                            const float bv = brow[j];
                            c0[j] += a0 * bv;
                            c1[j] += a1 * bv;
                            c2[j] += a2 * bv;
                            c3[j] += a3 * bv;
                        }
                    }
                } else {
                    for (r = 0; r < rows; ++r) {
                        float* crow = c + (i0 + r) * n;
                        for (kk = k0; kk < k1; ++kk) {
                            const float av = a[(i0 + r) * k + kk];
                            const float* brow = b + kk * n;
                            for (j = j0; j < j1; ++j) crow[j] += av * brow[j];
                        }
                    }
                }
            }
        }
    }
}

__attribute__((visibility("default")))
int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
