/* Thin C-ABI device layer of minicompiler-b200.
 *
 * Everything the C++17 host side (lowering, planner, executable, C API) needs
 * from CUDA goes through these calls: plain pointers, integers and opaque
 * handles only, so no CUDA or C++ type crosses the line and the layer can be
 * replaced by a fake in host-only tests. It takes the place of the direct
 * CUDA-runtime / driver / NVRTC calls the reference makes from
 * src/cuda/cuda_backend.cpp:154-257, src/cuda/kernel_compiler.cpp:24-57,
 * src/cuda/device_info.cpp:33-73 and src/cuda/matmul_kernels.hpp:46-59.
 *
 * Conventions: every call returns 0 on success; on failure it returns non-zero
 * and mcd_last_error() (thread-local) describes it as "<call>: <CUDA text>".
 * `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 * stream). Unless stated otherwise calls act on the current device
 * (mcd_set_device).
 */
#ifndef MINICOMPILER_B200_DEVICE_H
#define MINICOMPILER_B200_DEVICE_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MCD_API __attribute__((visibility("default")))

/* ------------------------------------------------------------- device query
 * Replaces query_device / current_sm_clock_mhz (src/cuda/device_info.cpp:33-73). */
typedef struct mcd_device_info {
    char name[128];
    int cc_major;
    int cc_minor;
    int sm_count;
    int fp32_lanes_per_sm;
    double sm_clock_mhz;
    double max_sm_clock_mhz; /* NVML; 0 when unavailable */
    double mem_clock_mhz;
    int bus_width_bits;
    unsigned long long total_memory;
    int runtime_version;
    int driver_version;
    int max_smem_per_block_optin;
} mcd_device_info;

MCD_API const char* mcd_last_error(void);
MCD_API int mcd_device_count(int* count);
MCD_API int mcd_query_device(int device, mcd_device_info* out);
MCD_API double mcd_current_sm_clock_mhz(int device);
MCD_API int mcd_set_device(int device);

/* ------------------------------------------------------- memory and streams
 * Replaces DeviceBuffer / cudaMemcpy* / stream handling
 * (src/cuda/cuda_backend.cpp:56-78, :154-165, :186-196, :217-219). */
MCD_API int mcd_malloc(void** ptr, size_t bytes);
MCD_API int mcd_free(void* ptr);
MCD_API int mcd_memset(void* ptr, int byte, size_t bytes, void* stream);
MCD_API int mcd_copy_h2d(void* dst, const void* src, size_t bytes, void* stream);
MCD_API int mcd_copy_d2h(void* dst, const void* src, size_t bytes, void* stream);
MCD_API int mcd_copy_d2d(void* dst, const void* src, size_t bytes, void* stream);
/* The device-side address of pinned, mapped host memory (cudaHostAlloc / cudaHostRegister), for kernels that
 * read or write caller memory in place; non-zero when `host` is pageable or not addressable by the GPU. */
MCD_API int mcd_host_device_pointer(const void* host, void** device_alias);
MCD_API int mcd_host_register(void* ptr, size_t bytes);   /* pin caller memory (optional fast path) */
MCD_API int mcd_host_unregister(void* ptr);
MCD_API int mcd_stream_create(void** stream);
MCD_API int mcd_stream_destroy(void* stream);
MCD_API int mcd_stream_synchronize(void* stream);
MCD_API int mcd_device_synchronize(void);
MCD_API int mcd_event_create(void** event);
MCD_API int mcd_event_destroy(void* event);
MCD_API int mcd_event_record(void* event, void* stream);
MCD_API int mcd_stream_wait_event(void* stream, void* event); /* later work on `stream` waits for `event` */
MCD_API int mcd_event_elapsed_ms(void* start, void* stop, float* ms); /* waits for `stop` */
/* Records `event` as a node of the CUDA graph being captured on `stream`, so that two of them bracket kernels
 * inside a replayed graph and their difference leaves out the host's launch cost - how the reference times a
 * single matmul (bench/bench_cuda.cpp:445-493). */
MCD_API int mcd_event_record_external(void* event, void* stream);
/* Named ranges for Nsight tools (NVTX), as the reference's profile suite wraps each launch
 * (bench/bench_cuda.cpp:860-928, nvtxRangePushA at :873). No-ops unless a tool is attached. */
MCD_API int mcd_range_push(const char* label);
MCD_API int mcd_range_pop(void);

/* -------------------------------------------------------- run-time kernels
 * Replaces KernelCompiler::get + cuLaunchKernel + the occupancy query
 * (src/cuda/kernel_compiler.cpp:24-57, src/cuda/cuda_backend.cpp:174-175,
 * :311-317). Compiles CUDA C++ to an sm_100a cubin with NVRTC and loads it
 * into `device`'s primary context; results are cached process-wide, keyed by
 * (device, options, hash of the source, kernel name), so a kernel is never
 * launched on a device other than the one its module was loaded for. NVRTC
 * runs outside the cache's lock. Each successful call takes one reference. */
MCD_API int mcd_jit_kernel(int device, const char* source, const char* kernel_name, const char* options,
                           void** function, double* compile_ms);
/* Gives back one reference taken by mcd_jit_kernel. A kernel nobody holds stays loaded while few such
 * kernels exist and is unloaded, least recently used first, beyond that; never launch it after the release. */
MCD_API int mcd_jit_release(void* function);
/* Loaded modules, and how many of them nobody holds (for tests and leak hunting). */
MCD_API int mcd_jit_cache_stats(long long* modules, long long* idle);
MCD_API int mcd_jit_occupancy(void* function, int block_threads, size_t dynamic_smem, int* blocks_per_sm);
MCD_API int mcd_jit_set_dynamic_smem(void* function, size_t bytes);
MCD_API int mcd_launch(void* function, unsigned grid_x, unsigned grid_y, unsigned grid_z, unsigned block_x,
                       size_t dynamic_smem, void* stream, void** params);
/* The same with thread-block clusters of `cluster_x` CTAs along x (grid_x a multiple of it). */
MCD_API int mcd_launch_cluster(void* function, unsigned grid_x, unsigned cluster_x, unsigned block_x, size_t dynamic_smem,
                               void* stream, void** params);
/* Launch as a programmatic dependent of the kernel launched before it on `stream`: the blocks may become resident
 * while that kernel drains (once all of its CTAs have executed griddepcontrol.launch_dependents or exited); the
 * kernel must execute griddepcontrol.wait before it touches what its predecessor wrote. */
MCD_API int mcd_launch_dependent(void* function, unsigned grid_x, unsigned block_x, size_t dynamic_smem, void* stream,
                                 void** params);
/* Launch-list replay (the reference names CUDA-graph replay of enqueue as its next step, README.md:554-556).
 * Between begin and end every launch issued on `stream` through this layer is recorded instead of run;
 * end returns an executable graph that mcd_graph_launch replays on any stream of the same device. */
MCD_API int mcd_graph_begin_capture(void* stream);
MCD_API int mcd_graph_end_capture(void* stream, void** graph_exec);
MCD_API int mcd_graph_launch(void* graph_exec, void* stream);
MCD_API int mcd_graph_destroy(void* graph_exec);
/* Number of kernel launches issued through this layer by the calling process. */
MCD_API unsigned long long mcd_launch_count(void);

/* ------------------------------------------------------------- collectives
 * NCCL over NVLink for the batch-sharded multi-GPU path: one broadcast replicates the packed constants at load
 * time, an all-gather assembles an output where the caller wants one. They take the place of the per-constant
 * blocking upload of src/cuda/cuda_backend.cpp:237-240 on every rank but the root. libnccl.so.2 (or the file named
 * by the environment variable MCD_NCCL_LIBRARY) is loaded at run time. Communicators are non-blocking: every call
 * polls the communicator's state for at most `timeout_s`; a call that does not finish in time, or an asynchronous
 * NCCL error, aborts the communicator (ncclCommAbort) and returns non-zero instead of leaving the rank hung.
 * `comm` handles are opaque; buffers are device pointers on the communicator's device. */
#define MCD_NCCL_ID_BYTES 128
MCD_API int mcd_nccl_available(void);                 /* 1 when NCCL could be loaded */
MCD_API int mcd_nccl_unique_id(char* id);             /* fills MCD_NCCL_ID_BYTES; call on one rank, share by any means */
MCD_API int mcd_nccl_init(void** comm, int world_size, int rank, const char* id, int device, double timeout_s);
MCD_API int mcd_nccl_broadcast(void* comm, void* buffer, size_t bytes, int root, void* stream);
MCD_API int mcd_nccl_all_gather(void* comm, const void* send, void* recv, size_t bytes_per_rank, void* stream);
/* Waits (bounded) until everything enqueued on `stream` has run, watching the communicator for errors. */
MCD_API int mcd_nccl_wait(void* comm, void* stream);
MCD_API int mcd_nccl_abort(void* comm);               /* after it every call on `comm` fails; destroy still frees it */
MCD_API int mcd_nccl_destroy(void* comm);
/* Host-only test hooks: replace NCCL by a stand-in that touches no GPU and no network. `failing_call` (an NCCL
 * function name, or NULL) returns `error_code`; with stay_in_progress the stand-in never leaves the in-progress
 * state, so the bounded polls run out. mcd_nccl_fake_aborts counts ncclCommAbort calls since installation. */
MCD_API int mcd_nccl_install_fake(const char* failing_call, int error_code, int stay_in_progress);
MCD_API int mcd_nccl_remove_fake(void);
MCD_API int mcd_nccl_fake_aborts(void);

/* ------------------------------------------------------- built-in kernels */

/* 16-bit formats of tensor-core operands. */
#define MCD_HALF_BF16 1
#define MCD_HALF_F16 2

/* dst[r*dst_pitch + c] = round-to-nearest-even(src[r*src_pitch + c]) for an
 * [rows, cols] matrix, or dst[c*dst_pitch + r] when `transpose` is non-zero.
 * This is the rounding the reference applies while staging tiles
 * (src/cuda/matmul_tensor_core.cu:45-57), done once per tensor instead. */
MCD_API int mcd_cast_f32_to_half(int half_kind, const float* src, void* dst, long long rows, long long cols,
                                 long long src_pitch, long long dst_pitch, int transpose, void* stream);
/* dst[c*dst_pitch + r] = src[r*src_pitch + c] in fp32 (operand re-layout for TF32). */
MCD_API int mcd_transpose_f32(const float* src, float* dst, long long rows, long long cols, long long src_pitch,
                              long long dst_pitch, void* stream);

/* Arithmetic of a matmul launch. */
#define MCD_GEMM_F32 0  /* FP32 FMA, exact path */
#define MCD_GEMM_TF32 1 /* tcgen05 kind::tf32 */
#define MCD_GEMM_BF16 2 /* tcgen05 kind::f16, bf16 operands */
#define MCD_GEMM_F16 3  /* tcgen05 kind::f16, fp16 operands */

/* Up to 6 extra operands of a fused epilogue. */
#define MCD_MAX_EPILOGUE_INPUTS 6

/* One matmul launch, C[m,n] = epilogue(A[m,k] * B[k,n]); replaces launch_matmul
 * (src/cuda/matmul_kernels.hpp:46-48) and its split-K helpers (:17-59).
 *
 *  a, b        operands. MCD_GEMM_F32 / TF32: float, row-major, leading dimensions lda/ldb in
 *              elements. BF16/F16: 16-bit, same layouts. When `b_transposed` is non-zero, b holds
 *              B^T, i.e. [n,k] row-major with leading dimension ldb.
 *  c, c16      outputs: float [m,n] with leading dimension ldc (may be NULL) and/or a 16-bit copy
 *              of kind `c16_kind` with leading dimension ldc16 (may be NULL).
 *  splits      > 1 divides K; partial sums go to `workspace` (splits*m*n floats) and are added in a
 *              fixed order, so results do not depend on scheduling. With variant bit 64 a tensor-core
 *              matmul whose effective split count is 2, 4 or 8 adds them inside one launch instead (the K
 *              slices of a tile form a thread-block cluster and meet in distributed shared memory, same
 *              order, same bits): it then needs no workspace and mcd_gemm_launches() is 1.
 *  function    NULL: the built-in kernel without epilogue. Otherwise a kernel obtained from
 *              mcd_jit_kernel for the source returned by mcd_gemm_source(arith) with a generated
 *              `mc_epilogue`; `epilogue_inputs` are its extra operands.
 *  reduce_function  same, for the split-K reduction kernel (mcd_gemm_source(-1)).
 */
typedef struct mcd_gemm_args {
    int arith;
    int m, n, k;
    const void* a;
    const void* b;
    long long lda, ldb;
    int b_transposed;
    float* c;
    long long ldc;
    void* c16;
    int c16_kind;
    long long ldc16;
    int splits;
    float* workspace;
    void* function;
    void* reduce_function;
    const float* epilogue_inputs[MCD_MAX_EPILOGUE_INPUTS];
    int num_epilogue_inputs;
    unsigned int* status; /* device word: a kernel that gives up a bounded wait ORs an error code in */
    int variant;          /* tuning variant, 0 = default. Bits: 2 no half-tile tails; 4 never / 8 always the SM-pair
                             kernel; 16 always / 32 never its two-tile form; 64 split tensor-core matmuls add their
                             partial tiles inside thread-block clusters instead of through the workspace and a second
                             launch; 128 outputs stored from registers instead of through the TMA unit; 512 never /
                             1024 always the TMA-fed FP32 kernel; 2048 the split-K reduction as a plain launch;
                             32768 the SM-pair kernels as plain launches (default: programmatic dependents of the
                             launch in front of them) */
    int tile_n;           /* tensor-core arithmetic: columns per tile, 0 or 256 = default, 128 or 64 = narrower tiles
                             (one-CTA kernel): small unsplit problems, and single rows of tiles with fewer K slices */
    int has_epilogue;     /* non-zero when the launch carries a generated epilogue; set it before asking for the
                             entry point as well, kernel selection depends on it */
} mcd_gemm_args;

MCD_API int mcd_gemm(const mcd_gemm_args* args, void* stream);
/* Kernel launches one mcd_gemm call issues (1, or 2 when it splits K). */
MCD_API int mcd_gemm_launches(const mcd_gemm_args* args);
/* CUDA C++ source of a GEMM kernel family, for epilogue specialisation: the caller puts a
 * generated `mc_epilogue` in front of it and compiles it with mcd_jit_kernel.
 * arith = MCD_GEMM_*, or -1 for the split-K reduction. */
MCD_API const char* mcd_gemm_source(int arith);
/* The entry point inside that source which mcd_gemm would launch for `args` (it depends on the
 * arithmetic, on operand alignment and on the layout of B); NULL args: the reduction kernel. */
MCD_API const char* mcd_gemm_entry_point(const mcd_gemm_args* args);
/* Dynamic shared memory the entry point needs (set it with mcd_jit_set_dynamic_smem). */
MCD_API size_t mcd_gemm_dynamic_smem(int arith);
/* Host-only check of the bookkeeping behind per-device kernel set-up (the opt-in to large dynamic shared
 * memory is kept per device): for a sequence of device ordinals, first[i] = 1 where a launch on
 * devices[i] would run the set-up, 0 where it was done by an earlier element. Touches no GPU. */
MCD_API int mcd_per_device_once_probe(const int* devices, int count, int* first);
/* How many thread-block clusters of `cluster_size` CTAs of the one-CTA tensor-core kernel the current device can run
 * at once (cudaOccupancyMaxActiveClusters): a split matmul that reduces inside clusters runs in one wave only when
 * its tiles do not exceed this. */
MCD_API int mcd_gemm_max_active_clusters(int arith, int b_transposed, int cluster_size, int* clusters);
/* Whether tcgen05 kernels can run on `device` (compute capability 10.x). */
MCD_API int mcd_tensor_core_supported(int device, int arith);

/* Bytes of built-in scratch behind mcd_gemm_f32_split_no_alloc (held, from the first call on it
 * until the process exits, by every GPU the entry point is used on). */
#define MCD_NO_ALLOC_SCRATCH_BYTES (16u << 20)

/* FP32 split-K matmul that allocates nothing: C[m,n] = A[m,k] * B[k,n], all dense row-major
 * float (lda = k, ldb = n, ldc = n), K divided into `splits` slices whose partial sums are
 * added in slice order, exactly as mcd_gemm(MCD_GEMM_F32) does with a caller workspace - and
 * bit-identical to it for the same split count.
 *
 * It has no counterpart in the reference. It exists for callers that cannot call cudaMalloc:
 * a process whose own pool already owns all of HBM, or code on a latency-critical path that
 * cannot take the device-wide synchronisation an allocation implies. The partial sums go to
 * an array built into the library instead of a workspace, so
 *   - slices * m * n * 4 bytes must not exceed MCD_NO_ALLOC_SCRATCH_BYTES (the call fails with
 *     a message otherwise; use fewer splits or mcd_gemm with your own workspace);
 *   - all calls on one GPU share that array: two calls that overlap on the GPU (different
 *     streams) race on it. Calls on one stream are safe. Nothing in it needs clearing between
 *     calls, every partial sum is rewritten before it is read;
 *   - the array comes into being on the first call per GPU: CUDA loads the module that owns it lazily, so
 *     that one call (cudaGetSymbolAddress, with that GPU current) makes the driver set aside the 16 MiB and may
 *     synchronise the device. Make it at start-up - a tiny problem with splits = 1 is enough - BEFORE the
 *     caller's own pool takes the rest of HBM (afterwards it can fail with out-of-memory) and before any stream
 *     capture. Every later call on that GPU allocates nothing and synchronises nothing.
 * The entry point itself calls no cudaMalloc, cudaFree or allocating library routine. */
MCD_API int mcd_gemm_f32_split_no_alloc(const float* a, const float* b, float* c, int m, int n, int k, int splits,
                                        void* stream);

#ifdef __cplusplus
}
#endif

#endif /* MINICOMPILER_B200_DEVICE_H */
