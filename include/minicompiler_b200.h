/* C ABI of minicompiler-b200: the drop-in surface for the reference's
 * `bench/capi.cpp` (what Python/ctypes and any other FFI binds), plus a small set
 * of host-only introspection calls (`mcb_*`) used by tools and tests.
 *
 * Every `mc_*` entry point has the reference's name, argument meaning and return
 * convention; the citation beside each one is the reference function it replaces.
 * Handles are opaque; the caller owns every host buffer; device buffers persist
 * between mc_upload and any number of mc_enqueue calls. No exceptions cross this
 * boundary: failures are a NULL handle plus a message, or a non-zero int.
 */
#ifndef MINICOMPILER_B200_H
#define MINICOMPILER_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MC_EXPORT __attribute__((visibility("default")))

/* Parses `graph_path` with dim overrides `dims` ("M=64,N=4096" or ""), runs the pass pipeline
 * `passes` ("default", "none" or a list such as "dne,fold") and compiles for `backend`.
 * Only "cuda" is available here: this library is the GPU backend and has no CPU execution path.
 * Returns NULL and writes a NUL-terminated message to `error` on failure.
 * Replaces mc_compile (bench/capi.cpp:62-109). */
MC_EXPORT void* mc_compile(const char* graph_path, const char* dims, const char* passes, const char* backend,
                           char* error, int error_size);

/* Same, with the knobs the reference exposes only in C++ (CudaOptions,
 * include/minicompiler/cuda/cuda_backend.hpp:51-56) spelled as "key=value,key=value":
 *   device=N  matmul=<kernel name>  vectorize=0|1  fuse_epilogue=0|1  b_layout=auto|kn|transposed
 *   unroll=N  streaming=0|1  gemm_variant=N
 * `graph_text` non-NULL compiles that text instead of reading `graph_path`.
 * No counterpart in bench/capi.cpp (the reference CLI and C ABI cannot select a matmul kernel). */
MC_EXPORT void* mc_compile_ex(const char* graph_path, const char* graph_text, const char* dims, const char* passes,
                              const char* options, char* error, int error_size);

/* Replaces mc_num_inputs / mc_num_outputs / mc_output_elements (bench/capi.cpp:111-123). */
MC_EXPORT int mc_num_inputs(const void* handle);
MC_EXPORT int mc_num_outputs(const void* handle);
MC_EXPORT long long mc_output_elements(const void* handle, int k);
/* Element count of input k (no counterpart; saves callers from re-parsing the graph). */
MC_EXPORT long long mc_input_elements(const void* handle, int k);

/* Runs the graph on float32 host buffers in graph order, copies included. 0 on success.
 * Replaces mc_run (bench/capi.cpp:127-132). */
MC_EXPORT int mc_run(void* handle, const float* const* inputs, float* const* outputs);

/* Copies the host inputs into the executable's device buffers, where they stay for any number of
 * mc_enqueue calls. Replaces mc_upload (bench/capi.cpp:136-146). */
MC_EXPORT int mc_upload(void* handle, const float* const* inputs);
/* Launches the graph's kernels on `stream` (a cudaStream_t; NULL = the executable's own stream):
 * no copies, no synchronization. Replaces mc_enqueue (bench/capi.cpp:150-158). */
MC_EXPORT int mc_enqueue(void* handle, void* stream);
/* Waits for the device, then copies the outputs to host buffers.
 * Replaces mc_download (bench/capi.cpp:161-171). */
MC_EXPORT int mc_download(void* handle, float* const* outputs);
/* Waits for the device and reports a kernel that gave up a bounded wait (no counterpart:
 * the reference's kernels have no waits). */
MC_EXPORT int mc_synchronize(void* handle);

/* Kernel launches per mc_enqueue. Replaces mc_kernel_launches (bench/capi.cpp:174-182). */
MC_EXPORT int mc_kernel_launches(void* handle);
/* The kernel each matmul runs, comma-separated. Replaces mc_matmul_kernels (bench/capi.cpp:186-201). */
MC_EXPORT int mc_matmul_kernels(void* handle, char* out, int size);
/* SM clock of GPU 0 in MHz right now, 0 if unavailable. Replaces mc_gpu_sm_clock_mhz (bench/capi.cpp:204-210). */
MC_EXPORT double mc_gpu_sm_clock_mhz(void);
/* JSON description of GPU 0 with `clocks` summarized; 0 ok, 1 no GPU, 2 buffer too small.
 * Replaces mc_gpu_device_json (bench/capi.cpp:215-231). */
MC_EXPORT int mc_gpu_device_json(const double* clocks, int n, char* out, int size);
/* Replaces mc_release (bench/capi.cpp:233-235). */
MC_EXPORT void mc_release(void* handle);

/* The message of the last failing mc_* / mcb_* call on this thread (no counterpart: the
 * reference's int-returning calls drop their message). */
MC_EXPORT const char* mc_last_error(void);

/* ---- additions for multi-GPU replication and zero-copy callers (no counterparts) ---- */

/* Device address and size of the packed constants of a compiled graph, so that one collective can
 * replicate them; after overwriting the range call mc_refresh_constants. */
MC_EXPORT int mc_constants_region(void* handle, void** device_ptr, size_t* bytes);
MC_EXPORT int mc_refresh_constants(void* handle);
/* The same two steps done by the library: one NCCL broadcast of `root`'s constants to every rank of `comm`
 * (a handle from mcd_nccl_init, include/minicompiler_b200_device.h) followed by mc_refresh_constants; and an
 * all-gather of output k, of which every rank holds its rows, into `device_dst` (world_size times the output's
 * size, a device pointer). Both return when the data is in place. A rank that does not answer within the
 * communicator's timeout aborts the communicator; the call then fails with a message in mc_last_error().
 * These replace, on every rank but the root, the reference's per-constant blocking upload at load time
 * (src/cuda/cuda_backend.cpp:237-240). */
MC_EXPORT int mc_replicate_constants(void* handle, void* comm, int root);
MC_EXPORT int mc_gather_output(void* handle, int k, void* comm, void* device_dst);
/* Device address of the 32-bit status word of a compiled graph, or NULL in *device_ptr when none of its
 * kernels can wait. A tensor-core matmul that gives up a bounded wait ORs a code into it; mc_synchronize and
 * mc_download then fail with a message and clear it. Exposed so that this error path can be exercised from
 * the host (write a non-zero value with mcd_copy_h2d) without making any kernel wait. */
MC_EXPORT int mc_status_word_ptr(void* handle, void** device_ptr);
/* Row slices mc_run cuts a call on pinned host buffers into, so that the copy-in of one slice, the kernels of
 * the previous and the copy-out of the one before overlap (option host_io_row_slices, default 16); 0 when the
 * graph's rows are not independent, it moves too little, or it is a single streaming kernel (which has a
 * pipeline of its own). Results are bit-identical to the unsliced run. */
MC_EXPORT int mc_row_slices(void* handle);
/* Device address of input / output k (float32, dense, graph layout). */
MC_EXPORT int mc_input_device_ptr(void* handle, int k, void** device_ptr, size_t* elements);
MC_EXPORT int mc_output_device_ptr(void* handle, int k, void** device_ptr, size_t* elements);
/* Bytes of intermediate storage after buffer reuse, and of the whole device arena. */
MC_EXPORT long long mc_intermediate_bytes(void* handle);
MC_EXPORT long long mc_arena_bytes(void* handle);
/* NVRTC time spent compiling this graph's kernels, in ms. */
MC_EXPORT double mc_jit_compile_ms(void* handle);
/* The generated kernel sources, separated by "\n// ----\n". Returns the length needed. */
MC_EXPORT int mc_kernel_sources(void* handle, char* out, int size);

/* Batch partitioning: rewrites `dims` so that dim `batch_dim` becomes the share of `rank` out of
 * `world_size` (dim value must divide evenly) after checking that every tensor carrying that dim
 * carries it only as its leading extent and that no constant or matmul right-hand side carries it.
 * Writes the new dims string to `out_dims` and this rank's first row to `row_offset`.
 * 0 ok; non-zero with a message in mc_last_error() when the graph cannot be sharded that way. */
MC_EXPORT int mc_shard_dims(const char* graph_path, const char* dims, const char* batch_dim, int rank, int world_size,
                            char* out_dims, int out_size, long long* row_offset, long long* rows);

/* ---- host-only introspection (needs no GPU) ---- */

/* Parses and optimizes without compiling. `text` non-NULL is parsed instead of reading `path`. */
MC_EXPORT void* mcb_graph_open(const char* path, const char* text, const char* dims, const char* passes, char* error,
                               int error_size);
MC_EXPORT void mcb_graph_close(void* graph);
/* Each writes a NUL-terminated string into `out` and returns the length needed (excluding NUL). */
MC_EXPORT int mcb_graph_print(const void* graph, char* out, int size);           /* print_graph */
MC_EXPORT int mcb_graph_stats_json(const void* graph, char* out, int size);      /* compute_stats + pass reports */
MC_EXPORT int mcb_graph_plan_json(const void* graph, int pool_outputs, char* out, int size); /* plan_memory */
MC_EXPORT int mcb_graph_fusion_groups(const void* graph, char* out, int size);   /* find_fusion_groups, names */
MC_EXPORT int mcb_graph_emit_cuda(const void* graph, const char* options, char* out, int size); /* --emit-cuda */
MC_EXPORT int mcb_graph_launch_plan(const void* graph, const char* options, int sm_count, char* out, int size);
/* Row slicing of mc_run on pinned memory (no counterpart: the reference copies in, runs, copies out): "none", or
 * "rows=<leading extent> cut=<names of the values cut by rows>"; with slice_rows > 0 followed by the printed graph
 * at that row count. -1 with a message when the slice-sized graph cannot be built. */
MC_EXPORT int mcb_graph_row_slicing(const void* graph, long long slice_rows, char* out, int size);
MC_EXPORT int mcb_graph_num_nodes(const void* graph);
/* Copies the values of constant node `name` (after the passes); returns the element count or -1. */
MC_EXPORT long long mcb_graph_constant(const void* graph, const char* name, float* out, long long capacity);
/* NVRTC-compiles every kernel the launch plan would generate, for sm_100a, without loading it. 0 ok. */
MC_EXPORT int mcb_graph_check_kernels(const void* graph, const char* options, int sm_count);
/* The CUDA text the launch plan generates, step by step (elementwise, reduction and row-fused kernels, matmul
 * epilogues); same return convention as mcb_graph_launch_plan. Unlike `--emit-cuda`, which follows the
 * reference and prints one kernel per graph node (tools/mcc.cpp:200-210), this is what actually runs. */
MC_EXPORT int mcb_graph_plan_sources(const void* graph, const char* options, int sm_count, char* out, int size);

/* 1 when kernels may read and write `count` caller buffers in place (mc_run on pinned memory): vectorised kernels
 * move 128 bits per access, so every buffer must start on a 16-byte boundary; otherwise mc_run stages copies. */
MC_EXPORT int mcb_in_place_pointers_ok(const void* const* pointers, int count, int any_vectorized);
MC_EXPORT void mcb_uniform_values(float* out, long long count, unsigned long long seed, float lo, float hi);
MC_EXPORT int mcb_split_k_splits(int m, int n, int k, int sm_count, int blocks_per_sm);
/* K splits `auto` adds on B200 to an FP32 problem the reference's rule leaves whole, when its 128 x 128 tiles share
 * out badly over the SMs (1 = none); no counterpart in the reference, whose rule was calibrated on one 30-SM GPU
 * (README.md:557-560). */
MC_EXPORT int mcb_balanced_fp32_splits(int m, int n, int k, int sm_count);
MC_EXPORT int mcb_tensor_core_splits(int m, int n, int k, int sm_count, int elem_bytes);
/* Columns per tile (256, 128 or 64) the tcgen05 path uses for an unsplit m x n x k problem; no counterpart in the
 * reference, whose tensor-core kernel has one tile shape (src/cuda/matmul_tensor_core.cu:27-35). */
MC_EXPORT int mcb_tensor_core_tile_n(int m, int n, int k, int sm_count, int elem_bytes);
/* Name of the kernel `kernel_name` resolves to for this shape ("auto" -> "split_k" / "double_buffered");
 * NULL with a message in mc_last_error() for an unknown name. */
MC_EXPORT const char* mcb_resolve_matmul_kernel(const char* kernel_name, int m, int n, int k, int sm_count);

#ifdef __cplusplus
}
#endif

#endif /* MINICOMPILER_B200_H */
