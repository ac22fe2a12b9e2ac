/* C ABI of libvesta_b200.so: the run-time under vesta_gpu_b200.launch.
 *
 * The reference reaches NVRTC and the CUDA driver through the Python packages cuda-bindings
 * and nvidia-cuda-nvrtc (vesta/launch.py:5-7). Each entry point below stands for the calls the
 * reference makes at the cited lines, behind plain pointers and sizes, so that any host
 * language with a C FFI can drive the decode-step kernel. Every function returns 0 on success
 * and a non-zero CUDA / NVRTC status otherwise; vesta_last_error() then describes the failure.
 * libcuda and libnvrtc are opened lazily, so the library loads on a machine with no GPU.
 */
#ifndef VESTA_B200_H
#define VESTA_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ABI version of this header. */
int vesta_rt_version(void);

/* Text of the last failure on the calling thread (never NULL). */
const char* vesta_last_error(void);

/* Optional: path of the libnvrtc to open (default: the system libnvrtc.so.12). */
int vesta_set_nvrtc_path(const char* path);

/* vesta/launch.py:17-27 compile_cubin: nvrtcCreateProgram, nvrtcCompileProgram,
 * nvrtcGetProgramLog, nvrtcGetCUBIN. arch e.g. "sm_100a". On return *cubin / *log are
 * malloc'ed (release with vesta_free); *log holds the compiler log also on failure. */
int vesta_nvrtc_compile(const char* src, const char* arch, const char* const* opts, int n_opts,
                        void** cubin, size_t* cubin_size, char** log);
void vesta_free(void* p);

/* vesta/launch.py:32 cuInit; makes sure a context is current on the calling thread
 * (the primary context of `device` is retained and set if none is). */
int vesta_init(int device);

/* vesta/launch.py:35-36 cuModuleLoadData / cuModuleGetFunction. */
int vesta_module_load(const void* cubin, void** module);
int vesta_module_unload(void* module);
int vesta_module_get_function(void* module, const char* name, void** function);

/* vesta/launch.py:38-40 cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES) and
 * cuOccupancyMaxActiveBlocksPerMultiprocessor. */
int vesta_func_set_max_dynamic_smem(void* function, int bytes);
int vesta_occupancy(void* function, int block_threads, size_t dynamic_smem, int* blocks_per_sm);

/* vesta/launch.py:68-70 cuLaunchCooperativeKernel: 1-D grid and block, on `stream`
 * (a CUstream, 0 for the default stream). args: one pointer per kernel parameter. */
int vesta_launch_cooperative(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                             void* stream, void** args);

/* Plain (non-cooperative) launch, used for the one-time weight packing kernel. */
int vesta_launch(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                 void* stream, void** args);

/* vesta/launch.py:57-70 bind + launch: the argument list is fixed once (every kernel parameter
 * is a device pointer), after which a step costs one call. vesta_step_run launches `steps`
 * decode steps back to back on `stream` without returning to the caller in between. */
int vesta_step_bind(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                    int n_args, const unsigned long long* device_pointers, void** bound);
/* A TMA descriptor (128 bytes, written to `out` in host memory; copy it to 64-byte aligned device memory) for a
 * cache of fp16 rows laid out [planes][rows][row_elems]: one copy brings `box_rows` consecutive rows of 64
 * elements (128 bytes, one head) of one plane into shared memory with the 128-byte swizzle. The step kernel
 * reads its K and V tiles through eight of these (K and V, boxes of 32, 64, 96 and 128 rows) and the embedding
 * table through a ninth (boxes of 128 rows). No counterpart in the
 * reference, whose generated folds read the cache with ordinary vector loads (vesta/lower.py:947-956). */
int vesta_tensor_map_rows(void* out, const void* base, unsigned long long row_elems, unsigned long long rows,
                          unsigned long long planes, unsigned box_elems, unsigned box_rows);
int vesta_step_run(void* bound, void* stream, int steps);
/* The same, with up to `per_launch` decode steps inside one launch (the kernel's last parameter is the number
 * of steps; it feeds its own token and position between them). The bound argument list must end with that
 * parameter. No counterpart in the reference, which launches once per step. */
int vesta_step_run_fused(void* bound, void* stream, int steps, int per_launch);
/* One decode step for a caller whose tokens live in host memory: copies `tokens_bytes` bytes from tokens_host to
 * the device address tokens_dev (the residue x), launches the bound step once, copies `result_bytes` bytes from
 * result_dev (e.g. the `next` values in the scratch) to result_host and waits for the stream. One call instead of
 * the copy / step / read-back / synchronise sequence of the reference's host loop (bench/g0_bench.py:175-177 with
 * the token copied from and to the host). Either copy is skipped when its host pointer is null. */
int vesta_step_host(void* bound, void* stream, unsigned long long tokens_dev, const void* tokens_host, size_t tokens_bytes,
                    unsigned long long result_dev, void* result_host, size_t result_bytes);
void vesta_step_release(void* bound);

/* No counterpart in the reference: one decode step for callers that must not allocate device
 * memory (a plugin inside a host that owns all of it, a serving loop with a frozen memory plan).
 * Launches the compiled step function `function` (from vesta_module_get_function) exactly as
 * vesta_launch_cooperative would, but with the kernel's work space (fp32 scratch, counters, timing
 * sums, normally allocated by the caller) in a fixed array inside the library's device image,
 * vesta_static_scratch_bytes() bytes (4 MiB) per GPU for the life of the process. The caller passes
 * the residues (inputs, the KV cache), the packed weights, the plan table and the nine TMA
 * descriptors (vesta_tensor_map_rows, in device memory) it already owns (the KV cache must hold finite values in
 * unused rows: the attention stages rows in boxes of 32 and weighs the ones past the position with zero), the
 * sizes the lowering reported (scratch_floats, counters) and where the logits and next lie in the
 * scratch; the results are copied to logits_out / next_out (device or pinned host memory) on
 * `stream`. Allocates nothing; a step that needs more scratch than the array holds is refused with
 * an error (vesta_static_last_error) and nothing is launched. The array is shared by every call and
 * keeps the last call's contents: each call clears the range it uses first, and calls that overlap
 * on the GPU race on it. The first call on a device resolves the array's address and should be
 * made before any stream capture. The kernel's status word lives in the array as well, so it is
 * copied to status_out (4 bytes, device or pinned host memory, may be NULL) on `stream` with the
 * results: 0 = the step ran; 0x900 = refused (a position outside the cache or a token outside the
 * vocabulary; logits and next are then zero and x, t and the cache untouched); anything else = a
 * bounded wait gave up (phase in bits 8-15, CTA in bits 16-31). At most 56 residues. */
size_t vesta_static_scratch_bytes(void);
const char* vesta_static_last_error(void);
int vesta_step_static(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                      int n_residues, const unsigned long long* residue_pointers,
                      unsigned long long packed_weights, unsigned long long plan_table,
                      unsigned long long tensor_maps,
                      size_t scratch_floats, size_t counters,
                      size_t logit_offset, size_t logit_count, float* logits_out,
                      size_t next_offset, size_t next_count, float* next_out,
                      unsigned* status_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif
