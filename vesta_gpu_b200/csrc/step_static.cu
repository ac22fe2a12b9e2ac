// vesta_step_static: one decode step for callers that must not allocate.
//
// Who needs it: code that runs where device allocation is off limits: inside a serving loop with a
// frozen memory plan, in a plugin whose host owns every byte of device memory, or after start-up in
// a process that has handed its allocator the whole GPU. The ordinary path (launch.Kernel) has
// PyTorch allocate the step kernel's work space: the fp32 scratch S (logits, next, the state
// vectors z, the query, the attention partials, the arg-max keys), the barrier and status counters
// and the timing sums. Here that work space is a fixed array in the library's own device image:
// every GPU that loads the library holds VESTA_STATIC_SCRATCH_BYTES of it until the process exits.
// The step kernel is the same compiled function the ordinary path launches; only its scratch
// lives somewhere else, and its results are copied out of the scratch into buffers the caller owns.
//
// Rules that follow from sharing one array:
//   * a step whose scratch needs exceed the array is refused with an error, nothing is launched;
//   * the array keeps the last call's contents, so every call first clears what the kernel expects
//     to find zero (counters, arg-max keys; the whole used range is cleared, it is small);
//   * calls that overlap on the GPU (two streams, two threads) race on the array: one call at a
//     time per device, or order them on one stream;
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress, with that
//     device current) and caches it; make that first call before any stream capture begins;
//   * the kernel's status word (0 = the step ran; otherwise why it was refused or where a bounded wait
//     gave up, as Kernel.status() of the ordinary path reports it) lives in the array too, so the call
//     copies it out to `status_out` with the results: a refused step leaves logits and next at zero,
//     which would otherwise read as "token 0".
#include <cuda_runtime.h>
#include <mutex>
#include <string>

#include "vesta_b200.h"

#define VESTA_STATIC_SCRATCH_BYTES (4u << 20)
#define COUNTER_WORDS 2048                      // barrier / status words at the front of the array
#define TIMING_WORDS 2048                       // 64-bit timing sums behind them
#define HEADER_BYTES (COUNTER_WORDS * 4 + TIMING_WORDS * 8)
#define VESTA_STATIC_MAX_RESIDUES 56            // kernel parameters that are residues (the step program has 20 to 22)

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char vesta_static_scratch[VESTA_STATIC_SCRATCH_BYTES];

namespace {

// clears the first `words` 32-bit words of the array; device code may name the array directly
__global__ void clear_static_scratch(size_t words) {
    unsigned* w = reinterpret_cast<unsigned*>(vesta_static_scratch);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < words; i += (size_t)gridDim.x * blockDim.x) w[i] = 0u;
}

const int MAX_DEVICES = 64;
std::mutex g_lock;
unsigned char* g_base[MAX_DEVICES] = {nullptr};
thread_local std::string g_msg;

int fail(const std::string& what) {
    g_msg = what;
    return -1;
}

// device address of the array on the current device, looked up once per device
int scratch_base(unsigned char** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail("device ordinal out of range");
    std::lock_guard<std::mutex> hold(g_lock);
    if (!g_base[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, vesta_static_scratch);
        if (e != cudaSuccess || !p) return fail(std::string("cudaGetSymbolAddress(vesta_static_scratch): ") + cudaGetErrorString(e));
        g_base[dev] = static_cast<unsigned char*>(p);
    }
    *out = g_base[dev];
    return 0;
}

}  // namespace

extern "C" {

const char* vesta_static_last_error(void) { return g_msg.c_str(); }

size_t vesta_static_scratch_bytes(void) { return VESTA_STATIC_SCRATCH_BYTES; }

int vesta_step_static(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                      int n_residues, const unsigned long long* residue_pointers,
                      unsigned long long packed_weights, unsigned long long plan_table,
                      unsigned long long tensor_maps,
                      size_t scratch_floats, size_t counters,
                      size_t logit_offset, size_t logit_count, float* logits_out,
                      size_t next_offset, size_t next_count, float* next_out,
                      unsigned* status_out, void* stream) {
    // the argument array below holds the residues and the seven pointers and counts that follow them
    if (!function || n_residues < 0 || n_residues > VESTA_STATIC_MAX_RESIDUES || (n_residues && !residue_pointers))
        return fail("vesta_step_static: bad argument (at most " + std::to_string(VESTA_STATIC_MAX_RESIDUES) + " residues)");
    if (counters > COUNTER_WORDS)
        return fail("vesta_step_static: the program needs " + std::to_string(counters) + " counter words, the static scratch holds " +
                    std::to_string(COUNTER_WORDS));
    // compared before multiplying: a huge count must not wrap around into range
    if (scratch_floats > (VESTA_STATIC_SCRATCH_BYTES - HEADER_BYTES) / sizeof(float))
        return fail("vesta_step_static: this step needs " + std::to_string(scratch_floats) + " floats of scratch, the static scratch holds " +
                    std::to_string((size_t)(VESTA_STATIC_SCRATCH_BYTES - HEADER_BYTES) / sizeof(float)) + " (batch x vocabulary is too large for the no-allocation path)");
    const size_t need = HEADER_BYTES + scratch_floats * sizeof(float);
    if (logit_offset > scratch_floats || logit_count > scratch_floats - logit_offset ||
        next_offset > scratch_floats || next_count > scratch_floats - next_offset)
        return fail("vesta_step_static: output range outside the scratch");
    unsigned char* base = nullptr;
    if (scratch_base(&base)) return -1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // what the kernel expects to find zero: counters, timing sums, arg-max keys; clear the used range
    const size_t words = need / 4;
    clear_static_scratch<<<64, 256, 0, st>>>(words);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(std::string("clear_static_scratch: ") + cudaGetErrorString(e));

    // the step kernel's parameters: residues, then S, bar, TS, packed weights, plan table, K/V descriptors, steps per launch
    unsigned long long vals[VESTA_STATIC_MAX_RESIDUES + 7];
    void* args[VESTA_STATIC_MAX_RESIDUES + 7];
    int n = 0;
    for (; n < n_residues; n++) vals[n] = residue_pointers[n];
    vals[n++] = (unsigned long long)(base + HEADER_BYTES);              // S
    vals[n++] = (unsigned long long)base;                               // bar
    vals[n++] = (unsigned long long)(base + COUNTER_WORDS * 4);         // TS
    vals[n++] = packed_weights;
    vals[n++] = plan_table;
    vals[n++] = tensor_maps;
    vals[n++] = 1ull;                                                   // one decode step per launch
    for (int i = 0; i < n; i++) args[i] = &vals[i];
    if (vesta_launch_cooperative(function, grid, block, dynamic_smem, stream, args) != 0)
        return fail(std::string("vesta_step_static: ") + vesta_last_error());

    const float* S = reinterpret_cast<const float*>(base + HEADER_BYTES);
    if (logits_out && logit_count) {
        e = cudaMemcpyAsync(logits_out, S + logit_offset, logit_count * sizeof(float), cudaMemcpyDefault, st);
        if (e != cudaSuccess) return fail(std::string("copy of the logits: ") + cudaGetErrorString(e));
    }
    if (next_out && next_count) {
        e = cudaMemcpyAsync(next_out, S + next_offset, next_count * sizeof(float), cudaMemcpyDefault, st);
        if (e != cudaSuccess) return fail(std::string("copy of next: ") + cudaGetErrorString(e));
    }
    if (status_out) {
        e = cudaMemcpyAsync(status_out, base, sizeof(unsigned), cudaMemcpyDefault, st);       // bar[0]: the kernel's status word
        if (e != cudaSuccess) return fail(std::string("copy of the status word: ") + cudaGetErrorString(e));
    }
    return 0;
}

}  // extern "C"
