// Run-time under vesta_gpu_b200.launch: NVRTC and the CUDA driver API behind a C ABI
// (declared in include/vesta_b200.h). libcuda and libnvrtc are opened on first use so that
// the library itself loads on a machine without a GPU driver.
#include <cuda.h>
#include <nvrtc.h>
#include <dlfcn.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>

#include "vesta_b200.h"

namespace {

thread_local std::string g_err = "";
std::string g_nvrtc_path;

int fail(int code, const std::string& what) {
    g_err = what;
    return code ? code : -1;
}

struct Driver {
    void* lib = nullptr;
    CUresult (*Init)(unsigned) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;
    CUresult (*CtxSetCurrent)(CUcontext) = nullptr;
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice) = nullptr;
    CUresult (*ModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*Occupancy)(int*, CUfunction, int, size_t) = nullptr;
    CUresult (*LaunchCooperative)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                                  unsigned, CUstream, void**) = nullptr;
    CUresult (*Launch)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                       CUstream, void**, void**) = nullptr;
    CUresult (*MemcpyHtoDAsync)(CUdeviceptr, const void*, size_t, CUstream) = nullptr;
    CUresult (*MemcpyDtoHAsync)(void*, CUdeviceptr, size_t, CUstream) = nullptr;
    CUresult (*StreamSynchronize)(CUstream) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                     const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};
Driver g_cu;

template <class F>
bool sym(void* lib, const char* name, F& out) {
    out = reinterpret_cast<F>(dlsym(lib, name));
    return out != nullptr;
}

int driver() {
    if (g_cu.lib) return 0;
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return fail(-1, std::string("cannot open libcuda.so.1: ") + dlerror());
    Driver d;
    bool ok = sym(lib, "cuInit", d.Init) && sym(lib, "cuGetErrorString", d.GetErrorString) &&
              sym(lib, "cuCtxGetCurrent", d.CtxGetCurrent) && sym(lib, "cuCtxSetCurrent", d.CtxSetCurrent) &&
              sym(lib, "cuDeviceGet", d.DeviceGet) && sym(lib, "cuDevicePrimaryCtxRetain", d.DevicePrimaryCtxRetain) &&
              sym(lib, "cuModuleLoadData", d.ModuleLoadData) && sym(lib, "cuModuleUnload", d.ModuleUnload) &&
              sym(lib, "cuModuleGetFunction", d.ModuleGetFunction) && sym(lib, "cuFuncSetAttribute", d.FuncSetAttribute) &&
              sym(lib, "cuOccupancyMaxActiveBlocksPerMultiprocessor", d.Occupancy) &&
              sym(lib, "cuLaunchCooperativeKernel", d.LaunchCooperative) && sym(lib, "cuLaunchKernel", d.Launch) &&
              sym(lib, "cuTensorMapEncodeTiled", d.TensorMapEncodeTiled) &&
              sym(lib, "cuMemcpyHtoDAsync_v2", d.MemcpyHtoDAsync) && sym(lib, "cuMemcpyDtoHAsync_v2", d.MemcpyDtoHAsync) &&
              sym(lib, "cuStreamSynchronize", d.StreamSynchronize);
    if (!ok) return fail(-1, "libcuda.so.1 lacks a required driver entry point");
    d.lib = lib;
    g_cu = d;
    return 0;
}

int cu(CUresult r, const char* call) {
    if (r == CUDA_SUCCESS) return 0;
    const char* s = nullptr;
    if (g_cu.GetErrorString) g_cu.GetErrorString(r, &s);
    return fail((int)r, std::string(call) + ": " + (s ? s : "unknown CUDA error") + " (" + std::to_string((int)r) + ")");
}

struct Nvrtc {
    void* lib = nullptr;
    nvrtcResult (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    nvrtcResult (*DestroyProgram)(nvrtcProgram*) = nullptr;
    nvrtcResult (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    nvrtcResult (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    nvrtcResult (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    nvrtcResult (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    const char* (*GetErrorString)(nvrtcResult) = nullptr;
};
Nvrtc g_rtc;

int rtc_open() {
    if (g_rtc.lib) return 0;
    std::vector<std::string> names;
    if (!g_nvrtc_path.empty()) names.push_back(g_nvrtc_path);
    if (const char* env = getenv("VESTA_NVRTC")) names.push_back(env);
    names.push_back("libnvrtc.so.12");
    names.push_back("/usr/local/cuda/lib64/libnvrtc.so.12");
    names.push_back("libnvrtc.so");
    void* lib = nullptr;
    std::string tried;
    for (auto& n : names) {
        lib = dlopen(n.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (lib) break;
        tried += n + " ";
    }
    if (!lib) return fail(-1, "cannot open libnvrtc (tried: " + tried + ")");
    Nvrtc r;
    bool ok = sym(lib, "nvrtcCreateProgram", r.CreateProgram) && sym(lib, "nvrtcDestroyProgram", r.DestroyProgram) &&
              sym(lib, "nvrtcCompileProgram", r.CompileProgram) && sym(lib, "nvrtcGetProgramLogSize", r.GetProgramLogSize) &&
              sym(lib, "nvrtcGetProgramLog", r.GetProgramLog) && sym(lib, "nvrtcGetCUBINSize", r.GetCUBINSize) &&
              sym(lib, "nvrtcGetCUBIN", r.GetCUBIN) && sym(lib, "nvrtcGetErrorString", r.GetErrorString);
    if (!ok) return fail(-1, "libnvrtc lacks a required entry point");
    r.lib = lib;
    g_rtc = r;
    return 0;
}

struct Bound {
    CUfunction fn;
    unsigned grid, block, smem;
    std::vector<unsigned long long> vals;
    std::vector<void*> ptrs;
};

}  // namespace

extern "C" {

int vesta_rt_version(void) { return 1; }

const char* vesta_last_error(void) { return g_err.c_str(); }

int vesta_set_nvrtc_path(const char* path) {
    g_nvrtc_path = path ? path : "";
    return 0;
}

void vesta_free(void* p) { free(p); }

int vesta_nvrtc_compile(const char* src, const char* arch, const char* const* opts, int n_opts,
                        void** cubin, size_t* cubin_size, char** log) {
    if (cubin) *cubin = nullptr;
    if (cubin_size) *cubin_size = 0;
    if (log) *log = nullptr;
    if (!src || !arch || !cubin || !cubin_size) return fail(-1, "vesta_nvrtc_compile: null argument");
    if (int e = rtc_open()) return e;
    nvrtcProgram prog;
    nvrtcResult r = g_rtc.CreateProgram(&prog, src, "vesta.cu", 0, nullptr, nullptr);
    if (r != NVRTC_SUCCESS) return fail((int)r, std::string("nvrtcCreateProgram: ") + g_rtc.GetErrorString(r));
    std::string a = std::string("--gpu-architecture=") + arch;
    std::vector<const char*> o{a.c_str(), "-std=c++17"};
    for (int i = 0; i < n_opts; i++) o.push_back(opts[i]);
    nvrtcResult cr = g_rtc.CompileProgram(prog, (int)o.size(), o.data());
    size_t ln = 0;
    g_rtc.GetProgramLogSize(prog, &ln);
    std::string text(ln ? ln : 1, '\0');
    if (ln) g_rtc.GetProgramLog(prog, &text[0]);
    if (log) {
        *log = (char*)malloc(text.size() + 1);
        if (*log) { memcpy(*log, text.c_str(), text.size()); (*log)[text.size()] = 0; }
    }
    if (cr != NVRTC_SUCCESS) {
        g_rtc.DestroyProgram(&prog);
        return fail((int)cr, std::string("NVRTC failed:\n") + text.c_str());
    }
    size_t n = 0;
    r = g_rtc.GetCUBINSize(prog, &n);
    if (r != NVRTC_SUCCESS || n == 0) {
        g_rtc.DestroyProgram(&prog);
        return fail(r ? (int)r : -1, "nvrtcGetCUBINSize: no cubin (is the architecture a real sm_ target?)");
    }
    char* buf = (char*)malloc(n);
    if (!buf) { g_rtc.DestroyProgram(&prog); return fail(-1, "out of host memory"); }
    r = g_rtc.GetCUBIN(prog, buf);
    g_rtc.DestroyProgram(&prog);
    if (r != NVRTC_SUCCESS) { free(buf); return fail((int)r, std::string("nvrtcGetCUBIN: ") + g_rtc.GetErrorString(r)); }
    *cubin = buf;
    *cubin_size = n;
    return 0;
}

int vesta_init(int device) {
    if (int e = driver()) return e;
    if (int e = cu(g_cu.Init(0), "cuInit")) return e;
    CUcontext ctx = nullptr;
    if (int e = cu(g_cu.CtxGetCurrent(&ctx), "cuCtxGetCurrent")) return e;
    if (!ctx) {
        CUdevice dev;
        if (int e = cu(g_cu.DeviceGet(&dev, device), "cuDeviceGet")) return e;
        if (int e = cu(g_cu.DevicePrimaryCtxRetain(&ctx, dev), "cuDevicePrimaryCtxRetain")) return e;
        if (int e = cu(g_cu.CtxSetCurrent(ctx), "cuCtxSetCurrent")) return e;
    }
    return 0;
}

int vesta_module_load(const void* cubin, void** module) {
    if (!cubin || !module) return fail(-1, "vesta_module_load: null argument");
    if (int e = driver()) return e;
    CUmodule m;
    if (int e = cu(g_cu.ModuleLoadData(&m, cubin), "cuModuleLoadData")) return e;
    *module = (void*)m;
    return 0;
}

int vesta_module_unload(void* module) {
    if (!module) return 0;
    if (int e = driver()) return e;
    return cu(g_cu.ModuleUnload((CUmodule)module), "cuModuleUnload");
}

int vesta_module_get_function(void* module, const char* name, void** function) {
    if (!module || !name || !function) return fail(-1, "vesta_module_get_function: null argument");
    if (int e = driver()) return e;
    CUfunction f;
    if (int e = cu(g_cu.ModuleGetFunction(&f, (CUmodule)module, name), "cuModuleGetFunction")) return e;
    *function = (void*)f;
    return 0;
}

int vesta_func_set_max_dynamic_smem(void* function, int bytes) {
    if (int e = driver()) return e;
    return cu(g_cu.FuncSetAttribute((CUfunction)function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, bytes),
              "cuFuncSetAttribute(MAX_DYNAMIC_SHARED_SIZE_BYTES)");
}

int vesta_occupancy(void* function, int block_threads, size_t dynamic_smem, int* blocks_per_sm) {
    if (!blocks_per_sm) return fail(-1, "vesta_occupancy: null argument");
    if (int e = driver()) return e;
    return cu(g_cu.Occupancy(blocks_per_sm, (CUfunction)function, block_threads, dynamic_smem),
              "cuOccupancyMaxActiveBlocksPerMultiprocessor");
}

int vesta_launch_cooperative(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                             void* stream, void** args) {
    if (int e = driver()) return e;
    return cu(g_cu.LaunchCooperative((CUfunction)function, grid, 1, 1, block, 1, 1, dynamic_smem, (CUstream)stream, args),
              "cuLaunchCooperativeKernel");
}

int vesta_launch(void* function, unsigned grid, unsigned block, unsigned dynamic_smem, void* stream, void** args) {
    if (int e = driver()) return e;
    return cu(g_cu.Launch((CUfunction)function, grid, 1, 1, block, 1, 1, dynamic_smem, (CUstream)stream, args, nullptr),
              "cuLaunchKernel");
}

int vesta_step_bind(void* function, unsigned grid, unsigned block, unsigned dynamic_smem,
                    int n_args, const unsigned long long* device_pointers, void** bound) {
    if (!function || !bound || n_args < 0 || (n_args && !device_pointers)) return fail(-1, "vesta_step_bind: bad argument");
    Bound* b = new Bound;
    b->fn = (CUfunction)function;
    b->grid = grid; b->block = block; b->smem = dynamic_smem;
    b->vals.assign(device_pointers, device_pointers + n_args);
    b->ptrs.resize(n_args);
    for (int i = 0; i < n_args; i++) b->ptrs[i] = &b->vals[i];
    *bound = b;
    return 0;
}

int vesta_step_run(void* bound, void* stream, int steps) {
    if (!bound) return fail(-1, "vesta_step_run: not bound");
    if (int e = driver()) return e;
    Bound* b = (Bound*)bound;
    for (int i = 0; i < steps; i++) {
        CUresult r = g_cu.LaunchCooperative(b->fn, b->grid, 1, 1, b->block, 1, 1, b->smem, (CUstream)stream, b->ptrs.data());
        if (r != CUDA_SUCCESS) return cu(r, "cuLaunchCooperativeKernel");
    }
    return 0;
}

int vesta_step_host(void* bound, void* stream, unsigned long long tokens_dev, const void* tokens_host, size_t tokens_bytes,
                    unsigned long long result_dev, void* result_host, size_t result_bytes) {
    if (!bound) return fail(-1, "vesta_step_host: not bound");
    if (int e = driver()) return e;
    Bound* b = (Bound*)bound;
    CUstream st = (CUstream)stream;
    CUresult r;
    if (tokens_host && tokens_bytes) {
        r = g_cu.MemcpyHtoDAsync((CUdeviceptr)tokens_dev, tokens_host, tokens_bytes, st);
        if (r != CUDA_SUCCESS) return cu(r, "cuMemcpyHtoDAsync");
    }
    r = g_cu.LaunchCooperative(b->fn, b->grid, 1, 1, b->block, 1, 1, b->smem, st, b->ptrs.data());
    if (r != CUDA_SUCCESS) return cu(r, "cuLaunchCooperativeKernel");
    if (result_host && result_bytes) {
        r = g_cu.MemcpyDtoHAsync(result_host, (CUdeviceptr)result_dev, result_bytes, st);
        if (r != CUDA_SUCCESS) return cu(r, "cuMemcpyDtoHAsync");
    }
    r = g_cu.StreamSynchronize(st);
    if (r != CUDA_SUCCESS) return cu(r, "cuStreamSynchronize");
    return 0;
}

int vesta_tensor_map_rows(void* out, const void* base, unsigned long long row_elems, unsigned long long rows,
                          unsigned long long planes, unsigned box_elems, unsigned box_rows) {
    if (!out || !base) return fail(-1, "vesta_tensor_map_rows: null argument");
    if (int e = driver()) return e;
    if (box_elems * 2u != 128u || box_rows == 0 || box_rows > 256u || (row_elems * 2ull) % 16ull)
        return fail(-1, "vesta_tensor_map_rows: the box must be 128 bytes wide, at most 256 rows, rows a multiple of 16 bytes");
    // fp16 [planes][rows][row_elems]; box = box_rows rows of 64 elements of one plane; 128-byte swizzle: the 16-byte
    // piece c of row r lands at piece c ^ (r % 8) of its 128-byte row in shared memory
    const cuuint64_t dims[3] = {row_elems, rows, planes};
    const cuuint64_t strides[2] = {row_elems * 2ull, rows * row_elems * 2ull};
    const cuuint32_t box[3] = {box_elems, box_rows, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMap tm;
    CUresult r = g_cu.TensorMapEncodeTiled(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cu(r, "cuTensorMapEncodeTiled");
    memcpy(out, &tm, sizeof(tm));
    return 0;
}

int vesta_step_run_fused(void* bound, void* stream, int steps, int per_launch) {
    if (!bound) return fail(-1, "vesta_step_run_fused: not bound");
    if (int e = driver()) return e;
    Bound* b = (Bound*)bound;
    if (b->vals.empty() || per_launch < 1) return fail(-1, "vesta_step_run_fused: bad argument");
    while (steps > 0) {
        const int n = steps < per_launch ? steps : per_launch;
        b->vals.back() = (unsigned long long)(unsigned)n;          // the kernel's last parameter: steps in this launch
        CUresult r = g_cu.LaunchCooperative(b->fn, b->grid, 1, 1, b->block, 1, 1, b->smem, (CUstream)stream, b->ptrs.data());
        if (r != CUDA_SUCCESS) return cu(r, "cuLaunchCooperativeKernel");
        steps -= n;
    }
    b->vals.back() = 1ull;
    return 0;
}

void vesta_step_release(void* bound) { delete (Bound*)bound; }

}  // extern "C"
