"""Device latency probe: cost of a grid-wide barrier on this GPU, for the variants considered for
the step kernel (one counter, fences, back-off, two levels, a go word, several counters, per-CTA
flags), alone and right after contended fp32 atomics. Cycles per barrier on CTA 0.

    python -m vesta_gpu_b200.latency_probe

Compiled with NVRTC and launched cooperatively through the C ABI, like the step kernel. Every spin
is bounded. The choice made in csrc/step_kernel.cuh (phase_end / phase_wait) rests on these numbers.
"""
import ctypes

import torch

from .launch import lib, ok, compile_cubin

SRC = r'''
typedef unsigned int u32; typedef unsigned long long u64;
__device__ __forceinline__ u32 ld_acquire(const u32* p) { u32 v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ u32 ld_relaxed(const u32* p) { u32 v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ u32 atom_add_acqrel(u32* p, u32 v) { u32 o; asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(o) : "l"(p), "r"(v) : "memory"); return o; }
#define LIMIT 4000000
extern "C" __global__ void micro(float* out, u32* bar, int iters, int variant) {
    const int tid = threadIdx.x, cta = blockIdx.x, ncta = gridDim.x;
    u32 gen = 0;
    float* vec = out + 64;
    __syncthreads();
    long long t0 = clock64();
    for (int i = 0; i < iters; i++) {
        if (variant >= 100) asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" :: "l"(vec + ((variant >= 200) ? (cta % 8) * 1024 : 0) + tid), "f"(1.0f) : "memory");
        const int v = variant % 100;
        __syncthreads();
        if (v == 1) {               // single counter, red.release + ld.acquire poll by thread 0
            gen += ncta;
            if (tid == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar) : "memory");
                int s = 0; while ((int)(ld_acquire(bar) - gen) < 0 && ++s < LIMIT) { }
            }
        } else if (v == 2) {        // fence + relaxed red, relaxed poll + fence
            gen += ncta;
            if (tid == 0) {
                asm volatile("fence.acq_rel.gpu;" ::: "memory");
                asm volatile("red.relaxed.gpu.global.add.u32 [%0], 1;" :: "l"(bar) : "memory");
                int s = 0; while ((int)(ld_relaxed(bar) - gen) < 0 && ++s < LIMIT) { }
                asm volatile("fence.acq_rel.gpu;" ::: "memory");
            }
        } else if (v == 3) {        // v1 + nanosleep in the poll loop
            gen += ncta;
            if (tid == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar) : "memory");
                int s = 0; while ((int)(ld_acquire(bar) - gen) < 0 && ++s < LIMIT) { __nanosleep(100); }
            }
        } else if (v == 4) {        // two-level: groups of 16 (atom), last of a group adds to the top counter; all poll the top
            gen += (ncta + 15) / 16;
            if (tid == 0) {
                const int g = cta / 16, gsz = min(16, ncta - g * 16);
                const u32 old = atom_add_acqrel(bar + 32 + g * 32, 1);
                if ((old % gsz) == gsz - 1) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar) : "memory");
                int s = 0; while ((int)(ld_acquire(bar) - gen) < 0 && ++s < LIMIT) { }
            }
        } else if (v == 5) {        // counter by atom, last arriver writes a go word that everybody polls
            gen += 1;
            if (tid == 0) {
                const u32 old = atom_add_acqrel(bar + 32, 1);
                if ((old % ncta) == ncta - 1) asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(bar), "r"(gen) : "memory");
                int s = 0; while ((int)(ld_acquire(bar) - gen) < 0 && ++s < LIMIT) { }
            }
        } else if (v == 6) {        // fence only
            if (tid == 0) asm volatile("fence.acq_rel.gpu;" ::: "memory");
        } else if (v == 7) {        // red.release only (no wait)
            if (tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar + 64 + (cta % 16) * 32) : "memory");
        } else if (v == 8) {        // 4 counters, thread 0 polls them one after the other
            gen += 1;
            if (tid == 0) {
                asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(bar + (cta % 4) * 32) : "memory");
                for (int k = 0; k < 4; k++) {
                    const u32 want = gen * ((ncta - k + 3) / 4);
                    int s = 0; while ((int)(ld_acquire(bar + k * 32) - want) < 0 && ++s < LIMIT) { }
                }
            }
        } else if (v == 9) {        // per-CTA flags, ONE poller thread per flag: thread i polls flag i
            gen += 1;
            if (tid == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(bar + cta), "r"(gen) : "memory");
            if (tid < ncta) { int s = 0; while ((int)(ld_relaxed(bar + tid) - gen) < 0 && ++s < LIMIT) { } }
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
        }
        __syncthreads();
    }
    long long t1 = clock64();
    if (cta == 0 && tid == 0) out[0] = (float)(t1 - t0) / iters;
}
'''


def main():
    L = lib(); torch.zeros(1, device='cuda'); ok(L.vesta_init(0))
    cubin = compile_cubin(SRC, cache=False)
    buf = ctypes.create_string_buffer(cubin, len(cubin))
    mod, fn = ctypes.c_void_p(), ctypes.c_void_p()
    ok(L.vesta_module_load(ctypes.cast(buf, ctypes.c_void_p), ctypes.byref(mod)))
    ok(L.vesta_module_get_function(mod, b'micro', ctypes.byref(fn)))
    out = torch.zeros(16384, device='cuda'); bar = torch.zeros(4096, dtype=torch.int32, device='cuda')
    names = {1: 'counter red.release/ld.acquire', 2: 'fence+relaxed', 3: 'counter+nanosleep', 4: 'two-level 16', 5: 'atom + go word', 6: 'fence only', 7: 'red.release only', 8: '4 counters serial poll', 9: 'flags, thread per flag'}
    for base in (0, 100, 200):
        for v in (1, 2, 3, 4, 5, 6, 7, 8, 9):
            bar.zero_(); torch.cuda.synchronize()
            vals = [out.data_ptr(), bar.data_ptr(), 300, base + v]
            store = (ctypes.c_ulonglong * 4)(*vals)
            ptrs = (ctypes.c_void_p * 4)(*[ctypes.addressof(store) + 8 * i for i in range(4)])
            ok(L.vesta_launch_cooperative(fn, torch.cuda.get_device_properties(0).multi_processor_count, 256, 0, None, ptrs)); torch.cuda.synchronize()
            print(('plain ' if base == 0 else 'after contended f32 atomics ' if base == 100 else 'after atomics spread over 8 copies '), names[v], round(float(out[0].item())), 'cycles', flush=True)


if __name__ == '__main__':
    main()
