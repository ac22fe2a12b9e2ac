// Shared by the step kernels (step_small.cuh: at most eight sequences; step_kernel.cuh: larger batches): types, thin
// wrappers around the PTX both use, the layout of the global counters and the bounded waits. lower.py places this
// text between the #defines of a configuration and the kernel text.

typedef unsigned int u32;
typedef unsigned long long u64;
typedef unsigned short u16;

#define NW V_NW
#define NCONS (NW * 32)
#ifndef V_NPROD
#define V_NPROD 1                       // producer warps behind the consumer warps
#endif
#define NTHREADS (NCONS + 32 * V_NPROD)
#define KT_D (V_D / 16)
#define JT_D (V_D / 16)
#define KT_F (V_F / 16)
#define FRAG_BYTES 512

// bar[] layout (u32): [0] status, [1] arrivals of the last phase, [2] abort flag, [3] steps done, [32] barrier counter
#define BAR_STATUS 0
#define BAR_DONE 1
#define BAR_ABORT 2
#define BAR_STEP 3                      // steps finished in this launch (0xffffffff: stop), cleared by its last step
#define BAR_COUNT 32

// every wait gives up after WAIT_NS nanoseconds (a step takes well under a millisecond; the lowering may set a
// shorter limit, which is how a test makes a wait run out)
#define WAIT_NS V_WAIT_NS
__device__ __forceinline__ u64 now_ns() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ u32 pack_h2(float lo, float hi) { u32 r; asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r; }
__device__ __forceinline__ float h_lo(u32 w) { float f; asm("{.reg .b16 l,h; mov.b32 {l,h}, %1; cvt.f32.f16 %0, l;}" : "=f"(f) : "r"(w)); return f; }
__device__ __forceinline__ float h_hi(u32 w) { float f; asm("{.reg .b16 l,h; mov.b32 {l,h}, %1; cvt.f32.f16 %0, h;}" : "=f"(f) : "r"(w)); return f; }
__device__ __forceinline__ float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 f2h(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }
__device__ __forceinline__ float fast_exp(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f)); return y; }

// tanh-GELU: a * v * (1 + tanh(b * (v + c * v^3))) with tanh(u) = 1 - 2 / (1 + e^(2u)) from the exponential and
// reciprocal units (absolute error of the tanh about 1e-7; the library tanhf costs some forty instructions)
__device__ __forceinline__ float gelu_tanh(float v) {
    const float u = V_GELU_B * (v + V_GELU_C * v * v * v);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u * 2.8853900817779268f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return V_GELU_A * v * (2.0f - 2.0f * r);
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint4& a, u32 b0, u32 b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" :: "n"(NCONS) : "memory"); }
// number of consumer threads with a non-zero predicate (a barrier over the consumer warps)
__device__ __forceinline__ int __syncthreads_count_cons(int pred) {
    int n;
    asm volatile("{.reg .pred p; setp.ne.s32 p, %1, 0; bar.red.popc.u32 %0, 1, %2, p;}" : "=r"(n) : "r"(pred), "n"(NCONS) : "memory");
    return n;
}
__device__ __forceinline__ u32 ld_acquire(const u32* p) { u32 v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ u32 ld_relaxed(const u32* p) { u32 v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void red_add(float* p, float v) { asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory"); }
__device__ __forceinline__ void mbar_init(u32 bar, u32 count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_arrive(u32 bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect(u32 bar, u32 bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_try(u32 bar, u32 parity) {
    u32 ok;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(u32 dst, const void* src, u32 bytes, u32 bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 16-byte asynchronous copies global (through L2 only) -> shared
__device__ __forceinline__ void cp16(void* dst, const void* src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory"); }
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ uint4 lds128(const unsigned char* p) { return *reinterpret_cast<const uint4*>(p); }
// the same from a 32-bit shared-memory address (explicit ld.shared: 32-bit address arithmetic, no generic-address path)
__device__ __forceinline__ uint4 lds128s(u32 a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint4 lds_acts(u32 a) {
#if V_ACT_LO
    return lds128s(a);
#else
    uint4 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    v.z = 0u; v.w = 0u;
    return v;
#endif
}
// one lane's part of an operand tile: (b0, b1) of the head and, if kept, (b0, b1) of the remainder
__device__ __forceinline__ uint4 lds_act(const unsigned char* p) {
#if V_ACT_LO
    return *reinterpret_cast<const uint4*>(p);
#else
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_uint4(v.x, v.y, 0u, 0u);
#endif
}

// a / w for small non-negative a (< 4096) and 1 <= w <= 64, with rcp = 1 / w: the integer division by a run-time
// divisor costs some thirty dependent instructions, this one four ((a + 0.5) / w is never within rounding of an integer)
__device__ __forceinline__ int qdiv(int a, float rcp) { return __float2int_rz(((float)a + 0.5f) * rcp); }
// 1 / w to within an ulp (one instruction): enough for qdiv, whose quotients stay 1/128 away from an integer
__device__ __forceinline__ float rcp_fast(int w) { float r; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"((float)w)); return r; }

// orderable key of (value, index): larger value wins, then the lower index
__device__ __forceinline__ u64 best_key(float v, u32 n) {
    u32 u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((u64)u << 32) | (u64)(0xFFFFFFFFu - n);
}

__device__ __noinline__ void give_up(u32* bar, u32 where, int cta) {
    atomicCAS(bar + BAR_STATUS, 0u, where | ((u32)cta << 16));
    atomicExch(bar + BAR_ABORT, 1u);
}

// slow path of a shared-memory barrier wait; returns false when the wait was abandoned
__device__ __noinline__ bool mbar_wait_slow(u32* bar, u32 mbar, u32 parity, u32 where, int cta, const volatile int* stop) {
    const u64 t0 = now_ns();
    u32 spins = 0;
    while (!mbar_try(mbar, parity)) {
        if (*stop) return false;                      // the consumers of this CTA have left (the launch ended early)
        if ((++spins & 63u) == 0) {
            if (ld_relaxed(bar + BAR_ABORT)) return false;
            if (now_ns() - t0 > WAIT_NS) { give_up(bar, where, cta); return false; }
        }
    }
    return true;
}

__device__ __forceinline__ void ldsm4(u32 (&r)[4], const unsigned char* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm4t(u32 (&r)[4], const unsigned char* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_r(float (&c)[4], const u32 (&a)[4], u32 b0, u32 b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}


// byte offset of the 16-byte piece `piece` of row `row` in a swizzled tile
__device__ __forceinline__ int kv_off(int row, int piece) { return row * 128 + ((piece ^ (row & 7)) << 4); }

__device__ __forceinline__ void tma_rows(u32 dst, const unsigned char* tmap, int x, int row, int plane, u32 bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 :: "r"(dst), "l"(tmap), "r"(x), "r"(row), "r"(plane), "r"(bar) : "memory");
}

