// One persistent cooperative kernel per decode step, written for sm_100a (B200, 148 SMs).
//
// This text is the body that vesta_gpu_b200/lower.py places behind a block of #defines (model
// sizes, placement constants, scratch offsets, parameter names) and a generated kernel signature.
// It compiles with NVRTC (no headers) and with nvcc.
//
// Execution model
//   * grid = one CTA per SM, block = NW consumer warps + 1 producer warp.
//   * Weights are read from a packed copy (built once by vesta_pack): for every CTA one contiguous
//     byte stream that holds, in the order the CTA consumes them, the 16x16 fp16 tiles of its share
//     of every contraction, each tile stored in the register order of mma.m16n8k16's A operand
//     (512 B, 16 B per lane). The producer warp walks that stream with cp.async.bulk into a ring
//     of shared-memory slots guarded by mbarriers; it runs ahead of the consumers through grid
//     barriers, so HBM keeps streaming while a phase waits for its inputs.
//   * Contractions run on mma.sync m16n8k16 with the weight tile as A (M = 16 outputs), the batch as
//     N (8 rows per tile) and the fp32 activation split into an fp16 head and an fp16 remainder
//     (two MMAs), accumulating in fp32: "fp16 weights, fp32 accumulation" at any batch <= 8*V_NB.
//   * NARROW placement: a CTA owns a few output tiles over the whole fold; its warps split the fold
//     and combine through shared memory; the epilogue sees complete sums (bias, GELU, KV emit).
//     WIDE placement: a CTA owns a range of the fold for many output tiles; each warp owns output
//     tiles; sums that span CTAs are combined with fp32 atomics into a zeroed vector.
//   * Per layer: [LN1 + QKV + KV emit] | [attention] | [attn-proj + residual] | [LN2 + FC + GELU +
//     MLP-proj + residual], grid barriers between them; then LN_f + logits + argmax + feedback,
//     finished by the last CTA to arrive (no barrier).
//   * Every wait (grid barrier, mbarrier) is bounded; on expiry the kernel records where in bar[]
//     and every later wait falls through, so the launch always ends.

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
typedef unsigned int u32;
typedef unsigned long long u64;
typedef unsigned short u16;

#define NW V_NW
#define NCONS (NW * 32)
#define NTHREADS (NCONS + 32)
#define KT_D (V_D / 16)
#define KT_F (V_F / 16)
#define JT_D (V_D / 16)
#define JT_J (3 * V_D / 16)
#define JT_N ((V_N + 15) / 16)
#define FRAG_BYTES 512
#define WN_MAX 4                      // widest NARROW placement (output tiles per CTA)
#define LNV ((V_D + 127) / 128)       // float4 per lane to hold one row of width D

// bar[] layout (u32): [0] status, [1] arrivals of the last phase, [2] abort flag, [32] barrier counter, cleared by the last CTA of every step
#define BAR_STATUS 0
#define BAR_DONE 1
#define BAR_ABORT 2
#define BAR_COUNT 32

// every wait gives up after WAIT_NS nanoseconds (a step takes well under a millisecond)
#define WAIT_NS 500000000ull
__device__ __forceinline__ u64 now_ns() { u64 t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }

__device__ __forceinline__ u32 smem_u32(const void* p) { return (u32)__cvta_generic_to_shared(p); }

__device__ __forceinline__ u32 pack_h2(float lo, float hi) {
    u32 r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float h_lo(u32 w) { float f; asm("{.reg .b16 l,h; mov.b32 {l,h}, %1; cvt.f32.f16 %0, l;}" : "=f"(f) : "r"(w)); return f; }
__device__ __forceinline__ float h_hi(u32 w) { float f; asm("{.reg .b16 l,h; mov.b32 {l,h}, %1; cvt.f32.f16 %0, h;}" : "=f"(f) : "r"(w)); return f; }
__device__ __forceinline__ float h2f(u16 h) { float f; asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h)); return f; }
__device__ __forceinline__ u16 f2h(float f) { u16 h; asm("cvt.rn.f16.f32 %0, %1;" : "=h"(h) : "f"(f)); return h; }

// fp32 pair -> fp16 head pair and fp16 remainder pair
__device__ __forceinline__ void split2(float a, float b, u32& hi, u32& lo) {
    hi = pack_h2(a, b);
    lo = pack_h2(a - h_lo(hi), b - h_hi(hi));
}

__device__ __forceinline__ void mma16816(float (&c)[4], const uint4& a, u32 b0, u32 b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" :: "n"(NCONS) : "memory"); }

__device__ __forceinline__ u32 ld_acquire(const u32* p) { u32 v; asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ u32 ld_relaxed(const u32* p) { u32 v; asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void st_release(u32* p, u32 v) { asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ void red_add(float* p, float v) { asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory"); }

__device__ __forceinline__ void mbar_init(u32 bar, u32 count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_arrive(u32 bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect(u32 bar, u32 bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ bool mbar_try(u32 bar, u32 parity) {
    u32 ok;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(u32 dst, const void* src, u32 bytes, u32 bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// orderable key of (value, index): larger value wins, then the lower index
__device__ __forceinline__ u64 best_key(float v, u32 n) {
    u32 u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((u64)u << 32) | (u64)(0xFFFFFFFFu - n);
}

// ---------------------------------------------------------------------------------------------
// per-CTA placement record (written by lower.py into the plan table PT, one per CTA)
// ---------------------------------------------------------------------------------------------
#define PT_STRIDE 16
#define PT_BASE 0        // first tile of this CTA's stream, in 512 B tiles
#define PT_LAYER 1       // tiles per layer
#define PT_QKV_J0 2      // NARROW: first output tile, tiles
#define PT_QKV_NJ 3
#define PT_PROJ_J0 4     // WIDE: output tiles [j0, j0+nj), fold tiles [k0, k0+nk)
#define PT_PROJ_NJ 5
#define PT_PROJ_K0 6
#define PT_PROJ_NK 7
#define PT_FC_J0 8       // NARROW; the same tiles are the fold range of the MLP projection
#define PT_FC_NJ 9
#define PT_LOG_J0 10     // WIDE over the whole fold
#define PT_LOG_NJ 11

struct Place {
    u32 base, layer;
    int qkv_j0, qkv_nj, proj_j0, proj_nj, proj_k0, proj_nk, fc_j0, fc_nj, log_j0, log_nj;
};

__device__ __forceinline__ Place load_place(const int* __restrict__ PT, int cta) {
    const int* p = PT + cta * PT_STRIDE;
    Place P;
    P.base = (u32)p[PT_BASE]; P.layer = (u32)p[PT_LAYER];
    P.qkv_j0 = p[PT_QKV_J0]; P.qkv_nj = p[PT_QKV_NJ];
    P.proj_j0 = p[PT_PROJ_J0]; P.proj_nj = p[PT_PROJ_NJ]; P.proj_k0 = p[PT_PROJ_K0]; P.proj_nk = p[PT_PROJ_NK];
    P.fc_j0 = p[PT_FC_J0]; P.fc_nj = p[PT_FC_NJ];
    P.log_j0 = p[PT_LOG_J0]; P.log_nj = p[PT_LOG_NJ];
    return P;
}

// A stream segment is a list of groups; a group is `rows` rows of `width` tiles, cut into chunks of
// whole rows, at most V_CH tiles per chunk. NARROW segment: one group (rows = fold tiles, width = nj).
// WIDE segment: one group per 8 output tiles (rows = fold tiles of the CTA, width <= 8).
__device__ __forceinline__ int rows_per_chunk(int width) { return V_CH / width; }
__device__ __forceinline__ u32 narrow_tiles(int nj, int kt) { return (u32)(nj * kt); }
__device__ __forceinline__ u32 wide_tiles(int nj, int nk) { return (u32)(nj * nk); }

// ---------------------------------------------------------------------------------------------
// shared memory
// ---------------------------------------------------------------------------------------------
#define SM_RING 0
#define SM_ACT (SM_RING + V_NSLOT * V_CH * FRAG_BYTES)
#define SM_GACT (SM_ACT + KT_D * V_NB * FRAG_BYTES)
#define SM_RED (SM_GACT + WN_MAX * V_NB * FRAG_BYTES)
#define SM_PRM (SM_RED + NW * WN_MAX * V_NB * 128 * 4)
#define PRM_TILE_HALVES (WN_MAX * 16)
#define SM_PRM_BYTES ((3 * V_D + PRM_TILE_HALVES) * 2)
#define SM_MISC ((SM_PRM + SM_PRM_BYTES + 15) & ~15)
#define SM_MISC_BYTES (NW * (V_E + 2) * 4 + V_B * 8 * NW + V_B * 4 + 64)
#define SM_BARS ((SM_MISC + SM_MISC_BYTES + 15) & ~15)
#define SM_TOTAL (SM_BARS + 2 * V_NSLOT * 8)

struct Ctx {
    unsigned char* smem;
    u32* bar;          // global counters
    u32 gen;           // barrier generation of this CTA
    u32 chunk;         // stream chunks consumed so far (same value in every consumer warp and the producer)
    int cta, ncta, tid, warp, lane;
    bool dead;         // a bounded wait expired somewhere: skip waits from now on
#if V_TIMING
    long long wait_clocks; u32 slow_waits;
#endif
};

__device__ __forceinline__ u32 full_bar(const Ctx& c, u32 slot) { return smem_u32(c.smem + SM_BARS) + slot * 8; }
__device__ __forceinline__ u32 empty_bar(const Ctx& c, u32 slot) { return smem_u32(c.smem + SM_BARS) + (V_NSLOT + slot) * 8; }

__device__ __noinline__ void give_up(Ctx& c, u32 where) {
    c.dead = true;
    atomicCAS(c.bar + BAR_STATUS, 0u, where | ((u32)c.cta << 16));
    atomicExch(c.bar + BAR_ABORT, 1u);
}

__device__ __forceinline__ void wait_mbar(Ctx& c, u32 bar, u32 parity, u32 where) {
    if (c.dead) return;
    if (mbar_try(bar, parity)) return;
#if V_TIMING
    c.slow_waits++;
    const long long k0_ = clock64();
    struct Acc_ { Ctx& c; long long k0; __device__ ~Acc_() { c.wait_clocks += clock64() - k0; } } acc_{c, k0_};
#endif
    const u64 t0 = now_ns();
    u32 spins = 0;
    while (!mbar_try(bar, parity)) {
        if ((++spins & 63u) == 0) {
            if (ld_relaxed(c.bar + BAR_ABORT)) { c.dead = true; return; }
            if (now_ns() - t0 > WAIT_NS) { give_up(c, where); return; }
        }
    }
}

// Grid barrier for the consumer warps of all CTAs, in two halves so that loads that do not depend
// on other CTAs (the next phase's parameters) can be issued in between. One monotonic counter:
// every CTA adds 1 (release), thread 0 of every CTA polls it until it reaches generation x CTAs.
// Measured on B200 with 148 CTAs arriving together: 2400 cycles (1.3 us) per barrier, of which the
// release fence is ~530 and the add ~270. Every variant tried was slower: one flag word per CTA
// polled by all (6100 cycles: 148 x 148 polling loads delay the flag stores), 4 or 16 counters on
// separate lines (4600), two levels of 16 (4000), an arrival counter plus a "go" word (3600).
__device__ __forceinline__ void phase_end(Ctx& c) {
    cons_sync();
    c.gen += (u32)c.ncta;
    if (c.tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(c.bar + BAR_COUNT) : "memory");
}
__device__ __forceinline__ void phase_wait(Ctx& c) {
    if (c.tid == 0 && !c.dead) {
        if ((int)(ld_acquire(c.bar + BAR_COUNT) - c.gen) < 0) {
            const u64 t0 = now_ns();
            u32 spins = 0;
            while ((int)(ld_acquire(c.bar + BAR_COUNT) - c.gen) < 0) {
                if ((++spins & 63u) == 0) {
                    if (ld_relaxed(c.bar + BAR_ABORT)) break;
                    if (now_ns() - t0 > WAIT_NS) { give_up(c, 0x100u); break; }
                }
            }
        }
    }
    cons_sync();
    if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
}

// 16-byte asynchronous copies global -> shared for the small per-phase parameters
__device__ __forceinline__ void cp16(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" :: "r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Parameters of the next phase into shared memory: LayerNorm gain and shift, the bias added when a
// combined vector is initialised (all three V_D halves), and the bias of this CTA's NARROW tiles.
__device__ __noinline__ void fetch_params(Ctx& c, const u16* gw, const u16* gb, const u16* ib, const u16* tb, int tiles) {
    u16* prm = reinterpret_cast<u16*>(c.smem + SM_PRM);
    const int per = V_D / 8;                       // 16-byte pieces per vector
    for (int i = c.tid; i < 3 * per; i += NCONS) {
        const int v = i / per, q = i % per;
        const u16* src = v == 0 ? gw : (v == 1 ? gb : ib);
        if (src) cp16(prm + v * V_D + q * 8, src + q * 8);
    }
    if (tb && c.tid < tiles * 2) cp16(prm + 3 * V_D + c.tid * 8, tb + c.tid * 8);
}

// ---------------------------------------------------------------------------------------------
// producer: walks this CTA's stream
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void produce_group(Ctx& c, const unsigned char* src, int rows, int width) {
    const int rpc = rows_per_chunk(width);
    for (int r = 0; r < rows; r += rpc) {
        const int nr = min(rpc, rows - r);
        const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
        wait_mbar(c, empty_bar(c, slot), (use & 1u) ^ 1u, 0x200u);
        if (c.dead) return;
        const u32 bytes = (u32)(nr * width) * FRAG_BYTES;
        mbar_expect(full_bar(c, slot), bytes);
        bulk_g2s(smem_u32(c.smem + SM_RING) + slot * (V_CH * FRAG_BYTES), src + (size_t)r * width * FRAG_BYTES, bytes, full_bar(c, slot));
        c.chunk++;
    }
}

__device__ __forceinline__ void produce_wide(Ctx& c, const unsigned char* src, int nj, int nk) {
    for (int j = 0; j < nj; j += 8) {
        const int w = min(8, nj - j);
        produce_group(c, src, nk, w);
        src += (size_t)nk * w * FRAG_BYTES;
    }
}

__device__ __noinline__ void producer(Ctx& c, const Place& P, const unsigned char* __restrict__ WP) {
    const unsigned char* base = WP + (size_t)P.base * FRAG_BYTES;
    for (int l = 0; l < V_L; l++) {
        const unsigned char* s = base + (size_t)l * P.layer * FRAG_BYTES;
        if (P.qkv_nj) produce_group(c, s, KT_D, P.qkv_nj);
        s += (size_t)narrow_tiles(P.qkv_nj, KT_D) * FRAG_BYTES;
        produce_wide(c, s, P.proj_nj, P.proj_nk);
        s += (size_t)wide_tiles(P.proj_nj, P.proj_nk) * FRAG_BYTES;
        if (P.fc_nj) produce_group(c, s, KT_D, P.fc_nj);
        s += (size_t)narrow_tiles(P.fc_nj, KT_D) * FRAG_BYTES;
        produce_wide(c, s, JT_D, P.fc_nj);
        if (c.dead) return;
    }
    produce_wide(c, base + (size_t)V_L * P.layer * FRAG_BYTES, P.log_nj, KT_D);
}

// ---------------------------------------------------------------------------------------------
// consumer side of the stream
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ const unsigned char* chunk_acquire(Ctx& c) {
    const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
    wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
    return c.smem + SM_RING + slot * (V_CH * FRAG_BYTES);
}
__device__ __forceinline__ void chunk_release(Ctx& c) {
    __syncwarp();
    if (c.lane == 0) mbar_arrive(empty_bar(c, c.chunk % V_NSLOT));
    c.chunk++;
}

__device__ __forceinline__ uint4 lds128(const unsigned char* p) { return *reinterpret_cast<const uint4*>(p); }

// NARROW group: rows = fold tiles [0, kt), width = nj (<= WN_MAX). Warp w takes rows r = w (mod NW).
// act: B operands, tile r at act + (r * V_NB + nb) * 512. Result: acc[jj][nb][4] partial per warp.
__device__ __forceinline__ void narrow_gemm(Ctx& c, int kt, int nj, const unsigned char* act, float (&acc)[WN_MAX][V_NB][4]) {
#pragma unroll
    for (int jj = 0; jj < WN_MAX; jj++)
#pragma unroll
        for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[jj][nb][i] = 0.f;
    if (nj == 0) return;
    const int rpc = rows_per_chunk(nj);
    for (int r0 = 0; r0 < kt; r0 += rpc) {
        const int nr = min(rpc, kt - r0);
        const unsigned char* slot = chunk_acquire(c);
        if (!c.dead) {
            // first row of this chunk owned by this warp
            int first = ((c.warp - (r0 % NW)) + NW) % NW;
            for (int rr = first; rr < nr; rr += NW) {
                const int r = r0 + rr;
                uint4 b[V_NB];
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++) b[nb] = lds128(act + ((size_t)(r * V_NB + nb) * 32 + c.lane) * 16);
#pragma unroll
                for (int jj = 0; jj < WN_MAX; jj++) {
                    if (jj < nj) {
                        const uint4 a = lds128(slot + ((size_t)(rr * nj + jj) * 32 + c.lane) * 16);
#pragma unroll
                        for (int nb = 0; nb < V_NB; nb++) {
                            mma16816(acc[jj][nb], a, b[nb].x, b[nb].y);
#if V_ACT_LO
                            mma16816(acc[jj][nb], a, b[nb].z, b[nb].w);
#endif
                        }
                    }
                }
            }
        }
        chunk_release(c);
    }
}

// Sum the NARROW partials of all warps. Afterwards red[(jj * V_NB + nb) * 128 + lane * 4 + i] of
// warp 0's block holds the complete sums for jj < nj.
__device__ __forceinline__ void narrow_reduce(Ctx& c, int nj, float (&acc)[WN_MAX][V_NB][4]) {
    float* red = reinterpret_cast<float*>(c.smem + SM_RED);
#pragma unroll
    for (int jj = 0; jj < WN_MAX; jj++)
        if (jj < nj)
#pragma unroll
            for (int nb = 0; nb < V_NB; nb++)
                *reinterpret_cast<float4*>(red + ((size_t)(c.warp * WN_MAX + jj) * V_NB + nb) * 128 + c.lane * 4) =
                    make_float4(acc[jj][nb][0], acc[jj][nb][1], acc[jj][nb][2], acc[jj][nb][3]);
    cons_sync();
    const int total = nj * V_NB * 128;
    for (int o = c.tid; o < total; o += NCONS) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) s += red[(size_t)w * WN_MAX * V_NB * 128 + o];
        red[o] = s;      // slot (warp 0, o): only this thread reads the other warps' value at o
    }
    cons_sync();
}

// Output coordinates of element o of a reduced NARROW block: jj, nb, then the C fragment layout.
__device__ __forceinline__ void narrow_coord(int o, int& jj, int& j_in, int& b) {
    const int i = o & 3, ln = (o >> 2) & 31, nb = (o >> 7) % V_NB;
    jj = (o >> 7) / V_NB;
    j_in = (ln >> 2) + ((i & 2) ? 8 : 0);
    b = nb * 8 + (ln & 3) * 2 + (i & 1);
}

// WIDE group: rows = fold tiles (nk), width = w (<= 8); warp w' < width owns output tile w'.
// act tile for row r: act + ((r_act0 + r) * V_NB + nb) * 512.
__device__ __forceinline__ void wide_gemm(Ctx& c, int nk, int width, const unsigned char* act, int r_act0, float (&acc)[V_NB][4]) {
    float lo[V_NB][4];
#pragma unroll
    for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) { acc[nb][i] = 0.f; lo[nb][i] = 0.f; }
    const int rpc = rows_per_chunk(width);
    for (int r0 = 0; r0 < nk; r0 += rpc) {
        const int nr = min(rpc, nk - r0);
        const unsigned char* slot = chunk_acquire(c);
        if (!c.dead && c.warp < width) {
            for (int rr = 0; rr < nr; rr++) {
                const uint4 a = lds128(slot + ((size_t)(rr * width + c.warp) * 32 + c.lane) * 16);
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++) {
                    const uint4 b = lds128(act + ((size_t)((r_act0 + r0 + rr) * V_NB + nb) * 32 + c.lane) * 16);
                    mma16816(acc[nb], a, b.x, b.y);
#if V_ACT_LO
                    mma16816(lo[nb], a, b.z, b.w);
#endif
                }
            }
        }
        chunk_release(c);
    }
#pragma unroll
    for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[nb][i] += lo[nb][i];
}

// ---------------------------------------------------------------------------------------------
// activations -> B operand tiles in shared memory
// element (b, k): tile k/16, batch tile b/8, lane (b%8)*4 + (k%8)/2, word (k%16)/8 (+2 for the
// remainder), half k%2
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void act_store4(unsigned char* act, int b, int k, float4 v) {
    // k is a multiple of 4: two words of the same register index
    u32 h0, l0, h1, l1;
    split2(v.x, v.y, h0, l0);
    split2(v.z, v.w, h1, l1);
    const int kt = k >> 4, kk = k & 15, reg = kk >> 3, t = (kk & 7) >> 1;
    u32* base = reinterpret_cast<u32*>(act + ((size_t)(kt * V_NB + (b >> 3)) * 32 + (b & 7) * 4) * 16);
    base[t * 4 + reg] = h0;
    base[t * 4 + 2 + reg] = l0;
    base[(t + 1) * 4 + reg] = h1;
    base[(t + 1) * 4 + 2 + reg] = l1;
}

__device__ __forceinline__ void act_store1(unsigned char* act, int b, int k, float v) {
    const u16 hi = f2h(v), lo = f2h(v - h2f(hi));
    const int kt = k >> 4, kk = k & 15, reg = kk >> 3, t = (kk & 7) >> 1, half = kk & 1;
    u16* base = reinterpret_cast<u16*>(act + ((size_t)(kt * V_NB + (b >> 3)) * 32 + (b & 7) * 4 + t) * 16);
    base[reg * 2 + half] = hi;
    base[(2 + reg) * 2 + half] = lo;
}

// LayerNorm of the rows of z (global, fp32, [V_B][V_D]) into the operand tiles, one warp per row;
// gain and shift come from the parameter block in shared memory. The same pass starts the vector
// the following projection is combined into: init[b][d] += z[b][d] + bias[d], every CTA adding
// its share of the elements (init was zeroed a phase earlier).
__device__ __noinline__ void ln_to_act(Ctx& c, const float* __restrict__ z, float* __restrict__ init, unsigned char* act) {
    const u16* prm = reinterpret_cast<const u16*>(c.smem + SM_PRM);
    for (int b = c.warp; b < V_B; b += NW) {
        float4 v[LNV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int d = (i * 32 + c.lane) * 4;
            v[i] = (d < V_D) ? __ldcg(reinterpret_cast<const float4*>(z + (size_t)b * V_D + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        const float mean = s * (1.0f / V_D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int d = (i * 32 + c.lane) * 4;
            if (d < V_D) {
                const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
                q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
            }
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
        const float rs = 1.0f / sqrtf(q * (1.0f / V_D) + V_EPS);
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int d = (i * 32 + c.lane) * 4;
            if (d < V_D) {
                const uint2 w = *reinterpret_cast<const uint2*>(prm + d);
                const uint2 bb = *reinterpret_cast<const uint2*>(prm + V_D + d);
                float4 o;
                o.x = (v[i].x - mean) * rs * h_lo(w.x) + h_lo(bb.x);
                o.y = (v[i].y - mean) * rs * h_hi(w.x) + h_hi(bb.x);
                o.z = (v[i].z - mean) * rs * h_lo(w.y) + h_lo(bb.y);
                o.w = (v[i].w - mean) * rs * h_hi(w.y) + h_hi(bb.y);
                act_store4(act, b, d, o);
                if (init && ((i * 32 + c.lane) % c.ncta) == c.cta) {
                    const uint2 ib = *reinterpret_cast<const uint2*>(prm + 2 * V_D + d);
                    float* dst = init + (size_t)b * V_D + d;
                    red_add(dst, v[i].x + h_lo(ib.x)); red_add(dst + 1, v[i].y + h_hi(ib.x));
                    red_add(dst + 2, v[i].z + h_lo(ib.y)); red_add(dst + 3, v[i].w + h_hi(ib.y));
                }
            }
        }
    }
    cons_sync();
}

// Attention output for the fold range [k0*16, (k0+nk)*16) of the projection, merged from the
// per-chunk partial results (m, sum, unnormalised o[V_E]) of the attention phase, into operand
// tiles 0..nk-1.
#define PART_STRIDE (V_E + 2)
__device__ __noinline__ void merge_to_act(Ctx& c, const float* __restrict__ part, int k0, int nk, unsigned char* act) {
    const int cols = nk * 16;
    for (int i = c.tid; i < V_B * cols; i += NCONS) {
        const int b = i / cols, kk = i % cols, d = k0 * 16 + kk, h = d / V_E, e = d % V_E;
        const float* p = part + (size_t)((b * V_H + h) * V_NCH) * PART_STRIDE;
        float m[V_NCH], M = -3.0e38f;
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) { m[ch] = __ldcg(p + ch * PART_STRIDE); M = fmaxf(M, m[ch]); }
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) {
            const float w = expf(m[ch] - M);
            den += w * __ldcg(p + ch * PART_STRIDE + 1);
            num += w * __ldcg(p + ch * PART_STRIDE + 2 + e);
        }
        act_store1(act, b, kk, num / den);
    }
    cons_sync();
}

// ---------------------------------------------------------------------------------------------
// attention of one (sequence, head): online softmax over positions 0..n-1, K and V from the cache
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void dot8(const uint4& kv, const float (&q)[8], float& s) {
    s = q[0] * h_lo(kv.x) + q[1] * h_hi(kv.x) + q[2] * h_lo(kv.y) + q[3] * h_hi(kv.y) +
        q[4] * h_lo(kv.z) + q[5] * h_hi(kv.z) + q[6] * h_lo(kv.w) + q[7] * h_hi(kv.w);
}

#define ATT_UNROLL 4
// positions [s_lo, s_hi) of one (sequence, head); result: (running max, sum, unnormalised o[V_E]) at out
__device__ __noinline__ void attention_item(Ctx& c, const u16* __restrict__ keys, const u16* __restrict__ vals, const float* __restrict__ qbuf,
                               float* __restrict__ out, int b, int h, int l, int s_lo, int n) {
    // 8 lanes per position (16 B each of the 128 B row), 4 positions per warp per round
    const int li = c.lane & 7, grp = c.warp * 4 + (c.lane >> 3);
    const int NG = NW * 4;
    float q[8];
    {
        const float* qp = qbuf + (size_t)b * V_D + h * V_E + li * 8;
        const float4 q0 = __ldcg(reinterpret_cast<const float4*>(qp)), q1 = __ldcg(reinterpret_cast<const float4*>(qp + 4));
        q[0] = q0.x; q[1] = q0.y; q[2] = q0.z; q[3] = q0.w; q[4] = q1.x; q[5] = q1.y; q[6] = q1.z; q[7] = q1.w;
    }
    const size_t row0 = ((size_t)(b * V_L + l) * V_TMAX) * V_D + (size_t)h * V_E + li * 8;
    float m = -3.0e38f, den = 0.f, acc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] = 0.f;
    // the trip count is the same for every lane of the warp (the shuffles below need all 32 lanes)
    for (int base = s_lo; base < n; base += NG * ATT_UNROLL) {
        const int s0 = base + grp;
        uint4 kk[ATT_UNROLL], vv[ATT_UNROLL];
#pragma unroll
        for (int u = 0; u < ATT_UNROLL; u++) {
            const int s = s0 + u * NG;
            if (s < n) {
                kk[u] = __ldcg(reinterpret_cast<const uint4*>(keys + row0 + (size_t)s * V_D));
                vv[u] = __ldcg(reinterpret_cast<const uint4*>(vals + row0 + (size_t)s * V_D));
            } else {
                kk[u] = make_uint4(0, 0, 0, 0); vv[u] = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int u = 0; u < ATT_UNROLL; u++) {
            const int s = s0 + u * NG;
            float sc;
            dot8(kk[u], q, sc);
            sc += __shfl_xor_sync(0xffffffffu, sc, 1);
            sc += __shfl_xor_sync(0xffffffffu, sc, 2);
            sc += __shfl_xor_sync(0xffffffffu, sc, 4);
            if (s < n) {
                sc = sc / V_SCALE;
                const float mn = fmaxf(m, sc);
                const float corr = expf(m - mn), p = expf(sc - mn);
                den = den * corr + p;
                acc[0] = acc[0] * corr + p * h_lo(vv[u].x); acc[1] = acc[1] * corr + p * h_hi(vv[u].x);
                acc[2] = acc[2] * corr + p * h_lo(vv[u].y); acc[3] = acc[3] * corr + p * h_hi(vv[u].y);
                acc[4] = acc[4] * corr + p * h_lo(vv[u].z); acc[5] = acc[5] * corr + p * h_hi(vv[u].z);
                acc[6] = acc[6] * corr + p * h_lo(vv[u].w); acc[7] = acc[7] * corr + p * h_hi(vv[u].w);
                m = mn;
            }
        }
    }
    // merge the 4 position groups of the warp (lanes li, li+8, li+16, li+24 hold the same dims)
#pragma unroll
    for (int x = 8; x <= 16; x <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, x), d2 = __shfl_xor_sync(0xffffffffu, den, x);
        const float mn = fmaxf(m, m2);
        const float c1 = expf(m - mn), c2 = expf(m2 - mn);
        den = den * c1 + d2 * c2;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float a2 = __shfl_xor_sync(0xffffffffu, acc[i], x);
            acc[i] = acc[i] * c1 + a2 * c2;
        }
        m = mn;
    }
    // merge the warps through shared memory: per warp (m, den, acc[V_E])
    float* ms = reinterpret_cast<float*>(c.smem + SM_MISC);
    if (c.lane < 8) {
        float* w = ms + c.warp * (V_E + 2);
        if (c.lane == 0) { w[0] = m; w[1] = den; }
#pragma unroll
        for (int i = 0; i < 8; i++) w[2 + li * 8 + i] = acc[i];
    }
    cons_sync();
    if (c.tid < V_E) {
        float M = -3.0e38f;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, ms[w * (V_E + 2)]);
        float num = 0.f, dd = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            const float sc = expf(ms[w * (V_E + 2)] - M);
            dd += ms[w * (V_E + 2) + 1] * sc;
            num += ms[w * (V_E + 2) + 2 + c.tid] * sc;
        }
        out[2 + c.tid] = num;
        if (c.tid == 0) { out[0] = M; out[1] = dd; }
    }
    cons_sync();
}

// ---------------------------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------------------------
struct Args {
    const int* x; const int* t;
    const u16 *wte, *wpe, *ln1w, *ln1b, *qkvb, *ob, *ln2w, *ln2b, *fcb, *pb, *lnfw, *lnfb;
    u16 *keys, *vals;
    int* x_out; int* t_out;
    float* S; u32* bar; u64* TS;
    const unsigned char* WP; const int* PT;
};

__device__ __forceinline__ int pos_of(const Args& a, int b) { return a.t[b * V_TSTRIDE]; }

#if V_TIMING
// thread 0 of CTA V_TIMING-1 sums clock64 deltas per site in shared memory (cheap) and adds them to TS at the end
#define TICK(k) do { if (c.cta == V_TIMING - 1 && c.tid == 0) { const long long now_ = clock64(); ts_[k] += now_ - tlast_; tlast_ = now_; } } while (0)
#else
#define TICK(k) do { } while (0)
#endif

__device__ void step_body(const Args& a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Ctx c;
    c.smem = smem; c.bar = a.bar; c.chunk = 0; c.dead = false;
#if V_TIMING
    c.wait_clocks = 0; c.slow_waits = 0;
#endif
    c.cta = blockIdx.x; c.ncta = gridDim.x; c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
#if V_TIMING
    __shared__ long long ts_[16];
    if (threadIdx.x == 0) for (int i = 0; i < 16; i++) ts_[i] = 0;
    long long tlast_ = clock64();
    const u64 t_begin_ = now_ns();
#endif

    // inputs outside their ranges would index outside the caches and tables: refuse the step
    // (every CTA sees the same values and takes the same branch)
    int* s_pos = reinterpret_cast<int*>(smem + SM_MISC + NW * (V_E + 2) * 4 + V_B * 8 * NW + 16);
    {
        bool bad = false;
        for (int b = 0; b < V_B; b++) {
            const int tb = pos_of(a, b), xb = a.x[b];
            bad |= (tb < 0) | (tb >= V_TMAX) | (tb >= V_CPOS) | (xb < 0) | (xb >= V_N);
            if (c.tid == 0) s_pos[b] = tb;
        }
        if (bad) {
            if (c.cta == 0 && c.tid == 0) atomicCAS(a.bar + BAR_STATUS, 0u, 0x900u);
            return;
        }
    }

    if (c.tid == 0) {
        for (int s = 0; s < V_NSLOT; s++) { mbar_init(full_bar(c, s), 1); mbar_init(empty_bar(c, s), NW); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // operand tiles start as zero: rows of a batch tile beyond V_B stay zero for the whole launch
    for (int i = c.tid; i < (SM_RED - SM_ACT) / 16; i += NTHREADS)
        reinterpret_cast<uint4*>(smem + SM_ACT)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    const Place P = load_place(a.PT, c.cta);
    if (c.warp == NW) {
        if (c.lane == 0) {
            producer(c, P, a.WP);
#if V_TIMING
            if (c.cta == V_TIMING - 1) { a.TS[18] += (u64)c.wait_clocks; a.TS[19] += c.slow_waits; a.TS[20] += c.chunk; }
#endif
        }
        return;
    }

    c.gen = 0;      // the barrier counter is zero at launch: the last CTA of every step clears it
    unsigned char* act = smem + SM_ACT;
    unsigned char* gact = smem + SM_GACT;
    float* red = reinterpret_cast<float*>(smem + SM_RED);
    const u16* prm = reinterpret_cast<const u16*>(smem + SM_PRM);
    float* Z = a.S + V_OFF_Z;
    float* qbuf = a.S + V_OFF_Q;
    float* part = a.S + V_OFF_PART;
    const int gtid = c.cta * NCONS + c.tid, gthreads = c.ncta * NCONS;
    const size_t ZS = (size_t)V_B * V_D;

    // Q1: z0 = wte[x] + wpe[t]; the vector the first projection is combined into starts at zero
    for (int i = gtid; i < V_B * V_D; i += gthreads) {
        const int b = i / V_D, d = i % V_D;
        Z[i] = h2f(a.wte[(size_t)a.x[b] * V_D + d]) + h2f(a.wpe[(size_t)s_pos[b] * V_D + d]);
        Z[ZS + i] = 0.f;
    }
    TICK(0);
    phase_end(c);
    fetch_params(c, a.ln1w, a.ln1b, a.ob, a.qkvb + P.qkv_j0 * 16, P.qkv_nj);
    phase_wait(c);
    TICK(1);

    for (int l = 0; l < V_L; l++) {
        float* zin = Z + (size_t)((2 * l) % 3) * ZS;
        float* z1 = Z + (size_t)((2 * l + 1) % 3) * ZS;
        float* z2 = Z + (size_t)((2 * l + 2) % 3) * ZS;

        // ---- LN1 + QKV (+bias): q to scratch, K and V rounded to fp16 into the cache at t.
        //      The same pass starts z1 = z + ob (the projection adds into it two phases later)
        //      and clears z2, which nobody reads any more.
        for (int i = gtid; i < V_B * V_D; i += gthreads) z2[i] = 0.f;
        cp_wait();
        cons_sync();
        ln_to_act(c, zin, z1, act);
        {
            float acc[WN_MAX][V_NB][4];
            narrow_gemm(c, KT_D, P.qkv_nj, act, acc);
            narrow_reduce(c, P.qkv_nj, acc);
            const int total = P.qkv_nj * V_NB * 128;
            for (int o = c.tid; o < total; o += NCONS) {
                int jj, j_in, b;
                narrow_coord(o, jj, j_in, b);
                if (b < V_B) {
                    const int j = (P.qkv_j0 + jj) * 16 + j_in;
                    const float v = red[o] + h2f(prm[3 * V_D + jj * 16 + j_in]);
                    if (j < V_D) qbuf[(size_t)b * V_D + j] = v;
                    else {
                        const size_t at = ((size_t)(b * V_L + l) * V_TMAX + s_pos[b]) * V_D + (j % V_D);
                        if (j < 2 * V_D) a.keys[at] = f2h(v); else a.vals[at] = f2h(v);
                    }
                }
            }
        }
        TICK(2);
        phase_end(c);
        phase_wait(c);
        TICK(3);

        // ---- attention: one (sequence, head, chunk of positions) at a time, partial results to scratch
        for (int it = c.cta; it < V_B * V_H * V_NCH; it += c.ncta) {
            const int ch = it % V_NCH, bh = it / V_NCH, b = bh / V_H, h = bh % V_H;
            const int n = s_pos[b] + 1, cs = (n + V_NCH - 1) / V_NCH;
            attention_item(c, a.keys, a.vals, qbuf, part + (size_t)it * PART_STRIDE, b, h, l, ch * cs, min(n, (ch + 1) * cs));
        }
        TICK(4);
        phase_end(c);
        phase_wait(c);
        TICK(5);

        // ---- attn-proj: z1 += o . ow, partial sums over this CTA's fold range
        if (P.proj_nj) {
            merge_to_act(c, part, P.proj_k0, P.proj_nk, act);
            float acc[V_NB][4];
            wide_gemm(c, P.proj_nk, P.proj_nj, act, 0, acc);
            if (c.warp < P.proj_nj) {
                const int jt = P.proj_j0 + c.warp;
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int j = jt * 16 + (c.lane >> 2) + ((i & 2) ? 8 : 0), b = nb * 8 + (c.lane & 3) * 2 + (i & 1);
                        if (b < V_B) red_add(z1 + (size_t)b * V_D + j, acc[nb][i]);
                    }
            }
        }
        TICK(6);
        phase_end(c);
        fetch_params(c, a.ln2w + (size_t)l * V_D, a.ln2b + (size_t)l * V_D, a.pb + (size_t)l * V_D,
                     a.fcb + (size_t)l * V_F + P.fc_j0 * 16, P.fc_nj);
        phase_wait(c);
        TICK(7);

        // ---- LN2 + FC + GELU on this CTA's slice of f, then its partial of the MLP projection.
        //      The LN pass starts z2 = z1 + pb; zin is free from here on and is cleared for the
        //      next layer's projection.
        for (int i = gtid; i < V_B * V_D; i += gthreads) zin[i] = 0.f;
        cp_wait();
        cons_sync();
        ln_to_act(c, z1, z2, act);
        TICK(12);
        {
            float acc[WN_MAX][V_NB][4];
            narrow_gemm(c, KT_D, P.fc_nj, act, acc);
            TICK(13);
            narrow_reduce(c, P.fc_nj, acc);
            // g = gelu(u + fcb) -> operand tiles of the projection: fold index = jj*16 + j_in
            const int total = P.fc_nj * V_NB * 128;
            for (int o = c.tid; o < total; o += NCONS) {
                int jj, j_in, b;
                narrow_coord(o, jj, j_in, b);
                float g = 0.f;
                if (b < V_B) {
                    const float u = red[o] + h2f(prm[3 * V_D + jj * 16 + j_in]);
                    g = V_GELU_A * u * (1.0f + tanhf(V_GELU_B * (u + V_GELU_C * u * u * u)));
                }
                act_store1(gact, b, jj * 16 + j_in, g);
            }
            cons_sync();
            TICK(14);
        }
        for (int jg = 0; jg < JT_D; jg += 8) {
            const int width = min(8, JT_D - jg);
            float acc[V_NB][4];
            wide_gemm(c, P.fc_nj, width, gact, 0, acc);
            if (c.warp < width && P.fc_nj) {
                const int jt = jg + c.warp;
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int j = jt * 16 + (c.lane >> 2) + ((i & 2) ? 8 : 0), b = nb * 8 + (c.lane & 3) * 2 + (i & 1);
                        if (b < V_B) red_add(z2 + (size_t)b * V_D + j, acc[nb][i]);
                    }
            }
        }
        TICK(8);
        phase_end(c);
        if (l + 1 < V_L)
            fetch_params(c, a.ln1w + (size_t)(l + 1) * V_D, a.ln1b + (size_t)(l + 1) * V_D, a.ob + (size_t)(l + 1) * V_D,
                         a.qkvb + (size_t)(l + 1) * 3 * V_D + P.qkv_j0 * 16, P.qkv_nj);
        else
            fetch_params(c, a.lnfw, a.lnfb, (const u16*)0, (const u16*)0, 0);
        phase_wait(c);
        TICK(9);
    }

    // ---- LN_f + logits + argmax
    float* zf = Z + (size_t)((2 * V_L) % 3) * ZS;
    cp_wait();
    cons_sync();
    ln_to_act(c, zf, (float*)0, act);
    u64 best[V_NB][2];
#pragma unroll
    for (int nb = 0; nb < V_NB; nb++) { best[nb][0] = 0; best[nb][1] = 0; }
    float* logit = a.S + V_OFF_LOGIT;
    for (int jg = 0; jg < P.log_nj; jg += 8) {
        const int width = min(8, P.log_nj - jg);
        float acc[V_NB][4];
        wide_gemm(c, KT_D, width, act, 0, acc);
        if (c.warp < width) {
            const int jt = P.log_j0 + jg + c.warp;
#pragma unroll
            for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const int n = jt * 16 + (c.lane >> 2) + ((i & 2) ? 8 : 0), b = nb * 8 + (c.lane & 3) * 2 + (i & 1);
                    if (b < V_B && n < V_N) {
                        logit[(size_t)b * V_N + n] = acc[nb][i];
                        const u64 k = best_key(acc[nb][i], (u32)n);
                        if (k > best[nb][i & 1]) best[nb][i & 1] = k;
                    }
                }
        }
    }
    // per batch row: max over the lanes that hold the same row (lanes with equal lane&3), then over warps
    u64* wbest = reinterpret_cast<u64*>(smem + ((SM_MISC + NW * (V_E + 2) * 4 + 7) & ~7));
#pragma unroll
    for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
        for (int p = 0; p < 2; p++) {
            u64 k = best[nb][p];
#pragma unroll
            for (int m = 4; m <= 16; m <<= 1) {
                const u64 o = __shfl_xor_sync(0xffffffffu, k, m);
                if (o > k) k = o;
            }
            const int b = nb * 8 + (c.lane & 3) * 2 + p;
            if ((c.lane >> 2) == 0 && b < V_B) wbest[b * NW + c.warp] = k;
        }
    cons_sync();
    u64* gbest = reinterpret_cast<u64*>(a.S + V_OFF_BEST);
    if (c.tid < V_B) {
        u64 k = 0;
        for (int w = 0; w < NW; w++) if (wbest[c.tid * NW + w] > k) k = wbest[c.tid * NW + w];
        if (k) atomicMax(gbest + c.tid, k);
    }
    TICK(10);
    // the last CTA to arrive publishes next, feeds it back into x and advances t
    cons_sync();
    if (c.tid == 0) {
        __threadfence();
        const u32 old = atomicAdd(a.bar + BAR_DONE, 1u);
        if (old == (u32)c.ncta - 1) {
            __threadfence();
            for (int b = 0; b < V_B; b++) {
                const u64 k = atomicExch(gbest + b, 0ull);
                const u32 n = 0xFFFFFFFFu - (u32)(k & 0xFFFFFFFFull);
                a.S[V_OFF_NEXT + b] = (float)n;
#if V_FEEDBACK
                a.x_out[b] = (int)n;
#endif
            }
#if V_FEEDBACK
            for (int b = 0; b < (V_TSTRIDE ? V_B : 1); b++) a.t_out[b] += V_TSTEP;
#endif
            atomicExch(a.bar + BAR_COUNT, 0u);     // every CTA is past its last barrier
            atomicExch(a.bar + BAR_DONE, 0u);
        }
    }
    TICK(11);
#if V_TIMING
    if (c.cta == V_TIMING - 1 && c.tid == 0) {
        for (int i = 0; i < 16; i++) a.TS[i] += (u64)ts_[i];
        a.TS[16] += (u64)c.wait_clocks; a.TS[17] += c.slow_waits;
        a.TS[21] += now_ns() - t_begin_;        // nanoseconds of this CTA's launch, to convert clocks
        a.TS[22] += (u64)(clock64() - (tlast_ - 0)) * 0 + 1;   // launches
    }
#endif
}

// ---------------------------------------------------------------------------------------------
// one-time packing of the weights into the per-CTA streams
// ---------------------------------------------------------------------------------------------
struct PackArgs {
    const u16 *wte, *qkvw, *ow, *fcw, *pw;
    unsigned char* WP; const int* PT;
};

// A(m = output j, k) of the five contractions
__device__ __forceinline__ u16 w_elem(const PackArgs& a, int kind, int l, int j, int k) {
    switch (kind) {
        case 0: return a.qkvw[((size_t)l * V_D + k) * (3 * V_D) + j];
        case 1: return a.ow[((size_t)l * V_D + k) * V_D + j];
        case 2: return a.fcw[((size_t)l * V_D + k) * V_F + j];
        case 3: return a.pw[((size_t)l * V_F + k) * V_D + j];
        default: return j < V_N ? a.wte[(size_t)j * V_D + k] : (u16)0;
    }
}

__device__ __forceinline__ void pack_tile(const PackArgs& a, unsigned char* dst, int kind, int l, int jt, int kt, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const int j0 = jt * 16 + g, j1 = j0 + 8, k0 = kt * 16 + 2 * t;
    uint4 v;
    v.x = (u32)w_elem(a, kind, l, j0, k0) | ((u32)w_elem(a, kind, l, j0, k0 + 1) << 16);
    v.y = (u32)w_elem(a, kind, l, j1, k0) | ((u32)w_elem(a, kind, l, j1, k0 + 1) << 16);
    v.z = (u32)w_elem(a, kind, l, j0, k0 + 8) | ((u32)w_elem(a, kind, l, j0, k0 + 9) << 16);
    v.w = (u32)w_elem(a, kind, l, j1, k0 + 8) | ((u32)w_elem(a, kind, l, j1, k0 + 9) << 16);
    reinterpret_cast<uint4*>(dst)[lane] = v;
}

// NARROW group: tile index = kt * nj + jj
__device__ void pack_narrow(const PackArgs& a, unsigned char* dst, int kind, int l, int j0, int nj, int kt_n, int wid, int nwarp, int lane) {
    const int n = nj * kt_n;
    for (int i = wid; i < n; i += nwarp) pack_tile(a, dst + (size_t)i * FRAG_BYTES, kind, l, j0 + i % nj, i / nj, lane);
}
// WIDE segment: groups of 8 output tiles; inside a group tile index = k_rel * width + w
__device__ void pack_wide(const PackArgs& a, unsigned char* dst, int kind, int l, int j0, int nj, int k0, int nk, int wid, int nwarp, int lane) {
    const int n = nj * nk;
    for (int i = wid; i < n; i += nwarp) {
        const int grp = i / (8 * nk);                      // full groups before this tile hold 8*nk tiles
        const int width = min(8, nj - grp * 8);
        const int r = i - grp * 8 * nk;
        pack_tile(a, dst + (size_t)i * FRAG_BYTES, kind, l, j0 + grp * 8 + r % width, k0 + r / width, lane);
    }
}

// grid: (V_L + 1) blocks per CTA of the step kernel: blockIdx.x = cta * (V_L + 1) + l; l == V_L packs the logits
__device__ void pack_body(const PackArgs& a) {
    const int cta = blockIdx.x / (V_L + 1), l = blockIdx.x % (V_L + 1);
    const Place P = load_place(a.PT, cta);
    const int wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5, lane = threadIdx.x & 31;
    unsigned char* base = a.WP + (size_t)P.base * FRAG_BYTES;
    if (l == V_L) {
        pack_wide(a, base + (size_t)V_L * P.layer * FRAG_BYTES, 4, 0, P.log_j0, P.log_nj, 0, KT_D, wid, nwarp, lane);
        return;
    }
    unsigned char* s = base + (size_t)l * P.layer * FRAG_BYTES;
    pack_narrow(a, s, 0, l, P.qkv_j0, P.qkv_nj, KT_D, wid, nwarp, lane);
    s += (size_t)narrow_tiles(P.qkv_nj, KT_D) * FRAG_BYTES;
    pack_wide(a, s, 1, l, P.proj_j0, P.proj_nj, P.proj_k0, P.proj_nk, wid, nwarp, lane);
    s += (size_t)wide_tiles(P.proj_nj, P.proj_nk) * FRAG_BYTES;
    pack_narrow(a, s, 2, l, P.fc_j0, P.fc_nj, KT_D, wid, nwarp, lane);
    s += (size_t)narrow_tiles(P.fc_nj, KT_D) * FRAG_BYTES;
    pack_wide(a, s, 3, l, 0, JT_D, P.fc_j0, P.fc_nj, wid, nwarp, lane);
}
