// The decode step for at most eight sequences (one batch tile of the tensor-core products), written for sm_100a
// (B200, 148 SMs): one persistent cooperative kernel, one CTA per SM, 8 consumer warps + 2 producer warps.
//
// A step of a small batch moves few bytes per phase (GPT-2 small: 96 KB of weights per CTA and layer), so what it
// costs is the chain of dependent operations between its grid-wide exchanges, not bandwidth. This text keeps that
// chain short:
//   * the weights stream through a ring of shared-memory slots (cp.async.bulk, mbarrier pairs), filled by the
//     producer warp from a packed copy in exactly the order the CTA consumes it; the producer runs ahead through
//     the grid barriers, so a phase never waits for memory;
//   * a contraction over the whole fold (QKV, FC) splits the fold over the eight warps: every warp multiplies its
//     fold tiles into all of the CTA's output tiles (one operand load per fold tile, products on mma.sync m16n8k16
//     with the weight tile as A and the batch as N), the warps' sums meet once in shared memory and the epilogue
//     (bias, q / K / V emit, GELU) works on complete sums;
//   * a contraction over a slice of the fold (attention projection, MLP projection) gives every warp whole output
//     tiles: no exchange inside the CTA, fp32 atomics into the vector the LayerNorm pass started;
//   * LayerNorm: one warp per row with the row in registers (8 sequences) or 8 / rows warps per row;
//   * attention: the (sequence, head, position chunk) items of a CTA are cut into tiles of 128 positions once per
//     step (the positions do not change between layers); the producer thread requests the K/V tiles by TMA from
//     that list, the first ones before the barrier that ends QKV; the row of the current position, written during
//     QKV by other CTAs, is copied into its place after the barrier; scores and output on mma.sync via ldmatrix,
//     online softmax in registers;
//   * per layer: [LN1 + QKV + KV emit] | [attention] | [attn-proj + residual] | [LN2 + FC + GELU + MLP-proj +
//     residual], a grid barrier after each; then LN_f + logits + argmax, finished by the last CTA to arrive.
// Activations are fp32, split into an fp16 head and an fp16 remainder for the products (two MMAs, fp32 accumulate).
// Every wait is bounded: on expiry the kernel records where in bar[0], raises the abort flag that all other waits
// poll, and runs to its end.

#define WN_MAX V_WN                     // most output tiles a CTA holds in a whole-fold contraction (at most 4)
#define CH V_CH                         // tiles per ring slot
#define SLOT_BYTES (CH * FRAG_BYTES)
#define ATILE 576                       // operand tiles (16 fold indices x 8 sequences; per lane head.x, head.y, rem.x, rem.y = 512 B) are
                                        // 576 B apart: the LayerNorm's 16-byte stores to eight tiles at once then spread over all banks
#define UMAX V_UMAX                     // deepest fold slice of a projection unit (tiles)

#define PT_STRIDE 16
#define PT_BASE 0        // first tile of this CTA's stream, in 512 B tiles
#define PT_LAYER 1       // tiles per layer
#define PT_QKV_J0 2      // whole fold: output tiles [j0, j0 + nj)
#define PT_QKV_NJ 3
#define PT_PROJ_J0 4     // fold slice: output tiles [j0, j0 + nj), fold tiles [k0, k0 + nk)
#define PT_PROJ_NJ 5
#define PT_PROJ_K0 6
#define PT_PROJ_NK 7
#define PT_FC_J0 8       // whole fold; the same tiles are the fold slice of the MLP projection
#define PT_FC_NJ 9
#define PT_LOG_J0 10     // vocabulary tiles, whole fold
#define PT_LOG_NJ 11

extern __shared__ __align__(1024) unsigned char smem[];

// The state vectors z (the sums the projections add into) are fp32, combined with floating-point atomics in arrival
// order: the last bits of a sum then depend on the order. V_FIXED (lowering option `ordered`) keeps them as 64-bit
// fixed point (36 fractional bits: finer than fp32 for |z| < 2^27) combined with integer atomics: integer addition is
// associative, so every run gives the same bits whatever the order, at the price of 8-byte scalar atomics and loads.
#if V_FIXED
typedef long long zacc;
#define ZSCALE 68719476736.0f
__device__ __forceinline__ zacc to_acc(float v) { return __float2ll_rn(v * ZSCALE); }
__device__ __forceinline__ float from_acc(zacc v) { return __ll2float_rn(v) * (1.0f / ZSCALE); }
__device__ __forceinline__ void acc_add(zacc* p, float v) {
    asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" :: "l"(p), "l"(to_acc(v)) : "memory");
}
__device__ __forceinline__ float2 acc_load2(const zacc* p) {
    const longlong2 v = __ldcg(reinterpret_cast<const longlong2*>(p));
    return make_float2(from_acc(v.x), from_acc(v.y));
}
#else
typedef float zacc;
__device__ __forceinline__ zacc to_acc(float v) { return v; }
__device__ __forceinline__ void acc_add(zacc* p, float v) { red_add(p, v); }
__device__ __forceinline__ float2 acc_load2(const zacc* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }
#endif

// shared memory: the offsets come from the lowering (V_SM_*); inside the last block:
#define MISC_ATT 0                                   // 2 x NW x (V_E + 2) floats: the warps' partial results of an item
#define MISC_BEST (2 * NW * (V_E + 2) * 4)           // 8 x NW u64
#define MISC_POS (MISC_BEST + 8 * NW * 8)            // 8 ints: positions of the sequences in this step
#define MISC_STAT (MISC_POS + 32)                    // 2 x 8 x 8 floats: LayerNorm partial sums of the warps of a row
#define MISC_FLAG (MISC_STAT + 512)
#define MISC_STOP (MISC_FLAG + 4)
#define MISC_ATTSEQ (MISC_FLAG + 8)                  // attention phases the consumers have opened
#define MISC_NTL (MISC_FLAG + 12)                    // entries of the tile list
#define MISC_TL (MISC_FLAG + 16)                     // V_MAXTL x int4
#define MISC_BYTES (MISC_TL + V_MAXTL * 16)

struct Ctx {
    u32* bar;          // global counters
    u32 gen;           // barrier generation x CTAs
    u32 chunk;         // ring slots used so far (the same count in every consumer warp and in the producer)
    u32 kvi, kvn;      // K/V tiles requested / used so far (stage = count % V_KVST)
    u32 seq;           // producer: attention phases entered
    int cta, ncta, tid, warp, lane;
    bool dead;         // a bounded wait expired somewhere: skip waits from now on
};
#if V_TIMING
// event trace of one CTA (V_TIMING - 1) in one layer: per warp up to TRACE_EVENTS (id, clock) pairs in shared memory
#define TRACE_EVENTS 96
__shared__ u64 trace_[(V_NW + 2) * TRACE_EVENTS];
__shared__ int trace_n[V_NW + 2];
__shared__ int trace_on;
__device__ __forceinline__ void trace_event(int id) {
    if ((threadIdx.x & 31) == 0 && *reinterpret_cast<volatile int*>(&trace_on)) {
        const int w = threadIdx.x >> 5, n = trace_n[w];
        if (n < TRACE_EVENTS) { trace_[w * TRACE_EVENTS + n] = ((u64)(id) << 48) | ((u64)clock64() & 0xFFFFFFFFFFFFull); trace_n[w] = n + 1; }
    }
}
#define TRACE(id) trace_event(id)
#else
#define TRACE(id) do { } while (0)
#endif

// per-CTA placement, read once
struct Plan {
    int qkv_j0, qkv_nj, proj_j0, proj_nj, proj_k0, proj_nk, fc_j0, fc_nj, log_j0, log_nj;
    int rpc_qkv, rpc_fc, upc_proj, upc_p2;       // fold rows / units per ring slot
};
// fold rows of a whole-fold contraction per ring slot: whole waves of eight rows (one per warp) where they fit
__device__ __forceinline__ int rows_per_slot(int nj) {
    const int k = CH / max(nj, 1), w = k & ~7;
    return (w * max(nj, 1) * 8 >= CH * 7) ? w : k;      // unless that leaves more than an eighth of the slot empty
}
__device__ __forceinline__ Plan load_plan(const int* __restrict__ P) {
    Plan p;
    p.qkv_j0 = P[PT_QKV_J0]; p.qkv_nj = P[PT_QKV_NJ]; p.proj_j0 = P[PT_PROJ_J0]; p.proj_nj = P[PT_PROJ_NJ];
    p.proj_k0 = P[PT_PROJ_K0]; p.proj_nk = P[PT_PROJ_NK]; p.fc_j0 = P[PT_FC_J0]; p.fc_nj = P[PT_FC_NJ];
    p.log_j0 = P[PT_LOG_J0]; p.log_nj = P[PT_LOG_NJ];
    p.rpc_qkv = rows_per_slot(p.qkv_nj); p.rpc_fc = rows_per_slot(p.fc_nj);
    p.upc_proj = rows_per_slot(p.proj_nk); p.upc_p2 = rows_per_slot(p.fc_nj);
    return p;
}

__device__ __forceinline__ u32 full_bar(u32 slot) { return smem_u32(smem + V_SM_BARS) + slot * 8; }
__device__ __forceinline__ u32 empty_bar(u32 slot) { return smem_u32(smem + V_SM_BARS) + (V_NSLOT + slot) * 8; }
__device__ __forceinline__ u32 kv_bar(u32 stage) { return smem_u32(smem + V_SM_BARS) + (2 * V_NSLOT + stage) * 8; }
__device__ __forceinline__ u32 kv_empty_bar(u32 stage) { return smem_u32(smem + V_SM_BARS) + (2 * V_NSLOT + V_KVST + stage) * 8; }

__device__ __forceinline__ void wait_mbar(Ctx& c, u32 mbar, u32 parity, u32 where) {
    if (c.dead || mbar_try(mbar, parity)) return;
    if (!mbar_wait_slow(c.bar, mbar, parity, where, c.cta, reinterpret_cast<const volatile int*>(smem + V_SM_MISC + MISC_STOP))) c.dead = true;
}

__device__ __forceinline__ u32 ctx_state(const Ctx& c) { return c.chunk | (c.dead ? 0x80000000u : 0u); }
__device__ __forceinline__ void ctx_set(Ctx& c, u32 st) { c.chunk = st & 0x7fffffffu; c.dead = (st >> 31) != 0; }

// Grid barrier of the consumer warps, in two halves so that loads that do not depend on other CTAs (the next
// phase's parameters) can be issued in between. One monotonic counter: every CTA adds 1 (release), thread 0 of
// every CTA polls it until it reaches generation x CTAs.
__device__ __forceinline__ void phase_end(Ctx& c) {
    cons_sync();
    c.gen += (u32)c.ncta;
    if (c.tid == 0) asm volatile("red.release.gpu.global.add.u32 [%0], 1;" :: "l"(c.bar + BAR_COUNT) : "memory");
}
__device__ __noinline__ bool grid_wait_slow(u32* bar, u32 gen, int cta) {
    const u64 t0 = now_ns();
    u32 spins = 0;
    while ((int)(ld_acquire(bar + BAR_COUNT) - gen) < 0) {
        if ((++spins & 63u) == 0) {
            if (ld_relaxed(bar + BAR_ABORT)) return false;
            if (now_ns() - t0 > WAIT_NS) { give_up(bar, 0x100u, cta); return false; }
        }
    }
    return true;
}
__device__ __forceinline__ void phase_wait(Ctx& c) {
    if (c.tid == 0 && !c.dead) grid_wait_slow(c.bar, c.gen, c.cta);
    cp_wait();                                 // this thread's share of the parameters has landed
    cons_sync();
    if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
}

// ---------------------------------------------------------------------------------------------
// attention work of this CTA in one step, as a list of K/V tiles
// ---------------------------------------------------------------------------------------------
#define ATT_ITEMS (V_B * V_H * V_NCH)            // (sequence, head, position chunk), dealt round-robin over the CTAs
#define KV_POS 128                               // positions per tile: sixteen per warp
#define KV_SMALL 32                              // TMA boxes of 32, 64, 96 and 128 rows
#define KV_TILE_BYTES (KV_POS * 128)             // the K (or V) rows of one tile
#define KV_STAGE_BYTES (2 * KV_TILE_BYTES)       // K rows, then V rows
#define TMAP_BYTES 128
#define PART_STRIDE (V_E + 2)
// a list entry: x = sequence | head << 8 | flags, y = first position, z = positions (0: an empty chunk), w = item
#define TL_LAST (1 << 16)                        // last tile of its item: the item's result is written after it
#define TL_PATCH (1 << 17)                       // may be requested before QKV has written the current position's row
// V_FUSE_PROJ (one chunk per (sequence, head)): the CTA that finishes an item also multiplies its 64 outputs by the 64
// rows of the projection that belong to the head (JT_D output tiles x 4 fold tiles, one copy per layer and head behind
// the per-CTA streams of the packed weights, fetched behind the item's K/V tiles) and adds the result into z1: no separate projection phase, one grid barrier less per layer.
#define FUSE_US (V_E / 16)
#define FUSE_PER (8 * FUSE_US)                   // eight output tiles (one per warp) per ring slot

// by one thread, once per step: the positions are the same in every layer
__device__ __noinline__ void build_tile_list(int cta, int ncta, const int* s_pos) {
    int4* tl = reinterpret_cast<int4*>(smem + V_SM_MISC + MISC_TL);
    int n = 0, live = 0;
#pragma unroll 1
    for (int it = cta; it < ATT_ITEMS && n < V_MAXTL; it += ncta) {
        const int bh = it / V_NCH, ch = it - bh * V_NCH, b = bh / V_H, h = bh - b * V_H;
        const int npos = s_pos[b] + 1;                                   // <= 0: a sequence that has not started
        const int cs = (max(npos, 1) + V_NCH - 1) / V_NCH;
        int s = ch * cs;
        const int hi = min(npos, (ch + 1) * cs);
        if (hi <= s) { tl[n++] = make_int4(b | (h << 8) | TL_LAST, 0, 0, it); continue; }
#pragma unroll 1
        for (; s < hi && n < V_MAXTL; s += KV_POS) {
            const int cnt = min(KV_POS, hi - s);
            const int flags = ((s + KV_POS >= hi) ? TL_LAST : 0) | (((V_FUSE_X2 || live < V_KVST) && s_pos[b] >= s && s_pos[b] < s + cnt) ? TL_PATCH : 0);
            tl[n++] = make_int4(b | (h << 8) | flags, s, cnt, it);
            live++;
        }
    }
    *reinterpret_cast<volatile int*>(smem + V_SM_MISC + MISC_NTL) = n;
}

// ---------------------------------------------------------------------------------------------
// producer: one thread walks this CTA's weight stream and requests its K/V tiles
// ---------------------------------------------------------------------------------------------
// leaving early: first let the copies still in flight land (bounded), so that none writes into shared memory
// after the CTA has gone
__device__ __noinline__ void producer_drain(Ctx& c) {
    for (u32 k = c.chunk > V_NSLOT ? c.chunk - V_NSLOT : 0u; k < c.chunk; k++) {
        const u64 t0 = now_ns();
        while (!mbar_try(full_bar(k % V_NSLOT), (k / V_NSLOT) & 1u) && now_ns() - t0 < WAIT_NS) { }
    }
    for (u32 k = c.kvi > V_KVST ? c.kvi - V_KVST : 0u; k < c.kvi; k++) {
        const u64 t0 = now_ns();
        while (!mbar_try(kv_bar(k % V_KVST), (k / V_KVST) & 1u) && now_ns() - t0 < WAIT_NS) { }
    }
}
// `ntiles` tiles from src into ring slots of at most `per` tiles
__device__ __forceinline__ void stream_tiles(Ctx& c, const unsigned char*& src, int ntiles, int per) {
#pragma unroll 1
    for (int i = 0; i < ntiles; i += per) {
        const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
        wait_mbar(c, empty_bar(slot), (use & 1u) ^ 1u, 0x200u);
        if (c.dead) return;
        const u32 bytes = (u32)min(per, ntiles - i) * FRAG_BYTES;
        mbar_expect(full_bar(slot), bytes);
        bulk_g2s(smem_u32(smem + V_SM_RING) + slot * SLOT_BYTES, src, bytes, full_bar(slot));
        src += bytes;
        c.chunk++;
    }
}
// The K/V tiles of one attention phase, in list order, each as soon as its stage has been released by all consumer
// warps. The consumers open the phase (a counter in shared memory) when they start the layer's QKV contraction: the
// first V_KVST requests then precede the grid barrier that ends QKV, and the consumers put the row of the current
// position in its place themselves; every later request follows a release made after that barrier.
__device__ __forceinline__ void producer_attention(Ctx& c, int l, const unsigned char* __restrict__ TM) {
    {
        const volatile u32* seq = reinterpret_cast<const volatile u32*>(smem + V_SM_MISC + MISC_ATTSEQ);
        const volatile int* stop = reinterpret_cast<const volatile int*>(smem + V_SM_MISC + MISC_STOP);
        c.seq++;
        const u64 t0 = now_ns();
        u32 spins = 0;
        while ((int)(*seq - c.seq) < 0) {
            __nanosleep(100);                      // this thread shares a scheduler with two consumer warps
            if (*stop) { c.dead = true; return; }
            if ((++spins & 63u) == 0) {
                if (ld_relaxed(c.bar + BAR_ABORT)) { c.dead = true; return; }
                if (now_ns() - t0 > WAIT_NS) { give_up(c.bar, 0x800u, c.cta); c.dead = true; return; }
            }
        }
        __threadfence_block();
    }
    const int4* tl = reinterpret_cast<const int4*>(smem + V_SM_MISC + MISC_TL);
    const int ntl = *reinterpret_cast<const volatile int*>(smem + V_SM_MISC + MISC_NTL);
#pragma unroll 1
    for (int k = 0; k < ntl; k++) {
        const int4 e = tl[k];
        if (e.z == 0) continue;
        const u32 stage = c.kvi % V_KVST;
        wait_mbar(c, kv_empty_bar(stage), ((c.kvi / V_KVST) & 1u) ^ 1u, 0x800u);
        if (c.dead) return;
        const int b = e.x & 255, h = (e.x >> 8) & 255;
        const int q = (e.z + KV_SMALL - 1) / KV_SMALL - 1;                  // the smallest box that covers the tile
        const u32 bar = kv_bar(stage), dst = smem_u32(smem + V_SM_KV) + stage * KV_STAGE_BYTES;
        // rows that other CTAs wrote with ordinary stores, a stage that was read and patched with ordinary accesses
        asm volatile("fence.proxy.async.global;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect(bar, 2 * (q + 1) * KV_SMALL * 128);
        tma_rows(dst, TM + (2 * q) * TMAP_BYTES, h * V_E, e.y, b * V_L + l, bar);
        tma_rows(dst + KV_TILE_BYTES, TM + (2 * q + 1) * TMAP_BYTES, h * V_E, e.y, b * V_L + l, bar);
        c.kvi++;
    }
}

// Two producer threads (lane 0 of two warps), each with a resource of its own and an order of its own:
//   * the weight producer walks this CTA's stream into the ring. Its order is fixed at lowering time (in the fused mode
//     the heads of this CTA's attention items are cta + k * grid modulo the head count), so it never waits for
//     anything but a free slot and runs ahead through barriers and attention phases;
//   * the K/V producer requests the tiles of the attention phases from the per-step list as stages become free.
__device__ __noinline__ void producer_weights(u32* bar, const int* __restrict__ P, const unsigned char* __restrict__ WP, int cta, int ncta, int nsteps) {
    Ctx c;
    c.bar = bar; c.chunk = 0; c.dead = false; c.cta = cta; c.ncta = ncta; c.kvi = 0; c.seq = 0;
    const Plan p = load_plan(P);
    const unsigned char* base = WP + (size_t)(u32)P[PT_BASE] * FRAG_BYTES;
    const int per_qkv = p.rpc_qkv * p.qkv_nj, per_fc = p.rpc_fc * p.fc_nj;
    const int per_proj = p.upc_proj * p.proj_nk, per_p2 = p.upc_p2 * p.fc_nj;
#pragma unroll 1
    for (int step = 0; step < nsteps; step++) {                  // every step reads the same stream again
        const unsigned char* src = base;
#pragma unroll 1
        for (int l = 0; l < V_L; l++) {
            stream_tiles(c, src, p.qkv_nj * KT_D, per_qkv);
#if V_FUSE_PROJ
#pragma unroll 1
            for (int it = cta; it < ATT_ITEMS && !c.dead; it += ncta) {
                const unsigned char* hs = WP + ((size_t)V_FUSE_BASE + (size_t)(l * V_H + it % V_H) * (JT_D * FUSE_US)) * FRAG_BYTES;
#if V_FUSE_X
                // only this CTA's share of the head's output tiles (the items of a head exchange their outputs)
                const int xb = it / V_H, j0 = (xb * JT_D) / V_B, j1 = ((xb + 1) * JT_D) / V_B;
                hs += (size_t)j0 * FUSE_US * FRAG_BYTES;
                stream_tiles(c, hs, (j1 - j0) * FUSE_US, FUSE_PER);
#else
                stream_tiles(c, hs, JT_D * FUSE_US, FUSE_PER);
#endif
            }
#else
            if (!c.dead) stream_tiles(c, src, p.proj_nj * p.proj_nk, per_proj);
#endif
            if (!c.dead) stream_tiles(c, src, p.fc_nj * KT_D, per_fc);
            if (!c.dead) stream_tiles(c, src, p.fc_nj * JT_D, per_p2);
            if (c.dead) { producer_drain(c); return; }
        }
#pragma unroll 1
        for (int j = 0; j < p.log_nj; j += 2 * NW) {
            const int width = min(2 * NW, p.log_nj - j);
            stream_tiles(c, src, width * KT_D, (CH / width) * width);
            if (c.dead) { producer_drain(c); return; }
        }
    }
}
__device__ __noinline__ void producer_kv(u32* bar, const unsigned char* __restrict__ TM, int cta, int ncta, int nsteps) {
    Ctx c;
    c.bar = bar; c.chunk = 0; c.dead = false; c.cta = cta; c.ncta = ncta; c.kvi = 0; c.seq = 0;
#pragma unroll 1
    for (int i = 0; i < nsteps * V_L; i++) {
        producer_attention(c, i % V_L, TM);
        if (c.dead) { producer_drain(c); return; }
    }
}

// ---------------------------------------------------------------------------------------------
// contractions
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 lds16(const unsigned char* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void mma_hl(float (&hi)[4], float (&lo)[4], const uint4& a, const uint4& b) {
    mma16816(hi, a, b.x, b.y);
    mma16816(lo, a, b.z, b.w);
}
// The contractions are out of line (one copy each: the kernel's code has to stay resident in the instruction cache
// while a layer runs), so they take what they need of the context by value: `st` = ring slots used so far, bit 31 set
// once a wait has been abandoned; they return the new value.
#define ST_DEAD 0x80000000u
__device__ __forceinline__ void wait_full(u32& st, u32* bar, int cta, u32 slot, u32 parity) {
    if ((st & ST_DEAD) || mbar_try(full_bar(slot), parity)) return;
    if (!mbar_wait_slow(bar, full_bar(slot), parity, 0x300u, cta, reinterpret_cast<const volatile int*>(smem + V_SM_MISC + MISC_STOP))) st |= ST_DEAD;
}

// Whole fold, NJ output tiles (stream order: fold tile major), operand tiles at V_SM_ACT. Warp w takes the fold
// tiles w, w + 8, ... and multiplies each into all NJ output tiles, alternating between two sets of accumulators
// (short dependency chains); the sums of the eight warps are left in shared memory (V_SM_RED: [warp][output tile]
// [lane] x 4 floats) for the epilogue, which runs after a block-wide sync. One instance per NJ: the loops are
// straight-line code for the CTA's own count.
template <int NJ>
__device__ __noinline__ u32 gemm_whole_fold_n(u32 st, u32* bar, int cta, int rpc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float acc[2][NJ][4], lo[2][NJ][4];
#pragma unroll
    for (int s = 0; s < 2; s++)
#pragma unroll
        for (int j = 0; j < NJ; j++)
#pragma unroll
            for (int i = 0; i < 4; i++) { acc[s][j][i] = 0.f; lo[s][j][i] = 0.f; }
    const unsigned char* actl = smem + V_SM_ACT + lane * 16;
#pragma unroll 1
    for (int r0 = 0; r0 < KT_D; r0 += rpc) {
        const u32 chunk = st & ~ST_DEAD, slot = chunk % V_NSLOT, use = chunk / V_NSLOT;
        wait_full(st, bar, cta, slot, use & 1u);
        const unsigned char* tiles = smem + V_SM_RING + slot * SLOT_BYTES + lane * 16;
        const int nr = (st & ST_DEAD) ? 0 : min(rpc, KT_D - r0);
        int r = warp;
#pragma unroll 1
        for (; r + NW < nr; r += 2 * NW) {
            const uint4 b0 = lds16(actl + (r0 + r) * ATILE), b1 = lds16(actl + (r0 + r + NW) * ATILE);
            const unsigned char* tp = tiles + (r * NJ) * FRAG_BYTES;
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                mma_hl(acc[0][j], lo[0][j], lds16(tp + j * FRAG_BYTES), b0);
                mma_hl(acc[1][j], lo[1][j], lds16(tp + (NW * NJ + j) * FRAG_BYTES), b1);
            }
        }
        if (r < nr) {
            const uint4 b0 = lds16(actl + (r0 + r) * ATILE);
            const unsigned char* tp = tiles + (r * NJ) * FRAG_BYTES;
#pragma unroll
            for (int j = 0; j < NJ; j++) mma_hl(acc[0][j], lo[0][j], lds16(tp + j * FRAG_BYTES), b0);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(slot));
        st++;
    }
    float* red = reinterpret_cast<float*>(smem + V_SM_RED);
#pragma unroll
    for (int j = 0; j < NJ; j++)
        *reinterpret_cast<float4*>(red + ((warp * WN_MAX + j) * 32 + lane) * 4) =
            make_float4((acc[0][j][0] + lo[0][j][0]) + (acc[1][j][0] + lo[1][j][0]), (acc[0][j][1] + lo[0][j][1]) + (acc[1][j][1] + lo[1][j][1]),
                        (acc[0][j][2] + lo[0][j][2]) + (acc[1][j][2] + lo[1][j][2]), (acc[0][j][3] + lo[0][j][3]) + (acc[1][j][3] + lo[1][j][3]));
    return st;
}
__device__ __forceinline__ u32 gemm_whole_fold(u32 st, u32* bar, int cta, int nj, int rpc) {
    switch (nj) {
        case 1: return gemm_whole_fold_n<1>(st, bar, cta, rpc);
#if WN_MAX >= 2
        case 2: return gemm_whole_fold_n<2>(st, bar, cta, rpc);
#endif
#if WN_MAX >= 3
        case 3: return gemm_whole_fold_n<3>(st, bar, cta, rpc);
#endif
#if WN_MAX >= 4
        case 4: return gemm_whole_fold_n<4>(st, bar, cta, rpc);
#endif
        default: return st;                     // the placement gives a CTA at most WN_MAX output tiles
    }
}
// complete sum of output `o` (tile o / 128, element (o % 128) of the accumulator layout: lane * 4 + register)
__device__ __forceinline__ float whole_fold_sum(const float* red, int o) {
    const int j = o >> 7, r = o & 127;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < NW; w++) v += red[(w * WN_MAX + j) * 128 + r];
    return v;
}

// The sums of one output tile (accumulator layout of mma.m16n8k16: lane (g, t) holds outputs g and g + 8 of sequences
// 2t and 2t + 1) added to z[b][unit * 16 + ...] with one 16-byte atomic per lane instead of four 4-byte ones: the
// four lanes g = 4i .. 4i + 3 transpose their 4 x 4 values (four shuffles), after which lane q = g % 4 holds four
// consecutive outputs of sequence 2t + q % 2 in the tile's half q / 2. A 148-way sum at eight sequences is bound by the
// number of atomic operations the L2 has to retire.
// `only` >= 0: only that sequence's sums are added (the operand held one live row).
__device__ __forceinline__ void red_tile(zacc* __restrict__ zu, const float (&v)[4], int lane, int only) {
    const int g = lane >> 2, t = lane & 3, q = g & 3;
    if (V_B <= 2 || V_FIXED) {
        // one or two sequences (only the lanes with t == 0 hold live sums: the transposition costs more than it
        // saves, measured), or fixed-point sums: scalar atomics
        zacc* o = zu + (size_t)(2 * t) * V_D + g;
        if (2 * t < V_B && (only < 0 || only == 2 * t)) { acc_add(o, v[0]); acc_add(o + 8, v[2]); }
        if (2 * t + 1 < V_B && (only < 0 || only == 2 * t + 1)) { acc_add(o + V_D, v[1]); acc_add(o + V_D + 8, v[3]); }
        return;
    }
    const bool odd = q & 1, hi = q & 2;
    // round 1, partner g ^ 1: even lanes keep registers 0 and 2, odd lanes 1 and 3
    const float s0 = odd ? v[0] : v[1], s1 = odd ? v[2] : v[3];
    const float r0 = __shfl_xor_sync(0xffffffffu, s0, 4), r1 = __shfl_xor_sync(0xffffffffu, s1, 4);
    const float ax = odd ? r0 : v[0], ay = odd ? v[1] : r0;          // register q % 2 of rows (g & ~1), (g & ~1) + 1
    const float bx = odd ? r1 : v[2], by = odd ? v[3] : r1;          // register 2 + q % 2 of the same rows
    // round 2, partner g ^ 2: lanes 0, 1 keep the a pair (tile half 0), lanes 2, 3 the b pair (tile half 1)
    const float t0 = hi ? ax : bx, t1 = hi ? ay : by;
    const float u0 = __shfl_xor_sync(0xffffffffu, t0, 8), u1 = __shfl_xor_sync(0xffffffffu, t1, 8);
    const float o0 = hi ? u0 : ax, o1 = hi ? u1 : ay, o2 = hi ? bx : u0, o3 = hi ? by : u1;
    const int b = 2 * t + (q & 1);
#if !V_FIXED
    if (b < V_B && (only < 0 || only == b))
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     :: "l"(zu + (size_t)b * V_D + (g & ~3) + (hi ? 8 : 0)), "f"(o0), "f"(o1), "f"(o2), "f"(o3) : "memory");
#endif
}

// A slice of US fold tiles for `nunits` output tiles (stream order: output tile major). Warp w takes the output
// tiles w, w + 8, ... of every ring slot, two at a time (independent chains of products); the sums are added to
// zt[b][unit * 16 + ...] with fp32 atomics (the other slices of the fold are other CTAs'). The operand tiles of
// the slice are read once, into registers. One instance per US.
template <int US>
__device__ __noinline__ u32 gemm_fold_slice_n(u32 st, u32* bar, int cta, int nunits, int upc, const unsigned char* act, zacc* __restrict__ zt, int only) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint4 bop[US];
#pragma unroll
    for (int r = 0; r < US; r++) bop[r] = lds16(act + r * ATILE + lane * 16);
#pragma unroll 1
    for (int u0 = 0; u0 < nunits; u0 += upc) {
        const u32 chunk = st & ~ST_DEAD, slot = chunk % V_NSLOT, use = chunk / V_NSLOT;
        wait_full(st, bar, cta, slot, use & 1u);
        TRACE(53);
        const unsigned char* tiles = smem + V_SM_RING + slot * SLOT_BYTES + lane * 16;
        const int nu = (st & ST_DEAD) ? 0 : min(upc, nunits - u0);
#pragma unroll 1
        for (int u = warp; u < nu; u += 2 * NW) {
            const bool two = u + NW < nu;
            float a0[4] = {0.f, 0.f, 0.f, 0.f}, l0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f}, l1[4] = {0.f, 0.f, 0.f, 0.f};
            const unsigned char* tp0 = tiles + (u * US) * FRAG_BYTES;
            const unsigned char* tp1 = tiles + ((two ? u + NW : u) * US) * FRAG_BYTES;
#pragma unroll
            for (int r = 0; r < US; r++) {
                const uint4 w0 = lds16(tp0 + r * FRAG_BYTES), w1 = lds16(tp1 + r * FRAG_BYTES);
                mma_hl(a0, l0, w0, bop[r]);
                mma_hl(a1, l1, w1, bop[r]);
            }
            const float f0[4] = {a0[0] + l0[0], a0[1] + l0[1], a0[2] + l0[2], a0[3] + l0[3]};
            red_tile(zt + (u0 + u) * 16, f0, lane, only);
            const float f1[4] = {a1[0] + l1[0], a1[1] + l1[1], a1[2] + l1[2], a1[3] + l1[3]};
            if (two) red_tile(zt + (u0 + u + NW) * 16, f1, lane, only);       // (warp-uniform)
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(slot));
        st++;
    }
    return st;
}
__device__ __forceinline__ u32 gemm_fold_slice(u32 st, u32* bar, int cta, int nunits, int us, int upc, const unsigned char* act, zacc* zt, int only = -1) {
    switch (us) {
        case 1: return gemm_fold_slice_n<1>(st, bar, cta, nunits, upc, act, zt, only);
#if UMAX >= 2
        case 2: return gemm_fold_slice_n<2>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 3
        case 3: return gemm_fold_slice_n<3>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 4
        case 4: return gemm_fold_slice_n<4>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 5
        case 5: return gemm_fold_slice_n<5>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 6
        case 6: return gemm_fold_slice_n<6>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 7
        case 7: return gemm_fold_slice_n<7>(st, bar, cta, nunits, upc, act, zt, only);
#endif
#if UMAX >= 8
        case 8: return gemm_fold_slice_n<8>(st, bar, cta, nunits, upc, act, zt, only);
#endif
        default: return st;                     // the lowering refuses placements with deeper slices
    }
}

// Exchange between CTAs without a grid barrier (every CTA holds at most one attention item): the producers write their
// values to global memory as (value, tag) pairs in one 8-byte store each, the tag being the number of the attention phase
// since the launch began (the buffer is cleared when a launch begins); a reader polls the pairs it needs until their
// tags are this phase's (bounded): the data is its own flag, no counter, no fence, no second trip to L2.
#define BAR_WHERE_HEAD 0xA00u
__device__ __forceinline__ void x_put(u64* p, float v, u32 tag) {
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" :: "l"(p), "l"(((u64)tag << 32) | (u64)__float_as_uint(v)) : "memory");
}
__device__ __forceinline__ u64 x_peek(const u64* p) {
    u64 v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __noinline__ bool x_get_slow(u32* bar, const u64* p, u32 tag, int cta, float& out) {
    const u64 t0 = now_ns();
    u32 spins = 0;
    for (;;) {
        const u64 v = x_peek(p);
        if ((u32)(v >> 32) == tag) { out = __uint_as_float((u32)v); return true; }
        if ((++spins & 63u) == 0) {
            if (ld_relaxed(bar + BAR_ABORT)) return false;
            if (now_ns() - t0 > WAIT_NS) { give_up(bar, BAR_WHERE_HEAD, cta); return false; }
        }
    }
}
#if V_FUSE_PROJ
// The projection of one attention item (fused mode): the head's 64 outputs (operand at V_SM_GACT, one live row `only`)
// times the head's 64 rows of the projection, JT_D output tiles x FUSE_US fold tiles, eight output tiles per ring slot.
// Several slots are taken at a time (the weight producer has had the whole attention phase to fill them): a warp then
// runs one independent chain of products per slot, so the chains overlap instead of following one another.
#define FUSE_GROUP (V_NSLOT - 1 < 6 ? V_NSLOT - 1 : 6)
__device__ __noinline__ u32 proj_head(u32 st, u32* bar, int cta, zacc* __restrict__ z1, int only) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint4 bop[FUSE_US];
#pragma unroll
    for (int r = 0; r < FUSE_US; r++) bop[r] = lds16(smem + V_SM_GACT + r * ATILE + lane * 16);
    constexpr int NSL = (JT_D + NW - 1) / NW;                    // ring slots of the item
#pragma unroll 1
    for (int s0 = 0; s0 < NSL; s0 += FUSE_GROUP) {
        const int g = min(FUSE_GROUP, NSL - s0);
        const u32 chunk = st & ~ST_DEAD;
        float a[FUSE_GROUP][4], l[FUSE_GROUP][4];
#pragma unroll
        for (int i = 0; i < FUSE_GROUP; i++) {
#pragma unroll
            for (int k = 0; k < 4; k++) { a[i][k] = 0.f; l[i][k] = 0.f; }
            if (i < g) wait_full(st, bar, cta, (chunk + i) % V_NSLOT, ((chunk + i) / V_NSLOT) & 1u);
        }
        TRACE(53);
        if (!(st & ST_DEAD)) {
            const unsigned char* tp[FUSE_GROUP];
#pragma unroll
            for (int i = 0; i < FUSE_GROUP; i++) tp[i] = smem + V_SM_RING + ((chunk + (i < g ? i : 0)) % V_NSLOT) * SLOT_BYTES + warp * (FUSE_US * FRAG_BYTES) + lane * 16;
#pragma unroll
            for (int r = 0; r < FUSE_US; r++) {
                // all loads of a round first, then its products: one chain per slot, none waits for another's load
                uint4 w[FUSE_GROUP];
#pragma unroll
                for (int i = 0; i < FUSE_GROUP; i++) w[i] = lds16(tp[i] + r * FRAG_BYTES);
#pragma unroll
                for (int i = 0; i < FUSE_GROUP; i++) mma_hl(a[i], l[i], w[i], bop[r]);
            }
#pragma unroll
            for (int i = 0; i < FUSE_GROUP; i++)
                if (i < g && (s0 + i) * NW + warp < JT_D) {
                    const float f[4] = {a[i][0] + l[i][0], a[i][1] + l[i][1], a[i][2] + l[i][2], a[i][3] + l[i][3]};
                    red_tile(z1 + ((s0 + i) * NW + warp) * 16, f, lane, only);
                }
        }
        __syncwarp();
        if (lane == 0)
            for (int i = 0; i < g; i++) mbar_arrive(empty_bar((chunk + i) % V_NSLOT));
        st += (u32)g;
    }
    return st;
}
#if V_FUSE_X
// This CTA's share [j0, j1) of the head's output tiles times the outputs of all V_B sequences (operand at V_SM_GACT, all
// rows live): eight output tiles per ring slot, one per warp.
__device__ __noinline__ u32 proj_head_x(u32 st, u32* bar, int cta, zacc* __restrict__ z1, int j0, int j1) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint4 bop[FUSE_US];
#pragma unroll
    for (int r = 0; r < FUSE_US; r++) bop[r] = lds16(smem + V_SM_GACT + r * ATILE + lane * 16);
#pragma unroll 1
    for (int jb = j0; jb < j1; jb += NW) {
        const u32 chunk = st & ~ST_DEAD;
        wait_full(st, bar, cta, chunk % V_NSLOT, (chunk / V_NSLOT) & 1u);
        TRACE(53);
        if (!(st & ST_DEAD) && jb + warp < j1) {
            const unsigned char* tp = smem + V_SM_RING + (chunk % V_NSLOT) * SLOT_BYTES + warp * (FUSE_US * FRAG_BYTES) + lane * 16;
            float a[4] = {0.f, 0.f, 0.f, 0.f}, l[4] = {0.f, 0.f, 0.f, 0.f};
            uint4 w[FUSE_US];
#pragma unroll
            for (int r = 0; r < FUSE_US; r++) w[r] = lds16(tp + r * FRAG_BYTES);
#pragma unroll
            for (int r = 0; r < FUSE_US; r++) mma_hl(a, l, w[r], bop[r]);
            const float f[4] = {a[0] + l[0], a[1] + l[1], a[2] + l[2], a[3] + l[3]};
            red_tile(z1 + (jb + warp) * 16, f, lane, -1);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_bar(chunk % V_NSLOT));
        st += 1u;
    }
    return st;
}
#endif
#endif

// ---------------------------------------------------------------------------------------------
// activations -> operand tiles in shared memory
// element (b, k): tile k / 16, lane b * 4 + (k % 8) / 2, word (k % 16) / 8 (+ 2 for the remainder), half k % 2
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void act_store1(unsigned char* act, int b, int k, float v) {
    const u16 hi = f2h(v);
    const int kt = k >> 4, kk = k & 15, reg = kk >> 3, t = (kk & 7) >> 1, half = kk & 1;
    u16* base = reinterpret_cast<u16*>(act + kt * ATILE + (b * 4 + t) * 16);
    base[reg * 2 + half] = hi;
    base[(2 + reg) * 2 + half] = f2h(v - h2f(hi));
}

// Parameters of the next LayerNorm phase into shared memory: gain and shift as fp32 (2 x V_D floats: the conversion
// happens here, in the shadow of the grid barrier, not in the LayerNorm pass), then as halves the bias added when the
// following combined vector is started (V_D) and the bias of this CTA's whole-fold output tiles. Warp 0 converts
// nothing: its first thread polls the barrier.
#define PRM_GAIN 0
#define PRM_SHIFT (V_D * 4)
#define PRM_INIT (V_D * 8)
#define PRM_TILE (V_D * 10)
__device__ __forceinline__ void fetch_params(Ctx& c, const u16* gw, const u16* gb, const u16* ib, const u16* tb, int tiles) {
    unsigned char* prm = smem + V_SM_PRM;
    const int per = V_D / 8;                       // 16-byte pieces per vector of halves
    if (ib) {
#pragma unroll 1
        for (int i = c.tid; i < per; i += NCONS) cp16(prm + PRM_INIT + i * 16, ib + i * 8);
    }
    if (tb && c.tid < tiles * 2) cp16(prm + PRM_TILE + c.tid * 16, tb + c.tid * 8);
#pragma unroll 1
    for (int i = c.tid - 32; i < 2 * per; i += NCONS - 32) {
        if (i < 0) continue;
        const int v = i >= per, q = v ? i - per : i;
        const uint4 h = __ldg(reinterpret_cast<const uint4*>((v ? gb : gw) + q * 8));
        float4* dst = reinterpret_cast<float4*>(prm + (v ? PRM_SHIFT : PRM_GAIN) + q * 32);
        dst[0] = make_float4(h_lo(h.x), h_hi(h.x), h_lo(h.y), h_hi(h.y));
        dst[1] = make_float4(h_lo(h.z), h_hi(h.z), h_lo(h.w), h_hi(h.w));
    }
}

// fp32 -> fp16 head + fp16 remainder of two values. The head is the value with its low 13 mantissa bits cleared (so
// its conversion to fp16 is exact in the normal range and needs no conversion back), the remainder what is left,
// rounded to fp16: together 21 to 22 bits of the value.
__device__ __forceinline__ void split_h2(float x, float y, u32& hi, u32& lo) {
    const float xh = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u), yh = __uint_as_float(__float_as_uint(y) & 0xFFFFE000u);
    hi = pack_h2(xh, yh);
    lo = pack_h2(x - xh, y - yh);
}

// LayerNorm of the rows of z (global, fp32, row stride V_D) into the operand tiles; gain and shift come from the
// parameter block in shared memory. LN_WPR warps share a row (eight sequences: one warp per row; one sequence: all
// eight warps on its row). A lane (u, t) of part wi holds the elements 2t, 2t+1, 2t+8, 2t+9 of the fold tiles
// u + 8 * (wi + LN_WPR * i): all loads independent (one round trip to L2), sums by warp shuffles (and through shared
// memory where several warps share the row), then the lane writes exactly the 16 bytes that thread (row, t) of a
// product reads from each of its tiles. Rows beyond the batch stay zero from the start of the kernel. The same pass
// starts the vector the following projection is combined into: init[b][d] += z[b][d] + bias[d], the fold tiles dealt
// over the CTAs (init was zeroed a phase earlier).
#define LN_ROWS (V_B <= 1 ? 1 : V_B <= 2 ? 2 : V_B <= 4 ? 4 : 8)
#define LN_WPR (NW / LN_ROWS)
#define LNI ((KT_D + 8 * LN_WPR - 1) / (8 * LN_WPR))
__device__ __noinline__ void ln_to_act(int cta, int ncta, const zacc* __restrict__ z, zacc* __restrict__ init) {
    unsigned char* act = smem + V_SM_ACT;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned char* prm = smem + V_SM_PRM;
    float* stat = reinterpret_cast<float*>(smem + V_SM_MISC + MISC_STAT);
    const int u = lane >> 2, t = lane & 3;
    const int rb = warp / LN_WPR, wi = warp % LN_WPR;
    const bool live = rb < V_B;
    const zacc* row = z + (size_t)rb * V_D + 2 * t;
    float2 v0[LNI], v1[LNI];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < LNI; i++) {
        const int kt = u + 8 * (wi + LN_WPR * i);
        v0[i] = make_float2(0.f, 0.f); v1[i] = make_float2(0.f, 0.f);
        if (live && kt < KT_D) {
            v0[i] = acc_load2(row + kt * 16);
            v1[i] = acc_load2(row + kt * 16 + 8);
        }
    }
#pragma unroll
    for (int i = 0; i < LNI; i++) s += (v0[i].x + v0[i].y) + (v1[i].x + v1[i].y);
#pragma unroll
    for (int m = 16; m; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
    if (LN_WPR > 1) {
        if (lane == 0) stat[warp] = s;
        cons_sync();
        s = 0.f;
#pragma unroll
        for (int w = 0; w < LN_WPR; w++) s += stat[rb * LN_WPR + w];
    }
    const float mean = s * (1.0f / V_D);
    TRACE(40);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < LNI; i++) {
        if (u + 8 * (wi + LN_WPR * i) < KT_D) {
            const float a0 = v0[i].x - mean, a1 = v0[i].y - mean, a2 = v1[i].x - mean, a3 = v1[i].y - mean;
            q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
        }
    }
#pragma unroll
    for (int m = 16; m; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
    if (LN_WPR > 1) {
        if (lane == 0) stat[64 + warp] = q;
        cons_sync();
        q = 0.f;
#pragma unroll
        for (int w = 0; w < LN_WPR; w++) q += stat[64 + rb * LN_WPR + w];
    }
    const float rs = rsqrtf(q * (1.0f / V_D) + V_EPS);
    TRACE(41);
    unsigned char* dst = act + (rb * 4 + t) * 16;
#pragma unroll
    for (int i = 0; i < LNI; i++) {
        const int kt = u + 8 * (wi + LN_WPR * i), k = kt * 16 + 2 * t;
        if (live && kt < KT_D) {
            const float2 w0 = *reinterpret_cast<const float2*>(prm + PRM_GAIN + k * 4), w1 = *reinterpret_cast<const float2*>(prm + PRM_GAIN + (k + 8) * 4);
            const float2 s0 = *reinterpret_cast<const float2*>(prm + PRM_SHIFT + k * 4), s1 = *reinterpret_cast<const float2*>(prm + PRM_SHIFT + (k + 8) * 4);
            const float o0 = (v0[i].x - mean) * rs * w0.x + s0.x, o1 = (v0[i].y - mean) * rs * w0.y + s0.y;
            const float o2 = (v1[i].x - mean) * rs * w1.x + s1.x, o3 = (v1[i].y - mean) * rs * w1.y + s1.y;
            uint4 out;
            split_h2(o0, o1, out.x, out.z);
            split_h2(o2, o3, out.y, out.w);
            *reinterpret_cast<uint4*>(dst + kt * ATILE) = out;
            if (init && ((KT_D <= V_MAXGRID) ? (kt == cta) : ((kt % ncta) == cta))) {
                const u32 i0 = *reinterpret_cast<const u32*>(prm + PRM_INIT + k * 2), i1 = *reinterpret_cast<const u32*>(prm + PRM_INIT + (k + 8) * 2);
                zacc* o = init + (size_t)rb * V_D + k;
                acc_add(o, v0[i].x + h_lo(i0)); acc_add(o + 1, v0[i].y + h_hi(i0));
                acc_add(o + 8, v1[i].x + h_lo(i1)); acc_add(o + 9, v1[i].y + h_hi(i1));
            }
        }
    }
    TRACE(42);
    cons_sync();
}

// Attention output for the fold tiles [k0, k0 + nk) of the projection, merged from the per-chunk partial results
// (m, sum, unnormalised o[V_E]) of the attention phase, into operand tiles 0 .. nk-1.
__device__ __forceinline__ void merge_to_act(Ctx& c, const float* __restrict__ part, int k0, int nk, unsigned char* act, u32 xphase) {
    const int cols = nk * 16;
    const float rcpk = rcp_fast(nk);
#pragma unroll 1
    for (int i = c.tid; i < V_B * cols; i += NCONS) {
        const int b = qdiv(i >> 4, rcpk), kk = i - b * cols, d = k0 * 16 + kk, h = d / V_E, e = d % V_E;
        const float* p = part + (size_t)((b * V_H + h) * V_NCH) * PART_STRIDE;
        // all loads first (independent, one round trip), then the arithmetic
        float mm[V_NCH], dd[V_NCH], oo[V_NCH], M = -3.0e38f;
#if V_FUSE_X3
        // (no grid barrier after the attention phase: the partial results are tagged values, polled until they are this phase's)
        const u64* p64 = reinterpret_cast<const u64*>(part) + (size_t)((b * V_H + h) * V_NCH) * PART_STRIDE;
        // all values of a round are requested together (one trip to L2 per round, not per value)
        u64 raw[V_NCH][3];
        const u64 t0 = now_ns();
        u32 spins = 0;
        for (;;) {
#pragma unroll
            for (int ch = 0; ch < V_NCH; ch++) { raw[ch][0] = x_peek(p64 + ch * PART_STRIDE); raw[ch][1] = x_peek(p64 + ch * PART_STRIDE + 1); raw[ch][2] = x_peek(p64 + ch * PART_STRIDE + 2 + e); }
            bool all = true;
#pragma unroll
            for (int ch = 0; ch < V_NCH; ch++) all = all && (u32)(raw[ch][0] >> 32) == xphase && (u32)(raw[ch][1] >> 32) == xphase && (u32)(raw[ch][2] >> 32) == xphase;
            if (all || c.dead) break;
            if ((++spins & 63u) == 0) {
                if (ld_relaxed(c.bar + BAR_ABORT)) { c.dead = true; break; }
                if (now_ns() - t0 > WAIT_NS) { give_up(c.bar, BAR_WHERE_HEAD, c.cta); c.dead = true; break; }
            }
        }
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) {
            mm[ch] = c.dead ? -3.0e38f : __uint_as_float((u32)raw[ch][0]);
            dd[ch] = c.dead ? 0.f : __uint_as_float((u32)raw[ch][1]);
            oo[ch] = c.dead ? 0.f : __uint_as_float((u32)raw[ch][2]);
        }
#else
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) { mm[ch] = __ldcg(p + ch * PART_STRIDE); dd[ch] = __ldcg(p + ch * PART_STRIDE + 1); oo[ch] = __ldcg(p + ch * PART_STRIDE + 2 + e); }
#endif
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) M = fmaxf(M, mm[ch]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int ch = 0; ch < V_NCH; ch++) {
            const float w = fast_exp(mm[ch] - M);
            den += w * dd[ch];
            num += w * oo[ch];
        }
        act_store1(act, b, kk, den > 0.f ? __fdividef(num, den) : 0.f);      // a sequence that has not started attends to nothing
    }
    cons_sync();
#if V_FUSE_X3
    if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
#endif
}

// ---------------------------------------------------------------------------------------------
// attention: the tiles of this CTA's list, each 128 positions (or fewer) of one (sequence, head). A tile's K rows
// and V rows (128 B per position and head) come into shared memory by TMA (two tensor copies that complete on the
// stage's mbarrier; the 128-byte swizzle spreads the rows over the banks for ldmatrix). A warp takes 16 positions of
// the tile. Scores: A = the K rows (ldmatrix, 16 positions x 16 dims per step), B = the query, its fp16 head in
// column 0 and its fp16 remainder in column 1, so that column 0 + column 1 is the fp32-accurate dot product. Online
// softmax on the 16 scores (held by the lanes with lane % 4 == 0). Output: A = V transposed (ldmatrix.trans, 16 dims
// x 16 positions), B = the weights, head and remainder again in columns 0 and 1. Result per item: (running max,
// sum, unnormalised o[V_E]) in global memory; the projection merges the chunks of a (sequence, head).
// ---------------------------------------------------------------------------------------------
// B operand of the scores: the query of (b, h), its fp16 head in column 0 (lanes with g == 0) and its fp16 remainder in
// column 1 (g == 1). The QKV epilogue stores the query in exactly this form (scaled where the divisor is a power of
// two): per (sequence, head) 128 halves ordered [column][t][k step][register][half], so a lane reads its eight
// registers with two 16-byte loads and no conversion.
__device__ __forceinline__ void att_load_q(u32 (&bq)[V_E / 16][2], const u32* __restrict__ qop, int b, int h, int g, int t) {
    uint4 x = make_uint4(0, 0, 0, 0), y = make_uint4(0, 0, 0, 0);
    if (g < 2) {
        const uint4* p = reinterpret_cast<const uint4*>(qop + (size_t)(b * V_H + h) * 64 + g * 32 + t * 8);
        x = __ldcg(p); y = __ldcg(p + 1);
    }
    bq[0][0] = x.x; bq[0][1] = x.y; bq[1][0] = x.z; bq[1][1] = x.w;
    bq[2][0] = y.x; bq[2][1] = y.y; bq[3][0] = y.z; bq[3][1] = y.w;
}
// one element of the query into that form: column 0 gets the fp16 head, column 1 the fp16 remainder
__device__ __forceinline__ void q_store(u16* __restrict__ qop16, int b, int jx, float v) {
    const float vs = V_SCALE_IS_POW2 ? v * (1.0f / V_SCALE) : v;
    const int h = jx / V_E, e = jx - h * V_E, kq = e >> 4, kk = e & 15;
    u16* q = qop16 + (size_t)(b * V_H + h) * 128 + ((kk & 7) >> 1) * 16 + kq * 4 + (kk >> 3) * 2 + (kk & 1);
    const u16 hi = f2h(vs);
    q[0] = hi;
    q[64] = f2h(vs - h2f(hi));
}

__device__ __forceinline__ void attention_phase(Ctx& c, const u16* __restrict__ keys, const u16* __restrict__ vals, const u32* __restrict__ qbuf,
                                                float* __restrict__ part, zacc* __restrict__ z1, int l, const int* s_pos, u32 xphase, u64* __restrict__ xbase) {
#if V_FUSE_X
    u64* xo = xbase;                                                           // [head][sequence][V_E] (value, tag): the items' outputs
#endif
#if V_FUSE_X2
    const u64* xq = xbase + (size_t)(V_FUSE_X ? 1 : 0) * V_H * V_B * V_E;      // the same for the queries (fp16 head | remainder << 16),
    const u64* xk = xq + (size_t)V_H * V_B * V_E;                              // the K rows and the V rows of the current position
    const u64* xv = xk + (size_t)V_H * V_B * V_E;
#endif
    const int4* tl = reinterpret_cast<const int4*>(smem + V_SM_MISC + MISC_TL);
    const int ntl = *reinterpret_cast<const volatile int*>(smem + V_SM_MISC + MISC_NTL);
    if (ntl == 0) return;
    const int g = c.lane >> 2, t = c.lane & 3;
    u32 bq[V_E / 16][2], bqn[V_E / 16][2];           // the query of this item and of the next one
#pragma unroll
    for (int kq = 0; kq < V_E / 16; kq++) { bqn[kq][0] = 0; bqn[kq][1] = 0; }
#if V_FUSE_X2
    // No grid barrier between the QKV phase and this one: the query of the item and the K / V rows of the current position
    // come as tagged values from the CTAs that computed them (x_put in the QKV epilogue); threads 0..63 poll the query
    // (fp16 head and remainder in one word) and leave it in shared memory in operand order, threads 64..191 poll the K
    // and V rows and keep their half until the tile that holds the position has landed.
    u32 kvhalf = 0;
    {
        const int4 e = tl[0];
        const int b = e.x & 255, h = (e.x >> 8) & 255;
        u16* qs = reinterpret_cast<u16*>(smem + V_SM_RED);
        if (c.tid < 3 * V_E) {
            const int part = c.tid / V_E, el = c.tid - part * V_E;
            const u64* src = (part == 0 ? xq : part == 1 ? xk : xv) + ((size_t)h * V_B + b) * V_E + el;
            float got = 0.f;
            const u64 w = x_peek(src);
            if ((u32)(w >> 32) == xphase) got = __uint_as_float((u32)w);
            else if (c.dead || !x_get_slow(c.bar, src, xphase, c.cta, got)) { c.dead = true; got = 0.f; }
            const u32 bits = __float_as_uint(got);
            if (part == 0) {
                const int kq = el >> 4, kk = el & 15;
                u16* q = qs + ((kk & 7) >> 1) * 16 + kq * 4 + (kk >> 3) * 2 + (kk & 1);
                q[0] = (u16)(bits & 0xffffu); q[64] = (u16)(bits >> 16);
            } else kvhalf = bits & 0xffffu;
        }
        cons_sync();
        if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
        uint4 x = make_uint4(0, 0, 0, 0), y = make_uint4(0, 0, 0, 0);
        if (g < 2) {
            const uint4* p = reinterpret_cast<const uint4*>(qs + g * 64 + t * 16);
            x = p[0]; y = p[1];
        }
        bq[0][0] = x.x; bq[0][1] = x.y; bq[1][0] = x.z; bq[1][1] = x.w;
        bq[2][0] = y.x; bq[2][1] = y.y; bq[3][0] = y.z; bq[3][1] = y.w;
    }
#else
    {
        const int4 e = tl[0];
        att_load_q(bq, qbuf, e.x & 255, (e.x >> 8) & 255, g, t);        // requested first: its trip to L2 overlaps the copies below
    }
    // Tiles requested before the barrier: where one holds the current position of its sequence, that row (written
    // by other CTAs during QKV) is copied into its place now, 16 bytes per thread, once the tile itself has landed.
    {
        u32 n = c.kvn;
        bool any = false;
#pragma unroll 1
        for (int k = 0; k < ntl && n != c.kvn + V_KVST; k++) {
            const int4 e = tl[k];
            if (e.z == 0) continue;
            if (e.x & TL_PATCH) {
                const u32 stage = n % V_KVST;
                wait_mbar(c, kv_bar(stage), (n / V_KVST) & 1u, 0x500u);
                if (c.tid < 16 && !c.dead) {
                    const int b = e.x & 255, h = (e.x >> 8) & 255, tp = s_pos[b];
                    const u16* src = ((c.tid & 8) ? vals : keys) + ((size_t)(b * V_L + l) * V_TMAX + tp) * V_D + (size_t)h * V_E + (c.tid & 7) * 8;
                    cp16(smem + V_SM_KV + stage * KV_STAGE_BYTES + ((c.tid & 8) ? KV_TILE_BYTES : 0) + kv_off(tp - e.y, c.tid & 7), src);
                }
                any = true;
            }
            n++;
        }
        if (any) { cp_wait(); cons_sync(); }
    }
#endif
    TRACE(44);

    float m = -3.0e38f, den = 0.f, o[V_E / 16][4];   // o[mt]: dims mt*16 + g (regs 0+1) and mt*16 + g + 8 (regs 2+3), lanes t == 0
    int item = 0;                                    // items finished by this CTA in this phase
#pragma unroll
    for (int mt = 0; mt < V_E / 16; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[mt][i] = 0.f;
#pragma unroll 1
    for (int k = 0; k < ntl; k++) {
        const int4 e = tl[k];
        const bool last = (e.x & TL_LAST) != 0;
        const int cnt = e.z;
#if !V_FUSE_X2
        if (last && k + 1 < ntl) {
            const int4 en = tl[k + 1];                  // the next item's query is requested now and used after this tile
            att_load_q(bqn, qbuf, en.x & 255, (en.x >> 8) & 255, g, t);
        }
#endif
        if (cnt > 0) {
            const u32 stage = c.kvn % V_KVST;
            wait_mbar(c, kv_bar(stage), (c.kvn / V_KVST) & 1u, 0x500u);
            TRACE(45);
            const unsigned char* kt = smem + V_SM_KV + stage * KV_STAGE_BYTES;
            const unsigned char* vt = kt + KV_TILE_BYTES;
#if V_FUSE_X2
            if (e.x & TL_PATCH) {
                // the row of the current position (the tile may have been fetched before the row reached the cache)
                if (c.tid >= V_E && c.tid < 3 * V_E) {
                    const int part = c.tid / V_E, el = c.tid - part * V_E, r = s_pos[e.x & 255] - e.y;
                    *reinterpret_cast<u16*>(smem + V_SM_KV + stage * KV_STAGE_BYTES + (part == 2 ? KV_TILE_BYTES : 0) + kv_off(r, el >> 3) + (el & 7) * 2) = (u16)kvhalf;
                }
                cons_sync();
            }
#endif
            const int p0 = c.warp * 16;                                 // this warp's positions of the tile
            if (p0 < cnt && !c.dead) {
                // scores of 16 positions: rows g and g + 8 of the tile slice, in the lanes with t == 0
                float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int kq = 0; kq < V_E / 16; kq++) {
                    u32 a[4];
                    ldsm4(a, kt + kv_off(p0 + (c.lane & 15), kq * 2 + (c.lane >> 4)));
                    mma_r(sacc, a, bq[kq][0], bq[kq][1]);
                }
                float s0 = sacc[0] + sacc[1], s1 = sacc[2] + sacc[3];
                if (!V_SCALE_IS_POW2) { s0 = s0 / V_SCALE; s1 = s1 / V_SCALE; }
                if (t != 0 || p0 + g >= cnt) s0 = -3.0e38f;
                if (t != 0 || p0 + g + 8 >= cnt) s1 = -3.0e38f;
                // the warp's maximum in one instruction: floats compare like integers once the negative ones are flipped
                int km = __float_as_int(fmaxf(s0, s1));
                km = __reduce_max_sync(0xffffffffu, km >= 0 ? km : km ^ 0x7fffffff);
                const float mx = __int_as_float(km >= 0 ? km : km ^ 0x7fffffff);
                const float mn = fmaxf(m, mx);
                const float corr = fast_exp(m - mn);
                const float pa = (s0 > -1.0e38f) ? fast_exp(s0 - mn) : 0.f, pb = (s1 > -1.0e38f) ? fast_exp(s1 - mn) : 0.f;
                den = den * corr + (pa + pb);                           // per lane: summed over the warp when the item ends
                m = mn;
#pragma unroll
                for (int mt = 0; mt < V_E / 16; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) o[mt][i] *= corr;
                // weights as the B operand: lane (g, t) holds positions 2t, 2t+1 (b0) and 2t+8, 2t+9 (b1); the weight
                // of position r < 8 is `pa` of lane 4r, that of position r + 8 is `pb` of lane 4r
                const float w00 = __shfl_sync(0xffffffffu, pa, 8 * t), w01 = __shfl_sync(0xffffffffu, pa, 8 * t + 4);
                const float w10 = __shfl_sync(0xffffffffu, pb, 8 * t), w11 = __shfl_sync(0xffffffffu, pb, 8 * t + 4);
                u32 b0 = pack_h2(w00, w01), b1 = pack_h2(w10, w11);
                if (g == 1) { b0 = pack_h2(w00 - h_lo(b0), w01 - h_hi(b0)); b1 = pack_h2(w10 - h_lo(b1), w11 - h_hi(b1)); }
                if (g > 1) { b0 = 0; b1 = 0; }
#pragma unroll
                for (int mt = 0; mt < V_E / 16; mt++) {
                    u32 a[4];
                    const int j = c.lane >> 3;
                    ldsm4t(a, vt + kv_off(p0 + (c.lane & 7) + ((j >> 1) ? 8 : 0), mt * 2 + (j & 1)));
                    mma_r(o[mt], a, b0, b1);
                }
            }
            TRACE(46);
        }
        // the warps' partial results of an item meet in shared memory; consecutive items use alternate buffers, so
        // that a warp that is already done with the next item does not overwrite what the merge is still reading
        float* ms = reinterpret_cast<float*>(smem + V_SM_MISC + MISC_ATT) + (item & 1) * (NW * (V_E + 2));
        if (last) {
            float* w = ms + c.warp * (V_E + 2);
#pragma unroll
            for (int x = 16; x; x >>= 1) den += __shfl_xor_sync(0xffffffffu, den, x);
            if (c.lane == 0) { w[0] = m; w[1] = den; }
            if (t == 0) {
#pragma unroll
                for (int mt = 0; mt < V_E / 16; mt++) { w[2 + mt * 16 + g] = o[mt][0] + o[mt][1]; w[2 + mt * 16 + g + 8] = o[mt][2] + o[mt][3]; }
            }
        }
        if (cnt > 0) {
            // this warp is done with the stage: the producer thread refills it when all eight are
            __syncwarp();
            if (c.lane == 0) mbar_arrive(kv_empty_bar(c.kvn % V_KVST));
            c.kvn++;
        }
        if (last) {
#if V_FUSE_PROJ
            // the operand of the item's projection: four fold tiles (the head's 64 outputs) with one live row
            if (c.tid >= 64 && c.tid < 64 + FUSE_US * 32) {
                const int i = c.tid - 64;
                *reinterpret_cast<uint4*>(smem + V_SM_GACT + (i >> 5) * ATILE + (i & 31) * 16) = make_uint4(0, 0, 0, 0);
            }
#endif
            cons_sync();                               // the warps' partial results of the item are in shared memory
            if (c.tid < V_E) {
                float M = -3.0e38f;
#pragma unroll
                for (int w = 0; w < NW; w++) M = fmaxf(M, ms[w * (V_E + 2)]);
                float num = 0.f, dd = 0.f;
#pragma unroll
                for (int w = 0; w < NW; w++) {
                    const float sc = fast_exp(ms[w * (V_E + 2)] - M);
                    dd += ms[w * (V_E + 2) + 1] * sc;
                    num += ms[w * (V_E + 2) + 2 + c.tid] * sc;
                }
#if V_FUSE_X
                // the item's outputs for the other CTAs of its head (a sequence that has not started attends to nothing)
                x_put(xo + ((size_t)((e.x >> 8) & 255) * V_B + (e.x & 255)) * V_E + c.tid, dd > 0.f ? __fdividef(num, dd) : 0.f, xphase);
#elif V_FUSE_PROJ
                act_store1(smem + V_SM_GACT, e.x & 255, c.tid, dd > 0.f ? __fdividef(num, dd) : 0.f);      // a sequence that has not started attends to nothing
#else
#if V_FUSE_X3
                u64* out = reinterpret_cast<u64*>(part) + (size_t)e.w * PART_STRIDE;
                x_put(out + 2 + c.tid, num, xphase);
                if (c.tid == 0) { x_put(out, M, xphase); x_put(out + 1, dd, xphase); }
#else
                float* out = part + (size_t)e.w * PART_STRIDE;
                out[2 + c.tid] = num;
                if (c.tid == 0) { out[0] = M; out[1] = dd; }
#endif
#endif
            }
#if V_FUSE_X
            {
                const int xb = e.x & 255, xh = (e.x >> 8) & 255;
                TRACE(48);
                // the outputs of all V_B sequences for this head as the operand of the projection (this CTA's own come
                // back the same way): every thread polls the pairs it converts
                {
                    constexpr int XN = (V_B * V_E + NCONS - 1) / NCONS;      // pairs per thread, requested together in every round
                    u64 got[XN];
                    const u64 t0 = now_ns();
                    u32 spins = 0;
                    for (;;) {
                        bool all = true;
#pragma unroll
                        for (int j = 0; j < XN; j++) {
                            const int i = c.tid + j * NCONS;
                            got[j] = i < V_B * V_E ? x_peek(xo + (size_t)xh * V_B * V_E + i) : ((u64)xphase << 32);
                        }
#pragma unroll
                        for (int j = 0; j < XN; j++) all = all && (u32)(got[j] >> 32) == xphase;
                        if (all || c.dead) break;
                        if ((++spins & 63u) == 0) {
                            if (ld_relaxed(c.bar + BAR_ABORT)) { c.dead = true; break; }
                            if (now_ns() - t0 > WAIT_NS) { give_up(c.bar, BAR_WHERE_HEAD, c.cta); c.dead = true; break; }
                        }
                    }
#pragma unroll
                    for (int j = 0; j < XN; j++) {
                        const int i = c.tid + j * NCONS;
                        if (i < V_B * V_E) act_store1(smem + V_SM_GACT, i / V_E, i % V_E, c.dead ? 0.f : __uint_as_float((u32)got[j]));
                    }
                }
                cons_sync();
                if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
                ctx_set(c, proj_head_x(ctx_state(c), c.bar, c.cta, z1, (xb * JT_D) / V_B, ((xb + 1) * JT_D) / V_B));
                cons_sync();                           // every warp has read the operand before the next item clears it
            }
#elif V_FUSE_PROJ
            cons_sync();
            TRACE(48);
            ctx_set(c, proj_head(ctx_state(c), c.bar, c.cta, z1, e.x & 255));
            cons_sync();                               // every warp has read the operand before the next item clears it
#endif
            item++;
#pragma unroll
            for (int kq = 0; kq < V_E / 16; kq++) { bq[kq][0] = bqn[kq][0]; bq[kq][1] = bqn[kq][1]; }
            m = -3.0e38f; den = 0.f;
#pragma unroll
            for (int mt = 0; mt < V_E / 16; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) o[mt][i] = 0.f;
            TRACE(47);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// logits: this CTA's vocabulary tiles over the whole fold, in groups of 16 (stream order inside a group: fold tile
// major); warp w owns the tiles w and w + 8 of the group. Stores the logits and keeps, per sequence, the best
// (value, lowest index) this lane has seen.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void logits_phase(Ctx& c, const Plan& p, const unsigned char* act, float* __restrict__ logit, u64 (&best)[2]) {
    const int g = c.lane >> 2, t = c.lane & 3;
    const unsigned char* actl = act + c.lane * 16;
#pragma unroll 1
    for (int j = 0; j < p.log_nj; j += 2 * NW) {
        const int width = min(2 * NW, p.log_nj - j);
        const int rpc = CH / width;
        const bool own0 = c.warp < width, own1 = c.warp + NW < width;
        float a0[4] = {0.f, 0.f, 0.f, 0.f}, l0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f}, l1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int r0 = 0; r0 < KT_D; r0 += rpc) {
            const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
            wait_mbar(c, full_bar(slot), use & 1u, 0x300u);
            const unsigned char* tiles = smem + V_SM_RING + slot * SLOT_BYTES + c.lane * 16 + c.warp * FRAG_BYTES;
            const int nr = c.dead ? 0 : min(rpc, KT_D - r0);
            if (own0) {
#pragma unroll 2
                for (int r = 0; r < nr; r++) {
                    const uint4 b = lds16(actl + (r0 + r) * ATILE);
                    const unsigned char* tp = tiles + (r * width) * FRAG_BYTES;
                    mma_hl(a0, l0, lds16(tp), b);
                    if (own1) mma_hl(a1, l1, lds16(tp + NW * FRAG_BYTES), b);
                }
            }
            __syncwarp();
            if (c.lane == 0) mbar_arrive(empty_bar(slot));
            c.chunk++;
        }
#pragma unroll
        for (int tw = 0; tw < 2; tw++) {
            if (!(tw ? own1 : own0)) continue;
            const int jt = p.log_j0 + j + c.warp + tw * NW;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int jx = jt * 16 + g + ((i & 2) ? 8 : 0), b = t * 2 + (i & 1);
                const float v = tw ? a1[i] + l1[i] : a0[i] + l0[i];
                if (b < V_B && jx < V_N) {
                    logit[(size_t)b * V_N + jx] = v;
                    const u64 key = best_key(v, (u32)jx);
                    if (key > best[i & 1]) best[i & 1] = key;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// the step
// ---------------------------------------------------------------------------------------------
struct Args {
    const int* x; const int* t;
    const u16 *wte, *wpe, *ln1w, *ln1b, *qkvb, *ob, *ln2w, *ln2b, *fcb, *pb, *lnfw, *lnfb;
    u16 *keys, *vals;
    int* x_out; int* t_out;
    const int* prompt; const int* plen;        // optional: tokens fed while t + 1 < plen[b] (V_PLEN > 0)
    const int* row_seq;                         // (not used by this kernel text: rows are sequences)
    float* S; u32* bar; u64* TS;
    const unsigned char* WP; const int* PT;
    const unsigned char* TM;                    // TMA descriptors of the K/V cache
    int nsteps;                                 // decode steps in this launch (the kernel feeds itself between them)
};

#if V_TIMING
// thread 0 of CTA V_TIMING-1 sums clock64 deltas per site in shared memory and adds them to TS at the end
#define TICK(k) do { if (c.cta == V_TIMING - 1 && c.tid == 0) { const long long now_ = clock64(); ts_[k] += now_ - tlast_; tlast_ = now_; } } while (0)
#else
#define TICK(k) do { } while (0)
#endif

__device__ __forceinline__ void step_body(const Args& a) {
    Ctx c;
    c.bar = a.bar; c.chunk = 0; c.dead = false; c.kvi = 0; c.kvn = 0; c.seq = 0;
    c.cta = blockIdx.x; c.ncta = gridDim.x; c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
#if V_TIMING
    __shared__ long long ts_[16];
    if (threadIdx.x == 0) { for (int i = 0; i < 16; i++) ts_[i] = 0; trace_on = 0; }
    if (threadIdx.x <= V_NW + 1) trace_n[threadIdx.x] = 0;
    long long tlast_ = clock64();
    const u64 t_begin_ = now_ns();
#endif

    // A launch that follows one that gave up does nothing (the abort flag stays until the host clears it). Positions
    // and tokens outside their ranges would index outside the caches and tables: refuse the step. Every CTA sees the
    // same values and takes the same branch, before any write. A negative position marks a sequence that has not
    // started yet: its row is carried along but reads and writes no cache.
    int* s_pos = reinterpret_cast<int*>(smem + V_SM_MISC + MISC_POS);
    {
        int bad = 0;
        if (c.tid < V_B) {
            const int tb = __ldcg(a.t + c.tid * V_TSTRIDE), xb = __ldcg(a.x + c.tid);
            bad = (tb >= V_TMAX) | (tb >= V_CPOS) | (xb < 0) | (xb >= V_N);
            s_pos[c.tid] = tb;
        }
        if (c.tid == 32 && ld_relaxed(a.bar + BAR_ABORT)) bad = 2;
        const int any = __syncthreads_or(bad);
        if (any) {
            if (c.cta == 0 && c.tid == 0) atomicCAS(a.bar + BAR_STATUS, 0u, 0x900u);      // (an earlier failure keeps its own code)
            return;
        }
    }
    const int nsteps = max(a.nsteps, 1);
    int* flag = reinterpret_cast<int*>(smem + V_SM_MISC + MISC_FLAG);
    volatile int* stop = reinterpret_cast<volatile int*>(smem + V_SM_MISC + MISC_STOP);
    if (c.tid == 0) {
        *stop = 0;
        if (c.cta == 0) asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(a.bar + BAR_STEP), "r"(0u) : "memory");   // nobody reads it before the first barrier
        for (int s = 0; s < V_NSLOT; s++) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), NW); }
        for (int s = 0; s < V_KVST; s++) { mbar_init(kv_bar(s), 1); mbar_init(kv_empty_bar(s), NW); }
        *reinterpret_cast<volatile u32*>(smem + V_SM_MISC + MISC_ATTSEQ) = 0;
        *reinterpret_cast<volatile int*>(smem + V_SM_MISC + MISC_NTL) = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // K/V stages and operand tiles start as zero: rows of the batch tile beyond the batch stay zero for the whole
    // launch, and staged rows past the end of a chunk only ever meet a weight of zero
#pragma unroll 1
    for (int i = c.tid; i < (V_SM_RED - V_SM_KV) / 16; i += NTHREADS) reinterpret_cast<uint4*>(smem + V_SM_KV)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

    const int* P = a.PT + c.cta * PT_STRIDE;
    if (c.warp >= NW) {
        if (c.lane == 0) {
            if (c.warp == NW) producer_weights(a.bar, P, a.WP, c.cta, c.ncta, nsteps);
            else producer_kv(a.bar, a.TM, c.cta, c.ncta, nsteps);
        }
        return;
    }
    const Plan p = load_plan(P);

    c.gen = 0;      // the barrier counter is zero at launch: the last CTA of every step clears it
    unsigned char* act = smem + V_SM_ACT;
    unsigned char* gact = smem + V_SM_GACT;
    float* red = reinterpret_cast<float*>(smem + V_SM_RED);
    const u16* tile_bias = reinterpret_cast<const u16*>(smem + V_SM_PRM + PRM_TILE);
    u64* wbest = reinterpret_cast<u64*>(smem + V_SM_MISC + MISC_BEST);
    zacc* Z = reinterpret_cast<zacc*>(a.S + V_OFF_Z);
    u32* qbuf = reinterpret_cast<u32*>(a.S + V_OFF_Q);
    float* part = a.S + V_OFF_PART;
    float* logit = a.S + V_OFF_LOGIT;
    u64* gbest = reinterpret_cast<u64*>(a.S + V_OFF_BEST);
    const int gtid = c.cta * NCONS + c.tid, gthreads = c.ncta * NCONS;
    const size_t ZS = (size_t)V_B * V_D;

#pragma unroll 1
  for (int step = 0; step < nsteps; step++) {
    if (step > 0) {
        // positions as the previous step of this launch left them (published before the step flag)
        if (c.tid < V_B) s_pos[c.tid] = __ldcg(a.t + c.tid * V_TSTRIDE);
        cons_sync();
    }
#if V_FUSE_X || V_FUSE_X2
    if (step == 0) {
        // the tags of the exchange buffers (a launch counts its attention phases from one; read after the next barrier)
#pragma unroll 1
        for (int i = gtid; i < ((V_FUSE_X ? 1 : 0) + (V_FUSE_X2 ? 3 : 0)) * V_H * V_B * V_E; i += gthreads) reinterpret_cast<u64*>(a.S + V_OFF_X)[i] = 0ull;
#if V_FUSE_X3
#pragma unroll 1
        for (int i = gtid; i < ATT_ITEMS * PART_STRIDE; i += gthreads) reinterpret_cast<u64*>(part)[i] = 0ull;
#endif
    }
#endif
    // Q1: z0 = wte[x] + wpe[t]; the vector the first projection is combined into starts at zero
#pragma unroll 1
    for (int i = gtid; i < V_B * V_D; i += gthreads) {
        const int b = i / V_D, d = i - b * V_D;
        Z[i] = to_acc(h2f(a.wte[(size_t)__ldcg(a.x + b) * V_D + d]) + h2f(a.wpe[(size_t)max(s_pos[b], 0) * V_D + d]));
        Z[ZS + i] = 0;
    }
    TICK(0);
    phase_end(c);
    fetch_params(c, a.ln1w, a.ln1b, a.ob, a.qkvb + p.qkv_j0 * 16, p.qkv_nj);
    if (c.tid == 0) build_tile_list(c.cta, c.ncta, s_pos);               // read after the barrier's block-wide sync
    phase_wait(c);
    TICK(1);

#pragma unroll 1
    for (int l = 0; l < V_L; l++) {
        zacc* zin = Z + (size_t)((2 * l) % 3) * ZS;          // layer input
        zacc* z1 = Z + (size_t)((2 * l + 1) % 3) * ZS;
        zacc* z2 = Z + (size_t)((2 * l + 2) % 3) * ZS;
#if V_TIMING
        if (c.tid == 0) trace_on = (c.cta == V_TIMING - 1) && (l == V_L / 2) && (step == 0);
#endif
        // ---- LN1 + QKV + K/V emit
        TRACE(1);
        if (c.tid == 0) {                                       // the producer thread may request this layer's K/V tiles
            volatile u32* seq = reinterpret_cast<volatile u32*>(smem + V_SM_MISC + MISC_ATTSEQ);
            __threadfence_block();                              // the tile list of this step is complete
            *seq = *seq + 1;
        }
#pragma unroll 1
        for (int i = gtid; i < V_B * V_D; i += gthreads) z2[i] = 0;      // the MLP adds into it two barriers later
        ln_to_act(c.cta, c.ncta, zin, z1);                             // starts z1 = z + ob
        TRACE(10);
        if (p.qkv_nj) {
            ctx_set(c, gemm_whole_fold(ctx_state(c), c.bar, c.cta, p.qkv_nj, p.rpc_qkv));
            TRACE(51);
            cons_sync();
            TRACE(52);
#pragma unroll 1
            for (int o = c.tid; o < p.qkv_nj * 128; o += NCONS) {
                const int r = o & 127, ln = r >> 2, i = r & 3;
                const int j_in = (ln >> 2) + ((i & 2) ? 8 : 0), b = (ln & 3) * 2 + (i & 1);
                const float v = whole_fold_sum(red, o) + h2f(tile_bias[(o >> 7) * 16 + j_in]);
                if (b < V_B) {
                    // q to scratch, K and V rounded to fp16 into the cache at t
                    const int jx = (p.qkv_j0 + (o >> 7)) * 16 + j_in;
#if V_FUSE_X2
                    // query, K and V of the current position as tagged values for the CTA that holds the attention item
                    // (it does not wait at a grid barrier for them); K and V also go to the cache, for the steps to come
                    const int prt = jx / V_D, jd = jx - prt * V_D, hh = jd / V_E, el = jd - hh * V_E;
                    u64* dst = reinterpret_cast<u64*>(a.S + V_OFF_X) + (size_t)((V_FUSE_X ? 1 : 0) + prt) * V_H * V_B * V_E + ((size_t)hh * V_B + b) * V_E + el;
                    if (prt == 0) {
                        const float vs = V_SCALE_IS_POW2 ? v * (1.0f / V_SCALE) : v;
                        const u16 hi = f2h(vs);
                        x_put(dst, __uint_as_float((u32)hi | ((u32)f2h(vs - h2f(hi)) << 16)), (u32)(step * V_L + l + 1));
                    } else {
                        const u16 hv = f2h(v);
                        if (s_pos[b] >= 0) (prt == 1 ? a.keys : a.vals)[((size_t)(b * V_L + l) * V_TMAX + s_pos[b]) * V_D + jd] = hv;
                        x_put(dst, __uint_as_float((u32)hv), (u32)(step * V_L + l + 1));
                    }
#else
                    if (jx < V_D) q_store(reinterpret_cast<u16*>(qbuf), b, jx, v);
                    else if (s_pos[b] >= 0) {
                        const size_t at = ((size_t)(b * V_L + l) * V_TMAX + s_pos[b]) * V_D + (jx % V_D);
                        if (jx < 2 * V_D) a.keys[at] = f2h(v); else a.vals[at] = f2h(v);
                    }
#endif
                }
            }
        }
        TRACE(20);
        TICK(2);
#if V_FUSE_X2
        cons_sync();                        // (the partial sums in shared memory have been read: the query is staged there next)
        TRACE(30);
#else
        phase_end(c);
        TRACE(30);
        phase_wait(c);
#endif
        TICK(3);

        // ---- attention
        TRACE(2);
        attention_phase(c, a.keys, a.vals, qbuf, part, z1, l, s_pos, (u32)(step * V_L + l + 1), reinterpret_cast<u64*>(a.S + V_OFF_X));
        TRACE(21);
        TICK(4);
#if !V_FUSE_X3
        phase_end(c);
        fetch_params(c, a.ln2w + (size_t)l * V_D, a.ln2b + (size_t)l * V_D, a.pb + (size_t)l * V_D,
                     a.fcb + (size_t)l * V_F + p.fc_j0 * 16, p.fc_nj);
        TRACE(31);
        phase_wait(c);
#endif
        TICK(5);

#if !V_FUSE_PROJ
        // ---- attention projection + residual (V_FUSE_X3: no barrier before it, the partial results of the attention items
        // are polled as tagged values)
        TRACE(3);
        if (p.proj_nj) {
            merge_to_act(c, part, p.proj_k0, p.proj_nk, act, (u32)(step * V_L + l + 1));
            TRACE(12);
            ctx_set(c, gemm_fold_slice(ctx_state(c), c.bar, c.cta, p.proj_nj, p.proj_nk, p.upc_proj, act, z1 + p.proj_j0 * 16));
        }
        TRACE(22);
        TICK(6);
        phase_end(c);
#if V_FUSE_X3
        fetch_params(c, a.ln2w + (size_t)l * V_D, a.ln2b + (size_t)l * V_D, a.pb + (size_t)l * V_D,
                     a.fcb + (size_t)l * V_F + p.fc_j0 * 16, p.fc_nj);
#endif
        TRACE(32);
        phase_wait(c);
        TICK(7);

#endif
        // ---- LN2 + FC + GELU + MLP projection + residual
        TRACE(4);
#pragma unroll 1
        for (int i = gtid; i < V_B * V_D; i += gthreads) zin[i] = 0;     // the next layer's projection adds into it
        ln_to_act(c.cta, c.ncta, z1, z2);                              // starts z2 = z1 + pb
        TRACE(13);
        if (p.fc_nj) {
            ctx_set(c, gemm_whole_fold(ctx_state(c), c.bar, c.cta, p.fc_nj, p.rpc_fc));
            TRACE(51);
            cons_sync();
            TRACE(52);
#pragma unroll 1
            for (int o = c.tid; o < p.fc_nj * 128; o += NCONS) {
                const int r = o & 127, ln = r >> 2, i = r & 3;
                const int j_in = (ln >> 2) + ((i & 2) ? 8 : 0), b = (ln & 3) * 2 + (i & 1);
                const float v = whole_fold_sum(red, o) + h2f(tile_bias[(o >> 7) * 16 + j_in]);
                // g = gelu(u) -> operand tiles of the MLP projection: fold index = tile * 16 + j_in
                if (b < V_B) act_store1(gact, b, (o >> 7) * 16 + j_in, gelu_tanh(v));
            }
            cons_sync();
            TRACE(23);
            ctx_set(c, gemm_fold_slice(ctx_state(c), c.bar, c.cta, JT_D, p.fc_nj, p.upc_p2, gact, z2));
        }
        TRACE(24);
        TICK(8);
        phase_end(c);
        if (l + 1 < V_L)
            fetch_params(c, a.ln1w + (size_t)(l + 1) * V_D, a.ln1b + (size_t)(l + 1) * V_D, a.ob + (size_t)(l + 1) * V_D,
                         a.qkvb + (size_t)(l + 1) * 3 * V_D + p.qkv_j0 * 16, p.qkv_nj);
        else
            fetch_params(c, a.lnfw, a.lnfb, (const u16*)0, (const u16*)0, 0);
        TRACE(34);
        phase_wait(c);
        TICK(9);
    }

    // ---- LN_f + logits + argmax
    {
#if V_TIMING
        if (c.tid == 0) trace_on = 0;
#endif
        zacc* zfin = Z + (size_t)((2 * V_L) % 3) * ZS;
        ln_to_act(c.cta, c.ncta, zfin, (zacc*)0);
        u64 best[2] = {0ull, 0ull};
        logits_phase(c, p, act, logit, best);
        // argmax: per row the max over the lanes that hold it (equal lane & 3), the warps, the CTAs
#pragma unroll
        for (int q = 0; q < 2; q++) {
            u64 k = best[q];
#pragma unroll
            for (int m = 4; m <= 16; m <<= 1) {
                const u64 o = __shfl_xor_sync(0xffffffffu, k, m);
                if (o > k) k = o;
            }
            if ((c.lane >> 2) == 0) wbest[((c.lane & 3) * 2 + q) * NW + c.warp] = k;
        }
        cons_sync();
        if (c.tid < V_B) {
            u64 k = 0;
#pragma unroll
            for (int w = 0; w < NW; w++) if (wbest[c.tid * NW + w] > k) k = wbest[c.tid * NW + w];
            if (k) atomicMax(gbest + c.tid, k);
        }
    }
    TICK(10);

    // ---- the last CTA to arrive publishes next, feeds it (or the next prompt token) back into x, advances t;
    //      between the steps of one launch everybody then waits for its step flag
    const bool final_step = step + 1 == nsteps;
    cons_sync();
    if (c.tid == 0) {
        __threadfence();
        flag[0] = (atomicAdd(a.bar + BAR_DONE, 1u) == (u32)c.ncta - 1);
        __threadfence();
    }
    cons_sync();
    if (flag[0]) {
        int bad = 0;
        if (c.tid < V_B) {
            const int b = c.tid;
            const u64 k = atomicExch(gbest + b, 0ull);
            const u32 n = 0xFFFFFFFFu - (u32)(k & 0xFFFFFFFFull);
            a.S[V_OFF_NEXT + b] = (float)n;
#if V_FEEDBACK
            int nx = (int)n;
            const int tn = s_pos[b] + V_TSTEP;
#if V_PLEN
            if (tn >= 0 && tn < a.plen[b]) nx = a.prompt[(size_t)b * V_PLEN + tn];
#endif
            a.x_out[b] = (nx < 0 || nx >= V_N) ? 0 : nx;
            if (V_TSTRIDE) a.t_out[b] = tn;
            bad |= (tn >= V_TMAX) | (tn >= V_CPOS);
#endif
        }
#if V_FEEDBACK
        if (!V_TSTRIDE && c.tid == 0) a.t_out[0] = s_pos[0] + V_TSTEP;
#else
        bad = 0;
#endif
        bad = __syncthreads_count_cons(bad);
        if (c.tid == 0) {
            const bool stop_now = !final_step && (bad || !V_FEEDBACK || c.dead);        // the next step would leave the cache or the tables
            if (stop_now && bad) atomicCAS(a.bar + BAR_STATUS, 0u, 0x900u);
            atomicExch(a.bar + BAR_DONE, 0u);
            if (final_step || stop_now) atomicExch(a.bar + BAR_COUNT, 0u);     // every CTA is past its last barrier
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(a.bar + BAR_STEP), "r"(final_step ? 0u : (stop_now ? 0xFFFFFFFFu : (u32)(step + 1))) : "memory");
        }
    }
    if (!final_step) {
        if (c.tid == 0) {
            u32 v = 0;
            if (!c.dead) {
                const u64 t0 = now_ns();
                u32 spins = 0;
                while ((v = ld_acquire(a.bar + BAR_STEP)) != (u32)(step + 1) && v != 0xFFFFFFFFu) {
                    if ((++spins & 63u) == 0) {
                        if (ld_relaxed(a.bar + BAR_ABORT)) { v = 0xFFFFFFFFu; break; }
                        if (now_ns() - t0 > WAIT_NS) { give_up(a.bar, 0x400u, c.cta); v = 0xFFFFFFFFu; break; }
                    }
                }
            } else v = 0xFFFFFFFFu;
            if (v == 0xFFFFFFFFu) *stop = 1;        // read by the other consumer warps below and by the producer warp
        }
        cons_sync();
        if (*stop) break;
    }
  }
    // a launch that gave up leaves the counters as a later launch expects them: the host clears status and abort flag
    if (c.dead && c.tid == 0) *stop = 1;
    TICK(11);
#if V_TIMING
    if (c.cta == V_TIMING - 1 && c.lane == 0)
        for (int i = 0; i < TRACE_EVENTS; i++) a.TS[64 + c.warp * TRACE_EVENTS + i] = i < trace_n[c.warp] ? trace_[c.warp * TRACE_EVENTS + i] : 0ull;
    if (c.cta == V_TIMING - 1 && c.tid == 0) {
        for (int i = 0; i < 16; i++) a.TS[i] += (u64)ts_[i];
        a.TS[21] += now_ns() - t_begin_;        // nanoseconds of this CTA's launch, to convert clocks
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
#define PK_QKV 0
#define PK_PROJ 1
#define PK_FC 2
#define PK_P2 3
#define PK_LOGITS 4

// A(m = output j, k) of the five contractions
__device__ __forceinline__ u16 w_elem(const PackArgs& a, int kind, int l, int j, int k) {
    switch (kind) {
        case PK_QKV: return a.qkvw[((size_t)l * V_D + k) * (3 * V_D) + j];
        case PK_PROJ: return a.ow[((size_t)l * V_D + k) * V_D + j];
        case PK_FC: return a.fcw[((size_t)l * V_D + k) * V_F + j];
        case PK_P2: return a.pw[((size_t)l * V_F + k) * V_D + j];
        default: return j < V_N ? a.wte[(size_t)j * V_D + k] : (u16)0;
    }
}
// one 16 x 16 tile in the register order of the A operand of mma.m16n8k16: 16 bytes per lane
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
// grid: (V_L + 1) blocks per CTA of the step kernel: blockIdx.x = cta * (V_L + 1) + l; l == V_L packs the logits
__device__ void pack_body(const PackArgs& a) {
    const int cta = blockIdx.x / (V_L + 1), l = blockIdx.x % (V_L + 1);
    const int* P = a.PT + cta * PT_STRIDE;
    const Plan p = load_plan(P);
    const int wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5, lane = threadIdx.x & 31;
    unsigned char* base = a.WP + (size_t)(u32)P[PT_BASE] * FRAG_BYTES;
    if (l == V_L) {
        unsigned char* dst = base + (size_t)V_L * (u32)P[PT_LAYER] * FRAG_BYTES;
        // groups of 16 vocabulary tiles, fold tile major inside a group
        for (int i = wid; i < p.log_nj * KT_D; i += nwarp) {
            const int grp = i / (2 * NW * KT_D), width = min(2 * NW, p.log_nj - grp * 2 * NW), r = i - grp * 2 * NW * KT_D;
            pack_tile(a, dst + (size_t)i * FRAG_BYTES, PK_LOGITS, 0, p.log_j0 + grp * 2 * NW + r % width, r / width, lane);
        }
        return;
    }
    unsigned char* dst = base + (size_t)l * (u32)P[PT_LAYER] * FRAG_BYTES;
    const int n_qkv = p.qkv_nj * KT_D, n_proj = p.proj_nj * p.proj_nk, n_fc = p.fc_nj * KT_D, n_p2 = p.fc_nj * JT_D;
    for (int i = wid; i < n_qkv; i += nwarp) pack_tile(a, dst + (size_t)i * FRAG_BYTES, PK_QKV, l, p.qkv_j0 + i % p.qkv_nj, i / p.qkv_nj, lane);
    dst += (size_t)n_qkv * FRAG_BYTES;
#if V_FUSE_PROJ
    // the heads' slices of the projection (64 rows each, output tile major), one copy per layer and head behind the
    // per-CTA streams; the blocks of the first CTAs pack them
    for (int h = cta; h < V_H; h += gridDim.x / (V_L + 1)) {
        unsigned char* hd = a.WP + ((size_t)V_FUSE_BASE + (size_t)(l * V_H + h) * (JT_D * FUSE_US)) * FRAG_BYTES;
        for (int i = wid; i < JT_D * FUSE_US; i += nwarp) pack_tile(a, hd + (size_t)i * FRAG_BYTES, PK_PROJ, l, i / FUSE_US, h * FUSE_US + i % FUSE_US, lane);
    }
#else
    for (int i = wid; i < n_proj; i += nwarp) pack_tile(a, dst + (size_t)i * FRAG_BYTES, PK_PROJ, l, p.proj_j0 + i / p.proj_nk, p.proj_k0 + i % p.proj_nk, lane);
    dst += (size_t)n_proj * FRAG_BYTES;
#endif
    for (int i = wid; i < n_fc; i += nwarp) pack_tile(a, dst + (size_t)i * FRAG_BYTES, PK_FC, l, p.fc_j0 + i % p.fc_nj, i / p.fc_nj, lane);
    dst += (size_t)n_fc * FRAG_BYTES;
    for (int i = wid; i < n_p2; i += nwarp) pack_tile(a, dst + (size_t)i * FRAG_BYTES, PK_P2, l, i / p.fc_nj, p.fc_j0 + i % p.fc_nj, lane);
}
