// One persistent cooperative kernel that runs one or several decode steps, written for sm_100a (B200, 148 SMs).
//
// This text is the body that vesta_gpu_b200/lower.py places behind a block of #defines (model
// sizes, placement constants, scratch offsets) and a generated kernel signature. It compiles with
// NVRTC (no headers) and with nvcc.
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
//     tiles; sums that span CTAs are combined with fp32 atomics into a vector zeroed a phase earlier.
//   * Per layer: [LN1 + QKV + KV emit] | [attention] | [attn-proj + residual] | [LN2 + FC + GELU +
//     MLP-proj + residual], grid barriers between them; then LN_f + logits + argmax + feedback,
//     finished by the last CTA to arrive (no barrier), which also releases the next step of the launch.
//   * Attention: the K/V cache comes into shared memory as TMA tensor copies (cp.async.bulk.tensor, 128-byte
//     swizzle), requested by the producer thread stage by stage as the consumer warps release them; scores and
//     output on mma.sync via ldmatrix, online softmax in registers.
//   * From 64 sequences the logits run on tcgen05.mma tiles (128 vocabulary rows x 64 sequences) with the
//     accumulators in tensor memory; the table's rows arrive by TMA tensor copies into the weight ring.
//   * Index arithmetic on the critical path avoids run-time integer division (qdiv): two consumer warps per
//     scheduler issue an instruction every ~10 cycles, so thirty dependent instructions per division were
//     measurable (6 % of a step).
//   * The whole step is ONE loop over phases with one GEMM site, one LayerNorm site and one barrier
//     site, and the big loops are kept rolled: measured on B200, a step kernel of 100 KB of code
//     ran instruction-fetch bound (88 % instruction-cache hit rate, ~90 cycles per 128 B of code,
//     every layer re-fetching the kernel), several times slower than its memory traffic allowed.
//   * Every wait (grid barrier, mbarrier) is bounded; on expiry the kernel records where in bar[]
//     and every later wait falls through, so the launch always ends.

#define WN_MAX 4                      // widest NARROW placement (output tiles per CTA)
#define TPW V_TPW                     // output tiles a warp owns in a WIDE group (more where the batch is small:
                                      // independent accumulators hide the latency of the tensor pipe)
#define NT (V_NB <= 2 ? 4 : 2)        // NARROW: tiles of a chunk a warp loads before it starts their products
#define WG (TPW * NW)                  // output tiles per WIDE group
#define G4 (V_D / 4)                  // float4 groups per activation row
#define ALB (V_ACT_LO ? 16 : 8)        // bytes per lane of an operand tile: fp16 head (b0, b1) and, if kept, the fp16 remainder
#define ATILE (32 * ALB)              // bytes per operand tile (16 fold indices x 8 batch rows)

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
#define PT_P2_J0 12      // V_KSPLIT: the MLP projection as output tiles [j0, j0+nj) x fold tiles [k0, k0+nk)
#define PT_P2_NJ 13
#define PT_P2_K0 14
#define PT_P2_NK 15

// A step is a sequence of phases separated by grid barriers: per layer QKV, ATT, PROJ, MLP (= FC then
// P2 inside the CTA), then LOGITS. Batches above one slab (SB = 8 * V_NB rows: what the operand
// tiles in shared memory hold) repeat the contraction phases slab by slab; the weight stream of
// the phase is then read once per slab (from L2 after the first).
// V_ROWSEQ: the rows of the batch are (cache sequence, position) pairs, several rows may belong to one sequence (a dense
// pass over prompt positions: every row's K and V are written before any row attends, so a row sees the rows before it).
// The sequence of row b follows the positions in shared memory.
#define SEQ_OF(s_pos, b) (V_ROWSEQ ? (s_pos)[V_B + (b)] : (b))
#define ROW_NO_LOGITS 0x40000000              // mark in row_seq[b]: nobody reads the logits of this row
#define PH_QKV 0
#define PH_ATT 1
#define PH_PROJ 2
#define PH_FC 3
#define PH_P2 4
#define PH_LOGITS 5
// V_KSPLIT (an option): the MLP projection, which combines partial sums with fp32 atomics, is placed as two
// output tiles x a slice of the fold per CTA (a 6-way instead of a 148-way sum); it then is a phase of its own,
// and the GELU output passes through global memory.
#define PH_PER_LAYER (4 + V_KSPLIT)   // QKV, ATT, PROJ, MLP (or FC, P2)
// the contractions of phase `pl` of a layer: first..last run inside the CTA without a barrier between them
__device__ __forceinline__ void phase_kinds(int pl, int& first, int& last) {
    first = (pl == 3) ? PH_FC : (pl == 4) ? PH_P2 : pl;
    last = (first == PH_FC && !V_KSPLIT) ? PH_P2 : first;
}
#define SB (8 * V_NB)                 // rows per slab
#define NSLAB ((V_B + SB - 1) / SB)

// A stream segment is a list of groups; a group is `rows` rows of `width` tiles, cut into chunks of
// whole rows, at most V_CH tiles per chunk. NARROW segment: one group (rows = fold tiles, width =
// output tiles). WIDE segment: one group per WG output tiles (rows = the CTA's fold tiles).
// off: first tile of the segment inside the layer's part of the stream.
struct Seg { int rows, nj, off; bool wide; };

__device__ __forceinline__ Seg seg_of(const int* __restrict__ P, int kind) {
    Seg s;
    const int n_qkv = P[PT_QKV_NJ] * KT_D, n_proj = P[PT_PROJ_NJ] * P[PT_PROJ_NK], n_fc = P[PT_FC_NJ] * KT_D;
    s.wide = (kind == PH_PROJ) | (kind == PH_P2 && !V_KSPLIT) | (kind == PH_LOGITS);
    s.rows = (kind == PH_PROJ) ? P[PT_PROJ_NK] : (kind == PH_P2) ? (V_KSPLIT ? P[PT_P2_NK] : P[PT_FC_NJ]) : KT_D;
    s.nj = (kind == PH_QKV) ? P[PT_QKV_NJ] : (kind == PH_PROJ) ? P[PT_PROJ_NJ] : (kind == PH_FC) ? P[PT_FC_NJ]
         : (kind == PH_P2) ? (V_KSPLIT ? P[PT_P2_NJ] : JT_D) : (kind == PH_LOGITS) ? P[PT_LOG_NJ] : 0;
    s.off = (kind == PH_PROJ) ? n_qkv : (kind == PH_FC) ? n_qkv + n_proj : (kind == PH_P2) ? n_qkv + n_proj + n_fc : 0;
    if (s.rows == 0) s.nj = 0;
    return s;
}

// ---------------------------------------------------------------------------------------------
// shared memory
// ---------------------------------------------------------------------------------------------
#define SM_RING 0
#define SM_KV (SM_RING + V_NSLOT * V_CH * FRAG_BYTES)             // K/V tiles of the attention phase
#define SM_ACT (SM_KV + V_KVST * 2 * NW * 16 * 128)                // B operands of the current contraction
#define SM_GACT (SM_ACT + KT_D * V_NB * ATILE)                    // B operands of the MLP projection (GELU output)
#define SM_RED (SM_GACT + WN_MAX * V_NB * ATILE)                  // NARROW partial sums, one tile per warp
#define SM_PRM (SM_RED + NW * V_NB * 512)                         // LayerNorm gain, shift, residual bias, tile bias
#define SM_PRM_BYTES ((3 * V_D + WN_MAX * 16) * 2)
#define SM_MISC ((SM_PRM + SM_PRM_BYTES + 15) & ~15)
#define MISC_ATT 0                                                // 2 x NW x (V_E + 2) floats (items alternate)
#define MISC_BEST (((2 * NW * (V_E + 2) * 4) + 15) & ~15)         // SB x NW u64
#define MISC_POS (MISC_BEST + SB * NW * 8)                        // V_B ints
#define MISC_STAT ((MISC_POS + V_B * 4 * (1 + V_ROWSEQ) + 15) & ~15)  // 8 x 2 floats (after the positions and, with V_ROWSEQ, the cache sequences of the rows)
#define MISC_FLAG (MISC_STAT + 8 * 8)                             // one int
#define MISC_STOP (MISC_FLAG + 4)                                 // one int: the consumers are leaving
#define MISC_ATTSEQ (MISC_FLAG + 12)                              // one u32: attention phases the consumers have opened
#define MISC_TMEM (MISC_FLAG + 8)                                 // one u32: base address of this CTA's tensor memory (V_TC)
#define MISC_SIDE (MISC_FLAG + 16)                                // per K/V stage: the K row and the V row of the current position
#define SM_MISC_BYTES (MISC_SIDE + V_KVST * 256)
#define SM_BARS ((SM_MISC + SM_MISC_BYTES + 15) & ~15)
#define SM_TOTAL (SM_BARS + (2 * V_NSLOT + 2 * V_KVST + 4) * 8)        // + operand-loaded (three thirds) and products-done barriers of the tensor-core phases

struct Ctx {
    unsigned char* smem;
    u32* bar;          // global counters
    u32 gen;           // barrier generation x CTAs
    u32 chunk;         // stream chunks consumed so far (same value in every consumer warp and the producer)
    u32 kvi, kvn;      // K/V tiles requested / used so far (stage = count % V_KVST)
    u32 tcl, tcd;      // tensor-core logits: operand loads / accumulator tiles finished so far (barrier parities)
    int cta, ncta, tid, warp, lane;
    bool dead;         // a bounded wait expired somewhere: skip waits from now on
#if V_TIMING
    int trn; bool tron; u64* trbuf;
#endif
};
#if V_TIMING
#define TRACE_EVENTS 96
#define TRACE(id) do { if (c.tron && c.lane == 0 && c.trn < TRACE_EVENTS) c.trbuf[c.warp * TRACE_EVENTS + c.trn++] = ((u64)(id) << 48) | ((u64)clock64() & 0xFFFFFFFFFFFFull); } while (0)
#else
#define TRACE(id) do { } while (0)
#endif

__device__ __forceinline__ u32 full_bar(const Ctx& c, u32 slot) { return smem_u32(c.smem + SM_BARS) + slot * 8; }
__device__ __forceinline__ u32 empty_bar(const Ctx& c, u32 slot) { return smem_u32(c.smem + SM_BARS) + (V_NSLOT + slot) * 8; }

__device__ __forceinline__ void wait_mbar(Ctx& c, u32 mbar, u32 parity, u32 where) {
    if (c.dead || mbar_try(mbar, parity)) return;
    if (!mbar_wait_slow(c.bar, mbar, parity, where, c.cta, reinterpret_cast<const volatile int*>(c.smem + SM_MISC + MISC_STOP))) c.dead = true;
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
    cp_wait();                                 // this thread's share of the parameters (and of a first K/V tile) has landed
    cons_sync();
    if (!c.dead && ld_relaxed(c.bar + BAR_ABORT)) c.dead = true;
}

// ---- K/V tiles of the attention phase (the arithmetic is further down, at attention_phase) ----
#define ATT_MAXCH (V_NCH > V_TS ? V_NCH : V_TS)
// work items of the attention phase: V_NCH position chunks for each of the first V_TAIL_BH (sequence, head) pairs,
// V_TS chunks for each of the rest (the pairs left over after whole rounds of the grid: split so that the last
// round is a fraction of an item for every CTA instead of a whole item for some)
#define ATT_ITEMS (V_TAIL_BH * V_NCH + (V_B * V_H - V_TAIL_BH) * V_TS)
#define KV_POS (NW * 16)                         // positions per tile: sixteen per warp
#define KV_SMALL 32                              // boxes of 32, 64, 96 and 128 rows
#define KV_TILE_BYTES (KV_POS * 128)             // K (or V) rows of one tile
#define KV_STAGE_BYTES (2 * KV_TILE_BYTES)       // K rows then V rows
#define TMAP_BYTES 128                           // descriptors at TM: K, V with boxes of 32 rows, of 64, of 96, of 128; then the embedding table

#if !V_TCL
struct AttIter { int it, s, hi, b, h; };         // item index, next position, end of its chunk

// (sequence, head), chunk and chunk count of item `it`
__device__ __forceinline__ void att_item(int it, int& b, int& h, int& ch, int& nch) {
    int bh;
    if (it < V_TAIL_BH * V_NCH) { bh = it / V_NCH; ch = it - bh * V_NCH; nch = V_NCH; }
    else { const int j = it - V_TAIL_BH * V_NCH; bh = V_TAIL_BH + j / V_TS; ch = j % V_TS; nch = V_TS; }
    b = bh / V_H; h = bh - b * V_H;
}
__device__ __forceinline__ void att_load_item(AttIter& a, const int* s_pos, int ncta) {
    if (a.it < ATT_ITEMS) {
        int ch, nch;
        att_item(a.it, a.b, a.h, ch, nch);
        const int n = s_pos[a.b] + 1;
        const int cs = (nch == V_NCH) ? (max(n, 1) + V_NCH - 1) / V_NCH : (max(n, 1) + V_TS - 1) / V_TS;     // divisions by constants
        a.s = ch * cs; a.hi = min(n, (ch + 1) * cs);
    }
}
__device__ __forceinline__ bool att_valid(const AttIter& a) { return a.it < ATT_ITEMS; }
__device__ __forceinline__ bool att_has_rows(const AttIter& a) { return a.hi > a.s; }      // an empty chunk is a tile without data
__device__ __forceinline__ void att_advance(AttIter& a, const int* s_pos, int ncta) {
    a.s += KV_POS;
    if (a.s >= a.hi) { a.it += ncta; att_load_item(a, s_pos, ncta); }
}
__device__ __forceinline__ void att_begin(AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta) { a.it = cta; att_load_item(a, s_pos, ncta); }
__device__ __forceinline__ void att_advance(AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta) { att_advance(a, s_pos, ncta); }
// the item after the current one of this CTA, as (sequence, head); false when there is none
__device__ __forceinline__ bool att_peek(const AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta, int& b, int& h) {
    if (a.it + ncta >= ATT_ITEMS) return false;
    int ch, nch;
    att_item(a.it + ncta, b, h, ch, nch);
    return true;
}
#else
// With tensor-core layer contractions (64 sequences and more, one work item per (sequence, head)) the items are dealt
// by length: the sequences are ranked by context length at the start of every step (longest first; the ranks live in
// the unused mma.sync operand tiles), the items in (rank, head) order go round-robin over the CTAs, every other round
// in reverse, so that the sums of lengths per CTA stay close whatever the contexts are (the items of the last,
// partial round are the shortest); the heads of a sequence still run on neighbouring CTAs at the same time (they
// share the rows of the cache). Consumer warps and the producer thread walk the items the same way.
// Measured and not kept: ranges of a cost line per CTA (contiguous items: 23 % slower, the CTAs no longer read the
// same cache rows at the same time), and cutting the items of the last round into runs of tiles merged by the CTA
// that finishes last (no gain at 64 sequences: a run costs its fixed part again).
struct AttIter { int r, b, h, s, hi; };
__device__ __forceinline__ int* att_order(unsigned char* smem) { return reinterpret_cast<int*>(smem + SM_ACT); }
__device__ __forceinline__ bool att_valid(const AttIter& a) { return a.r >= 0; }
__device__ __forceinline__ void att_load_item(AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta) {
    // (the grid is the lowered one: the placement of the weights depends on it too)
    const int i = a.r * V_MAXGRID + (((a.r & 1) && V_ATT_SNAKE) ? V_MAXGRID - 1 - cta : cta);
    if (i >= V_B * V_H) { a.r = -1; return; }
    const int sb = i / V_H;
    a.h = i - sb * V_H; a.b = att_order(smem)[sb];
    a.s = 0; a.hi = max(s_pos[a.b] + 1, 0);
}
__device__ __forceinline__ bool att_has_rows(const AttIter& a) { return a.hi > a.s; }      // a sequence that has not started: an item without data
__device__ __forceinline__ void att_advance(AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta) {
    a.s += KV_POS;
    if (a.s >= a.hi) { a.r++; att_load_item(a, smem, s_pos, cta, ncta); }
}
__device__ __forceinline__ void att_begin(AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta) { a.r = 0; att_load_item(a, smem, s_pos, cta, ncta); }
__device__ __forceinline__ bool att_peek(const AttIter& a, unsigned char* smem, const int* s_pos, int cta, int ncta, int& b, int& h) {
    AttIter n = a;
    n.r++;
    att_load_item(n, smem, s_pos, cta, ncta);
    b = n.b; h = n.h;
    return att_valid(n);
}
#endif
__device__ __forceinline__ u32 kv_bar(const Ctx& c, u32 stage) { return smem_u32(c.smem + SM_BARS) + (2 * V_NSLOT + stage) * 8; }
__device__ __forceinline__ u32 kv_empty_bar(const Ctx& c, u32 stage) { return smem_u32(c.smem + SM_BARS) + (2 * V_NSLOT + V_KVST + 2 + stage) * 8; }

// The producer thread's part of an attention phase: once the consumer warps have finished the QKV contraction of the
// layer (att_go), it requests this CTA's K/V tiles in order, each as soon as the stage it goes to has been released
// by all consumer warps. The first V_KVST requests can precede the grid barrier that ends the QKV phase (their row
// of the current position may be stale: the consumers patch it); every later one follows a release made after it.
__device__ __forceinline__ void producer_attention(Ctx& c, int l, const int* s_pos, const unsigned char* __restrict__ TM, int ncta) {
    {
        // a counter, not a barrier: the consumers may be a whole phase ahead of this thread in a CTA without weight tiles
        const volatile u32* seq = reinterpret_cast<const volatile u32*>(c.smem + SM_MISC + MISC_ATTSEQ);
        const volatile int* stop = reinterpret_cast<const volatile int*>(c.smem + SM_MISC + MISC_STOP);
        c.tcl++;
        const u64 t0 = now_ns();
        u32 spins = 0;
        while ((int)(*seq - c.tcl) < 0) {
            __nanosleep(200);                      // this thread shares a scheduler with two consumer warps
            if (*stop) { c.dead = true; return; }
            if ((++spins & 63u) == 0) {
                if (ld_relaxed(c.bar + BAR_ABORT)) { c.dead = true; return; }
                if (now_ns() - t0 > WAIT_NS) { give_up(c.bar, 0x800u, c.cta); c.dead = true; return; }
            }
        }
        __threadfence_block();
    }
    AttIter a;
    att_begin(a, c.smem, s_pos, c.cta, ncta);
#pragma unroll 1
    while (att_valid(a) && !c.dead) {
        if (att_has_rows(a)) {
            const u32 stage = c.kvi % V_KVST;
            wait_mbar(c, kv_empty_bar(c, stage), ((c.kvi / V_KVST) & 1u) ^ 1u, 0x800u);
            if (c.dead) break;
            // the smallest box that covers what is left of the item: 32, 64, 96 or 128 rows
            const int q = min((a.hi - a.s + KV_SMALL - 1) / KV_SMALL, KV_POS / KV_SMALL) - 1;
            const u32 bar = kv_bar(c, stage), dst = smem_u32(c.smem + SM_KV + stage * KV_STAGE_BYTES);
            // rows that other CTAs wrote with ordinary stores, a stage that was read and patched with ordinary accesses
            asm volatile("fence.proxy.async.global;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect(bar, 2 * (q + 1) * KV_SMALL * 128);
            tma_rows(dst, TM + (2 * q) * TMAP_BYTES, a.h * V_E, a.s, SEQ_OF(s_pos, a.b) * V_L + l, bar);
            tma_rows(dst + KV_TILE_BYTES, TM + (2 * q + 1) * TMAP_BYTES, a.h * V_E, a.s, SEQ_OF(s_pos, a.b) * V_L + l, bar);
            c.kvi++;
        }
        att_advance(a, c.smem, s_pos, c.cta, ncta);
    }
}

// ---------------------------------------------------------------------------------------------
// producer: walks this CTA's stream, segment by segment
// ---------------------------------------------------------------------------------------------
#define TC_SLABS_P ((V_B + 63) / 64)
#if V_TCL
// Layer contractions on the tensor cores (V_TCL: 64 sequences and more). The sequences are the rows of the tcgen05
// product (operand A, M = 64 of which the first V_TCL_RB are a block of sequences: the rest of the accumulator is
// never read), V_TCL_NW output columns of the weights its N. A unit = a block of V_TCL_RB sequences x V_TCL_NW
// output columns x TCL_UK k-blocks of 64 fold indices (the whole fold of width V_D; the MLP projection, whose fold
// is V_F, has V_F / V_D units per output block, their sums combined with atomics). Small units occupy all CTAs at
// 64 sequences (QKV: 2 x 72 units), their weights (V_TCL_NW x V_D x 2 bytes, one bulk copy) are already in the ring
// when the phase starts, and in the epilogue a thread holds consecutive output columns of one sequence: K / V
// rows, GELU outputs and queries leave in 16-byte stores. Units are numbered (row block, fold part, output block)
// and every CTA takes a contiguous run, so that its units share the operand of the row block.
// The weights come from a packed copy in the shared-memory image of operand B (K-major rows of 128 bytes, 128-byte
// swizzle): per layer [QKV | attn-proj | FC | MLP-proj], per (fold part, output block) TCL_UK tiles of V_TCL_NW rows.
#define TCL_KB_D (V_D / 64)
#define TCL_KB_F (V_F / 64)
#define TCL_UK TCL_KB_D                                        // k-blocks per unit
#define TCL_UB (V_TCL_NW * 128 * TCL_UK)                       // bytes of a unit's weights
#define TCL_SPU ((TCL_UB + V_CH * FRAG_BYTES - 1) / (V_CH * FRAG_BYTES))    // ring slots per unit
#define TCL_A_KB (V_TCL_RB * 128)                              // bytes of the operand of a row block per k-block
#define TCL_GS ((TCL_UK + 2) / 3)                              // k-blocks per third of a unit's fold
#define TCL_NRB ((V_B + V_TCL_RB - 1) / V_TCL_RB)
#define TCL_W_PROJ (3 * V_D / V_TCL_NW)                        // weight blocks of a layer before the attention projection's
#define TCL_W_FC (TCL_W_PROJ + V_D / V_TCL_NW)
#define TCL_W_P2 (TCL_W_FC + V_F / V_TCL_NW)
#define TCL_W_LAYER (TCL_W_P2 + (V_D / V_TCL_NW) * (TCL_KB_F / TCL_UK))
__device__ __forceinline__ int tcl_nfb(int kind) { return kind == PH_QKV ? 3 * V_D / V_TCL_NW : kind == PH_FC ? V_F / V_TCL_NW : V_D / V_TCL_NW; }
__device__ __forceinline__ int tcl_nks(int kind) { return kind == PH_P2 ? TCL_KB_F / TCL_UK : 1; }
__device__ __forceinline__ int tcl_ktot(int kind) { return kind == PH_P2 ? TCL_KB_F : TCL_KB_D; }
__device__ __forceinline__ int tcl_units(int kind) { return TCL_NRB * tcl_nks(kind) * tcl_nfb(kind); }
__device__ __forceinline__ int tcl_first_block(int kind) { return kind == PH_QKV ? 0 : kind == PH_PROJ ? TCL_W_PROJ : kind == PH_FC ? TCL_W_FC : TCL_W_P2; }
__device__ __forceinline__ void tcl_unit(int kind, int u, int& rb, int& ks, int& fb) {
    const int per = tcl_nks(kind) * tcl_nfb(kind);
    rb = u / per;
    const int r = u - rb * per;
    ks = r / tcl_nfb(kind); fb = r - ks * tcl_nfb(kind);
}
// the run of units of CTA `cta`
__device__ __forceinline__ void tcl_run(int kind, int cta, int ncta, int& u0, int& u1) {
    const int n = tcl_units(kind);
    u0 = (int)(((long long)cta * n) / ncta); u1 = (int)(((long long)(cta + 1) * n) / ncta);
}
#endif
#define TMAP_WTE 8                               // index of the embedding table's descriptor at TM (after the eight of K and V)
// leaving early: first let the copies still in flight land (bounded), so that none writes into shared memory
// after the CTA has gone
__device__ __noinline__ void producer_drain(Ctx& c) {
    for (u32 k = c.chunk > V_NSLOT ? c.chunk - V_NSLOT : 0u; k < c.chunk; k++) {
        const u64 t0 = now_ns();
        while (!mbar_try(full_bar(c, k % V_NSLOT), (k / V_NSLOT) & 1u) && now_ns() - t0 < WAIT_NS) { }
    }
}
__device__ __noinline__ void producer(unsigned char* smem, u32* bar, const int* __restrict__ P, const unsigned char* __restrict__ WP,
                                      const unsigned char* __restrict__ TM, int cta, int ncta, int nsteps, int log_slabs) {
    Ctx c;
    c.smem = smem; c.bar = bar; c.chunk = 0; c.dead = false; c.cta = cta; c.kvi = 0; c.tcl = 0;
    const int* s_pos = reinterpret_cast<const int*>(smem + SM_MISC + MISC_POS);
    const unsigned char* base = WP + (size_t)(u32)P[PT_BASE] * FRAG_BYTES;
#pragma unroll 1
    for (int ph = 0; ph < nsteps * (V_L * PH_PER_LAYER + 1); ph++) {          // every step reads the same stream again
        const int l = (ph % (V_L * PH_PER_LAYER + 1)) / PH_PER_LAYER, pl = ph % (V_L * PH_PER_LAYER + 1);
        int first, last;
        phase_kinds(pl - l * PH_PER_LAYER, first, last);
        if (l == V_L) { first = PH_LOGITS; last = PH_LOGITS; }
        if (first == PH_ATT) {
            producer_attention(c, l, s_pos, TM, ncta);
            if (c.dead) { producer_drain(c); return; }
            continue;
        }
#if V_TC
        if (first == PH_LOGITS) {
            // 128 rows x 64 k of the embedding table per slot, by tensor copy; once per slab of 64 sequences
            const int rows = P[PT_LOG_NJ] * 16, mtiles = (rows + 127) / 128;
#pragma unroll 1
            for (int i = 0; i < log_slabs * mtiles * (V_D / 64); i++) {
                const int kb = i % (V_D / 64), mt = (i / (V_D / 64)) % mtiles;
                const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
                wait_mbar(c, empty_bar(c, slot), (use & 1u) ^ 1u, 0x200u);
                if (c.dead) { producer_drain(c); return; }
                mbar_expect(full_bar(c, slot), 128 * 128);
                asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                             :: "r"(smem_u32(smem + SM_RING) + slot * (V_CH * FRAG_BYTES)), "l"(TM + TMAP_WTE * 128), "r"(kb * 64), "r"(P[PT_LOG_J0] * 16 + mt * 128), "r"(0),
                                "r"(full_bar(c, slot)) : "memory");
                c.chunk++;
            }
            continue;
        }
#endif
#if V_TCL
        {
            // the weights of this CTA's units, one bulk copy per unit into TCL_SPU consecutive ring slots (the first
            // slot's barrier counts the bytes; the others are passed so that every slot keeps its turn)
            int u0, u1;
            tcl_run(first, cta, ncta, u0, u1);
#pragma unroll 1
            for (int u = u0; u < u1; u++) {
                int rb, ks, fb;
                tcl_unit(first, u, rb, ks, fb);
                const unsigned char* src = WP + ((size_t)l * TCL_W_LAYER + tcl_first_block(first) + (size_t)ks * tcl_nfb(first) + fb) * TCL_UB;
                const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
#pragma unroll 1
                for (u32 i = 0; i < TCL_SPU; i++) wait_mbar(c, empty_bar(c, slot + i), (use & 1u) ^ 1u, 0x200u);
                if (c.dead) { producer_drain(c); return; }
                mbar_expect(full_bar(c, slot), TCL_UB);
                bulk_g2s(smem_u32(smem + SM_RING) + slot * (V_CH * FRAG_BYTES), src, TCL_UB, full_bar(c, slot));
#pragma unroll 1
                for (u32 i = 1; i < TCL_SPU; i++) mbar_arrive(full_bar(c, slot + i));
                c.chunk += TCL_SPU;
            }
            continue;
        }
#endif
#pragma unroll 1
        for (int slab = 0; slab < NSLAB; slab++)
#pragma unroll 1
            for (int kind = first; kind <= last; kind++) {
                const Seg s = seg_of(P, kind);
                const unsigned char* src = base + ((size_t)l * (u32)P[PT_LAYER] + s.off) * FRAG_BYTES;
#pragma unroll 1
                for (int j = 0; j < s.nj; j += (s.wide ? WG : WN_MAX * 4)) {
                    const int width = s.wide ? min(WG, s.nj - j) : s.nj;
                    const int rpc = qdiv(V_CH, rcp_fast(width));
#pragma unroll 1
                    for (int r = 0; r < s.rows; r += rpc) {
                        const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
                        wait_mbar(c, empty_bar(c, slot), (use & 1u) ^ 1u, 0x200u);
                        if (c.dead) { producer_drain(c); return; }
                        const u32 bytes = (u32)(min(rpc, s.rows - r) * width) * FRAG_BYTES;
                        mbar_expect(full_bar(c, slot), bytes);
                        bulk_g2s(smem_u32(smem + SM_RING) + slot * (V_CH * FRAG_BYTES), src, bytes, full_bar(c, slot));
                        src += bytes;
                        c.chunk++;
                    }
                }
            }
    }
}

// ---------------------------------------------------------------------------------------------
// one group of a contraction: `rows` x `width` tiles from the stream against the operand tiles at act.
// NARROW: warp w works on output tile w % width and on every cnt-th fold tile (cnt = warps that share
// the output tile); its tiles are those with index w + k * cnt * width in the group's row-major
// order; sums in acc[0]. WIDE: warp w owns output tiles w and w + NW (where < width) over all rows;
// sums in acc[0] and acc[1].
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void gemm_group(Ctx& c, int rows, int width, bool wide, const unsigned char* act, float (&acc)[TPW][V_NB][4]) {
    float lo[TPW][V_NB][4];
#pragma unroll
    for (int t = 0; t < TPW; t++)
#pragma unroll
        for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) { acc[t][nb][i] = 0.f; lo[t][nb][i] = 0.f; }
    const float rcpw = rcp_fast(width);
    const u32 act32 = smem_u32(act);
    const int rpc = qdiv(V_CH, rcpw), per = rpc * width, total = rows * width;
    if (wide) {
        bool own[TPW];
#pragma unroll
        for (int t = 0; t < TPW; t++) own[t] = c.warp + t * NW < width;
        int row = 0;
#pragma unroll 1
        for (int base = 0; base < total; base += per) {
            const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
            wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
            TRACE(53);
            const u32 tiles = smem_u32(c.smem + SM_RING) + slot * (V_CH * FRAG_BYTES) + (u32)c.lane * 16u;
            const int nr = c.dead ? 0 : min(rpc, rows - row);
#pragma unroll 2
            for (int r = 0; r < nr; r++) {
                const u32 tp = tiles + (u32)(r * width + c.warp) * FRAG_BYTES;
                uint4 a[TPW], b[V_NB];
#pragma unroll
                for (int t = 0; t < TPW; t++) a[t] = own[t] ? lds128s(tp + t * NW * FRAG_BYTES) : make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++) b[nb] = lds_acts(act32 + (u32)(((row + r) * V_NB + nb) * 32 + c.lane) * ALB);
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                    for (int t = 0; t < TPW; t++)
                        if (own[t]) { mma16816(acc[t][nb], a[t], b[nb].x, b[nb].y); if (V_ACT_LO) mma16816(lo[t][nb], a[t], b[nb].z, b[nb].w); }
            }
            row += rpc;
            __syncwarp();
            if (c.lane == 0) mbar_arrive(empty_bar(c, slot));
            c.chunk++;
        }
    } else {
        const int wq = qdiv(c.warp, rcpw), wm = c.warp - wq * width;             // warp / width, warp % width
        const int cnt = qdiv(NW - wm + width - 1, rcpw);                         // rows advance by cnt
        const int stride = cnt * width;
        const float rcps = rcp_fast(stride);
        int f = (wq < rows) ? c.warp : 0x3fffffff;                               // next tile of this warp
        int row = wq;
#pragma unroll 1
        for (int base = 0; base < total; base += per) {
            const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
            wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
            TRACE(53);
            const u32 tiles = smem_u32(c.smem + SM_RING) + slot * (V_CH * FRAG_BYTES) - (u32)base * FRAG_BYTES + (u32)c.lane * 16u;
            const int lim = c.dead ? 0 : min(base + per, total);
            int mine = f < lim ? qdiv(lim - f + stride - 1, rcps) : 0;           // this warp's tiles in the chunk
#pragma unroll 1
            for (; mine > 0; mine -= NT, f += NT * stride, row += NT * cnt) {
                // all loads of up to NT tiles first, then their products: the loads and the first product's latency overlap
                uint4 a[NT], b[NT][V_NB];
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    if (i < mine) {
                        a[i] = lds128s(tiles + (u32)(f + i * stride) * FRAG_BYTES);
#pragma unroll
                        for (int nb = 0; nb < V_NB; nb++) b[i][nb] = lds_acts(act32 + (u32)(((row + i * cnt) * V_NB + nb) * 32 + c.lane) * ALB);
                    }
                }
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    if (i < mine) {
#pragma unroll
                        for (int nb = 0; nb < V_NB; nb++) {
                            mma16816(acc[0][nb], a[i], b[i][nb].x, b[i][nb].y);
                            if (V_ACT_LO) mma16816(lo[0][nb], a[i], b[i][nb].z, b[i][nb].w);
                        }
                    }
                }
            }
            if (mine < 0) { f += mine * stride; row += mine * cnt; }             // the last batch was not full
            __syncwarp();
            if (c.lane == 0) mbar_arrive(empty_bar(c, slot));
            c.chunk++;
        }
    }
#pragma unroll
    for (int t = 0; t < TPW; t++)
#pragma unroll
        for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[t][nb][i] += lo[t][nb][i];
}

// ---------------------------------------------------------------------------------------------
// activations -> B operand tiles in shared memory
// element (b, k): tile k/16, batch tile b/8, lane (b%8)*4 + (k%8)/2, word (k%16)/8 (+2 for the
// remainder), half k%2
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void act_store4(unsigned char* act, int b, int k, float4 v) {
    // k is a multiple of 4: two lanes of the tile, the same register index in both
    const u32 h0 = pack_h2(v.x, v.y), h1 = pack_h2(v.z, v.w);
    const int kt = k >> 4, kk = k & 15, reg = kk >> 3, t = (kk & 7) >> 1;
    u32* base = reinterpret_cast<u32*>(act + ((size_t)(kt * V_NB + (b >> 3)) * 32 + (b & 7) * 4 + t) * ALB);
    base[reg] = h0;
    base[ALB / 4 + reg] = h1;
#if V_ACT_LO
    base[2 + reg] = pack_h2(v.x - h_lo(h0), v.y - h_hi(h0));
    base[ALB / 4 + 2 + reg] = pack_h2(v.z - h_lo(h1), v.w - h_hi(h1));
#endif
}
__device__ __forceinline__ void act_store1(unsigned char* act, int b, int k, float v) {
    const u16 hi = f2h(v);
    const int kt = k >> 4, kk = k & 15, reg = kk >> 3, t = (kk & 7) >> 1, half = kk & 1;
    u16* base = reinterpret_cast<u16*>(act + ((size_t)(kt * V_NB + (b >> 3)) * 32 + (b & 7) * 4 + t) * ALB);
    base[reg * 2 + half] = hi;
#if V_ACT_LO
    base[(2 + reg) * 2 + half] = f2h(v - h2f(hi));
#endif
}

// Parameters of the next LayerNorm phase into shared memory: gain, shift, the bias added when the
// following combined vector is started (each V_D halves), and the bias of this CTA's NARROW tiles.
__device__ __forceinline__ void fetch_params(Ctx& c, const u16* gw, const u16* gb, const u16* ib, const u16* tb, int tiles) {
    u16* prm = reinterpret_cast<u16*>(c.smem + SM_PRM);
    const int per = V_D / 8;                       // 16-byte pieces per vector
#pragma unroll 1
    for (int i = c.tid; i < 3 * per; i += NCONS) {
        const int v = i / per, q = i - v * per;
        const u16* src = v == 0 ? gw : (v == 1 ? gb : ib);
        if (src) cp16(prm + v * V_D + q * 8, src + q * 8);
    }
    if (tb && c.tid < tiles * 2) cp16(prm + 3 * V_D + c.tid * 8, tb + c.tid * 8);
}

// LayerNorm of `nrows` rows of z (global, fp32, row stride V_D: one slab) into the operand tiles; gain and shift come
// from the parameter block in shared memory. One warp per row, the row held in registers: lane (u, t) loads the
// elements 2t, 2t+1, 2t+8, 2t+9 of the fold tiles u, u + 8, ... (all loads independent: one round trip to L2),
// mean and variance by two warp reductions, then the lane writes exactly the 16 bytes that thread (row, t) of the
// contraction reads from each of its tiles (head and remainder of its four elements). Rows of the slab beyond
// `nrows` are written as zeros. The same pass starts the vector the following projection is combined into:
// init[b][d] += z[b][d] + bias[d], the fold tiles dealt over the CTAs (init was zeroed a phase earlier).
#define LNI ((KT_D + 7) / 8)
__device__ __forceinline__ void ln_to_act(Ctx& c, const float* __restrict__ z, float* __restrict__ init, unsigned char* act, int nrows) {
    const u16* prm = reinterpret_cast<const u16*>(c.smem + SM_PRM);
    const int u = c.lane >> 2, t = c.lane & 3;
#pragma unroll 1
    for (int rb = c.warp; rb < SB; rb += NW) {
        unsigned char* dst = act + ((size_t)(rb >> 3) * 32 + (rb & 7) * 4 + t) * ALB;
        if (rb >= nrows) {
#pragma unroll
            for (int i = 0; i < LNI; i++) {
                const int kt = u + 8 * i;
                if (kt < KT_D) {
#if V_ACT_LO
                    *reinterpret_cast<uint4*>(dst + (size_t)kt * V_NB * ATILE) = make_uint4(0, 0, 0, 0);
#else
                    *reinterpret_cast<uint2*>(dst + (size_t)kt * V_NB * ATILE) = make_uint2(0, 0);
#endif
                }
            }
            continue;
        }
        const float* row = z + (size_t)rb * V_D + 2 * t;
        float2 v0[LNI], v1[LNI];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < LNI; i++) {
            const int kt = u + 8 * i;
            v0[i] = make_float2(0.f, 0.f); v1[i] = make_float2(0.f, 0.f);
            if (kt < KT_D) {
                v0[i] = __ldcg(reinterpret_cast<const float2*>(row + kt * 16));
                v1[i] = __ldcg(reinterpret_cast<const float2*>(row + kt * 16 + 8));
            }
        }
#pragma unroll
        for (int i = 0; i < LNI; i++) s += (v0[i].x + v0[i].y) + (v1[i].x + v1[i].y);
#pragma unroll
        for (int m = 16; m; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        const float mean = s * (1.0f / V_D);
        TRACE(40);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < LNI; i++) {
            if (u + 8 * i < KT_D) {
                const float a0 = v0[i].x - mean, a1 = v0[i].y - mean, a2 = v1[i].x - mean, a3 = v1[i].y - mean;
                q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
            }
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
        const float rs = rsqrtf(q * (1.0f / V_D) + V_EPS);
        TRACE(41);
#pragma unroll
        for (int i = 0; i < LNI; i++) {
            const int kt = u + 8 * i, k = kt * 16 + 2 * t;
            if (kt < KT_D) {
                const u32 w0 = *reinterpret_cast<const u32*>(prm + k), w1 = *reinterpret_cast<const u32*>(prm + k + 8);
                const u32 s0 = *reinterpret_cast<const u32*>(prm + V_D + k), s1 = *reinterpret_cast<const u32*>(prm + V_D + k + 8);
                const float o0 = (v0[i].x - mean) * rs * h_lo(w0) + h_lo(s0), o1 = (v0[i].y - mean) * rs * h_hi(w0) + h_hi(s0);
                const float o2 = (v1[i].x - mean) * rs * h_lo(w1) + h_lo(s1), o3 = (v1[i].y - mean) * rs * h_hi(w1) + h_hi(s1);
                uint4 out;
                out.x = pack_h2(o0, o1); out.y = pack_h2(o2, o3);
#if V_ACT_LO
                out.z = pack_h2(o0 - h_lo(out.x), o1 - h_hi(out.x)); out.w = pack_h2(o2 - h_lo(out.y), o3 - h_hi(out.y));
                *reinterpret_cast<uint4*>(dst + (size_t)kt * V_NB * ATILE) = out;
#else
                *reinterpret_cast<uint2*>(dst + (size_t)kt * V_NB * ATILE) = make_uint2(out.x, out.y);
#endif
                if (init && ((KT_D <= V_MAXGRID) ? (kt == c.cta) : ((kt % c.ncta) == c.cta))) {
                    const u32 i0 = *reinterpret_cast<const u32*>(prm + 2 * V_D + k), i1 = *reinterpret_cast<const u32*>(prm + 2 * V_D + k + 8);
                    float* o = init + (size_t)rb * V_D + k;
                    red_add(o, v0[i].x + h_lo(i0)); red_add(o + 1, v0[i].y + h_hi(i0));
                    red_add(o + 8, v1[i].x + h_lo(i1)); red_add(o + 9, v1[i].y + h_hi(i1));
                }
            }
        }
        TRACE(42);
    }
    cons_sync();
}

// Distributed LayerNorm (batches of more than two batch tiles): instead of every CTA normalising every row
// of its slab, the rows are dealt over all warps of the grid; a warp normalises its row once and writes
// it as operand tiles to global memory (actg: per slab [fold tile][batch tile][lane][16 B], the layout
// of the shared-memory operand), and starts the vector the following projection is combined into
// (init[r] = z[r] + bias, a plain store: nothing has been added to it yet). After a grid barrier every
// CTA copies the tiles of the slab it works on into shared memory.
#define LNV ((G4 + 31) / 32)
#define SLAB_TILE_BYTES (KT_D * V_NB * ATILE)
__device__ __forceinline__ void ln_rows_to_global(Ctx& c, const float* __restrict__ z, float* __restrict__ init, unsigned char* __restrict__ actg) {
    const u16* prm = reinterpret_cast<const u16*>(c.smem + SM_PRM);
#pragma unroll 1
    for (int r = c.cta * NW + c.warp; r < V_B; r += c.ncta * NW) {
        float4 v[LNV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int g = i * 32 + c.lane;
            v[i] = (g < G4) ? __ldcg(reinterpret_cast<const float4*>(z + (size_t)r * V_D) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        const float mean = s * (1.0f / V_D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            if (i * 32 + c.lane < G4) {
                const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
                q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
            }
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
        const float rs = rsqrtf(q * (1.0f / V_D) + V_EPS);
        unsigned char* tiles = actg + (size_t)(r / SB) * SLAB_TILE_BYTES;
        const int rb = r % SB;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int g = i * 32 + c.lane, d = g * 4;
            if (g < G4) {
                const uint2 w = *reinterpret_cast<const uint2*>(prm + d);
                const uint2 bb = *reinterpret_cast<const uint2*>(prm + V_D + d);
                float4 o;
                o.x = (v[i].x - mean) * rs * h_lo(w.x) + h_lo(bb.x);
                o.y = (v[i].y - mean) * rs * h_hi(w.x) + h_hi(bb.x);
                o.z = (v[i].z - mean) * rs * h_lo(w.y) + h_lo(bb.y);
                o.w = (v[i].w - mean) * rs * h_hi(w.y) + h_hi(bb.y);
                act_store4(tiles, rb, d, o);
                if (init) {
                    const uint2 ib = *reinterpret_cast<const uint2*>(prm + 2 * V_D + d);
                    *reinterpret_cast<float4*>(init + (size_t)r * V_D + d) =
                        make_float4(v[i].x + h_lo(ib.x), v[i].y + h_hi(ib.x), v[i].z + h_lo(ib.y), v[i].w + h_hi(ib.y));
                }
            }
        }
    }
}
__device__ __forceinline__ void load_tiles(Ctx& c, const unsigned char* __restrict__ tiles, unsigned char* act, int bytes) {
#pragma unroll 1
    for (int i = c.tid; i < bytes / 16; i += NCONS) cp16(act + (size_t)i * 16, tiles + (size_t)i * 16);
    cp_wait();
    cons_sync();
}
__device__ __forceinline__ void load_act_tiles(Ctx& c, const unsigned char* __restrict__ tiles, unsigned char* act) {
    load_tiles(c, tiles, act, SLAB_TILE_BYTES);
}

// Attention output for the fold range [k0*16, (k0+nk)*16) of the projection, merged from the
// per-chunk partial results (m, sum, unnormalised o[V_E]) of the attention phase, into operand
// tiles 0..nk-1.
#define PART_STRIDE (V_E + 2)
__device__ __forceinline__ void merge_to_act(Ctx& c, const float* __restrict__ part, int k0, int nk, unsigned char* act, int row0, int nrows) {
    const int cols = nk * 16;
    const float rcpk = rcp_fast(nk);
#pragma unroll 1
    for (int i = c.tid; i < nrows * cols; i += NCONS) {
        const int b = (nk <= 64) ? qdiv(i >> 4, rcpk) : i / cols, kk = i - b * cols, d = k0 * 16 + kk, h = d / V_E, e = d % V_E;
        // the chunks of (sequence, head): V_NCH of them, or V_TS for the items of the last, split round
        const int bh = (row0 + b) * V_H + h;
        const bool tail = bh >= V_TAIL_BH;
        const int nchunks = tail ? V_TS : V_NCH;
        const float* p = part + (size_t)(tail ? V_TAIL_BH * V_NCH + (bh - V_TAIL_BH) * V_TS : bh * V_NCH) * PART_STRIDE;
        // all loads first (independent, one round trip), then the arithmetic
        float mm[ATT_MAXCH], dd[ATT_MAXCH], oo[ATT_MAXCH], M = -3.0e38f;
#pragma unroll
        for (int ch = 0; ch < ATT_MAXCH; ch++) {
            mm[ch] = -3.0e38f; dd[ch] = 0.f; oo[ch] = 0.f;
            if (ch < nchunks) { mm[ch] = __ldcg(p + ch * PART_STRIDE); dd[ch] = __ldcg(p + ch * PART_STRIDE + 1); oo[ch] = __ldcg(p + ch * PART_STRIDE + 2 + e); }
        }
#pragma unroll
        for (int ch = 0; ch < ATT_MAXCH; ch++) M = fmaxf(M, mm[ch]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int ch = 0; ch < ATT_MAXCH; ch++) {
            const float w = fast_exp(mm[ch] - M);
            den += w * dd[ch];
            num += w * oo[ch];
        }
        act_store1(act, b, kk, den > 0.f ? __fdividef(num, den) : 0.f);      // a sequence that has not started attends to nothing
    }
    cons_sync();
}

// ---------------------------------------------------------------------------------------------
// attention: this CTA's work items are (sequence, head, chunk of the positions); an item is processed
// in tiles of KV_POS positions. A tile's K rows and V rows (128 B per position and head) come into shared
// memory by TMA: one thread issues two tensor copies (cp.async.bulk.tensor, box = the rows of one head that are
// left of the item, rounded up to 32, at most KV_POS) that complete on the stage's mbarrier; the
// 128-byte swizzle of the copy spreads the rows over the banks for ldmatrix. V_KVST stages are in flight.
// The first V_KVST tiles are requested before the grid barrier that ends the QKV phase; the row of the
// current position, which another CTA writes during that phase, is fetched after the barrier with ordinary
// asynchronous copies and put in its place before the tile is used.
// Arithmetic on the tensor pipe: a warp takes 16 positions of the tile. Scores: A = the K rows
// (ldmatrix, 16 positions x 16 dims per step), B = the query, its fp16 head in column 0 and its fp16
// remainder in column 1, so that column 0 + column 1 is the fp32-accurate dot product. Online softmax
// on the 16 scores (held by the lanes with lane%4 == 0). Output: A = V transposed (ldmatrix.trans,
// 16 dims x 16 positions), B = the weights, head and remainder again in columns 0 and 1.
// Result per item: (running max, sum, unnormalised o[V_E]).
// ---------------------------------------------------------------------------------------------
// B operand of the scores: the query of (b, h), head in column 0 (lanes with g == 0), remainder in column 1 (g == 1)
// in two halves: the loads (the values are not touched, so the warp does not wait for them) and, when the operand is
// needed, the conversion
__device__ __forceinline__ void att_fetch_q(float2 (&raw)[V_E / 16][2], const float* __restrict__ qbuf, int b, int h, int g, int t) {
    const float* qp = qbuf + (size_t)b * V_D + h * V_E;
#pragma unroll
    for (int kq = 0; kq < V_E / 16; kq++) {
        raw[kq][0] = make_float2(0.f, 0.f); raw[kq][1] = make_float2(0.f, 0.f);
        if (g < 2) {
            raw[kq][0] = __ldcg(reinterpret_cast<const float2*>(qp + kq * 16 + 2 * t));
            raw[kq][1] = __ldcg(reinterpret_cast<const float2*>(qp + kq * 16 + 2 * t + 8));
        }
    }
}
__device__ __forceinline__ void att_pack_q(u32 (&bq)[V_E / 16][2], const float2 (&raw)[V_E / 16][2], int g) {
    const float sc = V_SCALE_IS_POW2 ? (1.0f / V_SCALE) : 1.0f;        // exact when the divisor is a power of two
#pragma unroll
    for (int kq = 0; kq < V_E / 16; kq++) {
        bq[kq][0] = 0; bq[kq][1] = 0;
        if (g < 2) {
            const float2 a0 = raw[kq][0], a1 = raw[kq][1];
            const u32 h0 = pack_h2(a0.x * sc, a0.y * sc), h1 = pack_h2(a1.x * sc, a1.y * sc);
            bq[kq][0] = g == 0 ? h0 : pack_h2(a0.x * sc - h_lo(h0), a0.y * sc - h_hi(h0));
            bq[kq][1] = g == 0 ? h1 : pack_h2(a1.x * sc - h_lo(h1), a1.y * sc - h_hi(h1));
        }
    }
}
__device__ __forceinline__ void att_load_q(u32 (&bq)[V_E / 16][2], const float* __restrict__ qbuf, int b, int h, int g, int t) {
    float2 raw[V_E / 16][2];
    att_fetch_q(raw, qbuf, b, h, g, t);
    att_pack_q(bq, raw, g);
}

#if V_TCL
// The sequences ranked by context length, longest first (ties by index): order[rank] = sequence. Rebuilt when the
// positions of a step are known; every thread ranks its sequences against all (the positions are read as broadcasts
// from shared memory). All consumer warps; ends with a block-wide sync.
__device__ __noinline__ void att_plan(Ctx& c, const int* s_pos) {
    int* order = att_order(c.smem);
#pragma unroll 1
    for (int b = c.tid; b < V_B; b += NCONS) {
        const int n = s_pos[b];
        int rank = 0;
#pragma unroll 4
        for (int o = 0; o < V_B; o++) { const int m = s_pos[o]; rank += (m > n || (m == n && o < b)) ? 1 : 0; }
        order[rank] = b;
    }
    __threadfence_block();
    cons_sync();
}

#endif

__device__ __forceinline__ void attention_phase(Ctx& c, const u16* __restrict__ keys, const u16* __restrict__ vals, const float* __restrict__ qbuf,
                                                float* __restrict__ part, int l, const int* s_pos, const unsigned char* __restrict__ TM, unsigned char* __restrict__ og) {
    const int g = c.lane >> 2, t = c.lane & 3;
    AttIter cur, pf;
    att_begin(cur, c.smem, s_pos, c.cta, c.ncta);
    if (!att_valid(cur)) return;
    u32 bq[V_E / 16][2];                             // the query of this item
    float2 qn[V_E / 16][2];                          // the query of the next one as loaded (converted when the item starts)
#pragma unroll
    for (int kq = 0; kq < V_E / 16; kq++) { qn[kq][0] = make_float2(0.f, 0.f); qn[kq][1] = make_float2(0.f, 0.f); }
    att_load_q(bq, qbuf, cur.b, cur.h, g, t);        // requested first: its trip to L2 overlaps the walk below
    // The first V_KVST tiles may have been requested before the barrier: where one holds the current position of its
    // sequence, that row is fetched now into a side buffer (one per stage) and moved into the tile when it is used.
    unsigned char* side = c.smem + SM_MISC + MISC_SIDE;
    u32 patch = 0;
    pf = cur;
    {
        u32 n = c.kvn;
#pragma unroll 1
        while (n != c.kvn + V_KVST && att_valid(pf)) {
            if (att_has_rows(pf)) {
                const int tp = s_pos[pf.b];
                if (tp >= pf.s && tp < min(pf.hi, pf.s + KV_POS)) {
                    const u32 stage = n % V_KVST;
                    patch |= 1u << stage;
                    if (c.tid < 16) {
                        const u16* src = ((c.tid & 8) ? vals : keys) + ((size_t)(SEQ_OF(s_pos, pf.b) * V_L + l) * V_TMAX + tp) * V_D + (size_t)pf.h * V_E + (c.tid & 7) * 8;
                        cp16(side + stage * 256 + c.tid * 16, src);
                    }
                }
                n++;
            }
            att_advance(pf, c.smem, s_pos, c.cta, c.ncta);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }

    float m = -3.0e38f, den = 0.f, o[V_E / 16][4];   // o[mt]: dims mt*16 + g (regs 0+1) and mt*16 + g + 8 (regs 2+3), lanes t == 0
    int item = 0;                                    // items finished by this CTA in this phase
#pragma unroll
    for (int mt = 0; mt < V_E / 16; mt++)
#pragma unroll
        for (int i = 0; i < 4; i++) o[mt][i] = 0.f;
#pragma unroll 1
    while (att_valid(cur)) {
        if (V_B <= 16) TRACE(44);
        const bool last = cur.s + KV_POS >= cur.hi;
        if (last) {
            // the next item's query is requested now and used after this tile
            int nb_, nh_;
            if (att_peek(cur, c.smem, s_pos, c.cta, c.ncta, nb_, nh_)) att_fetch_q(qn, qbuf, nb_, nh_, g, t);
        }
        const int cnt = min(KV_POS, cur.hi - cur.s);
        if (cnt > 0) {
            const u32 stage = c.kvn % V_KVST;
            wait_mbar(c, kv_bar(c, stage), (c.kvn / V_KVST) & 1u, 0x500u);
            unsigned char* kt = c.smem + SM_KV + stage * KV_STAGE_BYTES;
            unsigned char* vt = kt + KV_TILE_BYTES;
            if (patch & (1u << stage)) {
                patch &= ~(1u << stage);
                cp_wait();                              // the thread that fetched a piece is the one that places it
                if (c.tid < 16) {
                    const int r = s_pos[cur.b] - cur.s;
                    *reinterpret_cast<uint4*>(((c.tid & 8) ? vt : kt) + kv_off(r, c.tid & 7)) = *reinterpret_cast<const uint4*>(side + stage * 256 + c.tid * 16);
                }
                cons_sync();
            }
            if (V_B <= 16) TRACE(45);
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
        }
        if (V_B <= 16) TRACE(46);
#if !V_TCL
        float* out = part + (size_t)cur.it * PART_STRIDE;
#endif
        // the warps' partial results of an item meet in shared memory; consecutive items use alternate buffers, so
        // that a warp that is already done with the next item does not overwrite what the merge is still reading
        float* ms = reinterpret_cast<float*>(c.smem + SM_MISC + MISC_ATT) + (item & 1) * (NW * (V_E + 2));
        if (last) {
            // per warp (m, den, o[V_E]) into shared memory
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
            if (c.lane == 0) mbar_arrive(kv_empty_bar(c, c.kvn % V_KVST));
            c.kvn++;
        }
        if (last) {
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
#if V_TCL
                // one item per (sequence, head): the normalised output goes straight into the operand of the projection
                // (fp16, K-major swizzled rows: k-block = head, as the head width is 64)
                const int rb = cur.b % 64;
                *reinterpret_cast<u16*>(og + ((size_t)(cur.b / 64) * TCL_KB_D + cur.h) * (64 * 128) + rb * 128 + (((c.tid >> 3) ^ (rb & 7)) << 4) + (c.tid & 7) * 2) =
                    f2h(dd > 0.f ? __fdividef(num, dd) : 0.f);
#else
                out[2 + c.tid] = num;
                if (c.tid == 0) { out[0] = M; out[1] = dd; }
#endif
            }
            // start the next item
            item++;
            att_pack_q(bq, qn, g);
            m = -3.0e38f; den = 0.f;
#pragma unroll
            for (int mt = 0; mt < V_E / 16; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) o[mt][i] = 0.f;
        }
        att_advance(cur, c.smem, s_pos, c.cta, c.ncta);
    }
    cp_wait();                                         // (the phase ends with a block-wide sync before anything else uses this memory)
}

// ---------------------------------------------------------------------------------------------
// Logits on the 5th-generation tensor cores (V_TC: batches of 64 and more, where the contraction is dense).
// D[n][b] = sum_k wte[n][k] * y[b][k] per tile of 128 vocabulary rows x 64 batch rows, accumulated in tensor
// memory by tcgen05.mma (M = 128, N = 64, K = 16 per instruction, fp16 operands, fp32 accumulators):
//   A = 128 rows of the embedding table, 64 k at a time: the table is row-major, i.e. K-major, so the TMA
//       box (64 k x 128 rows, 128-byte swizzle) is the operand layout itself; 16 KB = one slot of the weight ring,
//       requested by the producer warp;
//   B = the normalised final state of 64 sequences, fp16, written by the distributed LayerNorm to global memory
//       in the same K-major swizzled layout (blocks of 64 k: 64 rows x 128 B) and copied into the K/V stages,
//       which are idle in this phase;
//   one thread issues the products of a block as soon as its slot is full and commits them to the slot's
//   empty barrier; after the last block of a tile it commits to the "done" barrier, and the eight consumer
//   warps read the accumulators (tcgen05.ld, a warp reads the lanes of its quarter), store the logits and
//   reduce the arg-max per sequence.
// ---------------------------------------------------------------------------------------------
#define TC_M 128
#define TC_N 64
#define TC_KB 64                                  // k per block (128 bytes of fp16)
#define TC_NKB (V_D / TC_KB)
#define TC_SLABS ((V_B + TC_N - 1) / TC_N)
#define TC_B_BYTES (TC_N * V_D * 2)               // operand B of one slab
#define TC_COLS 64                                // tensor-memory columns: one accumulator tile
// operand loaded: g = 0 (the whole operand, or its first third), 1 and 2 (the other thirds: the layer contractions start
// their products when a third has landed); the three complete once per operand, so one counter gives their parity
__device__ __forceinline__ u32 tc_load_bar(const Ctx& c, int g = 0) { return smem_u32(c.smem + SM_BARS) + (g == 0 ? 2 * V_NSLOT + V_KVST : 2 * V_NSLOT + 2 * V_KVST + 1 + g) * 8; }
__device__ __forceinline__ u32 tc_done_bar(const Ctx& c) { return smem_u32(c.smem + SM_BARS) + (2 * V_NSLOT + V_KVST + 1) * 8; }

// shared-memory matrix descriptor of a K-major operand in the 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2 (128-byte swizzle)
__device__ __forceinline__ u64 tc_desc(u32 smem_addr) {
    return (u64)((smem_addr & 0x3FFFFu) >> 4) | ((u64)1 << 16) | ((u64)(1024 >> 4) << 32) | ((u64)1 << 46) | ((u64)2 << 61);
}
// instruction descriptor: fp32 accumulate, fp16 A and B, both K-major, N = 64, M = 128
#define TC_IDESC ((1u << 4) | ((u32)(TC_N >> 3) << 17) | ((u32)(TC_M >> 4) << 24))

__device__ __forceinline__ void tc_mma(u32 d_tmem, u64 adesc, u64 bdesc, u32 accumulate, u32 idesc = TC_IDESC) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(u32 bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// The four products of one k-block of 64, for a warp that walks here as a whole: every lane carries the (uniform)
// descriptors, the lane that `elect_one` chose issues. Measured on B200 (48 products of 64 x 32 x 16 in a loop):
// issued by thread 0 inside a divergent branch, or under a predicate computed as lane == 0, a product costs 65 to
// 115 cycles (the descriptors pass from ordinary to uniform registers one by one); under the predicate of elect.sync
// it costs what the tensor core takes to read its operands from shared memory at 128 bytes per cycle
// ((rows of A + rows of B) x 32 bytes: 48 cycles at 128 x 64, 24 at 64 x 32). Polling warps beside it, more commits,
// the operand addresses and the data made no difference.
__device__ __forceinline__ u32 elect_one() {
    u32 leader;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
    return leader;
}
__device__ __forceinline__ void tc_mma_kb(u32 d_tmem, u64 adesc, u64 bdesc, bool first_kb, u32 idesc, u32 leader) {
#pragma unroll
    for (int k = 0; k < TC_KB / 16; k++)
        asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %4, 0;\n\tsetp.ne.b32 q, %5, 0;\n\t@q tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(adesc + 2 * k), "l"(bdesc + 2 * k), "r"(idesc), "r"((first_kb && k == 0) ? 0u : 1u), "r"(leader) : "memory");
}

// the normalised rows of the final state as operand B in global memory: row r of slab r / 64, block k / 64,
// 16-byte piece (k % 64) / 8 stored at piece ^ (row % 8) of its 128-byte row
// With `init` the same pass starts the vector the following projection is combined into: init[r] = z[r] + bias.
__device__ __forceinline__ void ln_rows_to_tc(Ctx& c, const float* __restrict__ z, float* __restrict__ init, unsigned char* __restrict__ tcg) {
    const u16* prm = reinterpret_cast<const u16*>(c.smem + SM_PRM);
#pragma unroll 1
    for (int r = c.cta * NW + c.warp; r < TC_SLABS * TC_N; r += c.ncta * NW) {
        float4 v[LNV];
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int g = i * 32 + c.lane;
            v[i] = (g < G4 && r < V_B) ? __ldcg(reinterpret_cast<const float4*>(z + (size_t)r * V_D) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
        const float mean = s * (1.0f / V_D);
        float q = 0.f;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            if (i * 32 + c.lane < G4) {
                const float a0 = v[i].x - mean, a1 = v[i].y - mean, a2 = v[i].z - mean, a3 = v[i].w - mean;
                q += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
            }
        }
#pragma unroll
        for (int m = 16; m; m >>= 1) q += __shfl_xor_sync(0xffffffffu, q, m);
        const float rs = rsqrtf(q * (1.0f / V_D) + V_EPS);
        const int rb = r % TC_N;
        unsigned char* dst = tcg + (size_t)(r / TC_N) * TC_B_BYTES + rb * 128;
#pragma unroll
        for (int i = 0; i < LNV; i++) {
            const int g = i * 32 + c.lane, d = g * 4;
            if (g < G4) {
                uint2 o = make_uint2(0, 0);                 // rows beyond the batch are zero
                if (r < V_B) {
                    const uint2 w = *reinterpret_cast<const uint2*>(prm + d);
                    const uint2 bb = *reinterpret_cast<const uint2*>(prm + V_D + d);
                    o.x = pack_h2((v[i].x - mean) * rs * h_lo(w.x) + h_lo(bb.x), (v[i].y - mean) * rs * h_hi(w.x) + h_hi(bb.x));
                    o.y = pack_h2((v[i].z - mean) * rs * h_lo(w.y) + h_lo(bb.y), (v[i].w - mean) * rs * h_hi(w.y) + h_hi(bb.y));
                }
                const int kb = d / TC_KB, piece = (d % TC_KB) >> 3;
                *reinterpret_cast<uint2*>(dst + (size_t)kb * (TC_N * 128) + ((piece ^ (rb & 7)) << 4) + ((d & 4) ? 8 : 0)) = o;
                if (init && r < V_B) {
                    const uint2 ib = *reinterpret_cast<const uint2*>(prm + 2 * V_D + d);
                    *reinterpret_cast<float4*>(init + (size_t)r * V_D + d) =
                        make_float4(v[i].x + h_lo(ib.x), v[i].y + h_hi(ib.x), v[i].z + h_lo(ib.y), v[i].w + h_hi(ib.y));
                }
            }
        }
    }
}

__device__ __forceinline__ void logits_tc(Ctx& c, const int* __restrict__ P, const unsigned char* __restrict__ tcg,
                                          float* __restrict__ logit, u64* __restrict__ gbest, int log_slabs) {
    const u32 tmem = *reinterpret_cast<const volatile u32*>(c.smem + SM_MISC + MISC_TMEM);
    const int rows = P[PT_LOG_NJ] * 16, n0 = P[PT_LOG_J0] * 16;
    const int mtiles = (rows + TC_M - 1) / TC_M;
    const int quarter = c.warp & 3, col0 = (c.warp >> 2) * 32;       // this warp reads lanes 32*quarter.., columns col0..col0+31
    const int wu = __shfl_sync(0xffffffffu, c.warp, 0);              // the warp index as a value the compiler knows to be uniform
    const u32 tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
#pragma unroll 1
    for (int slab = 0; slab < log_slabs; slab++) {
        // operand B of the slab: one bulk copy per block of 64 k into the K/V stages
        if (c.tid == 0 && mtiles > 0) {
            asm volatile("fence.proxy.async.global;" ::: "memory");          // the operand was written by other CTAs with ordinary stores
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_expect(tc_load_bar(c), TC_B_BYTES);
            mbar_arrive(tc_load_bar(c, 1)); mbar_arrive(tc_load_bar(c, 2));      // (their turn passes: one counter for the three)
#pragma unroll 1
            for (int kb = 0; kb < TC_NKB; kb++)
                bulk_g2s(smem_u32(c.smem + SM_KV) + kb * (TC_N * 128), tcg + (size_t)slab * TC_B_BYTES + (size_t)kb * (TC_N * 128), TC_N * 128, tc_load_bar(c));
        }
        if (mtiles > 0) { wait_mbar(c, tc_load_bar(c), c.tcl & 1u, 0x600u); c.tcl++; }
        u64 mybest = 0;                                              // best (value, index) of sequence slab*64 + col0 + lane in this CTA's rows
#pragma unroll 1
        for (int mt = 0; mt < mtiles; mt++) {
#if V_TCL
            // warp 0 alone waits for the slots and issues (see tc_contraction); the others meet it at the block barrier
            if (wu == 0) {
                const u32 leader = elect_one();
#pragma unroll 1
                for (int kb = 0; kb < TC_NKB; kb++) {
                    const u32 slot = (c.chunk + kb) % V_NSLOT, use = (c.chunk + kb) / V_NSLOT;
                    wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
                    const u32 slot_u = __shfl_sync(0xffffffffu, slot, 0);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (!(__shfl_sync(0xffffffffu, c.dead ? 1 : 0, 0) != 0)) {
                        tc_mma_kb(tmem_u, tc_desc(smem_u32(c.smem + SM_RING) + slot_u * (V_CH * FRAG_BYTES)), tc_desc(smem_u32(c.smem + SM_KV) + kb * (TC_N * 128)),
                                  kb == 0, TC_IDESC, leader);
                        if (leader) {
                            tc_commit(empty_bar(c, slot));               // the slot is free once these products have read it
                            if (kb == TC_NKB - 1) tc_commit(tc_done_bar(c));
                        }
                    } else if (c.lane == 0) mbar_arrive(empty_bar(c, slot));
                    __syncwarp();
                }
                wait_mbar(c, tc_done_bar(c), c.tcd & 1u, 0x700u);
            }
            c.chunk += TC_NKB; c.tcd++;
            cons_sync();
#else
#pragma unroll 1
            for (int kb = 0; kb < TC_NKB; kb++) {
                const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
                wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
                if (wu == 0) {
                    const u32 slot_u = __shfl_sync(0xffffffffu, slot, 0);
                    if (!(__shfl_sync(0xffffffffu, c.dead ? 1 : 0, 0) != 0)) {
                        const u32 leader = elect_one();
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        tc_mma_kb(tmem_u, tc_desc(smem_u32(c.smem + SM_RING) + slot_u * (V_CH * FRAG_BYTES)), tc_desc(smem_u32(c.smem + SM_KV) + kb * (TC_N * 128)),
                                  kb == 0, TC_IDESC, leader);                    // 32 bytes further per step of 16 k
                        if (leader) {
                            tc_commit(empty_bar(c, slot));               // the slot is free once these products have read it
                            if (kb == TC_NKB - 1) tc_commit(tc_done_bar(c));
                        }
                    } else if (c.lane == 0) mbar_arrive(empty_bar(c, slot));
                    __syncwarp();
                } else if (c.lane == 0) mbar_arrive(empty_bar(c, slot));
                c.chunk++;
            }
            // the accumulators of this tile: thread = vocabulary row, registers = 32 sequences
            wait_mbar(c, tc_done_bar(c), c.tcd & 1u, 0x700u); c.tcd++;
#endif
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            u32 r[32];
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                         : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                           "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                           "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                         : "r"(tmem + ((u32)(quarter * 32) << 16) + (u32)col0) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const int nl = mt * TC_M + quarter * 32 + c.lane, n = n0 + nl;       // this thread's vocabulary row
            const bool live = nl < rows && n < V_N && !c.dead;
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const int b = slab * TC_N + col0 + i;
                const float v = __uint_as_float(r[i]);
                if (live && b < V_B) logit[(size_t)b * V_N + n] = v;
                // the warp's best row for sequence b: maximum by redux, lowest row among the equal ones by ballot
                int kv = __float_as_int(live ? v : -3.0e38f);
                kv = kv >= 0 ? kv : kv ^ 0x7fffffff;
                const int km = __reduce_max_sync(0xffffffffu, kv);
                const u32 who = __ballot_sync(0xffffffffu, kv == km && live);
                if (who && c.lane == i) {
                    const u64 k = best_key(__int_as_float(km >= 0 ? km : km ^ 0x7fffffff), (u32)(n - c.lane + (__ffs(who) - 1)));
                    if (k > mybest) mybest = k;
                }
            }
            // every warp is done reading before the next tile's first product overwrites the accumulators
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            cons_sync();
        }
        const int b = slab * TC_N + col0 + c.lane;
        if (mybest && b < V_B) atomicMax(gbest + b, mybest);
    }
}

#if V_TCL
// One layer contraction on the tensor cores: this CTA's run of units of `kind`, one after the other. Per unit: the
// operand of its row block (V_TCL_RB sequences x TCL_UK k-blocks, fp16, K-major swizzled rows written to global memory
// by the previous phase) is bulk-copied into the K/V stages, which are idle outside the attention phase, unless the
// previous unit left it there; the unit's weights are in the ring (usually since before the phase started); one
// lane issues 4 x TCL_UK tcgen05.mma (64 x V_TCL_NW x 16: rows beyond the row block read whatever follows it in
// shared memory, their accumulator lanes are never read) and commits them to the slots' empty barriers and the
// "done" barrier; then the warps whose quarter of the tensor-memory lanes holds sequences read the accumulator
// (thread = sequence, 16 consecutive output columns) and run the epilogue of the kind.
struct TclOut {
    const u16 *bias;                 // QKV / FC: bias of the layer (halves), 0 otherwise
    float* sum;                      // the projections: the vector their partial sums are added into
    float* q;                        // QKV: queries, fp32 [sequence][V_D]
    u16 *keys, *vals;                // QKV: the caches
    unsigned char* gg;               // FC: GELU output as the operand of the MLP projection
    const int* s_pos;
};
#define TCL_M 64
#define TCL_IDESC ((1u << 4) | ((u32)(V_TCL_NW >> 3) << 17) | ((u32)(TCL_M >> 4) << 24))
#define TCL_EW (V_TCL_NW / 2)                      // output columns per epilogue thread: 8 or 16
__device__ __forceinline__ void tcl_ld(u32 (&r)[16], u32 addr) {
#if TCL_EW == 16
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
                   "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]) : "r"(addr) : "memory");
#else
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(addr) : "memory");
#endif
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The products of one unit, issued by a whole warp (`leader` comes from elect_one).
__device__ __forceinline__ void tcl_issue(u32 tmem, u32 a_addr, u32 b_addr, u32 leader, int k0, int k1) {
    const u64 ad = tc_desc(a_addr), bd = tc_desc(b_addr);
#pragma unroll 1
    for (int kb = k0; kb < k1; kb++)
        tc_mma_kb(tmem, ad + (u64)((kb * TCL_A_KB) >> 4), bd + (u64)((kb * (V_TCL_NW * 128)) >> 4), kb == 0, TCL_IDESC, leader);
}
__device__ __forceinline__ void tc_contraction(Ctx& c, int kind, int l, const unsigned char* __restrict__ opb, const TclOut& o) {
    const u32 tmem = *reinterpret_cast<const volatile u32*>(c.smem + SM_MISC + MISC_TMEM);
    const int ktot = tcl_ktot(kind);
    // A product of 64 rows leaves row m in tensor-memory lane 32 * (m / 16) + m % 16: the first 16 lanes of a warp's
    // quarter hold sequences, the others nothing.
    const int quarter = c.warp & 3, col0 = (c.warp >> 2) * TCL_EW;   // this warp reads lanes 32*quarter.., columns col0..col0+TCL_EW-1
    const int wu = __shfl_sync(0xffffffffu, c.warp, 0);              // the warp index as a value the compiler knows to be uniform
    const u32 tmem_u = __shfl_sync(0xffffffffu, tmem, 0);
    int u0, u1, staged = -1;
    tcl_run(kind, c.cta, c.ncta, u0, u1);
#pragma unroll 1
    for (int u = u0; u < u1; u++) {
        int rb, ks, fb;
        tcl_unit(kind, u, rb, ks, fb);
        // Warp 0 alone waits (for the operand, the weights and the products) and issues; the others go straight to the
        // block barrier below.
        const bool load = (rb * 64 + ks != staged);                          // (row block, fold part) of the operand in the stages
        staged = rb * 64 + ks;
        const u32 slot = c.chunk % V_NSLOT, use = c.chunk / V_NSLOT;
        if (wu == 0) {
            if (load) {
                if (c.lane == 0) {
                    asm volatile("fence.proxy.async.global;" ::: "memory");      // the operand was written by other CTAs with ordinary stores
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    // rows rb * V_TCL_RB .. of slab (rb * V_TCL_RB) / 64: V_TCL_RB rows of 128 bytes inside every 64-row k-block tile
                    const unsigned char* src = opb + ((size_t)((rb * V_TCL_RB) / 64) * ktot + (size_t)ks * TCL_UK) * (TC_N * 128) + ((rb * V_TCL_RB) % 64) * 128;
#pragma unroll
                    for (int g = 0; g < 3; g++) {
                        const int k0 = min(g * TCL_GS, TCL_UK), k1 = min(k0 + TCL_GS, TCL_UK);
                        if (k1 > k0) mbar_expect(tc_load_bar(c, g), (u32)(k1 - k0) * TCL_A_KB); else mbar_arrive(tc_load_bar(c, g));
                        if (V_TCL_RB == 64) {
                            // whole 64-row tiles follow one another in global and in shared memory: one copy per third
                            if (k1 > k0) bulk_g2s(smem_u32(c.smem + SM_KV) + k0 * TCL_A_KB, src + (size_t)k0 * (TC_N * 128), (u32)(k1 - k0) * TCL_A_KB, tc_load_bar(c, g));
                        } else {
#pragma unroll 1
                            for (int kb = k0; kb < k1; kb++)
                                bulk_g2s(smem_u32(c.smem + SM_KV) + kb * TCL_A_KB, src + (size_t)kb * (TC_N * 128), TCL_A_KB, tc_load_bar(c, g));
                        }
                    }
                }
                __syncwarp();
            }
            wait_mbar(c, full_bar(c, slot), use & 1u, 0x300u);
            TRACE(63);
            const u32 slot_u = __shfl_sync(0xffffffffu, slot, 0);
            // the products of a third of the fold as soon as that third of the operand has landed
#pragma unroll 1
            for (int g = 0; g < 3; g++) {
                if (load) wait_mbar(c, tc_load_bar(c, g), c.tcl & 1u, 0x600u);
                if (g == 0) TRACE(60);
                if (!(__shfl_sync(0xffffffffu, c.dead ? 1 : 0, 0) != 0)) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    tcl_issue(tmem_u, smem_u32(c.smem + SM_KV), smem_u32(c.smem + SM_RING) + slot_u * (V_CH * FRAG_BYTES), elect_one(),
                              min(g * TCL_GS, TCL_UK), min((g + 1) * TCL_GS, TCL_UK));
                }
            }
            const bool dead_u = __shfl_sync(0xffffffffu, c.dead ? 1 : 0, 0) != 0;
            if (!dead_u) {
                const u32 leader = elect_one();
                if (leader) {
#pragma unroll
                    for (u32 i = 0; i < TCL_SPU; i++) tc_commit(empty_bar(c, slot + i));     // the slots are free once these products have read them
                    tc_commit(tc_done_bar(c));
                }
            } else if (c.lane == 0) {
#pragma unroll
                for (u32 i = 0; i < TCL_SPU; i++) mbar_arrive(empty_bar(c, slot + i));
            }
            __syncwarp();
            TRACE(64);
            wait_mbar(c, tc_done_bar(c), c.tcd & 1u, 0x700u);
            TRACE(61);
        }
        if (load) c.tcl++;
        c.tcd++;
        c.chunk += TCL_SPU;
        cons_sync();                                                         // the products are done (warp 0 saw them complete)
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (quarter * 16 < V_TCL_RB && !c.dead) {
            u32 r[16];
            tcl_ld(r, tmem + ((u32)(quarter * 32) << 16) + (u32)col0);
            const int row = rb * V_TCL_RB + quarter * 16 + c.lane;           // this thread's sequence (row of the batch) where lane < 16
            const int j = fb * V_TCL_NW + col0;                              // its first output column
            if (c.lane < 16 && row < V_B) {
                if (kind == PH_QKV || kind == PH_FC) {
                    const u16* bp = o.bias + (size_t)l * (kind == PH_QKV ? 3 * V_D : V_F) + j;
#pragma unroll
                    for (int i = 0; i < TCL_EW; i += 8) {
                        const uint4 hb = __ldg(reinterpret_cast<const uint4*>(bp + i));
                        r[i + 0] = __float_as_uint(__uint_as_float(r[i + 0]) + h_lo(hb.x)); r[i + 1] = __float_as_uint(__uint_as_float(r[i + 1]) + h_hi(hb.x));
                        r[i + 2] = __float_as_uint(__uint_as_float(r[i + 2]) + h_lo(hb.y)); r[i + 3] = __float_as_uint(__uint_as_float(r[i + 3]) + h_hi(hb.y));
                        r[i + 4] = __float_as_uint(__uint_as_float(r[i + 4]) + h_lo(hb.z)); r[i + 5] = __float_as_uint(__uint_as_float(r[i + 5]) + h_hi(hb.z));
                        r[i + 6] = __float_as_uint(__uint_as_float(r[i + 6]) + h_lo(hb.w)); r[i + 7] = __float_as_uint(__uint_as_float(r[i + 7]) + h_hi(hb.w));
                    }
                }
                if (kind == PH_QKV) {
                    const int part = j / V_D, jj = j - part * V_D;           // 0: query, 1: key, 2: value (a unit never straddles two)
                    if (part == 0) {
                        float4* dst = reinterpret_cast<float4*>(o.q + (size_t)row * V_D + jj);
#pragma unroll
                        for (int i = 0; i < TCL_EW; i += 4)
                            dst[i >> 2] = make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                    } else if (o.s_pos[row] >= 0) {
                        uint4* dst = reinterpret_cast<uint4*>((part == 1 ? o.keys : o.vals) + ((size_t)(SEQ_OF(o.s_pos, row) * V_L + l) * V_TMAX + o.s_pos[row]) * V_D + jj);
#pragma unroll
                        for (int i = 0; i < TCL_EW; i += 8)
                            dst[i >> 3] = make_uint4(pack_h2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])), pack_h2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                                                     pack_h2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])), pack_h2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
                    }
                } else if (kind == PH_FC) {
                    const int rs = row & 63;                                 // row inside its slab of 64
                    unsigned char* dst = o.gg + ((size_t)(row >> 6) * TCL_KB_F + (j >> 6)) * (TC_N * 128) + rs * 128;
#pragma unroll
                    for (int i = 0; i < TCL_EW; i += 8) {
                        const int piece = ((j + i) & 63) >> 3;
                        float g[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) g[e] = gelu_tanh(__uint_as_float(r[i + e]));
                        *reinterpret_cast<uint4*>(dst + ((piece ^ (rs & 7)) << 4)) =
                            make_uint4(pack_h2(g[0], g[1]), pack_h2(g[2], g[3]), pack_h2(g[4], g[5]), pack_h2(g[6], g[7]));
                    }
                } else {
                    float* dst = o.sum + (size_t)row * V_D + j;
#pragma unroll
                    for (int i = 0; i < TCL_EW; i += 4)
                        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                                     :: "l"(dst + i), "f"(__uint_as_float(r[i])), "f"(__uint_as_float(r[i + 1])), "f"(__uint_as_float(r[i + 2])), "f"(__uint_as_float(r[i + 3])) : "memory");
                }
            }
        }
        TRACE(62);
        // every warp is done reading before the next unit's first product overwrites the accumulator (and before the
        // next unit's operand replaces this one in the K/V stages: its products have completed)
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        cons_sync();
    }
}
#endif

// The sums of one output tile of eight sequences (accumulator layout of mma.m16n8k16: lane (g, t) holds outputs g and
// g + 8 of sequences 2t and 2t + 1) added to zu[b][0..15] with one 16-byte atomic per lane instead of four 4-byte
// ones: the four lanes g = 4i .. 4i + 3 transpose their 4 x 4 values (four shuffles), after which lane q = g % 4 holds
// four consecutive outputs of sequence 2t + q % 2 in the tile's half q / 2. Sums of many CTAs into the same rows are
// bound by the number of atomic operations the L2 has to retire. `rows`: live sequences of the tile.
__device__ __forceinline__ void red_tile_v4(float* __restrict__ zu, const float (&v)[4], int lane, int rows) {
    const int g = lane >> 2, t = lane & 3, q = g & 3;
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
    if (b < rows)
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                     :: "l"(zu + (size_t)b * V_D + (g & ~3) + (hi ? 8 : 0)), "f"(o0), "f"(o1), "f"(o2), "f"(o3) : "memory");
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
    const int* row_seq;                         // optional (V_ROWSEQ): cache sequence of every row
    float* S; u32* bar; u64* TS;
    const unsigned char* WP; const int* PT;
    const unsigned char* TM;                    // TMA descriptors: eight of the K/V cache, one of the embedding table
    int nsteps;                                 // decode steps in this launch (the kernel feeds itself between them)
};

#if V_TIMING
// thread 0 of CTA V_TIMING-1 sums clock64 deltas per site in shared memory and adds them to TS at the end
#define TICK(k) do { if (c.cta == V_TIMING - 1 && c.tid == 0) { const long long now_ = clock64(); ts_[k] += now_ - tlast_; tlast_ = now_; } } while (0)
#else
#define TICK(k) do { } while (0)
#endif

__device__ __forceinline__ void step_body(const Args& a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    Ctx c;
    c.smem = smem; c.bar = a.bar; c.chunk = 0; c.dead = false; c.kvi = 0; c.kvn = 0; c.tcl = 0; c.tcd = 0;
    c.cta = blockIdx.x; c.ncta = gridDim.x; c.tid = threadIdx.x; c.warp = threadIdx.x >> 5; c.lane = threadIdx.x & 31;
#if V_TIMING
    __shared__ u64 trace_[(V_NW + 1) * TRACE_EVENTS];
    __shared__ long long ts_[16];
    c.trn = 0; c.tron = false; c.trbuf = trace_;
    if (threadIdx.x == 0) for (int i = 0; i < 16; i++) ts_[i] = 0;
    long long tlast_ = clock64();
    const u64 t_begin_ = now_ns();
#endif

    // Positions and tokens outside their ranges would index outside the caches and tables: refuse the
    // step (every CTA sees the same values and takes the same branch). A negative position marks a
    // sequence that has not started yet: its row is carried along but reads and writes no cache.
    int* s_pos = reinterpret_cast<int*>(smem + SM_MISC + MISC_POS);
    {
        int bad = 0;
#pragma unroll 1
        for (int b = c.tid; b < V_B; b += NTHREADS) {
            const int tb = __ldcg(a.t + b * V_TSTRIDE), xb = __ldcg(a.x + b);
            bad |= (tb >= V_TMAX) | (tb >= V_CPOS) | (xb < 0) | (xb >= V_N);
            s_pos[b] = tb;
#if V_ROWSEQ
            const int sq = __ldcg(a.row_seq + b) & ~ROW_NO_LOGITS;
            bad |= (sq < 0) | (sq >= V_BSEQ);
            s_pos[V_B + b] = sq;
#endif
        }
        // a launch that follows one that gave up does nothing: the abort flag stays until the host clears it
        if (c.tid == 0 && ld_relaxed(a.bar + BAR_ABORT)) bad |= 2;
        if (__syncthreads_or(bad)) {
            if (c.cta == 0 && c.tid == 0) atomicCAS(a.bar + BAR_STATUS, 0u, 0x900u);      // (an earlier failure keeps its own code)
            return;
        }
    }
    const int nsteps = max(a.nsteps, 1);
    // slabs of 64 rows whose logits are wanted: all of them, or (rows of a dense prompt pass) the slabs that hold the
    // rows without the ROW_NO_LOGITS mark, which the host places first
    int log_slabs = TC_SLABS_P;
#if V_ROWSEQ
    {
        int want = 0;
#pragma unroll 1
        for (int i = 0; i < (V_B + NTHREADS - 1) / NTHREADS; i++) {
            const int b = c.tid + i * NTHREADS;
            want += __syncthreads_count(b < V_B && !(__ldcg(a.row_seq + b) & ROW_NO_LOGITS));
        }
        log_slabs = (want + 63) / 64;
    }
#endif
    int* flag = reinterpret_cast<int*>(smem + SM_MISC + MISC_FLAG);
    volatile int* stop = reinterpret_cast<volatile int*>(smem + SM_MISC + MISC_STOP);
    if (c.tid == 0) {
        *stop = 0;
        if (c.cta == 0) asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" :: "l"(a.bar + BAR_STEP), "r"(0u) : "memory");   // nobody reads it before the first barrier
        // (with tensor-core layer contractions nothing but tensor-core products reads the ring: their commit is the one arrival)
        for (int s = 0; s < V_NSLOT; s++) { mbar_init(full_bar(c, s), 1); mbar_init(empty_bar(c, s), V_TCL ? 1 : NW); }
        for (int s = 0; s < V_KVST; s++) { mbar_init(kv_bar(c, s), 1); mbar_init(kv_empty_bar(c, s), NW); }
        *reinterpret_cast<volatile u32*>(smem + SM_MISC + MISC_ATTSEQ) = 0;
        mbar_init(tc_load_bar(c, 0), 1); mbar_init(tc_load_bar(c, 1), 1); mbar_init(tc_load_bar(c, 2), 1); mbar_init(tc_done_bar(c), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // operand tiles and K/V stages start as zero: rows of a batch tile beyond the batch stay zero for the whole
    // launch, and staged rows past the end of a chunk only ever meet a weight of zero
#pragma unroll 1
    for (int i = c.tid; i < (SM_RED - SM_KV) / 16; i += NTHREADS) reinterpret_cast<uint4*>(smem + SM_KV)[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();

#if V_TC
    // tensor memory for one accumulator tile; released by the same warp at the end of the kernel
    if (c.warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem + SM_MISC + MISC_TMEM)), "n"(TC_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#endif
    const int* P = a.PT + c.cta * PT_STRIDE;
    if (c.warp == NW) {
        if (c.lane == 0) producer(smem, a.bar, P, a.WP, a.TM, c.cta, c.ncta, nsteps, log_slabs);
        return;
    }

    c.gen = 0;      // the barrier counter is zero at launch: the last CTA of every step clears it
    unsigned char* act = smem + SM_ACT;
    unsigned char* gact = smem + SM_GACT;
    float* red = reinterpret_cast<float*>(smem + SM_RED);
    const u16* prm = reinterpret_cast<const u16*>(smem + SM_PRM);
    u64* wbest = reinterpret_cast<u64*>(smem + SM_MISC + MISC_BEST);
    float* Z = a.S + V_OFF_Z;
    float* qbuf = a.S + V_OFF_Q;
    float* part = a.S + V_OFF_PART;
    float* logit = a.S + V_OFF_LOGIT;
    unsigned char* actg = reinterpret_cast<unsigned char*>(a.S + V_OFF_ACTG);
#if V_TC
    unsigned char* tcg = reinterpret_cast<unsigned char*>(a.S + V_OFF_TC);
#endif
#if V_KSPLIT
    unsigned char* gg = reinterpret_cast<unsigned char*>(a.S + V_OFF_GG);     // GELU outputs as operand tiles: [slab][fold tile][batch tile]
#endif
#if V_TCL
    unsigned char* og = reinterpret_cast<unsigned char*>(a.S + V_OFF_OG);     // attention output as the operand of the projection
#else
    unsigned char* og = 0;
#endif
    u64* gbest = reinterpret_cast<u64*>(a.S + V_OFF_BEST);
    const int gtid = c.cta * NCONS + c.tid, gthreads = c.ncta * NCONS;
    const size_t ZS = (size_t)V_B * V_D;

#pragma unroll 1
  for (int step = 0; step < nsteps; step++) {
    if (step > 0) {
        // positions as the previous step of this launch left them (published before the step flag)
#pragma unroll 1
        for (int b = c.tid; b < V_B; b += NCONS) s_pos[b] = __ldcg(a.t + b * V_TSTRIDE);
        cons_sync();
    }
#if V_TCL
    att_plan(c, s_pos);
#endif
    // Q1: z0 = wte[x] + wpe[t]; the vector the first projection is combined into starts at zero
#pragma unroll 1
    for (int i = gtid; i < V_B * V_D; i += gthreads) {
        const int b = i / V_D, d = i - b * V_D;
        Z[i] = h2f(a.wte[(size_t)__ldcg(a.x + b) * V_D + d]) + h2f(a.wpe[(size_t)max(s_pos[b], 0) * V_D + d]);
        Z[ZS + i] = 0.f;
    }
    TICK(0);
    phase_end(c);
    fetch_params(c, a.ln1w, a.ln1b, a.ob, a.qkvb + P[PT_QKV_J0] * 16, P[PT_QKV_NJ]);
    phase_wait(c);
    TICK(1);

#pragma unroll 1
    for (int ph = 0; ph < V_L * PH_PER_LAYER + 1; ph++) {
        const int l = ph / PH_PER_LAYER;
        int first, last;
        phase_kinds(ph - l * PH_PER_LAYER, first, last);
        if (l == V_L) { first = PH_LOGITS; last = PH_LOGITS; }
        float* zin = Z + (size_t)((2 * l) % 3) * ZS;          // layer input (for LOGITS: the final state)
        float* z1 = Z + (size_t)((2 * l + 1) % 3) * ZS;
        float* z2 = Z + (size_t)((2 * l + 2) % 3) * ZS;
#if V_TIMING
        c.tron = (c.cta == V_TIMING - 1) && (l == V_L / 2);
#endif
        TRACE(1 + first);

        if (first == PH_ATT) {
#if V_TIMING
            const long long att_t0 = clock64();
#endif
            attention_phase(c, a.keys, a.vals, qbuf, part, l, s_pos, a.TM, og);
#if V_TIMING
            // every CTA's time in the attention phase of the middle layer (cycles), for the balance across the grid
            if (l == V_L / 2 && c.tid == 0) a.TS[1024 + c.cta] = (u64)(clock64() - att_t0);
#endif
        } else {
            // LN1 phase clears z2 (the MLP adds into it two barriers later); LN2 phase clears zin for the next layer
            // (not needed with the distributed LayerNorm, which starts those vectors with a plain store)
            float* clr = V_LN_DIST ? (float*)0 : (first == PH_QKV) ? z2 : (first == PH_FC) ? zin : (float*)0;
            if (clr) {
#pragma unroll 1
                for (int i = gtid; i < V_B * V_D; i += gthreads) clr[i] = 0.f;
            }
        }

#if V_LN_DIST
        if (first == PH_QKV || first == PH_FC || first == PH_LOGITS) {
#if V_TC
            if (first == PH_LOGITS) ln_rows_to_tc(c, zin, (float*)0, tcg);
            else
#endif
#if V_TCL
            ln_rows_to_tc(c, (first == PH_FC) ? z1 : zin, (first == PH_QKV) ? z1 : z2, tcg);
            if (false)
#endif
            ln_rows_to_global(c, (first == PH_FC) ? z1 : zin, (first == PH_QKV) ? z1 : (first == PH_FC) ? z2 : (float*)0, actg);
            phase_end(c);
            phase_wait(c);
        }
#endif
#if V_TC
        if (first == PH_LOGITS) { logits_tc(c, P, tcg, logit, gbest, log_slabs); break; }
#endif
#if V_TCL
        if (first != PH_ATT) {
            TclOut o;
            o.bias = (first == PH_QKV) ? a.qkvb : (first == PH_FC) ? a.fcb : (const u16*)0;
            o.sum = (first == PH_PROJ) ? z1 : z2;
            o.q = qbuf; o.keys = a.keys; o.vals = a.vals; o.gg = gg; o.s_pos = s_pos;
            tc_contraction(c, first, l, (first == PH_PROJ) ? og : (first == PH_P2) ? gg : tcg, o);
        }
#endif
#if !V_TCL
#pragma unroll 1
        for (int slab = 0; slab < ((first == PH_ATT) ? 0 : NSLAB); slab++) {
            const int row0 = slab * SB, nrows = min(SB, V_B - row0);
#pragma unroll 1
            for (int kind = first; kind <= last; kind++) {
                // ---- prologue: what the contraction reads from other CTAs, into operand tiles
                if (kind == PH_QKV || kind == PH_FC || kind == PH_LOGITS) {
                    // LN1 (starts z1 = z + ob) | LN2 (starts z2 = z1 + pb) | LNf
#if V_LN_DIST
                    load_act_tiles(c, actg + (size_t)slab * SLAB_TILE_BYTES, act);
#else
                    ln_to_act(c, ((kind == PH_FC) ? z1 : zin) + (size_t)row0 * V_D,
                              (kind == PH_QKV) ? z1 + (size_t)row0 * V_D : (kind == PH_FC) ? z2 + (size_t)row0 * V_D : (float*)0, act, nrows);
#endif
                }
                else if (kind == PH_PROJ && P[PT_PROJ_NJ])
                    merge_to_act(c, part, P[PT_PROJ_K0], P[PT_PROJ_NK], act, row0, nrows);
#if V_KSPLIT
                else if (kind == PH_P2 && P[PT_P2_NJ])
                    // the GELU outputs of the slab for this CTA's slice of the fold, written by the FC phase of all CTAs
                    load_tiles(c, gg + ((size_t)slab * KT_F + P[PT_P2_K0]) * (V_NB * ATILE), act, P[PT_P2_NK] * (V_NB * ATILE));
#endif
                TRACE(10 + kind);

                // ---- the contraction, group by group, each followed by its epilogue
                const Seg sg = seg_of(P, kind);
                u64 best[V_NB][2];
#pragma unroll
                for (int nb = 0; nb < V_NB; nb++) { best[nb][0] = 0; best[nb][1] = 0; }
#pragma unroll 1
                for (int j = 0; j < sg.nj; j += (sg.wide ? WG : WN_MAX * 4)) {
                    const int width = sg.wide ? min(WG, sg.nj - j) : sg.nj;
                    float acc[TPW][V_NB][4];
                    TRACE(50);
                    gemm_group(c, sg.rows, width, sg.wide, (kind == PH_P2 && !V_KSPLIT) ? gact : act, acc);
                    TRACE(51);
                    if (!sg.wide) {
                        // NARROW: sum the warps that share an output tile; thread (jj, o) then owns one output
#pragma unroll
                        for (int nb = 0; nb < V_NB; nb++)
                            *reinterpret_cast<float4*>(red + ((size_t)(c.warp * V_NB + nb) * 32 + c.lane) * 4) = make_float4(acc[0][nb][0], acc[0][nb][1], acc[0][nb][2], acc[0][nb][3]);
                        cons_sync();
                        TRACE(52);
                        // One batch tile: a thread per output (256 of them for two output tiles). More: a thread takes the
                        // four sums of one lane of an output tile and reads the warps' partial tiles 16 bytes at a time.
#define EPI4 (V_NB >= 2)
#pragma unroll 1
                        for (int o4 = c.tid; o4 < width * V_NB * (EPI4 ? 32 : 128); o4 += NCONS) {
                          const int per = V_NB * (EPI4 ? 32 : 128);
                          const int jj = o4 / per, r4 = o4 - jj * per;
                          float4 v4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
                          for (int w = jj; w < NW; w += width) {
                              if (EPI4) {
                                  const float4 p4 = *reinterpret_cast<const float4*>(red + ((size_t)w * V_NB * 32 + r4) * 4);
                                  v4.x += p4.x; v4.y += p4.y; v4.z += p4.z; v4.w += p4.w;
                              } else v4.x += red[(size_t)w * V_NB * 128 + r4];
                          }
                          const int ln = EPI4 ? (r4 & 31) : ((r4 >> 2) & 31), nb = EPI4 ? (r4 >> 5) : (r4 >> 7);
#pragma unroll 1
                          for (int i4 = 0; i4 < (EPI4 ? 4 : 1); i4++) {
                            const int i = EPI4 ? i4 : (r4 & 3);
                            float v = (!EPI4 || i4 == 0) ? v4.x : i4 == 1 ? v4.y : i4 == 2 ? v4.z : v4.w;
                            const int j_in = (ln >> 2) + ((i & 2) ? 8 : 0), rb = nb * 8 + (ln & 3) * 2 + (i & 1), b = row0 + rb;
                            if (kind == PH_PROJ || kind == PH_P2) {
                                // a slice of the fold: added to the vector the LayerNorm pass started (residual + bias)
                                if (rb < nrows) red_add(((kind == PH_PROJ) ? z1 : z2) + (size_t)b * V_D + (P[(kind == PH_PROJ) ? PT_PROJ_J0 : PT_P2_J0] + jj) * 16 + j_in, v);
                                continue;
                            }
                            v += h2f(prm[3 * V_D + jj * 16 + j_in]);
                            if (kind == PH_QKV) {
                                // q to scratch, K and V rounded to fp16 into the cache at t
                                if (rb < nrows) {
                                    const int jx = (P[PT_QKV_J0] + jj) * 16 + j_in;
                                    if (jx < V_D) qbuf[(size_t)b * V_D + jx] = v;
                                    else if (s_pos[b] >= 0) {
                                        const size_t at = ((size_t)(SEQ_OF(s_pos, b) * V_L + l) * V_TMAX + s_pos[b]) * V_D + (jx % V_D);
                                        if (jx < 2 * V_D) a.keys[at] = f2h(v); else a.vals[at] = f2h(v);
                                    }
                                }
                            } else {
                                // g = gelu(u) -> operand tiles of the MLP projection: fold index = jj*16 + j_in
                                const float g = (rb < nrows) ? gelu_tanh(v) : 0.f;
#if V_KSPLIT
                                act_store1(gg + (size_t)slab * KT_F * (V_NB * ATILE), rb, (P[PT_FC_J0] + jj) * 16 + j_in, g);
#else
                                act_store1(gact, rb, jj * 16 + j_in, g);
#endif
                            }
                          }
                        }
                        cons_sync();
                    } else {
                        float* zt = (kind == PH_PROJ) ? z1 : z2;
#pragma unroll
                        for (int tw = 0; tw < TPW; tw++) {
                            if (c.warp + tw * NW >= width) continue;
                            const int jt = ((kind == PH_PROJ) ? P[PT_PROJ_J0] : (kind == PH_LOGITS) ? P[PT_LOG_J0] : 0) + j + c.warp + tw * NW;
#pragma unroll
                            for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                                if (kind != PH_LOGITS) red_tile_v4(zt + (size_t)(row0 + nb * 8) * V_D + jt * 16, acc[tw][nb], c.lane, nrows - nb * 8);
#pragma unroll
                            for (int nb = 0; nb < V_NB; nb++)
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const int jx = jt * 16 + (c.lane >> 2) + ((i & 2) ? 8 : 0), rb = nb * 8 + (c.lane & 3) * 2 + (i & 1), b = row0 + rb;
                                    if (kind != PH_LOGITS) {
                                    } else if (rb < nrows && jx < V_N) {
                                        logit[(size_t)b * V_N + jx] = acc[tw][nb][i];
                                        const u64 k = best_key(acc[tw][nb][i], (u32)jx);
                                        if (k > best[nb][i & 1]) best[nb][i & 1] = k;
                                    }
                                }
                        }
                    }
                }
                if (kind == PH_LOGITS) {
                    // argmax of the slab: per row the max over the lanes that hold it (equal lane&3), the warps, the CTAs
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
                            if ((c.lane >> 2) == 0) wbest[(nb * 8 + (c.lane & 3) * 2 + p) * NW + c.warp] = k;
                        }
                    cons_sync();
                    if (c.tid < nrows) {
                        u64 k = 0;
#pragma unroll 1
                        for (int w = 0; w < NW; w++) if (wbest[c.tid * NW + w] > k) k = wbest[c.tid * NW + w];
                        if (k) atomicMax(gbest + row0 + c.tid, k);
                    }
                    cons_sync();
                }
                TRACE(20 + kind);
            }
        }
#endif
        if (first == PH_LOGITS) break;

        // ---- grid barrier; the next LayerNorm's parameters are fetched while waiting
        TICK(2 + 2 * min(ph - l * PH_PER_LAYER, 3));
        phase_end(c);
        if (first == PH_PROJ)
            fetch_params(c, a.ln2w + (size_t)l * V_D, a.ln2b + (size_t)l * V_D, a.pb + (size_t)l * V_D,
                         a.fcb + (size_t)l * V_F + P[PT_FC_J0] * 16, P[PT_FC_NJ]);
        else if (ph - l * PH_PER_LAYER == PH_PER_LAYER - 1) {
            if (l + 1 < V_L)
                fetch_params(c, a.ln1w + (size_t)(l + 1) * V_D, a.ln1b + (size_t)(l + 1) * V_D, a.ob + (size_t)(l + 1) * V_D,
                             a.qkvb + (size_t)(l + 1) * 3 * V_D + P[PT_QKV_J0] * 16, P[PT_QKV_NJ]);
            else
                fetch_params(c, a.lnfw, a.lnfb, (const u16*)0, (const u16*)0, 0);
        }
        // the producer thread may request this layer's K/V tiles: before the barrier (the consumers patch the row of the
        // current position in), or after it where several rows of this step may lie in one tile (V_ROWSEQ)
        if (first == PH_QKV && c.tid == 0 && !V_ROWSEQ) {
            volatile u32* seq = reinterpret_cast<volatile u32*>(smem + SM_MISC + MISC_ATTSEQ);
            __threadfence_block();
            *seq = *seq + 1;
        }
        TRACE(30 + first);
        phase_wait(c);
        if (first == PH_QKV && c.tid == 0 && V_ROWSEQ) {
            volatile u32* seq = reinterpret_cast<volatile u32*>(smem + SM_MISC + MISC_ATTSEQ);
            __threadfence_block();
            *seq = *seq + 1;
        }
        TICK(3 + 2 * min(ph - l * PH_PER_LAYER, 3));
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
#pragma unroll 1
        for (int b = c.tid; b < V_B; b += NCONS) {
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
#if V_TC
    cons_sync();
    if (c.warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(*reinterpret_cast<const volatile u32*>(smem + SM_MISC + MISC_TMEM)), "n"(TC_COLS) : "memory");
#endif
    TICK(11);
#if V_TIMING
    if (c.cta == V_TIMING - 1 && c.lane == 0)
        for (int i = 0; i < TRACE_EVENTS; i++) a.TS[64 + c.warp * TRACE_EVENTS + i] = i < c.trn ? trace_[c.warp * TRACE_EVENTS + i] : 0ull;
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

// A(m = output j, k) of the five contractions
__device__ __forceinline__ u16 w_elem(const PackArgs& a, int kind, int l, int j, int k) {
    switch (kind) {
        case PH_QKV: return a.qkvw[((size_t)l * V_D + k) * (3 * V_D) + j];
        case PH_PROJ: return a.ow[((size_t)l * V_D + k) * V_D + j];
        case PH_FC: return a.fcw[((size_t)l * V_D + k) * V_F + j];
        case PH_P2: return a.pw[((size_t)l * V_F + k) * V_D + j];
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

// one segment: NARROW tile index = k * nj + jj; WIDE groups of WG output tiles, inside a group
// tile index = k_rel * width + w. Returns the number of tiles.
__device__ int pack_segment(const PackArgs& a, unsigned char* dst, const int* __restrict__ P, int kind, int l, int wid, int nwarp, int lane) {
    const Seg s = seg_of(P, kind);
    const int n = s.rows * s.nj;
    const int j0 = (kind == PH_QKV) ? P[PT_QKV_J0] : (kind == PH_PROJ) ? P[PT_PROJ_J0] : (kind == PH_FC) ? P[PT_FC_J0]
                 : (kind == PH_LOGITS) ? P[PT_LOG_J0] : (kind == PH_P2 && V_KSPLIT) ? P[PT_P2_J0] : 0;
    const int k0 = (kind == PH_PROJ) ? P[PT_PROJ_K0] : (kind == PH_P2) ? (V_KSPLIT ? P[PT_P2_K0] : P[PT_FC_J0]) : 0;
    for (int i = wid; i < n; i += nwarp) {
        int jt, kt;
        if (!s.wide) { jt = j0 + i % s.nj; kt = k0 + i / s.nj; }
        else {
            const int grp = i / (WG * s.rows);                 // full groups before this tile hold WG*rows tiles
            const int width = min(WG, s.nj - grp * WG);
            const int r = i - grp * WG * s.rows;
            jt = j0 + grp * WG + r % width; kt = k0 + r / width;
        }
        pack_tile(a, dst + (size_t)i * FRAG_BYTES, kind, l, jt, kt, lane);
    }
    return n;
}

#if V_TCL
// The weight image of the tensor-core layer contractions: per layer [QKV | attn-proj | FC | MLP-proj], each a list of
// (fold part, output block) blocks of TCL_UK tiles; a tile = V_TCL_NW output columns x 64 fold indices in the
// shared-memory layout of a K-major operand with the 128-byte swizzle: row r (one output column) = 128 bytes at
// r * 128, its 16-byte piece p stored at p ^ (r % 8). One block of threads per weight block and pass over the grid;
// the logits read the embedding table itself (by TMA), nothing is packed for them.
__device__ void pack_body(const PackArgs& a) {
    for (int blk = blockIdx.x; blk < V_L * TCL_W_LAYER; blk += gridDim.x) {
        const int l = blk / TCL_W_LAYER, t = blk - l * TCL_W_LAYER;
        const int kind = t < TCL_W_PROJ ? PH_QKV : t < TCL_W_FC ? PH_PROJ : t < TCL_W_P2 ? PH_FC : PH_P2;
        const int i = t - tcl_first_block(kind), ks = i / tcl_nfb(kind), fb = i - ks * tcl_nfb(kind);
        unsigned char* dst = a.WP + (size_t)blk * TCL_UB;
        for (int e = threadIdx.x; e < V_TCL_NW * 64 * TCL_UK; e += blockDim.x) {
            // consecutive threads take consecutive output columns: the weights are stored with the output index contiguous
            const int r = e % V_TCL_NW, kk = e / V_TCL_NW, kb = kk >> 6, k = kk & 63;
            *reinterpret_cast<u16*>(dst + (size_t)kb * (V_TCL_NW * 128) + r * 128 + ((((k >> 3) ^ (r & 7))) << 4) + (k & 7) * 2) =
                w_elem(a, kind, l, fb * V_TCL_NW + r, (ks * TCL_UK + kb) * 64 + k);
        }
    }
}
#else
// grid: (V_L + 1) blocks per CTA of the step kernel: blockIdx.x = cta * (V_L + 1) + l; l == V_L packs the logits
__device__ void pack_body(const PackArgs& a) {
    const int cta = blockIdx.x / (V_L + 1), l = blockIdx.x % (V_L + 1);
    const int* P = a.PT + cta * PT_STRIDE;
    const int wid = threadIdx.x >> 5, nwarp = blockDim.x >> 5, lane = threadIdx.x & 31;
    unsigned char* base = a.WP + (size_t)(u32)P[PT_BASE] * FRAG_BYTES;
    if (l == V_L) {
        pack_segment(a, base + (size_t)V_L * (u32)P[PT_LAYER] * FRAG_BYTES, P, PH_LOGITS, 0, wid, nwarp, lane);
        return;
    }
    for (int kind = PH_QKV; kind <= PH_P2; kind++) {
        if (kind == PH_ATT) continue;
        pack_segment(a, base + ((size_t)l * (u32)P[PT_LAYER] + seg_of(P, kind).off) * FRAG_BYTES, P, kind, l, wid, nwarp, lane);
    }
}
#endif
