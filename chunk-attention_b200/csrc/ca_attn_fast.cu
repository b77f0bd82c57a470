// Decode attention over a prefix tree of KV chunks, fp16 / d_head 128 / chunk_size 64, sm_100a.
//
// attn_partial_kernel — ONE persistent kernel, two CTAs per SM, serves both phases of the
// reference's two-phase decode attention:
//   * chunk-first items (reference: attn_chunk_first_kernel_v2, cpp/chunk_attn/kernel_cuda.cu:796-883):
//     the queries of all rows sharing a run of chunks form a small dense contraction against
//     every K/V tile of the run.  Runs on tensor cores (mma.sync m16n8k16, fp32 accumulate) with
//     a flash-style online softmax kept in registers across the WHOLE run, so a run emits one
//     partial per row instead of one per chunk.
//   * sequence-first items (reference: attn_seq_first_kernel, kernel_cuda.cu:885-1086): one row's
//     private tail chunks.  Memory-bound; walked by default with the same tensor-core code (one
//     useful row out of 16 — the MMA path needs a third of the instructions of the CUDA-core
//     walk, and with a handful of warps per SM instruction latency, not HBM, was the limit), or,
//     selectably, on CUDA cores with 128-bit shared-memory loads, fp32 dot products and
//     warp-shuffle reductions.
// Both kinds read their K/V tiles from a ring of 32 KiB shared-memory stages, filled by a
// producer warp with 1-D TMA bulk copies (cp.async.bulk + mbarrier transaction counts) that run
// ahead across item boundaries.  Items (at most 8 tiles, cut by the host, ca_plan.h) are
// self-scheduled: each CTA's producer draws the next item from a device counter once the current
// one is issued in full and hands its description to the consumers through shared memory together with the item's
// first tile, so the split of the work follows what each SM actually achieves.  A CTA is one
// consumer warpgroup (4 warps) plus a producer warpgroup; two CTAs share an SM so that one CTA's
// item boundaries (queries, combining warps, storing a partial) hide behind the other CTA's
// steady state.
//
// attn_merge_kernel — combines the partials of each (row, head) with the usual
// max-rescaled sum (reference: the merge inlined in kernel_cuda.cu:962-984,1042-1085).
//
// Every wait on an mbarrier is bounded: when the bound is hit the kernel records a status code
// and unwinds instead of spinning forever.
#include <cuda_fp16.h>

#include <cstdlib>

#include "ca_kernels.h"
#include "ca_plan.h"
#include "ca_ptx.cuh"

namespace ca {
namespace {
using namespace ptx;

constexpr int NUM_STAGES = 3;
constexpr int NUM_CONSUMER_WARPS = FAST_CONSUMER_WARPS;  // one warpgroup
// The CTA is two warpgroups; the register file is re-split at run time: the producer group shrinks
// to 56 registers per thread, the consumers grow to 200 (2 CTAs * (128 * 56 + 128 * 200) = 65536).
constexpr int NUM_THREADS = (NUM_CONSUMER_WARPS + 4) * 32;
constexpr int PRODUCER_REGS = 56;
constexpr int CONSUMER_REGS = 200;
constexpr int SCRATCH_FLOATS_PER_WARP = 132;  // m, l, 2 pad, o[128]
constexpr int SCRATCH_BYTES = 2 * NUM_CONSUMER_WARPS * SCRATCH_FLOATS_PER_WARP * 4;
constexpr int NUM_BARRIERS = 2 * NUM_STAGES + 1;
// Query rows of items of up to 16 rows travel with the item's first tile: one slot per ring stage.
// Rows are pitched 16 bytes past their 256 so that the 8 rows an ldmatrix reads fall in 8 different
// bank groups.
constexpr int QSLOT_ROWS = 16;
constexpr int QSLOT_PITCH = FAST_D * 2 + 16;
constexpr int QSLOT_BYTES = QSLOT_ROWS * QSLOT_PITCH;
constexpr int SMEM_RING_BYTES = NUM_STAGES * FAST_STAGE_BYTES;
constexpr int SMEM_Q_OFFSET = SMEM_RING_BYTES;
constexpr int SMEM_SCRATCH_OFFSET = SMEM_Q_OFFSET + NUM_STAGES * QSLOT_BYTES;
constexpr int SMEM_BAR_OFFSET = SMEM_SCRATCH_OFFSET + SCRATCH_BYTES;
constexpr int SMEM_BYTES = SMEM_BAR_OFFSET + NUM_BARRIERS * 8 + 16;
// two CTAs per SM: 228 KiB per SM, 1 KiB of it reserved per resident CTA
static_assert(2 * (SMEM_BYTES + 1024) <= 233472, "two CTAs do not fit in one SM's shared memory");
constexpr float NEG_BIG = -1.0e30f;

struct ItemView {
    int n_tiles, head, row_begin, n_rows, slot_base, flags, last_tokens, end;  // end != 0: no more items
};
struct ItemChunks {
    int c[9];  // pool slots of the item's tiles
};

// The work list holds every item ONCE, for all heads: work piece v of a launch is item v / n_heads for head
// v % n_heads.  Partial rows are numbered per item as well; row ts of head h lives in slot ts * n_heads + h, so an
// item's description carries slot_base * n_heads + h and consecutive rows of one head are n_heads slots apart.
// Volatile so that the loads are issued where they are written (an item ahead of their use)
// instead of being sunk to the first use by the compiler.
__device__ __forceinline__ void load_item(const int4* items, int v, int n_heads, ItemView& it, ItemChunks& ch) {
    const int i = v / n_heads;
    const int h = v - i * n_heads;
    int4 a, b, c, d;
    asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(items + 4 * i));
    asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(items + 4 * i + 1));
    asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(c.x), "=r"(c.y), "=r"(c.z), "=r"(c.w) : "l"(items + 4 * i + 2));
    asm volatile("ld.global.nc.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(d.x), "=r"(d.y), "=r"(d.z), "=r"(d.w) : "l"(items + 4 * i + 3));
    it = ItemView{a.x, h, a.z, a.w, b.x, b.y, b.z, 0};
    ch = ItemChunks{{b.w, c.x, c.y, c.z, c.w, d.x, d.y, d.z, d.w}};
}

// tokens held by tile j of an item; only the last tile of a sequence-first item can be partial
__device__ __forceinline__ int tile_tokens(const ItemView& it, int j, int delta) {
    if (j != it.n_tiles - 1) return FAST_C;
    const int t = it.last_tokens + ((it.flags & ITEM_FLAG_TAIL) ? delta : 0);
    return t < FAST_C ? t : FAST_C;
}

// Byte offset, inside a K or V tile, of the 16-byte granule g (0..15) of token row t: the tile is two panels of
// 64 lines of 128 bytes (ca_layout.h), granule c of a line stored at c ^ (t & 7).
constexpr int PANEL_BYTES = FAST_C * 128;
__device__ __forceinline__ uint32_t tile_off(int t, int g) {
    return (uint32_t)(((g >> 3) * PANEL_BYTES) + (t << 7) + (((g & 7) ^ (t & 7)) << 4));
}

// Every index an item carries, checked against the bounds the launch was given (a bound of 0 is unchecked).
// The work list may come from device memory the host never saw (ca_attention_static), so nothing in it is
// trusted: an item that fails is skipped and the status word says so.
__device__ __forceinline__ bool item_in_bounds(const PartialParams& p, const ItemView& it, const ItemChunks& ch) {
    const int splits = it.flags >> ITEM_SPLITS_SHIFT;
    const int slots = it.n_rows == 1 ? 1 : it.n_rows * (splits > 1 ? splits : 1);
    const int max_rows = splits == 4 ? 16 : (splits == 2 ? 32 : (splits == 1 ? MAX_ROWS_PER_ITEM : (splits == 0 ? 1 : 0)));
    bool ok = (it.flags & ITEM_FLAG_WIDE) == 0 && it.n_tiles >= 1 && it.n_tiles <= MAX_TILES_PER_ITEM && it.n_rows >= 1 &&
              it.n_rows <= max_rows &&
              it.head >= 0 && it.head < p.n_heads && it.row_begin >= 0 && it.slot_base >= 0 && it.last_tokens >= 0 &&
              it.last_tokens <= FAST_C;
    if (p.n_slots > 0) ok = ok && (long long)(it.slot_base + slots) * p.n_heads <= p.n_slots;
    if (p.n_seqs > 0) ok = ok && it.row_begin + it.n_rows <= p.n_seqs;
    if (ok && p.max_chunks > 0) {
#pragma unroll
        for (int j = 0; j < MAX_TILES_PER_ITEM; j++)
            if (j < it.n_tiles) ok = ok && ch.c[j] >= 0 && ch.c[j] < p.max_chunks;
    }
    return ok;
}

// ---- pipeline bookkeeping shared by producer and consumers ----------------------------------------
struct Ring {
    uint32_t ring;        // shared address of stage 0
    uint32_t qslots;      // shared address of query slot 0 (slot s belongs to stage s)
    uint32_t full_bar;    // NUM_STAGES barriers, producer -> consumers (count 1 + tx bytes)
    uint32_t empty_bar;   // NUM_STAGES barriers, consumers -> producer (count NUM_CONSUMER_WARPS)
    uint32_t stage;
    uint32_t phase;
    long long wait_limit;     // cycles a wait may take before the kernel gives up
    bool timed;               // tracing on: accumulate stall cycles
    long long wait_cycles;    // cycles spent waiting on ring barriers
    long long tail_cycles;    // consumers: cycles spent combining warps and storing partials
    __device__ __forceinline__ void advance() {
        if (++stage == NUM_STAGES) {
            stage = 0;
            phase ^= 1;
        }
    }
};

__device__ __forceinline__ void report(int* status, int code) { atomicCAS(status, STATUS_OK, code); }

// The description of an item travels to the consumers in the padding of the first two query rows of
// the slot that belongs to the stage of the item's first tile (16 spare bytes after each 256-byte row).
__device__ __forceinline__ uint32_t desc_addr(const Ring& rg, uint32_t stage) {
    return rg.qslots + stage * QSLOT_BYTES + FAST_D * 2;
}

// ---- producer: one thread -----------------------------------------------------------------------------
// Post one stage: wait for it to be free, optionally publish an item description and the item's
// query rows, and start the tile's bulk copies.  bytes == 0 posts an empty stage (an item without
// tokens, or the end marker).
__device__ __forceinline__ bool producer_post(const PartialParams& p, Ring& rg, const ItemView* desc, bool stage_q,
                                              const uint8_t* src, uint32_t bytes) {
    const long long t0 = rg.timed ? clock64() : 0;
    const bool ok = mbar_wait_bounded(rg.empty_bar + 8 * rg.stage, rg.phase ^ 1, rg.wait_limit);
    if (rg.timed) rg.wait_cycles += clock64() - t0;
    if (!ok) return false;
    const uint32_t bar = rg.full_bar + 8 * rg.stage;
    uint32_t q_bytes = 0;
    if (desc) {
        const uint32_t da = desc_addr(rg, rg.stage);
        sts128(da, desc->n_tiles, desc->head, desc->row_begin, desc->n_rows);
        sts128(da + QSLOT_PITCH, desc->slot_base, desc->flags, desc->last_tokens, desc->end);
        if (stage_q) q_bytes = (uint32_t)desc->n_rows * (FAST_D * 2);
    }
    mbar_arrive_expect_tx(bar, 2 * bytes + q_bytes);  // release: the description is visible to whoever sees the phase
    if (bytes == FAST_TILE_BYTES) {
        const uint32_t dst = rg.ring + rg.stage * FAST_STAGE_BYTES;
        bulk_copy_g2s(dst, src, bytes, bar);
        bulk_copy_g2s(dst + FAST_TILE_BYTES, src + FAST_TILE_BYTES, bytes, bar);
    } else if (bytes) {
        // a partly filled tail: the first n token lines of each of the four panels (K, K, V, V)
        const uint32_t dst = rg.ring + rg.stage * FAST_STAGE_BYTES;
#pragma unroll
        for (int pnl = 0; pnl < 4; pnl++) bulk_copy_g2s(dst + pnl * PANEL_BYTES, src + pnl * PANEL_BYTES, bytes / 2, bar);
    }
    if (q_bytes) {
        const uint8_t* q = reinterpret_cast<const uint8_t*>(p.q) +
                           ((size_t)desc->row_begin * p.n_heads + desc->head) * (FAST_D * 2);
        const uint32_t qdst = rg.qslots + rg.stage * QSLOT_BYTES;
        for (int r = 0; r < desc->n_rows; r++)
            bulk_copy_g2s(qdst + r * QSLOT_PITCH, q + (size_t)r * p.n_heads * (FAST_D * 2), FAST_D * 2, bar);
    }
    rg.advance();
    return true;
}

__device__ __forceinline__ void producer_loop(const PartialParams& p, Ring& rg) {
    uint32_t issued = 0;
    bool ok = true;
    // The first two items of a CTA are fixed by its index, so that nothing waits for an atomic at
    // start-up; the counter hands out the items after those of all CTAs.  An item is drawn only
    // after the previous one has been issued in full: by then the ring holds NUM_STAGES tiles in
    // flight, which cover the round trips of the atomic and of the description, and no CTA sits on
    // work it has claimed but not started while other CTAs run dry at the end of the list (drawing
    // two items ahead left the last CTA 4 us behind the median one).
    const int n_fixed = 2 * (int)gridDim.x;
    int id0 = p.item_lo + (int)blockIdx.x;
    int id1 = p.item_lo + (int)gridDim.x + (int)blockIdx.x;  // < 0: draw from the counter
    ItemView it{};
    ItemChunks ch{};
    bool withheld = false;
    if (id0 < p.item_hi) load_item(p.items, id0, p.n_heads, it, ch);
    while (id0 < p.item_hi && ok) {
        if (id0 == p.withhold_item) {
            // failure-path test: this CTA's consumers are never told about the item (nor about the end of the
            // list), so their bounded wait runs out
            withheld = true;
            break;
        }
        if (!item_in_bounds(p, it, ch)) {
            report(p.status, STATUS_BAD_WORK_LIST);  // skipped: its partial rows keep whatever they held
        } else {
            it.slot_base = it.slot_base * p.n_heads + it.head;  // this head's first partial row
            // items of up to 16 rows get their query rows staged next to their first tile
            const bool stage_q = (it.flags >> ITEM_SPLITS_SHIFT) == NUM_CONSUMER_WARPS;
            bool first = true;
#pragma unroll
            for (int j = 0; j < 9; j++) {
                if (j < it.n_tiles && ok) {
                    const int nt = tile_tokens(it, j, p.delta_tokens);
                    if (nt > 0) {
                        const uint8_t* src = p.pool + ((size_t)ch.c[j] * p.n_heads + it.head) * (size_t)FAST_STAGE_BYTES;
                        ok = producer_post(p, rg, first ? &it : nullptr, stage_q, src, (uint32_t)nt * (FAST_D * 2));
                        issued += ok ? 1 : 0;
                        first = false;
                    }
                }
            }
            if (first && ok) {  // no token in the whole item: the description still has to travel
                ok = producer_post(p, rg, &it, false, nullptr, 0);
                issued += ok ? 1 : 0;
            }
        }
        id0 = id1 >= 0 ? id1 : p.item_lo + n_fixed + atomicAdd(p.counter, 1);
        id1 = -1;
        if (id0 < p.item_hi) load_item(p.items, id0, p.n_heads, it, ch);
    }
    if (ok && !withheld) {
        ItemView end_marker{};
        end_marker.end = 1;
        ok = producer_post(p, rg, &end_marker, false, nullptr, 0);
        issued += ok ? 1 : 0;
    }
    if (!ok) report(p.status, STATUS_EMPTY_WAIT_TIMEOUT);
    // Do not leave while a copy into this CTA's shared memory may still be in flight: wait
    // (bounded) for the completion of the last fills, newest NUM_STAGES at most.
    const uint32_t n_check = issued < (uint32_t)NUM_STAGES ? issued : (uint32_t)NUM_STAGES;
    for (uint32_t f = issued - n_check; f < issued; f++) {
        if (!mbar_wait_bounded(rg.full_bar + 8 * (f % NUM_STAGES), (f / NUM_STAGES) & 1, rg.wait_limit)) {
            report(p.status, STATUS_DRAIN_TIMEOUT);
            break;
        }
    }
}

// ---- consumers ---------------------------------------------------------------------------------------------
__device__ __forceinline__ bool consumer_wait_full(Ring& rg) {
    const long long t0 = rg.timed ? clock64() : 0;
    const bool ok = mbar_wait_bounded(rg.full_bar + 8 * rg.stage, rg.phase, rg.wait_limit);
    if (rg.timed) rg.wait_cycles += clock64() - t0;
    return __all_sync(0xffffffffu, ok);
}
__device__ __forceinline__ void consumer_release(Ring& rg, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(rg.empty_bar + 8 * rg.stage);
    rg.advance();
}

// Combine the warps' (max, sum, O[128]) of a ONE-row item and write its single partial.  Every
// warp has stored its state in its slot of the double-buffered scratch (buffer = item parity);
// one mbarrier phase per such item orders the stores before the loads, and because every warp
// waits for the phase, a warp can be at most one item ahead, so two buffers suffice.
__device__ __forceinline__ bool combine_row_and_store(const PartialParams& p, const ItemView& it, float* scratch,
                                                      uint32_t merge_bar, uint32_t& row_items, int warp, int lane,
                                                      Ring& rg) {
    const long long t0 = rg.timed ? clock64() : 0;
    __syncwarp();
    if (lane == 0) mbar_arrive(merge_bar);
    bool ok = mbar_wait_bounded(merge_bar, row_items & 1, rg.wait_limit);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) return false;
    {
        // warp w finishes outputs 32w .. 32w+31
        const float* base = scratch + (row_items & 1) * NUM_CONSUMER_WARPS * SCRATCH_FLOATS_PER_WARP;
        const int d = warp * 32 + lane;
        float mm = NEG_BIG;
#pragma unroll
        for (int w = 0; w < NUM_CONSUMER_WARPS; w++) mm = fmaxf(mm, base[w * SCRATCH_FLOATS_PER_WARP]);
        float ll = 0.f, od = 0.f;
#pragma unroll
        for (int w = 0; w < NUM_CONSUMER_WARPS; w++) {
            const float wl = base[w * SCRATCH_FLOATS_PER_WARP + 1];
            // a warp that saw no token keeps l = 0 and contributes nothing whatever its weight
            const float wgt = fast_exp2(base[w * SCRATCH_FLOATS_PER_WARP] - mm);
            ll = fmaf(wgt, wl, ll);
            od = fmaf(wgt, base[w * SCRATCH_FLOATS_PER_WARP + 4 + d], od);
        }
        p.part_o[(size_t)it.slot_base * FAST_D + d] = od;
        if (d == 0) p.part_ml[it.slot_base] = make_float2(mm, ll);
    }
    row_items++;
    if (rg.timed) rg.tail_cycles += clock64() - t0;
    return true;
}

// Tensor-core item.  The 4 warps form MT = 4 / TS row tiles of 16 rows times TS token splits; a
// warp owns 16 query rows and the TW = 64 / TS tokens [split * TW, ...) of every tile and keeps its
// own (max, sum, O) for the whole item:
//   TS = 4: up to 16 rows, 16 tokens per warp — chunk-first items of narrow runs AND a sequence's
//           private tail (one row).  Its queries arrive through shared memory with the first
//           tile; a partially filled tail tile is handled by masking the scores of absent tokens
//           and zeroing their V rows in the staged copy; a one-row item combines its 4 warps
//           through shared memory and writes a single partial.
//   TS = 2: up to 32 rows, 32 tokens per warp;   TS = 1: up to 64 rows, all 64 tokens.
//           Queries come straight from global memory; each warp writes its own partial rows.
template <int TS>
__device__ __forceinline__ bool mma_item(const PartialParams& p, const ItemView& it, Ring& rg, float* scratch,
                                         uint32_t merge_bar, uint32_t& row_items, int warp, int lane) {
    constexpr int MT = NUM_CONSUMER_WARPS / TS;
    constexpr int TW = FAST_C / TS;   // tokens per warp per tile
    constexpr int NT_S = TW / 8;      // 8-token column tiles of S
    constexpr bool STAGED_Q = (TS == NUM_CONSUMER_WARPS);
    const int mt = warp % MT;
    const int split = warp / MT;
    const int tok0 = split * TW;
    const int quad = lane & 3;
    const int r_lo = mt * 16 + (lane >> 2);
    const int r_hi = r_lo + 8;
    const bool v_lo = r_lo < it.n_rows;
    const bool v_hi = r_hi < it.n_rows;
    const int mi = lane >> 3;  // which of the four 8x8 matrices of an ldmatrix.x4 this lane addresses

    // Q as A fragments for the 8 k-steps over d_head; rows past the item are zero
    uint32_t qa[8][4];
    bool have_q = !STAGED_Q;
    if (!STAGED_Q) {
        const __half* q = reinterpret_cast<const __half*>(p.q);
        const size_t row_stride = (size_t)p.n_heads * FAST_D;
        const __half* q_lo = q + (size_t)(it.row_begin + r_lo) * row_stride + (size_t)it.head * FAST_D;
        const __half* q_hi = q + (size_t)(it.row_begin + r_hi) * row_stride + (size_t)it.head * FAST_D;
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
            const int col = ks * 16 + 2 * quad;
            qa[ks][0] = v_lo ? __ldg(reinterpret_cast<const uint32_t*>(q_lo + col)) : 0u;
            qa[ks][1] = v_hi ? __ldg(reinterpret_cast<const uint32_t*>(q_hi + col)) : 0u;
            qa[ks][2] = v_lo ? __ldg(reinterpret_cast<const uint32_t*>(q_lo + col + 8)) : 0u;
            qa[ks][3] = v_hi ? __ldg(reinterpret_cast<const uint32_t*>(q_hi + col + 8)) : 0u;
        }
    }

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; n++) {
        o[n][0] = 0.f; o[n][1] = 0.f; o[n][2] = 0.f; o[n][3] = 0.f;
    }
    float m_lo = NEG_BIG, m_hi = NEG_BIG, l_lo = 0.f, l_hi = 0.f;

    // per-lane row offsets for the two ldmatrix address patterns
    const int k_tok = (lane & 7) + ((mi >> 1) << 3);   // K: matrices 2,3 are the next 8 tokens
    const int k_gsel = mi & 1;                         //    matrices 1,3 are the next granule
    const int v_tok = (lane & 7) + ((mi & 1) << 3);    // V: matrices 1,3 are the next 8 tokens
    const int v_gsel = mi >> 1;                        //    matrices 2,3 are the next granule

    bool waited = true;  // the caller has waited for the item's first stage (it carried the description)
    for (int j = 0; j < it.n_tiles; j++) {
        const int nt = tile_tokens(it, j, p.delta_tokens);
        if (nt == 0) continue;  // an empty reserved tail: it occupies no stage
        if (!waited && !consumer_wait_full(rg)) return false;
        waited = false;
        const uint32_t kbase = rg.ring + rg.stage * FAST_STAGE_BYTES;
        const uint32_t vbase = kbase + FAST_TILE_BYTES;
        if (STAGED_Q && !have_q) {
            // The producer staged this item's query rows next to its first non-empty tile, in the
            // slot of that tile's stage; they arrived with it.  Copy them to registers as the A
            // fragments of the 8 k-steps before this stage is released.
            const uint32_t qrow = rg.qslots + rg.stage * QSLOT_BYTES + ((lane & 7) + (mi & 1) * 8) * QSLOT_PITCH + (mi >> 1) * 16;
#pragma unroll
            for (int ks = 0; ks < 8; ks++) {
                ldsm_x4(qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], qrow + ks * 32);
                // rows past the item hold stale bytes: make them exact zeros
                if (!v_lo) { qa[ks][0] = 0u; qa[ks][2] = 0u; }
                if (!v_hi) { qa[ks][1] = 0u; qa[ks][3] = 0u; }
            }
            have_q = true;
        }
        // only a private tail (a one-row item, TS = 4) can be partially filled
        if (STAGED_Q && tok0 >= nt) {
            // none of this warp's tokens exists in the tile: its state stays as it is
            consumer_release(rg, lane);
            continue;
        }
        const bool partial = STAGED_Q && (tok0 + TW > nt);
        if (partial) {
            // Absent tokens: the bulk copy did not fill their rows, so they hold stale bytes.  Their
            // scores are masked below; their V rows are zeroed here because 0 * NaN is NaN.
            const int first_absent = nt > tok0 ? nt : tok0;
            for (int idx = lane; idx < (tok0 + TW - first_absent) * 16; idx += 32)
                sts128_zero(vbase + tile_off(first_absent + (idx >> 4), idx & 15));
            __syncwarp();
        }

        // S = Q K^T for this warp's TW tokens.  The 8 k-steps over d_head are spread over KG
        // independent accumulator sets (summed afterwards) so that narrow warp slices do not
        // serialise on the latency of 8 dependent MMAs.
        constexpr int KG = NT_S >= 8 ? 1 : (NT_S >= 4 ? 2 : 4);
        float sg[KG][NT_S][4];
#pragma unroll
        for (int kg = 0; kg < KG; kg++)
#pragma unroll
            for (int n = 0; n < NT_S; n++) {
                sg[kg][n][0] = 0.f; sg[kg][n][1] = 0.f; sg[kg][n][2] = 0.f; sg[kg][n][3] = 0.f;
            }
#pragma unroll
        for (int ks = 0; ks < 8; ks++) {
#pragma unroll
            for (int np = 0; np < NT_S / 2; np++) {
                const int t = tok0 + np * 16 + k_tok;
                const int g = 2 * ks + k_gsel;
                uint32_t b0, b1, b2, b3;
                ldsm_x4(b0, b1, b2, b3, kbase + tile_off(t, g));
                mma_16816(sg[ks % KG][2 * np], qa[ks], b0, b1);
                mma_16816(sg[ks % KG][2 * np + 1], qa[ks], b2, b3);
            }
        }
        float s[NT_S][4];
#pragma unroll
        for (int n = 0; n < NT_S; n++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float acc = sg[0][n][c];
#pragma unroll
                for (int kg = 1; kg < KG; kg++) acc += sg[kg][n][c];
                s[n][c] = acc;
            }
        if (partial) {
            // column c of 8-token tile n is token tok0 + 8n + 2*quad + (c & 1)
#pragma unroll
            for (int n = 0; n < NT_S; n++) {
                const int t = tok0 + 8 * n + 2 * quad;
                if (t >= nt) { s[n][0] = NEG_BIG; s[n][2] = NEG_BIG; }
                if (t + 1 >= nt) { s[n][1] = NEG_BIG; s[n][3] = NEG_BIG; }
            }
        }

        // online softmax in log2 units; a thread holds rows r_lo (c0, c1) and r_hi (c2, c3)
        float mx_lo = NEG_BIG, mx_hi = NEG_BIG;
#pragma unroll
        for (int n = 0; n < NT_S; n++) {
            mx_lo = fmaxf(mx_lo, fmaxf(s[n][0], s[n][1]));
            mx_hi = fmaxf(mx_hi, fmaxf(s[n][2], s[n][3]));
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        // a warp whose tokens are all absent keeps its state (masked scores must not set the maximum)
        const float mn_lo = fmaxf(m_lo, mx_lo > 0.5f * NEG_BIG ? mx_lo * p.scale_log2 : NEG_BIG);
        const float mn_hi = fmaxf(m_hi, mx_hi > 0.5f * NEG_BIG ? mx_hi * p.scale_log2 : NEG_BIG);
        const float a_lo = fast_exp2(m_lo - mn_lo);
        const float a_hi = fast_exp2(m_hi - mn_hi);
        m_lo = mn_lo;
        m_hi = mn_hi;
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t pa[TW / 16][4];
#pragma unroll
        for (int n = 0; n < NT_S; n++) {
            float p0 = fast_exp2(fmaf(s[n][0], p.scale_log2, -mn_lo));
            float p1 = fast_exp2(fmaf(s[n][1], p.scale_log2, -mn_lo));
            float p2 = fast_exp2(fmaf(s[n][2], p.scale_log2, -mn_hi));
            float p3 = fast_exp2(fmaf(s[n][3], p.scale_log2, -mn_hi));
            if (partial) {
                const int t = tok0 + 8 * n + 2 * quad;
                if (t >= nt) { p0 = 0.f; p2 = 0.f; }
                if (t + 1 >= nt) { p1 = 0.f; p3 = 0.f; }
            }
            sum_lo += p0 + p1;
            sum_hi += p2 + p3;
            // the accumulator layout of two adjacent 8-token tiles is the A layout of one k-step
            pa[n >> 1][(n & 1) * 2 + 0] = pack_half2(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2, p3);
        }
        l_lo = l_lo * a_lo + sum_lo;
        l_hi = l_hi * a_hi + sum_hi;
        // once the running maxima have settled the factors are exactly 1: skip the 64 multiplies
        if (__any_sync(0xffffffffu, a_lo != 1.f || a_hi != 1.f)) {
#pragma unroll
            for (int n = 0; n < 16; n++) {
                o[n][0] *= a_lo; o[n][1] *= a_lo; o[n][2] *= a_hi; o[n][3] *= a_hi;
            }
        }

        // O += P V
#pragma unroll
        for (int kk = 0; kk < TW / 16; kk++) {
#pragma unroll
            for (int dp = 0; dp < 8; dp++) {
                const int t = tok0 + kk * 16 + v_tok;
                const int g = 2 * dp + v_gsel;
                uint32_t b0, b1, b2, b3;
                ldsm_x4_trans(b0, b1, b2, b3, vbase + tile_off(t, g));
                mma_16816(o[2 * dp], pa[kk], b0, b1);
                mma_16816(o[2 * dp + 1], pa[kk], b2, b3);
            }
        }
        if (partial) fence_proxy_async();
        consumer_release(rg, lane);
    }

    if (waited) consumer_release(rg, lane);  // the item held no token: its first stage was empty
    // the four lanes of a quad hold partial sums of the same two rows
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    if (STAGED_Q && it.n_rows == 1) {
        if (!have_q) {
            // the item held no token at all (an empty reserved tail): mark its partial as empty
            if (warp == 0 && lane == 0) p.part_ml[it.slot_base] = make_float2(NEG_BIG, 0.f);
            return true;
        }
        // row 0 lives in the first quad: lane q holds outputs 8n + 2q, 8n + 2q + 1
        float* mine = scratch + ((row_items & 1) * NUM_CONSUMER_WARPS + warp) * SCRATCH_FLOATS_PER_WARP;
        if (lane == 0) {
            mine[0] = m_lo;
            mine[1] = l_lo;
        }
        if (lane < 4) {
#pragma unroll
            for (int n = 0; n < 16; n++)
                *reinterpret_cast<float2*>(mine + 4 + 8 * n + 2 * quad) = make_float2(o[n][0], o[n][1]);
        }
        return combine_row_and_store(p, it, scratch, merge_bar, row_items, warp, lane, rg);
    }
    // rows of one head are n_heads slots apart
    const int slot_lo = it.slot_base + (split * it.n_rows + r_lo) * p.n_heads;
    const int slot_hi = it.slot_base + (split * it.n_rows + r_hi) * p.n_heads;
    if (v_lo) {
        float* dst = p.part_o + (size_t)slot_lo * FAST_D + 2 * quad;
#pragma unroll
        for (int n = 0; n < 16; n++) *reinterpret_cast<float2*>(dst + 8 * n) = make_float2(o[n][0], o[n][1]);
        if (quad == 0) p.part_ml[slot_lo] = make_float2(m_lo, l_lo);
    }
    if (v_hi) {
        float* dst = p.part_o + (size_t)slot_hi * FAST_D + 2 * quad;
#pragma unroll
        for (int n = 0; n < 16; n++) *reinterpret_cast<float2*>(dst + 8 * n) = make_float2(o[n][2], o[n][3]);
        if (quad == 0) p.part_ml[slot_hi] = make_float2(m_hi, l_hi);
    }
    return true;
}

// Sequence-first item on CUDA cores (selectable alternative to the tensor-core walk).  Warp w owns
// tokens 16w..16w+15 of every tile; a half-warp reads one 256-byte token row per 128-bit load
// (lane = granule), so K rows are dotted against q held in registers and V rows are accumulated
// into 8 output elements per lane.  The warps' states are combined through shared memory at the
// end of the item and one partial is written.
__device__ __forceinline__ bool simt_item(const PartialParams& p, const ItemView& it, Ring& rg, float* scratch,
                                          uint32_t merge_bar, uint32_t& row_items, int warp, int lane) {
    constexpr int TPW = FAST_C / NUM_CONSUMER_WARPS;  // tokens per warp per tile
    constexpr int NJ = TPW / 2;                       // a warp reads two token rows per load
    const int g = lane & 15;
    const int half = lane >> 4;
    float qf[8];
    {
        const __half* q = reinterpret_cast<const __half*>(p.q) +
                          ((size_t)it.row_begin * p.n_heads + it.head) * FAST_D + 8 * g;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(q));
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(h[i]);
            qf[2 * i] = f.x * p.scale_log2;
            qf[2 * i + 1] = f.y * p.scale_log2;
        }
    }
    float m = NEG_BIG, l = 0.f;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] = 0.f;

    bool waited = true;  // the caller has waited for the item's first stage (it carried the description)
    for (int j = 0; j < it.n_tiles; j++) {
        const int nt = tile_tokens(it, j, p.delta_tokens);
        if (nt == 0) continue;
        if (!waited && !consumer_wait_full(rg)) return false;
        waited = false;
        if (warp * TPW < nt) {
            const uint32_t kt = rg.ring + rg.stage * FAST_STAGE_BYTES;
            const uint32_t vt = kt + FAST_TILE_BYTES;
            float s[NJ];
#pragma unroll
            for (int jj = 0; jj < NJ; jj++) {
                const int t = warp * TPW + 2 * jj + half;
                float acc = 0.f;
                if (t < nt) {
                    const uint4 raw = lds128(kt + tile_off(t, g));
                    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(h[i]);
                        acc = fmaf(qf[2 * i], f.x, acc);
                        acc = fmaf(qf[2 * i + 1], f.y, acc);
                    }
                }
                s[jj] = acc;
            }
            // sum over the 16 lanes of a half-warp (the 16 granules of a token row)
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) {
#pragma unroll
                for (int jj = 0; jj < NJ; jj++) s[jj] += __shfl_xor_sync(0xffffffffu, s[jj], off);
            }
            float mx = NEG_BIG;
#pragma unroll
            for (int jj = 0; jj < NJ; jj++) {
                const int t = warp * TPW + 2 * jj + half;
                if (t < nt) mx = fmaxf(mx, s[jj]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
            const float mn = fmaxf(m, mx);
            const float alpha = fast_exp2(m - mn);
            m = mn;
            l *= alpha;
#pragma unroll
            for (int i = 0; i < 8; i++) o[i] *= alpha;
#pragma unroll
            for (int jj = 0; jj < NJ; jj++) {
                const int t = warp * TPW + 2 * jj + half;
                if (t < nt) {
                    const float pj = fast_exp2(s[jj] - mn);
                    l += pj;
                    const uint4 raw = lds128(vt + tile_off(t, g));
                    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(h[i]);
                        o[2 * i] = fmaf(pj, f.x, o[2 * i]);
                        o[2 * i + 1] = fmaf(pj, f.y, o[2 * i + 1]);
                    }
                }
            }
        }
        consumer_release(rg, lane);
    }

    if (waited) consumer_release(rg, lane);  // the item held no token: its first stage was empty
    // the two half-warps walked different tokens against the same running max
    l += __shfl_xor_sync(0xffffffffu, l, 16);
#pragma unroll
    for (int i = 0; i < 8; i++) o[i] += __shfl_xor_sync(0xffffffffu, o[i], 16);

    // lanes 0..15 of a warp hold the warp's 128 outputs, 8 each
    float* mine = scratch + ((row_items & 1) * NUM_CONSUMER_WARPS + warp) * SCRATCH_FLOATS_PER_WARP;
    if (lane == 0) {
        mine[0] = m;
        mine[1] = l;
    }
    if (lane < 16) {
        *reinterpret_cast<float4*>(mine + 4 + 8 * g) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(mine + 8 + 8 * g) = make_float4(o[4], o[5], o[6], o[7]);
    }
    return combine_row_and_store(p, it, scratch, merge_bar, row_items, warp, lane, rg);
}

__global__ void __launch_bounds__(NUM_THREADS, 2) attn_partial_kernel(const PartialParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    float* scratch = reinterpret_cast<float*>(smem + SMEM_SCRATCH_OFFSET);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BAR_OFFSET);

    Ring rg;
    rg.ring = smem_u32(smem);
    rg.qslots = smem_u32(smem + SMEM_Q_OFFSET);
    rg.full_bar = smem_u32(bars);
    rg.empty_bar = smem_u32(bars + NUM_STAGES);
    rg.stage = 0;
    rg.phase = 0;
    rg.wait_limit = p.wait_limit;
    rg.timed = p.trace != nullptr;
    rg.wait_cycles = 0;
    rg.tail_cycles = 0;
    const long long t_begin = rg.timed ? clock64() : 0;
    const uint32_t merge_bar = smem_u32(bars + 2 * NUM_STAGES);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NUM_STAGES; i++) {
            mbar_init(rg.full_bar + 8 * i, 1);
            mbar_init(rg.empty_bar + 8 * i, NUM_CONSUMER_WARPS);
        }
        mbar_init(merge_bar, NUM_CONSUMER_WARPS);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    // no block-wide barrier below this line: the warps run decoupled
    // Launched as a programmatic dependent of whatever precedes it in the stream, the CTA has set
    // itself up while that kernel was finishing; nothing in global memory has been touched so far.
    // Every thread waits here until the predecessor's writes (queries, appended K/V rows, the
    // previous step's merge still reading the partial buffers) are complete and visible.  A no-op
    // for an ordinary launch.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // let the merge kernel (a programmatic dependent launch) be scheduled as soon as SMs drain
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // the launch after this one draws from the other counter: zero it now (launches are stream-ordered)
    if (blockIdx.x == 0 && threadIdx.x == 0) *p.counter_next = 0;

    if (p.trace && threadIdx.x == 0) p.trace[8 * blockIdx.x + 0] = global_timer_ns();
    if (warp >= NUM_CONSUMER_WARPS) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
        if (warp == NUM_CONSUMER_WARPS && lane == 0) {
            producer_loop(p, rg);
            if (p.trace) {
                p.trace[8 * blockIdx.x + 1] = global_timer_ns();
                p.trace[8 * blockIdx.x + 6] = (unsigned long long)rg.wait_cycles;
            }
        }
        return;
    }
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(CONSUMER_REGS));

    uint32_t row_items = 0;  // one-row items finished so far (scratch buffer and merge-barrier parity)
    while (true) {
        // the next item announces itself with its first stage
        if (!consumer_wait_full(rg)) {
            if (lane == 0) report(p.status, STATUS_FULL_WAIT_TIMEOUT);
            break;
        }
        const uint32_t da = desc_addr(rg, rg.stage);
        const uint4 d0 = lds128(da);
        const uint4 d1 = lds128(da + QSLOT_PITCH);
        const ItemView it{(int)d0.x, (int)d0.y, (int)d0.z, (int)d0.w, (int)d1.x, (int)d1.y, (int)d1.z, (int)d1.w};
        if (it.end) {
            consumer_release(rg, lane);
            break;
        }
        const int splits = it.flags >> ITEM_SPLITS_SHIFT;
        bool ok;
        if (splits == 4) {
            ok = mma_item<4>(p, it, rg, scratch, merge_bar, row_items, warp, lane);
        } else if (splits == 0) {
            ok = simt_item(p, it, rg, scratch, merge_bar, row_items, warp, lane);
        } else if (splits == 2) {
            ok = mma_item<2>(p, it, rg, scratch, merge_bar, row_items, warp, lane);
        } else {
            ok = mma_item<1>(p, it, rg, scratch, merge_bar, row_items, warp, lane);
        }
        if (!ok) {
            if (lane == 0) report(p.status, STATUS_FULL_WAIT_TIMEOUT);
            break;
        }
    }
    if (p.trace && lane == 0 && (warp == 0 || warp == NUM_CONSUMER_WARPS - 1)) {
        p.trace[8 * blockIdx.x + (warp == 0 ? 2 : 3)] = global_timer_ns();
        if (warp == 0) {
            p.trace[8 * blockIdx.x + 4] = (unsigned long long)rg.wait_cycles;
            p.trace[8 * blockIdx.x + 5] = (unsigned long long)rg.tail_cycles;
            p.trace[8 * blockIdx.x + 7] = (unsigned long long)(clock64() - t_begin);
        }
    }
}

// One warp per (row, head): out = sum_i 2^(m_i - M) O_i / sum_i 2^(m_i - M) l_i.
// The kernel is a chain of dependent lookups (list bounds -> slot numbers -> max and sum -> O rows),
// so it is organised to pay each round trip once: a lane looks up one partial's slot, max and sum
// (32 partials per pass, usually all of them), the maximum is found with shuffles, and the O rows
// are then fetched eight at a time with the slot numbers passed around by shuffles.
// FIRST: O rows requested ahead of the weights (registers: 4 per row).  Three instances, chosen so that
// the whole grid is resident at once: 16 rows ahead (3 CTAs per SM), 8 ahead (5 per SM), none ahead
// (two round trips, 72 registers, 7 per SM) for large batches, where a second wave of CTAs would cost
// more than the round trip saved.
// ---- short private tails ---------------------------------------------------------------------------------
// A (sequence, head) whose private part is a single, usually partly filled, chunk is too small an item
// for the persistent kernel (an item costs its warps the same whatever it holds).  When a batch has
// many of them the planner puts them at the end of the item list and this kernel walks them instead:
// one HALF-WARP per item, straight from global memory, eight tokens per round with all of a round's loads
// (K rows and V rows) issued before any is used, so a tail of up to eight tokens costs one round trip after
// the item's description.  Lane g of the half-warp owns granule g of every row: 16 bytes of each K row (the
// products are summed over the 16 lanes with shuffles, which leaves every lane with every score, so the
// softmax needs no further exchange) and 16 bytes = 8 output elements of each V row.  The result is an
// ordinary partial (max and sum in log2 units, un-normalised O), combined with the row's other partials by
// the merge kernel.
// FINISH: when EVERY row of the batch has such a tail (many requests with short suffixes over shared prompts) the
// kernel runs LAST in the step and finishes the rows itself: the half-warp keeps its partial in registers, fetches
// the row's other partials (the shared runs', written by the kernels before it), combines, normalises and stores the
// fp16 output row — the tail's partial never travels through memory and the merge kernel is not launched.
__device__ __forceinline__ int checked_slot(const MergeParams& p, int entry, int head);
__device__ __forceinline__ void checked_bounds(const MergeParams& p, int& b, int& e);
__device__ __forceinline__ void store_row8(const MergeParams& p, int row, int head, int g, const float (&o)[8], float inv);

constexpr int SHORT_WARPS = 4;   // small CTAs: they fit beside the wide-runs kernel's CTAs when the two overlap
constexpr int SHORT_ITEMS_PER_CTA = 2 * SHORT_WARPS;
constexpr int SHORT_BLOCK = 8;   // tokens per round

template <bool FINISH>
__global__ void __launch_bounds__(SHORT_WARPS * 32, 4) attn_short_tails_kernel(const PartialParams p, const MergeParams mp) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane & 15, half = lane >> 4;
    const int vid = p.item_lo + ((int)blockIdx.x * SHORT_WARPS + warp) * 2 + half;  // work piece = (item, head)
    // every lane runs every round (the shuffles below need the whole warp); a half-warp without an item, or with a
    // rejected one, simply has no tokens
    int nt = 0, row = 0, head = 0, chunk = 0, slot = -1;
    if (vid < p.item_hi) {
        const int idx = vid / p.n_heads;
        head = vid - idx * p.n_heads;
        const int4 d0 = __ldg(p.items + 4 * idx), d1 = __ldg(p.items + 4 * idx + 1);
        row = d0.z;
        chunk = d1.w;
        slot = d1.x * p.n_heads + head;
        if (row < 0 || d1.x < 0 || chunk < 0 || d1.z < 0 || (p.n_slots > 0 && slot >= p.n_slots) ||
            (p.n_seqs > 0 && row >= p.n_seqs) || (p.max_chunks > 0 && chunk >= p.max_chunks)) {
            if (g == 0) report(p.status, STATUS_BAD_WORK_LIST);  // skipped
            slot = -1;
        } else {
            nt = min(FAST_C, d1.z + ((d1.y & ITEM_FLAG_TAIL) ? p.delta_tokens : 0));
        }
    }
    const int nt_warp = max(nt, __shfl_xor_sync(0xffffffffu, nt, 16));
    // FINISH: where the row's other partials are is looked up now, in the shadow of the tail's own loads
    constexpr int AHEAD = 4;   // lists of up to four other pieces cost one round trip after the tail
    int lb = 0, le = 0, sl[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; u++) sl[u] = -1;
    if (FINISH && slot >= 0) {
        lb = __ldg(mp.merge_off + row);
        le = __ldg(mp.merge_off + row + 1);
        checked_bounds(mp, lb, le);
#pragma unroll
        for (int u = 0; u < AHEAD; u++)
            if (lb + u < le) sl[u] = __ldg(mp.merge_slots + lb + u);   // entries; checked when they are used
    }
    const uint8_t* ktile = p.pool + ((size_t)chunk * p.n_heads + head) * (size_t)FAST_STAGE_BYTES;
    const uint8_t* vtile = ktile + FAST_TILE_BYTES;
    uint4 qraw = make_uint4(0u, 0u, 0u, 0u);
    if (nt > 0)
        qraw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p.q) + ((size_t)row * p.n_heads + head) * FAST_D + 8 * g));
    float qf[8];
    float m = NEG_BIG, l = 0.f;
    float o[8];
#pragma unroll
    for (int e = 0; e < 8; e++) o[e] = 0.f;
    for (int t0 = 0; t0 < nt_warp; t0 += SHORT_BLOCK) {
        uint4 kr[SHORT_BLOCK], vr[SHORT_BLOCK];
#pragma unroll
        for (int i = 0; i < SHORT_BLOCK; i++) {
            kr[i] = make_uint4(0u, 0u, 0u, 0u);
            vr[i] = make_uint4(0u, 0u, 0u, 0u);
            if (t0 + i < nt) {
                kr[i] = __ldg(reinterpret_cast<const uint4*>(ktile + tile_off(t0 + i, g)));
                vr[i] = __ldg(reinterpret_cast<const uint4*>(vtile + tile_off(t0 + i, g)));
            }
        }
        if (t0 == 0) {  // the query granule of this lane, pre-scaled to log2 units
            const __half2* h = reinterpret_cast<const __half2*>(&qraw);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float2 f = __half22float2(h[k]);
                qf[2 * k] = f.x * p.scale_log2;
                qf[2 * k + 1] = f.y * p.scale_log2;
            }
        }
        const int n_here = min(SHORT_BLOCK, nt_warp - t0);  // warp-uniform: rounds are cut short together
        float sc[SHORT_BLOCK];
        float mx = NEG_BIG;
#pragma unroll
        for (int i = 0; i < SHORT_BLOCK; i++) {
            sc[i] = NEG_BIG;
            if (i < n_here) {
                const __half2* h = reinterpret_cast<const __half2*>(&kr[i]);
                float a = 0.f;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    const float2 f = __half22float2(h[k]);
                    a = fmaf(qf[2 * k], f.x, a);
                    a = fmaf(qf[2 * k + 1], f.y, a);
                }
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
                if (t0 + i < nt) sc[i] = a;
                mx = fmaxf(mx, sc[i]);
            }
        }
        if (t0 < nt) {  // this half-warp's item still has tokens in the round
            const float mn = fmaxf(m, mx);
            const float alpha = fast_exp2(m - mn);
            m = mn;
            l *= alpha;
#pragma unroll
            for (int e = 0; e < 8; e++) o[e] *= alpha;
#pragma unroll
            for (int i = 0; i < SHORT_BLOCK; i++) {
                if (i < n_here) {
                    const float pw = t0 + i < nt ? fast_exp2(sc[i] - mn) : 0.f;
                    l += pw;
                    const __half2* h = reinterpret_cast<const __half2*>(&vr[i]);
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const float2 f = __half22float2(h[k]);
                        o[2 * k] = fmaf(pw, f.x, o[2 * k]);
                        o[2 * k + 1] = fmaf(pw, f.y, o[2 * k + 1]);
                    }
                }
            }
        }
    }
    if (slot < 0) return;
    if (!FINISH) {
        if (nt > 0) {
            float4* dst = reinterpret_cast<float4*>(p.part_o + (size_t)slot * FAST_D + 8 * g);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
        }
        if (g == 0) p.part_ml[slot] = make_float2(nt > 0 ? m : NEG_BIG, l);  // an empty reserved tail: (none, 0)
        return;
    }
    // ---- the row's other partials (no shuffles from here on: half-warps proceed on their own)
    if (nt == 0) m = NEG_BIG;
    for (int b = lb; b < le; b += AHEAD) {
        if (b > lb) {
#pragma unroll
            for (int u = 0; u < AHEAD; u++) sl[u] = b + u < le ? __ldg(mp.merge_slots + b + u) : -1;
        }
        float2 ml[AHEAD];
        float4 v[AHEAD][2];
#pragma unroll
        for (int u = 0; u < AHEAD; u++) {
            ml[u] = make_float2(NEG_BIG, 0.f);
            v[u][0] = v[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b + u < le) {
                const int s = checked_slot(mp, sl[u], head);
                if (s >= 0 && s != slot) {   // this half-warp's own piece is in its registers
                    ml[u] = mp.part_ml[s];
                    const float4* src = reinterpret_cast<const float4*>(mp.part_o + (size_t)s * FAST_D + 8 * g);
                    v[u][0] = src[0];
                    v[u][1] = src[1];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < AHEAD; u++) {
            if (!(ml[u].y > 0.f)) continue;   // no piece, this half-warp's own, or one without tokens (it has no O row)
            const float mn = fmaxf(m, ml[u].x);
            const float a = fast_exp2(m - mn), w = fast_exp2(ml[u].x - mn);
            m = mn;
            l = l * a + ml[u].y * w;
            o[0] = o[0] * a + v[u][0].x * w;
            o[1] = o[1] * a + v[u][0].y * w;
            o[2] = o[2] * a + v[u][0].z * w;
            o[3] = o[3] * a + v[u][0].w * w;
            o[4] = o[4] * a + v[u][1].x * w;
            o[5] = o[5] * a + v[u][1].y * w;
            o[6] = o[6] * a + v[u][1].z * w;
            o[7] = o[7] * a + v[u][1].w * w;
        }
    }
    store_row8(mp, row, head, g, o, l > 0.f ? 1.f / l : 0.f);  // a row with no token yields zeros
}

// The un-normalised combination of the partials merge_slots[b .. e) by one warp: on return mm is their
// maximum, acc this lane's four output elements weighted by 2^(m_i - mm), ll the warp-wide sum of the
// weighted sums.  slot0: this lane's slot among the first 32 (-1: none), read by the caller.
// A slot number from a merge list, or -1 (and the status word set) when it lies outside the partial rows.
// `entry` numbers a partial row per head-agnostic item; head h's copy of it is slot entry * n_heads + h.
__device__ __forceinline__ int checked_slot(const MergeParams& p, int entry, int head) {
    const long long slot = (long long)entry * p.n_heads + head;
    if (entry < 0 || (p.n_slots > 0 && slot >= p.n_slots)) {
        if (p.status) atomicCAS(p.status, STATUS_OK, STATUS_BAD_WORK_LIST);
        return -1;
    }
    return (int)slot;
}
// The bounds [b, e) of a pair's list inside merge_slots; an impossible pair of offsets yields an empty list.
__device__ __forceinline__ void checked_bounds(const MergeParams& p, int& b, int& e) {
    if (p.n_merge_entries > 0 && (b < 0 || e < b || e > p.n_merge_entries)) {
        if (p.status) atomicCAS(p.status, STATUS_OK, STATUS_BAD_WORK_LIST);
        b = e = 0;
    }
}

template <int FIRST>
__device__ __forceinline__ void merge_list(const MergeParams& p, int lane, int head, int b, int e, int slot0, float& mm,
                                           float& ll, float4& acc) {
    // The first 32 partials stay in registers; longer lists are re-read pass by pass.  The O rows of
    // the first 16 partials are requested together with the (max, sum) pairs, before the weights are
    // known, so the usual row (a dozen partials) costs ONE round trip after the wait instead of two;
    // a partial without tokens has no O row (its slot holds stale data), so its row is discarded by
    // a select, not by a multiplication with zero.
    float2 ml0 = make_float2(NEG_BIG, 0.f);
    if (slot0 >= 0) ml0 = p.part_ml[slot0];
    float4 v0[FIRST > 0 ? FIRST : 1];
    if (FIRST > 0) {
        const int n0 = min(FIRST, e - b);
#pragma unroll
        for (int u = 0; u < FIRST; u++) {
            const int sk = __shfl_sync(0xffffffffu, slot0, u);
            v0[u] = (u < n0 && sk >= 0) ? *reinterpret_cast<const float4*>(p.part_o + (size_t)sk * FAST_D + 4 * lane)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    mm = ml0.y > 0.f ? ml0.x : NEG_BIG;
    for (int i = b + 32 + lane; i < e; i += 32) {
        const int si = checked_slot(p, __ldg(p.merge_slots + i), head);
        if (si < 0) continue;
        const float2 ml = p.part_ml[si];
        if (ml.y > 0.f) mm = fmaxf(mm, ml.x);
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));

    acc = make_float4(0.f, 0.f, 0.f, 0.f);
    ll = 0.f;
    for (int base = b; base < e; base += 32) {
        int slot = slot0;
        float2 ml = ml0;
        if (base != b) {
            slot = -1;
            ml = make_float2(NEG_BIG, 0.f);
            if (base + lane < e) {
                slot = checked_slot(p, __ldg(p.merge_slots + base + lane), head);
                if (slot >= 0) ml = p.part_ml[slot];
            }
        }
        float w = 0.f;
        if (ml.y > 0.f) {  // an empty piece has no O row
            w = fast_exp2(ml.x - mm);
            ll = fmaf(w, ml.y, ll);
        } else {
            slot = -1;
        }
        const int n = min(32, e - base);
        int k_begin = 0;
        if (FIRST > 0 && base == b) {  // the rows requested ahead
#pragma unroll
            for (int u = 0; u < FIRST; u++) {
                const float wu = __shfl_sync(0xffffffffu, w, u);
                const bool live = wu != 0.f;
                acc.x = fmaf(wu, live ? v0[u].x : 0.f, acc.x);
                acc.y = fmaf(wu, live ? v0[u].y : 0.f, acc.y);
                acc.z = fmaf(wu, live ? v0[u].z : 0.f, acc.z);
                acc.w = fmaf(wu, live ? v0[u].w : 0.f, acc.w);
            }
            k_begin = FIRST;
        }
        for (int k0 = k_begin; k0 < n; k0 += 8) {
            float4 v[8];
            float wk[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int sk = __shfl_sync(0xffffffffu, slot, (k0 + u) & 31);
                wk[u] = __shfl_sync(0xffffffffu, w, (k0 + u) & 31);
                const bool live = (k0 + u < n) && sk >= 0;
                if (!live) wk[u] = 0.f;
                v[u] = live ? *reinterpret_cast<const float4*>(p.part_o + (size_t)sk * FAST_D + 4 * lane)
                            : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                acc.x = fmaf(wk[u], v[u].x, acc.x);
                acc.y = fmaf(wk[u], v[u].y, acc.y);
                acc.z = fmaf(wk[u], v[u].z, acc.z);
                acc.w = fmaf(wk[u], v[u].w, acc.w);
            }
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
}

// fp16 output row of a pair: to `out`, or into every rank's full-width buffer
__device__ __forceinline__ void store_row(const MergeParams& p, int pair, int lane, const float4& acc, float inv) {
    const __half2 h01 = __floats2half2_rn(acc.x * inv, acc.y * inv);
    const __half2 h23 = __floats2half2_rn(acc.z * inv, acc.w * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t*>(&h01);
    packed.y = *reinterpret_cast<const uint32_t*>(&h23);
    if (p.n_peers == 0) {
        *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + (size_t)pair * FAST_D + 4 * lane) = packed;
    } else {
        // head-sharded: the row goes into every rank's full-width output
        const int row = pair / p.n_heads;
        const int head = pair - row * p.n_heads;
        const size_t off = ((size_t)row * p.total_heads + p.head_offset + head) * FAST_D + 4 * lane;
        if (p.mc_out) {
            // one store to the multicast address: the switch replicates it into every rank's buffer
            asm volatile("multimem.st.weak.global.v2.f16x2 [%0], {%1, %2};" ::"l"(reinterpret_cast<__half*>(p.mc_out) + off),
                         "r"(packed.x), "r"(packed.y)
                         : "memory");
        } else {
            // plain stores to peer memory over NVLink
#pragma unroll
            for (int i = 0; i < MERGE_MAX_PEERS; i++)
                if (i < p.n_peers) *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.peer_out[i]) + off) = packed;
        }
    }
}

// The same for a lane that owns eight consecutive output elements (granule g of the row)
__device__ __forceinline__ void store_row8(const MergeParams& p, int row, int head, int g, const float (&o)[8], float inv) {
    uint4 packed;
    packed.x = pack_half2(o[0] * inv, o[1] * inv);
    packed.y = pack_half2(o[2] * inv, o[3] * inv);
    packed.z = pack_half2(o[4] * inv, o[5] * inv);
    packed.w = pack_half2(o[6] * inv, o[7] * inv);
    if (p.n_peers == 0) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + ((size_t)row * p.n_heads + head) * FAST_D + 8 * g) = packed;
    } else {
        const size_t off = ((size_t)row * p.total_heads + p.head_offset + head) * FAST_D + 8 * g;
        if (p.mc_out) {
            asm volatile("multimem.st.weak.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(reinterpret_cast<__half*>(p.mc_out) + off),
                         "r"(packed.x), "r"(packed.y), "r"(packed.z), "r"(packed.w)
                         : "memory");
        } else {
#pragma unroll
            for (int i = 0; i < MERGE_MAX_PEERS; i++)
                if (i < p.n_peers) *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.peer_out[i]) + off) = packed;
        }
    }
}

// Large batches whose rows have at most four pieces each (one long shared prefix plus a short private tail, the
// usual serving shape): eight lanes per (row, head), each owning 16 output elements, every piece's (max, sum)
// and O segment requested at once, so the whole combination is one round trip after the list lookups and a warp
// finishes four pairs instead of one.
constexpr int SMALL_MAX_LIST = 4;
__global__ void __launch_bounds__(128) attn_merge_small_kernel(const MergeParams p) {
    const int pair = blockIdx.x * 16 + (threadIdx.x >> 3);
    const int sub = threadIdx.x & 7;
    int slot[SMALL_MAX_LIST];
#pragma unroll
    for (int u = 0; u < SMALL_MAX_LIST; u++) slot[u] = -1;
    if (pair < p.n_pairs) {
        const int row = pair / p.n_heads, head = pair - row * p.n_heads;
        int b = __ldg(p.merge_off + row), e = __ldg(p.merge_off + row + 1);
        checked_bounds(p, b, e);
#pragma unroll
        for (int u = 0; u < SMALL_MAX_LIST; u++)
            if (b + u < e) slot[u] = checked_slot(p, __ldg(p.merge_slots + b + u), head);
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (pair >= p.n_pairs) return;
    float2 ml[SMALL_MAX_LIST];
    float4 v[SMALL_MAX_LIST][4];
#pragma unroll
    for (int u = 0; u < SMALL_MAX_LIST; u++) {
        ml[u] = make_float2(NEG_BIG, 0.f);
#pragma unroll
        for (int k = 0; k < 4; k++) v[u][k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (slot[u] >= 0) {
            ml[u] = p.part_ml[slot[u]];
            const float4* src = reinterpret_cast<const float4*>(p.part_o + (size_t)slot[u] * FAST_D + 16 * sub);
#pragma unroll
            for (int k = 0; k < 4; k++) v[u][k] = src[k];
        }
    }
    float mm = NEG_BIG;
#pragma unroll
    for (int u = 0; u < SMALL_MAX_LIST; u++)
        if (ml[u].y > 0.f) mm = fmaxf(mm, ml[u].x);
    float ll = 0.f;
    float4 o[4];
#pragma unroll
    for (int k = 0; k < 4; k++) o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int u = 0; u < SMALL_MAX_LIST; u++) {
        if (ml[u].y > 0.f) {  // a piece without tokens has no O row: its slot holds stale data
            const float w = fast_exp2(ml[u].x - mm);
            ll = fmaf(w, ml[u].y, ll);
#pragma unroll
            for (int k = 0; k < 4; k++) {
                o[k].x = fmaf(w, v[u][k].x, o[k].x);
                o[k].y = fmaf(w, v[u][k].y, o[k].y);
                o[k].z = fmaf(w, v[u][k].z, o[k].z);
                o[k].w = fmaf(w, v[u][k].w, o[k].w);
            }
        }
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;  // a row with no token yields zeros
    uint4 packed[2];
    {
        uint32_t h[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            h[2 * k] = pack_half2(o[k].x * inv, o[k].y * inv);
            h[2 * k + 1] = pack_half2(o[k].z * inv, o[k].w * inv);
        }
        packed[0] = make_uint4(h[0], h[1], h[2], h[3]);
        packed[1] = make_uint4(h[4], h[5], h[6], h[7]);
    }
    if (p.n_peers == 0) {
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.out) + (size_t)pair * FAST_D + 16 * sub);
        dst[0] = packed[0];
        dst[1] = packed[1];
    } else {
        const int row = pair / p.n_heads, head = pair - row * p.n_heads;
        const size_t off = ((size_t)row * p.total_heads + p.head_offset + head) * FAST_D + 16 * sub;
        if (p.mc_out) {
            __half* dst = reinterpret_cast<__half*>(p.mc_out) + off;
            asm volatile("multimem.st.weak.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(packed[0].x),
                         "r"(packed[0].y), "r"(packed[0].z), "r"(packed[0].w)
                         : "memory");
            asm volatile("multimem.st.weak.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst + 8), "r"(packed[1].x),
                         "r"(packed[1].y), "r"(packed[1].z), "r"(packed[1].w)
                         : "memory");
            return;
        }
#pragma unroll
        for (int i = 0; i < MERGE_MAX_PEERS; i++)
            if (i < p.n_peers) {
                uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p.peer_out[i]) + off);
                dst[0] = packed[0];
                dst[1] = packed[1];
            }
    }
}

template <int FIRST, int MIN_CTAS>
__global__ void __launch_bounds__(128, MIN_CTAS) attn_merge_kernel(const MergeParams p) {
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    // The merge lists belong to the work list, which was uploaded before the partial kernel started:
    // as a programmatic dependent this kernel reads them while that kernel is still draining, and
    // only the partials themselves are read after the wait.
    int b = 0, e = 0, slot0 = -1, head = 0;
    if (pair < p.n_pairs) {
        const int row = pair / p.n_heads;   // the lists are per row; every head of the row combines the same pieces
        head = pair - row * p.n_heads;
        b = __ldg(p.merge_off + row);
        e = __ldg(p.merge_off + row + 1);
        checked_bounds(p, b, e);
        if (b + lane < e) slot0 = checked_slot(p, __ldg(p.merge_slots + b + lane), head);
    }
    // wait until the partial kernel's results are visible; a no-op for an ordinary launch
    asm volatile("griddepcontrol.wait;" ::: "memory");
    // the partial kernel is complete: a following kernel launched as a programmatic dependent (the
    // next step's partial kernel) may set itself up while the rows below are combined; it waits for
    // this kernel's completion before it touches global memory
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (pair >= p.n_pairs) return;
    float mm, ll;
    float4 acc;
    merge_list<FIRST>(p, lane, head, b, e, slot0, mm, ll, acc);
    store_row(p, pair, lane, acc, ll > 0.f ? 1.f / ll : 0.f);  // a row with no token yields zeros
}

// Few rows with long lists (one long sequence cut into many pieces, a long shared prefix under a
// handful of sequences): one CTA per (row, head), each of its 4 warps combines a quarter of the list
// and the quarters are combined through shared memory.
__global__ void __launch_bounds__(128, 3) attn_merge_wide_kernel(const MergeParams p) {
    __shared__ float4 s_acc[4][32];
    __shared__ float2 s_ml[4];
    const int pair = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = pair / p.n_heads, head = pair - row * p.n_heads;
    int b0 = __ldg(p.merge_off + row), e0 = __ldg(p.merge_off + row + 1);
    checked_bounds(p, b0, e0);
    const int per = (e0 - b0 + 3) >> 2;
    const int b = min(e0, b0 + warp * per), e = min(e0, b + per);
    const int slot0 = b + lane < e ? checked_slot(p, __ldg(p.merge_slots + b + lane), head) : -1;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    float mm, ll;
    float4 acc;
    merge_list<16>(p, lane, head, b, e, slot0, mm, ll, acc);
    s_acc[warp][lane] = acc;
    if (lane == 0) s_ml[warp] = make_float2(mm, ll);
    __syncthreads();
    if (warp != 0) return;
    float top = NEG_BIG;
#pragma unroll
    for (int w = 0; w < 4; w++)
        if (s_ml[w].y > 0.f) top = fmaxf(top, s_ml[w].x);
    float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
        if (s_ml[w].y > 0.f) {  // a quarter without tokens contributes nothing
            const float wgt = fast_exp2(s_ml[w].x - top);
            const float4 a = s_acc[w][lane];
            out.x = fmaf(wgt, a.x, out.x);
            out.y = fmaf(wgt, a.y, out.y);
            out.z = fmaf(wgt, a.z, out.z);
            out.w = fmaf(wgt, a.w, out.w);
            sum = fmaf(wgt, s_ml[w].y, sum);
        }
    }
    store_row(p, pair, lane, out, sum > 0.f ? 1.f / sum : 0.f);
}

// ---- barrier among the ranks of a node ------------------------------------------------------------------------
// Lane i tells rank i that this rank has arrived (a release store of the epoch into word `rank` of rank i's flag
// array, over NVLink), then waits -- for a bounded time -- until rank i's arrival shows in this rank's own array.
// The kernel before it in the stream has completed, so the rows it stored into the peers are ordered before the
// release.  A peer that never arrives costs the time limit and a status code, not a hung GPU.
__global__ void peer_barrier_kernel(const PeerBarrierParams p) {
    // launched as a programmatic dependent of the kernel whose rows it publishes: resident early, it waits here
    // for that kernel's completion (a no-op for an ordinary launch) and lets the next kernel set itself up
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int i = threadIdx.x;
    if (i >= p.n_peers) return;
    uint32_t* theirs = p.flags[i] + p.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(p.epoch) : "memory");
    const uint32_t* mine = p.flags[p.rank] + i;
    const unsigned long long t0 = global_timer_ns();
    while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
        if ((int32_t)(v - p.epoch) >= 0) break;
        if ((long long)(global_timer_ns() - t0) > p.timeout_ns) {
            if (p.status) atomicCAS(p.status, STATUS_OK, STATUS_PEER_WAIT_TIMEOUT);
            break;
        }
    }
}

}  // namespace

cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t stream) {
    static const bool pdl_disabled = std::getenv("CA_DISABLE_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(32);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_disabled ? 0 : 1;
    cudaError_t err = cudaLaunchKernelEx(&cfg, peer_barrier_kernel, p);
    if (err != cudaSuccess && cfg.numAttrs == 1) {
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        err = cudaLaunchKernelEx(&cfg, peer_barrier_kernel, p);
    }
    return err;
}

cudaError_t configure_fast_kernels() {
    // opt in to the large dynamic shared-memory carve-out, once per device (per context creation)
    cudaError_t e = cudaFuncSetAttribute(attn_partial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_partial_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                cudaSharedmemCarveoutMaxShared);
}

cudaError_t launch_attn_partials(const PartialParams& p, int n_ctas, cudaStream_t stream, bool dependent_launch) {
    if (n_ctas <= 0) return cudaSuccess;
    static const bool pdl_disabled = std::getenv("CA_DISABLE_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_ctas);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (dependent_launch && !pdl_disabled) ? 1 : 0;
    cudaError_t err = cudaLaunchKernelEx(&cfg, attn_partial_kernel, p);
    if (err != cudaSuccess && cfg.numAttrs == 1) {
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        err = cudaLaunchKernelEx(&cfg, attn_partial_kernel, p);
    }
    return err;
}

cudaError_t launch_attn_short_tails(const PartialParams& p, cudaStream_t stream, bool dependent_launch, const MergeParams* finish) {
    const int n = p.item_hi - p.item_lo;
    if (n <= 0) return cudaSuccess;
    static const bool pdl_disabled = std::getenv("CA_DISABLE_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((n + SHORT_ITEMS_PER_CTA - 1) / SHORT_ITEMS_PER_CTA);
    cfg.blockDim = dim3(SHORT_WARPS * 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (dependent_launch && !pdl_disabled) ? 1 : 0;
    auto* kernel = finish ? attn_short_tails_kernel<true> : attn_short_tails_kernel<false>;
    const MergeParams mp = finish ? *finish : MergeParams{};
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, p, mp);
    if (err != cudaSuccess && cfg.numAttrs == 1) {
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        err = cudaLaunchKernelEx(&cfg, kernel, p, mp);
    }
    return err;
}

cudaError_t launch_attn_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch) {
    if (p.n_pairs <= 0) return cudaSuccess;
    static const bool pdl_disabled = std::getenv("CA_DISABLE_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.n_pairs + 3) / 4);
    cfg.blockDim = dim3(128);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (dependent_launch && !pdl_disabled) ? 1 : 0;
    // pick the instance whose single wave holds the grid
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int)cfg.gridDim.x;
    // long lists under few rows: a CTA per row instead of a warp per row (a couple of waves at most)
    const bool wide = p.n_pairs <= 8 * sms && p.n_merge_entries * (long long)p.n_heads > 48LL * p.n_pairs;
    if (wide) cfg.gridDim = dim3(p.n_pairs);
    // many rows of at most four pieces each: eight lanes per row instead of a warp
    const bool small = !wide && p.max_list > 0 && p.max_list <= SMALL_MAX_LIST && grid > 3 * sms;
    if (small) cfg.gridDim = dim3((p.n_pairs + 15) / 16);
    auto launch = [&]() {
        if (wide) return cudaLaunchKernelEx(&cfg, attn_merge_wide_kernel, p);
        if (small) return cudaLaunchKernelEx(&cfg, attn_merge_small_kernel, p);
        if (grid <= 3 * sms) return cudaLaunchKernelEx(&cfg, attn_merge_kernel<16, 3>, p);
        if (grid <= 5 * sms) return cudaLaunchKernelEx(&cfg, attn_merge_kernel<8, 5>, p);
        return cudaLaunchKernelEx(&cfg, attn_merge_kernel<0, 7>, p);
    };
    cudaError_t err = launch();
    if (err != cudaSuccess && cfg.numAttrs == 1) {
        // the stream or driver refused the programmatic launch: fall back to a plain ordered launch
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        err = launch();
    }
    return err;
}

}  // namespace ca
