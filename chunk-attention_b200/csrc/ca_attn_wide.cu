// Chunk-first attention for WIDE shared runs on the Blackwell tensor path: tcgen05.mma with accumulators in
// tensor memory (TMEM), K/V tiles staged by 1-D TMA bulk copies, sm_100a.
//
// When many sequences share a long prefix (one system prompt under hundreds of requests), the chunk-first
// phase is a real contraction: n query rows against every K/V tile of the run, n flop per K/V byte.  The
// mma.sync walk of the persistent kernel (ca_attn_fast.cu) is then bound by the latency of its dependent
// m16n8k16 chains, not by memory; this kernel serves those runs instead (the planner routes them, ca_plan.cpp).
// Counterpart in the reference: attn_chunk_first_kernel_v2 (cpp/chunk_attn/kernel_cuda.cu:796-883, wmma).
//
// One CTA per item = (head, block of up to 128 query rows, piece of up to 32 consecutive chunks of a run):
//   S = Q K^T      tcgen05.mma.kind::f16, M = 128 query rows, N = 64 tokens, 8 steps over d_head = 128;
//                  A = the item's queries, staged once in shared memory in the 128-byte-swizzled K-major layout,
//                  B = the K tile exactly as the pool stores it (two panels of 64 elements, ca_layout.h);
//                  D = S in TMEM (fp32), two buffers so that S of tile j+1 is computed under the softmax of tile j
//   softmax        a warpgroup, one thread per query row (= TMEM lane): tcgen05.ld S, running maximum in log2
//                  units, P = 2^(s - m) as fp16 written back over S with tcgen05.st; the accumulator O is only
//                  rescaled (tcgen05.ld / st) when a row's maximum has grown by more than 8 since the scale in
//                  use was fixed, which bounds P by 2^8 and makes rescaling rare
//   O += P V       tcgen05.mma with A = P read from TMEM, B = the V tile as stored (MN-major panels), N = 128,
//                  4 steps of 16 tokens; D = O in TMEM (fp32)
// and emits one ordinary partial per row (running max, sum, un-normalised O) for the merge kernel.
// Warp roles: warps 0-3 softmax and epilogue, warp 4 (one thread) TMA producer over a ring of four 16 KiB
// slots (K and V tiles take slots of their own, so a K slot is free again as soon as S is computed), warp 5
// allocates and frees the 256 TMEM columns and (one thread) issues every MMA.  Completion travels through
// mbarriers (tcgen05.commit).  Two CTAs share an SM (2 x 256 TMEM columns, 2 x 97 KiB of shared memory).
//
// Every wait is bounded: on expiry the kernel records a status code, every role falls through to the common
// exit, and the TMEM columns are freed there on every path.
#include <cuda_fp16.h>

#include <cstdlib>

#include "ca_kernels.h"
#include "ca_plan.h"
#include "ca_ptx.cuh"

namespace ca {
namespace {
using namespace ptx;

constexpr int W_ROWS = WIDE_MAX_ROWS;                  // MMA M: query rows of an item (padded)
constexpr int W_SLOTS = 4;                             // ring slots, one K or V tile each
constexpr int W_Q_PANEL = W_ROWS * 128;                // one 64-element panel of the staged queries
constexpr int W_SMEM_RING = 2 * W_Q_PANEL;             // queries first (32 KiB), then the ring
constexpr int W_SMEM_BAR = W_SMEM_RING + W_SLOTS * FAST_TILE_BYTES;
constexpr int W_NUM_BARS = 2 * W_SLOTS + 6;            // full, empty, s_full[2], p_full[2], o_done, q_ready
constexpr int W_SMEM_BYTES = W_SMEM_BAR + W_NUM_BARS * 8 + 24;
constexpr int W_THREADS = 192;
constexpr int W_TMEM_COLS = 256;                       // O: 0..127, S buffers: 128..191 and 192..255
constexpr int W_COL_S = 128;
constexpr int W_STAGE_PITCH = FAST_D + 4;               // floats per staged output row (528 bytes: conflict-free 128-bit stores)
static_assert(W_ROWS * W_STAGE_PITCH * 4 <= W_SMEM_BAR, "the output staging must fit under the barriers");
constexpr float W_NEG_BIG = -1.0e30f;
constexpr float W_RESCALE_STEP = 8.f;                  // log2 units a row's maximum may drift above the scale in use
static_assert(2 * (W_SMEM_BYTES + 1024) <= 233472, "two CTAs do not fit in one SM's shared memory");

constexpr uint32_t IDESC_QK = umma_idesc_f16(W_ROWS, FAST_C, false, false);
constexpr uint32_t IDESC_PV = umma_idesc_f16(W_ROWS, FAST_D, false, true);

__device__ __forceinline__ void report(int* status, int code) { atomicCAS(status, STATUS_OK, code); }

// ACCT: instead of the timestamps 1-5 of the trace, the CTA records where the cycles of its two serial roles go
// (see WideParams::trace_cycles); a separate instantiation, so the kernel that serves carries none of it.
template <bool ACCT>
__global__ void __launch_bounds__(W_THREADS, 2) attn_wide_kernel(const WideParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t sbase = smem_u32(smem);
    const uint32_t ring = sbase + W_SMEM_RING;
    const uint32_t full_bar = sbase + W_SMEM_BAR;
    const uint32_t empty_bar = full_bar + 8 * W_SLOTS;
    const uint32_t s_full = empty_bar + 8 * W_SLOTS;
    const uint32_t p_full = s_full + 16;
    const uint32_t o_done = p_full + 16;
    const uint32_t q_ready = o_done + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + W_SMEM_BAR + W_NUM_BARS * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long* tr = p.trace ? p.trace + 8 * blockIdx.x : nullptr;
    if (tr && threadIdx.x == 0) tr[0] = global_timer_ns();

    if (threadIdx.x == 0) {
        for (int i = 0; i < W_SLOTS; i++) {
            mbar_init(full_bar + 8 * i, 1);
            mbar_init(empty_bar + 8 * i, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, 4 * 32);
        }
        mbar_init(o_done, 1);
        mbar_init(q_ready, 4 * 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 5) {  // the warp that allocates is the warp that frees
        tmem_alloc(smem_u32(tmem_slot), W_TMEM_COLS);
        tmem_relinquish_alloc_permit();
    }
    // as a programmatic dependent launch the CTA has set itself up while the kernel before it was finishing;
    // nothing in global memory has been touched so far
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    // the work list holds every item once for all heads: piece v = (item v / n_heads, head v % n_heads)
    const int vid = p.item_lo + (int)blockIdx.x;
    const int idx = vid / p.n_heads, head = vid - idx * p.n_heads;
    const int4 d0 = __ldg(p.items + 4 * idx), d1 = __ldg(p.items + 4 * idx + 1);
    const int n_tiles = d0.x, row_begin = d0.z, n_rows = d0.w, slot_base = d1.x, chunk_off = d1.w;
    // the work list may come from memory the host never saw: nothing in it is trusted
    bool ok = n_tiles >= 1 && n_tiles <= WIDE_MAX_TILES && n_rows >= 1 && n_rows <= W_ROWS &&
              row_begin >= 0 && slot_base >= 0 && chunk_off >= 0 && chunk_off + n_tiles <= p.n_wide_chunks &&
              (p.n_slots <= 0 || (long long)(slot_base + n_rows) * p.n_heads <= p.n_slots) &&
              (p.n_seqs <= 0 || row_begin + n_rows <= p.n_seqs);
    tc_fence_before_thread_sync();
    __syncthreads();   // barriers initialised, TMEM address published
    tc_fence_after_thread_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (!ACCT && tr && threadIdx.x == 0) tr[1] = global_timer_ns();
    if (!ok && threadIdx.x == 0) report(p.status, STATUS_BAD_WORK_LIST);  // skipped: its partial rows keep what they held

    if (ok) {
        if (warp < 4) {
            // ---- queries -> shared memory, K-major 128-byte-swizzled: two panels of 128 lines; rows past the item
            // are zero.  The producer is already fetching K/V tiles meanwhile.
            const uint4* q = reinterpret_cast<const uint4*>(p.q);
            uint4 v[16];   // all sixteen loads of a thread in flight together
#pragma unroll
            for (int u = 0; u < 16; u++) {
                const int i = threadIdx.x + u * (4 * 32), r = i >> 4, g = i & 15;
                v[u] = make_uint4(0u, 0u, 0u, 0u);
                if (r < n_rows) v[u] = __ldg(q + ((size_t)(row_begin + r) * p.n_heads + head) * 16 + g);
            }
#pragma unroll
            for (int u = 0; u < 16; u++) {
                const int i = threadIdx.x + u * (4 * 32), r = i >> 4, g = i & 15;
                const uint32_t dst = sbase + (g >> 3) * W_Q_PANEL + r * 128 + (((g & 7) ^ (r & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w) : "memory");
            }
            fence_proxy_async();  // the tensor core reads shared memory through the async proxy
            mbar_arrive(q_ready);
        }

        if (warp == 4) {
            // ---- producer: one thread, slot i & 3 takes K of tile i / 2 (even i) or its V (odd i)
            if (lane == 0) {
                int issued = 0;
                for (int i = 0; i < 2 * n_tiles; i++) {
                    const int slot = i & (W_SLOTS - 1), use = i / W_SLOTS;
                    if (!mbar_wait_bounded(empty_bar + 8 * slot, (use & 1) ^ 1, p.wait_limit)) {
                        report(p.status, STATUS_EMPTY_WAIT_TIMEOUT);
                        break;
                    }
                    int chunk = __ldg(p.wide_chunks + chunk_off + (i >> 1));
                    if (chunk < 0 || (p.max_chunks > 0 && chunk >= p.max_chunks)) {
                        report(p.status, STATUS_BAD_WORK_LIST);  // keep the pipeline moving on a chunk that exists
                        chunk = 0;
                    }
                    const uint8_t* src = p.pool + ((size_t)chunk * p.n_heads + head) * (size_t)FAST_STAGE_BYTES +
                                         (size_t)(i & 1) * FAST_TILE_BYTES;
                    mbar_arrive_expect_tx(full_bar + 8 * slot, FAST_TILE_BYTES);
                    bulk_copy_g2s(ring + slot * FAST_TILE_BYTES, src, FAST_TILE_BYTES, full_bar + 8 * slot);
                    issued++;
                }
                // do not leave while a copy into this CTA's shared memory may still be in flight
                for (int f = issued > W_SLOTS ? issued - W_SLOTS : 0; f < issued; f++) {
                    if (!mbar_wait_bounded(full_bar + 8 * (f & (W_SLOTS - 1)), (f / W_SLOTS) & 1, p.wait_limit)) {
                        report(p.status, STATUS_DRAIN_TIMEOUT);
                        break;
                    }
                }
            }
        } else if (warp == 5) {
            // ---- MMA issuer: one thread
            if (elect_one()) {
                bool live = true;
                constexpr uint32_t DESC_HI = umma_desc_sw128_hi(1024);   // 8-line groups are 1024 bytes apart in every operand
                const uint32_t q_lo = umma_desc_sw128_lo(sbase, 16);
                long long c_issue_qk = 0, c_issue_pv = 0, c_wait_p = 0, c_wait_k = 0, w0 = 0, w1 = 0;
                auto issue_qk = [&](int j) {
                    const int i = 2 * j, slot = i & (W_SLOTS - 1);
                    if (ACCT) w0 = clock64();
                    if (!mbar_wait_bounded(full_bar + 8 * slot, (i / W_SLOTS) & 1, p.wait_limit)) {
                        report(p.status, STATUS_FULL_WAIT_TIMEOUT);
                        live = false;
                        return;
                    }
                    if (ACCT) {
                        w1 = clock64();
                        c_wait_k += w1 - w0;
                    }
                    tc_fence_after_thread_sync();
                    const uint32_t kaddr = ring + slot * FAST_TILE_BYTES;
                    const uint32_t d = tmem_base + W_COL_S + (j & 1) * FAST_C;
                    // K step ks: 32 bytes further along the 128-byte line, the second panel of 64 elements after four
                    const uint32_t b_lo = umma_desc_sw128_lo(kaddr, 16);
#pragma unroll
                    for (int ks = 0; ks < 8; ks++) {
                        const uint64_t a = umma_desc_pack(q_lo + (((ks >> 2) * W_Q_PANEL + (ks & 3) * 32) >> 4), DESC_HI);
                        const uint64_t b = umma_desc_pack(b_lo + (((ks >> 2) * (FAST_C * 128) + (ks & 3) * 32) >> 4), DESC_HI);
                        umma_ss_f16(d, a, b, IDESC_QK, ks > 0 ? 1u : 0u);
                    }
                    umma_commit(s_full + 8 * (j & 1));   // S of tile j is complete ...
                    umma_commit(empty_bar + 8 * slot);   // ... and its K tile may be overwritten
                    if (ACCT) c_issue_qk += clock64() - w1;
                };
                if (!mbar_wait_bounded(q_ready, 0, p.wait_limit)) {
                    report(p.status, STATUS_FULL_WAIT_TIMEOUT);
                    live = false;
                }
                if (live) issue_qk(0);
                for (int j = 0; j < n_tiles && live; j++) {
                    if (j + 1 < n_tiles) issue_qk(j + 1);  // S of the next tile is computed under this tile's softmax
                    if (!live) break;
                    const int i = 2 * j + 1, slot = i & (W_SLOTS - 1);
                    if (ACCT) w0 = clock64();
                    if (!mbar_wait_bounded(p_full + 8 * (j & 1), (j >> 1) & 1, p.wait_limit) ||
                        !mbar_wait_bounded(full_bar + 8 * slot, (i / W_SLOTS) & 1, p.wait_limit)) {
                        report(p.status, STATUS_FULL_WAIT_TIMEOUT);
                        break;
                    }
                    if (ACCT) {
                        w1 = clock64();
                        c_wait_p += w1 - w0;
                    }
                    tc_fence_after_thread_sync();
                    const uint32_t vaddr = ring + slot * FAST_TILE_BYTES;
                    const uint32_t a_tmem = tmem_base + W_COL_S + (j & 1) * FAST_C;  // P over S, two fp16 per column
                    // 16 tokens = two groups of 8 lines; the two 64-element panels of d_head are 8 KiB apart
                    const uint32_t v_lo = umma_desc_sw128_lo(vaddr, FAST_C * 128);
#pragma unroll
                    for (int kk = 0; kk < 4; kk++) {
                        const uint64_t b = umma_desc_pack(v_lo + ((kk * 2048) >> 4), DESC_HI);
                        umma_ts_f16(tmem_base, a_tmem + kk * 8, b, IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar + 8 * slot);
                    umma_commit(o_done);
                    if (ACCT) c_issue_pv += clock64() - w1;
                }
                if (ACCT && tr) {
                    uint32_t smid;
                    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                    tr[1] = (unsigned long long)c_issue_pv;
                    tr[2] = (unsigned long long)c_issue_qk;
                    tr[3] = (unsigned long long)c_wait_p;
                    tr[7] = (unsigned long long)c_wait_k | ((unsigned long long)smid << 48);
                }
            }
        } else {
            // ---- softmax and epilogue: thread r owns query row r = TMEM lane r
            const int r = threadIdx.x;
            const bool active = r < n_rows;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
            float m_used = W_NEG_BIG, l = 0.f;
            bool live = true;
            long long c_wait_s = 0, c_chain = 0, w0 = 0, w1 = 0;
            for (int j = 0; j < n_tiles && live; j++) {
                const int b = j & 1;
                if (ACCT) w0 = clock64();
                live = mbar_wait_bounded(s_full + 8 * b, (j >> 1) & 1, p.wait_limit);
                live = __all_sync(0xffffffffu, live);
                if (!live) {
                    if (lane == 0) report(p.status, STATUS_FULL_WAIT_TIMEOUT);
                    break;
                }
                tc_fence_after_thread_sync();
                if (!ACCT && tr && j == 0 && threadIdx.x == 0) tr[2] = global_timer_ns();
                if (ACCT) {
                    w1 = clock64();
                    c_wait_s += w1 - w0;
                }
                uint32_t s0[32], s1[32];
                tmem_ld32(lane_addr + W_COL_S + b * FAST_C, s0);
                tmem_ld32(lane_addr + W_COL_S + b * FAST_C + 32, s1);
                tmem_wait_ld();
                float alpha = 1.f;
                bool rescale = false;
                uint32_t pk[32];
                if (active) {
                    float mx = W_NEG_BIG;
#pragma unroll
                    for (int i = 0; i < 32; i++) mx = fmaxf(mx, fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])));
                    mx *= p.scale_log2;
                    if (j == 0) {
                        m_used = mx;
                    } else if (mx > m_used + W_RESCALE_STEP) {
                        alpha = fast_exp2(m_used - mx);
                        m_used = mx;
                        l *= alpha;
                        rescale = true;
                    }
                    float sum = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float a0 = fast_exp2(fmaf(__uint_as_float(s0[2 * i]), p.scale_log2, -m_used));
                        const float a1 = fast_exp2(fmaf(__uint_as_float(s0[2 * i + 1]), p.scale_log2, -m_used));
                        const float c0 = fast_exp2(fmaf(__uint_as_float(s1[2 * i]), p.scale_log2, -m_used));
                        const float c1 = fast_exp2(fmaf(__uint_as_float(s1[2 * i + 1]), p.scale_log2, -m_used));
                        sum += (a0 + a1) + (c0 + c1);
                        pk[i] = pack_half2(a0, a1);        // tokens 2i, 2i + 1
                        pk[16 + i] = pack_half2(c0, c1);   // tokens 32 + 2i, 33 + 2i
                    }
                    l += sum;
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++) pk[i] = 0u;
                }
                tmem_st32(lane_addr + W_COL_S + b * FAST_C, pk);
                if (j > 0) {
                    // Every thread follows o_done phase by phase (an mbarrier wait only tells a phase from its
                    // neighbour, so nobody may fall two behind): O += P V of tile j - 1 is complete.  It was issued
                    // before this tile's softmax began, so this rarely waits; and O may now be rescaled.
                    live = mbar_wait_bounded(o_done, (j - 1) & 1, p.wait_limit);
                    live = __all_sync(0xffffffffu, live);
                    if (!live) {
                        if (lane == 0) report(p.status, STATUS_FULL_WAIT_TIMEOUT);
                        break;
                    }
                }
                if (__any_sync(0xffffffffu, rescale)) {
                    // O holds the tiles before this one, scaled by the old maximum
                    tc_fence_after_thread_sync();
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        uint32_t o[32];
                        tmem_ld32(lane_addr + c * 32, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st32(lane_addr + c * 32, o);
                    }
                }
                tmem_wait_st();
                tc_fence_before_thread_sync();
                mbar_arrive(p_full + 8 * b);
                if (ACCT) c_chain += clock64() - w1;
            }
            if (ACCT && tr && threadIdx.x == 0) {
                tr[4] = (unsigned long long)c_wait_s;
                tr[5] = (unsigned long long)c_chain;
            }
            if (!ACCT && tr && threadIdx.x == 0) tr[3] = global_timer_ns();
            if (live) {
                live = mbar_wait_bounded(o_done, (n_tiles - 1) & 1, p.wait_limit);
                live = __all_sync(0xffffffffu, live);
                if (!live && lane == 0) report(p.status, STATUS_FULL_WAIT_TIMEOUT);
            }
            if (!ACCT && tr && threadIdx.x == 0) tr[4] = global_timer_ns();
            if (live) {
                tc_fence_after_thread_sync();
                // O leaves through shared memory (the staged queries and the ring are free now: every MMA has
                // completed): a thread holds one ROW, but a row must reach global memory as whole 512-byte lines.
                // Each warp stages and writes its own 32 rows, so a warp-level barrier is all the ordering it needs.
                float* stage = reinterpret_cast<float*>(smem);
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    uint32_t o[32];
                    tmem_ld32(lane_addr + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        *reinterpret_cast<uint4*>(stage + r * W_STAGE_PITCH + c * 32 + 4 * i) =
                            make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
                }
                __syncwarp();
                const int rows_here = min(32, n_rows - warp * 32);   // <= 0 for a warp past the item's rows
                for (int rr = 0; rr < rows_here; rr++) {
                    const int row = warp * 32 + rr;
                    const size_t slot = (size_t)(slot_base + row) * p.n_heads + head;  // row `row` of this head
                    const uint4 v = *reinterpret_cast<const uint4*>(stage + row * W_STAGE_PITCH + 4 * lane);
                    *reinterpret_cast<uint4*>(p.part_o + slot * FAST_D + 4 * lane) = v;
                }
                if (active) p.part_ml[(size_t)(slot_base + r) * p.n_heads + head] = make_float2(m_used, l);
            }
            if (!ACCT && tr && threadIdx.x == 0) tr[5] = global_timer_ns();
        }
    }
    // ---- common exit of every path: nobody touches TMEM after this barrier, then the allocating warp frees it
    tc_fence_before_thread_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_thread_sync();
        tmem_dealloc(tmem_base, W_TMEM_COLS);
        if (tr && lane == 0) tr[6] = global_timer_ns();
    }
}

}  // namespace

cudaError_t configure_wide_kernel() {
    cudaError_t e = cudaFuncSetAttribute(attn_wide_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_wide_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, W_SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_wide_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_wide_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

cudaError_t launch_attn_wide(const WideParams& p, cudaStream_t stream, bool dependent_launch) {
    const int n = p.item_hi - p.item_lo;
    if (n <= 0) return cudaSuccess;
    static const bool pdl_disabled = std::getenv("CA_DISABLE_PDL") != nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n);
    cfg.blockDim = dim3(W_THREADS);
    cfg.dynamicSmemBytes = W_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (dependent_launch && !pdl_disabled) ? 1 : 0;
    auto* kernel = (p.trace && p.trace_cycles) ? attn_wide_kernel<true> : attn_wide_kernel<false>;
    cudaError_t err = cudaLaunchKernelEx(&cfg, kernel, p);
    if (err != cudaSuccess && cfg.numAttrs == 1) {
        (void)cudaGetLastError();
        cfg.numAttrs = 0;
        err = cudaLaunchKernelEx(&cfg, kernel, p);
    }
    return err;
}

}  // namespace ca
