// Launchers of the CUDA kernels (internal to the library; the public surface is the C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "ca_layout.h"

namespace ca {

void set_last_error(const std::string& msg);  // message returned by ca_last_error() on this thread

// Device status word values (first failure wins).
constexpr int STATUS_OK = 0;
constexpr int STATUS_FULL_WAIT_TIMEOUT = 1;   // a consumer warp gave up waiting for a tile
constexpr int STATUS_EMPTY_WAIT_TIMEOUT = 2;  // the producer gave up waiting for a free stage
constexpr int STATUS_DRAIN_TIMEOUT = 3;       // copies still in flight at kernel exit
constexpr int STATUS_BAD_WORK_LIST = 4;       // an item or merge entry named a slot, row, head or chunk out of range: skipped
constexpr int STATUS_BAD_POSITION = 5;        // rotary embedding: a position outside the cos/sin table: row skipped
constexpr long long DEFAULT_WAIT_LIMIT_CYCLES = 4000000000LL;  // about two seconds of SM clock

// ---- fast path: fp16, d_head 128, chunk_size 64 -----------------------------------------------
constexpr int FAST_D = 128;
constexpr int FAST_C = 64;
constexpr int FAST_TILE_BYTES = FAST_C * FAST_D * 2;  // one K or V tile
constexpr int FAST_STAGE_BYTES = 2 * FAST_TILE_BYTES; // K tile + V tile of one (chunk, head)
constexpr int FAST_CONSUMER_WARPS = 4;                // warps of a CTA that walk tiles
constexpr int FAST_CTAS_PER_SM = 2;                   // persistent CTAs resident per SM
constexpr int FAST_MAX_ROWS_PER_ITEM = 16 * FAST_CONSUMER_WARPS;  // query rows one item can serve

struct PartialParams {
    const uint8_t* pool;         // chunk pool base
    int n_heads;
    const void* q;               // fp16 [n_seqs, n_heads, 128]
    const int4* items;           // PlanItem as four int4, each standing for n_heads pieces of work
    int item_lo, item_hi;        // the launch works through pieces [item_lo, item_hi); piece v = item v / n_heads, head v % n_heads
    int* counter;                // next item to hand out (relative to item_lo); zero when the launch starts
    int* counter_next;           // the counter of the following launch: zeroed by this one
    float* part_o;               // [n_slots][128]
    float2* part_ml;             // [n_slots] (running max in log2 units, sum of exponentials)
    int delta_tokens;            // tokens appended to every tail since the plan was built
    float scale_log2;            // log2(e) / sqrt(d_head)
    int* status;
    // Bounds every index of the work list is checked against on the device (an item that fails is skipped and
    // STATUS_BAD_WORK_LIST is recorded); 0 switches the corresponding check off.
    int n_slots = 0;             // partial rows behind part_o / part_ml
    int n_seqs = 0;              // rows of q
    int max_chunks = 0;          // chunks in the pool
    long long wait_limit = DEFAULT_WAIT_LIMIT_CYCLES;  // SM cycles a wait on a ring barrier may take
    int withhold_item = -1;      // failure-path tests only: the producer that draws this item stops feeding its CTA
    unsigned long long* trace = nullptr;  // optional [n_ctas][8], null = off: ns timestamps of start,
                                 // producer end, first and last consumer warp end; then cycles: warp 0 waiting for
                                 // tiles, warp 0 combining/storing partials, producer waiting for free stages, warp 0 total
};

// Persistent kernel: chunk-first and sequence-first items, both fed by one TMA ring per CTA.
// grid = n_ctas (FAST_CTAS_PER_SM per SM).
// dependent_launch: allow the CTAs to be set up while the preceding kernel of the stream is finishing
cudaError_t launch_attn_partials(const PartialParams& p, int n_ctas, cudaStream_t stream, bool dependent_launch = false);
// one half-warp per item over items [item_lo, item_hi): single-tile one-row items only (short private tails).
// finish != null: every row of the batch has such an item and every other partial of the step is already in the
// stream; the kernel then combines each row's partials itself and stores the output rows (no merge launch follows)
struct MergeParams;
cudaError_t launch_attn_short_tails(const PartialParams& p, cudaStream_t stream, bool dependent_launch = false,
                                    const MergeParams* finish = nullptr);
cudaError_t configure_fast_kernels();  // once per device before the first launch

// ---- wide shared runs on tcgen05 / TMEM (ca_attn_wide.cu): one CTA per item ---------------------------------
struct WideParams {
    const uint8_t* pool;
    int n_heads;
    const void* q;               // fp16 [n_seqs, n_heads, 128]
    const int4* items;           // PlanItem; chunk[0] is the offset of the item's chunk list in wide_chunks
    int item_lo, item_hi;
    const int32_t* wide_chunks;
    int n_wide_chunks;           // entries of wide_chunks
    float* part_o;
    float2* part_ml;
    float scale_log2;
    int* status;
    int n_slots = 0, n_seqs = 0, max_chunks = 0;  // bounds the work list is checked against (0: unchecked)
    long long wait_limit = DEFAULT_WAIT_LIMIT_CYCLES;
    unsigned long long* trace = nullptr;  // optional [n_ctas][8] ns timestamps: entry, set-up done, first S ready,
                                          // last P written, O complete, partial rows stored, exit
    int trace_cycles = 0;                 // 1: entries 1-5 and 7 hold SM cycles summed over the item's tiles instead: the MMA
                                          // thread issuing [1] the P V and [2] the Q K^T MMAs with their commits, [3] that
                                          // thread waiting for P and the V tile, [4] the first softmax thread waiting for
                                          // S, [5] that thread from S ready to P handed over, [7] bits 0-47 the MMA thread
                                          // waiting for the K tile, bits 48-63 the SM the CTA ran on
};
cudaError_t launch_attn_wide(const WideParams& p, cudaStream_t stream, bool dependent_launch = false);
cudaError_t configure_wide_kernel();  // once per device before the first launch

constexpr int MERGE_MAX_PEERS = 8;
struct MergeParams {
    const float* part_o;
    const float2* part_ml;
    const int32_t* merge_off;    // [n_rows + 1]: the lists are per row, shared by the row's heads
    const int32_t* merge_slots;  // partial rows numbered per head-agnostic item; head h's is entry * n_heads + h
    void* out;                   // fp16 [n_rows, n_heads, 128]; unused when n_peers > 0
    int n_pairs;                 // n_rows * n_heads
    long long n_merge_entries = 0; // length of merge_slots
    int max_list = 0;            // longest list of a row (0: unknown); picks the kernel instance
    // Head-sharded output written straight into every rank's full-width buffer (peer memory over
    // NVLink): row s, local head h goes to peer_out[i] + ((s * total_heads) + head_offset + h) * 128.
    int n_heads = 0;             // local heads
    int n_peers = 0;             // 0: write `out` only
    int total_heads = 0;
    int head_offset = 0;
    void* peer_out[MERGE_MAX_PEERS] = {};
    void* mc_out = nullptr;      // optional multicast address of the same buffer on all ranks (NVLink SHARP): one
                                 // multimem.st per row segment then replaces the n_peers unicast stores
    int n_slots = 0;             // partial rows behind part_o / part_ml; a list entry outside [0, n_slots) is skipped
    int* status = nullptr;       // and STATUS_BAD_WORK_LIST recorded here (0 / null: unchecked)
};
cudaError_t launch_attn_merge(const MergeParams& p, cudaStream_t stream, bool dependent_launch);

constexpr int STATUS_PEER_WAIT_TIMEOUT = 6;   // a peer did not reach the barrier within the time allowed
// One-phase barrier among the ranks of a node over flag words in each other's memory: rank r stores `epoch` into
// word r of every peer's flag array, then waits until every word of its own array has reached `epoch`.
struct PeerBarrierParams {
    uint32_t* flags[MERGE_MAX_PEERS];  // flags[i]: rank i's array of n_peers words (this rank's own included)
    int n_peers;
    int rank;
    uint32_t epoch;                    // grows by one per barrier; the words only ever grow
    long long timeout_ns;              // of the GPU's global timer
    int* status;                       // may be null
};
cudaError_t launch_peer_barrier(const PeerBarrierParams& p, cudaStream_t stream);

// ---- generic path: any d_head <= 256, any chunk size, fp16 or fp32 ----------------------------------
struct GenericParams {
    const void* pool;
    Geometry geo;
    const void* q;
    void* out;
    const int32_t* path_off;     // [n_seqs + 1]
    const int32_t* path_chunks;
    const int32_t* path_tokens;
    int n_seqs;
    int delta_tokens;
    float scale;                 // 1 / sqrt(d_head)
};
cudaError_t launch_attn_seq_generic(const GenericParams& p, int dtype, cudaStream_t stream);

// ---- pool maintenance ------------------------------------------------------------------------------------
struct AppendParams {
    void* pool;
    Geometry geo;
    const void* k;               // [n_seqs, n_heads, d_head]
    const void* v;
    const int32_t* tail_chunk;   // [n_seqs]
    const int32_t* tail_tokens;  // [n_seqs]
    int n_seqs;
    int delta_tokens;
};
// vec16: rows are whole 16-byte granules and k, v are 16-byte aligned
cudaError_t launch_append_kv(const AppendParams& p, bool vec16, cudaStream_t stream);

constexpr int SCATTER_MAX_CHUNKS = 512;
struct ScatterParams {
    void* pool;
    Geometry geo;
    const void* k;
    const void* v;
    int64_t stride_token, stride_head;  // in elements
    int n_tokens;
    int32_t chunk_ids[SCATTER_MAX_CHUNKS];
};
cudaError_t launch_scatter_prefill(const ScatterParams& p, bool vec16, cudaStream_t stream);

// token i of k / v goes to row rows[i] of chunk chunk_ids[i]
constexpr int SCATTER_MAX_ROWS = 256;
struct ScatterRowsParams {
    void* pool;
    Geometry geo;
    const void* k;
    const void* v;
    int64_t stride_token, stride_head;  // in elements
    int n_tokens;
    int32_t chunk_ids[SCATTER_MAX_ROWS];
    int32_t rows[SCATTER_MAX_ROWS];
};
cudaError_t launch_scatter_rows(const ScatterRowsParams& p, bool vec16, cudaStream_t stream);

constexpr int COPY_MAX_PAIRS = 256;
struct CopyParams {
    void* pool;
    int64_t chunk_bytes;
    int n;
    int32_t src[COPY_MAX_PAIRS];
    int32_t dst[COPY_MAX_PAIRS];
};
cudaError_t launch_copy_chunks(const CopyParams& p, cudaStream_t stream);

struct ReadChunkParams {
    const void* pool;
    Geometry geo;
    int chunk_id;
    int n_tokens;
    void* k_out;                 // [n_heads, n_tokens, d_head]
    void* v_out;
};
cudaError_t launch_read_chunk(const ReadChunkParams& p, cudaStream_t stream);

}  // namespace ca
