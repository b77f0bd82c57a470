// Host-side work-list builder ("plan") for one decode step.
//
// Input: the depth-first list of live chunks with the row range each one serves (what the
// reference's Attention::get_chunks produces, cpp/chunk_attn/attention.cpp:342-372).
// Output: everything the kernels read — the reference builds the equivalent tables in
// refresh_kernel_context (cpp/chunk_attn/kernel_cuda.cu:1331-1445), but the decomposition
// here is different:
//
//  * shared chunks (more sharers than tpp_threshold, always full) are grouped into RUNS, the
//    maximal chains of chunks that serve the identical row range; one run x head x row block
//    is a chunk-first unit and produces ONE partial per row for a whole piece of the chain
//    instead of one per chunk;
//  * the remaining chunks of a sequence (its private tail) x head are a sequence-first unit;
//  * every unit is a list of 32 KiB K+V tiles and is cut into ITEMS of at most 8 tiles (9 when a
//    tail chunk rides along), each
//    emitting its own partial.  Items are self-scheduled: the persistent CTAs draw the next item
//    from a device counter, so the split of the work adapts to whatever each SM achieves.  Item
//    sizes follow guided self-scheduling — as large as allowed while much work remains, shrinking
//    towards single tiles at the end of the list — so that all CTAs finish within about one tile
//    of each other;
//  * wide shared runs (many rows under a long prefix, where the contraction and not memory bounds the step) are
//    cut into items of their own for the tcgen05 / TMEM kernel: up to 128 rows x up to 32 chunks, one CTA each,
//    about one wave of them;
//  * merge lists name, per (row, head), the partial slots the merge kernel combines.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/chunk_attn_b200.h"

namespace ca {

constexpr int ITEM_FLAG_TAIL = 1;     // last tile of the item is the sequence's tail chunk
constexpr int ITEM_FLAG_WIDE = 2;     // an item of the tcgen05 kernel: chunk[0] is an offset into Plan::wide_chunks
constexpr int ITEM_SPLITS_SHIFT = 8;  // flags >> 8: token splits of a tensor-core item (4, 2, 1);
                                      // 0 = one-row item walked on CUDA cores
constexpr int MAX_ROWS_PER_ITEM = 64; // 4 consumer warps x 16 rows
constexpr int MAX_TILES_PER_ITEM = 9;  // 8 by size, plus a sequence's tail chunk riding along
constexpr int WIDE_MAX_ROWS = 128;    // query rows of a wide item (the M of tcgen05.mma)
constexpr int WIDE_MAX_TILES = 32;    // chunks of a wide item
// Wide routing (wide_mode 1 = automatic): shared runs of more than WIDE_MIN_ROWS rows go to the tcgen05 kernel when
// walking them with mma.sync would take longer than half the time the step's unique K/V needs at HBM rate — only then
// is the step bound by the tensor path rather than by memory.  Rates measured on B200.
constexpr int WIDE_MIN_ROWS = 32;
constexpr double WIDE_MMA_SYNC_FLOPS = 200e12;
constexpr double WIDE_HBM_BYTES_PER_S = 6.4e12;

struct PlanItem {
    int32_t n_tiles;      // 1 .. MAX_TILES_PER_ITEM
    int32_t head;
    int32_t row_begin;    // first row of q / out this item serves
    int32_t n_rows;       // 1: sequence-first item; >= 2: chunk-first item
    int32_t slot_base;    // first partial slot
    int32_t flags;
    int32_t last_tokens;  // tokens in the last tile when the plan was built
    int32_t chunk[MAX_TILES_PER_ITEM];  // pool slots of the tiles
};
static_assert(sizeof(PlanItem) == 64, "PlanItem is read on the device as four int4");

struct Plan {
    int n_seqs = 0, n_heads = 0, chunk_size = 0, tpp_threshold = 1, n_ctas = 1;
    bool split_phases = false;
    std::vector<PlanItem> items;          // chunk-first items first, short tails last
    int n_items_cf = 0;                   // how many of them are chunk-first items
    int n_items_short = 0;                // how many, after the persistent kernel's items, are short tails for the warp-per-item kernel
    bool short_all_empty = false;         // every short tail was empty when the plan was built (freshly reserved tails)
    int32_t short_slot_base = 0;          // first partial row (per-item numbering) of the short tails
    int n_items_wide = 0;                 // how many at the END of the list are wide items for the tcgen05 kernel
    std::vector<int32_t> wide_chunks;     // chunk lists of the wide items
    std::vector<int32_t> merge_off, merge_slots;
    int max_merge_len = 0;                // pieces of the row that has most
    std::vector<ca_chunk_info> infos;     // the input, kept so that the path lists can be built later
    bool has_paths = false;               // path_* are filled (build_paths)
    std::vector<int32_t> path_off, path_chunks, path_tokens;
    std::vector<int32_t> tail_chunk, tail_tokens;
    ca_plan_stats stats{};
};

// partial rows an item emits: a one-row item combines its warps on chip and writes one row, a
// wider item writes one row per (token split, query row)
inline int item_slots(int n_rows, int splits) { return n_rows == 1 ? 1 : n_rows * (splits > 1 ? splits : 1); }

// Returns an empty string on success, else the reason the input was rejected.
std::string build_plan(Plan& plan, const ca_chunk_info* infos, int n_infos, int n_seqs, int n_heads,
                       int chunk_size, int tpp_threshold, int n_ctas, int64_t max_chunks,
                       bool split_phases, int d_head, int esize, bool fast_path, bool seq_first_tensor,
                       int wide_mode = 1,   // 0: never route runs to the tcgen05 kernel, 1: by cost, 2: every shared run
                       bool want_paths = true);  // also build the per-row path lists of the any-geometry kernel
// The per-row path lists (path_off / path_chunks / path_tokens) from plan.infos, for a plan built without them.
void build_paths(Plan& plan);

}  // namespace ca
