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
//    is a chunk-first unit and produces ONE partial per row for the whole chain instead of one
//    per chunk;
//  * the remaining chunks of a sequence (its private tail) x head are a sequence-first unit;
//  * every unit is a list of 32 KiB K+V tiles.  The units are laid end to end into one stream
//    of weighted tiles, and the stream is cut into n_ctas equal parts; a unit that straddles a
//    cut becomes two ITEMS, each emitting its own partial.  Each persistent CTA walks its
//    items in order, so its TMA ring never drains between items;
//  * merge lists name, per (row, head), the partial slots the merge kernel combines.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/chunk_attn_b200.h"

namespace ca {

constexpr int ITEM_FLAG_TAIL = 1;     // last tile of the item is the sequence's tail chunk
constexpr int ITEM_SPLITS_SHIFT = 8;  // flags >> 8: token splits of a tensor-core item (4, 2, 1);
                                      // 0 = one-row item walked on CUDA cores
constexpr int MAX_ROWS_PER_ITEM = 64; // 4 consumer warps x 16 rows

struct PlanItem {
    int32_t tile_begin;   // index into tile_chunks
    int32_t n_tiles;
    int32_t head;
    int32_t row_begin;    // first row of q / out this item serves
    int32_t n_rows;       // 1: sequence-first item; >= 2: chunk-first item
    int32_t slot_base;    // first partial slot
    int32_t flags;
    int32_t last_tokens;  // tokens in the last tile when the plan was built
};
static_assert(sizeof(PlanItem) == 32, "PlanItem is read on the device as two int4");

struct Plan {
    int n_seqs = 0, n_heads = 0, chunk_size = 0, tpp_threshold = 1, n_ctas = 1;
    bool split_phases = false;
    std::vector<PlanItem> items;          // chunk-first items first when split_phases
    std::vector<int32_t> tile_chunks;
    std::vector<int32_t> cta_item_begin;     // fused schedule (n_ctas + 1)
    std::vector<int32_t> cta_item_begin_cf;  // split schedules
    std::vector<int32_t> cta_item_begin_sf;
    std::vector<int32_t> merge_off, merge_slots;
    std::vector<int32_t> path_off, path_chunks, path_tokens;
    std::vector<int32_t> tail_chunk, tail_tokens;
    int n_items_cf = 0;
    ca_plan_stats stats{};
};

// Returns an empty string on success, else the reason the input was rejected.
std::string build_plan(Plan& plan, const ca_chunk_info* infos, int n_infos, int n_seqs, int n_heads,
                       int chunk_size, int tpp_threshold, int n_ctas, int64_t max_chunks,
                       bool split_phases, int d_head, int esize, bool fast_path, bool seq_first_tensor);

}  // namespace ca
