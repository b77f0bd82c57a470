// Host-side work-list builder; see ca_plan.h for what it produces and why.
#include "ca_plan.h"

#include <algorithm>
#include <cstdio>
#include <unordered_map>

namespace ca {
namespace {

// A unit is the same for every head (heads differ only in which tile of a chunk they read and where their partial
// rows go), so units, items and merge lists are built ONCE and the kernels expand them over the heads.
struct Unit {
    const int32_t* chunks;        // pool slots, root to leaf
    int32_t n_chunks;
    int32_t row_begin, n_rows, splits, last_tokens;
    bool tail;                    // last tile is a sequence's tail chunk
};

std::string fmt(const char* f, long a = 0, long b = 0, long c = 0) {
    char buf[256];
    snprintf(buf, sizeof(buf), f, a, b, c);
    return buf;
}

// Cut the units [ubegin, uend) into items.  Guided self-scheduling: an item takes
// remaining_tiles / n_ctas tiles, clamped to [1, MAX_TILES_PER_ITEM], so the list starts with
// full-size items and ends with single tiles.
void cut_units(Plan& plan, const std::vector<Unit>& units, size_t ubegin, size_t uend, int n_ctas, int n_heads,
               int32_t& n_slots, int64_t tiles_elsewhere = 0) {
    // tiles_elsewhere: work of the same step that other kernels do (the short tails); counting it keeps
    // the pieces of shared runs long - every piece of a run costs a partial row per sharer, so they
    // are not tapered down to single tiles for the sake of the last microsecond
    // every item exists once per head: the work that remains is counted in (tile, head) pairs
    int64_t remaining = tiles_elsewhere;
    for (size_t u = ubegin; u < uend; u++) remaining += (int64_t)units[u].n_chunks * n_heads;
    for (size_t u = ubegin; u < uend; u++) {
        const Unit& un = units[u];
        const int n_tiles = un.n_chunks;
        int j = 0;
        while (j < n_tiles) {
            int want = (int)std::min<int64_t>(MAX_TILES_PER_ITEM - 1, std::max<int64_t>(1, remaining / n_ctas));
            // a sequence's tail chunk (partially filled or still empty) rides along with the piece
            // before it instead of becoming an item of its own
            if (n_tiles - (j + want) == 1 && un.tail) want++;
            const int len = std::min(want, n_tiles - j);
            plan.items.emplace_back();
            PlanItem& it = plan.items.back();
            it.n_tiles = len;
            it.head = 0;
            it.row_begin = un.row_begin;
            it.n_rows = un.n_rows;
            it.slot_base = n_slots;
            const bool has_last = (j + len == n_tiles);
            it.flags = ((un.tail && has_last) ? ITEM_FLAG_TAIL : 0) | (un.splits << ITEM_SPLITS_SHIFT);
            it.last_tokens = has_last ? un.last_tokens : plan.chunk_size;
            for (int k = 0; k < len; k++) it.chunk[k] = un.chunks[j + k];
            n_slots += item_slots(un.n_rows, un.splits);
            j += len;
            remaining -= (int64_t)len * n_heads;
        }
    }
}

}  // namespace

// The root-to-leaf chunk list of every row (CSR), read by the any-geometry kernel only.
void build_paths(Plan& plan) {
    const int n_seqs = plan.n_seqs;
    plan.path_off.assign((size_t)n_seqs + 1, 0);
    for (const ca_chunk_info& ci : plan.infos)
        for (int s = ci.seq_begin; s < ci.seq_end; s++) plan.path_off[s + 1]++;
    for (int s = 0; s < n_seqs; s++) plan.path_off[s + 1] += plan.path_off[s];
    const int64_t total = plan.path_off[n_seqs];
    plan.path_chunks.resize(total);
    plan.path_tokens.resize(total);
    std::vector<int32_t> cursor(plan.path_off.begin(), plan.path_off.end() - 1);
    for (const ca_chunk_info& ci : plan.infos)
        for (int s = ci.seq_begin; s < ci.seq_end; s++) {
            const int32_t p = cursor[s]++;
            plan.path_chunks[p] = ci.chunk_id;
            plan.path_tokens[p] = ci.n_tokens;
        }
    plan.has_paths = true;
}

std::string build_plan(Plan& plan, const ca_chunk_info* infos, int n_infos, int n_seqs, int n_heads,
                       int chunk_size, int tpp_threshold, int n_ctas, int64_t max_chunks,
                       bool split_phases, int d_head, int esize, bool fast_path, bool seq_first_tensor, int wide_mode,
                       bool want_paths) {
    // the vectors keep their capacity from one rebuild to the next
    plan.items.clear();
    plan.wide_chunks.clear();
    plan.n_items_wide = 0;
    plan.merge_slots.clear();
    plan.path_chunks.clear();
    plan.path_tokens.clear();
    plan.tail_chunk.clear();
    plan.tail_tokens.clear();
    plan.n_items_cf = 0;
    plan.n_items_short = 0;
    plan.n_ctas = 1;
    plan.stats = ca_plan_stats{};
    if (n_infos < 0 || n_seqs < 0 || n_heads <= 0 || chunk_size <= 0 || n_ctas <= 0)
        return "negative or zero size";
    if (n_infos > 0 && infos == nullptr) return "infos is null";
    if (tpp_threshold < 1) tpp_threshold = 1;
    plan.n_seqs = n_seqs;
    plan.n_heads = n_heads;
    plan.chunk_size = chunk_size;
    plan.tpp_threshold = tpp_threshold;
    plan.split_phases = split_phases;

    // ---- validate; every row must be covered and end in a chunk of its own ---------------------------------
    // (nothing here expands a shared chunk over its rows: the per-row path lists, which only the any-geometry
    // kernel reads, are built on demand by build_paths)
    plan.infos.assign(infos, infos + n_infos);
    plan.has_paths = false;
    std::vector<int32_t> cover((size_t)n_seqs + 1, 0);   // difference array of the rows the entries serve
    std::vector<int32_t> leaf((size_t)n_seqs, -1);       // the last single-row entry of each row
    int64_t unique_tokens = 0;
    for (int i = 0; i < n_infos; i++) {
        const ca_chunk_info& ci = infos[i];
        if (ci.chunk_id < 0 || ci.chunk_id >= max_chunks)
            return fmt("chunk_id %ld of entry %ld outside the pool (%ld chunks)", ci.chunk_id, i, (long)max_chunks);
        if (ci.n_tokens < 0 || ci.n_tokens > chunk_size)
            return fmt("n_tokens %ld of entry %ld outside [0, %ld]", ci.n_tokens, i, chunk_size);
        if (ci.seq_begin < 0 || ci.seq_begin >= ci.seq_end || ci.seq_end > n_seqs)
            return fmt("row range [%ld, %ld) of entry %ld is empty or outside the batch", ci.seq_begin, ci.seq_end, i);
        cover[ci.seq_begin]++;
        cover[ci.seq_end]--;
        if (ci.seq_end - ci.seq_begin == 1) leaf[ci.seq_begin] = i;
        unique_tokens += ci.n_tokens;
    }
    for (int s = 0, run = 0; s < n_seqs; s++) {
        run += cover[s];
        if (run == 0) return fmt("row %ld is served by no chunk", s);
        if (leaf[s] < 0) return fmt("last chunk of row %ld is shared with other rows; every row needs its own tail", s);
    }
    // the list is depth-first: an entry that serves several rows lies before the leaf of each of them
    for (int i = 0; i < n_infos; i++) {
        const ca_chunk_info& ci = infos[i];
        if (ci.seq_end - ci.seq_begin == 1) continue;
        for (int s = ci.seq_begin; s < ci.seq_end; s++)
            if (leaf[s] < i)
                return fmt("last chunk of row %ld is shared by %ld rows; every row needs its own tail", s, ci.seq_end - ci.seq_begin);
    }
    // the leaf of every row is private to it: new tokens are appended there
    plan.tail_chunk.resize(n_seqs);
    plan.tail_tokens.resize(n_seqs);
    for (int s = 0; s < n_seqs; s++) {
        plan.tail_chunk[s] = infos[leaf[s]].chunk_id;
        plan.tail_tokens[s] = infos[leaf[s]].n_tokens;
    }

    plan.stats.unique_kv_bytes = unique_tokens * (int64_t)n_heads * d_head * 2 * esize;
    plan.stats.n_chunks = n_infos;
    plan.stats.fast_path = fast_path ? 1 : 0;
    plan.stats.kernels_per_step = 1;
    plan.merge_off.assign((size_t)n_seqs + 1, 0);
    if (want_paths || !fast_path) build_paths(plan);
    if (!fast_path) {
        plan.n_ctas = 0;
        return "";
    }

    // ---- classify chunks, group shared ones into runs ----------------------------------------------
    struct Run { int32_t b, e; std::vector<int32_t> chunks; };
    std::vector<Run> runs;
    std::unordered_map<uint64_t, int> run_of;
    std::vector<char> shared(n_infos, 0);
    for (int i = 0; i < n_infos; i++) {
        const ca_chunk_info& ci = infos[i];
        const int n = ci.seq_end - ci.seq_begin;
        if (n > tpp_threshold && ci.n_tokens == chunk_size) {
            shared[i] = 1;
            plan.stats.n_shared_chunks++;
            const uint64_t key = ((uint64_t)(uint32_t)ci.seq_begin << 32) | (uint32_t)ci.seq_end;
            auto f = run_of.find(key);
            int r;
            if (f == run_of.end()) {
                r = (int)runs.size();
                run_of.emplace(key, r);
                runs.push_back(Run{ci.seq_begin, ci.seq_end, {}});
            } else {
                r = f->second;
            }
            runs[r].chunks.push_back(ci.chunk_id);
        }
    }
    plan.stats.n_runs = (int)runs.size();

    // ---- which runs go to the tcgen05 kernel ---------------------------------------------------------------
    std::vector<char> run_wide(runs.size(), 0);
    if (wide_mode == 2) {
        for (size_t r = 0; r < runs.size(); r++) run_wide[r] = 1;
    } else if (wide_mode == 1) {
        double flops = 0;
        for (const Run& r : runs)
            if (r.e - r.b > WIDE_MIN_ROWS) flops += 4.0 * chunk_size * d_head * (double)(r.e - r.b) * (double)r.chunks.size() * n_heads;
        const double t_mma = flops / WIDE_MMA_SYNC_FLOPS, t_hbm = (double)plan.stats.unique_kv_bytes / WIDE_HBM_BYTES_PER_S;
        if (t_mma > 0.5 * t_hbm)
            for (size_t r = 0; r < runs.size(); r++) run_wide[r] = runs[r].e - runs[r].b > WIDE_MIN_ROWS ? 1 : 0;
    }

    // ---- units ---------------------------------------------------------------------------------------------
    std::vector<Unit> units;
    units.reserve(runs.size() * 2 + (size_t)n_seqs);
    for (size_t ri = 0; ri < runs.size(); ri++) {
        Run& r = runs[ri];
        if (run_wide[ri]) continue;
        const int n = r.e - r.b;
        const int n_blocks = (n + MAX_ROWS_PER_ITEM - 1) / MAX_ROWS_PER_ITEM;
        const int rows_per_block = (n + n_blocks - 1) / n_blocks;
        for (int blk = 0; blk < n_blocks; blk++) {
            const int rb = r.b + blk * rows_per_block;
            const int rows = std::min(rows_per_block, r.e - rb);
            if (rows <= 0) continue;
            const int splits = rows <= 16 ? 4 : (rows <= 32 ? 2 : 1);
            units.push_back(Unit{r.chunks.data(), (int32_t)r.chunks.size(), rb, rows, splits, chunk_size, false});
        }
    }
    const size_t n_units_cf = units.size();
    // The private chunks of every row, in path order (CSR): only the chunks that are NOT shared are expanded over
    // their rows, and those serve a single row unless tpp_threshold was raised.
    std::vector<int32_t> priv_off((size_t)n_seqs + 1, 0);
    for (int i = 0; i < n_infos; i++)
        if (!shared[i])
            for (int s = infos[i].seq_begin; s < infos[i].seq_end; s++) {
                // a non-final private tile must be full: only the tail may be partially filled
                if (i != leaf[s] && infos[i].n_tokens != chunk_size)
                    return fmt("row %ld has a partially filled chunk that is not its tail", s);
                priv_off[s + 1]++;
            }
    for (int s = 0; s < n_seqs; s++) priv_off[s + 1] += priv_off[s];
    std::vector<int32_t> priv_arena((size_t)priv_off[n_seqs]);
    {
        std::vector<int32_t> cursor(priv_off.begin(), priv_off.end() - 1);
        for (int i = 0; i < n_infos; i++)
            if (!shared[i])
                for (int s = infos[i].seq_begin; s < infos[i].seq_end; s++) priv_arena[cursor[s]++] = infos[i].chunk_id;
    }
    // Sequences whose private part is a single chunk (a short tail).  When there are many of them they
    // are not walked by the persistent kernel, where an item costs the same whatever its size, but by
    // a kernel of their own with one half-warp per (sequence, head); their items follow the persistent kernel's.
    std::vector<Unit> short_units;
    bool route_short = false;
    if (seq_first_tensor) {
        int64_t n_short = 0;
        for (int s = 0; s < n_seqs; s++) n_short += priv_off[s + 1] - priv_off[s] == 1 ? 1 : 0;
        route_short = n_short * n_heads > 4 * (int64_t)n_ctas;  // fewer are cheaper inside the persistent kernel than a launch of their own
        if (route_short) short_units.reserve((size_t)n_seqs);
    }
    for (int s = 0; s < n_seqs; s++) {
        const int32_t n_priv = priv_off[s + 1] - priv_off[s];
        std::vector<Unit>& dst = (route_short && n_priv == 1) ? short_units : units;
        dst.push_back(Unit{priv_arena.data() + priv_off[s], n_priv, s, 1, seq_first_tensor ? 4 : 0, plan.tail_tokens[s], true});
    }

    // ---- items ---------------------------------------------------------------------------------------------
    int32_t n_slots = 0;
    {
        int64_t tiles = 0;
        for (const Unit& u : units) tiles += u.n_chunks;
        plan.items.reserve((size_t)(tiles / 4 + units.size() + 4 * (size_t)n_ctas / n_heads + 16));
    }
    const int64_t short_tiles = (int64_t)short_units.size() * n_heads;
    if (!split_phases) {
        cut_units(plan, units, 0, units.size(), n_ctas, n_heads, n_slots, short_tiles);
        plan.n_items_cf = 0;
        for (const PlanItem& it : plan.items) plan.n_items_cf += it.n_rows > 1 ? 1 : 0;
    } else {
        // each phase is a launch of its own, with its own taper towards small items
        cut_units(plan, units, 0, n_units_cf, n_ctas, n_heads, n_slots);
        plan.n_items_cf = (int)plan.items.size();
        cut_units(plan, units, n_units_cf, units.size(), n_ctas, n_heads, n_slots);
    }
    plan.n_ctas = (int)std::min<int64_t>(n_ctas, std::max<int64_t>(1, (int64_t)plan.items.size() * n_heads));
    // the short tails: one single-tile item each, after the persistent kernel's items
    plan.n_items_short = (int)short_units.size();
    plan.short_slot_base = n_slots;
    plan.short_all_empty = !short_units.empty();
    for (const Unit& un : short_units) {
        if (un.last_tokens != 0) plan.short_all_empty = false;
        plan.items.emplace_back();
        PlanItem& it = plan.items.back();
        it.n_tiles = 1;
        it.head = 0;
        it.row_begin = un.row_begin;
        it.n_rows = 1;
        it.slot_base = n_slots++;
        it.flags = ITEM_FLAG_TAIL | (un.splits << ITEM_SPLITS_SHIFT);
        it.last_tokens = un.last_tokens;
        it.chunk[0] = un.chunks[0];
    }
    // the wide runs: (run, head, block of up to 128 rows) cut into about one wave of pieces of up to 32 chunks
    {
        int64_t n_wide_units = 0;
        for (size_t ri = 0; ri < runs.size(); ri++)
            if (run_wide[ri]) n_wide_units += (int64_t)((runs[ri].e - runs[ri].b + WIDE_MAX_ROWS - 1) / WIDE_MAX_ROWS) * n_heads;  // one per head
        const int pieces_wanted = n_wide_units > 0 ? (int)std::max<int64_t>(1, n_ctas / n_wide_units) : 1;
        for (size_t ri = 0; ri < runs.size(); ri++) {
            if (!run_wide[ri]) continue;
            const Run& r = runs[ri];
            const int n = r.e - r.b, n_chunks = (int)r.chunks.size();
            const int n_blocks = (n + WIDE_MAX_ROWS - 1) / WIDE_MAX_ROWS;
            const int rows_per_block = (n + n_blocks - 1) / n_blocks;
            // pieces of 2 .. 32 chunks, equal up to one
            int n_pieces = std::min(pieces_wanted, std::max(1, n_chunks / 2));
            n_pieces = std::max(n_pieces, (n_chunks + WIDE_MAX_TILES - 1) / WIDE_MAX_TILES);
            const int32_t list_off = (int32_t)plan.wide_chunks.size();
            plan.wide_chunks.insert(plan.wide_chunks.end(), r.chunks.begin(), r.chunks.end());
            for (int blk = 0; blk < n_blocks; blk++) {
                const int rb = r.b + blk * rows_per_block;
                const int rows = std::min(rows_per_block, r.e - rb);
                if (rows <= 0) continue;
                for (int pc = 0; pc < n_pieces; pc++) {
                    const int c0 = (int)((int64_t)n_chunks * pc / n_pieces), c1 = (int)((int64_t)n_chunks * (pc + 1) / n_pieces);
                    if (c1 <= c0) continue;
                    plan.items.emplace_back();
                    PlanItem& it = plan.items.back();
                    it.n_tiles = c1 - c0;
                    it.head = 0;
                    it.row_begin = rb;
                    it.n_rows = rows;
                    it.slot_base = n_slots;
                    it.flags = ITEM_FLAG_WIDE | (1 << ITEM_SPLITS_SHIFT);
                    it.last_tokens = chunk_size;
                    it.chunk[0] = list_off + c0;
                    n_slots += rows;
                    plan.n_items_wide++;
                }
            }
        }
    }
    {
        // launches of one step: the persistent kernel (one per phase when the phases are split), the short-tails
        // kernel, the wide-runs kernel, each only when it has items, and the merge kernel
        const int n_persistent = (int)plan.items.size() - plan.n_items_short - plan.n_items_wide;
        int k = 1;
        if (!split_phases) k += n_persistent > 0 ? 1 : 0;
        else k += (plan.n_items_cf > 0 ? 1 : 0) + (n_persistent - plan.n_items_cf > 0 ? 1 : 0);
        k += (plan.n_items_short > 0 ? 1 : 0) + (plan.n_items_wide > 0 ? 1 : 0);
        plan.stats.kernels_per_step = k;
    }

    // ---- merge lists: per ROW, the partial rows (numbered per head-agnostic item) that hold a piece of it ---------
    for (const PlanItem& it : plan.items) {
        const int splits = it.n_rows == 1 ? 1 : std::max(1, it.flags >> ITEM_SPLITS_SHIFT);
        int32_t* off = plan.merge_off.data() + (size_t)it.row_begin + 1;
        for (int r = 0; r < it.n_rows; r++, off++) *off += splits;
    }
    plan.max_merge_len = 0;
    for (size_t i = 1; i < plan.merge_off.size(); i++) {
        plan.max_merge_len = std::max(plan.max_merge_len, (int)plan.merge_off[i]);
        plan.merge_off[i] += plan.merge_off[i - 1];
    }
    plan.merge_slots.resize(plan.merge_off.back());
    {
        std::vector<int32_t> cursor(plan.merge_off.begin(), plan.merge_off.end() - 1);
        for (const PlanItem& it : plan.items) {
            const int splits = it.n_rows == 1 ? 1 : std::max(1, it.flags >> ITEM_SPLITS_SHIFT);
            // per row the slots are listed split by split, as the loops below visit them
            int32_t* cur = cursor.data() + (size_t)it.row_begin;
            for (int r = 0; r < it.n_rows; r++, cur++) {
                int32_t* dst = plan.merge_slots.data() + *cur;
                for (int sp = 0; sp < splits; sp++) dst[sp] = it.slot_base + sp * it.n_rows + r;
                *cur += splits;
            }
        }
    }
    // the counters describe the expanded work list (every item once per head)
    plan.stats.n_items = (int)plan.items.size() * n_heads;
    plan.stats.n_items_cf = plan.n_items_cf * n_heads;
    plan.stats.n_items_short = plan.n_items_short * n_heads;
    plan.stats.n_items_wide = plan.n_items_wide * n_heads;
    plan.stats.n_slots = n_slots * n_heads;
    plan.stats.n_ctas = plan.n_ctas;
    return "";
}

}  // namespace ca
