// Pool and tile layout shared by host and device code.
//
// Pool: [max_chunks][n_heads][2 (K, V)] tiles in one allocation; a tile is the chunk_size x d_head block of
// one (chunk, head, K|V).  A token row is cut into 16-byte granules.  When a row holds a multiple of 8
// granules (every geometry the tensor-core kernels serve), the tile is stored as PANELS:
//
//     tile = [d_head * esize / 128 panels][chunk_size token rows][8 granules of 16 bytes]
//
// panel p holds bytes [128 p, 128 p + 128) of every token row, one 128-byte line per token, and inside a line
// granule c of token row t sits at position c ^ (t & 7).  This is exactly the canonical 128-byte-swizzled
// shared-memory layout of the Blackwell tensor cores (tcgen05.mma matrix descriptors, SWIZZLE_128B): a K
// panel is a K-major operand of 64 elements (fp16), a V panel an MN-major one, so a tile bulk-copied VERBATIM
// into shared memory (1024-byte aligned) can be handed to tcgen05.mma by descriptor, with no tensor map and
// no TMA swizzle mode.  The same XOR makes the ldmatrix patterns of the mma.sync path (8 consecutive tokens x
// one granule, plain for K, .trans for V) and row-wise 128-bit readers bank-conflict free.
// Other geometries (rows that are not a multiple of 128 bytes) are stored row-major, unswizzled.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define CA_HD __host__ __device__ __forceinline__
#else
#define CA_HD inline
#endif

namespace ca {

struct Geometry {
    int n_heads;
    int d_head;
    int chunk_size;
    int esize;  // bytes per element
    int epg;    // elements per 16-byte granule, or 1 when rows are not a whole number of granules
    int gpr;    // granules per token row (d_head / epg)
    int swz;    // 7 when the tile is stored as swizzled 128-byte panels, else 0 (row-major)
    int64_t tile_elems;   // chunk_size * d_head
    int64_t chunk_elems;  // n_heads * 2 * tile_elems
};

CA_HD Geometry make_geometry(int n_heads, int d_head, int chunk_size, int esize) {
    Geometry g;
    g.n_heads = n_heads;
    g.d_head = d_head;
    g.chunk_size = chunk_size;
    g.esize = esize;
    int per16 = 16 / esize;
    g.epg = (d_head % per16 == 0) ? per16 : 1;
    g.gpr = d_head / g.epg;
    g.swz = (g.epg > 1 && g.gpr % 8 == 0) ? 7 : 0;
    g.tile_elems = (int64_t)chunk_size * d_head;
    g.chunk_elems = (int64_t)n_heads * 2 * g.tile_elems;
    return g;
}

// index, in 16-byte units from the start of the tile, of granule `gran` of token row t (geometries with
// whole-granule rows only)
CA_HD int64_t tile_granule_index(const Geometry& g, int t, int gran) {
    if (g.swz) return ((int64_t)(gran >> 3) * g.chunk_size + t) * 8 + ((gran & 7) ^ (t & 7));
    return (int64_t)t * g.gpr + gran;
}

// element offset of (token row t, element e) inside a tile
CA_HD int64_t tile_elem_offset(const Geometry& g, int t, int e) {
    int gran = e / g.epg;
    int within = e - gran * g.epg;
    if (g.epg == 1) return (int64_t)t * g.d_head + e;
    return tile_granule_index(g, t, gran) * g.epg + within;
}

// element offset of the K tile (kv = 0) or V tile (kv = 1) of (chunk, head) inside the pool
CA_HD int64_t tile_base_elems(const Geometry& g, int64_t chunk, int head, int kv) {
    return chunk * g.chunk_elems + ((int64_t)head * 2 + kv) * g.tile_elems;
}

}  // namespace ca
