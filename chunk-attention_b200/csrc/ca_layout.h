// Pool and tile layout shared by host and device code.
//
// Pool: [max_chunks][n_heads][2 (K, V)][chunk_size][d_head] elements in one allocation.
// Tile: the chunk_size x d_head block of one (chunk, head, K|V).  A token row is cut into
// 16-byte granules; when a row holds a multiple of 8 granules, granule g of token row t is
// stored at position g ^ (t & 7).  The XOR spreads the eight rows an ldmatrix reads (same
// logical granule, consecutive tokens) over all 32 shared-memory banks after a tile has been
// bulk-copied verbatim into shared memory, and keeps a row's granules inside the row, so a
// row is still one contiguous 16-byte-aligned span for row-wise readers.
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
    int swz;    // 7 when granules are XOR-swizzled, else 0
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

// element offset of (token row t, element e) inside a tile
CA_HD int64_t tile_elem_offset(const Geometry& g, int t, int e) {
    int gran = e / g.epg;
    int within = e - gran * g.epg;
    return (int64_t)t * g.d_head + (int64_t)((gran ^ (t & g.swz)) * g.epg) + within;
}

// element offset of the K tile (kv = 0) or V tile (kv = 1) of (chunk, head) inside the pool
CA_HD int64_t tile_base_elems(const Geometry& g, int64_t chunk, int head, int kv) {
    return chunk * g.chunk_elems + ((int64_t)head * 2 + kv) * g.tile_elems;
}

}  // namespace ca
