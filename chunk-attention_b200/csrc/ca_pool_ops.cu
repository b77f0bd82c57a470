// Device-side maintenance of the chunk pool: append one token per sequence, ingest a prefill,
// write single token rows (beam forks), clone chunks (copy-on-write), read a chunk back in logical order.  All of them are pure data
// movement into / out of the swizzled tile layout (ca_layout.h) with 16-byte accesses wherever
// the geometry allows.
//
// Reference counterparts: append_kv_kernel (cpp/chunk_attn/kernel_cuda.cu:1088-1115),
// Chunk::append_tokens' two strided slice copies per chunk (cpp/chunk_attn/chunk.cpp:63-71),
// Chunk::deep_copy (cpp/chunk_attn/chunk.cpp:93-107).
#include <algorithm>

#include "ca_kernels.h"

namespace ca {
namespace {

// One thread moves one unit of K or V of one token row into its tile: a 16-byte granule (U = uint4,
// requires whole-granule rows and 16-byte aligned source rows) or a single element (U = uint16_t /
// uint32_t, any geometry and alignment).  Both land in the same swizzled positions.
template <typename U>
__device__ __forceinline__ int units_per_row(const Geometry& g) {
    return sizeof(U) == 16 ? g.gpr : g.d_head;
}
template <typename U>
__device__ __forceinline__ void move_unit(void* dst_tile, const void* src_row, const Geometry& g, int t, int unit) {
    if (sizeof(U) == 16) {
        reinterpret_cast<U*>(dst_tile)[tile_granule_index(g, t, unit)] = reinterpret_cast<const U*>(src_row)[unit];
    } else {
        reinterpret_cast<U*>(dst_tile)[tile_elem_offset(g, t, unit)] = reinterpret_cast<const U*>(src_row)[unit];
    }
}

template <typename U>
__global__ void append_kv_kernel(const AppendParams p) {
    const Geometry& g = p.geo;
    const int upr = units_per_row<U>(g);
    const int64_t total = (int64_t)p.n_seqs * g.n_heads * 2 * upr;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int unit = (int)(idx % upr);
    int64_t r = idx / upr;
    const int kv = (int)(r & 1);
    r >>= 1;
    const int h = (int)(r % g.n_heads);
    const int s = (int)(r / g.n_heads);
    const int t = p.tail_tokens[s] + p.delta_tokens;  // slot inside the tail chunk
    if (t >= g.chunk_size) return;                    // rejected on the host; never write past the tile
    const char* src = reinterpret_cast<const char*>(kv ? p.v : p.k) +
                      ((int64_t)s * g.n_heads + h) * g.d_head * g.esize;
    char* dst = reinterpret_cast<char*>(p.pool) + tile_base_elems(g, p.tail_chunk[s], h, kv) * g.esize;
    move_unit<U>(dst, src, g, t, unit);
}

template <typename U>
__global__ void scatter_prefill_kernel(const ScatterParams p) {
    const Geometry& g = p.geo;
    const int upr = units_per_row<U>(g);
    const int64_t total = (int64_t)p.n_tokens * g.n_heads * 2 * upr;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int unit = (int)(idx % upr);
    int64_t r = idx / upr;
    const int kv = (int)(r & 1);
    r >>= 1;
    const int h = (int)(r % g.n_heads);
    const int tok = (int)(r / g.n_heads);
    const int chunk = p.chunk_ids[tok / g.chunk_size];
    const int t = tok % g.chunk_size;
    const char* src = reinterpret_cast<const char*>(kv ? p.v : p.k) +
                      ((int64_t)tok * p.stride_token + (int64_t)h * p.stride_head) * g.esize;
    char* dst = reinterpret_cast<char*>(p.pool) + tile_base_elems(g, chunk, h, kv) * g.esize;
    move_unit<U>(dst, src, g, t, unit);
}

template <typename U>
__global__ void scatter_rows_kernel(const ScatterRowsParams p) {
    const Geometry& g = p.geo;
    const int upr = units_per_row<U>(g);
    const int64_t total = (int64_t)p.n_tokens * g.n_heads * 2 * upr;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int unit = (int)(idx % upr);
    int64_t r = idx / upr;
    const int kv = (int)(r & 1);
    r >>= 1;
    const int h = (int)(r % g.n_heads);
    const int tok = (int)(r / g.n_heads);
    const char* src = reinterpret_cast<const char*>(kv ? p.v : p.k) +
                      ((int64_t)tok * p.stride_token + (int64_t)h * p.stride_head) * g.esize;
    char* dst = reinterpret_cast<char*>(p.pool) + tile_base_elems(g, p.chunk_ids[tok], h, kv) * g.esize;
    move_unit<U>(dst, src, g, p.rows[tok], unit);
}

template <typename U>
__global__ void copy_chunks_kernel(const CopyParams p) {
    const int pair = blockIdx.y;
    const U* src = reinterpret_cast<const U*>(reinterpret_cast<const char*>(p.pool) + p.src[pair] * p.chunk_bytes);
    U* dst = reinterpret_cast<U*>(reinterpret_cast<char*>(p.pool) + p.dst[pair] * p.chunk_bytes);
    const int64_t n = p.chunk_bytes / (int64_t)sizeof(U);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        dst[i] = src[i];
}

template <typename E>
__global__ void read_chunk_kernel(const ReadChunkParams p) {
    const Geometry& g = p.geo;
    const int64_t total = (int64_t)g.n_heads * p.n_tokens * g.d_head;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int e = (int)(idx % g.d_head);
    const int t = (int)((idx / g.d_head) % p.n_tokens);
    const int h = (int)(idx / ((int64_t)g.d_head * p.n_tokens));
    const E* pool = reinterpret_cast<const E*>(p.pool);
    const int64_t off = tile_elem_offset(g, t, e);
    reinterpret_cast<E*>(p.k_out)[idx] = pool[tile_base_elems(g, p.chunk_id, h, 0) + off];
    reinterpret_cast<E*>(p.v_out)[idx] = pool[tile_base_elems(g, p.chunk_id, h, 1) + off];
}

inline int blocks_for(int64_t total, int threads) { return (int)((total + threads - 1) / threads); }

}  // namespace

cudaError_t launch_append_kv(const AppendParams& p, bool vec16, cudaStream_t stream) {
    const int upr = vec16 ? p.geo.gpr : p.geo.d_head;
    const int64_t total = (int64_t)p.n_seqs * p.geo.n_heads * 2 * upr;
    if (total <= 0) return cudaSuccess;
    if (vec16) {
        append_kv_kernel<uint4><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else if (p.geo.esize == 2) {
        append_kv_kernel<uint16_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else {
        append_kv_kernel<uint32_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t launch_scatter_prefill(const ScatterParams& p, bool vec16, cudaStream_t stream) {
    const int upr = vec16 ? p.geo.gpr : p.geo.d_head;
    const int64_t total = (int64_t)p.n_tokens * p.geo.n_heads * 2 * upr;
    if (total <= 0) return cudaSuccess;
    if (vec16) {
        scatter_prefill_kernel<uint4><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else if (p.geo.esize == 2) {
        scatter_prefill_kernel<uint16_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else {
        scatter_prefill_kernel<uint32_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t launch_scatter_rows(const ScatterRowsParams& p, bool vec16, cudaStream_t stream) {
    const int upr = vec16 ? p.geo.gpr : p.geo.d_head;
    const int64_t total = (int64_t)p.n_tokens * p.geo.n_heads * 2 * upr;
    if (total <= 0) return cudaSuccess;
    if (vec16) {
        scatter_rows_kernel<uint4><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else if (p.geo.esize == 2) {
        scatter_rows_kernel<uint16_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else {
        scatter_rows_kernel<uint32_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t launch_copy_chunks(const CopyParams& p, cudaStream_t stream) {
    if (p.n <= 0) return cudaSuccess;
    const bool aligned = (reinterpret_cast<uintptr_t>(p.pool) % 16 == 0);
    if (aligned && p.chunk_bytes % 16 == 0) {
        const int bx = (int)std::min<int64_t>(64, (p.chunk_bytes / 16 + 255) / 256);
        copy_chunks_kernel<uint4><<<dim3(bx, p.n), 256, 0, stream>>>(p);
    } else if (p.chunk_bytes % 4 == 0) {
        const int bx = (int)std::min<int64_t>(64, (p.chunk_bytes / 4 + 255) / 256);
        copy_chunks_kernel<uint32_t><<<dim3(bx, p.n), 256, 0, stream>>>(p);
    } else {
        const int bx = (int)std::min<int64_t>(64, (p.chunk_bytes / 2 + 255) / 256);
        copy_chunks_kernel<uint16_t><<<dim3(bx, p.n), 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

cudaError_t launch_read_chunk(const ReadChunkParams& p, cudaStream_t stream) {
    const int64_t total = (int64_t)p.geo.n_heads * p.n_tokens * p.geo.d_head;
    if (total <= 0) return cudaSuccess;
    if (p.geo.esize == 2) {
        read_chunk_kernel<uint16_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    } else {
        read_chunk_kernel<uint32_t><<<blocks_for(total, 256), 256, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace ca
