// Sequence-first-only decode attention for any geometry (fp16 or fp32, d_head <= 256, any chunk
// size).  One warp walks the whole root-to-leaf chunk path of one (row, head) with a scalar online
// softmax in fp32 and accurate expf.  It serves the geometries the tensor-core/TMA kernels do not
// (the reference's CPU tests use fp32 with d_head 4..128 and chunk sizes 2..1024,
// tests/test_chunk_attn_cpu.py:24-385), `partition = 2` requests (the reference's
// sequence-first-only mode, cpp/chunk_attn/kernel_cpu_mkl.cpp:122-242), and is the in-library
// cross-check of the fast path.  Correctness first: it is not a performance path.
#include <cuda_fp16.h>

#include "ca_kernels.h"

namespace ca {
namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

constexpr int MAX_PER_LANE = 8;  // d_head <= 256

template <typename T>
__global__ void __launch_bounds__(128) attn_seq_generic_kernel(const GenericParams p) {
    const int pair = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (pair >= p.n_seqs * p.geo.n_heads) return;
    const int lane = threadIdx.x & 31;
    const int s = pair / p.geo.n_heads;
    const int h = pair - s * p.geo.n_heads;
    const int d = p.geo.d_head;
    const T* q = reinterpret_cast<const T*>(p.q) + (size_t)pair * d;
    const T* pool = reinterpret_cast<const T*>(p.pool);

    float qr[MAX_PER_LANE], o[MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; i++) {
        const int e = lane + 32 * i;
        qr[i] = e < d ? to_f32<T>(q[e]) * p.scale : 0.f;
        o[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int pb = p.path_off[s], pe = p.path_off[s + 1];
    for (int pi = pb; pi < pe; pi++) {
        int nt = p.path_tokens[pi];
        if (pi == pe - 1) nt = min(nt + p.delta_tokens, p.geo.chunk_size);  // the row's tail
        const T* kt = pool + tile_base_elems(p.geo, p.path_chunks[pi], h, 0);
        const T* vt = kt + p.geo.tile_elems;
        for (int t = 0; t < nt; t++) {
            float sc = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; i++) {
                const int e = lane + 32 * i;
                if (e < d) sc = fmaf(qr[i], to_f32<T>(kt[tile_elem_offset(p.geo, t, e)]), sc);
            }
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, off);
            const float mn = fmaxf(m, sc);
            const float alpha = expf(m - mn);  // exp(-inf) = 0 on the first token
            const float pj = expf(sc - mn);
            l = l * alpha + pj;
            m = mn;
#pragma unroll
            for (int i = 0; i < MAX_PER_LANE; i++) {
                const int e = lane + 32 * i;
                if (e < d) o[i] = fmaf(pj, to_f32<T>(vt[tile_elem_offset(p.geo, t, e)]), o[i] * alpha);
            }
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;  // a row with no token yields zeros
    T* out = reinterpret_cast<T*>(p.out) + (size_t)pair * d;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; i++) {
        const int e = lane + 32 * i;
        if (e < d) out[e] = from_f32<T>(o[i] * inv);
    }
}

}  // namespace

cudaError_t launch_attn_seq_generic(const GenericParams& p, int dtype, cudaStream_t stream) {
    const int pairs = p.n_seqs * p.geo.n_heads;
    if (pairs <= 0) return cudaSuccess;
    const int blocks = (pairs + 3) / 4;
    if (dtype == 0) {
        attn_seq_generic_kernel<__half><<<blocks, 128, 0, stream>>>(p);
    } else {
        attn_seq_generic_kernel<float><<<blocks, 128, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace ca
