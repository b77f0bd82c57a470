// Sequence-first-only decode attention for any geometry (fp16 or fp32, d_head <= 256, any chunk
// size), fp32 arithmetic with accurate expf.  It serves the geometries the tensor-core/TMA kernels
// do not (the reference's CPU tests use fp32 with d_head 4..128 and chunk sizes 2..1024,
// tests/test_chunk_attn_cpu.py:24-385), `partition = 2` requests (the reference's
// sequence-first-only mode, cpp/chunk_attn/kernel_cpu_mkl.cpp:122-242), and is the in-library
// cross-check of the fast path.
//
// One CTA of 4 warps per (row, head).  The row's root-to-leaf chunk path is cut into blocks of 32
// tokens which the warps take in turn.  For a block, lane j computes the score of token j (a dot
// product along the token's K row, read in 16-byte granules against the query held in shared
// memory), the block's maximum and sum come from warp shuffles, and the P.V update walks the 32
// tokens with each lane owning one or two 16-byte granules of the output row (coalesced V reads).
// The four warps' (max, sum, O) are combined through shared memory at the end.  Rows whose length
// is not a whole number of 16-byte granules (odd d_head), or an unaligned pool, take an element-wise
// variant of the same walk.
#include <cuda_fp16.h>

#include "ca_kernels.h"

namespace ca {
namespace {

constexpr int GEN_WARPS = 4;
constexpr int GEN_MAX_D = 256;

template <typename T> struct Gran;  // one 16-byte granule of T as floats
template <> struct Gran<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Gran<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __half* p, float* out) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(h[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
};
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// VEC: rows are whole 16-byte granules (geo.epg > 1); a lane owns granules lane and lane + 32 of the
// output row.  Otherwise a lane owns elements lane + 32 i.
template <typename T, bool VEC>
__global__ void __launch_bounds__(GEN_WARPS * 32) attn_seq_generic_kernel(const GenericParams p) {
    constexpr int EPG = Gran<T>::N;
    constexpr int OWN = VEC ? 2 * EPG : GEN_MAX_D / 32;  // output elements a lane may own
    __shared__ float q_s[GEN_MAX_D];
    __shared__ float part[GEN_WARPS][GEN_MAX_D + 2];

    const int pair = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int s = pair / p.geo.n_heads;
    const int h = pair - s * p.geo.n_heads;
    const int d = p.geo.d_head;
    const int gpr = p.geo.gpr;
    const T* pool = reinterpret_cast<const T*>(p.pool);
    {
        const T* q = reinterpret_cast<const T*>(p.q) + (size_t)pair * d;
        for (int e = threadIdx.x; e < d; e += blockDim.x) q_s[e] = to_f32<T>(q[e]) * p.scale;
    }
    __syncthreads();

    float o[OWN];
#pragma unroll
    for (int i = 0; i < OWN; i++) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int pb = p.path_off[s], pe = p.path_off[s + 1];
    int turn = 0;  // blocks are dealt to the warps round-robin
    for (int pi = pb; pi < pe; pi++) {
        int nt = p.path_tokens[pi];
        if (pi == pe - 1) nt = min(nt + p.delta_tokens, p.geo.chunk_size);  // the row's tail
        const T* kt = pool + tile_base_elems(p.geo, p.path_chunks[pi], h, 0);
        const T* vt = kt + p.geo.tile_elems;
        for (int t0 = 0; t0 < nt; t0 += 32, turn++) {
            if ((turn & (GEN_WARPS - 1)) != warp) continue;
            const int nv = min(32, nt - t0);
            const int t = t0 + lane;
            // ---- scores: lane j <-> token t0 + j
            float sc = -INFINITY;
            if (lane < nv) {
                float acc = 0.f;
                if (VEC) {
                    for (int g = 0; g < gpr; g++) {
                        float kf[EPG];
                        Gran<T>::load(kt + tile_granule_index(p.geo, t, g) * EPG, kf);
#pragma unroll
                        for (int k = 0; k < EPG; k++) acc = fmaf(q_s[g * EPG + k], kf[k], acc);
                    }
                } else {
                    for (int e = 0; e < d; e++) acc = fmaf(q_s[e], to_f32<T>(kt[tile_elem_offset(p.geo, t, e)]), acc);
                }
                sc = acc;
            }
            // ---- online softmax over the block
            const float mn = fmaxf(m, warp_max(sc));
            const float alpha = expf(m - mn);  // exp(-inf) = 0 before the first token
            const float pj = lane < nv ? expf(sc - mn) : 0.f;
            l = l * alpha + warp_sum(pj);
            m = mn;
#pragma unroll
            for (int i = 0; i < OWN; i++) o[i] *= alpha;
            // ---- O += P V: every lane walks the block's tokens over the elements it owns
            for (int j = 0; j < nv; j++) {
                const float pw = __shfl_sync(0xffffffffu, pj, j);
                const int tj = t0 + j;
                if (VEC) {
#pragma unroll
                    for (int gi = 0; gi < 2; gi++) {
                        const int g = lane + 32 * gi;
                        if (g < gpr) {
                            float vf[EPG];
                            Gran<T>::load(vt + tile_granule_index(p.geo, tj, g) * EPG, vf);
#pragma unroll
                            for (int k = 0; k < EPG; k++) o[gi * EPG + k] = fmaf(pw, vf[k], o[gi * EPG + k]);
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < OWN; i++) {
                        const int e = lane + 32 * i;
                        if (e < d) o[i] = fmaf(pw, to_f32<T>(vt[tile_elem_offset(p.geo, tj, e)]), o[i]);
                    }
                }
            }
        }
    }

    // ---- combine the warps
    if (lane == 0) {
        part[warp][GEN_MAX_D] = m;
        part[warp][GEN_MAX_D + 1] = l;
    }
    if (VEC) {
#pragma unroll
        for (int gi = 0; gi < 2; gi++) {
            const int g = lane + 32 * gi;
            if (g < gpr) {
#pragma unroll
                for (int k = 0; k < EPG; k++) part[warp][g * EPG + k] = o[gi * EPG + k];
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < OWN; i++) {
            const int e = lane + 32 * i;
            if (e < d) part[warp][e] = o[i];
        }
    }
    __syncthreads();
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; w++) mm = fmaxf(mm, part[w][GEN_MAX_D]);
    float wgt[GEN_WARPS];
    float ll = 0.f;
#pragma unroll
    for (int w = 0; w < GEN_WARPS; w++) {
        // a warp that saw no token has max -inf and sum 0: it contributes nothing
        wgt[w] = part[w][GEN_MAX_D + 1] > 0.f ? expf(part[w][GEN_MAX_D] - mm) : 0.f;
        ll = fmaf(wgt[w], part[w][GEN_MAX_D + 1], ll);
    }
    const float inv = ll > 0.f ? 1.f / ll : 0.f;  // a row with no token yields zeros
    T* out = reinterpret_cast<T*>(p.out) + (size_t)pair * d;
    for (int e = threadIdx.x; e < d; e += blockDim.x) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < GEN_WARPS; w++) acc = fmaf(wgt[w], part[w][e], acc);
        out[e] = from_f32<T>(acc * inv);
    }
}

}  // namespace

cudaError_t launch_attn_seq_generic(const GenericParams& p, int dtype, cudaStream_t stream) {
    const int pairs = p.n_seqs * p.geo.n_heads;
    if (pairs <= 0) return cudaSuccess;
    if (p.geo.d_head > GEN_MAX_D) return cudaErrorInvalidValue;
    // 16-byte granule reads need the pool base aligned (rows and tiles then are, too)
    const bool vec = p.geo.epg > 1 && reinterpret_cast<uintptr_t>(p.pool) % 16 == 0;
    if (dtype == 0) {
        if (vec) attn_seq_generic_kernel<__half, true><<<pairs, GEN_WARPS * 32, 0, stream>>>(p);
        else attn_seq_generic_kernel<__half, false><<<pairs, GEN_WARPS * 32, 0, stream>>>(p);
    } else {
        if (vec) attn_seq_generic_kernel<float, true><<<pairs, GEN_WARPS * 32, 0, stream>>>(p);
        else attn_seq_generic_kernel<float, false><<<pairs, GEN_WARPS * 32, 0, stream>>>(p);
    }
    return cudaGetLastError();
}

}  // namespace ca
