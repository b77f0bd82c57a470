// Element-wise companions of the attention path that the reference's model code imports from the
// same extension module (`chunk_attn.ops`): RMS normalisation, residual-add + RMS normalisation,
// rotary position embedding.  Written from their published semantics; the reference's own versions
// are cpp/chunk_attn/layernorm_kernels.cu:26-131 and cpp/chunk_attn/pos_encoding_kernels.cu:7-139.
//
// All three are HBM / latency bound: one CTA per token, 128-bit accesses whenever a row is a whole
// number of 16-byte granules and 16-byte aligned, the row re-read from L1 for the second pass.
// Rounding follows the reference so that results agree bit for bit: the normalised value is
// rounded to the element type BEFORE it is multiplied by the weight (in the element type), and the
// rotation's two products and their difference / sum are each rounded to the element type.
#include <cuda_fp16.h>

#include "../../include/chunk_attn_b200.h"
#include "ca_kernels.h"

namespace ca {
namespace {

template <typename T> struct Elem;
template <> struct Elem<float> {
    static __device__ __forceinline__ float to_f(float x) { return x; }
    static __device__ __forceinline__ float from_f(float x) { return x; }
    static __device__ __forceinline__ float mul(float a, float b) { return a * b; }
    static __device__ __forceinline__ float rot_x(float x, float y, float c, float s) { return x * c - y * s; }
    static __device__ __forceinline__ float rot_y(float x, float y, float c, float s) { return y * c + x * s; }
};
template <> struct Elem<__half> {
    static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
    static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
    // Each product and sum goes through float and back, one rounding to fp16 per operation, exactly
    // as the reference's element type does on the device; plain fp16 intrinsics without a rounding
    // modifier could be fused into one multiply-add with a single rounding.
    static __device__ __forceinline__ __half mul(__half a, __half b) {
        return __float2half_rn(__half2float(a) * __half2float(b));
    }
    static __device__ __forceinline__ __half rot_x(__half x, __half y, __half c, __half s) {
        return __float2half_rn(__half2float(mul(x, c)) - __half2float(mul(y, s)));
    }
    static __device__ __forceinline__ __half rot_y(__half x, __half y, __half c, __half s) {
        return __float2half_rn(__half2float(mul(y, c)) + __half2float(mul(x, s)));
    }
};

__device__ __forceinline__ float block_sum(float v) {
    __shared__ float warp_sums[32];
    __shared__ float total;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_sums[warp] = v;
    __syncthreads();
    if (warp == 0) {
        const int n_warps = (blockDim.x + 31) >> 5;
        float s = lane < n_warps ? warp_sums[lane] : 0.f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) total = s;
    }
    __syncthreads();
    return total;
}

// VEC elements per access (16 bytes when the row allows it, else 1).  ADD: x = input + residual is
// written back to residual first and the output overwrites input (the fused form); otherwise
// out = norm(input).
template <typename T, int VEC, bool ADD>
__global__ void rms_norm_kernel(T* __restrict__ out, T* __restrict__ input, T* __restrict__ residual,
                                const T* __restrict__ weight, float epsilon, int hidden) {
    struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
    const size_t row = (size_t)blockIdx.x * hidden;
    const int n_vec = hidden / VEC;
    const Pack* in_v = reinterpret_cast<const Pack*>(input + row);
    Pack* res_v = reinterpret_cast<Pack*>(residual ? residual + row : nullptr);
    float ss = 0.f;
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        Pack a = in_v[i];
        if (ADD) {
            Pack r = res_v[i];
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                const float x = Elem<T>::to_f(a.v[k]) + Elem<T>::to_f(r.v[k]);
                ss += x * x;                  // the sum of squares uses the unrounded sum
                r.v[k] = Elem<T>::from_f(x);  // the residual stream keeps the rounded one
            }
            res_v[i] = r;
        } else {
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                const float x = Elem<T>::to_f(a.v[k]);
                ss += x * x;
            }
        }
    }
    const float inv = rsqrtf(block_sum(ss) / hidden + epsilon);
    const Pack* w_v = reinterpret_cast<const Pack*>(weight);
    const Pack* src_v = ADD ? res_v : in_v;  // second pass: this CTA's own lines, still in L1
    Pack* dst_v = reinterpret_cast<Pack*>((ADD ? input : out) + row);
    for (int i = threadIdx.x; i < n_vec; i += blockDim.x) {
        const Pack a = src_v[i];
        const Pack w = w_v[i];
        Pack o;
#pragma unroll
        for (int k = 0; k < VEC; k++) o.v[k] = Elem<T>::mul(Elem<T>::from_f(Elem<T>::to_f(a.v[k]) * inv), w.v[k]);
        dst_v[i] = o;
    }
}

// Rows of up to 32 * PPL packs: one WARP per token, the whole row in registers (PPL 16-byte packs per
// lane, all requested before the first is used), the sum of squares by shuffles alone - no block-wide
// barrier and eight rows in flight per CTA.  Same per-element arithmetic as rms_norm_kernel.
template <typename T, int VEC, bool ADD, int PPL>
__global__ void __launch_bounds__(256) rms_norm_warp_kernel(T* __restrict__ out, T* __restrict__ input, T* __restrict__ residual,
                                                            const T* __restrict__ weight, float epsilon, int hidden,
                                                            int num_tokens) {
    struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };
    const int token = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (token >= num_tokens) return;
    const int lane = threadIdx.x & 31;
    const size_t row = (size_t)token * hidden;
    const int n_vec = hidden / VEC;
    const Pack* in_v = reinterpret_cast<const Pack*>(input + row);
    Pack* res_v = reinterpret_cast<Pack*>(residual ? residual + row : nullptr);
    Pack a[PPL];
    float ss = 0.f;
    // four packs of the row (and of the residual) at a time: enough loads in flight, and only four
    // residual packs alive next to the row
#pragma unroll
    for (int k0 = 0; k0 < PPL; k0 += 4) {
        Pack r[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int i = lane + 32 * (k0 + k);
            if (i < n_vec) {
                a[k0 + k] = in_v[i];
                if (ADD) r[k] = res_v[i];
            }
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int i = lane + 32 * (k0 + k);
            if (i < n_vec) {
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    float x = Elem<T>::to_f(a[k0 + k].v[e]);
                    if (ADD) {
                        x += Elem<T>::to_f(r[k].v[e]);
                        a[k0 + k].v[e] = Elem<T>::from_f(x);  // the rounded sum: new residual and the value normalised
                    }
                    ss += x * x;                              // the sum of squares uses the unrounded value
                }
                if (ADD) res_v[i] = a[k0 + k];
            }
        }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = rsqrtf(ss / hidden + epsilon);
    const Pack* w_v = reinterpret_cast<const Pack*>(weight);
    Pack* dst_v = reinterpret_cast<Pack*>((ADD ? input : out) + row);
#pragma unroll
    for (int k = 0; k < PPL; k++) {
        const int i = lane + 32 * k;
        if (i < n_vec) {
            const Pack w = w_v[i];
            Pack o;
#pragma unroll
            for (int e = 0; e < VEC; e++) o.v[e] = Elem<T>::mul(Elem<T>::from_f(Elem<T>::to_f(a[k].v[e]) * inv), w.v[e]);
            dst_v[i] = o;
        }
    }
}

// One CTA per token.  A thread rotates one (x, y) pair of one head: pairs are (i, i + rot/2) in the
// NeoX layout and (2i, 2i + 1) in the GPT-J layout.
template <typename T, bool NEOX>
__global__ void rotary_kernel(const int64_t* __restrict__ positions, T* __restrict__ query, T* __restrict__ key,
                              const T* __restrict__ cos_sin_cache, int rot_dim, int64_t q_stride, int64_t k_stride,
                              int n_heads, int n_kv_heads, int head_size, int64_t max_position, int* status) {
    const int half_rot = rot_dim / 2;
    const int64_t pos = positions[blockIdx.x];
    if (max_position > 0 && (pos < 0 || pos >= max_position)) {  // outside the table: leave the token as it is
        if (status && threadIdx.x == 0) atomicCAS(status, 0, 5);
        return;
    }
    const T* cs = cos_sin_cache + pos * rot_dim;  // [cos(half_rot) | sin(half_rot)]
    const int nq = n_heads * half_rot, nk = n_kv_heads * half_rot;
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const bool is_q = i < nq;
        const int j = is_q ? i : i - nq;
        const int head = j / half_rot, r = j - head * half_rot;
        T* base = is_q ? query + (size_t)blockIdx.x * q_stride + (size_t)head * head_size
                       : key + (size_t)blockIdx.x * k_stride + (size_t)head * head_size;
        const int xi = NEOX ? r : 2 * r, yi = NEOX ? half_rot + r : 2 * r + 1;
        const T c = cs[r], s = cs[half_rot + r];
        const T x = base[xi], y = base[yi];
        base[xi] = Elem<T>::rot_x(x, y, c, s);
        base[yi] = Elem<T>::rot_y(x, y, c, s);
    }
}

// The same rotation, 16 bytes at a time.  NeoX layout: a thread takes granule u of the x half of a head and
// the matching granule of the y half (and of the cos and sin halves of the table row).  GPT-J layout: a
// granule holds EPG / 2 interleaved (x, y) pairs and needs half a granule each of cos and sin.  Element
// arithmetic is that of rotary_kernel, so the results are bit-identical.
template <typename T, bool NEOX>
__global__ void rotary_vec_kernel(const int64_t* __restrict__ positions, T* __restrict__ query, T* __restrict__ key,
                                  const T* __restrict__ cos_sin_cache, int rot_dim, int64_t q_stride, int64_t k_stride,
                                  int n_heads, int n_kv_heads, int head_size, int64_t max_position, int* status) {
    constexpr int EPG = 16 / sizeof(T);
    struct alignas(16) Pack { T v[EPG]; };
    struct alignas(8) HalfPack { T v[EPG / 2]; };
    const int half_rot = rot_dim / 2;
    const int64_t pos = positions[blockIdx.x];
    if (max_position > 0 && (pos < 0 || pos >= max_position)) {  // outside the table: leave the token as it is
        if (status && threadIdx.x == 0) atomicCAS(status, 0, 5);
        return;
    }
    const T* cs = cos_sin_cache + pos * rot_dim;
    const int units_per_head = NEOX ? half_rot / EPG : rot_dim / EPG;
    const int nq = n_heads * units_per_head, nk = n_kv_heads * units_per_head;
    for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
        const bool is_q = i < nq;
        const int j = is_q ? i : i - nq;
        const int head = j / units_per_head, u = j - head * units_per_head;
        T* base = is_q ? query + (size_t)blockIdx.x * q_stride + (size_t)head * head_size
                       : key + (size_t)blockIdx.x * k_stride + (size_t)head * head_size;
        if (NEOX) {
            Pack* xp = reinterpret_cast<Pack*>(base + u * EPG);
            Pack* yp = reinterpret_cast<Pack*>(base + half_rot + u * EPG);
            const Pack c = *reinterpret_cast<const Pack*>(cs + u * EPG);
            const Pack sn = *reinterpret_cast<const Pack*>(cs + half_rot + u * EPG);
            const Pack x = *xp, y = *yp;
            Pack xo, yo;
#pragma unroll
            for (int k = 0; k < EPG; k++) {
                xo.v[k] = Elem<T>::rot_x(x.v[k], y.v[k], c.v[k], sn.v[k]);
                yo.v[k] = Elem<T>::rot_y(x.v[k], y.v[k], c.v[k], sn.v[k]);
            }
            *xp = xo;
            *yp = yo;
        } else {
            Pack* pp = reinterpret_cast<Pack*>(base + u * EPG);
            const HalfPack c = *reinterpret_cast<const HalfPack*>(cs + u * (EPG / 2));
            const HalfPack sn = *reinterpret_cast<const HalfPack*>(cs + half_rot + u * (EPG / 2));
            const Pack v = *pp;
            Pack o;
#pragma unroll
            for (int k = 0; k < EPG / 2; k++) {
                o.v[2 * k] = Elem<T>::rot_x(v.v[2 * k], v.v[2 * k + 1], c.v[k], sn.v[k]);
                o.v[2 * k + 1] = Elem<T>::rot_y(v.v[2 * k], v.v[2 * k + 1], c.v[k], sn.v[k]);
            }
            *pp = o;
        }
    }
}

int threads_for(int work) {
    int t = ((work + 31) / 32) * 32;
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

template <typename T, bool ADD>
cudaError_t launch_norm(void* out, void* input, void* residual, const void* weight, float eps, int num_tokens,
                        int hidden, cudaStream_t stream) {
    constexpr int VEC = 16 / sizeof(T);
    auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    const bool vec = hidden % VEC == 0 && aligned(input) && aligned(weight) && (ADD ? aligned(residual) : aligned(out));
    const int n_vec = hidden / VEC;
    if (!ADD && vec && n_vec <= 32 * 16 && num_tokens >= 1024) {
        // rows that fit a warp's registers, and enough of them to fill the GPU with warps (measured at
        // 65 536 x 4096 fp16: 164 us against 304 us for the CTA-per-row kernel; the fused add + norm form
        // is faster CTA-per-row, 359 us against 462 us, and stays there)
        const int blocks = (num_tokens + 7) / 8;
#define CA_NORM_WARP(PPL)                                                                                         \
    rms_norm_warp_kernel<T, VEC, ADD, PPL><<<blocks, 256, 0, stream>>>(static_cast<T*>(out), static_cast<T*>(input), \
                                                                       static_cast<T*>(residual),                    \
                                                                       static_cast<const T*>(weight), eps, hidden, num_tokens)
        if (n_vec <= 32 * 4) CA_NORM_WARP(4);
        else if (n_vec <= 32 * 8) CA_NORM_WARP(8);
        else CA_NORM_WARP(16);
#undef CA_NORM_WARP
    } else if (vec) {
        rms_norm_kernel<T, VEC, ADD><<<num_tokens, threads_for(hidden / VEC), 0, stream>>>(
            static_cast<T*>(out), static_cast<T*>(input), static_cast<T*>(residual), static_cast<const T*>(weight), eps, hidden);
    } else {
        rms_norm_kernel<T, 1, ADD><<<num_tokens, threads_for(hidden), 0, stream>>>(
            static_cast<T*>(out), static_cast<T*>(input), static_cast<T*>(residual), static_cast<const T*>(weight), eps, hidden);
    }
    return cudaGetLastError();
}

int ops_fail(int code, const char* msg) {
    set_last_error(msg);
    return code;
}

}  // namespace
}  // namespace ca

extern "C" {

int ca_rms_norm(void* out, const void* input, const void* weight, float epsilon, int64_t num_tokens, int hidden_size,
                int dtype, ca_stream stream) {
    if (num_tokens < 0 || hidden_size <= 0) return ca::ops_fail(CA_ERR_INVALID, "rms_norm: bad shape");
    if (num_tokens == 0) return CA_OK;
    if (!out || !input || !weight) return ca::ops_fail(CA_ERR_INVALID, "rms_norm: null pointer");
    cudaError_t e;
    if (dtype == CA_DTYPE_F16) {
        e = ca::launch_norm<__half, false>(out, const_cast<void*>(input), nullptr, weight, epsilon, (int)num_tokens, hidden_size,
                                           static_cast<cudaStream_t>(stream));
    } else if (dtype == CA_DTYPE_F32) {
        e = ca::launch_norm<float, false>(out, const_cast<void*>(input), nullptr, weight, epsilon, (int)num_tokens, hidden_size,
                                          static_cast<cudaStream_t>(stream));
    } else {
        return ca::ops_fail(CA_ERR_INVALID, "rms_norm: fp16 and fp32 only");
    }
    if (e != cudaSuccess) return ca::ops_fail(CA_ERR_CUDA, cudaGetErrorString(e));
    return CA_OK;
}

int ca_fused_add_rms_norm(void* input, void* residual, const void* weight, float epsilon, int64_t num_tokens,
                          int hidden_size, int dtype, ca_stream stream) {
    if (num_tokens < 0 || hidden_size <= 0) return ca::ops_fail(CA_ERR_INVALID, "fused_add_rms_norm: bad shape");
    if (num_tokens == 0) return CA_OK;
    if (!input || !residual || !weight) return ca::ops_fail(CA_ERR_INVALID, "fused_add_rms_norm: null pointer");
    cudaError_t e;
    if (dtype == CA_DTYPE_F16) {
        e = ca::launch_norm<__half, true>(nullptr, input, residual, weight, epsilon, (int)num_tokens, hidden_size,
                                          static_cast<cudaStream_t>(stream));
    } else if (dtype == CA_DTYPE_F32) {
        e = ca::launch_norm<float, true>(nullptr, input, residual, weight, epsilon, (int)num_tokens, hidden_size,
                                         static_cast<cudaStream_t>(stream));
    } else {
        return ca::ops_fail(CA_ERR_INVALID, "fused_add_rms_norm: fp16 and fp32 only");
    }
    if (e != cudaSuccess) return ca::ops_fail(CA_ERR_CUDA, cudaGetErrorString(e));
    return CA_OK;
}

int ca_rotary_embedding(const int64_t* positions, void* query, void* key, const void* cos_sin_cache, int rot_dim,
                        int64_t query_stride, int64_t key_stride, int num_heads, int num_kv_heads, int head_size,
                        int64_t num_tokens, int is_neox, int dtype, int64_t max_position, int32_t* status,
                        ca_stream stream) {
    if (num_tokens < 0 || rot_dim <= 0 || rot_dim % 2 || rot_dim > head_size || num_heads < 0 || num_kv_heads < 0)
        return ca::ops_fail(CA_ERR_INVALID, "rotary_embedding: bad shape");
    if (num_tokens == 0) return CA_OK;
    if (!positions || !query || !key || !cos_sin_cache) return ca::ops_fail(CA_ERR_INVALID, "rotary_embedding: null pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int n = (int)num_tokens;
    // 16-byte path: every granule a thread touches must be 16-byte aligned (8 for the half granules of
    // cos / sin in the GPT-J layout)
    const int es = dtype == CA_DTYPE_F16 ? 2 : 4;
    const int epg = 16 / es;
    auto mult = [](int64_t v, int64_t m) { return v % m == 0; };
    const bool vec = (dtype == CA_DTYPE_F16 || dtype == CA_DTYPE_F32) &&
                     mult(reinterpret_cast<uintptr_t>(query), 16) && mult(reinterpret_cast<uintptr_t>(key), 16) &&
                     mult(reinterpret_cast<uintptr_t>(cos_sin_cache), 16) && mult(query_stride * es, 16) &&
                     mult(key_stride * es, 16) && mult((int64_t)head_size * es, 16) && mult((int64_t)rot_dim * es, 16) &&
                     (is_neox ? mult(rot_dim / 2, epg) : mult(rot_dim / 2, epg / 2) && mult((int64_t)(rot_dim / 2) * es, 8));
    const int units = vec ? (num_heads + num_kv_heads) * (is_neox ? rot_dim / 2 / epg : rot_dim / epg)
                          : (num_heads + num_kv_heads) * rot_dim / 2;
    const int threads = ca::threads_for(units < 512 ? units : 512);
#define CA_ROTV(T, NEOX)                                                                                            \
    ca::rotary_vec_kernel<T, NEOX><<<n, threads, 0, s>>>(positions, static_cast<T*>(query), static_cast<T*>(key),    \
                                                         static_cast<const T*>(cos_sin_cache), rot_dim, query_stride, \
                                                         key_stride, num_heads, num_kv_heads, head_size, max_position, status)
#define CA_ROT(T, NEOX)                                                                                             \
    ca::rotary_kernel<T, NEOX><<<n, threads, 0, s>>>(positions, static_cast<T*>(query), static_cast<T*>(key),        \
                                                     static_cast<const T*>(cos_sin_cache), rot_dim, query_stride,    \
                                                     key_stride, num_heads, num_kv_heads, head_size, max_position,  \
                                                     status)
    if (dtype == CA_DTYPE_F16) {
        if (vec) {
            if (is_neox) CA_ROTV(__half, true); else CA_ROTV(__half, false);
        } else {
            if (is_neox) CA_ROT(__half, true); else CA_ROT(__half, false);
        }
    } else if (dtype == CA_DTYPE_F32) {
        if (vec) {
            if (is_neox) CA_ROTV(float, true); else CA_ROTV(float, false);
        } else {
            if (is_neox) CA_ROT(float, true); else CA_ROT(float, false);
        }
    } else {
        return ca::ops_fail(CA_ERR_INVALID, "rotary_embedding: fp16 and fp32 only");
    }
#undef CA_ROT
#undef CA_ROTV
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return ca::ops_fail(CA_ERR_CUDA, cudaGetErrorString(e));
    return CA_OK;
}

}  // extern "C"
