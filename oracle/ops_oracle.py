"""CPU oracle for the element-wise companions of the attention path: TEST INFRASTRUCTURE ONLY.

numpy restatement of the three functions the reference exports as `chunk_attn.ops`
(cpp/chunk_attn/python_exports_ops.cpp:11-19).  Only the tests and the smoke check may import
it; the shipped engine never does and has no CPU path for these functions.

Parity status: PINNED on a GPU box through the unmodified reference kernels built into
oracle/_ref/cuda (tests/test_gpu_ops.py compares the engine with them bit for bit where the
arithmetic is order-independent and within one unit in the last place where a reduction order
enters); the reference has no CPU implementation of these functions and its repository holds
no golden vectors for them, so on a CPU-only machine this file is checked against a float64
statement of the same formulas (tests/test_ops_oracle_cpu.py).

Rounding follows the reference kernels: arithmetic on fp16 tensors rounds every product and sum
to fp16 where the reference computes in the element type, and stays in float32 where it
converts to float first.
"""
import numpy as np


def _f32(x):
    return np.asarray(x, dtype=np.float32)


def rms_norm(x, weight, epsilon):
    """out = T(x * rsqrt(mean(x^2) + eps)) * weight, T the element type
    (cpp/chunk_attn/layernorm_kernels.cu:26-50: the variance is a float sum of squares, the
    normalised value is cast to the element type and only then multiplied by the weight)."""
    dt = x.dtype
    xf = _f32(x)
    var = np.sum(xf * xf, axis=-1, keepdims=True, dtype=np.float32) / np.float32(x.shape[-1])
    inv = np.float32(1.0) / np.sqrt(var + np.float32(epsilon), dtype=np.float32)
    return (xf * inv).astype(dt) * weight.astype(dt)


def fused_add_rms_norm(x, residual, weight, epsilon):
    """Returns (out, new_residual): z = x + residual in float, new_residual = T(z),
    out = T(z_rounded * rsqrt(mean(z^2) + eps)) * weight
    (cpp/chunk_attn/layernorm_kernels.cu:53-79: the variance uses the unrounded float sum, the
    second pass re-reads the rounded residual)."""
    dt = x.dtype
    z = _f32(x) + _f32(residual)
    var = np.sum(z * z, axis=-1, keepdims=True, dtype=np.float32) / np.float32(x.shape[-1])
    inv = np.float32(1.0) / np.sqrt(var + np.float32(epsilon), dtype=np.float32)
    new_res = z.astype(dt)
    return (_f32(new_res) * inv).astype(dt) * weight.astype(dt), new_res


def make_cos_sin_cache(rot_dim, max_position, base=10000.0, dtype=np.float16):
    """[max_position, rot_dim] = [cos | sin] of position * base^(-2i/rot_dim), the layout the
    kernels read (src/chunk_attn/models/llama_hf/rotary_embedding_vllm.py:62-90)."""
    inv_freq = 1.0 / (base ** (np.arange(0, rot_dim, 2, dtype=np.float32) / np.float32(rot_dim)))
    freqs = np.outer(np.arange(max_position, dtype=np.float32), inv_freq.astype(np.float32))
    return np.concatenate([np.cos(freqs), np.sin(freqs)], axis=-1).astype(dtype)


def _rotate(t, positions, cache, head_size, is_neox):
    """t: [num_tokens, n_heads * head_size]; returns the rotated copy
    (cpp/chunk_attn/pos_encoding_kernels.cu:7-31: x' = x cos - y sin, y' = y cos + x sin, every
    product and the sum rounded in the element type)."""
    dt = t.dtype
    n_tok = t.shape[0]
    rot = cache.shape[1]
    half = rot // 2
    out = t.reshape(n_tok, -1, head_size).copy()
    cs = cache[positions]                 # [n_tok, rot]
    cos = cs[:, None, :half].astype(dt)
    sin = cs[:, None, half:].astype(dt)
    if is_neox:
        x, y = out[:, :, :half].copy(), out[:, :, half:rot].copy()
    else:
        x, y = out[:, :, 0:rot:2].copy(), out[:, :, 1:rot:2].copy()
    if dt == np.float32:
        # nvcc contracts x*cos - y*sin into one fused multiply-add; emulate it in float64
        # (the float64 product of two floats is exact) and round once
        xo = ((x.astype(np.float64) * cos) - (y * sin).astype(np.float64)).astype(np.float32)
        yo = ((y.astype(np.float64) * cos) + (x * sin).astype(np.float64)).astype(np.float32)
    else:
        xo = (x * cos).astype(dt) - (y * sin).astype(dt)
        yo = (y * cos).astype(dt) + (x * sin).astype(dt)
    if is_neox:
        out[:, :, :half], out[:, :, half:rot] = xo, yo
    else:
        out[:, :, 0:rot:2], out[:, :, 1:rot:2] = xo, yo
    return out.reshape(t.shape)


def rotary_embedding(positions, query, key, head_size, cos_sin_cache, is_neox):
    """Returns (query', key').  query: [num_tokens, num_heads * head_size], key likewise with
    its own head count; positions: [num_tokens] int64
    (cpp/chunk_attn/pos_encoding_kernels.cu:33-90)."""
    positions = np.asarray(positions, dtype=np.int64).reshape(-1)
    return (_rotate(query, positions, cos_sin_cache, head_size, is_neox),
            _rotate(key, positions, cos_sin_cache, head_size, is_neox))
