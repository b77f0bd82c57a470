"""The numpy oracle of `chunk_attn.ops` against a float64 statement of the same formulas, and the
host-side argument checks of the shipped functions (no GPU needed)."""
import numpy as np
import pytest
import torch

import ops_oracle as oo


def _rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("dtype,tol", [(np.float16, 2e-3), (np.float32, 2e-6)])
@pytest.mark.parametrize("hidden", [8, 100, 4096])
def test_rms_norm_oracle(dtype, tol, hidden):
    r = _rng(hidden)
    x = r.standard_normal((5, hidden)).astype(dtype)
    w = (1.0 + 0.1 * r.standard_normal(hidden)).astype(dtype)
    got = oo.rms_norm(x, w, 1e-5)
    assert got.dtype == dtype
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(-1, keepdims=True) + 1e-5) * w.astype(np.float64)
    np.testing.assert_allclose(got.astype(np.float64), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype,tol", [(np.float16, 2e-3), (np.float32, 2e-6)])
def test_fused_add_rms_norm_oracle(dtype, tol):
    r = _rng(7)
    x = r.standard_normal((6, 256)).astype(dtype)
    res = r.standard_normal((6, 256)).astype(dtype)
    w = (1.0 + 0.1 * r.standard_normal(256)).astype(dtype)
    out, new_res = oo.fused_add_rms_norm(x, res, w, 1e-6)
    z = x.astype(np.float64) + res.astype(np.float64)
    np.testing.assert_array_equal(new_res, z.astype(dtype))  # the residual stream is the rounded sum
    want = z / np.sqrt((z ** 2).mean(-1, keepdims=True) + 1e-6) * w.astype(np.float64)
    np.testing.assert_allclose(out.astype(np.float64), want, rtol=2 * tol, atol=2 * tol)
    # the fused form equals the plain norm of the new residual up to the variance's rounding
    np.testing.assert_allclose(out.astype(np.float64), oo.rms_norm(new_res, w, 1e-6).astype(np.float64),
                               rtol=2 * tol, atol=2 * tol)


@pytest.mark.parametrize("dtype,tol", [(np.float16, 4e-3), (np.float32, 1e-6)])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("rot_dim,head_size", [(128, 128), (64, 128), (32, 32)])
def test_rotary_oracle(dtype, tol, is_neox, rot_dim, head_size):
    r = _rng(rot_dim + is_neox)
    n_tok, hq, hk = 7, 4, 2
    q = r.standard_normal((n_tok, hq * head_size)).astype(dtype)
    k = r.standard_normal((n_tok, hk * head_size)).astype(dtype)
    pos = r.integers(0, 512, n_tok)
    cache = oo.make_cos_sin_cache(rot_dim, 512, dtype=dtype)
    q2, k2 = oo.rotary_embedding(pos, q, k, head_size, cache, is_neox)
    assert q2.shape == q.shape and k2.shape == k.shape

    def want(t, heads):
        t = t.astype(np.float64).reshape(n_tok, heads, head_size).copy()
        cs = cache[pos].astype(np.float64)
        c, s = cs[:, None, :rot_dim // 2], cs[:, None, rot_dim // 2:]
        if is_neox:
            x, y = t[..., :rot_dim // 2].copy(), t[..., rot_dim // 2:rot_dim].copy()
            t[..., :rot_dim // 2], t[..., rot_dim // 2:rot_dim] = x * c - y * s, y * c + x * s
        else:
            x, y = t[..., 0:rot_dim:2].copy(), t[..., 1:rot_dim:2].copy()
            t[..., 0:rot_dim:2], t[..., 1:rot_dim:2] = x * c - y * s, y * c + x * s
        return t.reshape(n_tok, -1)

    np.testing.assert_allclose(q2.astype(np.float64), want(q, hq), rtol=tol, atol=tol)
    np.testing.assert_allclose(k2.astype(np.float64), want(k, hk), rtol=tol, atol=tol)
    # elements past rot_dim are untouched, and a rotation preserves each pair's norm
    if rot_dim < head_size:
        np.testing.assert_array_equal(q2.reshape(n_tok, hq, head_size)[..., rot_dim:],
                                      q.reshape(n_tok, hq, head_size)[..., rot_dim:])
    n0 = (q.astype(np.float64).reshape(n_tok, hq, head_size)[..., :rot_dim] ** 2).sum(-1)
    n1 = (q2.astype(np.float64).reshape(n_tok, hq, head_size)[..., :rot_dim] ** 2).sum(-1)
    np.testing.assert_allclose(n1, n0, rtol=20 * tol)


def test_position_zero_is_identity():
    r = _rng(3)
    q = r.standard_normal((3, 2 * 64)).astype(np.float16)
    k = r.standard_normal((3, 64)).astype(np.float16)
    cache = oo.make_cos_sin_cache(64, 16)
    q2, k2 = oo.rotary_embedding(np.zeros(3, np.int64), q, k, 64, cache, True)
    np.testing.assert_array_equal(q2, q)
    np.testing.assert_array_equal(k2, k)


def test_shipped_ops_have_no_cpu_path():
    from chunk_attn import ops
    x = torch.randn(2, 64, dtype=torch.float16)
    w = torch.ones(64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensors are required"):
        ops.rms_norm(torch.empty_like(x), x, w, 1e-5)
    with pytest.raises(RuntimeError, match="CUDA tensors are required"):
        ops.fused_add_rms_norm(x, x.clone(), w, 1e-5)
    with pytest.raises(RuntimeError, match="CUDA tensors are required"):
        ops.rotary_embedding(torch.zeros(2, dtype=torch.int64), x, x.clone(), 64, torch.zeros(4, 64, dtype=torch.float16), True)


def test_c_abi_rejects_bad_arguments():
    from chunk_attn import cabi
    L = cabi.lib
    assert L.ca_rms_norm(None, None, None, 1e-5, 4, 64, cabi.CA_DTYPE_F16, None) == cabi.CA_ERR_INVALID
    assert L.ca_rms_norm(None, None, None, 1e-5, 0, 64, cabi.CA_DTYPE_F16, None) == cabi.CA_OK  # nothing to do
    assert L.ca_rms_norm(None, None, None, 1e-5, 4, 0, cabi.CA_DTYPE_F16, None) == cabi.CA_ERR_INVALID
    assert L.ca_fused_add_rms_norm(None, None, None, 1e-5, 4, 64, cabi.CA_DTYPE_F16, None) == cabi.CA_ERR_INVALID
    # odd rot_dim, rot_dim > head_size
    assert L.ca_rotary_embedding(None, None, None, None, 63, 64, 64, 1, 1, 64, 4, 1, 0, 0, None, None) == cabi.CA_ERR_INVALID
    assert L.ca_rotary_embedding(None, None, None, None, 128, 64, 64, 1, 1, 64, 4, 1, 0, 0, None, None) == cabi.CA_ERR_INVALID
    assert b"rotary_embedding" in L.ca_last_error()
