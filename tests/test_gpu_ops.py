"""`chunk_attn.ops` on the GPU: the shipped kernels against the numpy oracle and, when the unmodified
reference's CUDA build is present (oracle/_ref/cuda), against its own kernels on the same inputs."""
import numpy as np
import pytest
import torch

import ops_oracle as oo
from chunk_attn import cabi, ops
from ref_loader import load_reference

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NP = {torch.float16: np.float16, torch.float32: np.float32}
# one unit in the last place of the element type, relative
ULP = {torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -23}


def _ref_ops():
    ref = load_reference("cuda")
    return getattr(ref, "ops", None) if ref is not None else None


def _close(got, want, dtype, ulps):
    got, want = got.astype(np.float64), want.astype(np.float64)
    if dtype == torch.float32:
        ulps *= 2  # the factor's last-bit difference passes through two more float roundings
    tol = ulps * ULP[dtype]
    np.testing.assert_allclose(got, want, rtol=tol, atol=tol * 1e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,hidden", [(1, 8), (7, 100), (33, 4096), (4, 5120), (3, 8200), (2, 1)])
def test_rms_norm(dtype, tokens, hidden):
    g = torch.Generator().manual_seed(tokens * 10007 + hidden)
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    xd, wd = x.to(DEV), w.to(DEV)
    out = torch.full_like(xd, float("nan"))
    ops.rms_norm(out, xd, wd, 1e-5)
    want = oo.rms_norm(x.numpy(), w.numpy(), 1e-5)
    # the sum of squares is accumulated in a different order: the float factor may differ in its last
    # bits, which can move a rounded result by one unit
    _close(out.cpu().numpy(), want, dtype, 2)
    assert torch.equal(xd.cpu(), x)  # the input is not modified
    rops = _ref_ops()
    if rops is not None:
        rout = torch.empty_like(xd)
        rops.rms_norm(rout, xd, wd, 1e-5)
        _close(out.cpu().numpy(), rout.cpu().numpy(), dtype, 2)
        # a last-bit difference of a row's float factor moves every fp32 element of that row, but only
        # the fp16 results that sat on a rounding boundary
        assert dtype == torch.float32 or (out == rout).float().mean().item() > 0.99


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("tokens,hidden", [(1, 8), (5, 100), (17, 4096), (2, 8200)])
def test_fused_add_rms_norm(dtype, tokens, hidden):
    g = torch.Generator().manual_seed(tokens * 31 + hidden)
    x = torch.randn(tokens, hidden, generator=g).to(dtype)
    res = torch.randn(tokens, hidden, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    xd, rd, wd = x.to(DEV), res.to(DEV), w.to(DEV)
    ops.fused_add_rms_norm(xd, rd, wd, 1e-6)
    want, want_res = oo.fused_add_rms_norm(x.numpy(), res.numpy(), w.numpy(), 1e-6)
    np.testing.assert_array_equal(rd.cpu().numpy(), want_res)  # the residual stream: bit exact
    _close(xd.cpu().numpy(), want, dtype, 2)
    rops = _ref_ops()
    if rops is not None:
        x2, r2 = x.to(DEV), res.to(DEV)
        rops.fused_add_rms_norm(x2, r2, wd, 1e-6)
        assert torch.equal(rd, r2)
        _close(xd.cpu().numpy(), x2.cpu().numpy(), dtype, 2)
        assert dtype == torch.float32 or (xd == x2).float().mean().item() > 0.99


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("is_neox", [True, False])
@pytest.mark.parametrize("tokens,hq,hk,head,rot", [(1, 1, 1, 32, 32), (9, 32, 32, 128, 128), (5, 8, 2, 128, 64),
                                                   (3, 40, 40, 128, 128), (4, 3, 1, 80, 20)])
def test_rotary_embedding(dtype, is_neox, tokens, hq, hk, head, rot):
    g = torch.Generator().manual_seed(tokens + 7 * hq + rot)
    q = torch.randn(tokens, hq * head, generator=g).to(dtype)
    k = torch.randn(tokens, hk * head, generator=g).to(dtype)
    pos = torch.randint(0, 2048, (tokens,), generator=g)
    cache = torch.from_numpy(oo.make_cos_sin_cache(rot, 2048, dtype=NP[dtype]))
    qd, kd, pd, cd = q.to(DEV), k.to(DEV), pos.to(DEV), cache.to(DEV)
    ops.rotary_embedding(pd, qd, kd, head, cd, is_neox)
    wq, wk = oo.rotary_embedding(pos.numpy(), q.numpy(), k.numpy(), head, cache.numpy(), is_neox)
    if dtype == torch.float16:  # every operation is a correctly rounded fp16 one: bit exact
        np.testing.assert_array_equal(qd.cpu().numpy(), wq)
        np.testing.assert_array_equal(kd.cpu().numpy(), wk)
    else:                       # the compiler may fuse a multiply into the add
        np.testing.assert_allclose(qd.cpu().numpy(), wq, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(kd.cpu().numpy(), wk, rtol=1e-6, atol=1e-6)
    rops = _ref_ops()
    if rops is not None:
        q2, k2 = q.to(DEV), k.to(DEV)
        rops.rotary_embedding(pd, q2, k2, head, cd, is_neox)
        if dtype == torch.float16:
            assert torch.equal(qd, q2) and torch.equal(kd, k2)
        else:
            torch.testing.assert_close(qd, q2, rtol=1e-6, atol=1e-6)
            torch.testing.assert_close(kd, k2, rtol=1e-6, atol=1e-6)


def test_rotary_on_strided_batch_views():
    """[batch, seq, heads * head] query with a token stride larger than the row (a slice of a fused
    qkv projection), 2-D positions: the layout the reference's llama layer passes."""
    b, s, hq, hk, head = 2, 5, 4, 2, 64
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(b, s, (hq + 2 * hk) * head, generator=g).half()
    pos = torch.randint(0, 128, (b, s), generator=g)
    cache = torch.from_numpy(oo.make_cos_sin_cache(head, 128))
    qkv_d = qkv.to(DEV)
    q_d, k_d = qkv_d[..., :hq * head], qkv_d[..., hq * head:(hq + hk) * head]
    ops.rotary_embedding(pos.to(DEV), q_d, k_d, head, cache.to(DEV), True)
    wq, wk = oo.rotary_embedding(pos.numpy().reshape(-1), qkv[..., :hq * head].reshape(b * s, -1).numpy(),
                                 qkv[..., hq * head:(hq + hk) * head].reshape(b * s, -1).numpy(), head,
                                 cache.numpy(), True)
    np.testing.assert_array_equal(q_d.cpu().numpy().reshape(b * s, -1), wq)
    np.testing.assert_array_equal(k_d.cpu().numpy().reshape(b * s, -1), wk)
    # v is untouched
    assert torch.equal(qkv_d[..., (hq + hk) * head:].cpu(), qkv[..., (hq + hk) * head:])


def test_ops_on_a_side_stream_and_unaligned_rows():
    """The C ABI directly: an explicit stream, and rows that start off a 16-byte boundary (the
    element-wise kernel variant)."""
    hidden, tokens = 72, 6
    g = torch.Generator().manual_seed(11)
    base = torch.randn(tokens * hidden + 1, generator=g).half().to(DEV)
    x = base[1:].view(tokens, hidden)  # 2 bytes off alignment
    w = (1 + 0.1 * torch.randn(hidden, generator=g)).half().to(DEV)
    out = torch.empty(tokens, hidden, dtype=torch.float16, device=DEV)
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    cabi.check(cabi.lib.ca_rms_norm(out.data_ptr(), x.data_ptr(), w.data_ptr(), 1e-5, tokens, hidden,
                                    cabi.CA_DTYPE_F16, st.cuda_stream))
    st.synchronize()
    _close(out.cpu().numpy(), oo.rms_norm(x.cpu().numpy(), w.cpu().numpy(), 1e-5), torch.float16, 2)


def test_llama_layer_sequence_matches_oracle():
    """The order a decoder layer uses them in: residual add + norm, rotary on q/k, over a decode
    batch of 32 tokens at hidden 4096."""
    g = torch.Generator().manual_seed(2)
    n, hidden, heads, head = 32, 4096, 32, 128
    h = torch.randn(n, hidden, generator=g).half()
    res = torch.randn(n, hidden, generator=g).half()
    w = (1 + 0.05 * torch.randn(hidden, generator=g)).half()
    pos = torch.randint(0, 4096, (n,), generator=g)
    cache = torch.from_numpy(oo.make_cos_sin_cache(head, 4096))
    hd, rd = h.to(DEV), res.to(DEV)
    ops.fused_add_rms_norm(hd, rd, w.to(DEV), 1e-5)
    qd, kd = hd.clone(), hd.clone()
    ops.rotary_embedding(pos.to(DEV), qd, kd, head, cache.to(DEV), True)
    wn, wr = oo.fused_add_rms_norm(h.numpy(), res.numpy(), w.numpy(), 1e-5)
    np.testing.assert_array_equal(rd.cpu().numpy(), wr)
    _close(hd.cpu().numpy(), wn, torch.float16, 2)
    # rotary of the GPU's own normalised rows must match the oracle bit for bit
    wq, _ = oo.rotary_embedding(pos.numpy(), hd.cpu().numpy(), hd.cpu().numpy(), head, cache.numpy(), True)
    np.testing.assert_array_equal(qd.cpu().numpy(), wq)
