"""`ca_attention_host` / `Attention.forward_host`: queries and result in host memory (pinned buffers used in
place, pageable ones staged), bit-identical to the device-tensor call."""
import pytest
import torch

from chunk_attn import Attention, cabi
import synthetic_workloads as W
from gpu_helpers import CabiEngine

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def small_engine(dtype, H, d, C):
    g = torch.Generator().manual_seed(0)
    attn = Attention(n_heads=H, d_head=d, chunk_size=C, memory_mb=64, dtype=dtype, device=DEV)
    shared = list(range(2 * C + 5))
    sk, sv = torch.randn(len(shared), H, d, generator=g), torch.randn(len(shared), H, d, generator=g)
    for s in range(5):
        own = 3 + 11 * s
        toks = shared + [1000 * (s + 1) + j for j in range(own)]
        k = torch.cat([sk, torch.randn(own, H, d, generator=g)])
        v = torch.cat([sv, torch.randn(own, H, d, generator=g)])
        attn.add_seq(tokens=toks, k=k.to(DEV, dtype), v=v.to(DEV, dtype))
    return attn, torch.randn(5, H, d, generator=g).to(dtype)


@pytest.mark.parametrize("dtype,H,d,C", [(torch.float16, 4, 128, 64), (torch.float32, 2, 64, 16)])
@pytest.mark.parametrize("pin_q", [True, False])
@pytest.mark.parametrize("pin_out", [True, False, None])
def test_forward_host_equals_forward(dtype, H, d, C, pin_q, pin_out):
    attn, q = small_engine(dtype, H, d, C)
    want = attn.forward(q=q.to(DEV)).cpu()
    q_cpu = q.clone().pin_memory() if pin_q else q.clone()
    if pin_out is None:
        got = attn.forward_host(q=q_cpu)
        assert got.is_pinned()
    else:
        out = torch.full_like(q, float("nan"))
        out = out.pin_memory() if pin_out else out
        got = attn.forward_host(q=q_cpu, out=out)
        assert got.data_ptr() == out.data_ptr()
    assert torch.equal(got, want)
    assert torch.equal(attn.forward_host(q=q_cpu, partition=2), attn.forward(q=q.to(DEV), partition=2).cpu())
    # repeated calls reuse the staging buffers; a decode step in between is picked up
    k = torch.randn(5, H, d).to(dtype)
    attn.append_token(tokens=[9] * 5, k=k.to(DEV), v=k.to(DEV))
    assert torch.equal(attn.forward_host(q=q_cpu), attn.forward(q=q.to(DEV)).cpu())
    assert attn.device_status() == 0


def test_forward_host_argument_checks():
    attn, q = small_engine(torch.float16, 4, 128, 64)
    with pytest.raises(RuntimeError, match="must be a CPU tensor"):
        attn.forward_host(q=q.to(DEV))
    with pytest.raises(RuntimeError, match="one query row per live sequence"):
        attn.forward_host(q=q[:3].contiguous())
    with pytest.raises(RuntimeError, match="shaped and typed like q"):
        attn.forward_host(q=q, out=torch.empty(5, 4, 128))
    with pytest.raises(RuntimeError, match="dtype of the cache"):
        attn.forward_host(q=q.float())


def test_c_abi_host_call_on_config2():
    w = W.config2()
    eng = CabiEngine(w.n_heads, w.d_head, w.chunk_size, torch.float16, max_chunks=32 + 32 * 9 + 8)
    rows = W.populate(eng, w)
    q = w.q[rows].half().contiguous()
    want = eng.forward(q.to(DEV)).cpu()
    qp, outp = q.pin_memory(), torch.empty_like(q).pin_memory()
    eng.ctx.attention_host(qp, outp)
    assert torch.equal(outp, want)
    out2 = torch.empty_like(q)
    eng.ctx.attention_host(q, out2)  # pageable both ways
    assert torch.equal(out2, want)
    # stale work list is refused like in ca_attention
    eng.tree.remove_seq(0)
    eng.ctx.refresh(eng.tree.get_chunks(), len(eng.tree.tails))
    with pytest.raises(cabi.CAError, match="n_seqs differs"):
        eng.ctx.attention_host(qp, outp)
