"""tcgen05 flash attention against an fp32 softmax(QK^T)V of the same bf16 inputs."""
import math

import pytest
import torch

from solarwm_b200 import ops
from solarwm_b200.ops import reference as R
from solarwm_b200.ops.attention_native import attn_fwd

pytestmark = pytest.mark.gpu


def _mk(B, S, H, D, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(B, S, H, D, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("B,Sq,Sk,H,D", [(1, 256, 256, 2, 128), (1, 128, 128, 1, 128), (2, 384, 512, 3, 128),
                                          (1, 300, 200, 2, 128), (1, 1000, 1111, 2, 128), (1, 640, 512, 4, 64),
                                          (2, 250, 77, 2, 64), (1, 2000, 3000, 1, 128)])
def test_attention_forward(B, Sq, Sk, H, D):
    q, k, v = _mk(B, Sq, H, D, 1), _mk(B, Sk, H, D, 2), _mk(B, Sk, H, D, 3)
    scale = 1.0 / math.sqrt(D)
    o, lse = attn_fwd(q, k, v, scale)
    ops.check_status()
    ref = R.attention(q.float(), k.float(), v.float(), scale=scale)
    err = (o.float() - ref).abs().max().item()
    rel = ((o.float() - ref).norm() / ref.norm()).item()
    assert rel < 1e-2 and err < 5e-2, (rel, err)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    lse_ref = torch.logsumexp(s, dim=-1)
    assert (lse - lse_ref).abs().max().item() < 2e-2


def test_attention_large_scores_trigger_rescale():
    """Scores that grow along the key axis force the running-maximum rescale path."""
    B, S, H, D = 1, 1024, 1, 128
    q = _mk(B, S, H, D, 5, 2.0)
    k = _mk(B, S, H, D, 6, 2.0)
    ramp = torch.linspace(0.2, 3.0, S, device="cuda").view(1, S, 1, 1)
    k = (k.float() * ramp).to(torch.bfloat16)
    v = _mk(B, S, H, D, 7)
    scale = 1.0 / math.sqrt(D)
    o, _ = attn_fwd(q, k, v, scale)
    ops.check_status()
    ref = R.attention(q.float(), k.float(), v.float(), scale=scale)
    assert ((o.float() - ref).norm() / ref.norm()).item() < 1.5e-2


def test_attention_strided_views_of_fused_qkv():
    B, S, H, D = 1, 512, 2, 128
    qkv = _mk(B, S, 3 * H, D, 9).view(B, S, 3, H, D)
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    scale = 1.0 / math.sqrt(D)
    o, _ = attn_fwd(q, k, v, scale)
    ops.check_status()
    ref = R.attention(q.float(), k.float(), v.float(), scale=scale)
    assert ((o.float() - ref).norm() / ref.norm()).item() < 1e-2


@pytest.mark.parametrize("B,Sq,Sk,H,D", [(1, 256, 256, 2, 128), (1, 128, 64, 1, 128), (2, 300, 520, 2, 128),
                                          (1, 1000, 777, 2, 128), (1, 384, 512, 3, 64), (1, 2100, 2100, 1, 128)])
def test_attention_backward(B, Sq, Sk, H, D):
    q, k, v = (_mk(B, n, H, D, s).requires_grad_(True) for n, s in ((Sq, 21), (Sk, 22), (Sk, 23)))
    ops.reset_counters()
    o = ops.attention(q, k, v, backend="native")
    g = _mk(B, Sq, H, D, 24)
    o.backward(g)
    ops.check_status()
    assert ops.COUNTERS.get("attn_bwd", 0) == 3 and "library_sdpa_bwd" not in ops.COUNTERS
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    R.attention(q2, k2, v2).backward(g.float())
    for name, a, b in (("dq", q.grad, q2.grad), ("dk", k.grad, k2.grad), ("dv", v.grad, v2.grad)):
        rel = ((a.float() - b).norm() / b.norm()).item()
        assert rel < 2e-2, (name, rel)


def test_attention_autograd_path():
    B, S, H, D = 1, 256, 2, 128
    q, k, v = (_mk(B, S, H, D, s).requires_grad_(True) for s in (11, 12, 13))
    o = ops.attention(q, k, v, backend="native")
    g = torch.randn_like(o)
    o.backward(g)
    q2, k2, v2 = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    o2 = R.attention(q2, k2, v2)
    o2.backward(g.float())
    for a, b in ((q.grad, q2.grad), (k.grad, k2.grad), (v.grad, v2.grad)):
        assert ((a.float() - b).norm() / b.norm()).item() < 2e-2


def test_attention_backward_tail_overlap_is_bit_identical_and_ordered():
    """dQ on the side stream: same gradients as the single-stream order, and work queued right after the call on
    the caller's stream sees all three outputs complete."""
    import math

    from solarwm_b200.ops.attention_bwd_native import attn_bwd_native, set_tail_overlap
    from solarwm_b200.ops.attention_native import attn_fwd

    q, k, v, do = (_mk(1, n, 3, 128, s) for n, s in ((1500, 31), (1300, 32), (1300, 33), (1500, 34)))
    scale = 1.0 / math.sqrt(128)
    o, lse = attn_fwd(q, k, v, scale)
    previous = set_tail_overlap(False)
    try:
        want = [t.clone() for t in attn_bwd_native(q, k, v, o, lse, do, scale)]
        set_tail_overlap(True)
        for _ in range(3):
            got = attn_bwd_native(q, k, v, o, lse, do, scale)
            sums = [t.float().sum() for t in got]          # consumers on the caller's stream, no host sync before
            for a, b, s in zip(got, want, sums):
                assert torch.equal(a, b)
                assert float(s) == float(b.float().sum())
    finally:
        set_tail_overlap(previous)
    ops.check_status()


@pytest.mark.parametrize("D,kind", [(128, "tf"), (64, "tf"), (128, "causal"), (128, "w6")])
def test_masked_attention_matches_fp32_dense_mask_reference(D, kind):
    """One masked kernel call (forward + both backward kernels) against fp32 attention under the same dense mask; the
    geometry puts chunk boundaries off every tile boundary (chunks of 200 / 136 rows against 64- and 128-wide tiles)."""
    from solarwm_b200 import ops
    from solarwm_b200.ops import attention_mask as am

    torch.manual_seed(1)
    if kind == "tf":
        mask = am.teacher_forcing_segment_mask(L=1000, chunk=200, window_chunks=2, sink=72, prefix=0)
    elif kind == "w6":
        mask = am.teacher_forcing_segment_mask(L=680, chunk=136, window_chunks=1, sink=0, prefix=90)
    else:
        mask = am.block_causal_mask(1500, 200, 2, sink=40)
    S, H = mask.Sq, 3
    q, k, v = (torch.randn(1, S, H, D, device="cuda").bfloat16().requires_grad_(True) for _ in range(3))
    do = torch.randn(1, S, H, D, device="cuda").bfloat16()
    ops.reset_counters()
    o = am.masked_attention(q, k, v, mask)
    o.backward(do)
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.COUNTERS.get("attn_fwd_masked") == 1 and ops.COUNTERS.get("attn_bwd_masked") == 3
    t = mask.tables("cuda")
    assert t["tiles_visited"] < t["tiles_dense"]                       # tiles nobody sees are skipped
    qf, kf, vf = (x.detach().float().requires_grad_(True) for x in (q, k, v))
    dense = mask.dense().cuda()
    s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) / D ** 0.5
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s.masked_fill(~dense, float("-inf")), -1), vf)
    ref.backward(do.float())
    rel = lambda a, b: ((a.float() - b).norm() / b.norm()).item()     # noqa: E731
    assert rel(o, ref) < 1e-2
    assert rel(q.grad, qf.grad) < 2e-2 and rel(k.grad, kf.grad) < 2e-2 and rel(v.grad, vf.grad) < 2e-2
    assert torch.isfinite(o).all() and torch.isfinite(q.grad).all()
