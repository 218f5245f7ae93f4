"""Row kernels (norm+modulate, gated residual, RMSNorm+RoPE, GELU/SwiGLU, AdamW, MSE, flow, RGB8)
against the fp32 PyTorch statements in ops.reference."""
import pytest
import torch

from solarwm_b200 import ops
from solarwm_b200.ops import reference as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("D", [128, 3072, 5376])
def test_norm_modulate_fwd_bwd(mode, D):
    torch.manual_seed(D + mode)
    rows, rpg, G = 96, 16, 8
    x = torch.randn(rows, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    mod = (torch.randn(G, 6, D, device=DEV) * 0.3).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).requires_grad_(mode >= 1)
    b = (0.1 * torch.randn(D, device=DEV)).requires_grad_(mode == 2)
    kw = dict(mode=mode, w=w if mode >= 1 else None, b=b if mode == 2 else None, eps=1e-6,
              rows_per_group=rpg, group_offset=1)
    y = ops.norm_modulate(x, mod[:, 0], mod[:, 1], **kw)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    modr = mod.detach().clone().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(mode >= 1)
    br = b.detach().clone().requires_grad_(mode == 2)
    kwr = dict(kw, w=wr if mode >= 1 else None, b=br if mode == 2 else None)
    yr = R.norm_modulate(xr.float(), modr[:, 0], modr[:, 1], **kwr)
    yr.backward(g.float())
    assert _rel(y, yr) < 5e-3
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(mod.grad, modr.grad) < 1e-2
    if mode >= 1:
        assert _rel(w.grad, wr.grad) < 1e-2
    if mode == 2:
        assert _rel(b.grad, br.grad) < 1e-2


def test_gated_residual_fwd_bwd():
    torch.manual_seed(0)
    rows, D, rpg, G = 80, 3072, 20, 4
    res = torch.randn(rows, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = torch.randn(rows, D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    gate = (torch.randn(G, 6, D, device=DEV) * 0.5).requires_grad_(True)
    out = ops.gated_residual(res, y, gate[:, 2], rows_per_group=rpg)
    g = torch.randn_like(out)
    out.backward(g)
    r2, y2, g2 = (t.detach().clone().requires_grad_(True) for t in (res, y, gate))
    outr = R.gated_residual(r2.float(), y2.float(), g2[:, 2], rows_per_group=rpg)
    outr.backward(g.float())
    assert _rel(out, outr) < 5e-3
    assert _rel(res.grad, r2.grad) < 5e-3
    assert _rel(y.grad, y2.grad) < 1e-2
    assert _rel(gate.grad, g2.grad) < 1e-2
    plain = ops.gated_residual(res.detach(), y.detach(), None)
    assert _rel(plain, res.detach().float() + y.detach().float()) < 5e-3


@pytest.mark.parametrize("D,hd", [(128, 32), (3072, 128), (2048, 64)])
def test_rmsnorm_rope_fwd_bwd(D, hd):
    from solarwm_b200.models.wan import rope_table

    torch.manual_seed(D)
    grid = (3, 4, 5)
    rows = 60
    rope = rope_table(grid, hd, DEV)
    big = torch.randn(rows, 3 * D, device=DEV).to(torch.bfloat16).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, device=DEV)).requires_grad_(True)
    y = ops.rmsnorm_rope(big[:, D:2 * D], w, rope, eps=1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    b2 = big.detach().clone().requires_grad_(True)
    w2 = w.detach().clone().requires_grad_(True)
    yr = R.rmsnorm_rope(b2[:, D:2 * D].float(), w2, rope, eps=1e-6)
    yr.backward(g.float())
    assert _rel(y, yr) < 5e-3
    assert _rel(big.grad, b2.grad) < 1e-2
    assert _rel(w.grad, w2.grad) < 1e-2
    # rotation only
    y0 = ops.rmsnorm_rope(big.detach()[:, :D], None, rope, no_norm=True)
    assert _rel(y0, R.rmsnorm_rope(big.detach()[:, :D].float(), None, rope, no_norm=True)) < 5e-3


def test_rope_table_matches_complex_fp64():
    """The (cos, sin) table equals the reference's fp64 complex multiplication on interleaved pairs."""
    from solarwm_b200.models.wan import rope_axis_dims, rope_table

    hd, grid = 128, (2, 3, 4)
    x = torch.randn(24, 2, hd, dtype=torch.float64)
    tab = rope_table(grid, hd, "cpu").double()
    ours = R.rmsnorm_rope(x.reshape(24, 2 * hd), None, tab, no_norm=True).reshape(24, 2, hd)
    c = hd // 2
    parts = []
    for n_pairs in rope_axis_dims(hd):
        d = 2 * n_pairs
        fr = torch.outer(torch.arange(1024, dtype=torch.float64),
                         1.0 / torch.pow(10000, torch.arange(0, d, 2, dtype=torch.float64) / d))
        parts.append(torch.polar(torch.ones_like(fr), fr))
    f, h, w = grid
    freqs = torch.cat([parts[0][:f].view(f, 1, 1, -1).expand(f, h, w, -1),
                       parts[1][:h].view(1, h, 1, -1).expand(f, h, w, -1),
                       parts[2][:w].view(1, 1, w, -1).expand(f, h, w, -1)], -1).reshape(24, 1, c)
    xc = torch.view_as_complex(x.reshape(24, 2, c, 2))
    ref = torch.view_as_real(xc * freqs).flatten(2)
    assert (ours.double() - ref).abs().max().item() < 1e-5


def test_gelu_swiglu():
    torch.manual_seed(1)
    x = torch.randn(64, 512, device=DEV).to(torch.bfloat16).requires_grad_(True)
    y = ops.gelu(x)
    g = torch.randn_like(y)
    y.backward(g)
    x2 = x.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(x2, approximate="tanh")
    yr.backward(g.float())
    assert _rel(y, yr) < 5e-3 and _rel(x.grad, x2.grad) < 1e-2
    gu = torch.randn(48, 1024, device=DEV).to(torch.bfloat16).requires_grad_(True)
    s = ops.swiglu(gu)
    gs = torch.randn_like(s)
    s.backward(gs)
    gu2 = gu.detach().float().requires_grad_(True)
    sr = R.swiglu(gu2)
    sr.backward(gs.float())
    assert _rel(s, sr) < 5e-3 and _rel(gu.grad, gu2.grad) < 1e-2


@pytest.mark.parametrize("grad_dtype", [torch.float32, torch.bfloat16])
def test_adamw_matches_fp32_reference(grad_dtype):
    torch.manual_seed(2)
    n = 4096 * 3
    master = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    live = master.to(torch.bfloat16)
    ema = master.clone()
    rm, rmm, rv, rema = master.clone(), m.clone(), v.clone(), ema.clone()
    scale = torch.tensor([0.5], device=DEV)
    skip = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(grad_dtype)
        ops.adamw_(master, m, v, g, live=live, ema=ema, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, wd=0.1,
                   step=step, grad_scale=scale, skip=skip, ema_decay=0.9)
        R.adamw_step(rm, rmm, rv, g, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, wd=0.1, step=step, grad_scale=0.5)
        rema.mul_(0.9).add_(rm, alpha=0.1)
    assert _rel(master, rm) < 1e-5 and _rel(m, rmm) < 1e-5 and _rel(v, rv) < 1e-5 and _rel(ema, rema) < 1e-5
    assert torch.equal(live, master.to(torch.bfloat16))
    before = master.clone()
    skip.fill_(1)
    ops.adamw_(master, m, v, g, live=live, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, wd=0.1, step=4, skip=skip)
    assert torch.equal(before, master)


def test_sumsq_mse_flow():
    torch.manual_seed(3)
    x = torch.randn(1 << 20, device=DEV)
    assert abs(ops.sumsq(x).item() / x.double().pow(2).sum().item() - 1) < 1e-5
    xb = x.to(torch.bfloat16)
    assert abs(ops.sumsq(xb).item() / xb.double().pow(2).sum().item() - 1) < 1e-5
    G, E = 6, 4096
    x0 = torch.randn(G, E, device=DEV).to(torch.bfloat16)
    n = torch.randn(G, E, device=DEV).to(torch.bfloat16)
    s = torch.rand(G, device=DEV)
    xt, tgt = ops.add_noise(x0, n, s)
    assert _rel(xt, (1 - s[:, None]) * x0.float() + s[:, None] * n.float()) < 4e-3
    assert _rel(tgt, n.float() - x0.float()) < 4e-3
    assert _rel(ops.flow_to_x0(xt, tgt, s), xt.float() - s[:, None] * tgt.float()) < 4e-3
    s2 = torch.rand(G, device=DEV)
    assert _rel(ops.euler_step(xt, tgt, s, s2), xt.float() + (s2 - s)[:, None] * tgt.float()) < 4e-3
    pred = torch.randn(G, E, device=DEV).to(torch.bfloat16).requires_grad_(True)
    w = torch.rand(G, device=DEV) + 0.5
    mask = torch.tensor([0., 1, 1, 1, 0, 1], device=DEV)
    loss = ops.weighted_masked_mse(pred, tgt, w, mask)
    loss.backward()
    p2 = pred.detach().float().requires_grad_(True)
    lr = R.weighted_masked_mse(p2, tgt.float(), w, mask)
    lr.backward()
    assert abs(loss.item() / lr.item() - 1) < 1e-4
    assert _rel(pred.grad, p2.grad) < 1e-2


def test_rgb8_device_equals_host_twin():
    torch.manual_seed(4)
    frame = (torch.randn(3, 48, 84) * 1.5).to(torch.bfloat16)
    host, _ = ops.rgb8(frame)
    dev, flag = ops.rgb8(frame.to(DEV))
    assert flag.item() == 0
    assert torch.equal(host, dev.cpu())
    v = frame.float() * torch.tensor([.229, .224, .225]).view(3, 1, 1) + torch.tensor([.485, .456, .406]).view(3, 1, 1)
    ref = torch.round(v.clamp(0, 1) * 255).to(torch.uint8).permute(1, 2, 0)
    assert (host.int() - ref.int()).abs().max().item() <= 1
