import numpy as np
import pytest
import torch

from solarwm_b200 import ops
from solarwm_b200.engine import anyflow as af
from solarwm_b200.engine import sgf
from solarwm_b200.engine.flow import (FlowMatchScheduler, first_frame_loss_mask, rectified_interpolate_array,
                                      velocity_target_array, weighted_masked_mse_array)
from solarwm_b200.engine.schedule import warmup_cosine_factor


def test_flow_scheduler_matches_closed_form_and_numpy_twins():
    s = FlowMatchScheduler(shift=5.0)
    lin = torch.linspace(1, 0, 1001)[:-1]
    assert torch.allclose(s.sigmas, 5 * lin / (1 + 4 * lin))
    assert abs(s.linear_timesteps_weights.mean().item() - 1.0) < 1e-5 and s.linear_timesteps_weights.min() == 0
    t = s.timesteps[[0, 400, 999]]
    x0, n = torch.randn(3, 4, 8), torch.randn(3, 4, 8)
    xt, target = s.add_noise(x0, n, t)
    assert np.allclose(xt.numpy(), rectified_interpolate_array(x0, n, s.sigma_of(t)), atol=1e-6)
    assert np.allclose(target.numpy(), velocity_target_array(x0, n), atol=1e-6)
    mask = first_frame_loss_mask(1, 3, torch.tensor([False]))[0]
    w = torch.tensor([0.5, 1.0, 2.0])
    got = ops.weighted_masked_mse(xt, target, w, mask.float())
    want = weighted_masked_mse_array(xt, target, mask.numpy()[:, None, None], w.numpy()[:, None, None])
    assert abs(got.item() - want) < 1e-5
    assert torch.allclose(ops.flow_to_x0(xt, target, s.sigma_of(t)), x0, atol=1e-5)


def test_warmup_cosine():
    f = lambda i: warmup_cosine_factor(i, warmup_steps=10, total_steps=110, min_lr_ratio=0.1)
    assert f(0) == 0.1 and f(9) == 1.0 and abs(f(60) - 0.55) < 1e-9 and abs(f(110) - 0.1) < 1e-9


def test_anyflow_time_pairs_types_and_windows():
    g = torch.Generator().manual_seed(0)
    pairs = [af.sample_time_pairs(4, dp_rank=r, dp_world=2, generator=torch.Generator().manual_seed(r)) for r in range(2)]
    kinds = torch.cat([p.sample_type for p in pairs]).tolist()
    assert kinds == [0, 0, 0, 0, 1, 1, 2, 2]
    p = pairs[1]
    assert torch.equal(p.r[p.is_consistency], torch.zeros(2))
    fm = p.sample_type == af.FLOW_MAP
    assert bool(((p.r[fm] > 0) & (p.r[fm] < p.t[fm])).all())
    assert torch.equal(pairs[0].r, pairs[0].t)
    tp, tm = af.difference_window(torch.tensor([998.0, 3.0, 500.0]), torch.tensor([0.0, 1.0, 499.0]))
    assert tp.tolist() == [1000.0, 8.0, 505.0] and tm.tolist() == [993.0, 1.0, 499.0]
    u_plus, u_minus = torch.full((3, 2), 4.0), torch.full((3, 2), 1.0)
    d = af.central_difference(u_plus, u_minus, tp, tm)
    assert torch.allclose(d[:, 0], torch.tensor([3 / 7, 3 / 7, 3 / 6]))
    w = af.gaussian_timestep_weights(torch.tensor([500.0, 0.0]), shift=5.0)
    assert w[0] > w[1]
    with pytest.raises(ValueError):
        af.sample_time_pairs(2, diffusion_ratio=0.8, consistency_ratio=0.5)


def test_anyflow_adaptive_rescale():
    loss = torch.tensor([2.0, 4.0, 8.0, 1.0])
    is_diff = torch.tensor([True, True, False, False])
    out = af.adaptive_rescale(loss, is_diff)
    assert torch.allclose(out[:2], loss[:2]) and torch.allclose(out[2:], torch.tensor([3.0, 3.0]), atol=1e-3)
    assert torch.equal(af.adaptive_rescale(loss, torch.zeros(4, dtype=torch.bool)), loss)
    gathered = af.adaptive_rescale(loss, is_diff, gather_fn=lambda x: [x, x * 0 + (10.0 if x.dtype != torch.bool else 1)])
    assert gathered.shape == loss.shape


def test_sgf_gradient_masks_before_reducing():
    assert [sgf.should_update_student(s, 5) for s in (0, 4, 5, 10)] == [False, False, True, True]
    fake, real, out = torch.randn(2, 3, 4), torch.randn(2, 3, 4), torch.randn(2, 3, 4, requires_grad=True)
    real[:, 0] = float("nan")
    mask = torch.tensor([False, True, True]).view(1, 3, 1)
    g = sgf.sgf_kl_gradient(fake_x0=fake, real_x0=real, student_output=out.detach(), mask=mask)
    assert torch.isfinite(g).all() and g[:, 0].abs().sum() == 0
    norm = (out.detach() - real)[:, 1:].abs().mean(dim=(1, 2), keepdim=True)
    assert torch.allclose(g[:, 1:], (fake - real)[:, 1:] / norm, atol=1e-5)
    loss = sgf.sgf_student_loss(out, g, mask=mask)
    loss.backward()
    assert torch.allclose(out.grad[:, 1:], g[:, 1:] / (2 * 2 * 4), atol=1e-6) and out.grad[:, 0].abs().sum() == 0


def test_prope_matrices_and_wan_camera_path():
    import torch

    from solarwm_b200.models import camera_prope
    from solarwm_b200.models.wan import WanConfig, WanDiT

    q, _ = torch.linalg.qr(torch.randn(3, 3, 3))
    view = torch.eye(4).repeat(3, 1, 1)
    view[:, :3, :3] = q
    view[:, :3, 3] = torch.randn(3, 3)
    Ks = torch.eye(3).repeat(3, 1, 1)
    Ks[:, 0, 0], Ks[:, 1, 1], Ks[:, 0, 2] = 0.6, 0.9, 0.5
    PT, Pinv, P = camera_prope.prope_matrices(view, Ks)
    assert torch.allclose(P @ Pinv, torch.eye(4).expand(3, 4, 4), atol=1e-5)
    assert torch.allclose(PT, P.transpose(1, 2))
    # attention logits are invariant to a common rigid change of the world frame
    g = torch.eye(4)
    g[:3, :3] = torch.linalg.qr(torch.randn(3, 3))[0]
    g[:3, 3] = torch.randn(3)
    PT2, Pinv2, _ = camera_prope.prope_matrices(view @ g, Ks)
    a, b = torch.randn(4), torch.randn(4)
    s1 = (PT[0] @ a) @ (Pinv[1] @ b)
    s2 = (PT2[0] @ a) @ (Pinv2[1] @ b)
    assert torch.allclose(s1, s2, atol=1e-4)
    # logd4 compresses long translations, keeps rotation
    far = view.clone()
    far[:, :3, 3] *= 100
    z = camera_prope.transform_translation(far, "logd4")
    assert torch.equal(z[:, :3, :3], far[:, :3, :3]) and (z[:, :3, 3].norm(dim=-1) < far[:, :3, 3].norm(dim=-1)).all()
    # Wan forward with identity cameras equals the forward without cameras; other cameras change it
    cfg = WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=256, ffn_dim=256, num_heads=2, num_layers=1,
                    text_dim=32, text_len=8, freq_dim=32)
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    x, t, ctx = torch.randn(1, 4, 3, 4, 4), torch.tensor([[100.0, 500.0, 900.0]]), torch.randn(1, 8, 32)
    base = m(x, t, ctx)
    ident = {"viewmats": torch.eye(4).repeat(1, 3, 1, 1), "Ks": None}
    assert torch.allclose(m(x, t, ctx, y_camera=ident), base, atol=1e-5)
    moved = {"viewmats": view.unsqueeze(0), "Ks": Ks.unsqueeze(0), "transform": "logd4"}
    assert not torch.allclose(m(x, t, ctx, y_camera=moved), base, atol=1e-4)


def test_unipc_exact_for_constant_data_and_beats_euler():
    import torch

    from solarwm_b200.engine.unipc import FlowUniPC, sample

    torch.manual_seed(0)
    x0 = torch.randn(4, 8)
    noise = torch.randn(4, 8)
    # a model whose data prediction is exactly x0: every consistent solver must return x0
    out = sample(lambda x, t: (x - x0) / max(t / 1000.0, 1e-9), noise, num_steps=8, shift=3.0)
    assert torch.allclose(out, x0, atol=1e-4)

    # the exact denoiser of Gaussian data N(mu, sd^2): 10 UniPC steps must beat 10 Euler steps by a wide margin
    mu, sd = 0.7, 0.5

    def vel(x, t):
        s = t / 1000.0
        a = 1 - s
        x0p = mu + a * sd * sd / (a * a * sd * sd + s * s) * (x - a * mu)
        return (x - x0p) / max(s, 1e-9)

    def euler(n):
        solver = FlowUniPC(n, 1.0)
        x = noise.double()
        for i in range(n):
            s, sn = float(solver.sigmas[i]), float(solver.sigmas[i + 1])
            x = x + (sn - s) * vel(x, s * 1000.0)
        return x

    ref = euler(20000)
    uni = sample(vel, noise.double(), num_steps=10, shift=1.0, order=2)
    err_uni, err_euler = (uni - ref).abs().max(), (euler(10) - ref).abs().max()
    assert err_uni < 0.1 * err_euler, (err_uni, err_euler)


def test_a14b_expert_switch_and_i2v_condition():
    import pytest
    import torch

    from solarwm_b200.backends.wan22.experts import (ExpertPair, expert_for_sigma, pack_i2v_condition,
                                                     sample_expert_sigmas)

    assert expert_for_sigma(0.9) == "high_noise" and expert_for_sigma(0.875) == "high_noise"
    assert expert_for_sigma(0.5) == "low_noise"
    g = torch.Generator().manual_seed(0)
    hi = sample_expert_sigmas(1000, "high_noise", generator=g)
    lo = sample_expert_sigmas(1000, "low_noise", generator=g)
    assert hi.min() >= 0.875 - 1e-6 and hi.max() <= 1.0 and lo.max() < 0.875 + 1e-6 and lo.min() >= 0
    y = pack_i2v_condition(torch.ones(1, 16, 1, 4, 4), frames=5)
    assert y.shape == (1, 20, 5, 4, 4) and y[:, :4, 0].min() == 1 and y[:, :4, 1:].abs().max() == 0
    assert y[:, 4:, 0].min() == 1 and y[:, 4:, 1:].abs().max() == 0
    calls = []

    class M(torch.nn.Module):
        def __init__(self, name):
            super().__init__()
            self.name = name

        def forward(self, x, t, c, **kw):
            calls.append(self.name)
            return x

    pair = ExpertPair(low_noise=M("low"), load=lambda n: M("loaded-" + n))
    x = torch.zeros(1, 4, 3, 2, 2)
    pair(x, torch.tensor([[0.0, 950.0, 950.0]]), None)
    pair(x, torch.tensor([[0.0, 300.0, 300.0]]), None)
    assert calls == ["loaded-high_noise", "low"]
    with pytest.raises(ValueError):
        pair(x, torch.tensor([[0.0, 950.0, 300.0]]), None)


def test_ltx_guided_sampler_and_provider():
    import torch

    from solarwm_b200.backends.ltx25.backend import RuntimeProvider, guided_x0, sample, sample_guided
    from solarwm_b200.models.ltx import LTXDiT, ltx_preset

    c, u, p = torch.full((4,), 2.0), torch.full((4,), 1.0), torch.full((4,), 0.5)
    assert torch.allclose(guided_x0(c, u, p, cfg_scale=3.0, stg_scale=1.0), torch.full((4,), 2.0 + 2.0 + 1.5))
    r = torch.randn(64)
    out = guided_x0(r, 0.5 * r, 0.5 * r, cfg_scale=3.0, stg_scale=1.0, rescale=1.0)
    assert abs(float(out.std()) - float(r.std())) < 1e-5               # full rescale restores the conditional spread
    m = LTXDiT(ltx_preset("tiny"), device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    text = torch.randn(1, 16, 64)
    x = torch.randn(1, 16, 2, 4, 4)
    t = torch.full((1, 2), 500.0)
    base, pert = m(x, t, text), m(x, t, text, perturb_blocks=(0,))
    assert not torch.allclose(base, pert, atol=1e-4)
    plain = sample(m, text, frames=2, height=4, width=4, steps=2, seed=1)
    same = sample_guided(m, text, torch.zeros_like(text), frames=2, height=4, width=4, steps=2, seed=1, cfg_scale=1.0,
                         stg_scale=0.0, rescale=0.0)
    assert torch.allclose(plain, same, atol=1e-5)                        # no guidance = the plain Euler sampler
    guided = sample_guided(m, text, torch.zeros_like(text), frames=2, height=4, width=4, steps=2, seed=1)
    assert torch.isfinite(guided).all() and not torch.allclose(plain, guided, atol=1e-3)
    prov = RuntimeProvider({"model": {"architecture": "tiny", "assets": {"vae": "/nonexistent/vae.pt"}},
                            "runtime": {"device": "cpu"}})
    rep = prov.readiness()
    assert not rep["ready"] and any("vae" in p for p in rep["problems"])


def test_lean_resident_blocks_rebuild_activations_with_identical_gradients():
    """Blocks that drop their norm outputs and FFN hidden activation (rebuilt inside backward) give the same
    parameter and input gradients as blocks that keep them."""
    from solarwm_b200.models.wan import WanConfig, WanDiT

    cfg = WanConfig(dim=64, ffn_dim=128, num_heads=2, num_layers=2, in_dim=4, out_dim=4, text_dim=32, freq_dim=32, text_len=8)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 4, 3, 4, 4, generator=g)
    t = torch.tensor([[500.0, 300.0, 100.0]])
    ctx = torch.randn(1, 8, 32, generator=g)
    grads = {}
    for lean in (False, True):
        m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=2)
        with torch.no_grad():
            m.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator().manual_seed(1))
        m.lean_kept = lean
        xin = x.clone().requires_grad_(True)
        m(xin, t, ctx).pow(2).mean().backward()
        grads[lean] = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
        grads[lean]["__input__"] = xin.grad.clone()
    assert set(grads[False]) == set(grads[True]) and len(grads[True]) > 20
    for n in grads[False]:
        assert torch.allclose(grads[False][n], grads[True][n], rtol=1e-5, atol=1e-7), n


def test_ltx_fixed_focal_camera_condition_changes_only_with_the_cameras():
    from solarwm_b200.models import camera_prope
    from solarwm_b200.models.ltx import FIXED_FX_NORM, LTXDiT, ltx_camera_condition, ltx_preset

    cfg = ltx_preset("tiny")                                  # 2 heads x 64
    m = LTXDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05, generator=g)     # the head starts at zero
    x, t, ctx = torch.randn(1, 16, 3, 4, 4, generator=g), torch.tensor([[400.0, 400.0, 400.0]]), torch.randn(1, 16, 64, generator=g)
    eye = torch.eye(4).repeat(1, 3, 1, 1)
    moved = eye.clone()
    moved[0, 1:, 0, 3] = 0.3
    cond = ltx_camera_condition(eye)
    assert abs(float(cond["Ks"][0, 0, 0, 0]) - FIXED_FX_NORM) < 1e-7 and cond["Ks"].shape == (1, 3, 3, 3)
    with torch.no_grad():
        plain, same, other = m(x, t, ctx), m(x, t, ctx, y_camera=cond), m(x, t, ctx, y_camera=ltx_camera_condition(moved, "logd4"))
    # identical cameras: P cancels between q^T k and the output transform (same frame <-> same P), up to rounding
    assert torch.allclose(plain, same, atol=1e-4)
    assert (other - plain).abs().max() > 1e-4
    # 64-wide heads ride the 128-wide camera kernel as pseudo-heads: same numbers as the dense 4x4 products
    rows = torch.randn(5, 128, generator=g)
    mats = torch.randn(5, 4, 4, generator=g)
    want = torch.einsum("rij,rnj->rni", mats, rows.view(5, 32, 4)).reshape(5, 128)
    assert torch.allclose(camera_prope.apply(rows, mats, heads=2), want, atol=1e-5)
    with pytest.raises(ValueError):
        ltx_camera_condition(torch.eye(4))
