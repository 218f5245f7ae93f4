"""Teacher-forcing forward and Stage1 trainers (CPU, fp32 oracle path)."""
import pytest
import torch

from solarwm_b200.models.wan import WanConfig, WanDiT
from solarwm_b200.models.wan_causal import teacher_forcing_mask
from solarwm_b200.models import wan_tf
from solarwm_b200.ops import reference as R


def tiny():
    cfg = WanConfig(model_type="ti2v", in_dim=4, out_dim=4, dim=64, ffn_dim=128, num_heads=2, num_layers=2,
                    text_dim=32, text_len=8, freq_dim=32)
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    return cfg, m


@pytest.mark.parametrize("F", [4, 5])          # 5 frames: the last chunk is ragged
def test_teacher_forcing_matches_dense_mask(monkeypatch, F):
    cfg, m = tiny()
    H, W = 4, 4
    g = torch.Generator().manual_seed(0)
    clean = torch.randn(1, 4, F, H, W, generator=g)
    noisy = torch.randn(1, 4, F, H, W, generator=g)
    t = torch.tensor([[700.0, 700.0, 300.0, 300.0, 500.0][:F]])
    ctx = torch.randn(1, 8, 32, generator=g)
    out = wan_tf.forward_teacher_forcing(m, clean, noisy, t, ctx, chunk_frames=2, window_chunks=1)
    ft = (H // 2) * (W // 2)
    mask = teacher_forcing_mask(F, ft, 2, 1)

    def dense(qc, kc, vc, qn, kn, vn, **kw):
        q, k, v = torch.cat([qc, qn], 1), torch.cat([kc, kn], 1), torch.cat([vc, vn], 1)
        o = R.attention(q, k, v, mask=mask.view(1, 1, *mask.shape))
        L = qc.shape[1]
        return o[:, :L], o[:, L:]

    monkeypatch.setattr(wan_tf, "teacher_forcing_attention", dense)
    ref = wan_tf.forward_teacher_forcing(m, clean, noisy, t, ctx, chunk_frames=2, window_chunks=1)
    assert out.shape == (1, 4, F, H, W)
    assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)


def test_first_chunk_equals_plain_forward():
    cfg, m = tiny()
    g = torch.Generator().manual_seed(1)
    clean = torch.randn(1, 4, 4, 4, 4, generator=g)
    noisy = torch.randn(1, 4, 4, 4, 4, generator=g)
    t = torch.tensor([[500.0, 500.0, 200.0, 200.0]])
    ctx = torch.randn(1, 8, 32, generator=g)
    out = wan_tf.forward_teacher_forcing(m, clean, noisy, t, ctx, chunk_frames=2, window_chunks=3)
    plain = m(noisy[:, :, :2], t[:, :2], ctx)
    assert torch.allclose(out[:, :, :2], plain, atol=1e-5, rtol=1e-4)


def test_window_forward_matches_teacher_forcing_last_chunk():
    cfg, m = tiny()
    g = torch.Generator().manual_seed(2)
    clean = torch.randn(1, 4, 4, 4, 4, generator=g)
    noisy = torch.randn(1, 4, 4, 4, 4, generator=g)
    t = torch.tensor([[500.0, 500.0, 200.0, 200.0]])
    ctx = torch.randn(1, 8, 32, generator=g)
    tf = wan_tf.forward_teacher_forcing(m, clean, noisy, t, ctx, chunk_frames=2, window_chunks=3)
    frames = torch.cat([clean[:, :, :2], noisy[:, :, 2:]], dim=2)
    tw = torch.tensor([[0.0, 0.0, 200.0, 200.0]])
    win = wan_tf.forward_window(m, frames, tw, ctx, first_frame=0, current_frames=2, chunk_frames=2, window_chunks=3)
    assert torch.allclose(win, tf[:, :, 2:], atol=1e-5, rtol=1e-4)


def test_stage1_trainers_step():
    from solarwm_b200.backends.wan22.stage1 import Stage1Options, WanStage1Trainer

    cfg, m = tiny()
    for objective in ("tf_fm", "anyflow"):
        tr = WanStage1Trainer(cfg, "cpu", Stage1Options(objective=objective, chunk_frames=2, window_chunks=2, lr=1e-3,
                                                        diffusion_ratio=0.34, consistency_ratio=0.33),
                              model=WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0))
        with torch.no_grad():
            tr.model.get_parameter("head.head.weight").normal_(0, 0.05)
        before = tr.model.get_parameter("blocks.0.ffn.0.weight").detach().clone()
        batch = {"latents": torch.randn(1, 6, 4, 4, 4), "text": torch.randn(1, 8, 32)}
        loss = tr.train_step(batch)
        assert torch.isfinite(loss)
        assert not torch.equal(before, tr.model.get_parameter("blocks.0.ffn.0.weight"))


def test_stage2_outer_steps_and_role_state():
    from solarwm_b200.backends.wan22.stage2 import Stage2Options, WanStage2Trainer

    cfg, _ = tiny()
    tr = WanStage2Trainer(cfg, "cpu", Stage2Options(chunk_frames=2, window_chunks=2, critic_updates_per_student=2,
                                                    denoising_steps=(1000.0, 500.0)), dtype=torch.float32)
    for m in (tr.student, tr.teacher, tr.critic):
        with torch.no_grad():
            m.get_parameter("head.head.weight").normal_(0, 0.05)
    batch = {"latents": torch.randn(1, 4, 4, 4, 4), "text": torch.randn(1, 8, 32)}
    teacher_before = tr.teacher.get_parameter("blocks.0.ffn.0.weight").detach().clone()
    student_before = tr.student.get_parameter("blocks.0.ffn.0.weight").detach().clone()
    r0 = tr.train_outer_step(batch)
    assert "critic" in r0 and "student" not in r0            # step 0 trains the critic only
    assert torch.equal(student_before, tr.student.get_parameter("blocks.0.ffn.0.weight"))
    tr.train_outer_step(batch)
    r2 = tr.train_outer_step(batch)                           # step 2: student too
    assert "student" in r2 and r2["student"] == r2["student"]
    assert not torch.equal(student_before, tr.student.get_parameter("blocks.0.ffn.0.weight"))
    assert torch.equal(teacher_before, tr.teacher.get_parameter("blocks.0.ffn.0.weight"))
    state = tr.role_state()
    tr2 = WanStage2Trainer(cfg, "cpu", tr.opts, dtype=torch.float32)
    tr2.load_role_state(state)
    assert tr2.global_step == 3
    assert torch.equal(tr2.student.get_parameter("blocks.0.ffn.0.weight"), tr.student.get_parameter("blocks.0.ffn.0.weight"))


def test_stage2_student_ema_follows_student_steps_only_and_round_trips():
    from solarwm_b200.backends.wan22.stage2 import Stage2Options, WanStage2Trainer
    from solarwm_b200.errors import BackendContractError

    cfg, _ = tiny()
    opts = Stage2Options(chunk_frames=2, window_chunks=2, critic_updates_per_student=2, denoising_steps=(1000.0, 500.0),
                         ema_decay=0.5, ema_start_step=0, lr_student=1e-3)
    tr = WanStage2Trainer(cfg, "cpu", opts, dtype=torch.float32)
    for m in (tr.student, tr.teacher, tr.critic):
        with torch.no_grad():
            m.get_parameter("head.head.weight").normal_(0, 0.05)
    tr.ema_student.load_state_dict({n: p.detach().float().clone() for n, p in tr.student.named_parameters()}, num_updates=0)
    name = "blocks.0.ffn.0.weight"
    start = tr.student.get_parameter(name).detach().clone()
    batch = {"latents": torch.randn(1, 4, 4, 4, 4), "text": torch.randn(1, 8, 32)}
    tr.train_outer_step(batch)
    tr.train_outer_step(batch)
    assert tr.ema_student.num_updates == 0                                   # critic-only steps leave the average alone
    tr.train_outer_step(batch)
    assert tr.ema_student.num_updates == 1
    live = tr.student.get_parameter(name).detach()
    assert torch.allclose(tr.ema_student.shadow[name], 0.5 * start + 0.5 * live, atol=1e-6)
    state = tr.role_state()
    tr2 = WanStage2Trainer(cfg, "cpu", opts, dtype=torch.float32)
    tr2.load_role_state(state)
    assert tr2.ema_student.num_updates == 1 and torch.equal(tr2.ema_student.shadow[name], tr.ema_student.shadow[name])
    state.pop("ema_student")
    with pytest.raises(BackendContractError):
        tr2.load_role_state(state)
    # before ``ema_start_step`` the shadow follows the student exactly
    early = WanStage2Trainer(cfg, "cpu", Stage2Options(chunk_frames=2, window_chunks=2, critic_updates_per_student=1,
                                                       denoising_steps=(1000.0, 500.0), ema_decay=0.9, lr_student=1e-3),
                             dtype=torch.float32)
    for m in (early.student, early.teacher, early.critic):
        with torch.no_grad():
            m.get_parameter("head.head.weight").normal_(0, 0.05)
    early.train_outer_step(batch)
    assert torch.equal(early.ema_student.shadow[name], early.student.get_parameter(name).detach().float())


@pytest.mark.parametrize("F,sink", [(4, 0), (5, 1)])
def test_noisy_suffix_on_captured_clean_half_matches_full_teacher_forcing(F, sink):
    cfg, m = tiny()
    g = torch.Generator().manual_seed(0)
    clean = torch.randn(1, 4, F, 4, 4, generator=g)
    ctx = torch.randn(1, 8, 32, generator=g)
    kw = dict(chunk_frames=2, window_chunks=1, sink_frames=sink)
    t0 = torch.tensor([[700.0, 700.0, 300.0, 300.0, 500.0][:F]])
    t1 = t0 + 5.0
    with torch.no_grad():
        prefix = []
        wan_tf.forward_teacher_forcing(m, clean, torch.randn(1, 4, F, 4, 4, generator=g), t0, ctx, capture=prefix, **kw)
        assert len(prefix) == len(m.blocks) and prefix[0][0].shape[1] == F * 4
        noisy = torch.randn(1, 4, F, 4, 4, generator=g)
        want = wan_tf.forward_teacher_forcing(m, clean, noisy, t1, ctx, **kw)
        got = wan_tf.forward_noisy_suffix(m, noisy, t1, ctx, prefix, **kw)
    assert got.shape == want.shape and torch.allclose(got, want, atol=1e-5, rtol=1e-4)


def test_stage1_anyflow_step_with_and_without_prefix_reuse_agree():
    from solarwm_b200.backends.wan22.stage1 import Stage1Options, WanStage1Trainer

    cfg, _ = tiny()
    cfg.flow_objective = "anyflow_forward_map"
    losses, grads = [], []
    for reuse in (False, True):
        opts = Stage1Options(objective="anyflow", chunk_frames=2, window_chunks=1, diffusion_ratio=0.0, consistency_ratio=0.5,
                             seed=5, reuse_prefix=reuse)
        tr = WanStage1Trainer(cfg, "cpu", opts, dtype=torch.float32)
        with torch.no_grad():
            tr.model.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator().manual_seed(1))
        lat = torch.randn(1, 4, 4, 4, 4, generator=torch.Generator().manual_seed(2))
        text = torch.randn(1, 8, 32, generator=torch.Generator().manual_seed(3))
        losses.append(float(tr.microbatch(lat, text)))
        grads.append(tr.model.get_parameter("blocks.0.ffn.0.weight").grad.clone())
    assert abs(losses[0] - losses[1]) < 1e-5 * max(1.0, abs(losses[0]))
    assert torch.allclose(grads[0], grads[1], atol=1e-6, rtol=1e-4)


def test_stage2_rollouts_share_one_preallocated_cache():
    """The rollout cache is allocated once per token grid and reset between rollouts; a rollout that follows another
    one (and therefore runs in used buffers) equals the same rollout in a fresh trainer."""
    from solarwm_b200.backends.wan22.stage2 import Stage2Options, WanStage2Trainer

    cfg, _ = tiny()
    opts = Stage2Options(chunk_frames=2, window_chunks=1, critic_updates_per_student=1, denoising_steps=(1000.0, 500.0))

    def make():
        tr = WanStage2Trainer(cfg, "cpu", opts, dtype=torch.float32)
        with torch.no_grad():
            tr.student.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator().manual_seed(3))
        return tr

    text = torch.randn(1, 8, 32, generator=torch.Generator().manual_seed(4))
    a, b = make(), make()
    a.rollout(text, (1, 6, 4, 4, 4), torch.float32, exit_index=0)           # leaves the buffers used (window slid)
    cache = a.rollout_cache((2, 2))
    assert a.rollout_cache((2, 2)) is cache and cache.committed_frames == 0 and cache.layers[0].text_k is None
    b.gen.set_state(a.gen.get_state())
    got, _, _ = a.rollout(text, (1, 6, 4, 4, 4), torch.float32, exit_index=1)
    want, _, _ = b.rollout(text, (1, 6, 4, 4, 4), torch.float32, exit_index=1)
    assert torch.equal(got, want)
