"""Renderer: observation plans, omni flow-matching trainer, pinned rendering, DMD distillation (CPU)."""
import numpy as np
import pytest
import torch

from solarwm_b200.renderer import known_degree as kd


def test_observation_plans_cover_patterns_and_invariants():
    prof = kd.ObservationProfile(patterns=tuple((p, 1.0) for p in kd.PATTERNS), dropout=(("camera", 0.5), ("observation", 0.3)))
    rng = np.random.default_rng(0)
    seen = set()
    for _ in range(200):
        plan = kd.sample_plan(prof, frames=6, grid_height=6, grid_width=8, base_time=float(rng.random()), shift=12.0, rng=rng,
                              given=np.clip(rng.random((6, 6, 8)) - 0.3, 0, 1))
        seen.add(plan.pattern)
        assert plan.row_times.shape == (6 * 6 * 8,) and plan.loss_rows.any()
        assert plan.row_times.min() >= 0 and plan.row_times.max() <= prof.hard_level + 1e-6
        assert np.allclose(plan.row_times * prof.levels, np.round(plan.row_times * prof.levels), atol=1e-3)
        assert (plan.row_times[plan.loss_rows] < prof.hard_level).all()
        assert (plan.row_times >= min(plan.base_time, plan.row_times.min()) - 1e-6).all()
    assert seen == set(kd.PATTERNS)
    # same generator state -> same plan
    a = kd.sample_plan(prof, frames=4, grid_height=3, grid_width=3, base_time=0.3, shift=12.0, rng=np.random.default_rng(5))
    b = kd.sample_plan(prof, frames=4, grid_height=3, grid_width=3, base_time=0.3, shift=12.0, rng=np.random.default_rng(5))
    assert a.pattern == b.pattern and np.array_equal(a.row_times, b.row_times)
    assert kd.confidence_to_known_degree(0.0) == 1.0 and kd.confidence_to_known_degree(np.inf) == 0.0
    with pytest.raises(ValueError):
        kd.ObservationProfile(patterns=(("nope", 1.0),))
    assert abs(kd.unshift_time(float(kd.shift_time(0.37, 12.0)), 12.0) - 0.37) < 1e-12


def test_trainer_render_and_distillation():
    from solarwm_b200.renderer.cli import _sample, main
    from solarwm_b200.renderer.core import OmniFlowTrainer, render
    from solarwm_b200.renderer.dmd import RendererDMDTrainer, structure_guided
    from solarwm_b200.models.h3 import h3_preset

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    prof = kd.ObservationProfile(patterns=(("known_frames", 1.0), ("known_region", 1.0)))
    tr = OmniFlowTrainer(cfg, "cpu", prof, lr=1e-3)
    before = [p.detach().clone() for p in tr.model.trainable_parameters()]
    loss = tr.train_step(_sample(cfg, 0))
    assert torch.isfinite(loss) and 0 < tr.last_plan.generated_fraction < 1
    assert any(not torch.equal(a, b) for a, b in zip(before, tr.model.trainable_parameters()))
    # rendering with fully known rows returns them (degree 1 rows are pinned to the known clip)
    s = _sample(cfg, 1)
    known = s["target_latents"]
    deg = torch.zeros(4 * 4 * 4)
    deg[:16] = 1.0                                    # the first frame is given
    out = render(tr.model, s, steps=3, known=known, known_degree=deg)
    assert out.shape == known.shape and torch.isfinite(out).all()
    assert torch.allclose(out[:, 0].float(), known[:, 0].float(), atol=2e-2)
    assert not torch.allclose(out[:, 1].float(), known[:, 1].float(), atol=1e-1)
    assert torch.equal(structure_guided(torch.ones(2), torch.zeros(2), 2.0), torch.full((2,), 2.0))
    d = RendererDMDTrainer(cfg, "cpu", student_steps=2, critic_updates_per_student=2, lr_student=1e-3, lr_critic=1e-3)
    r0 = d.train_outer_step(s)
    d.train_outer_step(s)
    r2 = d.train_outer_step(s)
    assert "student" not in r0 and "student" in r2 and r2["critic"] == r2["critic"]
    assert main(["train", "--steps", "1", "--device", "cpu"]) == 0


def test_render_service_caches_reproduce_the_plain_renderer_and_refuse_unprepared_times():
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.renderer.cli import _sample
    from solarwm_b200.renderer.core import render
    from solarwm_b200.renderer.service import RenderService, schedule_time_sets

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    s = _sample(cfg, 3)
    with torch.no_grad():
        want = render(model, s, steps=3, seed=5)
    svc = RenderService(model, steps=3, free_projection=True)
    with pytest.raises(RuntimeError):
        svc.render(s)
    report = svc.prepare()
    assert len(report["time_sets"]) == 3 == len(schedule_time_sets(3)) and report["adaln_weight_bytes_removed"] > 0
    assert all(blk.adaln_proj.numel() == 0 for blk in model.blocks)       # projection weights are gone
    got = svc.render(s, seed=5)
    assert torch.equal(got, want)
    assert model.text_cache["hits"] == 2                                     # steps 2 and 3 reuse the refined prompt
    svc.render(_sample(cfg, 4), seed=5)                                      # another prompt: cache refills, no stale hit
    assert model.text_cache["hits"] == 4
    with torch.no_grad(), pytest.raises(ValueError, match="not prepared"):
        render(model, s, steps=2, seed=5)                                    # a different grid of times


def test_render_service_http_transport(tmp_path):
    import http.client
    import json
    import threading

    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.renderer.cli import _sample
    from solarwm_b200.renderer.service import RenderService, make_server

    cfg = h3_preset("tiny")
    svc = RenderService(H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0), steps=2)
    svc.prepare()
    server = make_server(svc, {"s0": _sample(cfg, 0)}, tmp_path / "out")
    threading.Thread(target=server.serve_forever, daemon=True).start()
    try:
        def call(method, path, body=None):
            c = http.client.HTTPConnection("127.0.0.1", server.server_address[1], timeout=60)
            c.request(method, path, None if body is None else json.dumps(body), {"Content-Type": "application/json"})
            r = c.getresponse()
            return r.status, json.loads(r.read())

        assert call("GET", "/health")[1]["prepared"] is True and call("GET", "/samples")[1] == ["s0"]
        st, job = call("POST", "/render", {"sample": "s0", "seed": 3})
        assert st == 200 and (tmp_path / "out" / job["file"]).exists() and job["shape"] == list(_sample(cfg, 0)["shape"])
        assert torch.equal(torch.load(tmp_path / "out" / job["file"]), svc.render(_sample(cfg, 0), seed=3).cpu())
        assert call("POST", "/render", {"sample": "nope"})[0] == 404 and call("POST", "/render", {"seed": 1})[0] == 400
        assert call("GET", "/jobs")[1] == [job] and call("GET", "/x")[0] == 404
        c = http.client.HTTPConnection("127.0.0.1", server.server_address[1], timeout=60)
        c.request("GET", "/")
        page = c.getresponse()
        html = page.read().decode()
        assert page.status == 200 and page.getheader("Content-Type").startswith("text/html")
        assert all(path in html for path in ("'/health'", "'/samples'", "'/render'", "'/jobs'")) and "<script src" not in html
    finally:
        server.shutdown()


def test_node_graph_front_end_follows_the_node_protocol_and_renders():
    from solarwm_b200 import ops
    from solarwm_b200.models.h3 import h3_preset
    from solarwm_b200.renderer import comfy_nodes as cn
    from solarwm_b200.renderer.cli import _sample

    assert set(cn.NODE_CLASS_MAPPINGS) == set(cn.NODE_DISPLAY_NAME_MAPPINGS)
    for cls in cn.NODE_CLASS_MAPPINGS.values():
        spec = cls.INPUT_TYPES()
        assert "required" in spec and isinstance(cls.RETURN_TYPES, tuple) and hasattr(cls, cls.FUNCTION) and cls.CATEGORY == "SolarRenderer"
    (svc,) = cn.SolarRendererModelLoader().load(architecture="tiny", steps=2, device="cpu")
    (sig,) = cn.SolarRendererSigmas().sigmas(2)
    assert len(sig) == 3 and float(sig[0]) == 1.0 and float(sig[-1]) == 0.0
    from solarwm_b200.ops.attention import get_backend

    before = get_backend()
    try:
        (svc,) = cn.SolarRendererAttention().patch(svc, "auto")
        with pytest.raises(RuntimeError):
            cn.SolarRendererAttention().patch(svc, "native")
        (prompt,) = cn.SolarRendererPrompt().build("near_depth", " a harbour at dusk ")
        assert prompt.endswith("a harbour at dusk") and "depth map" in prompt
        with pytest.raises(ValueError):
            cn.SolarRendererPrompt().build("custom", "x", "")
        s = _sample(h3_preset("tiny"), 2)
        (lat,) = cn.SolarRendererSampler().sample(svc, s, seed=1, sigmas=sig)
        assert lat["samples"].shape == (1, *s["shape"]) and torch.isfinite(lat["samples"]).all()
        with pytest.raises(ValueError):
            cn.SolarRendererSampler().sample(svc, s, seed=1, sigmas=sig[:2])
    finally:
        ops.set_backend(before)


def test_conditioning_lora_and_capture_nodes(tmp_path):
    import numpy as np

    from solarwm_b200.models.h3 import h3_preset
    from solarwm_b200.renderer import comfy_nodes as cn

    assert [cn.snap_frames(200, n) for n in (22, 38, 39, 158, 500)] == [22, 22, 39, 158, 192]
    with pytest.raises(ValueError):
        cn.snap_frames(21, 158)
    wide = torch.zeros(2, 20, 60, 3)
    wide[:, :, 25:35] = 1.0
    fitted = cn.fit_images(wide, 16, 16)
    assert fitted.shape == (2, 16, 16, 3) and float(fitted[0, 8, 8, 0]) > 0.9 and float(fitted[0, 8, 0, 0]) < 0.1

    class Codec:                                                     # the host's VAE protocol, at the codec's cadence
        def encode(self, images):
            T = images.shape[0]
            F = 1 if T < 22 else 5 * ((T - 5) // 17) + 2
            return images[:1].mean(dim=(0, 3))[None, None, ::4, ::4].repeat(24, F, 1, 1)

    cfg = h3_preset("tiny")
    node = cn.SolarRendererConditioning()
    structure = torch.rand(30, 20, 30, 3)
    cond, latent = node.encode(lambda p: torch.full((5, cfg.text_dim), float(len(p))), Codec(), structure, "a harbour", width=32, height=16,
                               length=158, first_frame=torch.rand(1, 20, 30, 3))
    assert cond["shape"] == (24, 7, 4, 8) and cond["pixel_frames"] == 22 and cond["has_first_frame"]
    assert latent["samples"].shape == (1, 24, 7, 4, 8) and cond["anchor_latents"].shape == (24, 1, 4, 8)
    no_first, _ = node.encode(lambda p: torch.zeros(5, cfg.text_dim), Codec(), structure, "x", width=32, height=16, length=22)
    assert float(no_first["anchor_latents"].abs().sum()) == 0.0
    with pytest.raises(ValueError):
        node.encode(lambda p: torch.zeros(5, cfg.text_dim), Codec(), structure[:10], "x", width=32, height=16)
    # the conditioning renders through the sampler node
    (svc,) = cn.SolarRendererModelLoader().load(architecture="tiny", steps=2, device="cpu")
    (lat,) = cn.SolarRendererSampler().sample(svc, cond, seed=0)
    assert lat["samples"].shape == (1, 24, 7, 4, 8) and torch.isfinite(lat["samples"]).all()
    # key / mouse scripts
    plan = cn.capture_plan("0.5:KeyW:1.0, 1.0:mouse:30:0:0.1\n2:click, 0.2:down:ShiftLeft, 3:up:ShiftLeft")
    assert plan[0] == (0.2, "down", "ShiftLeft") and (0.5, "down", "KeyW") in plan and (1.5, "up", "KeyW") in plan
    moves = [e for e in plan if e[1] == "move"]
    assert len(moves) == 3 and sum(m[2][0] for m in moves) == pytest.approx(30.0) and plan[-1] == (3.0, "up", "ShiftLeft")
    assert [e[1] for e in plan if e[1].startswith("m") and e[1] != "move"] == ["mdown", "mup"]
    for bad in ("oops", "-1:KeyW"):
        with pytest.raises(ValueError):
            cn.capture_plan(bad)
    # a capture made by an external process is loaded as host images; the command is run with its fields filled in
    out = tmp_path / "cap"
    import sys

    maker = tmp_path / "fake_capture.py"
    maker.write_text("import sys, numpy as np\nnp.save(sys.argv[2] + '.npy', np.full((int(sys.argv[3]), 6, 8, 3), 128, np.uint8))\n")
    (images,) = cn.SolarRendererWebCapture().capture("http://127.0.0.1/x", frames=24, out=str(out), script="0:KeyW",
                                                     command=f"{sys.executable} {maker} {{url}} {{out}} {{frames}}")
    assert images.shape == (24, 6, 8, 3) and float(images.mean()) == pytest.approx(128 / 255, abs=1e-6)
    with pytest.raises(FileNotFoundError):
        cn.SolarRendererWebCapture().capture("u", out=str(tmp_path / "absent"))
    with pytest.raises(RuntimeError):
        cn.SolarRendererWebCapture().capture("u", out=str(out), command=f"{sys.executable} -c 'raise SystemExit(3)'")


def test_lora_loader_node_fills_adapters_and_scales_the_up_projection(tmp_path):
    from solarwm_b200.backends.minimax_h3.runtime import ADAPTER_SCHEMA
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.renderer import comfy_nodes as cn
    from solarwm_b200.renderer.service import RenderService

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    svc = RenderService(model, steps=2)
    svc.prepare()
    g = torch.Generator().manual_seed(1)
    state = {n: torch.randn(p.shape, generator=g) for n, p in model.named_parameters() if "lora_" in n}
    torch.save({"schema": ADAPTER_SCHEMA, "state": state, "rank": 4}, tmp_path / "adapter.pt")
    (svc,) = cn.SolarRendererLoraLoader().load(svc, str(tmp_path / "adapter.pt"), strength=0.5)
    got = dict(model.named_parameters())
    a = next(n for n in state if "lora_A" in n)
    b = next(n for n in state if "lora_B" in n)
    assert torch.equal(got[a], state[a]) and torch.allclose(got[b], 0.5 * state[b])
    torch.save({"schema": ADAPTER_SCHEMA, "state": {"other": torch.zeros(1)}, "rank": 4}, tmp_path / "bad.pt")
    with pytest.raises(ValueError):
        cn.SolarRendererLoraLoader().load(svc, str(tmp_path / "bad.pt"))
