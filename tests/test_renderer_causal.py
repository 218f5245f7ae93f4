"""Block-causal renderer: the visibility plan against its dense oracle, segment attention against masked attention, and
the stream's chunk evaluations against the training document's predictions."""
import pytest
import torch

from solarwm_b200.backends.minimax_h3.layout import patchify_latents
from solarwm_b200.models.h3 import H3DiT, h3_preset
from solarwm_b200.renderer.causal import (CLEAN_LEVEL, CausalRenderer, ChunkKVCache, chunk_spans, document_rows, plan_mask,
                                          segment_attention, teacher_forcing_prediction, training_plan)
from solarwm_b200.renderer.cli import _sample


def test_plan_follows_the_visibility_rule():
    assert chunk_spans(12, 5) == [(0, 5), (5, 10), (10, 12)]
    with pytest.raises(ValueError):
        chunk_spans(0, 5)
    rows = document_rows(3, [2, 2, 2], structure=True, clean_copy=True)
    assert rows.static == (0, 3) and rows.structure[1] == (5, 7) and rows.clean[0] == (9, 11) and rows.noisy[2] == (19, 21) and rows.total == 21
    m = plan_mask(training_plan(rows, window=2), rows.total)
    static, s, c, n = slice(0, 3), rows.structure, rows.clean, rows.noisy
    sl = lambda span: slice(*span)                                    # noqa: E731
    assert m[static, static].all() and not m[static, 3:].any()
    assert m[sl(s[1]), static].all() and m[sl(s[1]), sl(s[1])].all() and not m[sl(s[1]), sl(s[0])].any() and not m[sl(s[1]), 9:].any()
    # noisy chunk 2 with a window of two: structure 1-2, clean 1, itself; not structure 0, clean 0, clean 2, other noisy chunks
    q = sl(n[2])
    assert m[q, static].all() and m[q, sl(s[1])].all() and m[q, sl(s[2])].all() and m[q, sl(c[1])].all() and m[q, q].all()
    assert not m[q, sl(s[0])].any() and not m[q, sl(c[0])].any() and not m[q, sl(c[2])].any() and not m[q, sl(n[1])].any()
    # clean chunk 2 sees the same with its own rows in place of the noisy ones
    qc = sl(c[2])
    assert m[qc, sl(c[1])].all() and m[qc, qc].all() and not m[qc, sl(n[2])].any() and not m[qc, sl(c[0])].any()
    # nothing sees a later chunk
    for j in range(3):
        for later in range(j + 1, 3):
            for kind in (s, c, n):
                assert not m[sl(n[j]), sl(kind[later])].any() and not m[sl(c[j]), sl(kind[later])].any()
    # diffusion forcing (no clean copy): the history is the noisy chunks themselves
    df = document_rows(3, [2, 2, 2], structure=False, clean_copy=False)
    md = plan_mask(training_plan(df, window=2), df.total)
    assert md[sl(df.noisy[2]), sl(df.noisy[1])].all() and not md[sl(df.noisy[2]), sl(df.noisy[0])].any()


def test_segment_attention_equals_masked_attention():
    torch.manual_seed(0)
    rows = document_rows(3, [2, 4, 2], structure=True, clean_copy=True)
    plan = training_plan(rows, window=2)
    S = rows.total
    q, k, v = (torch.randn(1, S, 2, 16) for _ in range(3))
    got = segment_attention(q, k, v, plan)
    mask = plan_mask(plan, S)
    want = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask).transpose(1, 2)
    assert torch.allclose(got, want, atol=1e-5)


def _model_and_sample(frames=6):
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    s = _sample(cfg, 3, frames=frames, size=4)
    g = torch.Generator().manual_seed(9)
    cams = torch.eye(4).repeat(frames + 1, 1, 1)
    cams[:, 0, 3] = torch.arange(frames + 1) * 0.05
    s["camera_w2c"] = cams
    return model, s, g


def test_the_stream_computes_what_the_training_document_predicts():
    model, s, g = _model_and_sample()
    C, F, H, W = s["shape"]
    per = (H // 2) * (W // 2)
    noisy = torch.randn(F * per, C * 4, generator=g)
    t_chunks = torch.tensor([0.3, 0.5, 0.7])
    with torch.no_grad():
        want = teacher_forcing_prediction(model, s, noisy, t_chunks, chunk=2, window=2)
        r = CausalRenderer(model, chunk=2, window=2, steps=2)
        cache = ChunkKVCache(2)
        prompt = s["prompt_embeds"].float()
        anchor_rows = patchify_latents(s["anchor_latents"]).float()
        s_rows, clean = patchify_latents(s["structure_latents"]).float(), patchify_latents(s["target_latents"]).float()
        for j, (a, b) in enumerate(chunk_spans(F, 2)):
            kw = dict(prompt=prompt, anchor_rows=anchor_rows, structure_rows=s_rows[a * per:b * per], frames=(a, b), total_frames=F,
                      grid_hw=(H // 2, W // 2), cameras=s["camera_w2c"])
            got = r._evaluate(cache, target_rows=noisy[a * per:b * per], t=float(t_chunks[j]), commit=False, **kw)
            assert torch.allclose(got, want[a * per:b * per], atol=2e-4, rtol=1e-4), (j, (got - want[a * per:b * per]).abs().max())
            assert cache.chunks == min(j, 1)                           # a window of two keeps one committed chunk
            r._evaluate(cache, target_rows=clean[a * per:b * per], t=CLEAN_LEVEL, commit=True, **kw)
    # a wider window changes what chunk 2 sees
    with torch.no_grad():
        wide = teacher_forcing_prediction(model, s, noisy, t_chunks, chunk=2, window=3)
    assert torch.allclose(wide[:2 * 2 * per], want[:2 * 2 * per], atol=1e-5) and not torch.allclose(wide[4 * per:], want[4 * per:], atol=1e-4)


def test_rendering_is_chunked_seeded_and_bounded():
    model, s, _ = _model_and_sample(frames=7)
    record = []
    r = CausalRenderer(model, chunk=3, window=2, steps=2)
    a = r.render(s, seed=5, record=record)
    assert a.shape == tuple(s["shape"]) and torch.isfinite(a).all()
    assert [x["frames"] for x in record] == [[0, 3], [3, 6], [6, 7]] and max(x["cached_chunks"] for x in record) == 1
    assert torch.equal(a, r.render(s, seed=5)) and not torch.equal(a, r.render(s, seed=6))
    plain = dict(s)
    plain.pop("structure_latents")
    b = r.render(plain, seed=5)                                       # no structure stream: still a valid document
    assert b.shape == a.shape and not torch.equal(a, b)


def test_causal_sampler_node_and_cli(tmp_path, capsys):
    import json

    from solarwm_b200.renderer import comfy_nodes as cn
    from solarwm_b200.renderer.cli import main

    (svc,) = cn.SolarRendererModelLoader().load(architecture="tiny", steps=2, device="cpu")
    s = _sample(h3_preset("tiny"), 2, frames=6, size=4)
    (lat,) = cn.SolarRendererCausalSampler().sample(svc, s, seed=1, chunk=2, window=2, steps=2)
    assert lat["samples"].shape == (1, *s["shape"]) and svc.model.fixed_tables is not None
    assert main(["render", "--causal", "--frames", "6", "--chunk", "2", "--window", "2", "--device", "cpu", "--out", str(tmp_path)]) == 0
    assert json.loads(capsys.readouterr().out)["finite"] is True and (tmp_path / "latents.pt").is_file()


def test_causal_training_runs_behind_the_renderer_runtime(tmp_path):
    from solarwm_b200.checkpoint.store import verify_checkpoint
    from solarwm_b200.errors import BackendContractError, ConfigurationError
    from solarwm_b200.renderer.runtime import RendererTrainingRuntime, run_control_training, validate_config
    from tests.test_renderer_runtime import _config, _corpus

    _corpus(tmp_path / "corpus", n=4, frames=lambda i: 4)
    cfg = _config(tmp_path / "corpus", tmp_path / "run", train={"causal_omni": {"chunk": 2, "window": 2}, "max_steps": 2,
                                                                "gradient_accumulation_steps": 1})
    out = run_control_training(cfg)
    assert out["final_step"] == 2 and out["last_loss"] == out["last_loss"]
    ck = verify_checkpoint(out["checkpoint"])
    assert ck.contract.causal_mode == "block_causal"
    # the causal chunking is part of the resume identity
    other = _config(tmp_path / "corpus", tmp_path / "run2", train={"causal_omni": {"chunk": 4, "window": 2}, "max_steps": 3,
                                                                   "gradient_accumulation_steps": 1}, checkpoint={"resume_from": out["checkpoint"]})
    with pytest.raises(BackendContractError):
        RendererTrainingRuntime(other)
    with pytest.raises(ConfigurationError):
        validate_config(_config(tmp_path / "corpus", tmp_path / "x", train={"causal_omni": {"chunk": 0}}))
    # gradients reach the adapters through the segment-attention document
    rt = RendererTrainingRuntime(_config(tmp_path / "corpus", tmp_path / "run3", train={"causal_omni": {"chunk": 2, "window": 2}}))
    try:
        with torch.no_grad():
            rt.optimizer.master.add_(0.02)
            rt.optimizer.live.copy_(rt.optimizer.master.to(rt.optimizer.live.dtype))
        rt.train_microbatch(0, 1)
        grads = [p.grad for p in rt.optimizer.params if p.grad is not None]
        assert grads and any(float(g.abs().sum()) > 0 for g in grads)
    finally:
        rt.close()


def test_render_command_from_media(tmp_path, capsys):
    import json

    import cv2
    import numpy as np

    from solarwm_b200.renderer.cli import main

    rng = np.random.default_rng(0)
    frames = rng.integers(0, 255, (30, 40, 60, 3), dtype=np.uint8)
    wr = cv2.VideoWriter(str(tmp_path / "structure.mp4"), cv2.VideoWriter_fourcc(*"mp4v"), 24.0, (60, 40))
    for f in frames:
        wr.write(f)
    wr.release()
    cv2.imwrite(str(tmp_path / "first.png"), frames[0])
    base = ["render", "--structure", str(tmp_path / "structure.mp4"), "--prompt", "a harbour at dusk", "--codecs", "tests.helpers.stub_codecs:factory",
            "--canvas", "32x48", "--device", "cpu", "--steps", "2"]
    assert main(base + ["--out", str(tmp_path / "a"), "--first-frame", str(tmp_path / "first.png")]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["pixel_frames"] == 22 and rec["latents"] == [24, 7, 4, 6] and rec["mode"] == "bidirectional" and rec["finite"]
    assert main(base + ["--out", str(tmp_path / "b"), "--causal", "--chunk", "3", "--window", "2"]) == 0
    assert json.loads((tmp_path / "b" / "render.json").read_text())["mode"] == "causal"
    assert torch.load(tmp_path / "b" / "latents.pt", weights_only=True).shape == (24, 7, 4, 6)
    with pytest.raises(SystemExit):
        main(["render", "--structure", str(tmp_path / "structure.mp4"), "--out", str(tmp_path / "c"), "--device", "cpu"])
