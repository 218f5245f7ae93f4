"""Interactive memory sessions: camera packets at the latent cadence, absolute cameras, retrieval invariants, the noise
schedule, sticky failure, session reports."""
import json

import numpy as np
import pytest
import torch

from solarwm_b200.models.h3 import H3DiT, h3_preset
from solarwm_b200.serve.h3_stream import H3StreamConfig
from solarwm_b200.serve.memory_engine import MemorySessionEngine, cache_key, check_selection, noise_window


def test_noise_window_and_selection_invariants():
    assert [noise_window(i) for i in (0, 7, 57)] == [(0, False), (7, False), (57, False)]
    assert noise_window(58) == (0, True) and noise_window(59) == (1, False) and noise_window(68) == (0, True)
    with pytest.raises(ValueError):
        noise_window(-1)
    check_selection({"chunk": 3, "memory_latent_indices": [], "cached_chunks": 3})
    check_selection({"chunk": 7, "memory_latent_indices": [0, 9, 3, 4, 5], "cached_chunks": 5})
    for bad in ({"chunk": 7, "memory_latent_indices": [0, 9, 3, 4], "cached_chunks": 5},            # too few
                {"chunk": 7, "memory_latent_indices": [0, 0, 3, 4, 5], "cached_chunks": 5},         # repeated
                {"chunk": 7, "memory_latent_indices": [0, 10, 3, 4, 5], "cached_chunks": 5},        # inside the recent window
                {"chunk": 7, "memory_latent_indices": [0, 9, 3, 4, 5], "cached_chunks": 6}):
        with pytest.raises(RuntimeError):
            check_selection(bad)
    a = cache_key(sources_sha256="x", runtime={"sp": 8}, inference={"top_k": 5})
    assert a == cache_key(sources_sha256="x", runtime={"sp": 8}, inference={"top_k": 5}) != cache_key(sources_sha256="y", runtime={"sp": 8}, inference={"top_k": 5})


def _engine(tmp_path, **kw):
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=5, window_chunks=2, denoise_steps=1, use_cuda_graph=False, memory_latents=2)
    eng = MemorySessionEngine(model, scfg, run_dir=tmp_path, top_k=2, identity={"adapter": "unit"}, **kw)
    eng.set_condition(text=torch.randn(6, cfg.text_dim), anchor_latent=torch.randn(24, 1, 4, 6), scene_id="scene-1")
    return eng


def test_session_walks_out_and_back_and_retrieves_old_latents(tmp_path):
    eng = _engine(tmp_path)
    with pytest.raises(RuntimeError):
        eng.generate()                                              # no session
    eng.start(seed=7)
    with pytest.raises(ValueError):
        eng.advance_camera([["w"]] * 5)                             # the first chunk takes 4 packets
    chunks = []
    for j in range(6):
        keys = ["w"] if j < 3 else ["s"]                            # walk forward, then back over the same ground
        eng.advance_camera([keys] * (4 if j == 0 else 5))
        with pytest.raises(ValueError):
            eng.advance_camera([keys] * 5)                          # one packet per chunk
        chunk, ms = eng.generate()
        chunks.append(chunk)
        assert chunk.shape == (24, 5, 4, 6) and ms > 0
    # poses: one per latent at the 1, 4, 4, 4, 4 cadence, absolute in the first camera's frame
    assert len(eng.poses) == 30 and np.allclose(eng.poses[0], np.eye(4))
    z = [p[2, 3] for p in eng.poses]
    assert z[1] > 0 and (z[2] - z[1]) > 2.5 * (z[1] - z[0]) * 0.5 and max(z) == pytest.approx(z[14], abs=0.2) and z[-1] < z[14]
    assert eng.views.shape[0] >= 30 and torch.allclose(eng.views[0], torch.eye(4))
    assert torch.allclose(eng.views[14, 2, 3], torch.tensor(-z[14], dtype=torch.float32), atol=1e-5)       # world-to-camera
    recs = eng.records
    assert [len(r["memory_latent_indices"]) for r in recs] == [0, 0, 0, 2, 2, 2]
    assert all(i < 5 for i in recs[3]["memory_latent_indices"]) and all(i < 15 for i in recs[5]["memory_latent_indices"])
    assert all(r["cached_chunks"] <= 2 for r in recs)
    report = eng.stop()
    assert report["chunks"] == 6 and report["scene_id"] == "scene-1" and report["memory"] == {"adapter": "unit"}
    saved = json.loads((tmp_path / "memory-session-1-rank0.json").read_text())
    assert saved["retrieval"][5]["memory_latent_indices"] == recs[5]["memory_latent_indices"]
    assert eng.poses == [] and eng.gen is None
    # a second session of the same engine: same seed, same cameras -> the same chunks; its report has its own file
    eng.start(seed=7)
    eng.advance_camera([["w"]] * 4)
    again, _ = eng.generate()
    assert torch.equal(again, chunks[0])
    eng.stop()
    assert (tmp_path / "memory-session-2-rank0.json").is_file()
    with pytest.raises(RuntimeError):
        eng.stop()


def test_failure_is_sticky(tmp_path):
    eng = _engine(tmp_path)
    eng.start()
    eng.advance_camera([[]] * 4)
    real = eng.gen.next_chunk
    eng.gen.next_chunk = lambda views: torch.full((24, 5, 4, 6), float("nan"))
    with pytest.raises(FloatingPointError):
        eng.generate()
    eng.gen.next_chunk = real
    assert eng.failed
    with pytest.raises(RuntimeError):
        eng.generate()
    eng.close()
    with pytest.raises(RuntimeError):
        eng.start()
    with pytest.raises(ValueError):
        MemorySessionEngine(eng.model, H3StreamConfig(grid_hw=(2, 3), memory_latents=1), run_dir=tmp_path, top_k=5)


def test_memory_bank_attaches_beside_merged_generation_adapters(tmp_path):
    from solarwm_b200.serve.memory import adapter_digest, attach_memory_adapter

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with pytest.raises(ValueError):
        attach_memory_adapter(model, rank=4)                        # trainable generation adapters: not a frozen parent
    from solarwm_b200.models.h3 import LoRALinear

    with torch.no_grad():
        for m in model.modules():
            if isinstance(m, LoRALinear):
                m.lora_B.normal_(0, 0.02)
                m.merge_()
                m.rank = 0
    ident = attach_memory_adapter(model, rank=4, frozen_identity="stage2:ema:step=12")
    assert ident["memory_adapter"] == "fresh-zero" and ident["parameter_count"] > 0 and ident["frozen_adapter"].startswith("stage2")
    assert not any(p.requires_grad for p in model.parameters())
    with pytest.raises(ValueError):
        attach_memory_adapter(model, rank=4)                        # already attached
    # a trained bank loads strictly and is identified by its digest
    state = {k: torch.randn_like(v) * 0.01 for k, v in model.named_parameters() if k.endswith("__memory")}
    fresh = H3DiT(h3_preset("tiny"), device="cpu", dtype=torch.float32, seed=0)
    got = attach_memory_adapter(fresh, rank=4, memory_state=state)
    assert got["memory_adapter"] == adapter_digest(state) and got["tensors"] == len(state)
    other = H3DiT(h3_preset("tiny"), device="cpu", dtype=torch.float32, seed=0)
    with pytest.raises(ValueError):
        attach_memory_adapter(other, rank=4, memory_state={k: v for k, v in list(state.items())[:-1]})
    # the engine runs with the bank switched on while memory rows are installed
    scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=5, window_chunks=2, denoise_steps=1, use_cuda_graph=False, memory_latents=2,
                          memory_adapter="memory")
    eng = MemorySessionEngine(fresh, scfg, run_dir=tmp_path, top_k=2, identity=got)
    eng.set_condition(text=torch.randn(6, fresh.cfg.text_dim), anchor_latent=torch.randn(24, 1, 4, 6), scene_id="s")
    eng.start()
    for j in range(4):
        eng.advance_camera([["w"]] * (4 if j == 0 else 5))
        eng.generate()
    assert eng.stop()["memory"]["memory_adapter"] == got["memory_adapter"]


def test_worker_runs_the_memory_family(tmp_path, capsys):
    import json

    from solarwm_b200.serve.worker import main

    assert main(["--smoke", "--family", "memory", "--height", "4", "--width", "6", "--chunks", "7", "--window-frames", "10",
                 "--output", str(tmp_path)]) == 0
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["family"] == "memory" and line["retrieved"] == [0, 0, 0, 5, 5, 5, 5]
    assert (tmp_path / "memory-session-1-rank0.json").is_file() and (tmp_path / "exit-rank0.json").is_file()
