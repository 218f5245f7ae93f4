"""H3 validation: source-balanced slots with reserves, frozen selection, seeded scoring, the runtime hook."""
import json
from types import SimpleNamespace

import pytest
import torch

from solarwm_b200.backends.minimax_h3.validation import IndexedValidation, balanced_candidates, score, source_video_id
from solarwm_b200.errors import DataContractError


def _rows():
    rows = []
    for ds, n in (("alpha", 4), ("beta", 3)):
        for v in range(n):
            for w in range(2):                                       # two windows per source video
                rows.append(SimpleNamespace(sample_id=f"{ds}/video{v}/h3-158f-occ-{w:02d}", values={}))
    rows.append(SimpleNamespace(sample_id="beta/loose", values={"source_sample_id": "beta/video0"}))
    return rows


def test_slots_are_balanced_disjoint_and_have_reserves():
    assert source_video_id("a/b/h3-158f-occ-03") == "a/b" and source_video_id("x", {"source_sample_id": "s"}) == "s"
    slots = balanced_candidates(_rows(), sample_count=4, seed=1)
    firsts = [c[0].sample_id for c in slots]
    assert [f.split("/")[0] for f in firsts] == ["alpha", "beta", "alpha", "beta"]
    videos = [source_video_id(c.sample_id, c.values) for cs in slots for c in cs]
    assert len(videos) == len(set(videos)) == 7                       # every source video appears once, as a choice or a reserve
    assert [len(c) for c in slots] == [2, 2, 2, 1]
    assert slots == balanced_candidates(_rows(), sample_count=4, seed=1) != balanced_candidates(_rows(), sample_count=4, seed=2)
    assert len(balanced_candidates(_rows(), sample_count=3, seed=1, balance=False)) == 3
    with pytest.raises(DataContractError):
        balanced_candidates(_rows(), sample_count=1, seed=1)          # fewer slots than datasets
    with pytest.raises(DataContractError):
        balanced_candidates(_rows(), sample_count=9, seed=1)          # beta has 3 source videos for a quota of 4


def test_unreadable_first_choice_falls_back_and_the_selection_is_frozen(tmp_path):
    rows = _rows()
    slots = balanced_candidates(rows, sample_count=4, seed=1)
    broken = {slots[0][0].sample_id}
    reads = []

    def read(row):
        reads.append(row.sample_id)
        if row.sample_id in broken:
            raise DataContractError("camera filter")
        return {"x": torch.full((2,), float(len(row.sample_id)))}

    v = IndexedValidation(rows, read, sample_count=4, seed=1, freeze_path=tmp_path / "sel.json")
    chosen = v.prepare()
    assert chosen[0] == slots[0][1].sample_id and chosen[1] == slots[1][0].sample_id
    frozen = json.loads((tmp_path / "sel.json").read_text())
    assert frozen["selected"]["0"] == chosen[0] and frozen["slots"] == 4
    # later the broken clip became readable: the frozen choice still stands, and only the chosen clips are read
    broken.clear()
    reads.clear()
    again = IndexedValidation(rows, read, sample_count=4, seed=1, freeze_path=tmp_path / "sel.json")
    assert again.prepare() == chosen and sorted(reads) == sorted(chosen.values())
    with pytest.raises(DataContractError):
        IndexedValidation(rows, read, sample_count=4, seed=2, freeze_path=tmp_path / "sel.json").prepare()
    broken.update(c.sample_id for c in slots[3])                      # a slot without any usable clip
    with pytest.raises(DataContractError):
        IndexedValidation(rows, read, sample_count=4, seed=1).prepare()
    # two replicas split the slots; five slots round down to two whole waves
    broken.clear()
    r1 = IndexedValidation(rows, read, sample_count=5, seed=1, dp_rank=1, dp_size=2)
    assert r1.count == 4 and r1.my_slots == [1, 3]
    with pytest.raises(DataContractError):
        IndexedValidation(rows, read, sample_count=1, seed=1, dp_rank=0, dp_size=2)


def test_scoring_is_a_pure_function_of_the_weights():
    rows = _rows()
    v = IndexedValidation(rows, lambda row: {"x": torch.full((4,), float(len(row.sample_id)))}, sample_count=2, seed=3)
    v.prepare()
    weight = torch.tensor(2.0)

    def loss_at(sample, t, gen):
        noise = torch.randn(4, generator=gen)
        return ((weight * sample["x"] * t + noise) ** 2).mean()

    a, b = score(v, loss_at, device=torch.device("cpu")), score(v, loss_at, device=torch.device("cpu"))
    assert a == b and a["clips"] == 2 and set(a) >= {"loss", "loss_t0.25", "loss_t0.5", "loss_t0.75", "selected"}
    assert a["loss_t0.75"] > a["loss_t0.25"]
    weight = torch.tensor(3.0)
    assert score(v, loss_at, device=torch.device("cpu"))["loss"] > a["loss"]
    with pytest.raises(FloatingPointError):
        score(v, lambda s, t, g: torch.tensor(float("nan")), device=torch.device("cpu"))


def test_runtime_validates_on_its_frozen_clips(tmp_path):
    from solarwm_b200.backends.minimax_h3.runtime import H3TrainingRuntime
    from solarwm_b200.registry import load_backend

    be = load_backend("minimax_h3")
    pre = {"data": {"pixel_frames": 9, "pixel_height": 64, "pixel_width": 64, "seed": 1}, "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 4, "output_root": str(tmp_path / "enc"),
                         "codecs": {"vae_base": 4, "t5": {"vocab": 512, "dim": 64, "dim_attn": 32, "dim_ffn": 64, "num_heads": 2,
                                                         "num_layers": 1, "text_len": 8}}}}
    assert be.preencode(pre)["samples"] == 4
    config = {"schema": "solarwm.run.v1", "action": "train",
              "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
              "data": {"source": "index", "index": str(tmp_path / "enc" / "index.jsonl"), "seed": 0, "pixel_frames": 158},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 2, "optimizer": {"lr": 1e-2}},
              "validation": {"index": str(tmp_path / "enc" / "index.jsonl"), "sample_count": 2, "seed": 5, "balance_sources": False},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")}}
    rt = H3TrainingRuntime(config, model_config=be._cfg(config))
    try:
        first = rt.validate(0)["validation"]
        assert first["clips"] == 2 and first["loss"] > 0 and (tmp_path / "run" / "validation-selection.json").is_file()
        assert rt.validate(0)["validation"] == first                   # same weights, same number
        with torch.no_grad():                                           # LoRA B starts at zero: move the adapters
            rt.optimizer.master.add_(0.05)
            rt.optimizer.live.copy_(rt.optimizer.master.to(rt.optimizer.live.dtype))
        moved = rt.validate(1)["validation"]
        assert moved["selected"] == first["selected"] and moved["loss"] != first["loss"]
    finally:
        rt.close()


def test_inference_uses_the_trained_adapters_of_a_checkpoint(tmp_path):
    from solarwm_b200.registry import load_backend

    be = load_backend("minimax_h3")
    train = {"schema": "solarwm.run.v1", "action": "train",
             "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
             "data": {"source": "synthetic", "seed": 3, "pixel_frames": 158, "latent_frames": 3, "latent_height": 8, "latent_width": 8},
             "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 6,
                       "optimizer": {"lr": 2e-2}, "ema": {"decay": 0.5}},
             "runtime": {"device": "cpu", "output_dir": str(tmp_path / "train")}}
    out = be.train(train)
    infer = {"schema": "solarwm.run.v1", "action": "infer", "model": train["model"], "data": {"seed": 3},
             "inference": {"source": "synthetic", "grid_hw": [2, 2], "chunk_latents": 2, "chunks": 1, "denoise_steps": 1, "seed": 1}}
    runs = {}
    for name, ck in (("base", {}), ("live", {"resume_from": out["checkpoint"], "weight_source": "live"}),
                     ("ema", {"resume_from": out["checkpoint"]})):
        model, weights_id = be._inference_model({**infer, "checkpoint": ck}, "cpu")
        runs[name] = (weights_id, {n: p.detach().clone() for n, p in model.named_parameters() if n.endswith("q.weight") or ".q." in n})
        assert not any(p.requires_grad for p in model.parameters()) or name == "base"
        r = be.infer({**infer, "checkpoint": ck, "runtime": {"device": "cpu", "output_dir": str(tmp_path / name)}})
        assert r["chunks"] == 1 and r["weights_id"] == weights_id
    assert runs["base"][0] == "init:random" and runs["live"][0].endswith(":live") and runs["ema"][0].endswith(":ema")
    import pytest as _pytest
    from solarwm_b200.errors import BackendContractError

    with _pytest.raises(BackendContractError):
        be._inference_model({**infer, "checkpoint": {"resume_from": out["checkpoint"], "weight_source": "other"}}, "cpu")
