"""Renderer pre-encoding: frame rules, media fitting, known-degree pooling, resumable shards, and the corpus it writes
is the corpus the training reader takes."""
import json

import numpy as np
import pytest
import torch

from solarwm_b200.errors import DataContractError
from solarwm_b200.renderer.data import MemberContract, OmniStream
from solarwm_b200.renderer.preencode import (Codecs, FetchFailed, fit, known_degrees, latent_frames, member_name, merge_indexes,
                                             on_grid, read_media, region, run_shard, usable_frames)


def test_frame_rules_and_media_fitting():
    assert [usable_frames(n) for n in (10, 22, 38, 39, 100)] == [0, 22, 22, 39, 90]
    assert latent_frames(22) == 7 and latent_frames(39) == 12
    with pytest.raises(DataContractError):
        latent_frames(23)
    frames = np.arange(30, dtype=np.uint8).reshape(30, 1, 1, 1).repeat(3, axis=3)
    assert on_grid(frames, 24.0) is frames
    g = on_grid(frames, 30.0)                                       # 30 fps -> every 1.25th source frame
    assert len(g) == 24 and g[:5, 0, 0, 0].tolist() == [0, 1, 2, 4, 5]
    wide = np.zeros((2, 40, 100, 3), dtype=np.uint8)
    wide[:, :, 40:60] = 255
    out = fit(wide, (16, 24))
    assert out.shape == (2, 16, 24, 3) and out[0, 8, 12, 0] > 200 and out[0, 8, 0, 0] < 50     # the centre survives the crop
    assert region(wide, [0.4, 0.0, 0.6, 1.0]).shape == (2, 40, 20, 3) and region(wide, None) is wide
    with pytest.raises(DataContractError):
        region(wide, [0.6, 0, 0.4, 1])
    mask = np.zeros((22, 16, 24, 3), dtype=np.uint8)
    mask[:, :, :12] = 255                                          # the left half is known
    k = known_degrees(mask, 7, (4, 6)).view(7, 4, 6)
    assert k.shape == (7, 4, 6) and torch.allclose(k[:, :, :3], torch.ones(7, 4, 3)) and float(k[:, :, 3:].max()) == 0.0
    with pytest.raises(FetchFailed):
        read_media("/nonexistent/clip.mp4")
    assert member_name("a/b c") != member_name("a_b_c") and member_name("x").endswith(".safetensors")


def _write_video(path, frames, fps=24.0):
    import cv2

    h, w = frames.shape[1:3]
    wr = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), fps, (w, h))
    assert wr.isOpened()
    for f in frames:
        wr.write(cv2.cvtColor(f, cv2.COLOR_RGB2BGR))
    wr.release()


def test_shards_encode_resume_and_feed_the_training_reader(tmp_path):
    import cv2

    rng = np.random.default_rng(0)
    media = tmp_path / "media"
    media.mkdir()
    for name, n in (("a.mp4", 24), ("b.mp4", 45), ("c.mp4", 24)):
        _write_video(media / name, rng.integers(0, 255, (n, 32, 48, 3), dtype=np.uint8))
    cv2.imwrite(str(media / "still.png"), rng.integers(0, 255, (32, 48, 3), dtype=np.uint8))
    mask = np.zeros((24, 32, 48, 3), dtype=np.uint8)
    mask[:, :, :24] = 255
    _write_video(media / "mask.mp4", mask)
    rows = [{"id": "clip/a", "target": "a.mp4", "text": "a street", "source": "unit",
             "observations": [{"media": "still.png", "frames": [0], "degree": 0.9}, {"media": "a.mp4", "frames": "all"},
                              {"media": "c.mp4", "frames": None, "box": [0.0, 0.0, 0.5, 1.0]}], "known_mask": "mask.mp4"},
            {"id": "clip/b", "target": "b.mp4", "text": "a hall"},
            {"id": "clip/late", "target": "not-there-yet.mp4", "text": "x"}]
    calls = {"video": 0}

    def video(frames):                                             # stand-in codec with the real geometry rules
        calls["video"] += 1
        T = frames.shape[0]
        return torch.from_numpy(frames[:, ::4, ::4].astype(np.float32).mean(-1) / 255.0)[:latent_frames(T)].unsqueeze(0).repeat(24, 1, 1, 1) \
            if (T - 5) % 17 == 0 else None

    codecs = Codecs(video=video, text=lambda s: (torch.full((5, 64), float(len(s))), torch.zeros(5)), canvas=(32, 48))
    first = run_shard(rows, out=tmp_path / "corpus", media_root=media, codecs=codecs)
    assert first["encoded"] == ["clip/a", "clip/b"] and first["pending"][0]["id"] == "clip/late" and not first["skipped"]
    n_calls = calls["video"]
    again = run_shard(rows, out=tmp_path / "corpus", media_root=media, codecs=codecs)
    assert again["skipped"] == ["clip/a", "clip/b"] and not again["encoded"] and calls["video"] == n_calls
    assert merge_indexes(tmp_path / "corpus") == 2
    index = [json.loads(l) for l in (tmp_path / "corpus" / "index.jsonl").read_text().splitlines()]
    assert [r["latent_frames"] for r in index] == [7, 12] and index[0]["observations"] == 3 and index[0]["pixel_frames"] == 22
    # the training reader takes what was written
    contract = MemberContract(latent_channels=24, text_dim=64, grids=((8, 12),))
    stream = OmniStream(root=tmp_path / "corpus", index=tmp_path / "corpus" / "index.jsonl", dp_rank=0, dp_size=1, seed=0,
                        shuffle=False, contract=contract)
    a, b = stream.next(), stream.next()
    assert a.sample_id == "clip/a" and a.target_latents.shape == (24, 7, 8, 12) and b.target_latents.shape[1] == 12
    still, aligned, free = a.observations
    assert still.frames == (0,) and still.degree == 0.9 and still.latents.shape[1] == 1
    assert aligned.frames == tuple(range(7)) and free.frames is None and free.boxes == ((0.0, 0.0, 0.5, 1.0),)
    k = a.known_degree.view(7, 4, 6)
    assert float(k[:, :, :3].min()) > 0.9 and float(k[:, :, 3:].max()) < 0.1 and a.source == "unit"
    # two shards split the rows and may not both claim a sample
    s0 = run_shard(rows[:2], out=tmp_path / "two", media_root=media, codecs=codecs, shard=0, shards=2)
    s1 = run_shard(rows[:2], out=tmp_path / "two", media_root=media, codecs=codecs, shard=1, shards=2)
    assert s0["encoded"] == ["clip/a"] and s1["encoded"] == ["clip/b"] and merge_indexes(tmp_path / "two") == 2
    with pytest.raises(DataContractError):
        run_shard(rows[:1] + rows[:1], out=tmp_path / "dup", media_root=media, codecs=codecs)
    with pytest.raises(DataContractError):                         # 10 frames: below the shortest clip
        _write_video(media / "short.mp4", rng.integers(0, 255, (10, 32, 48, 3), dtype=np.uint8))
        run_shard([{"id": "s", "target": "short.mp4", "text": ""}], out=tmp_path / "short", media_root=media, codecs=codecs)
