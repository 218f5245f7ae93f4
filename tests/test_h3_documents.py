"""Packed H3 documents: anchors, free and aligned observations, audio, the duplicated Stage-1 clip."""
import numpy as np
import pytest

from solarwm_b200.backends.minimax_h3 import documents as doc
from solarwm_b200.backends.minimax_h3.layout import build_layout, temporal_positions


def test_plain_document_matches_the_trainer_layout_rules():
    d = doc.stage0p5_document([1] * 6, 4, (2, 3))
    assert d.sequence_length == 6 + 6 + 4 * 6 and d.stage == "stage0p5"
    assert list(d.text_indices) == list(range(6)) and list(d.condition_video_indices) == list(range(6, 12))
    assert d.target_video_output_slice == slice(6, 30)
    # text clock, the anchor at the first frame's time, the clip on the non-uniform grid starting at the text length
    assert np.array_equal(d.position_ids[:6, 0], np.arange(6)) and np.all(d.position_ids[6:12, 0] == 6.0)
    assert np.allclose(d.position_ids[d.noisy_video_indices, 0].reshape(4, 6)[:, 0], temporal_positions(4, 6.0))
    ref = build_layout(n_text=6, latent_frames=4, grid_hw=(2, 3))             # same spatial grid as the trainer layout
    assert np.allclose(d.position_ids[6:12, 1:], ref.position_ids[6:12, 1:].numpy())
    assert list(d.camera_frame[6:12]) == [0] * 6 and list(d.camera_frame[-6:]) == [3] * 6 and np.all(d.camera_frame[:6] == -1)
    cams = np.stack([np.eye(4) * (i + 1) for i in range(4)])
    rows = d.camera_rows(cams)
    assert rows.shape == (36, 4, 4) and rows[0, 0, 0] == 1.0 and rows[12, 0, 0] == 1.0 and rows[-1, 0, 0] == 4.0
    last = doc.stage0p5_document([1] * 6, 4, (2, 3), anchors=("first", "last"))
    t_last = temporal_positions(5, 6.0)[-1] - 5.0 / 3.0
    assert np.allclose(last.position_ids[12:18, 0], t_last) and list(last.camera_frame[12:18]) == [3] * 6
    with pytest.raises(ValueError):
        doc.stage0p5_document([1], 4, (2, 3), anchors=("middle",))


def test_observations_free_ones_use_the_clock_aligned_ones_the_canvas():
    free1 = doc.Observation(frames=1, height=2, width=2)
    free3 = doc.Observation(frames=3, height=1, width=2)
    aligned = doc.Observation(frames=2, height=1, width=1, at=(1, 3), boxes=((0.0, 0.0, 0.5, 0.5), (0.5, 0.5, 1.0, 1.0)))
    d = doc.stage0p5_document([1] * 4, 4, (2, 2), observations=(free1, free3, aligned), audio_latents=3)
    assert d.observation_rows == (4, 6, 2) and len(d.observation_indices) == 12
    ob = d.position_ids[d.observation_indices]
    assert np.all(ob[:4, 0] == 4.0)                                            # one slot on the clock
    assert np.allclose(ob[4:10, 0].reshape(3, 2)[:, 0], temporal_positions(3, 5.0))
    origin = 5.0 + float(np.diff(temporal_positions(4, 0.0)).sum())            # what the free observations used
    clip = d.position_ids[d.noisy_video_indices, 0].reshape(4, 4)[:, 0]
    assert np.allclose(clip, temporal_positions(4, origin))
    assert np.allclose(ob[10:, 0], clip[[1, 3]])                               # aligned: their frames' times
    assert list(d.camera_frame[d.observation_indices]) == [-1] * 10 + [1, 3]   # ... and their frames' cameras
    # a 1 x 1 observation over the upper-left / lower-right quarter of a square canvas sits at 0 and 16
    assert np.allclose(ob[10, 1:], [0.0, 0.0]) and np.allclose(ob[11, 1:], [16.0, 16.0])
    audio = d.position_ids[d.audio_indices]
    assert audio.shape == (6, 3) and np.allclose(audio[:3, 0], origin + np.arange(3)) and audio[0, 2] != audio[3, 2]
    for bad in (doc.Observation(1, 1, 1, at=(4,)), doc.Observation(2, 1, 1, at=(0,)), doc.Observation(1, 1, 1, boxes=((0, 0, 1, 1),)),
                doc.Observation(1, 1, 1, at=(0,), boxes=((0.2, 0.2, 0.1, 0.9),))):
        with pytest.raises(ValueError):
            doc.stage0p5_document([1], 4, (2, 2), observations=(bad,))


def test_stage1_document_holds_the_clip_twice_with_identical_structure():
    d = doc.stage1_document([1, 1, 0], 10, (2, 2), chunk_latent_frames=5, window_chunks=6)
    c, n = d.clean_video_indices, d.noisy_video_indices
    assert len(c) == len(n) == 40 and c[-1] + 1 == n[0] and d.stage == "stage1" and d.window_chunks == 6
    assert np.array_equal(d.position_ids[c], d.position_ids[n]) and np.array_equal(d.chunk_ids[c], d.chunk_ids[n])
    assert np.array_equal(d.camera_frame[c], d.camera_frame[n]) and list(np.unique(d.chunk_ids[n])) == [0, 1]
    assert np.all(d.roles[c] == doc.ROLE_CLEAN) and np.all(d.roles[n] == doc.ROLE_NOISY) and np.all(d.chunk_ids[:7] == -1)
    assert d.target_video_output_slice == slice(4 + 40, 4 + 80)
    t = d.to_layout_tensors()
    assert t["position_ids"].shape == (3 + 4 + 80, 3) and int(t["tags"][0]) == 1
    with pytest.raises(ValueError):
        doc.stage1_document([1], 7, (2, 2), chunk_latent_frames=5)
