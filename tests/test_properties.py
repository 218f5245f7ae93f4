"""Property tests of the pure planning / geometry functions (hypothesis; small example budgets)."""
from types import SimpleNamespace

import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from solarwm_b200.backends.minimax_h3.geometry import align_pixel_frames, latent_pixel_indices, latent_to_pixel_frames, pixel_to_latent_frames
from solarwm_b200.backends.minimax_h3.validation import balanced_candidates, source_video_id
from solarwm_b200.renderer.causal import chunk_spans, document_rows, plan_mask, training_plan
from solarwm_b200.renderer.preencode import usable_frames
from solarwm_b200.serve.h3_source_length import full_length_geometry
from solarwm_b200.serve.memory_engine import check_selection, noise_window

FAST = settings(max_examples=60, deadline=None)


@FAST
@given(st.integers(1, 4000))
def test_frame_rules_round_trip(n):
    a = align_pixel_frames(n)
    assert a >= n and a - n < 17 and (a - 5) % 17 == 0
    lat = pixel_to_latent_frames(a)
    assert latent_to_pixel_frames(lat) == a
    idx = latent_pixel_indices(a)
    assert len(idx) == lat and idx[0] == 0 and idx[-1] < a and (np.diff(idx) >= 1).all() and (np.diff(idx) <= 4).all()
    u = usable_frames(n)
    assert u <= n and (u == 0) == (n < 22) and (u == 0 or (u - 5) % 17 == 0) and n - u < 17 + 22


@FAST
@given(st.integers(22, 3000))
def test_source_length_geometry(frames):
    g = full_length_geometry(frames)
    assert g.decoded_frames >= frames and g.decoded_frames - frames < 17
    assert g.rollout_latents % 5 == 0 and 0 <= g.rollout_latents - g.decode_latents < 5 and len(g.camera_indices) == g.rollout_latents
    cams = np.asarray(g.camera_indices)
    assert cams[0] == 0 and cams.max() < frames and (np.diff(cams) >= 0).all() and g.tail_camera_rows == int((np.diff(cams) == 0).sum())


@FAST
@given(st.integers(1, 40), st.integers(1, 9), st.integers(1, 6), st.booleans(), st.booleans())
def test_causal_plan_never_looks_ahead_and_covers_every_row(frames, chunk, window, structure, clean_copy):
    spans = chunk_spans(frames, chunk)
    assert spans[0][0] == 0 and spans[-1][1] == frames and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    rows = document_rows(3, [2 * (b - a) for a, b in spans], structure=structure, clean_copy=clean_copy)
    plan = training_plan(rows, window)
    m = plan_mask(plan, rows.total)
    assert m.any(dim=1).all() and m.diagonal().all()                  # every row attends something, at least itself
    order = {}                                                        # chunk index of every non-static row
    for kind in (rows.structure, rows.clean, rows.noisy):
        for j, (a, b) in enumerate(kind):
            for r in range(a, b):
                order[r] = j
    qs, ks = torch.nonzero(m, as_tuple=True)
    for q, k in zip(qs.tolist(), ks.tolist()):
        if q in order and k in order:
            assert order[k] <= order[q] and order[q] - order[k] < window
        if q < 3:
            assert k < 3                                              # static rows see static rows only


@FAST
@given(st.integers(2, 5), st.integers(2, 6), st.integers(0, 10 ** 6))
def test_validation_slots_never_share_a_source_video(datasets, videos, seed):
    rows = [SimpleNamespace(sample_id=f"d{d}/v{v}/h3-158f-occ-{w:02d}", values={}) for d in range(datasets) for v in range(videos) for w in range(2)]
    count = datasets * min(videos, 3)
    slots = balanced_candidates(rows, sample_count=count, seed=seed)
    firsts = [source_video_id(c[0].sample_id) for c in slots]
    everything = [source_video_id(r.sample_id) for c in slots for r in c]
    assert len(set(firsts)) == len(firsts) and len(set(everything)) == len(everything)
    per = {}
    for f in firsts:
        per[f.split("/")[0]] = per.get(f.split("/")[0], 0) + 1
    assert max(per.values()) - min(per.values()) <= 1                 # balanced over the datasets


@FAST
@given(st.integers(0, 400))
def test_noise_window_walks_ten_chunk_buffers(index):
    offset, refill = noise_window(index)
    assert 0 <= offset < (58 if index < 58 else 10) and refill == (index >= 58 and (index - 58) % 10 == 0)
    stop = max(0, index - 5) * 5
    ids = list(range(min(5, stop)))
    check_selection({"chunk": index, "memory_latent_indices": ids, "cached_chunks": min(index, 5)})
