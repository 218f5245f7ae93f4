"""Structured masks: the run description, its dense form, the tile tables and the CPU oracle against the per-chunk
loops that the models used to run."""
import torch

from solarwm_b200.backends.minimax_h3.stage1 import w6_mask
from solarwm_b200.models.wan_causal import teacher_forcing_attention, teacher_forcing_mask
from solarwm_b200.ops import attention_mask as am


def test_masks_equal_the_dense_oracles():
    tf = am.teacher_forcing_segment_mask(L=7 * 6, chunk=2 * 6, window_chunks=2, sink=6, prefix=0)
    want = teacher_forcing_mask(7, 6, 2, 2, sink_frames=1)
    assert torch.equal(tf.dense(), want)
    w6 = am.teacher_forcing_segment_mask(L=4 * 10, chunk=10, window_chunks=2, sink=0, prefix=13)
    assert torch.equal(w6.dense(), w6_mask(13, 10, 4, 2))
    bc = am.block_causal_mask(50, 8, 1, sink=3)
    d = bc.dense()
    assert d[0:8, 0:8].all() and not d[0:8, 8:].any()
    assert d[24:32, 16:32].all() and d[24:32, 0:3].all() and not d[24:32, 3:16].any() and not d[24:32, 32:].any()
    assert 0.0 < w6.density() < 1.0


def test_tile_tables_cover_exactly_the_visible_tiles_and_flag_partial_ones():
    m = am.teacher_forcing_segment_mask(L=600, chunk=200, window_chunks=1, sink=0, prefix=100)       # S = 1300
    dense = m.dense()
    for lists, qb, kt in ((m._tiles_over_keys(256, 128), 256, 128), (m._tiles_over_keys(128, 64), 128, 64)):
        for b, entries in enumerate(lists):
            rows = dense[b * qb:(b + 1) * qb]
            seen = {e & (am.PARTIAL - 1) for e in entries}
            for t in range(-(-m.Sk // kt)):
                block = rows[:, t * kt:(t + 1) * kt]
                assert (t in seen) == bool(block.any()), (b, t)
                if t in seen:
                    partial = any(e == (t | am.PARTIAL) for e in entries)
                    assert partial == (not bool(block.all())), (b, t)
    for b, entries in enumerate(m._tiles_over_queries(128, 64)):
        cols = dense[:, b * 128:(b + 1) * 128]
        for e in entries:
            t = e & (am.PARTIAL - 1)
            block = cols[t * 64:(t + 1) * 64]
            assert block.any() and bool(e & am.PARTIAL) == (not bool(block.all()))
        seen = {e & (am.PARTIAL - 1) for e in entries}
        for t in range(-(-m.Sq // 64)):
            assert (t in seen) == bool(cols[t * 64:(t + 1) * 64].any())
    rr = m.row_ranges()
    assert rr.shape == (1300, 6) and (rr[:100, :2] == [0, 100]).all() and (rr[:100, 2:] == 0).all()


def test_cpu_masked_attention_equals_the_chunk_loop():
    torch.manual_seed(0)
    F, ft, H, D = 5, 4, 2, 16
    L = F * ft
    q, k, v = (torch.randn(1, 2 * L, H, D) for _ in range(3))
    mask = am.teacher_forcing_segment_mask(L, 2 * ft, 1, sink=ft, prefix=0)
    got = am.masked_attention(q, k, v, mask)
    oc, on = teacher_forcing_attention(q[:, :L], k[:, :L], v[:, :L], q[:, L:], k[:, L:], v[:, L:], frame_tokens=ft,
                                       chunk_frames=2, window_chunks=1, sink_frames=1)
    assert torch.allclose(got, torch.cat([oc, on], 1), atol=1e-5)


def test_invalid_runs_are_refused():
    import pytest

    with pytest.raises(ValueError):
        am.SegmentMask(10, 10, [am.Run(0, 5, ((0, 5),))])                    # rows 5..9 uncovered
    with pytest.raises(ValueError):
        am.SegmentMask(4, 4, [am.Run(0, 4, ())])                             # sees nothing
    with pytest.raises(ValueError):
        am.SegmentMask(4, 20, [am.Run(0, 4, ((0, 1), (2, 3), (4, 5), (6, 7)))])   # four disjoint ranges
