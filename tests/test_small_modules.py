"""Direct tests of small host-side modules: shard prefetch, fp32-master AdamW, text encoder, environment probe,
frame sink."""
import threading
import time
from types import SimpleNamespace

import pytest
import torch


def test_prefetcher_keeps_lookahead_shards_in_flight_and_preserves_order():
    from solarwm_b200.data.prefetch import ShardPrefetcher, warm_cache

    calls, lock = [], threading.Lock()

    class Resolver:
        def resolve(self, shard, size=None):
            with lock:
                calls.append(shard)
            time.sleep(0.01)
            return f"/local/{shard}"

    plans = [SimpleNamespace(shard=f"s{i // 3}", i=i) for i in range(15)]          # 5 shards, 3 samples each
    pf = ShardPrefetcher(Resolver(), lookahead=2, max_workers=2)
    out = list(pf.iterate(plans))
    pf.close()
    assert [p.i for p, _ in out] == list(range(15)) and all(path == f"/local/{p.shard}" for p, path in out)
    assert sorted(set(calls)) == [f"s{i}" for i in range(5)] and len(calls) == 5     # every shard resolved once
    rows = [SimpleNamespace(shard=f"s{i % 3}", values={"shard_size": 10 + i % 3}) for i in range(9)]
    calls.clear()
    done = warm_cache(Resolver(), rows)
    assert (done.shards, done.bytes) == (3, 10 + 11 + 12) and sorted(calls) == ["s0", "s1", "s2"]


def test_fp32_master_adamw_matches_torch_adamw_and_refuses_casting_loads():
    from solarwm_b200.engine.master_adamw import FP32MasterAdamW

    torch.manual_seed(0)
    a, b = torch.nn.Parameter(torch.randn(7, 5)), torch.nn.Parameter(torch.randn(11))
    ra, rb = torch.nn.Parameter(a.detach().clone()), torch.nn.Parameter(b.detach().clone())
    frozen = torch.nn.Parameter(torch.randn(3), requires_grad=False)
    ours = FP32MasterAdamW([a, b, frozen], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ref = torch.optim.AdamW([ra, rb], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(4):
        ga, gb = torch.randn(7, 5) * 0.1, torch.randn(11) * 0.1
        a.grad, b.grad, ra.grad, rb.grad = ga.clone(), gb.clone(), ga.clone(), gb.clone()
        ours.gather_grads()
        norm = ours.clip_(None)
        assert torch.allclose(norm, torch.sqrt(ga.pow(2).sum() + gb.pow(2).sum()), rtol=1e-5)
        ours.step()
        ours.zero_grad()
        ref.step()
    assert a.grad is None and torch.allclose(a, ra, atol=1e-6) and torch.allclose(b, rb, atol=1e-6)
    # clipping scales the step; a non-finite gradient skips it
    before = a.detach().clone()
    a.grad, b.grad = torch.full((7, 5), float("nan")), torch.zeros(11)
    ours.gather_grads()
    ours.clip_(1.0)
    ours.step()
    assert torch.equal(a, before)
    state = ours.state_dict()
    other = FP32MasterAdamW([torch.nn.Parameter(torch.zeros(7, 5)), torch.nn.Parameter(torch.zeros(11))], lr=1e-2)
    other.load_state_dict(state)
    assert other.step_count == ours.step_count and torch.equal(other.master, ours.master)
    state["master"] = state["master"].double()
    with pytest.raises(ValueError, match="casting"):
        other.load_state_dict(state)
    with pytest.raises(ValueError):
        FP32MasterAdamW([frozen])


def test_text_encoder_is_deterministic_masks_padding_and_keeps_the_contract_shape():
    from solarwm_b200.models.t5 import HashTokenizer, T5Config, WanTextEncoder

    cfg = T5Config.tiny()
    enc = WanTextEncoder(cfg, device="cpu", dtype=torch.float32, seed=0)
    out = enc(["a red bicycle", "a red bicycle", "something much longer than the first prompt, with more words in it"])
    assert out.shape == (3, cfg.text_len, cfg.dim) and torch.equal(out[0], out[1]) and not torch.equal(out[0], out[2])
    ids, mask = HashTokenizer(cfg.vocab, cfg.text_len)(["two words"])
    assert ids.shape == (1, cfg.text_len) and int(mask.sum()) < cfg.text_len
    n = int(mask[0].sum())
    assert float(out[0, int(HashTokenizer(cfg.vocab, cfg.text_len)(["a red bicycle"])[1][0].sum()):].abs().sum()) == 0.0   # padding rows are zero
    assert n >= 2
    again = WanTextEncoder(cfg, device="cpu", dtype=torch.float32, seed=0)(["a red bicycle"])
    assert torch.equal(again[0], out[0])


def test_environment_probe_reports_versions():
    from solarwm_b200.runtime.env_probe import probe_python_runtime

    info = probe_python_runtime()
    assert info["packages"]["torch"] == torch.__version__ and "python" in info
    assert info["cuda_available"] == torch.cuda.is_available() and "native_library" in info


def test_frame_sink_writes_raw_rgb_and_checks_geometry(tmp_path):
    from solarwm_b200.serve.media import FragmentStore, FrameSink

    sink = FrameSink(tmp_path, width=8, height=6, use_ffmpeg=False)
    sink.push(torch.rand(3, 6, 8).to(torch.bfloat16))
    sink.push(torch.rand(3, 6, 8).to(torch.bfloat16))
    with pytest.raises(ValueError):
        sink.push(torch.rand(3, 5, 8).to(torch.bfloat16))
    with pytest.raises(FloatingPointError):
        sink.push(torch.full((3, 6, 8), float("nan")).to(torch.bfloat16))
    report = sink.close()
    assert report["frames"] == 2 and (tmp_path / "video.rgb").stat().st_size == 2 * 6 * 8 * 3
    store = FragmentStore(keep=2)
    ids = [store.add(bytes([i])) for i in range(3)]
    assert ids == [0, 1, 2] and [i for i, _ in store.since(0)] == [1, 2]


def test_frame_sink_normalization_maps_signed_unit_frames_to_full_range(tmp_path):
    import numpy as np

    from solarwm_b200.serve.media import SIGNED_UNIT, FrameSink, frame_to_rgb8

    frame = torch.stack([torch.full((4, 4), -1.0), torch.zeros(4, 4), torch.ones(4, 4)])
    rgb = frame_to_rgb8(frame, SIGNED_UNIT)
    assert rgb.shape == (4, 4, 3) and (rgb[..., 0] == 0).all() and (rgb[..., 2] == 255).all() and abs(int(rgb[0, 0, 1]) - 128) <= 1
    sink = FrameSink(tmp_path, 4, 4, use_ffmpeg=False, normalization=SIGNED_UNIT)
    sink.push(frame)
    sink.close()
    raw = np.frombuffer((tmp_path / "video.rgb").read_bytes(), np.uint8).reshape(4, 4, 3)
    assert np.array_equal(raw, rgb)
