"""Pre-encode contracts, shard writer and the Wan preencode runner (CPU)."""
import pytest
import torch

from solarwm_b200.data.index import read_index
from solarwm_b200.errors import DataContractError
from solarwm_b200.preencode.contracts import EncoderContract, validate_encoded_tensors, wan_contract
from solarwm_b200.preencode.shards import EncodedShardWriter, read_encoded_sample


def _contract():
    return wan_contract("wan22_ti2v_5b", pixel_frames=9, height=64, width=64, z_dim=48, text_len=8, text_dim=16)


def test_contract_digest_roundtrip_and_validation():
    c = _contract()
    assert EncoderContract.from_dict(c.as_dict()).digest == c.digest
    good = {"latents": torch.zeros(3, 48, 4, 4).bfloat16(), "text": torch.zeros(8, 16).bfloat16()}
    validate_encoded_tensors(c, good)
    with pytest.raises(DataContractError):
        validate_encoded_tensors(c, {**good, "latents": torch.zeros(3, 48, 4, 5).bfloat16()})
    with pytest.raises(DataContractError):
        validate_encoded_tensors(c, {**good, "text": torch.zeros(8, 16)})
    bad = good["latents"].clone()
    bad[0, 0, 0, 0] = float("nan")
    with pytest.raises(DataContractError):
        validate_encoded_tensors(c, {**good, "latents": bad})
    with pytest.raises(DataContractError):
        validate_encoded_tensors(c, {"latents": good["latents"]})


def test_shard_writer_commit_last_and_readback(tmp_path):
    c = _contract()
    w = EncodedShardWriter(tmp_path, c, samples_per_shard=2)
    ref = {}
    for i in range(3):
        t = {"latents": torch.randn(3, 48, 4, 4).bfloat16(), "text": torch.randn(8, 16).bfloat16()}
        ref[f"s{i}"] = t
        w.add(f"s{i}", t, {"caption": f"c{i}"})
        assert not (tmp_path / "index.jsonl").exists()
    rows = read_index(w.finish())
    assert [r.shard for r in rows] == ["encoded-000000.tar", "encoded-000000.tar", "encoded-000001.tar"]
    for r in rows:
        got = read_encoded_sample(tmp_path, r.values, c)
        assert torch.equal(got["latents"], ref[r.sample_id]["latents"])
        assert torch.equal(got["text"], ref[r.sample_id]["text"])
    other = wan_contract("wan22_ti2v_5b", pixel_frames=13, height=64, width=64, z_dim=48, text_len=8, text_dim=16)
    with pytest.raises(DataContractError):
        read_encoded_sample(tmp_path, rows[0].values, other)
    with pytest.raises(DataContractError):           # published shards are never overwritten
        EncodedShardWriter(tmp_path, c, samples_per_shard=2).add("again", ref["s0"])


def test_wan_preencode_runner(tmp_path):
    from solarwm_b200.backends.wan22.preencode import run_preencode

    cfg = {"data": {"pixel_frames": 9, "pixel_height": 32, "pixel_width": 32, "seed": 3},
           "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 3, "output_root": str(tmp_path / "enc"),
                         "samples_per_shard": 2, "codecs": {"z_dim": 8, "vae_base": 8}}}
    out = run_preencode(cfg, "wan22_ti2v_5b")
    assert out["samples"] == 3
    rows = read_index(tmp_path / "enc" / "index.jsonl")
    c = EncoderContract.from_dict(__import__("json").loads((tmp_path / "enc" / "encoder-contract.json").read_text()))
    s = read_encoded_sample(tmp_path / "enc", rows[0].values, c)
    assert s["latents"].shape == (3, 8, 4, 4) and s["text"].shape == (8, 32)


def test_vae_streaming_decode_matches_full():
    from solarwm_b200.models.vae import StreamingDecoder, VAEConfig, VideoVAE

    torch.manual_seed(0)
    vae = VideoVAE(VAEConfig(z_dim=4, base=8)).eval()
    z = torch.randn(1, 4, 5, 4, 4)
    full = vae.decode(z)
    assert full.shape == (1, 3, 17, 32, 32)          # 1 + 4 * (5 - 1) frames, 8x spatial
    dec = StreamingDecoder(vae)
    parts = [dec.push(z[:, :, :1]), dec.push(z[:, :, 1:3]), dec.push(z[:, :, 3:])]
    assert torch.allclose(torch.cat(parts, dim=2), full, atol=1e-5)
    enc = vae.encode(torch.randn(1, 3, 17, 32, 32))
    assert enc.shape == (1, 4, 5, 4, 4)


def test_parameter_free_resample_shortcuts():
    from solarwm_b200.models.vae import AvgDown3D, DupUp3D

    x = torch.arange(2 * 4 * 4 * 4 * 4, dtype=torch.float32).view(2, 4, 4, 4, 4)
    down = AvgDown3D(4, 8, factor_t=2, factor_s=2)(x)
    assert down.shape == (2, 8, 2, 2, 2)
    assert torch.allclose(down.mean(), x.mean())                       # averaging preserves the mean
    up = DupUp3D(8, 4, factor_t=2, factor_s=2)(down)
    assert up.shape == (2, 4, 4, 4, 4)
    first = DupUp3D(8, 4, factor_t=2, factor_s=2)(down, first_chunk=True)
    assert first.shape == (2, 4, 3, 4, 4) and torch.equal(first, up[:, :, 1:])
    const = torch.full((1, 4, 3, 2, 2), 1.5)
    assert torch.allclose(AvgDown3D(4, 4, 2, 2)(const)[:, :, 1:], torch.full((1, 4, 1, 1, 1), 1.5))


def test_ltx_and_h3_preencode_share_the_corpus_assembly(tmp_path):
    from solarwm_b200.registry import load_backend

    for family, z, frames, hw, shape in (("ltx25_video", 128, 9, 64, (2, 128, 2, 2)), ("minimax_h3", 24, 9, 32, (3, 24, 2, 2))):
        out_root = tmp_path / family
        cfg = {"data": {"pixel_frames": frames, "pixel_height": hw, "pixel_width": hw, "seed": 1}, "runtime": {"device": "cpu"},
               "preencode": {"source": "synthetic", "num_samples": 2, "output_root": str(out_root), "codecs": {"vae_base": 4}}}
        res = load_backend(family).preencode(cfg)
        assert res["samples"] == 2
        rows = read_index(out_root / "index.jsonl")
        c = EncoderContract.from_dict(__import__("json").loads((out_root / "encoder-contract.json").read_text()))
        assert c.family == family
        s = read_encoded_sample(out_root, rows[0].values, c)
        assert tuple(s["latents"].shape) == shape, s["latents"].shape


def test_ltx_backend_trains_from_its_own_preencoded_corpus(tmp_path):
    from solarwm_b200.registry import load_backend

    be = load_backend("ltx25_video")
    pre = {"data": {"pixel_frames": 9, "pixel_height": 64, "pixel_width": 64, "seed": 1}, "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 2, "output_root": str(tmp_path / "enc"),
                         "codecs": {"z_dim": 16, "vae_base": 4, "t5": {"vocab": 512, "dim": 64, "dim_attn": 32, "dim_ffn": 64,
                                                                      "num_heads": 2, "num_layers": 1, "text_len": 16}}}}
    assert be.preencode(pre)["samples"] == 2
    config = {"schema": "solarwm.run.v1", "action": "train",
              "model": {"family": "ltx25_video", "architecture": "tiny", "camera_translation_transform": "linear"},
              "data": {"source": "index", "index": str(tmp_path / "enc" / "index.jsonl"), "seed": 0, "pixel_frames": 153},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "native_rectified_flow", "max_steps": 2,
                        "optimizer": {"lr": 1e-3}},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")}}
    out = be.train(config)
    assert out["final_step"] == 2 and out["last_loss"] == out["last_loss"]
