"""The published Wan VAE topologies: parity with the unmodified reference class (when it is installed under
``baseline/_ref``), chunked == whole, and the published-name tables."""
import sys
from pathlib import Path

import pytest
import torch

from solarwm_b200.errors import BackendContractError
from solarwm_b200.models.vae import StreamingDecoder
from solarwm_b200.models.wan_vae_released import (ReleasedVAE, ReleasedVAEConfig, adopt_released_state, from_diffusers_wan21,
                                                  load_released, pixel_shuffle, pixel_unshuffle, released_names)

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _randomise(module, seed=0):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in module.named_parameters():
            p.copy_(torch.randn(p.shape, generator=g) * (0.3 if p.dim() > 1 and p.shape[-1] > 1 or "gamma" not in n else 0.1))
            if n.endswith("gamma"):
                p.add_(1.0)


def _reference_vae(**kw):
    if not (REF / "solar").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    for p in (str(ROOT / "baseline" / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        from solar.backends.wan22.runtime.modeling.vae import WanVAE_
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference VAE not importable: {exc!r}")
    return WanVAE_(**kw).eval()


def test_wan22_topology_matches_the_reference_class_whole_and_streamed():
    ref = _reference_vae(dim=8, dec_dim=8, z_dim=4, temperal_downsample=[False, True, True])
    _randomise(ref)
    cfg = ReleasedVAEConfig.wan22(enc_dim=8, dec_dim=8, z_dim=4)
    mean, std = [0.1, -0.2, 0.3, 0.0], [1.5, 0.7, 1.0, 2.0]
    ours = ReleasedVAE(cfg, mean, std).eval()
    names = released_names(ours)
    assert set(names) == set(ref.state_dict()) and set(names.values()) == {n for n, _ in ours.named_parameters()}
    adopt_released_state(ours, ref.state_dict())
    scale = [torch.tensor(mean), 1.0 / torch.tensor(std)]
    video = torch.randn(1, 3, 9, 32, 32)
    with torch.no_grad():
        want = ref.encode(video, scale)
        got = ours.encode(video)
        assert got.shape == want.shape == (1, 4, 3, 2, 2)
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (got - want).abs().max()
        assert torch.allclose(ours.encode(video, chunk_frames=4), want, atol=2e-4, rtol=1e-4)
        z = torch.randn(1, 4, 4, 2, 2)
        want_px = ref.decode(z, scale)
        got_px = ours.decode(z)
        assert got_px.shape == want_px.shape == (1, 3, 13, 32, 32)
        assert torch.allclose(got_px, want_px, atol=5e-4, rtol=1e-4), (got_px - want_px).abs().max()
        dec = StreamingDecoder(ours)
        pieces = torch.cat([dec.push(z[:, :, :1]), dec.push(z[:, :, 1:3]), dec.push(z[:, :, 3:])], dim=2)
        assert torch.allclose(pieces, want_px, atol=5e-4, rtol=1e-4)


def test_wan21_topology_names_shapes_and_streaming():
    cfg = ReleasedVAEConfig.wan21(dim=8, z_dim=4)
    vae = ReleasedVAE(cfg).eval()
    _randomise(vae, 1)
    names = released_names(vae)
    # the published Wan2.1 checkpoint numbers blocks and resamplers in one list per side
    for key in ("encoder.conv1.weight", "encoder.downsamples.2.resample.1.weight", "encoder.downsamples.3.shortcut.weight",
                "encoder.downsamples.5.time_conv.weight", "encoder.downsamples.10.residual.6.bias", "encoder.middle.1.to_qkv.weight",
                "encoder.head.0.gamma", "conv1.weight", "conv2.bias", "decoder.upsamples.3.time_conv.weight",
                "decoder.upsamples.4.shortcut.weight", "decoder.upsamples.11.resample.1.bias", "decoder.upsamples.14.residual.0.gamma",
                "decoder.head.2.weight"):
        assert key in names, key
    assert "decoder.upsamples.11.time_conv.weight" not in names and "encoder.downsamples.2.time_conv.weight" not in names
    assert len(set(names.values())) == len(names) == len(list(vae.named_parameters()))
    own = dict(vae.named_parameters())
    assert own[names["decoder.upsamples.3.resample.1.weight"]].shape == (16, 32, 3, 3)      # the up-sampling conv halves the channels
    assert own[names["decoder.upsamples.4.residual.2.weight"]].shape[:2] == (32, 16)
    video = torch.randn(1, 3, 9, 16, 16)
    with torch.no_grad():
        z = vae.encode(video)
        assert z.shape == (1, 4, 3, 2, 2) and torch.allclose(vae.encode(video, chunk_frames=4), z, atol=1e-4)
        px = vae.decode(z)
        assert px.shape == (1, 3, 9, 16, 16)
        dec = StreamingDecoder(vae)
        assert torch.allclose(torch.cat([dec.push(z[:, :, :2]), dec.push(z[:, :, 2:])], dim=2), px, atol=1e-4)
    # diffusers naming maps onto the same table
    pairs = {"quant_conv.weight": "conv1.weight", "post_quant_conv.bias": "conv2.bias", "encoder.conv_in.weight": "encoder.conv1.weight",
             "encoder.down_blocks.3.conv_shortcut.weight": "encoder.downsamples.3.shortcut.weight",
             "encoder.down_blocks.5.time_conv.bias": "encoder.downsamples.5.time_conv.bias",
             "encoder.down_blocks.2.resample.1.weight": "encoder.downsamples.2.resample.1.weight",
             "encoder.mid_block.resnets.1.norm2.gamma": "encoder.middle.2.residual.3.gamma",
             "decoder.mid_block.attentions.0.to_qkv.weight": "decoder.middle.1.to_qkv.weight",
             "decoder.up_blocks.1.resnets.0.conv_shortcut.bias": "decoder.upsamples.4.shortcut.bias",
             "decoder.up_blocks.0.upsamplers.0.time_conv.weight": "decoder.upsamples.3.time_conv.weight",
             "decoder.up_blocks.2.upsamplers.0.resample.1.weight": "decoder.upsamples.11.resample.1.weight",
             "decoder.up_blocks.3.resnets.2.conv2.weight": "decoder.upsamples.14.residual.6.weight",
             "decoder.norm_out.gamma": "decoder.head.0.gamma", "decoder.conv_out.bias": "decoder.head.2.bias"}
    for theirs, original in pairs.items():
        assert from_diffusers_wan21(theirs) == original and original in names


def test_checkpoint_files_load_strictly(tmp_path):
    cfg = ReleasedVAEConfig.wan22(enc_dim=8, dec_dim=8, z_dim=4)
    src = ReleasedVAE(cfg).eval()
    _randomise(src, 2)
    names = released_names(src)
    own = dict(src.named_parameters())
    state = {theirs: (own[ours].detach().reshape(-1, 1, 1, 1) if theirs.endswith("gamma") and ".residual." in theirs or theirs.endswith("head.0.gamma")
                      else own[ours].detach().clone()) for theirs, ours in names.items()}
    torch.save(state, tmp_path / "Wan2.2_VAE.pth")
    got = load_released(tmp_path / "Wan2.2_VAE.pth", cfg)
    z = torch.randn(1, 4, 2, 2, 2)
    assert torch.equal(got.decode(z), src.decode(z))
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in state.items()}, str(tmp_path / "vae.safetensors"))
    assert torch.equal(load_released(tmp_path / "vae.safetensors", cfg).decode(z), src.decode(z))
    broken = dict(state)
    broken.pop("decoder.conv1.bias")
    broken["decoder.extra"] = torch.zeros(1)
    with pytest.raises(BackendContractError) as err:
        adopt_released_state(ReleasedVAE(cfg), broken)
    assert "decoder.conv1.bias" in str(err.value) and "decoder.extra" in str(err.value)
    wrong = dict(state)
    wrong["conv2.weight"] = torch.zeros(5, 4, 1, 1, 1)
    with pytest.raises(BackendContractError):
        adopt_released_state(ReleasedVAE(cfg), wrong)
    with pytest.raises(BackendContractError):
        load_released(tmp_path / "missing.pth", cfg)


def test_pixel_shuffle_round_trip_and_frame_rule():
    x = torch.arange(2 * 3 * 2 * 4 * 6, dtype=torch.float32).view(2, 3, 2, 4, 6)
    assert torch.equal(pixel_shuffle(pixel_unshuffle(x, 2), 2), x) and pixel_unshuffle(x, 2).shape == (2, 12, 2, 2, 3)
    with pytest.raises(ValueError):
        ReleasedVAE(ReleasedVAEConfig.wan21(dim=8, z_dim=4)).encode(torch.zeros(1, 3, 4, 16, 16))


def test_text_encoder_matches_the_reference_class_and_loads_its_file(tmp_path):
    if not (REF / "solar").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    for p in (str(ROOT / "baseline" / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        from solar.backends.wan22.runtime.modeling.t5 import T5Encoder as RefEncoder
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference text encoder not importable: {exc!r}")
    from solarwm_b200.models.t5 import PromptTokenizer, T5Config, T5Encoder, WanTextEncoder, clean_prompt

    cfg = T5Config(vocab=64, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=2, num_buckets=32, text_len=12)
    torch.manual_seed(0)
    ref = RefEncoder(vocab=64, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=2, num_buckets=32, shared_pos=False, dropout=0.0).eval()
    ours = T5Encoder(cfg).eval()
    assert {k: tuple(v.shape) for k, v in ref.state_dict().items()} == {k: tuple(v.shape) for k, v in ours.state_dict().items()}
    ours.load_state_dict(ref.state_dict(), strict=True)
    ids = torch.randint(2, 64, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.bool)
    mask[1, 7:] = False
    with torch.no_grad():
        want, got = ref(ids, mask.long()), ours(ids, mask)
    assert torch.allclose(got[mask], want[mask], atol=2e-5, rtol=1e-4), (got - want)[mask].abs().max()
    # the published file is that state dict; the tokenizer directory holds a tokenizer.json
    torch.save(ref.state_dict(), tmp_path / "enc.pth")
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    tk = Tokenizer(WordLevel({"<pad>": 0, "</s>": 1, "<unk>": 2, "a": 3, "red": 4, "car": 5, "&": 6}, unk_token="<unk>"))
    tk.pre_tokenizer = Whitespace()
    (tmp_path / "tok").mkdir()
    tk.save(str(tmp_path / "tok" / "tokenizer.json"))
    enc = WanTextEncoder.from_released(tmp_path / "enc.pth", tmp_path / "tok", cfg=cfg, dtype=torch.float32)
    ids2, mask2 = enc.tok(["  a   red &amp;amp; car ", "car " * 40])
    assert ids2[0].tolist()[:6] == [3, 4, 6, 5, 1, 0] and mask2[0].sum() == 5
    assert ids2[1].tolist() == [5] * 11 + [1] and clean_prompt(" x\n\ty ") == "x y"
    out = enc(["a red car"])
    assert out.shape == (1, 12, 32) and bool((out[0, 4:] == 0).all()) and bool(out[0, :4].abs().sum() > 0)
    with pytest.raises(FileNotFoundError):
        PromptTokenizer(tmp_path, 12)
    bad = dict(ref.state_dict())
    bad.pop("norm.weight")
    torch.save(bad, tmp_path / "bad.pth")
    with pytest.raises((RuntimeError, ValueError)):
        WanTextEncoder.from_released(tmp_path / "bad.pth", tmp_path / "tok", cfg=cfg)


def test_codec_adapters_take_the_published_files(tmp_path):
    from solarwm_b200.backends.wan22.codec import Wan5BVAE, WanA14BVAE

    assert len(Wan5BVAE.mean) == len(Wan5BVAE.std) == 48 and min(Wan5BVAE.std) > 0 and len(WanA14BVAE.mean) == 16
    # full-size architectures are built on the meta device only: count what the published files hold
    with torch.device("meta"):
        big22, big21 = ReleasedVAE(ReleasedVAEConfig.wan22()), ReleasedVAE(ReleasedVAEConfig.wan21())
    n22, n21 = sum(p.numel() for p in big22.parameters()), sum(p.numel() for p in big21.parameters())
    assert 600e6 < n22 < 800e6 and 120e6 < n21 < 135e6, (n22, n21)
    own = dict(big22.named_parameters())
    names = released_names(big22)
    assert own[names["encoder.conv1.weight"]].shape == (160, 12, 3, 3, 3) and own[names["decoder.head.2.weight"]].shape == (12, 256, 3, 3, 3)
    assert own[names["decoder.conv1.weight"]].shape == (1024, 48, 3, 3, 3)
    # a small Wan2.1-shaped file through the adapter (the class checks the channel count)
    small = ReleasedVAE(ReleasedVAEConfig.wan21(dim=8, z_dim=16)).eval()
    _randomise(small, 3)
    state = {theirs: dict(small.named_parameters())[ours].detach().clone() for theirs, ours in released_names(small).items()}
    torch.save(state, tmp_path / "Wan2.1_VAE.pth")
    import solarwm_b200.models.wan_vae_released as mod

    original = mod.ReleasedVAEConfig.wan21
    try:
        mod.ReleasedVAEConfig.wan21 = classmethod(lambda cls, dim=8, z_dim=16: original(dim, z_dim))
        codec = WanA14BVAE.from_checkpoint(tmp_path / "Wan2.1_VAE.pth")
    finally:
        mod.ReleasedVAEConfig.wan21 = original
    video = torch.rand(1, 5, 3, 16, 16) * 2 - 1
    z = codec.encode(video)
    assert z.shape == (1, 2, 16, 2, 2)
    px = codec.decode(z)
    assert px.shape == (1, 5, 3, 16, 16) and float(px.abs().max()) <= 1.0
    pieces = list(codec.decode_streaming_chunks(z, chunk_latent_frames=1))
    assert torch.allclose(torch.cat(pieces, dim=1), px, atol=1e-4)


def test_online_encoding_batches_come_from_raw_clips_through_the_codecs():
    from solarwm_b200.backends.wan22.runtime import build_online_codecs, online_batches
    from solarwm_b200.models.wan import wan_preset

    arch = wan_preset("tiny")
    config = {"model": {"family": "wan22_ti2v_5b"}, "train": {"micro_batch_size": 2},
              "data": {"source": "synthetic", "encoding": "online", "num_samples": 3, "seed": 1, "pixel_frames": 9, "pixel_height": 32,
                       "pixel_width": 32,
                       "online_codecs": {"t5": {"vocab": 512, "dim": 256, "dim_attn": 64, "dim_ffn": 128, "num_heads": 2, "num_layers": 1, "text_len": 32},
                                         "vae": {"z_dim": 16, "base": 8, "temporal_ups": [True, True, False]}}}}
    stream = online_batches(config, arch, torch.device("cpu"))
    a, b = next(stream), next(stream)
    assert a["latents"].shape == (2, 3, 16, 4, 4) and a["text"].shape == (2, 32, 256) and a["sample_ids"] == ["synthetic-000000", "synthetic-000001"]
    # 3 clips, micro batch 2: the third clip is dropped at the epoch's end and the epoch repeats with the same encodings
    assert b["sample_ids"] == a["sample_ids"] and torch.equal(a["latents"], b["latents"])
    text, codec = build_online_codecs(config, torch.device("cpu"))
    assert codec.vae.cfg.z_dim == 16 and text(["a caption"]).shape == (1, 32, 256)
    bad = {**config, "data": {**config["data"], "online_codecs": {**config["data"]["online_codecs"], "vae": {"z_dim": 8, "base": 8}}}}
    from solarwm_b200.errors import DataContractError

    with pytest.raises(DataContractError):
        next(online_batches(bad, arch, torch.device("cpu")))
