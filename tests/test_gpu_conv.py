"""Implicit-GEMM convolution kernel against torch's fp32 convolution, and the VAE decoder on it."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _reference(x_cl, weight, bias, history):
    """x_cl [T, H, W, Cin] -> [T, H, W, Cout] in fp32: same padding in H / W, causal in T."""
    kt, kh, kw = weight.shape[2:]
    x = x_cl.float().permute(3, 0, 1, 2).unsqueeze(0)
    left = history.float().permute(3, 0, 1, 2).unsqueeze(0) if history is not None else x.new_zeros(1, x.shape[1], kt - 1, *x.shape[3:])
    x = torch.cat([left, x], 2) if kt > 1 else x
    x = F.pad(x, (kw // 2, kw // 2, kh // 2, kh // 2))
    y = F.conv3d(x, weight.float(), None if bias is None else bias.float())
    return y[0].permute(1, 2, 3, 0)


@pytest.mark.parametrize("shape", [
    # T, H, W, Cin, Cout, kernel, with_history
    (3, 16, 32, 64, 256, (3, 3, 3), False),
    (2, 11, 23, 48, 24, (3, 3, 3), True),       # ragged borders, channel padding on both sides
    (4, 8, 16, 96, 320, (3, 1, 1), True),       # temporal-only kernel, two N tiles, 1.5 K blocks per tap
    (1, 20, 20, 128, 64, (1, 3, 3), False),     # one-frame-deep (2-D) convolution
    (2, 9, 17, 32, 12, (1, 1, 1), False),       # pointwise; Cout padded to 16
])
def test_conv3d_kernel_matches_fp32_convolution(shape):
    from solarwm_b200 import ops
    from solarwm_b200.ops import functional as F_

    T, H, W, cin, cout, k, with_hist = shape
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, H, W, cin, generator=g).cuda().bfloat16()
    w = (torch.randn(cout, cin, *k, generator=g) / (cin * k[0] * k[1] * k[2]) ** 0.5).cuda().bfloat16()
    b = torch.randn(cout, generator=g).cuda().bfloat16()
    hist = torch.randn(k[0] - 1, H, W, cin, generator=g).cuda().bfloat16() if with_hist and k[0] > 1 else None
    pw, pb = F_.pack_conv_weight(w, b)
    y = F_.conv3d_channels_last(x, pw, pb, k, history=hist, out_channels=cout)
    ops.check_status()
    want = _reference(x, w, b, hist)
    assert y.shape == want.shape
    err = (y.float() - want).abs().max() / want.abs().max()
    assert err < 1.5e-2, float(err)


def test_vae_decoder_on_native_convolutions_matches_library_path_and_streams():
    from solarwm_b200.models.vae import CausalConv3d, StreamingDecoder, VAEConfig, VideoVAE
    from solarwm_b200.ops import _lib

    torch.manual_seed(0)
    cfg = VAEConfig(z_dim=16, base=16, temporal_ups=(True, False), out_channels=3)
    vae = VideoVAE(cfg).cuda().bfloat16().eval()
    z = torch.randn(1, 16, 3, 6, 10).cuda().bfloat16()
    before = _lib.COUNTERS.get("conv3d", 0)
    with torch.no_grad():
        native = vae.decode(z).float()
    assert _lib.COUNTERS.get("conv3d", 0) > before
    # the same weights through torch's convolutions (fp32)
    ref_vae = VideoVAE(cfg).cuda().float().eval()
    ref_vae.load_state_dict({k: v.float() for k, v in vae.state_dict().items()})
    with torch.no_grad():
        want = ref_vae.decode(z.float())
    assert native.shape == want.shape
    assert (native - want).abs().max() / want.abs().max() < 6e-2
    # chunked decode with the feature cache equals the one-shot decode
    dec = StreamingDecoder(vae)
    parts = [dec.push(z[:, :, :1]), dec.push(z[:, :, 1:])]
    streamed = torch.cat(parts, 2).float()
    assert (streamed - native).abs().max() / native.abs().max() < 2e-2
    assert isinstance(vae.decoder.conv_in, CausalConv3d)


def test_published_topology_decoder_on_native_convolutions_matches_fp32_and_streams():
    from solarwm_b200.models.vae import StreamingDecoder
    from solarwm_b200.models.wan_vae_released import ReleasedVAE, ReleasedVAEConfig
    from solarwm_b200.ops import _lib

    for cfg in (ReleasedVAEConfig.wan22(enc_dim=16, dec_dim=16, z_dim=16), ReleasedVAEConfig.wan21(dim=16, z_dim=16)):
        torch.manual_seed(0)
        vae = ReleasedVAE(cfg).cuda().bfloat16().eval()
        z = torch.randn(1, 16, 3, 6, 10).cuda().bfloat16()
        before = _lib.COUNTERS.get("conv3d", 0)
        with torch.no_grad():
            native = vae.decode(z).float()
        assert _lib.COUNTERS.get("conv3d", 0) > before
        ref_vae = ReleasedVAE(cfg).cuda().float().eval()
        ref_vae.load_state_dict({k: v.float() for k, v in vae.state_dict().items()})
        with torch.no_grad():
            want = ref_vae.decode(z.float())
        assert native.shape == want.shape == (1, 3, 9, 48 * cfg.patch, 80 * cfg.patch)
        assert (native - want).abs().max() / want.abs().max() < 6e-2
        dec = StreamingDecoder(vae)
        streamed = torch.cat([dec.push(z[:, :, :1]), dec.push(z[:, :, 1:])], 2).float()
        assert (streamed - native).abs().max() / native.abs().max() < 2e-2


@pytest.mark.parametrize("C", [16, 64, 160, 1024])
def test_rms_silu_channels_last_matches_unfused_composition(C):
    from solarwm_b200.models.vae import RMSNormC
    from solarwm_b200.ops import functional as F_

    g = torch.Generator().manual_seed(C)
    x = (torch.randn(2, 3, 5, 7, C, generator=g) * 3).cuda().bfloat16()
    norm = RMSNormC(C).cuda()
    norm.gamma.data = (torch.rand(C, generator=g) + 0.5).cuda()
    for silu in (False, True):
        got = F_.rms_silu_channels_last(x, norm.gamma, silu)
        xf = x.float()
        want = xf / xf.norm(dim=-1, keepdim=True).clamp_min(1e-12) * C ** 0.5 * norm.gamma.float()
        want = F.silu(want) if silu else want
        assert (got.float() - want).abs().max() < 4e-2 * want.abs().max()
