"""Parity tool: streaming (chunk by chunk, cached) decode against one-shot decode of the same latents.

    python -m solarwm_b200.serve.decode_parity --decoder conv --frames 9 --chunk 2
    python -m solarwm_b200.serve.decode_parity --decoder vit  --frames 9

``conv``: the causal-conv VAE decoded through ``StreamingDecoder`` in chunks of ``--chunk`` latents against
``VideoVAE.decode`` of the whole clip.  ``vit``: ``StreamingViTDecoder.push`` latent by latent against the windowed
oracle ``ViTVideoDecoder.decode_window`` (window by window, with the emission rule of the stream).  Prints one JSON
line with the largest absolute difference and whether the two are bit-identical; exits 1 when the difference exceeds
``--tolerance`` (reference: tools/h3_stream_decode_parity.py:11-62).
"""
from __future__ import annotations

import argparse
import json

import torch


def conv_parity(frames: int, chunk: int, device: str, seed: int = 0) -> dict:
    from ..models.vae import StreamingDecoder, VAEConfig, VideoVAE

    torch.manual_seed(seed)
    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    vae = VideoVAE(VAEConfig(z_dim=8, base=16, temporal_ups=(True, False))).to(device, dtype).eval()
    z = torch.randn(1, 8, frames, 6, 10, generator=torch.Generator().manual_seed(seed)).to(device, dtype)
    with torch.no_grad():
        full = vae.decode(z).float()
        dec = StreamingDecoder(vae)
        parts = [dec.push(z[:, :, i:i + chunk]) for i in range(0, frames, chunk)]
    streamed = torch.cat(parts, 2).float()
    return {"decoder": "conv", "frames": int(full.shape[2]), "max_abs_diff": float((streamed - full).abs().max()),
            "bit_identical": bool(torch.equal(streamed, full))}


def vit_parity(frames: int, device: str, seed: int = 0) -> dict:
    from ..models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder

    dtype = torch.bfloat16 if device.startswith("cuda") else torch.float32
    cfg = ViTDecoderConfig(latent_channels=8, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256, registers=8, patch=2)
    model = ViTVideoDecoder(cfg, device=device, dtype=dtype, seed=seed)
    lat = torch.randn(frames, 8, 8, 8, generator=torch.Generator().manual_seed(seed + 1)).to(device)
    dec = StreamingViTDecoder(model, (8, 8))
    with torch.no_grad():
        outs = [dec.push(lat[i]) for i in range(frames)]
    F, worst, same = cfg.frames_per_latent, 0.0, True
    shared = cfg.window - cfg.stride
    for i, got in enumerate(outs):
        start = ((i - shared) // cfg.stride) * cfg.stride if i >= cfg.window else 0
        hi = min(start + cfg.window, frames)
        with torch.no_grad():
            window = model.decode_window(lat[start:hi].permute(1, 0, 2, 3).unsqueeze(0))[0].float()
        s = i - start
        want = window[:, s * F:(s + 1) * F]
        want = want[:, -1:] if i % cfg.stride == 0 else want
        worst = max(worst, float((got.float() - want).abs().max()))
        same = same and bool(torch.equal(got.float(), want))
    return {"decoder": "vit", "frames": frames, "max_abs_diff": worst, "bit_identical": same}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--decoder", choices=["conv", "vit"], default="conv")
    ap.add_argument("--frames", type=int, default=9)
    ap.add_argument("--chunk", type=int, default=2)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tolerance", type=float, default=5e-2)
    args = ap.parse_args(argv)
    report = conv_parity(args.frames, args.chunk, args.device) if args.decoder == "conv" else vit_parity(args.frames, args.device)
    print(json.dumps(report))
    return 0 if report["max_abs_diff"] <= args.tolerance else 1


if __name__ == "__main__":
    raise SystemExit(main())
