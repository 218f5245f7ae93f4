"""Wan pre-encoding: raw clips + captions -> latent / text-embedding shards.

Commit-last corpus assembly: every shard is written under a temporary name and published
create-only, the encoder contract next, and the index last; a crashed run leaves no index, and a
rerun refuses to overwrite published shards.  Ranks split the work by ``ordinal % world`` and write
disjoint shard prefixes; rank 0 merges the per-rank indices after a collective error exchange
(reference: solar/backends/wan22/runtime/preencode.py:277-699, solar/preencode/shards.py).

Sources: ``preencode.source: synthetic`` (deterministic random clips; used by tests and smoke runs)
or ``index`` (rows of a raw dataset index whose members are a video -- a ``.npy`` array ``[T, H, W, 3]`` uint8 or a
compressed container decoded by ``data.raw_video`` -- and a caption).
"""
from __future__ import annotations

from pathlib import Path
from typing import Any, Iterator, Mapping, Tuple

import numpy as np
import torch

from ...data.index import read_index, write_index
from ...errors import BackendContractError
from ...models.t5 import T5Config, WanTextEncoder
from ...models.vae import VAEConfig, VideoVAE
from ...preencode.contracts import wan_contract
from ...preencode.shards import EncodedShardWriter
from .contracts import PROFILES


def _camera_of(blob: bytes, frame_indices, source_hw, target_hw):
    """Absolute poses and normalised intrinsics of the latent frames out of a clip's camera archive."""
    from ..minimax_h3.geometry import ResizeCrop, decode_camera

    how = ResizeCrop(source_hw[1], source_hw[0], target_hw[1], target_hw[0], target_hw[1], target_hw[0])     # plain resize
    c2w, K = decode_camera(blob, [int(i) for i in frame_indices], how, focal_guard=False)
    return torch.from_numpy(c2w), torch.from_numpy(K)


def _clips(config: Mapping[str, Any], rank: int, world: int) -> Iterator[Tuple[str, torch.Tensor, str]]:
    pre = config["preencode"]
    data = config["data"]
    T, H, W = int(data["pixel_frames"]), int(data["pixel_height"]), int(data["pixel_width"])
    if str(pre.get("source", "synthetic")) == "synthetic":
        n = int(pre.get("num_samples", 4))
        for i in range(rank, n, world):
            g = torch.Generator().manual_seed(int(data.get("seed", 0)) * 7919 + i)
            clip = torch.rand(3, T, H, W, generator=g) * 2 - 1
            if pre.get("cameras"):                  # a seeded dolly so that camera-conditioned paths have something to read
                c2w = torch.eye(4).repeat(T, 1, 1)
                c2w[:, 2, 3] = torch.arange(T) * 0.01 * (1 + i)
                K = torch.tensor([[0.505, 0.0, 0.5], [0.0, 0.898, 0.5], [0.0, 0.0, 1.0]]).repeat(T, 1, 1)
                yield f"synthetic-{i:06d}", clip, f"synthetic clip {i}", (c2w, K)
            else:
                yield f"synthetic-{i:06d}", clip, f"synthetic clip {i}"
        return
    from ...data.archive import TarShardReader

    root = Path(pre["raw_root"])
    reader = TarShardReader()
    try:
        for row in read_index(pre["raw_index"]):
            if row.ordinal % world != rank:
                continue
            members = row.values.get("members", {})
            got = reader.read_members(root / row.shard, [members["video"], members["caption"]])
            from ...data.raw_video import load_clip

            vid = load_clip(members["video"], got[members["video"]], T)     # .npy array or a compressed container
            clip = torch.from_numpy(np.ascontiguousarray(vid)).permute(3, 0, 1, 2).float() / 127.5 - 1.0
            if clip.shape[2:] != (H, W):
                clip = torch.nn.functional.interpolate(clip.permute(1, 0, 2, 3), size=(H, W), mode="bilinear",
                                                       align_corners=False).permute(1, 0, 2, 3)
            caption = got[members["caption"]].decode("utf-8").strip()
            if pre.get("cameras"):
                if "camera" not in members:
                    raise BackendContractError(f"{row.sample_id}: preencode.cameras is on and the sample has no camera member")
                blob = reader.read_members(root / row.shard, [members["camera"]])[members["camera"]]
                yield row.sample_id, clip, caption, _camera_of(blob, range(T), vid.shape[1:3], (H, W))
            else:
                yield row.sample_id, clip, caption
    finally:
        reader.close()


def run_preencode(config: Mapping[str, Any], family: str, *, latent_channels: int = None,
                  temporal_ups: Tuple[bool, ...] = None) -> Mapping[str, Any]:
    """``latent_channels`` / ``temporal_ups`` describe the codec geometry of families outside the Wan profiles
    (LTX: 128 channels, 8 x 32 x 32; H3: 24 channels, 4 x 16 x 16); the corpus assembly is the same."""
    import torch.distributed as dist

    from ...runtime import distributed as rdist

    prof = PROFILES.get(family)
    if prof is None and latent_channels is None:
        raise BackendContractError(f"no codec geometry known for family {family!r}")
    pre, data = config["preencode"], config["data"]
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = torch.device(str(config.get("runtime", {}).get("device", "cpu")).replace("auto", "cuda" if torch.cuda.is_available() else "cpu"))
    dtype = torch.bfloat16
    codecs = pre.get("codecs", {}) or {}
    ups = tuple(bool(u) for u in codecs.get("temporal_ups", temporal_ups or VAEConfig().temporal_ups))
    vcfg = VAEConfig(z_dim=int(codecs.get("z_dim", latent_channels or prof.latent_channels)),
                     base=int(codecs.get("vae_base", 16)), temporal_ups=ups)
    tcfg = T5Config(**codecs["t5"]) if "t5" in codecs else T5Config.tiny()
    released = codecs.get("released_vae")           # "wan2.2" / "wan2.1": the published topology + ``vae_checkpoint``
    if released:
        from .codec import Wan5BVAE, WanA14BVAE

        kind = {"wan2.2": Wan5BVAE, "wan2.1": WanA14BVAE}.get(str(released))
        if kind is None or not codecs.get("vae_checkpoint"):
            raise BackendContractError("preencode.codecs.released_vae is 'wan2.2' or 'wan2.1' and needs vae_checkpoint")
        vae = kind.from_checkpoint(codecs["vae_checkpoint"], device=device).vae
        t_stride, s_stride = 4, 8 * vae.cfg.patch
        vcfg = vae.cfg
    else:
        vae = VideoVAE(vcfg).to(device=device, dtype=torch.float32).eval()
        if codecs.get("vae_checkpoint"):
            vae.load_state_dict(torch.load(codecs["vae_checkpoint"], map_location=device, weights_only=True))
        t_stride = 2 ** sum(vcfg.temporal_ups)
        s_stride = 2 ** len(vcfg.temporal_ups)
    if codecs.get("t5_checkpoint") and codecs.get("tokenizer"):     # the published encoder file + tokenizer directory
        text = WanTextEncoder.from_released(codecs["t5_checkpoint"], codecs["tokenizer"], cfg=tcfg, device=device, dtype=torch.float32)
    else:
        text = WanTextEncoder(tcfg, device=device, dtype=torch.float32)
        if codecs.get("t5_checkpoint"):
            text.model.load_state_dict(torch.load(codecs["t5_checkpoint"], map_location=device, weights_only=True))
    contract = wan_contract(family, pixel_frames=int(data["pixel_frames"]), height=int(data["pixel_height"]),
                            width=int(data["pixel_width"]), z_dim=vcfg.z_dim, text_len=tcfg.text_len,
                            text_dim=tcfg.dim, temporal_stride=t_stride, spatial_stride=s_stride,
                            video_codec=str(codecs.get("video_codec", "causal-vae-random-init")),
                            text_codec=str(codecs.get("text_codec", "t5-random-init")), cameras=bool(pre.get("cameras")))
    out = Path(pre["output_root"])
    writer = EncodedShardWriter(out, contract, samples_per_shard=int(pre.get("samples_per_shard", 64)),
                                prefix=f"encoded-r{rank:03d}")
    error = None
    try:
        for sample_id, clip, caption, *camera in _clips(config, rank, world):
            with torch.no_grad():
                z = vae.encode(clip.unsqueeze(0).to(device))[0].permute(1, 0, 2, 3)      # [F, z, h, w]
                e = text([caption])[0]
            tensors = {"latents": z.to(dtype).cpu(), "text": e.to(dtype).cpu()}
            if camera:                              # per pixel frame -> the frame each latent starts at
                at = torch.arange(z.shape[0]) * t_stride
                tensors["camera_c2w"], tensors["camera_K"] = camera[0][0][at].float(), camera[0][1][at].float()
            writer.add(sample_id, tensors, {"caption": caption})
        index = writer.finish(index_name=f"index-r{rank:03d}.jsonl") if writer.rows or writer._pending else None
    except Exception as exc:  # noqa: BLE001 - exchanged so that every rank fails together
        error, index = exc, None
    rdist.propagate_collective_error(None if error is None else f"{type(error).__name__}: {error}",
                                     dist=dist if world > 1 else None, label=f"{family} preencode")
    if world > 1:
        dist.barrier()
    total = 0
    if rank == 0:
        rows = []
        for r in range(world):
            part = out / f"index-r{r:03d}.jsonl"
            if part.exists():
                rows.extend(dict(x.values) for x in read_index(part))
        total = write_index(out / "index.jsonl", rows)     # the corpus index is the last file written
    return {"samples": total, "contract_digest": contract.digest, "output_root": str(out)}
