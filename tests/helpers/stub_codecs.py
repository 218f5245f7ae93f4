"""Stand-in codecs with the renderer's frame cadence (17 n + 5 pixel frames -> 5 n + 2 latents) for command-line tests."""
import numpy as np
import torch

from solarwm_b200.renderer.preencode import Codecs, latent_frames


def factory() -> Codecs:
    def video(frames: np.ndarray) -> torch.Tensor:
        T = frames.shape[0]
        n = latent_frames(T)
        plane = torch.from_numpy(frames[:n, ::8, ::8].astype(np.float32).mean(-1) / 255.0)
        return plane.unsqueeze(0).repeat(24, 1, 1, 1)

    return Codecs(video=video, text=lambda s: (torch.full((6, 64), float(len(s)) / 100.0), torch.zeros(6)), canvas=(32, 48))
