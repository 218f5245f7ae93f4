"""Node-graph front end of the renderer (the node protocol of ComfyUI-style hosts, no host import needed).

A host discovers nodes through ``NODE_CLASS_MAPPINGS``; every node class declares ``INPUT_TYPES`` (a classmethod
returning ``{"required": {name: (type, options)}}``), ``RETURN_TYPES``, ``FUNCTION`` (the method the host calls with
the inputs as keyword arguments) and ``CATEGORY``, and returns a tuple.  The graph mirrors how the renderer is used:

    ModelLoader -> (Attention) -> Sampler <- Conditioning <- Prompt
                       Sigmas ---^

``MODEL`` is a prepared ``renderer.service.RenderService`` (precomputed modulation tables, text cache); ``SIGMAS`` the
schedule's noise levels; ``CONDITIONING`` the packed sample dictionary ``renderer.core.render`` takes; ``LATENT`` a
dictionary ``{"samples": [1, C, F, H, W]}``.  The attention node switches between this package's kernels
(``native``) and the library path (``library``); ``auto`` takes the kernels whenever the model sits on a GPU
(reference: deploy/solar_renderer/comfyui/nodes.py:96-431, whose choice is FlashAttention-4 / cuDNN).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..backends.minimax_h3 import flow
from ..models.h3 import H3DiT, h3_preset
from .service import RenderService

CATEGORY = "SolarRenderer"

STRUCTURE_SENTENCES: Dict[str, str] = {
    "scene_graybox": "The structure video is an untextured gray-box model of the scene.",
    "scene_whitebox": "The structure video is a white, shaded blocking model of the scene.",
    "semantic": "The structure video paints every object class in one flat colour.",
    "mask_skeleton": "The structure video shows subject masks with their pose skeletons.",
    "smpl_mesh": "The structure video shows body meshes of the people in the shot.",
    "near_depth": "The structure video is a depth map, brighter where the surface is nearer.",
}


class SolarRendererModelLoader:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"architecture": (["tiny", "h3_33b"], {"default": "tiny"}),
                             "steps": ("INT", {"default": 4, "min": 1, "max": 50}),
                             "device": (["auto", "cpu", "cuda"], {"default": "auto"}),
                             "free_projection": ("BOOLEAN", {"default": False,
                                                             "tooltip": "drop the adaLN projection weights once the tables exist"})}}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load"
    CATEGORY = CATEGORY

    def load(self, architecture="tiny", steps=4, device="auto", free_projection=False, seed=0):
        dev = ("cuda" if torch.cuda.is_available() else "cpu") if device == "auto" else device
        model = H3DiT(h3_preset(architecture), device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32, seed=seed)
        service = RenderService(model, steps=int(steps), free_projection=bool(free_projection))
        service.prepare()
        return (service,)


class SolarRendererSigmas:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"steps": ("INT", {"default": 4, "min": 1, "max": 50,
                                               "tooltip": "model evaluations; the distilled adapter was trained for 4"})}}

    RETURN_TYPES = ("SIGMAS",)
    FUNCTION = "sigmas"
    CATEGORY = CATEGORY

    def sigmas(self, steps=4):
        return (torch.tensor([1.0 - t for t in flow.rollout_times(int(steps))], dtype=torch.float32),)


class SolarRendererAttention:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",),
                             "backend": (["auto", "native", "library"],
                                         {"tooltip": "auto: this package's kernels on a GPU, the library path on CPU"})}}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "patch"
    CATEGORY = CATEGORY

    def patch(self, model, backend="auto"):
        on_gpu = model.model.proj_in.is_cuda
        if backend == "native" and not on_gpu:
            raise RuntimeError("the native attention kernels need the model on a CUDA device")
        ops.set_backend("native" if (backend == "native" or (backend == "auto" and on_gpu)) else "library")
        return (model,)


class SolarRendererPrompt:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"structure_type": (list(STRUCTURE_SENTENCES) + ["custom"], {"default": "scene_graybox"}),
                             "description": ("STRING", {"multiline": True, "default": ""}),
                             "custom_structure": ("STRING", {"default": ""})}}

    RETURN_TYPES = ("STRING",)
    FUNCTION = "build"
    CATEGORY = CATEGORY

    def build(self, structure_type="scene_graybox", description="", custom_structure=""):
        if structure_type == "custom":
            if not custom_structure.strip():
                raise ValueError("describe the custom structure video in one sentence")
            lead = custom_structure.strip().rstrip(".") + "."
        else:
            lead = STRUCTURE_SENTENCES[structure_type]
        text = description.strip()
        if not text:
            raise ValueError("the scene description is empty")
        return (f"{lead} {text}",)


def snap_frames(available: int, wanted: int) -> int:
    """The longest ``17 n + 5`` frames within both the request and the structure video (at least 22)."""
    frames = min(int(wanted), int(available))
    if frames < 22:
        raise ValueError(f"the renderer needs at least 22 frames of structure video, got {frames}")
    return 17 * ((frames - 5) // 17) + 5


def fit_images(images: torch.Tensor, width: int, height: int) -> torch.Tensor:
    """Host images ``[T, H, W, 3]`` in [0, 1] -> cover-resized and centre-cropped to ``height x width``."""
    import torch.nn.functional as F

    T, h, w, _ = images.shape
    scale = max(height / h, width / w)
    nh, nw = max(height, round(h * scale)), max(width, round(w * scale))
    x = F.interpolate(images.permute(0, 3, 1, 2).float(), size=(nh, nw), mode="bilinear", align_corners=False, antialias=scale < 1)
    top, left = (nh - height) // 2, (nw - width) // 2
    return x[:, :, top:top + height, left:left + width].permute(0, 2, 3, 1).clamp(0, 1)


class SolarRendererConditioning:
    """Structure video + prompt (+ the look's first frame) -> what the sampler consumes.  ``TEXT_ENCODER`` is a callable
    ``prompt -> [L, D]``; ``VAE`` an object whose ``encode(images [T, H, W, 3] in [0, 1])`` returns latents
    ``[C, F, h, w]`` (both are the host's own loaders; the renderer does not bundle the official codecs)."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"text_encoder": ("TEXT_ENCODER",), "vae": ("VAE",),
                             "structure": ("IMAGE", {"tooltip": "the structure video at 24 fps; the render follows it frame for frame"}),
                             "prompt": ("STRING", {"multiline": True}),
                             "width": ("INT", {"default": 1344, "min": 64, "max": 2048, "step": 32}),
                             "height": ("INT", {"default": 768, "min": 64, "max": 2048, "step": 32}),
                             "length": ("INT", {"default": 158, "min": 22, "max": 3609,
                                                "tooltip": "frames to render, snapped down to 17 n + 5 and to the structure video"})},
                "optional": {"first_frame": ("IMAGE", {"tooltip": "the look of the shot: its first frame, already in that look"}),
                             "structure_vae": ("VAE", {"tooltip": "a faster codec for the structure video; the first frame keeps vae"})}}

    RETURN_TYPES = ("CONDITIONING", "LATENT")
    RETURN_NAMES = ("positive", "latent")
    FUNCTION = "encode"
    CATEGORY = CATEGORY

    def encode(self, text_encoder, vae, structure, prompt, width=1344, height=768, length=158, first_frame=None, structure_vae=None):
        frames = snap_frames(structure.shape[0], length)
        video = fit_images(structure[:frames], int(width), int(height))
        structure_latents = (structure_vae or vae).encode(video)
        if structure_latents.ndim != 4 or structure_latents.shape[1] != 5 * ((frames - 5) // 17) + 2:
            raise ValueError(f"the codec returned {tuple(structure_latents.shape)} for {frames} frames")
        C, F, H, W = structure_latents.shape
        if first_frame is not None:
            anchor = vae.encode(fit_images(first_frame[:1], int(width), int(height)))[:, :1]
            if tuple(anchor.shape) != (C, 1, H, W):
                raise ValueError("the first frame's latent does not sit on the structure video's grid")
        else:
            anchor = torch.zeros(C, 1, H, W, dtype=structure_latents.dtype, device=structure_latents.device)
        text = text_encoder(str(prompt))
        if text.ndim != 2:
            raise ValueError("the text encoder returns [tokens, width]")
        cond = {"prompt_embeds": text, "anchor_latents": anchor, "structure_latents": structure_latents, "shape": (C, F, H, W),
                "pixel_frames": frames, "has_first_frame": first_frame is not None}
        return (cond, {"samples": torch.zeros(1, C, F, H, W)})


class SolarRendererLoraLoader:
    """Fill the model's adapters from an exported adapter file (``renderer.runtime.export_adapter``) and re-prepare it."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",), "adapter_path": ("STRING", {"default": ""}),
                             "strength": ("FLOAT", {"default": 1.0, "min": 0.0, "max": 2.0, "step": 0.05})}}

    RETURN_TYPES = ("MODEL",)
    FUNCTION = "load"
    CATEGORY = CATEGORY

    def load(self, model, adapter_path, strength=1.0):
        from .runtime import read_adapter

        state = read_adapter(adapter_path)
        own = {n: p for n, p in model.model.named_parameters() if "lora_" in n}
        if set(own) != set(state):
            raise ValueError("the adapter file does not fit this model's adapters")
        with torch.no_grad():
            for n, p in own.items():
                # the product B A scales linearly in either factor: the strength goes on the up-projection
                p.copy_((state[n] * (float(strength) if "lora_B" in n else 1.0)).to(p))
        model.prepare()
        return (model,)


def capture_plan(script: str) -> list:
    """A key / mouse script as time-ordered ``(seconds, action, argument)`` events.  Items are separated by commas or new
    lines: ``t:Key[:hold]`` (a key press), ``t:down:Key`` / ``t:up:Key``, ``t:mouse:dx:dy[:over]`` (a move spread over
    ``over`` seconds in 1/30 s steps), ``t:click[:hold]``."""
    plan = []
    for item in (x.strip() for x in script.replace("\n", ",").split(",")):
        if not item:
            continue
        parts = item.split(":")
        if len(parts) < 2:
            raise ValueError(f"capture script item {item!r} is not seconds:action")
        t, kind = float(parts[0]), parts[1]
        if t < 0:
            raise ValueError("capture script times are non-negative")
        if kind in ("down", "up"):
            plan.append((t, kind, parts[2]))
        elif kind == "mouse":
            dx, dy = float(parts[2]), float(parts[3])
            over = float(parts[4]) if len(parts) > 4 else 0.4
            steps = max(1, int(over * 30))
            plan += [(t + over * i / steps, "move", (dx / steps, dy / steps)) for i in range(steps)]
        elif kind == "click":
            hold = float(parts[2]) if len(parts) > 2 else 0.15
            plan += [(t, "mdown", None), (t + hold, "mup", None)]
        else:
            hold = float(parts[2]) if len(parts) > 2 else 0.12
            plan += [(t, "down", kind), (t + hold, "up", kind)]
    return sorted(plan, key=lambda e: e[0])


class SolarRendererWebCapture:
    """A recorded web page (a game, a 3-D scene) as a structure video.  The recording itself is done by a separate
    process -- ``command`` with ``{url} {out} {frames} {script}`` filled in -- so a browser that hangs never takes the
    host with it; that process needs a headless browser with a GPU canvas, which this package does not bundle.  The node
    checks the script, runs the command when one is given, and loads ``<out>.npy`` (RGB8 ``[T, H, W, 3]``)."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"url": ("STRING", {"default": ""}), "frames": ("INT", {"default": 158, "min": 22, "max": 3609}),
                             "out": ("STRING", {"default": "capture"})},
                "optional": {"script": ("STRING", {"multiline": True, "default": ""}), "command": ("STRING", {"default": ""}),
                             "timeout_seconds": ("INT", {"default": 600, "min": 10, "max": 7200})}}

    RETURN_TYPES = ("IMAGE",)
    FUNCTION = "capture"
    CATEGORY = CATEGORY

    def capture(self, url, frames=158, out="capture", script="", command="", timeout_seconds=600):
        import shlex
        import subprocess
        from pathlib import Path

        import numpy as np

        capture_plan(script)                                            # refuse a malformed script before anything runs
        target = Path(f"{out}.npy")
        if command:
            argv = [a.format(url=url, out=out, frames=int(frames), script=script) for a in shlex.split(command)]
            done = subprocess.run(argv, capture_output=True, text=True, timeout=int(timeout_seconds))
            if done.returncode != 0:
                raise RuntimeError(f"the capture process failed ({done.returncode}): {done.stderr[-400:]}")
        if not target.is_file():
            raise FileNotFoundError(f"{target} was not recorded")
        data = np.load(target, allow_pickle=False)
        if data.ndim != 4 or data.shape[-1] != 3 or data.dtype != np.uint8 or len(data) < 22:
            raise ValueError("a capture is RGB8 [T >= 22, H, W, 3]")
        return (torch.from_numpy(data[:int(frames)].astype(np.float32) / 255.0),)


class SolarRendererSampler:
    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",), "conditioning": ("CONDITIONING",),
                             "seed": ("INT", {"default": 0, "min": 0, "max": 2 ** 31 - 1})},
                "optional": {"sigmas": ("SIGMAS",)}}

    RETURN_TYPES = ("LATENT",)
    FUNCTION = "sample"
    CATEGORY = CATEGORY

    def sample(self, model, conditioning, seed=0, sigmas=None):
        if sigmas is not None and len(sigmas) != model.steps + 1:
            raise ValueError(f"the model was prepared for {model.steps} steps, the schedule has {len(sigmas) - 1}")
        latents = model.render(conditioning, seed=int(seed))
        return ({"samples": latents.unsqueeze(0)},)


class SolarRendererCausalSampler:
    """Chunk-by-chunk sampling with a key / value window: clips longer than the training length."""

    @classmethod
    def INPUT_TYPES(cls):
        return {"required": {"model": ("MODEL",), "conditioning": ("CONDITIONING",),
                             "seed": ("INT", {"default": 0, "min": 0, "max": 2 ** 31 - 1}),
                             "chunk": ("INT", {"default": 5, "min": 1, "max": 16}), "window": ("INT", {"default": 6, "min": 1, "max": 32}),
                             "steps": ("INT", {"default": 8, "min": 2, "max": 50})}}

    RETURN_TYPES = ("LATENT",)
    FUNCTION = "sample"
    CATEGORY = CATEGORY

    def sample(self, model, conditioning, seed=0, chunk=5, window=6, steps=8):
        from .causal import CausalRenderer

        held = model.model.fixed_tables                  # the prepared tables cover the fixed schedule only
        model.model.fixed_tables = None
        try:
            latents = CausalRenderer(model.model, chunk=int(chunk), window=int(window), steps=int(steps)).render(conditioning, seed=int(seed))
        finally:
            model.model.fixed_tables = held
        return ({"samples": latents.unsqueeze(0)},)


NODE_CLASS_MAPPINGS = {
    "SolarRendererModelLoader": SolarRendererModelLoader,
    "SolarRendererSigmas": SolarRendererSigmas,
    "SolarRendererAttention": SolarRendererAttention,
    "SolarRendererPrompt": SolarRendererPrompt,
    "SolarRendererConditioning": SolarRendererConditioning,
    "SolarRendererLoraLoader": SolarRendererLoraLoader,
    "SolarRendererWebCapture": SolarRendererWebCapture,
    "SolarRendererSampler": SolarRendererSampler,
    "SolarRendererCausalSampler": SolarRendererCausalSampler,
}
NODE_DISPLAY_NAME_MAPPINGS = {
    "SolarRendererModelLoader": "SolarRenderer model",
    "SolarRendererSigmas": "SolarRenderer sigmas",
    "SolarRendererAttention": "SolarRenderer attention backend",
    "SolarRendererPrompt": "SolarRenderer prompt",
    "SolarRendererConditioning": "SolarRenderer conditioning",
    "SolarRendererLoraLoader": "SolarRenderer LoRA loader",
    "SolarRendererWebCapture": "SolarRenderer web capture",
    "SolarRendererSampler": "SolarRenderer sampler",
    "SolarRendererCausalSampler": "SolarRenderer causal sampler",
}
