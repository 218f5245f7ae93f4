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


NODE_CLASS_MAPPINGS = {
    "SolarRendererModelLoader": SolarRendererModelLoader,
    "SolarRendererSigmas": SolarRendererSigmas,
    "SolarRendererAttention": SolarRendererAttention,
    "SolarRendererPrompt": SolarRendererPrompt,
    "SolarRendererSampler": SolarRendererSampler,
}
NODE_DISPLAY_NAME_MAPPINGS = {
    "SolarRendererModelLoader": "SolarRenderer model",
    "SolarRendererSigmas": "SolarRenderer sigmas",
    "SolarRendererAttention": "SolarRenderer attention backend",
    "SolarRendererPrompt": "SolarRenderer prompt",
    "SolarRendererSampler": "SolarRenderer sampler",
}
