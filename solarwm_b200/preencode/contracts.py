"""What a pre-encoded sample must look like.

``TensorSpec`` fixes the dtype, rank and (possibly symbolic) extents of one stored tensor;
``EncoderContract`` names the encoder (family, codec ids, pixel geometry, latent strides) and the
tensor specs, and has a stable digest that goes into every shard and index so a reader can refuse
data produced under a different contract (reference: solar/preencode/contracts.py:14-159).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

import numpy as np

from ..errors import DataContractError

_DTYPES = ("float16", "bfloat16", "float32", "float64", "int32", "int64", "uint8", "bool")


@dataclass(frozen=True)
class TensorSpec:
    name: str
    dtype: str
    shape: Tuple[Any, ...]          # ints are exact extents, strings are symbols shared across tensors
    finite: bool = True

    def __post_init__(self):
        if not self.name or not isinstance(self.name, str):
            raise DataContractError("tensor spec needs a non-empty name")
        if self.dtype not in _DTYPES:
            raise DataContractError(f"tensor spec {self.name!r}: unsupported dtype {self.dtype!r}")
        for d in self.shape:
            if not (isinstance(d, str) and d) and not (type(d) is int and d > 0):
                raise DataContractError(f"tensor spec {self.name!r}: extents are positive ints or symbols")

    def as_dict(self) -> dict:
        return {"name": self.name, "dtype": self.dtype, "shape": list(self.shape), "finite": self.finite}


@dataclass(frozen=True)
class EncoderContract:
    family: str
    video_codec: str
    text_codec: str
    pixel_frames: int
    pixel_height: int
    pixel_width: int
    temporal_stride: int
    spatial_stride: int
    tensors: Tuple[TensorSpec, ...]
    extras: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        names = [t.name for t in self.tensors]
        if len(set(names)) != len(names) or not names:
            raise DataContractError("encoder contract tensor names must be unique and non-empty")
        if min(self.pixel_frames, self.pixel_height, self.pixel_width, self.temporal_stride, self.spatial_stride) < 1:
            raise DataContractError("encoder contract geometry must be positive")

    def as_dict(self) -> dict:
        return {"family": self.family, "video_codec": self.video_codec, "text_codec": self.text_codec,
                "pixel_frames": self.pixel_frames, "pixel_height": self.pixel_height, "pixel_width": self.pixel_width,
                "temporal_stride": self.temporal_stride, "spatial_stride": self.spatial_stride,
                "tensors": [t.as_dict() for t in self.tensors], "extras": dict(self.extras)}

    @property
    def digest(self) -> str:
        blob = json.dumps(self.as_dict(), sort_keys=True, separators=(",", ":")).encode()
        return hashlib.blake2s(blob).hexdigest()

    @classmethod
    def from_dict(cls, v: Mapping[str, Any]) -> "EncoderContract":
        try:
            return cls(family=str(v["family"]), video_codec=str(v["video_codec"]), text_codec=str(v["text_codec"]),
                       pixel_frames=int(v["pixel_frames"]), pixel_height=int(v["pixel_height"]),
                       pixel_width=int(v["pixel_width"]), temporal_stride=int(v["temporal_stride"]),
                       spatial_stride=int(v["spatial_stride"]),
                       tensors=tuple(TensorSpec(t["name"], t["dtype"], tuple(t["shape"]), bool(t.get("finite", True)))
                                     for t in v["tensors"]), extras=dict(v.get("extras", {})))
        except (KeyError, TypeError, ValueError) as exc:
            raise DataContractError("invalid encoder contract") from exc

    @property
    def latent_frames(self) -> int:
        return (self.pixel_frames - 1) // self.temporal_stride + 1


def _dtype_name(arr) -> str:
    name = str(getattr(arr, "dtype", ""))
    return name.replace("torch.", "")


def validate_encoded_tensors(contract: EncoderContract, tensors: Mapping[str, Any]) -> Mapping[str, int]:
    """Check names, dtypes, ranks, exact extents, symbol consistency and finiteness; returns the symbol
    bindings.  Accepts numpy arrays or torch tensors."""
    want = {t.name for t in contract.tensors}
    if set(tensors) != want:
        raise DataContractError(f"encoded tensor names {sorted(tensors)} differ from the contract {sorted(want)}")
    bound: dict = {}
    for spec in contract.tensors:
        arr = tensors[spec.name]
        if _dtype_name(arr) != spec.dtype:
            raise DataContractError(f"{spec.name}: dtype {_dtype_name(arr)} != {spec.dtype}")
        shape = tuple(int(d) for d in arr.shape)
        if len(shape) != len(spec.shape):
            raise DataContractError(f"{spec.name}: rank {len(shape)} != {len(spec.shape)}")
        for got, exp in zip(shape, spec.shape):
            if isinstance(exp, str):
                if bound.setdefault(exp, got) != got:
                    raise DataContractError(f"{spec.name}: symbol {exp} bound to {bound[exp]} and {got}")
            elif got != exp:
                raise DataContractError(f"{spec.name}: extent {got} != {exp}")
        if spec.finite and spec.dtype.startswith(("float", "bfloat")):
            a = arr.float().numpy() if hasattr(arr, "numpy") and not isinstance(arr, np.ndarray) else np.asarray(arr, dtype=np.float32)
            if not np.isfinite(a).all():
                raise DataContractError(f"{spec.name}: non-finite values")
    return bound


def wan_contract(family: str, *, pixel_frames: int, height: int, width: int, z_dim: int, text_len: int,
                 text_dim: int, temporal_stride: int = 4, spatial_stride: int = 16,
                 video_codec: str = "wan2.2-vae", text_codec: str = "umt5-xxl",
                 dtype: str = "bfloat16", extras: Optional[Mapping[str, Any]] = None, cameras: bool = False) -> EncoderContract:
    """``cameras``: every sample also carries the absolute camera-to-world pose and the normalised intrinsics of each
    latent frame (``camera_c2w`` [F, 4, 4], ``camera_K`` [F, 3, 3], fp32)."""
    f = (pixel_frames - 1) // temporal_stride + 1
    tensors = (TensorSpec("latents", dtype, (f, z_dim, height // spatial_stride, width // spatial_stride)),
               TensorSpec("text", dtype, (text_len, text_dim)))
    if cameras:
        tensors += (TensorSpec("camera_c2w", "float32", (f, 4, 4)), TensorSpec("camera_K", "float32", (f, 3, 3)))
    return EncoderContract(family, video_codec, text_codec, pixel_frames, height, width, temporal_stride, spatial_stride, tensors,
                           dict(extras or {}))
