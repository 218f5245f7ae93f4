"""``solar environment probe``: versions of python / torch / CUDA / NCCL and of the native library
(reference: solar/runtime/images.py:10-39)."""
from __future__ import annotations

import importlib
import platform
import sys


def probe_python_runtime() -> dict:
    out = {"python": sys.version.split()[0], "platform": platform.platform(), "packages": {}}
    for name in ("numpy", "yaml", "torch", "einops", "safetensors"):
        try:
            mod = importlib.import_module(name)
            out["packages"][name] = getattr(mod, "__version__", "unknown")
        except Exception:  # noqa: BLE001
            out["packages"][name] = None
    try:
        import torch

        out["cuda"] = torch.version.cuda
        out["cuda_available"] = torch.cuda.is_available()
        out["nccl"] = ".".join(str(v) for v in torch.cuda.nccl.version()) if torch.cuda.is_available() else None
        if torch.cuda.is_available():
            out["devices"] = [{"name": torch.cuda.get_device_name(i),
                               "capability": list(torch.cuda.get_device_capability(i))}
                              for i in range(torch.cuda.device_count())]
    except Exception as exc:  # noqa: BLE001
        out["torch_error"] = repr(exc)
    from ..ops import _lib

    out["native_library"] = {"path": str(_lib.lib_path()), "built": _lib.available()}
    return out
