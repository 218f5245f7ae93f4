"""Model FLOPs of a DiT training step and the fraction of the measured tensor-core rate a step time achieves.

Counting rule (multiply-add = 2 FLOPs), per transformer block and per sample of S tokens, T text tokens, width d,
FFN width f:  q/k/v/o projections ``8 S d^2``; self-attention scores + values ``4 S^2 d``; cross-attention q/o
``4 S d^2``, k/v ``4 T d^2``, scores + values ``4 S T d``; FFN ``4 S d f``.  Backward is twice the forward; recomputed
work is NOT counted (model FLOPs, not hardware FLOPs), so a run that recomputes less does not look better than it is.
The denominator is the pool's measured cuBLAS bf16 rate: the sustained figure for a whole step, the burst figure for a
kernel timed alone (``MEASURED_PEAKS.json`` at the repository root, with the stated fallback when it is absent).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping, Optional


def block_forward_flops(tokens: int, text_tokens: int, dim: int, ffn_dim: int) -> float:
    s, t, d, f = float(tokens), float(text_tokens), float(dim), float(ffn_dim)
    return 8 * s * d * d + 4 * s * s * d + 4 * s * d * d + 4 * t * d * d + 4 * s * t * d + 4 * s * d * f


def training_step_flops(cfg, tokens: int, batch: int = 1) -> float:
    """Forward + backward model FLOPs of one step (embeddings and the head are under 0.1 % and left out)."""
    return 3.0 * batch * cfg.num_layers * block_forward_flops(tokens, cfg.text_len, cfg.dim, cfg.ffn_dim)


def measured_peaks(root: Optional[Path] = None) -> Mapping[str, object]:
    path = (root or Path(__file__).resolve().parents[2]) / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def step_utilization(cfg, tokens: int, ms_per_step: float, n_gpus: int, batch: int = 1, root: Optional[Path] = None) -> Mapping[str, object]:
    flops = training_step_flops(cfg, tokens, batch)
    peaks = measured_peaks(root)
    achieved = flops / (ms_per_step * 1e-3) / 1e12                     # TFLOP/s over the whole job
    return {"model_tflop_per_step": round(flops / 1e12, 1), "achieved_tflops": round(achieved, 1),
            "fraction_of_sustained_peak": round(achieved / (n_gpus * peaks["bf16_tflops_sustained"]), 3),
            "peak_source": peaks["source"]}
