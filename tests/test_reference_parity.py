"""Parity of the Wan DiT with the unmodified reference class (when it is installed under
``baseline/_ref``): identical parameter names and shapes, state-dict interchange, and the same
forward output (bf16 weights, CPU)."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def _reference_model(**kw):
    if not (REF / "solar").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    for p in (str(ROOT / "baseline" / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        from solar.backends.wan22.runtime.modeling import attention as ref_attention
        from solar.backends.wan22.runtime.modeling.causal_model import CausalWanModel
    except Exception as exc:  # noqa: BLE001
        pytest.skip(f"reference model not importable: {exc!r}")
    # CPU run: route the reference's attention shim to its SDPA branch
    ref_attention.FLASH_ATTN_2_AVAILABLE = False
    ref_attention.FLASH_ATTN_3_AVAILABLE = False
    # the cross-attention calls the CUDA-only flash_attention directly; on CPU send it through the
    # reference's own SDPA branch as well
    from solar.backends.wan22.runtime.modeling import model as ref_model

    ref_model.flash_attention = lambda q, k, v, k_lens=None, **kw: ref_attention.attention(q, k, v)
    return CausalWanModel(cam_self_attn_layers=[], add_control_adapter=False, **kw)


def test_tiny_wan_matches_reference_forward_and_names():
    from solarwm_b200.models.wan import WanDiT, wan_preset

    cfg = wan_preset("tiny")
    ref = _reference_model(model_type="t2v", in_dim=16, out_dim=16, dim=128, ffn_dim=512, num_heads=4,
                           num_layers=2, text_dim=256, text_len=32, freq_dim=64, frame_seq_length=64)
    # the reference's attention shim casts q/k/v to bf16, so the whole model has to run in bf16
    ours = WanDiT(cfg, device="cpu", dtype=torch.bfloat16, seed=0)
    ref_names = {n: tuple(p.shape) for n, p in ref.named_parameters()}
    our_names = {n: tuple(p.shape) for n, p in ours.named_parameters()}
    assert ref_names == our_names
    torch.manual_seed(0)
    with torch.no_grad():
        for p in ref.parameters():
            p.normal_(0, 0.05)
        for n, p in ref.named_parameters():
            if "norm" in n and n.endswith("weight"):
                p.add_(1.0)
    ref = ref.to(torch.bfloat16)
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    x = torch.randn(1, 16, 5, 16, 16)
    ctx = torch.randn(1, 32, 256)
    t_frames = torch.tensor([[0.0, 250.0, 500.0, 750.0, 999.0]])
    t_tokens = t_frames.repeat_interleave(64, dim=1)
    with torch.no_grad():
        out_ref = ref(x.bfloat16(), t=t_tokens, context=ctx.bfloat16(), seq_len=320).float()
        out = ours(x, t_frames, ctx).float()
    rel = ((out - out_ref).norm() / out_ref.norm()).item()
    assert rel < 3e-2, rel
