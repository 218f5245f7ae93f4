"""Low-rank adapters over the Wan / LTX blocks, per-head attention gates, and the LTX adapter training route."""
import pytest
import torch

from solarwm_b200.errors import BackendContractError
from solarwm_b200.models.lora import TARGET_SUFFIX, adapter_parameter_count, inject_lora
from solarwm_b200.models.wan import WanConfig, WanDiT, wan_preset


def _model(**kw):
    cfg = WanConfig(model_type="t2v", patch_size=(1, 1, 1), in_dim=8, out_dim=8, dim=64, ffn_dim=128, num_heads=2,
                    num_layers=2, text_dim=32, text_len=8, freq_dim=32, norm_type="rms", cross_attn_norm=False, **kw)
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    g = torch.Generator().manual_seed(0)
    return m, (torch.randn(1, 8, 2, 4, 4, generator=g), torch.full((1, 2), 500.0), torch.randn(1, 8, 32, generator=g)), g


def test_released_recipe_adapter_inventory():
    cfg = wan_preset("ltx25_video_13b")
    assert (cfg.num_layers, cfg.num_heads, cfg.head_dim, cfg.gated_attention) == (48, 32, 128, True)
    # r = 384 on q / k / v / out of both attentions and on both FFN linears of 48 blocks
    assert adapter_parameter_count(cfg, 384) == 1_962_934_272 and len(TARGET_SUFFIX) == 10


def test_adapters_start_as_the_base_model_train_alone_and_merge():
    m, args, g = _model()
    base = m(*args)
    rt = inject_lora(m, rank=4, alpha=8)
    assert len(rt.keys) == 2 * 10 * 2 and rt.keys[0] == "transformer_blocks.0.attn1.to_q.lora_A.weight"
    assert sum(p.numel() for p in rt.parameters) == adapter_parameter_count(m.cfg, 4)
    assert torch.equal(m(*args), base)                                            # B = 0: nothing changes
    assert {n for n, p in m.named_parameters() if p.requires_grad} == \
        {n for n, _ in m.named_parameters() if ".lora." in n}                      # the base is frozen
    with torch.no_grad():
        for p in rt.parameters:
            if p.shape[1] == 4:                                                    # the B matrices
                p.normal_(0, 0.05, generator=g)
    adapted = m(*args)
    assert not torch.allclose(adapted, base, atol=1e-4)
    adapted.square().mean().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in rt.parameters)
    # gradient of one adapter against finite differences of the loss
    p = rt.parameter_by_key["transformer_blocks.1.ff.net.2.lora_B.weight"]
    with torch.no_grad():
        d = torch.zeros_like(p)
        d[3, 1] = 1e-3
        p.add_(d)
        up = m(*args).square().mean()
        p.sub_(2 * d)
        down = m(*args).square().mean()
        p.add_(d)
    assert abs(float((up - down) / 2e-3) - float(p.grad[3, 1])) < 2e-3 * max(1.0, abs(float(p.grad[3, 1])))
    # state round trip is strict
    state = {k: v.clone() for k, v in rt.state_dict().items()}
    meta = rt.metadata()
    assert meta["schema"] == "solarwm.ltx25.peft-lora.v1" and meta["state_shapes"][rt.keys[1]] == [64, 4]
    with pytest.raises(BackendContractError):
        rt.load_state_dict({k: v for k, v in list(state.items())[1:]})
    with pytest.raises(BackendContractError):
        rt.load_state_dict({**state, rt.keys[0]: state[rt.keys[0]].double()})
    rt.load_state_dict(state)
    with torch.no_grad():
        rt.merge_()
        merged = m(*args)
    assert torch.allclose(merged, adapted, atol=1e-5)
    assert all(float(p.detach().abs().max()) == 0 for k, p in rt.parameter_by_key.items() if "lora_B" in k)
    with pytest.raises(BackendContractError):
        inject_lora(m, rank=4)


def test_attention_gates_are_identity_at_init_and_scale_heads():
    gated, args, g = _model(gated_attention=True)
    plain, _, _ = _model()
    own = dict(gated.named_parameters())
    with torch.no_grad():
        for n, p in plain.named_parameters():
            p.copy_(own[n])
    assert "blocks.0.self_attn.to_gate_logits.weight" in own and torch.allclose(gated(*args), plain(*args), atol=1e-6)
    with torch.no_grad():
        for b in gated.blocks:
            b._p("self_attn.to_gate_logits.bias").fill_(-30.0)                     # gate -> 0: self-attention is switched off
        off = gated(*args)
        for b in plain.blocks:
            b._p("self_attn.o.weight").zero_()
        assert torch.allclose(off, plain(*args), atol=1e-5)


def test_ltx_backend_trains_adapters_and_writes_them(tmp_path):
    from solarwm_b200.registry import load_backend

    config = {"schema": "solarwm.run.v1", "action": "train", "name": "ltx-lora",
              "model": {"family": "ltx25_video", "architecture": "tiny", "adapter": {"rank": 4}},
              "data": {"source": "synthetic", "seed": 0, "pixel_frames": 153, "latent_frames": 2, "latent_height": 4, "latent_width": 4},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 3,
                        "optimizer": {"lr": 1e-3}},
              "runtime": {"output_dir": str(tmp_path), "device": "cpu"}}
    out = load_backend("ltx25_video").train(config)
    assert out["final_step"] == 3
    saved = torch.load(tmp_path / "checkpoint_model_000003" / "adapter.pt", weights_only=True)
    assert saved["metadata"]["rank"] == 4 and len(saved["state"]) == 2 * 10 * 2
    assert any(float(v.abs().max()) > 0 for k, v in saved["state"].items() if "lora_B" in k)       # the adapters moved
