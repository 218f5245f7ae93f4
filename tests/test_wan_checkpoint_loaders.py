"""Wan checkpoint loaders: name normalisation, weights-only starts that re-base the optimizer, LIVE + EMA starts,
flow-matching -> AnyFlow upgrades, and resume from a name-keyed AdamW state."""
import dataclasses

import pytest
import torch

from solarwm_b200.backends.wan22 import checkpoint as ckpt
from solarwm_b200.checkpoint import CheckpointContract
from solarwm_b200.engine.optim import FlatAdamW
from solarwm_b200.errors import CheckpointError
from solarwm_b200.models.wan import WanConfig, WanDiT


def _cfg(**kw):
    return WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=32, ffn_dim=64, num_heads=2, num_layers=1, text_dim=16,
                     text_len=4, freq_dim=16, **kw)


def _contract():
    return CheckpointContract(family="wan22_ti2v_5b", stage="stage0p5", causal_mode="bidirectional", objective="flow_matching",
                              objective_variant="", camera_translation_transform="linear", parameterization="full",
                              sp_size=1, data_generation="synthetic", extras={"timestep_shift": 5.0})


class _Sched:
    def state_dict(self):
        return {"last_step": 3}

    def load_state_dict(self, s):
        self.loaded = s


def _trained(tmp_path, seed=1, steps=3):
    m = WanDiT(_cfg(), device="cpu", dtype=torch.float32, seed=seed)
    m.ensure_grads()
    opt = FlatAdamW(m.units(), lr=1e-2, ema_decay=0.5)
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        for u in m.units():
            u.grad.copy_(torch.randn(u.grad.shape, generator=g))
            u.grad_v.copy_(torch.randn(u.grad_v.shape, generator=g))
        opt.set_clip(torch.tensor(1.0), None)
        opt.step()
    state = opt.state_dict()
    ckpt.save_checkpoint(tmp_path, steps, model=m, scheduler=_Sched(), contract=_contract(), config={"name": "t"},
                         ema_state=opt.ema_state_dict(m, gathered=state), ema_num_updates=steps,
                         rank_states=[{"batches_consumed": steps}], is_main=True, optimizer_state=state)
    return m, opt, tmp_path / f"checkpoint_model_{steps:06d}"


def test_name_normalisation():
    good = ckpt.normalize_weight_names({"model.blocks.0._fsdp_wrapped_module.ffn.0.weight": 1, "model.head.head.bias": 2})
    assert good == {"blocks.0.ffn.0.weight": 1, "head.head.bias": 2}
    with pytest.raises(CheckpointError):
        ckpt.normalize_weight_names({"model.a": 1, "b": 2})                       # mixed root namespace
    with pytest.raises(CheckpointError):
        ckpt.normalize_weight_names({"a._orig_mod.b": 1, "a.b": 2})               # collision
    with pytest.raises(CheckpointError):
        ckpt.normalize_weight_names({})


def test_weights_only_start_rebases_master_and_ema(tmp_path):
    src, src_opt, path = _trained(tmp_path)
    for ema_source, want_ema in ((None, "live"), ("ema", "ema")):
        m = WanDiT(_cfg(), device="cpu", dtype=torch.bfloat16, seed=9)           # bf16: the optimizer keeps fp32 masters
        m.ensure_grads()
        opt = FlatAdamW(m.units(), lr=0.0, ema_decay=0.5)
        ckpt.load_checkpoint(path, model=m, optimizer=opt, mode="weights_only", ema_source=ema_source)
        want = dict(src.named_parameters())
        for n, p in m.named_parameters():
            assert torch.equal(p.detach().float(), want[n].detach().to(p.dtype).float()), n
        # a step with lr 0 and zero gradients must leave the loaded weights in place (the masters were re-based)
        for u in m.units():
            u.grad.zero_()
            u.grad_v.zero_()
        opt.set_clip(torch.tensor(0.0), None)
        opt.weight_decay = 0.0
        opt.step()
        for n, p in m.named_parameters():
            assert torch.equal(p.detach().float(), want[n].detach().to(p.dtype).float()), n
        ema = opt.ema_state_dict(m)
        ref = src_opt.ema_state_dict(src) if want_ema == "ema" else {n: p.detach().float() for n, p in want.items()}
        assert opt.step_count == 1
        for n in ema:
            assert torch.allclose(ema[n], ref[n].float(), atol=1e-2), n
        if want_ema == "ema":
            assert any(not torch.allclose(ema[n], want[n].detach().float(), atol=1e-3) for n in ema)   # it IS the average


def test_flow_matching_weights_start_an_anyflow_model(tmp_path):
    src, _, path = _trained(tmp_path)
    m = WanDiT(_cfg(flow_objective="anyflow_forward_map"), device="cpu", dtype=torch.float32, seed=5)
    _, payload = ckpt.load_checkpoint(path, model=m, mode="weights_only")
    assert sorted(payload["initialised_from_time_embedding"]) == sorted(
        n for n, _ in m.named_parameters() if n.startswith("delta_embedding."))
    for n, p in m.named_parameters():
        if n.startswith("delta_embedding."):
            assert torch.equal(p, m.get_parameter(n.replace("delta_embedding.", "time_embedding.", 1)))
    broken = {n: p.detach() for n, p in src.named_parameters() if n != "head.head.bias"}
    with pytest.raises(CheckpointError):
        ckpt.upgrade_flow_matching_to_anyflow(broken, m)                          # anything else missing is an error


def test_resume_from_a_name_keyed_adamw_state(tmp_path):
    """The reference stores ``torch.optim.AdamW`` state under parameter names (with a ``model.`` root); such a payload
    resumes into the flat optimizer: moments, step and EMA land where the parameters live."""
    src, src_opt, path = _trained(tmp_path)
    full = src_opt.state_dict()
    named, idx = {}, {id(u): i for i, u in enumerate(src_opt.units)}
    for n, p in src.named_parameters():
        slot = p.flat_unit.slots[p.flat_name]
        st = full["units"][idx[id(p.flat_unit)]]["v" if slot.is_vector else "m"]
        cut = lambda t: t[slot.offset:slot.offset + slot.numel].view(slot.shape).clone()   # noqa: E731
        named["model." + n] = {"step": torch.tensor(3.0), "exp_avg": cut(st["exp_avg"]), "exp_avg_sq": cut(st["exp_avg_sq"])}
    payload = torch.load(path / "model.pt", weights_only=True)
    payload["optimizer"] = {"state": named, "param_groups": [{"params": list(named), "lr": 1e-2}]}
    payload["generator"] = {"model." + k: v for k, v in payload["generator"].items()}
    other = tmp_path / "ref"
    from solarwm_b200.checkpoint import CheckpointTransaction

    with CheckpointTransaction(other / "checkpoint_model_000003") as tx:
        torch.save(payload, tx.path / "model.pt")
        tx.commit(step=3, contract=_contract(), required_components=["model.pt"], metadata={})
    m = WanDiT(_cfg(), device="cpu", dtype=torch.float32, seed=4)
    m.ensure_grads()
    opt = FlatAdamW(m.units(), lr=1e-2, ema_decay=0.5)
    ckpt.load_checkpoint(other / "checkpoint_model_000003", model=m, optimizer=opt, scheduler=_Sched(), mode="full_resume",
                         expected=_contract())
    assert opt.step_count == 3
    mine = opt.state_dict()
    idx2 = {id(u): i for i, u in enumerate(opt.units)}
    for n, p in m.named_parameters():                      # (the padding between parameters carries no state)
        slot = p.flat_unit.slots[p.flat_name]
        a = mine["units"][idx2[id(p.flat_unit)]]["v" if slot.is_vector else "m"]
        b = full["units"][idx2[id(p.flat_unit)]]["v" if slot.is_vector else "m"]
        for field in ("exp_avg", "exp_avg_sq", "ema"):
            lo, hi = slot.offset, slot.offset + slot.numel
            assert torch.allclose(a[field][lo:hi], b[field][lo:hi]), (n, field)
    bad = dict(payload, optimizer={"state": named, "param_groups": [{"params": list(named)[1:]}]})
    with pytest.raises(CheckpointError):
        ckpt.named_optimizer_moments(bad["optimizer"])
