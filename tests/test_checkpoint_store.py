import json

import pytest

from solarwm_b200.checkpoint import (CheckpointContract, CheckpointTransaction, assert_resume_compatible,
                                     verify_checkpoint)
from solarwm_b200.errors import CheckpointError


def _contract(**kw):
    base = dict(family="wan22_ti2v_5b", stage="stage0p5", causal_mode="bidirectional", objective="flow_matching",
                objective_variant="", camera_translation_transform="linear", parameterization="full", sp_size=2,
                data_generation="g1")
    base.update(kw)
    return CheckpointContract(**base)


def test_transaction_commit_verify_and_layout(tmp_path):
    target = tmp_path / "checkpoint_model_000010"
    with CheckpointTransaction(target) as tx:
        assert tx.path.name.startswith(".checkpoint_model_000010.") and tx.path.name.endswith(".partial")
        (tx.path / "model.pt").write_bytes(b"x" * 100)
        (tx.path / "critic.pt").write_bytes(b"y" * 10)
        done = tx.commit(step=10, contract=_contract(), required_components=["model.pt", "critic.pt"], metadata={"a": 1})
    assert target.is_dir() and not tx.path.exists()
    manifest = json.loads((target / "checkpoint-manifest.json").read_text())
    assert manifest["schema"] == "solarwm.checkpoint.v2" and manifest["step"] == 10
    assert manifest["files"] == [{"path": "critic.pt", "size": 10}, {"path": "model.pt", "size": 100}]
    assert json.loads((target / "COMPLETE.json").read_text())["manifest_digest"] == done.manifest_digest
    v = verify_checkpoint(target)
    assert v.step == 10 and v.contract == _contract() and v.metadata == {"a": 1}


def test_missing_component_leaves_partial_and_no_target(tmp_path):
    target = tmp_path / "ck"
    with pytest.raises(CheckpointError):
        with CheckpointTransaction(target) as tx:
            (tx.path / "model.pt").write_bytes(b"x")
            tx.commit(step=1, contract=_contract(), required_components=["model.pt", "optimizer.pt"], metadata={})
    assert not target.exists() and tx.path.exists()


def test_tamper_detection_and_existing_target(tmp_path):
    target = tmp_path / "ck"
    with CheckpointTransaction(target) as tx:
        (tx.path / "model.pt").write_bytes(b"x" * 8)
        tx.commit(step=3, contract=_contract(), required_components=["model.pt"], metadata={})
    (target / "model.pt").write_bytes(b"x" * 9)
    with pytest.raises(CheckpointError, match="size differs"):
        verify_checkpoint(target)
    (target / "model.pt").write_bytes(b"x" * 8)
    m = target / "checkpoint-manifest.json"
    m.write_bytes(m.read_bytes().replace(b'"step":3', b'"step":4'))
    with pytest.raises(CheckpointError):
        verify_checkpoint(target)
    with pytest.raises(CheckpointError, match="already exists"):
        with CheckpointTransaction(target):
            pass
    (tmp_path / "nocomplete").mkdir()
    with pytest.raises(CheckpointError, match="not complete"):
        verify_checkpoint(tmp_path / "nocomplete")


def test_resume_contract_and_validation():
    assert_resume_compatible(_contract(), _contract())
    with pytest.raises(CheckpointError, match="sp_size"):
        assert_resume_compatible(_contract(), _contract(sp_size=4))
    with pytest.raises(CheckpointError):
        _contract(family="")
    with pytest.raises(CheckpointError):
        _contract(sp_size=0)


def test_safetensors_inventory_and_strict_load(tmp_path):
    import json

    import pytest
    import torch
    from safetensors.torch import save_file

    from solarwm_b200.backends.wan22.loader import ARCHITECTURES, inventory, strict_load
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.models.wan import WanConfig, WanDiT

    assert ARCHITECTURES["ti2v_5b"]["num_layers"] == 30 and ARCHITECTURES["i2v_a14b"]["dim"] == 5120
    cfg = WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=64, ffn_dim=128, num_heads=2, num_layers=2, text_dim=32,
                    text_len=8, freq_dim=32)
    src = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=1)
    state = {k: v.clone().contiguous() for k, v in src.state_dict().items()}
    names = sorted(state)
    half = len(names) // 2
    save_file({k: state[k] for k in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: state[k] for k in names[half:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {
        **{k: "model-00001-of-00002.safetensors" for k in names[:half]},
        **{k: "model-00002-of-00002.safetensors" for k in names[half:]}}}))
    inv = inventory(tmp_path)
    assert set(inv) == set(names) and inv[names[0]].dtype == "F32"
    dst = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=2)
    copied = strict_load(dst, tmp_path)
    assert sum(copied.values()) == len(names)
    assert all(torch.equal(dst.state_dict()[k], state[k]) for k in names)
    other = WanDiT(WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=64, ffn_dim=128, num_heads=2, num_layers=3,
                             text_dim=32, text_len=8, freq_dim=32), device="cpu", dtype=torch.float32)
    with pytest.raises(BackendContractError):
        strict_load(other, tmp_path)


def test_h3_released_layout_strict_mapped_load(tmp_path):
    import pytest
    import torch
    from safetensors.torch import save_file

    from solarwm_b200.backends.minimax_h3.loader import export_released_layout, plan_load, strict_load_mapped
    from solarwm_b200.backends.wan22.loader import inventory
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.models.h3 import H3DiT, h3_preset

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    src = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=1)
    released = export_released_layout(src)
    assert "transformer_blocks.0.ffn.gate_proj.weight" in released and "token_refiner.0.attn.to_out.0.weight" in released
    names = sorted(released)
    half = len(names) // 2                                  # two shards, bf16 on disk
    save_file({k: released[k].to(torch.bfloat16) for k in names[:half]}, str(tmp_path / "model-00001-of-00002.safetensors"))
    save_file({k: released[k].to(torch.bfloat16) for k in names[half:]}, str(tmp_path / "model-00002-of-00002.safetensors"))
    dst = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=2)
    lora_before = dst.blocks[0].to_q.lora_A.detach().clone()
    copied = strict_load_mapped(dst, tmp_path)
    assert sum(copied.values()) == len(names) and len(copied) == 2
    for k, v in src.state_dict().items():
        if "lora_" in k:
            continue
        assert torch.equal(dst.state_dict()[k], v.to(torch.bfloat16).to(v.dtype)), k
    assert dst.blocks[0].norm1.dtype == torch.float32 and torch.equal(dst.blocks[0].to_q.lora_A, lora_before)   # adapters untouched
    # refusals happen before any copy
    entries = dict(inventory(tmp_path))
    some = next(iter(entries.values()))
    with pytest.raises(BackendContractError, match="match no rule"):
        plan_load({**entries, "transformer_blocks.0.attn.rotary.weight": some}, dst)
    entries = dict(inventory(tmp_path))
    gone = entries.pop("transformer_blocks.1.ffn.up_proj.weight")
    with pytest.raises(BackendContractError, match="do not tile|not in the checkpoint"):
        plan_load(entries, dst)
    entries["transformer_blocks.1.ffn.up_proj.weight"] = gone._replace(shape=(3, 3))
    with pytest.raises(BackendContractError, match="do not tile"):
        plan_load(entries, dst)
    entries["transformer_blocks.1.ffn.up_proj.weight"] = gone
    entries["norm_out.weight"] = entries["norm_out.weight"]._replace(shape=(7,))
    with pytest.raises(BackendContractError, match="shape"):
        plan_load(entries, dst)


def test_release_manifest_selects_the_default_weight_role(tmp_path):
    import json

    import pytest

    from solarwm_b200.checkpoint.release import resolve_default_weights, write_release_manifest
    from solarwm_b200.errors import BackendContractError

    pkg = tmp_path / "pkg"
    pkg.mkdir()
    with pytest.raises(BackendContractError, match="readable"):
        resolve_default_weights(pkg)
    with pytest.raises(BackendContractError):
        write_release_manifest(pkg, family="wan22_ti2v_5b", stage="stage2", weight_roles=["live"], default_weights="ema")
    path = write_release_manifest(pkg, family="wan22_ti2v_5b", stage="stage2", weight_roles=["live", "ema"], default_weights="ema")
    assert resolve_default_weights(pkg) == "ema" and resolve_default_weights(pkg / "model.pt") == "ema"
    with pytest.raises(FileExistsError):
        write_release_manifest(pkg, family="x", stage="y", weight_roles=["live"], default_weights="live")
    m = json.loads(path.read_text())
    for mutate in (lambda d: d.update(schema="other"), lambda d: d["load"].update(entrypoint="sub"),
                   lambda d: d["load"].update(default_weights="teacher"), lambda d: d["identity"]["model"].update(weight_role="live")):
        bad = json.loads(json.dumps(m))
        mutate(bad)
        path.write_text(json.dumps(bad))
        with pytest.raises(BackendContractError):
            resolve_default_weights(pkg)
