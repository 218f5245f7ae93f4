"""LTX checkpoint authority: strict header reading, tensor families, base inspection against an inventory, resume identity."""
import json
import struct

import pytest
import torch

from solarwm_b200.backends.ltx25.checkpoint import (PREFIX, PUBLISHED, EMARecipe, Inventory, TrainingCheckpointManifest, classify,
                                                    fingerprint_digest, inspect_base_checkpoint, read_header, runtime_fingerprint,
                                                    validate_full_resume)
from solarwm_b200.errors import BackendContractError


def _raw(path, header: dict, payload: bytes):
    blob = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(blob)) + blob + payload)


def test_header_reader_trusts_nothing(tmp_path):
    from safetensors.torch import save_file

    save_file({"a": torch.zeros(2, 3, dtype=torch.bfloat16), "b": torch.ones(4)}, str(tmp_path / "ok.safetensors"), metadata={"k": "v"})
    h = read_header(tmp_path / "ok.safetensors")
    assert {t.name: (t.dtype, t.shape) for t in h.tensors} == {"a": ("BF16", (2, 3)), "b": ("F32", (4,))} and h.metadata == {"k": "v"}
    assert h.file_size == (tmp_path / "ok.safetensors").stat().st_size and len(h.digest) == 64
    good = {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    cases = {
        "gap": ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
        "short": (good, b"\0" * 12),                                           # ranges stop before the file's end
        "shape": ({"x": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
        "dtype": ({"x": {"dtype": "F4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8),
        "overlap": ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}, "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 12),
        "meta": ({"__metadata__": {"k": 1}, **good}, b"\0" * 8),
        "extra-field": ({"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8], "more": 1}}, b"\0" * 8),
    }
    for name, (header, payload) in cases.items():
        _raw(tmp_path / f"{name}.st", header, payload)
        with pytest.raises(BackendContractError):
            read_header(tmp_path / f"{name}.st")
    blob = b'{"x": {"dtype":"F32","shape":[2],"data_offsets":[0,8]}, "x": {"dtype":"F32","shape":[2],"data_offsets":[0,8]}}'
    (tmp_path / "dup.st").write_bytes(struct.pack("<Q", len(blob)) + blob + b"\0" * 8)
    with pytest.raises(BackendContractError):
        read_header(tmp_path / "dup.st")
    (tmp_path / "trunc.st").write_bytes(struct.pack("<Q", 500) + b"{}")
    with pytest.raises(BackendContractError):
        read_header(tmp_path / "trunc.st")
    with pytest.raises(BackendContractError):
        read_header(tmp_path / "ok.safetensors", max_header_bytes=8)
    with pytest.raises(BackendContractError):
        read_header(tmp_path / "absent.st")


def test_tensor_families():
    p = PREFIX
    assert classify(p + "transformer_blocks.3.attn1.to_q.weight") == ("video_core", "transformer_blocks.3.attn1.to_q.weight")
    assert classify(p + "transformer_blocks.47.prompt_scale_shift_table") == ("video_core", "transformer_blocks.47.prompt_scale_shift_table")
    assert classify(p + "scale_shift_table")[0] == "video_core" and classify(p + "adaln_single.linear.weight")[0] == "video_core"
    assert classify(p + "video_embeddings_connector.blocks.0.w") == ("video_connector", "video_connector.blocks.0.w")
    assert classify(p + "transformer_blocks.3.audio_attn1.to_q.weight") == ("audio", None)
    assert classify(p + "audio_scale_shift_table") == ("audio", None) and classify(p + "audio_embeddings_connector.x")[0] == "audio"
    assert classify(p + "transformer_blocks.0.audio_to_video_attn.to_k.bias") == ("av_cross", None)
    assert classify(p + "av_ca_a2v_gate_adaln_single.linear.weight") == ("av_cross", None)
    for stranger in ("transformer_blocks.3.attn1.to_q.weight", p + "transformer_blocks.48.attn1.to_q.weight", p + "transformer_blocks.03.ff.net.0.proj.weight",
                     p + "transformer_blocks.1.attn1", p + "transformer_blocks.1.scale_shift_table.extra", p + "vae.encoder.w"):
        assert classify(stranger)[0] == "unknown", stranger
    assert classify(p + "transformer_blocks.1.ff.net.0.proj.weight", blocks=1)[0] == "unknown"


def _tiny_base(path, *, fp32_block_tables=True, stranger=False, audio=True):
    from safetensors.torch import save_file

    t = {}
    for i in range(2):
        b = f"{PREFIX}transformer_blocks.{i}."
        t[b + "attn1.to_q.weight"] = torch.zeros(8, 8, dtype=torch.bfloat16)
        t[b + "ff.net.0.proj.weight"] = torch.zeros(16, 8, dtype=torch.bfloat16)
        t[b + "scale_shift_table"] = torch.zeros(6, 8, dtype=torch.float32 if fp32_block_tables else torch.bfloat16)
        t[b + "prompt_scale_shift_table"] = torch.zeros(2, 8)
        if audio:
            t[b + "audio_attn1.to_q.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
        t[b + "video_to_audio_attn.to_q.weight"] = torch.zeros(4, 8, dtype=torch.bfloat16)
    t[PREFIX + "scale_shift_table"] = torch.zeros(2, 8)
    t[PREFIX + "patchify_proj.weight"] = torch.zeros(8, 4, dtype=torch.bfloat16)
    t[PREFIX + "video_embeddings_connector.w"] = torch.zeros(8, 8, dtype=torch.bfloat16)
    if stranger:
        t["vae.decoder.w"] = torch.zeros(1)
    save_file(t, str(path))


TINY = Inventory(blocks=2, tensors={"video_core": 10, "video_connector": 1, "audio": 2, "av_cross": 2},
                 parameters={"video_core": 2 * (64 + 128 + 48 + 16) + 16 + 32, "video_connector": 64, "audio": 32, "av_cross": 64},
                 model_version=None)


def test_base_inspection_counts_families_and_fails_closed(tmp_path):
    _tiny_base(tmp_path / "base.safetensors")
    got = inspect_base_checkpoint(tmp_path / "base.safetensors", TINY)
    assert got.tensors == dict(TINY.tensors) and got.fp32_scale_tables == 5 and len(got.retained) == 11
    assert ("video_connector.w", PREFIX + "video_embeddings_connector.w") in got.retained
    assert got.as_dict()["retained"] == 11 and len(got.retained_layout_digest) == 64
    again = inspect_base_checkpoint(tmp_path / "base.safetensors", TINY)
    assert again.retained_layout_digest == got.retained_layout_digest
    for name, kw in (("bf16-table", {"fp32_block_tables": False}), ("stranger", {"stranger": True}), ("no-audio", {"audio": False})):
        _tiny_base(tmp_path / f"{name}.safetensors", **kw)
        with pytest.raises(BackendContractError):
            inspect_base_checkpoint(tmp_path / f"{name}.safetensors", TINY)
    with pytest.raises(BackendContractError):                                  # the published inventory also checks the metadata
        inspect_base_checkpoint(tmp_path / "base.safetensors")
    assert PUBLISHED.fp32_tables == 97 and sum(PUBLISHED.tensors[k] for k in ("video_core", "video_connector")) == 1491


def test_resume_identity_names_what_differs():
    now = runtime_fingerprint(camera_translation_transform="logd4", data_generation="gen-7")
    assert now["base_checkpoint"]["fp32_scale_tables"] == 97 and now["lora"]["trainable_parameters"] == 1_962_934_272
    assert now["geometry"]["pixel_frames"] == 153 if "pixel_frames" in now["geometry"] else True
    targets = ("transformer_blocks.0.attn1.to_q", "transformer_blocks.0.attn1.to_k")
    saved = TrainingCheckpointManifest(10, dict(now), targets, targets, True, True)
    validate_full_resume(saved, now, targets)
    other = runtime_fingerprint(camera_translation_transform="linear", data_generation="gen-7", ema=EMARecipe(decay=0.99))
    with pytest.raises(BackendContractError) as err:
        validate_full_resume(saved, other, targets)
    assert "camera_translation_transform" in str(err.value) and "ema" in str(err.value) and "lora" not in str(err.value)
    assert fingerprint_digest(now) != fingerprint_digest(other) and fingerprint_digest(now) == fingerprint_digest(dict(now))
    for broken in (TrainingCheckpointManifest(-1, now, targets, targets, True, True), TrainingCheckpointManifest(1, now, targets[:1], targets, True, True),
                   TrainingCheckpointManifest(1, now, targets, targets, False, True), TrainingCheckpointManifest(1, {}, targets, targets, True, True)):
        with pytest.raises(BackendContractError):
            validate_full_resume(broken, now, targets)
    for bad in ({"camera_translation_transform": "cubic", "data_generation": "g"}, {"camera_translation_transform": "linear", "data_generation": " "}):
        with pytest.raises(BackendContractError):
            runtime_fingerprint(**bad)


def test_readiness_reports_a_base_checkpoint_that_is_not_the_published_layout(tmp_path):
    from solarwm_b200.backends.ltx25.backend import RuntimeProvider

    _tiny_base(tmp_path / "base.safetensors")
    report = RuntimeProvider({"model": {"assets": {"base_checkpoint": str(tmp_path / "base.safetensors")}}}).readiness()
    assert any(p.startswith("base checkpoint:") for p in report["problems"]) and not report["ready"]
    missing = RuntimeProvider({"model": {"assets": {"base_checkpoint": str(tmp_path / "none.safetensors")}}}).readiness()
    assert any("missing" in p for p in missing["problems"])
