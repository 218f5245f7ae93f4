"""The release-recipe pins of the Wan families (``metadata.contract: release``)."""
import copy

import pytest

from solarwm_b200.backends.wan22.contracts import (RELEASE_PROFILES, pixel_to_latent_frames, release_recipe_problems,
                                                   validate_release_recipe, whole_frame_splits)
from solarwm_b200.errors import BackendContractError


def recipe(family="wan22_ti2v_5b", stage="stage0p5", pixel_frames=81, **over):
    prof = RELEASE_PROFILES[family]
    latent = 1 + (pixel_frames - 1) // 4
    sp = prof.sequence_parallel_size
    causal = {"stage0p5": "bidirectional", "stage1": "teacher_forcing", "stage2": "self_gradient_forcing"}[stage]
    cfg = {
        "schema": "solarwm.run.v1", "action": "train", "name": "recipe", "metadata": {"contract": "release"},
        "model": {"family": family, "name": prof.model_name, "timestep_shift": prof.timestep_shift,
                  "latent_channels": prof.latent_channels, "frame_sequence_length": prof.frame_sequence_length,
                  "camera_attention_mode": "fused_prope", "camera_translation_transform": "linear",
                  "causal": stage != "stage0p5", "base_path": "/models/wan", "num_output_frames": latent,
                  "num_frame_per_block": 3, "local_attn_size": latent if family == "wan22_i2v_a14b" else 21,
                  "assets": {"transformer_config": "builtin", "transformer_weights": "dit", "text_encoder": "t5",
                             "tokenizer": "tok", "vae": "vae.pth"}},
        "data": {"encoding": "online", "pixel_frames": pixel_frames, "latent_frames": latent, "height": prof.height,
                 "width": prof.width, "max_rel_translation": 20.0, "max_camera_abs": 20.0, "streaming_index": True,
                 "random_start": pixel_frames == 81, "train_index": "idx/train.jsonl.gz", "test_index": "idx/test.jsonl.gz",
                 "partition_mode": "node_shard", "num_workers": 4, "camera_array_key": "c2w",
                 "transport": {"kind": "local", "root": "/data"}},
        "distributed": {"world_size": 8, "sequence_parallel_size": sp, "sample_sharding": "logical_dp",
                        "rng_scope": "logical_dp"},
        "train": {"stage": stage, "causal_mode": causal, "objective": "flow_matching", "micro_batch_size": 1, "grad_accum": 2,
                  "global_batch_size": 8 // sp * 2, "timestep_mode": "uniform_per_video" if stage == "stage0p5" else "per_block",
                  "num_train_timesteps": 1000, "i2v_image_condition_dropout": 0.1,
                  "optimizer": {"lr": 5.0e-5, "betas": [0.9, 0.95]},
                  "fsdp": {"strategy": prof.fsdp_strategy, "param_dtype": "bfloat16", "reduce_dtype": "float32"},
                  "ema": {"enabled": True, "device": "cuda", "dtype": "float32", "sharded": True, "decay": 0.9999,
                          "start_step": 0}},
        "checkpoint": {"mode": "none"}, "runtime": {"output_dir": "/out"},
    }
    if family == "wan22_i2v_a14b":
        splits = list(whole_frame_splits(latent, sp))
        cfg["distributed"].update(sequence_layout="whole_frame_uneven", sp_frame_splits=splits,
                                  sp_token_splits=[n * prof.frame_sequence_length for n in splits])
    for dotted, value in over.items():
        node = cfg
        parts = dotted.split("__")
        for part in parts[:-1]:
            node = node[part]
        node[parts[-1]] = value
    return cfg


def test_conforming_recipes_pass_for_both_families():
    assert release_recipe_problems(recipe(), "wan22_ti2v_5b") == []
    a14b = recipe("wan22_i2v_a14b")
    assert a14b["distributed"]["sp_frame_splits"] == [11, 10] and a14b["distributed"]["sp_token_splits"] == [17160, 15600]
    assert release_recipe_problems(a14b, "wan22_i2v_a14b") == []
    assert validate_release_recipe(a14b, "wan22_i2v_a14b").key == "wan22_i2v_a14b:stage0p5:bidirectional:flow_matching"
    long = recipe("wan22_i2v_a14b", pixel_frames=153, data__random_start=False, checkpoint__mode="weights_only",
                  checkpoint__path="/ckpt", checkpoint__source_step=2000, checkpoint__weights=["live", "ema"],
                  checkpoint__source_contract={"stage": "stage0p5", "objective": "flow_matching"})
    assert long["distributed"]["sp_frame_splits"] == [20, 19]
    assert release_recipe_problems(long, "wan22_i2v_a14b") == []
    assert pixel_to_latent_frames(153) == 39
    with pytest.raises(BackendContractError):
        pixel_to_latent_frames(82)


@pytest.mark.parametrize("field,value,needle", [
    ("model__name", "Wan2.2", "model.name"),
    ("model__timestep_shift", 3.0, "model.timestep_shift"),
    ("model__causal", True, "model.causal"),
    ("model__local_attn_size", 12, "model.local_attn_size"),
    ("data__height", 720, "data.height"),
    ("data__latent_frames", 20, "data.latent_frames"),
    ("data__random_start", False, "data.random_start"),
    ("data__train_index", "/abs/train.jsonl", "data.train_index"),
    ("data__max_camera_abs", 10.0, "data.max_camera_abs"),
    ("distributed__sequence_parallel_size", 2, "sequence_parallel_size"),
    ("distributed__rng_scope", "raw_rank", "distributed.rng_scope"),
    ("train__global_batch_size", 7, "global_batch_size"),
    ("train__optimizer__lr", 1e-4, "train.optimizer.lr"),
    ("train__optimizer__betas", [0.9, 0.999], "train.optimizer.betas"),
    ("train__ema__decay", 0.99, "train.ema.decay"),
    ("train__ema__sharded", False, "train.ema.sharded"),
    ("train__fsdp__strategy", "FULL_SHARD", "train.fsdp.strategy"),
    ("train__num_train_timesteps", True, "train.num_train_timesteps"),
    ("checkpoint__mode", "stage2_roles", None),
])
def test_departures_are_named(field, value, needle):
    cfg = recipe(**{field: value})
    problems = release_recipe_problems(cfg, "wan22_ti2v_5b")
    if needle is None:
        return                                              # (a mode that is legal for another stage: no single field to name)
    assert any(needle in p for p in problems), problems
    with pytest.raises(BackendContractError, match="release recipe"):
        validate_release_recipe(cfg, "wan22_ti2v_5b")


def test_stage_specific_pins_and_sp_override():
    s2 = recipe(stage="stage2", train__optimizer={"lr": 2.0e-6, "betas": [0.0, 0.999]}, train__i2v_image_condition_dropout=0.0,
                train__ema={"enabled": True, "device": "cuda", "dtype": "float32", "sharded": True, "decay": 0.99, "start_step": 39},
                checkpoint__mode="stage2_roles", data__random_start=True)
    assert release_recipe_problems(s2, "wan22_ti2v_5b") == []
    s2["train"]["ema"]["start_step"] = 0
    assert any("start_step" in p for p in release_recipe_problems(s2, "wan22_ti2v_5b"))
    s1 = recipe(stage="stage1", model__use_echorope=False, model__max_prior_clean_chunks=5,
                train__noise_augmentation_max_timestep=0, checkpoint__mode="weights_only", checkpoint__path="/c",
                checkpoint__weights="ema", checkpoint__source_step=10,
                checkpoint__source_contract={"stage": "stage0p5", "objective": "flow_matching"})
    assert release_recipe_problems(s1, "wan22_ti2v_5b") == []
    s1["checkpoint"]["source_contract"]["camera_translation_transform"] = "logd4"
    assert any("translation transform" in p for p in release_recipe_problems(s1, "wan22_ti2v_5b"))
    # the SP pin can be lifted: any divisor of the head count, with the frame splits recomputed
    sp8 = recipe(distributed__sequence_parallel_size=8, distributed__allow_sequence_parallel_override=True,
                 train__global_batch_size=2)
    assert release_recipe_problems(sp8, "wan22_ti2v_5b") == []
    sp5 = copy.deepcopy(sp8)
    sp5["distributed"].update(sequence_parallel_size=5, world_size=5)
    sp5["train"]["global_batch_size"] = 2
    assert any("attention heads" in p for p in release_recipe_problems(sp5, "wan22_ti2v_5b"))


def test_backend_applies_the_release_level_only_when_asked():
    from solarwm_b200.backends.wan22.backend import Wan22Backend

    cfg = recipe()
    cfg["data"]["source"] = "synthetic"
    cfg["train"]["max_steps"] = 1
    Wan22Backend("wan22_ti2v_5b").validate_config(cfg)
    cfg["model"]["name"] = "something else"
    with pytest.raises(BackendContractError, match="model.name"):
        Wan22Backend("wan22_ti2v_5b").validate_config(cfg)
    cfg["metadata"]["contract"] = "structural"
    Wan22Backend("wan22_ti2v_5b").validate_config(cfg)
