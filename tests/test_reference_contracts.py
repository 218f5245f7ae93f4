"""Contracts shared with the reference, checked against the UNMODIFIED reference package when it is installed under
``baseline/_ref`` (skipped otherwise): sample-plan sequences and fingerprints, config digests and canonical JSON,
checkpoint directories that each side can verify, window start rules, EMA arithmetic.  These are the oracles that
let the modules behind them be written independently of the reference's code."""
import json
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


@pytest.fixture(scope="module")
def ref():
    if not (REF / "solar").exists():
        pytest.skip("reference package not installed under baseline/_ref")
    for p in (str(ROOT / "baseline" / "shims"), str(REF)):
        if p not in sys.path:
            sys.path.insert(0, p)
    import importlib

    class Ref:
        sampling = importlib.import_module("solar.data.sampling")
        index = importlib.import_module("solar.data.index")
        loader = importlib.import_module("solar.config.loader")
        store = importlib.import_module("solar.checkpoint.store")
        ema = importlib.import_module("solar.training.ema")
        windows = importlib.import_module("solar.backends.wan22.windows")

    return Ref


def _rows():
    rows = []
    for i in range(23):
        shard = f"ds{'AB'[i % 2]}/shards/part-{i // 4:03d}.tar"
        rows.append({"sample_id": f"ds/clip-{i:03d}", "key": f"clip{i:03d}", "shard": shard, "epoch_repeats": 1 + (i % 3 == 0),
                     "num_frames": 200 + 7 * i, "fps": 24.0 if i % 2 else 30.0, "start_frame": i % 5})
    return rows


SAMPLER_CASES = [
    dict(cfg=dict(seed=3, pixel_frames=81), ident=dict(rank=0, world_size=1)),
    dict(cfg=dict(seed=3, pixel_frames=81, shuffle_buffer=1), ident=dict(rank=1, world_size=2)),
    dict(cfg=dict(seed=9, pixel_frames=81, shuffle_buffer=4), ident=dict(rank=2, world_size=3, worker_id=1, num_workers=2)),
    dict(cfg=dict(seed=5, pixel_frames=81, random_start=False, fixed_start_from_index=True), ident=dict(rank=0, world_size=2)),
    dict(cfg=dict(seed=5, pixel_frames=81, random_start=False), ident=dict(rank=1, world_size=2)),
    dict(cfg=dict(seed=1, pixel_frames=81, clip_seconds=5.0, output_fps=16.0), ident=dict(rank=0, world_size=1)),
    dict(cfg=dict(seed=7, pixel_frames=81, partition_mode="node_shard", shuffle_buffer=2),
         ident=dict(rank=1, world_size=4, node_id=0, node_count=2, local_rank=1, local_world_size=2)),
    dict(cfg=dict(seed=7, pixel_frames=81, partition_mode="node_shard", shard_partition_scope="collection_relative"),
         ident=dict(rank=2, world_size=4, node_id=1, node_count=2, local_rank=0, local_world_size=2)),
]


@pytest.mark.parametrize("case", SAMPLER_CASES)
def test_sample_plans_match_the_reference(ref, case):
    from solarwm_b200.data import index as our_index, sampling as ours

    theirs = ref.sampling
    r_rows = [ref.index.IndexRow.from_mapping(i, r) for i, r in enumerate(_rows())]
    o_rows = [our_index.IndexRow.from_mapping(i, r) for i, r in enumerate(_rows())]
    a = ours.CanonicalSampler(o_rows, ours.SamplingConfig(**case["cfg"]), ours.ReaderIdentity(**case["ident"]))
    b = theirs.CanonicalSampler(r_rows, theirs.SamplingConfig(**case["cfg"]), theirs.ReaderIdentity(**case["ident"]))
    for epoch in (0, 1, 4):
        pa, pb = list(a.iter_epoch(epoch)), list(b.iter_epoch(epoch))
        assert [(p.sample_id, p.repeat_ordinal, p.start_frame, tuple(p.source_frame_indices)) for p in pa] == \
               [(p.sample_id, p.repeat_ordinal, p.start_frame, tuple(p.source_frame_indices)) for p in pb]
        assert ours.plan_fingerprint(pa) == theirs.plan_fingerprint(pb)


CONFIG = """
schema: solarwm.run.v1
action: train
name: parity
model: {family: wan2.2-ti2v-5b, camera_translation_transform: linear, note: "${PARITY_ROOT}/x"}
data: {pixel_frames: 81, root: "${PARITY_ROOT}", ratios: [0.5, 1, 2.25e-3], flag: true, nothing: null}
train: {stage: stage0p5, causal_mode: bidirectional, objective: flow_matching, unicode: "café"}
runtime: {output_dir: /tmp/x}
"""


def test_config_digests_and_canonical_json_match_the_reference(ref, tmp_path, monkeypatch):
    from solarwm_b200.config import loader as ours

    monkeypatch.setenv("PARITY_ROOT", "/corpus")
    path = tmp_path / "c.yaml"
    path.write_text(CONFIG, encoding="utf-8")
    overrides = ["train.max_steps=12", "data.nested.deep={a: [1, {b: 2}]}", "name=renamed"]
    ok = lambda values: None                                       # noqa: E731 - route tables are checked elsewhere
    a = ours.load_config(path, overrides, route_validator=ok)
    b = ref.loader.load_config(path, overrides, route_validator=ok)
    assert a.values == b.values
    assert (a.source_digest, a.resolved_digest) == (b.source_digest, b.resolved_digest)
    assert ours.canonical_json(a.values) == ref.loader.canonical_json(b.values)
    a.write_json(tmp_path / "ours.json")
    b.write_json(tmp_path / "theirs.json")
    assert (tmp_path / "ours.json").read_bytes() == (tmp_path / "theirs.json").read_bytes()
    for bad in ("schema: other", "name: ''", "bogus: 1"):
        text = CONFIG.replace("schema: solarwm.run.v1", bad) if bad.startswith("schema") else CONFIG + bad + "\n" \
            if bad.startswith("bogus") else CONFIG.replace("name: parity", bad)
        path.write_text(text, encoding="utf-8")
        for mod, err in ((ours, None), (ref.loader, None)):
            with pytest.raises(Exception):
                mod.load_config(path, route_validator=ok)


def test_checkpoint_directories_verify_on_both_sides(ref, tmp_path):
    from solarwm_b200.checkpoint import store as ours

    kw = dict(family="wan22_ti2v_5b", stage="stage0p5", causal_mode="bidirectional", objective="flow_matching",
              objective_variant="", camera_translation_transform="linear", parameterization="full", sp_size=2,
              data_generation="index", extras={"timestep_shift": 5.0})
    for writer, reader, name in ((ours, ref.store, "ours"), (ref.store, ours, "theirs")):
        target = tmp_path / name / "checkpoint_model_000007"
        target.parent.mkdir(parents=True)
        with writer.CheckpointTransaction(target) as tx:
            (tx.path / "model.pt").write_bytes(b"weights" * 100)
            (tx.path / "extra").mkdir()
            (tx.path / "extra" / "notes.txt").write_text("hello")
            tx.commit(step=7, contract=writer.CheckpointContract(**kw), required_components=["model.pt"],
                      metadata={"ema_num_updates": 7})
        seen = reader.verify_checkpoint(target)
        assert seen.step == 7 and seen.contract.as_dict() == writer.CheckpointContract(**kw).as_dict()
        mine = writer.verify_checkpoint(target)
        assert mine.manifest_digest == seen.manifest_digest
        reader.assert_resume_compatible(reader.CheckpointContract(**kw), seen.contract)
        with pytest.raises(Exception):
            reader.assert_resume_compatible(reader.CheckpointContract(**{**kw, "sp_size": 4}), seen.contract)
    a = json.loads((tmp_path / "ours" / "checkpoint_model_000007" / "checkpoint-manifest.json").read_text())
    b = json.loads((tmp_path / "theirs" / "checkpoint_model_000007" / "checkpoint-manifest.json").read_text())
    assert a.keys() == b.keys() and a["schema"] == b["schema"] == "solarwm.checkpoint.v2"
    assert a["files"] == b["files"] and a["contract"] == b["contract"]
    # a damaged component is caught by either verifier
    victim = tmp_path / "ours" / "checkpoint_model_000007" / "model.pt"
    victim.write_bytes(b"short")
    for mod in (ours, ref.store):
        with pytest.raises(Exception):
            mod.verify_checkpoint(victim.parent)


def test_window_rules_match_the_reference(ref):
    from solarwm_b200.backends.wan22 import windows as ours

    for n in range(81, 400, 13):
        count = ours.window_count_81f(n)
        assert count == ref.windows.expected_81f_window_count(n)
        for i in range(count):
            meta = {"window_index": i, "window_count": count}
            assert ours.window_start_81f(meta, n) == ref.windows.expected_81f_window_start(meta, n)
    for n in range(153, 900, 37):
        for ds, count in (("miradata", 6), ("re10k", 1)):
            for i in range(count):
                meta = {"source_sample_id": f"{ds}/c{n}", "source_dataset": ds, "window_index": i, "window_count": count}
                assert ours.window_start_153f(meta, n) == ref.windows.expected_153f_window_start(meta, n)


def test_ema_matches_the_reference(ref):
    from solarwm_b200.engine import ema as ours

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Linear(7, 3))
    net[1].bias.requires_grad_(False)
    for trainable_only in (False, True):
        a = ours.ShardedEMA(net, decay=0.9, device="cpu", dtype=torch.float32, trainable_only=trainable_only)
        b = ref.ema.ShardedEMA(net, decay=0.9, device="cpu", dtype=torch.float32, trainable_only=trainable_only)
        for step in range(4):
            with torch.no_grad():
                for p in net.parameters():
                    p.add_(torch.randn_like(p) * 0.1)
            d = ours.ema_decay_for_step(target_decay=0.9, global_step=step, warmup_steps=2)
            assert d == ref.ema.ema_decay_for_step(target_decay=0.9, global_step=step, warmup_steps=2)
            a.update(net, decay=d)
            b.update(net, decay=d)
        sa, sb = a.state_dict(), b.state_dict()
        assert sa.keys() == sb.keys() and all(torch.allclose(sa[k], sb[k], atol=1e-7) for k in sa)
        assert a.num_updates == b.num_updates == 4
        b.load_state_dict(sa, num_updates=4)                       # state dicts interchange
        live = {n: p.detach().clone() for n, p in net.named_parameters()}
        with a.swapped_into(net):
            assert all(torch.allclose(p, sa[n]) for n, p in net.named_parameters() if n in sa)
        assert all(torch.equal(p, live[n]) for n, p in net.named_parameters())
