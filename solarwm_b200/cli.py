"""``solar`` / ``solarwm`` command line.

    solar train|infer|preencode --config FILE [--set a.b=YAML ...]
    solar infer ... [--memory | --no-memory] [--memory-lora PATH]
    solar config resolve --config FILE [--set ...] [--output FILE]
    solar config routes
    solar data inspect --index FILE
    solar data plan --config FILE [--epoch N] [--limit N]
    solar data warm-cache --config FILE
    solar data materialize-wan153f --train-index F --test-index F --train-window-index F --test-window-index F --output F
    solar environment probe
    solar publish-validation (--source DIR | --run-dir DIR [--node-rank I --num-nodes N]) --destination URI

``train/infer/preencode`` resolve the config, reject inline secrets, check that the config's action
matches the command, validate the route, load the backend lazily, let it validate its own section
contracts, write ``resolved-config.json`` and ``launch-manifest.json`` (rank 0), dispatch, and write
``run-result.json`` (schema ``solarwm.run-result.v1``).  Expected failures (``SolarWMError``,
``OSError``, ``ValueError``) exit with code 2 (reference: solar/cli.py:47-446).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import Sequence

from .config.loader import canonical_json, load_config
from .config.routes import supported_routes, validate_route
from .errors import ConfigurationError, SolarWMError

RESULT_SCHEMA = "solarwm.run-result.v1"


def _add_config_args(p):
    p.add_argument("--config", required=True)
    p.add_argument("--set", dest="overrides", action="append", default=[], metavar="KEY=VALUE")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="solar", description="Blackwell-native video world-model framework")
    sub = ap.add_subparsers(dest="command", required=True)
    for name in ("train", "infer", "preencode"):
        p = sub.add_parser(name)
        _add_config_args(p)
        if name == "infer":
            g = p.add_mutually_exclusive_group()
            g.add_argument("--memory", dest="memory", action="store_true", default=None)
            g.add_argument("--no-memory", dest="memory", action="store_false")
            p.add_argument("--memory-lora", default=None)
    cfg = sub.add_parser("config").add_subparsers(dest="config_command", required=True)
    r = cfg.add_parser("resolve")
    _add_config_args(r)
    r.add_argument("--output", default=None)
    cfg.add_parser("routes")
    data = sub.add_parser("data").add_subparsers(dest="data_command", required=True)
    i = data.add_parser("inspect")
    i.add_argument("--index", required=True)
    pl = data.add_parser("plan")
    _add_config_args(pl)
    pl.add_argument("--epoch", type=int, default=0)
    pl.add_argument("--limit", type=int, default=16)
    w = data.add_parser("warm-cache")
    _add_config_args(w)
    mw = data.add_parser("materialize-wan153f", help="join raw Wan 153-frame sources to the released fixed-window indexes")
    for flag in ("--train-index", "--test-index", "--train-window-index", "--test-window-index", "--output"):
        mw.add_argument(flag, required=True, type=Path)
    env = sub.add_parser("environment").add_subparsers(dest="environment_command", required=True)
    env.add_parser("probe")
    rd = env.add_parser("readiness", help="dependencies, assets, weights, indexes and device a configuration needs")
    _add_config_args(rd)
    rd.add_argument("--require-cuda", action="store_true")
    pub = sub.add_parser("publish-validation")
    pub.add_argument("--source", help="one pass directory (or a folder of them) to upload as it is")
    pub.add_argument("--run-dir", help="a run directory: publish the comparison views under <run-dir>/validation through the store protocol")
    pub.add_argument("--destination", required=True)
    pub.add_argument("--node-rank", type=int, default=int(os.environ.get("NODE_RANK", "0")))
    pub.add_argument("--num-nodes", type=int, default=int(os.environ.get("NUM_NODES", "1")))
    return ap


def _rank() -> int:
    return int(os.environ.get("RANK", "0"))


def _write_json(path: Path, payload) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(f".{path.name}.{os.getpid()}.tmp")
    tmp.write_bytes(canonical_json(payload))
    os.replace(tmp, path)


def run_backend(args) -> int:
    from .registry import load_backend
    from .runtime.output_layout import output_root
    from .runtime.provenance import build_launch_manifest, reject_inline_secrets

    resolved = load_config(args.config, args.overrides)
    values = resolved.mutable_copy()
    reject_inline_secrets(values)
    action = str(values.get("action", "")).lower()
    if action != args.command:
        raise ConfigurationError(f"config action {action!r} does not match command {args.command!r}")
    route = validate_route(values)
    if args.command == "infer":
        inference = values.setdefault("inference", {})
        if getattr(args, "memory", None) is not None:
            inference["memory"] = bool(args.memory)
        if getattr(args, "memory_lora", None):
            inference["memory_lora"] = str(args.memory_lora)
    backend = load_backend(route.family)
    backend.validate_config(values)
    root = output_root(values)
    started = time.time()
    if _rank() == 0:
        resolved.write_json(root / "resolved-config.json")
        _write_json(root / "launch-manifest.json",
                    build_launch_manifest(resolved=resolved, route=route, command=args.command))
    report = getattr(backend, args.command)(values)
    if _rank() == 0:
        _write_json(root / "run-result.json", {
            "schema": RESULT_SCHEMA, "command": args.command, "route": route.key, "name": values.get("name"),
            "resolved_digest": resolved.resolved_digest, "seconds": time.time() - started,
            "report": dict(report or {})})
    return 0


def config_command(args) -> int:
    if args.config_command == "routes":
        for route in supported_routes():
            print(route.key)
        return 0
    resolved = load_config(args.config, args.overrides)
    if args.output:
        resolved.write_json(args.output)
    else:
        sys.stdout.write(canonical_json(resolved.values).decode())
    print(f"source_digest={resolved.source_digest} resolved_digest={resolved.resolved_digest}", file=sys.stderr)
    return 0


def data_command(args) -> int:
    from .data import index as index_mod

    if args.data_command == "inspect":
        inv = index_mod.inventory(args.index)
        print(json.dumps(inv.__dict__, sort_keys=True))
        return 0
    if args.data_command == "materialize-wan153f":
        from .backends.wan22.windows import write_window_index

        summary = write_window_index(args.train_index, args.test_index, args.train_window_index,
                                     args.test_window_index, args.output)
        print(json.dumps(summary.as_dict(), sort_keys=True))
        return 0
    resolved = load_config(args.config, args.overrides)
    data = resolved.values["data"]
    if not data.get("index"):
        raise ConfigurationError("this command reads the corpus index: set data.index (synthetic runs have no plan)")
    rows = index_mod.read_index(data["index"])
    if args.data_command == "warm-cache":
        from .data.prefetch import warm_cache
        from .data.transport import resolver_from_config

        done = warm_cache(resolver_from_config(data), rows)
        print(json.dumps({"shards": done.shards, "bytes": done.bytes, "seconds": round(done.seconds, 3)}))
        return 0
    from .data.sampling import CanonicalSampler, ReaderIdentity, SamplingConfig, plan_fingerprint

    cfg = SamplingConfig(seed=int(data.get("seed", 0)), pixel_frames=int(data["pixel_frames"]),
                         random_start=bool(data.get("random_start", True)),
                         shuffle_buffer=int(data.get("shuffle_buffer", 4096)))
    sampler = CanonicalSampler(rows, cfg, ReaderIdentity(0, 1))
    plans = []
    for plan in sampler.iter_epoch(args.epoch):
        plans.append(plan)
        if len(plans) >= args.limit:
            break
    for p in plans:
        print(json.dumps({"sample_id": p.sample_id, "shard": p.shard, "start_frame": p.start_frame}))
    print(json.dumps({"plan_fingerprint": plan_fingerprint(plans)}))
    return 0


def environment_command(args) -> int:
    if args.environment_command == "readiness":
        from .registry import load_backend

        resolved = load_config(args.config, args.overrides)
        backend = load_backend(str(resolved.values["model"]["family"]))
        if not hasattr(backend, "readiness"):
            raise ConfigurationError(f"the {resolved.values['model']['family']} backend has no readiness report")
        report = backend.readiness(resolved.values, require_cuda=bool(args.require_cuda))
        report = report.as_dict() if hasattr(report, "as_dict") else dict(report)
        print(json.dumps(report, sort_keys=True, indent=1))
        return 0 if report.get("ready") else 3
    from .runtime.env_probe import probe_python_runtime

    print(json.dumps(probe_python_runtime(), sort_keys=True, indent=1))
    return 0


def publish_validation_command(args) -> int:
    from .runtime.validation_publish import ValidationPublisher, publish_validation

    if args.run_dir:
        from .runtime.object_store import store_for

        report = ValidationPublisher(args.run_dir, store_for(args.destination), node=args.node_rank, nodes=args.num_nodes).scan()
        print(json.dumps(report, sort_keys=True))
        return 3 if report["errors"] else 0
    if not args.source:
        raise ValueError("publish-validation needs --source or --run-dir")
    print(json.dumps(publish_validation(args.source, args.destination, node=args.node_rank, nodes=args.num_nodes), sort_keys=True))
    return 0


def main(argv: Sequence[str] = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command in ("train", "infer", "preencode"):
            return run_backend(args)
        if args.command == "config":
            return config_command(args)
        if args.command == "data":
            return data_command(args)
        if args.command == "environment":
            return environment_command(args)
        if args.command == "publish-validation":
            return publish_validation_command(args)
    except (SolarWMError, OSError, ValueError) as exc:
        print(f"solar: error: {exc}", file=sys.stderr)
        return 2
    return 1


if __name__ == "__main__":
    raise SystemExit(main())
