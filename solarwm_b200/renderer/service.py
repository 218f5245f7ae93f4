"""Inference host of the renderer: the caches that make the fixed few-step schedule cheap.

* **Precomputed modulation**: a distilled renderer only ever sees a handful of timestep sets (one per denoise
  step: ``{text, anchor, t_k}``), so the time MLP and every block's adaLN projection are evaluated once per set
  and the per-block tables kept; the projection weights (``18 * hidden * time_embed_dim`` per block) can then be
  dropped.  An unprepared set is refused rather than served from a stale table.
* **Text cache**: the embedded + refined prompt rows are kept while the prompt tensor stays bit-identical.
* **Tile-parallel decode**: frames leave through ``models.vit_decoder.StreamingViTDecoder(distributed=True)``.

Reference behaviour: deploy/solar_renderer/reactor/solarrenderer_optimizations.py:18-110 (one-entry exact-input
cache, modulation tables, refusal of unprepared timestep sets), solarrenderer_distributed.py:10-108.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch

from ..backends.minimax_h3 import flow
from ..models.h3 import H3DiT
from . import core

TEXT_TIME, ANCHOR_TIME = 1.0, 0.999


def time_key(values: Iterable[float]) -> Tuple[float, ...]:
    """Sorted unique timesteps, rounded the way ``H3DiT.forward`` looks them up."""
    t = torch.unique(torch.tensor(list(values), dtype=torch.float32))
    return tuple(round(float(v), 6) for v in t.tolist())


def schedule_time_sets(steps: int, shift: float = flow.VIDEO_SHIFT) -> List[List[float]]:
    """The timestep sets ``core.render`` produces without pinned rows: text, anchor and the step's own time."""
    return [[TEXT_TIME, ANCHOR_TIME, float(t)] for t in flow.rollout_times(steps, shift)[:steps]]


@torch.no_grad()
def precompute_modulation(model: H3DiT, time_sets: Sequence[Sequence[float]], *, free_projection: bool = False) -> Dict:
    """Evaluate the adaLN tables of every block for each timestep set and install them on ``model``."""
    dev = model.proj_in.device
    tables = {}
    for ts in time_sets:
        key = time_key(ts)
        exact = torch.unique(torch.tensor(list(ts), dtype=torch.float32))      # the lookup key is rounded, the values are not
        temb = model.time_embed(exact.to(dev))
        tables[key] = [blk.tables(temb) for blk in model.blocks]
    model.fixed_tables = tables
    freed = 0
    if free_projection:
        for blk in model.blocks:
            freed += blk.adaln_proj.numel() * blk.adaln_proj.element_size()
            blk.adaln_proj.data = blk.adaln_proj.data.new_empty(0)
    return {"time_sets": list(tables), "adaln_weight_bytes_removed": freed,
            "table_bytes": sum(t.numel() * t.element_size() for ts in tables.values() for t in ts)}


def enable_text_cache(model: H3DiT) -> None:
    model.text_cache = {"input": None, "output": None, "hits": 0}


class RenderService:
    """``prepare`` once, then ``render`` per request on the prepared schedule."""

    def __init__(self, model: H3DiT, *, steps: int = 4, shift: float = flow.VIDEO_SHIFT, free_projection: bool = False):
        self.model, self.steps, self.shift = model, steps, shift
        self.free_projection = free_projection
        self.report: Optional[Mapping] = None

    def prepare(self) -> Mapping:
        self.report = precompute_modulation(self.model, schedule_time_sets(self.steps, self.shift),
                                            free_projection=self.free_projection)
        enable_text_cache(self.model)
        return self.report

    @torch.no_grad()
    def render(self, sample: Mapping[str, torch.Tensor], *, seed: int = 0) -> torch.Tensor:
        if self.report is None:
            raise RuntimeError("RenderService.prepare() must run before render()")
        return core.render(self.model, sample, steps=self.steps, seed=seed, shift=self.shift)


# ------------------------------------------------------------------------------------------ HTTP transport
CLIENT_PAGE = """<!doctype html>
<html lang="en"><head><meta charset="utf-8"><title>SolarRenderer</title>
<style>
 body{font:14px/1.4 system-ui,sans-serif;margin:2rem;max-width:60rem;color:#ddd;background:#181818}
 h1{font-size:1.2rem} select,input,button{font:inherit;padding:.3rem .5rem;margin-right:.5rem}
 table{border-collapse:collapse;margin-top:1rem;width:100%} td,th{border-bottom:1px solid #333;padding:.3rem .6rem;text-align:left}
 #status{margin:.6rem 0;color:#9c9} .err{color:#e88}
</style></head><body>
<h1>SolarRenderer service</h1>
<div id="status">connecting...</div>
<div><select id="sample"></select><input id="seed" type="number" min="0" value="0" size="6">
<button id="go">Render</button></div>
<table><thead><tr><th>sample</th><th>seed</th><th>latents</th><th>seconds</th><th>file</th></tr></thead><tbody id="jobs"></tbody></table>
<script>
const $ = id => document.getElementById(id);
const get = path => fetch(path).then(r => r.json());
function row(j){ const tr=document.createElement('tr');
  for (const v of [j.sample,j.seed,(j.shape||[]).join(' x '),j.seconds,j.file]){ const td=document.createElement('td'); td.textContent=v; tr.appendChild(td);} return tr; }
async function refresh(){
  const h = await get('/health');
  $('status').textContent = h.prepared ? `ready: ${h.steps} steps, ${h.time_sets.length} prepared time sets` : 'not prepared';
  const jobs = await get('/jobs'); $('jobs').replaceChildren(...jobs.slice().reverse().map(row));
}
async function start(){
  for (const s of await get('/samples')){ const o=document.createElement('option'); o.value=o.textContent=s; $('sample').appendChild(o); }
  await refresh();
}
$('go').onclick = async () => {
  $('go').disabled = true; $('status').className=''; $('status').textContent = 'rendering...';
  try {
    const r = await fetch('/render',{method:'POST',headers:{'Content-Type':'application/json'},
                                     body:JSON.stringify({sample:$('sample').value,seed:Number($('seed').value)})});
    const j = await r.json();
    if (!r.ok) { $('status').className='err'; $('status').textContent = j.error; } else await refresh();
  } finally { $('go').disabled = false; }
};
start().catch(e => { $('status').className='err'; $('status').textContent = String(e); });
</script></body></html>
"""


def make_server(service: "RenderService", samples: Mapping[str, Mapping[str, torch.Tensor]], out_dir, *,
                host: str = "127.0.0.1", port: int = 0):
    """Stdlib HTTP front of the service: ``GET /health`` (the prepare report), ``GET /samples`` (ids),
    ``POST /render {"sample": id, "seed": n}`` -> renders on the serving thread under a lock (one request on the
    device at a time), saves the latents under ``out_dir`` and answers with the file name and the latency,
    ``GET /jobs`` (history), ``GET /`` (a dependency-free browser client of these four calls).  Unknown samples and
    malformed bodies are refused with 4xx, never forwarded."""
    import json
    import threading
    import time
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
    from pathlib import Path

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    lock, jobs = threading.Lock(), []

    class Handler(BaseHTTPRequestHandler):
        def log_message(self, *a):
            return

        def _send(self, code, payload):
            body = json.dumps(payload).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path in ("/", "/index.html"):
                page = CLIENT_PAGE.encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/html; charset=utf-8")
                self.send_header("Content-Length", str(len(page)))
                self.end_headers()
                return self.wfile.write(page)
            if self.path == "/health":
                rep = service.report
                return self._send(200, {"prepared": rep is not None, "steps": service.steps,
                                        "time_sets": None if rep is None else [list(k) for k in rep["time_sets"]]})
            if self.path == "/samples":
                return self._send(200, sorted(samples))
            if self.path == "/jobs":
                return self._send(200, list(jobs))
            self._send(404, {"error": "not found"})

        def do_POST(self):
            if self.path != "/render":
                return self._send(404, {"error": "not found"})
            n = int(self.headers.get("Content-Length", "0"))
            if n > 1 << 20:
                return self._send(413, {"error": "body too large"})
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
                sid, seed = str(body["sample"]), int(body.get("seed", 0))
            except (KeyError, ValueError, TypeError, json.JSONDecodeError) as exc:
                return self._send(400, {"error": f"bad request: {exc}"})
            if sid not in samples:
                return self._send(404, {"error": f"unknown sample {sid!r}"})
            with lock:
                t0 = time.perf_counter()
                try:
                    latents = service.render(samples[sid], seed=seed)
                except Exception as exc:  # noqa: BLE001 - reported to the client, the service stays up
                    return self._send(500, {"error": f"{type(exc).__name__}: {exc}"})
                name = f"{sid}-seed{seed}.pt"
                torch.save(latents.detach().cpu(), out / name)
                job = {"sample": sid, "seed": seed, "file": name, "seconds": round(time.perf_counter() - t0, 4),
                       "shape": list(latents.shape)}
                jobs.append(job)
            self._send(200, job)

    return ThreadingHTTPServer((host, port), Handler)
