"""Minimal HTTP front end (stdlib ``ThreadingHTTPServer``): ``GET /`` (a one-page client), ``GET /state`` (JSON snapshot),
``POST /key`` ({"key": "w", "down": true}), ``POST /command`` ({"op": "start"}), ``POST /speeds``
({"move": 1.0, "turn": 1.0}), ``GET /fragments?since=N`` (reference: deploy/solar_wm/web/server.py)."""
from __future__ import annotations

import base64
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

MAX_BODY = 8 * 1024 * 1024

# The whole client: keys go to /key, the buttons to /command, the status line polls /state.
INDEX_HTML = """<!doctype html><html><head><meta charset="utf-8"><title>solarwm_b200 realtime</title>
<style>body{font:14px system-ui;margin:2em;max-width:48em}kbd{border:1px solid #999;border-radius:3px;padding:1px 5px}
#state{white-space:pre;font-family:ui-monospace,monospace;background:#f4f4f4;padding:1em}</style></head><body>
<h1>Realtime session</h1>
<p>Move with <kbd>W</kbd><kbd>A</kbd><kbd>S</kbd><kbd>D</kbd>, turn with <kbd>I</kbd><kbd>J</kbd><kbd>K</kbd><kbd>L</kbd>.
<button onclick="cmd('start')">start</button> <button onclick="cmd('chunk')">one chunk</button>
<button onclick="cmd('stop')">stop</button></p>
<p>move speed <input id="move" type="range" min="0.25" max="4" step="0.05" value="1" oninput="speeds()">
turn speed <input id="turn" type="range" min="0.1" max="3" step="0.1" value="1" oninput="speeds()"></p>
<div id="state">...</div>
<script>
const post=(path,body)=>fetch(path,{method:'POST',headers:{'Content-Type':'application/json'},body:JSON.stringify(body)});
const cmd=op=>post('/command',{op});
const speeds=()=>post('/speeds',{move:+move.value,turn:+turn.value});
const keys=new Set('wasdijkl');
for(const [ev,down] of [['keydown',true],['keyup',false]])
  addEventListener(ev,e=>{const k=e.key.toLowerCase();if(keys.has(k)&&!e.repeat){post('/key',{key:k,down});e.preventDefault();}});
setInterval(async()=>{const r=await fetch('/state');state.textContent=JSON.stringify(await r.json(),null,1);},500);
</script></body></html>"""


def make_server(state, navigation, fragments=None, host: str = "127.0.0.1", port: int = 8900,
                media=None) -> ThreadingHTTPServer:
    """``media``: a ``serve.fragments.MediaStore``; ``GET /media?scene=&sequence=&cursor=&limit=`` then serves whole
    fMP4 fragments of a live (or finished) preview to clients that resume by cursor."""
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
            url = urlparse(self.path)
            if url.path in ("/", "/index.html"):
                body = INDEX_HTML.encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/html; charset=utf-8")
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)
                return None
            if url.path == "/state":
                return self._send(200, state.snapshot())
            if url.path == "/fragments" and fragments is not None:
                since = int(parse_qs(url.query).get("since", ["0"])[0])
                return self._send(200, [{"index": i, "data": base64.b64encode(b).decode()} for i, b in fragments.since(since)])
            if url.path == "/media" and media is not None:
                q = parse_qs(url.query)
                try:
                    got = media.fragments(q.get("scene", [""])[0], int(q.get("sequence", ["0"])[0]),
                                          int(q.get("cursor", ["0"])[0]), int(q.get("limit", ["16"])[0]))
                except FileNotFoundError:
                    return self._send(404, {"error": "no such preview"})
                except ValueError as exc:
                    return self._send(400, {"error": str(exc)})
                enc = lambda b: None if b is None else base64.b64encode(b).decode()    # noqa: E731
                return self._send(200, {"rows": got["rows"], "data": [enc(b) for b in got["data"]], "init": enc(got["init"]),
                                        "produced": got["produced"], "done": got["done"], "next_cursor": got["next_cursor"]})
            self._send(404, {"error": "not found"})

        def do_POST(self):
            n = int(self.headers.get("Content-Length", "0"))
            if n > MAX_BODY:
                return self._send(413, {"error": "body too large"})
            try:
                body = json.loads(self.rfile.read(n) or b"{}")
                if self.path == "/key":
                    navigation.set_key(str(body["key"]), bool(body["down"]))
                elif self.path == "/speeds":
                    navigation.set_speeds(float(body.get("move", 1.0)), float(body.get("turn", 1.0)))
                elif self.path == "/command":
                    state.submit(str(body["op"]), **{k: v for k, v in body.items() if k != "op"})
                else:
                    return self._send(404, {"error": "not found"})
            except (KeyError, ValueError, TypeError, json.JSONDecodeError) as exc:
                return self._send(400, {"error": str(exc)})
            self._send(200, {"ok": True})

    return ThreadingHTTPServer((host, port), Handler)


def serve_in_thread(server: ThreadingHTTPServer) -> threading.Thread:
    t = threading.Thread(target=server.serve_forever, daemon=True)
    t.start()
    return t
