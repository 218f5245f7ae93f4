"""Minimal HTTP front end (stdlib ``ThreadingHTTPServer``): ``GET /state`` (JSON snapshot),
``POST /key`` ({"key": "w", "down": true}), ``POST /command`` ({"op": "start"}), ``POST /speeds``
({"move": 1.0, "turn": 1.0}), ``GET /fragments?since=N`` (reference: deploy/solar_wm/web/server.py)."""
from __future__ import annotations

import base64
import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from urllib.parse import parse_qs, urlparse

MAX_BODY = 8 * 1024 * 1024


def make_server(state, navigation, fragments=None, host: str = "127.0.0.1", port: int = 8900) -> ThreadingHTTPServer:
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
            if url.path == "/state":
                return self._send(200, state.snapshot())
            if url.path == "/fragments" and fragments is not None:
                since = int(parse_qs(url.query).get("since", ["0"])[0])
                return self._send(200, [{"index": i, "data": base64.b64encode(b).decode()} for i, b in fragments.since(since)])
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
