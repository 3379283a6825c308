"""A decision task behind HTTP: JSON wire bodies in, JSON answers out, rows of concurrent requests scored together.

    POST /v1/decide     one wire body -> its response body; a list of bodies -> a list (a refused body becomes {"error": ...})
    GET  /metrics       counters in the Prometheus text format (requests, refusals by reason, passes, rows per pass, token share)
    GET  /healthz       200 once the scoring thread runs

Each connection's handler thread submits to one ``ScoringServer``, whose thread batches the waiting rows into passes, so many
small requests share forward passes.  Query flags ``?details=1`` and ``?whole=1`` select the matching wire options per request.

Reference: examples/serve_decisions.py and the served scoring task of src/dew/inference/scoring.py.
"""
from __future__ import annotations

import json
import threading
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Dict, Optional, Tuple
from urllib.parse import parse_qs, urlparse

from ..inference.scoring import ScoringServer
from .task import Decide


class DecisionService:
    def __init__(self, task: Decide, host: str = "127.0.0.1", port: int = 0, max_rows: int = 256, max_wait: float = 0.005, max_body: int = 4 << 20,
                 timeout: float = 60.0):
        self.task, self.max_body, self.timeout = task, max_body, timeout
        # one scoring server per combination of wire options (they change what ``admit`` refuses and what ``answer`` reports)
        self._servers: Dict[Tuple[bool, bool], ScoringServer] = {}
        self._max_rows, self._max_wait = max_rows, max_wait
        self._lock = threading.Lock()
        service = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *args):                               # quiet by default
                pass

            def _send(self, code: int, body: bytes, kind: str = "application/json"):
                self.send_response(code)
                self.send_header("Content-Type", kind)
                self.send_header("Content-Length", str(len(body)))
                self.end_headers()
                self.wfile.write(body)

            def do_GET(self):
                path = urlparse(self.path).path
                if path == "/healthz":
                    return self._send(200, b'{"status": "ok"}')
                if path == "/metrics":
                    return self._send(200, service.metrics_text().encode(), "text/plain; version=0.0.4")
                self._send(404, b'{"error": "not found"}')

            def do_POST(self):
                url = urlparse(self.path)
                if url.path != "/v1/decide":
                    return self._send(404, b'{"error": "not found"}')
                n = int(self.headers.get("Content-Length") or 0)
                if n <= 0 or n > service.max_body:
                    return self._send(413 if n > service.max_body else 400, json.dumps({"error": "the body is empty or too large"}).encode())
                try:
                    body = json.loads(self.rfile.read(n))
                except ValueError:
                    return self._send(400, b'{"error": "the body is not JSON"}')
                q = parse_qs(url.query)
                flag = lambda name: q.get(name, ["0"])[0] not in ("0", "", "false")
                try:
                    out = service.decide(body, details=flag("details"), whole=flag("whole"))
                except ValueError as refused:
                    return self._send(422, json.dumps({"error": str(refused), "reason": getattr(refused, "reason", "malformed")}).encode())
                except Exception as failed:                              # a failed pass: the server stays up
                    return self._send(500, json.dumps({"error": f"{type(failed).__name__}: {failed}"}).encode())
                self._send(200, json.dumps(out).encode())

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.httpd.daemon_threads = True
        self.address = self.httpd.server_address
        self._thread: Optional[threading.Thread] = None

    def _server(self, details: bool, whole: bool) -> ScoringServer:
        with self._lock:
            key = (details, whole)
            if key not in self._servers:
                self._servers[key] = ScoringServer(self.task.scoring(details=details, whole=whole), self._max_rows, self._max_wait).start()
            return self._servers[key]

    def decide(self, body: Any, details: bool = False, whole: bool = False):
        server = self._server(details, whole)
        if isinstance(body, list):
            futures = []
            for b in body:
                try:
                    futures.append(server.submit(b))
                except ValueError as refused:
                    futures.append(refused)
            return [{"error": str(f), "reason": getattr(f, "reason", "malformed")} if isinstance(f, ValueError) else f.result(self.timeout) for f in futures]
        return server.submit(body).result(self.timeout)

    def metrics_text(self) -> str:
        lines = []
        with self._lock:
            servers = dict(self._servers)
        for (details, whole), s in servers.items():
            labels = f'{{details="{int(details)}",whole="{int(whole)}"}}'
            for k, v in s.metrics().items():
                name = "dew_decide_" + k.replace("/", "_")
                lines.append(f"{name}{labels} {v:g}")
        return "\n".join(lines) + "\n"

    def start(self) -> "DecisionService":
        self._thread = threading.Thread(target=self.httpd.serve_forever, name="decision-http", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
        with self._lock:
            for s in self._servers.values():
                s.stop()
            self._servers.clear()

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
