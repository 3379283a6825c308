"""The continuous-batching server behind HTTP, in the request / response shapes OpenAI-compatible clients send.

    POST /v1/completions        {"prompt": "text" | [ids], "max_tokens", "temperature", "top_p", "top_k", "seed", "stream"}
    POST /v1/chat/completions   {"messages": [{"role", "content"}, ...], ...the same sampling fields}
    GET  /v1/models             the served model's name
    GET  /metrics               Prometheus text: requests, tokens, queue depth, occupancy, time-to-first-token and per-token latency sums
    GET  /healthz

One thread runs the server's step loop while anything is queued or seated; each connection's handler thread submits a ticket and
waits for it (or, with ``"stream": true``, relays tokens as server-sent events the moment they settle).  Tokens of concurrent
requests share decode steps - that is the server's continuous batching, unchanged.

Reference: src/dew/inference/serving.py (the serving loop and its clients), examples/evaluate_and_serve.py.
"""
from __future__ import annotations

import json
import queue
import threading
import time
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer
from typing import Any, Dict, List, Optional

from ..sampling.text import Sampling
from .serving import Server


class CompletionService:
    def __init__(self, server: Server, tokenizer=None, name: str = "dew-b200", host: str = "127.0.0.1", port: int = 0, timeout: float = 300.0,
                 template=None, max_body: int = 8 << 20):
        self.server, self.tokenizer, self.name, self.timeout, self.template, self.max_body = server, tokenizer or server.tokenizer, name, timeout, template, max_body
        self._wake = threading.Condition()
        self._stop = False
        self._loop: Optional[threading.Thread] = None
        self.requests = self.completion_tokens = self.prompt_tokens = self.failed = 0
        self.ttft_sum = self.latency_sum = 0.0
        service = self

        class Handler(BaseHTTPRequestHandler):
            protocol_version = "HTTP/1.1"

            def log_message(self, *a):
                pass

            def _json(self, code: int, body: Dict[str, Any]):
                data = json.dumps(body).encode()
                self.send_response(code)
                self.send_header("Content-Type", "application/json")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def do_GET(self):
                if self.path == "/healthz":
                    return self._json(200, {"status": "ok"})
                if self.path == "/v1/models":
                    return self._json(200, {"object": "list", "data": [{"id": service.name, "object": "model", "owned_by": "local"}]})
                if self.path == "/metrics":
                    data = service.metrics_text().encode()
                    self.send_response(200)
                    self.send_header("Content-Type", "text/plain; version=0.0.4")
                    self.send_header("Content-Length", str(len(data)))
                    self.end_headers()
                    return self.wfile.write(data)
                self._json(404, {"error": {"message": "not found"}})

            def do_POST(self):
                if self.path not in ("/v1/completions", "/v1/chat/completions"):
                    return self._json(404, {"error": {"message": "not found"}})
                n = int(self.headers.get("Content-Length") or 0)
                if n <= 0 or n > service.max_body:
                    return self._json(400, {"error": {"message": "the body is empty or too large"}})
                try:
                    body = json.loads(self.rfile.read(n))
                    chat = self.path.endswith("chat/completions")
                    prompt = service.chat_prompt(body["messages"]) if chat else service.prompt_ids(body["prompt"])
                    ticket, events = service.submit(prompt, body)
                except (ValueError, KeyError, TypeError) as e:
                    service.failed += 1
                    return self._json(400, {"error": {"message": f"{type(e).__name__}: {e}"}})
                rid = ("chatcmpl-" if chat else "cmpl-") + uuid.uuid4().hex[:24]
                if body.get("stream"):
                    return self._stream(rid, chat, ticket, events)
                if not service.wait(ticket):
                    return self._json(504, {"error": {"message": "the request did not finish in time"}})
                if ticket.error is not None:
                    service.failed += 1
                    return self._json(500, {"error": {"message": str(ticket.error)}})
                self._json(200, service.response(rid, chat, ticket))

            def _stream(self, rid, chat, ticket, events):
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()

                def send(obj):
                    data = ("data: " + (obj if isinstance(obj, str) else json.dumps(obj)) + "\n\n").encode()
                    self.wfile.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
                    self.wfile.flush()
                deadline = time.monotonic() + service.timeout
                sent = 0
                while True:
                    try:
                        tok = events.get(timeout=0.05)
                    except queue.Empty:
                        if ticket.done and events.empty():
                            break
                        if time.monotonic() > deadline:
                            break
                        continue
                    sent += 1
                    text = service.text([tok])
                    delta = {"delta": {"content": text}} if chat else {"text": text, "token_ids": [tok]}
                    send({"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "model": service.name,
                          "choices": [{"index": 0, **delta, "finish_reason": None}]})
                send({"id": rid, "object": "chat.completion.chunk" if chat else "text_completion", "model": service.name,
                      "choices": [{"index": 0, **({"delta": {}} if chat else {"text": ""}), "finish_reason": service.finish_reason(ticket)}]})
                send("[DONE]")
                self.wfile.write(b"0\r\n\r\n")
                service.account(ticket)

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.httpd.daemon_threads = True
        self.address = self.httpd.server_address
        self._http: Optional[threading.Thread] = None

    # ------------------------------------------------------------------ requests
    def prompt_ids(self, prompt) -> List[int]:
        if isinstance(prompt, str):
            if self.tokenizer is None:
                raise ValueError("a text prompt needs a tokenizer; send token ids")
            return [int(t) for t in self.tokenizer.encode(prompt)]
        if isinstance(prompt, list) and all(isinstance(t, int) for t in prompt) and prompt:
            return prompt
        raise ValueError("the prompt is a string or a non-empty list of token ids")

    def chat_prompt(self, messages) -> List[int]:
        if self.tokenizer is None:
            raise ValueError("chat completions need a tokenizer")
        from ..data.chat import render_prompt
        return render_prompt(self.tokenizer, list(messages), self.template).tolist()

    def text(self, ids: List[int]) -> str:
        if self.tokenizer is None or not hasattr(self.tokenizer, "decode"):
            return ""
        return self.tokenizer.decode(ids)

    def submit(self, prompt: List[int], body: Dict[str, Any]):
        temperature = float(body.get("temperature", 1.0))
        sampling = Sampling(temperature=temperature, top_p=float(body.get("top_p") or 1.0), top_k=body.get("top_k"), min_p=float(body.get("min_p") or 0.0),
                            repetition_penalty=float(body.get("repetition_penalty") or 1.0), presence_penalty=float(body.get("presence_penalty") or 0.0),
                            frequency_penalty=float(body.get("frequency_penalty") or 0.0)) if temperature > 0 else Sampling(temperature=0.0)
        events: "queue.Queue[int]" = queue.Queue()
        max_tokens = int(body.get("max_tokens", 16))
        if max_tokens < 1:
            raise ValueError("max_tokens is at least 1")
        with self._wake:
            ticket = self.server.submit(prompt, max_tokens, key=int(body.get("seed", 0) or 0), sampling=sampling, on_token=events.put)
            self.requests += 1
            self._wake.notify_all()
        return ticket, events

    def wait(self, ticket) -> bool:
        deadline = time.monotonic() + self.timeout
        with self._wake:
            while not ticket.done:
                left = deadline - time.monotonic()
                if left <= 0:
                    return False
                self._wake.wait(min(left, 0.1))
        self.account(ticket)
        return True

    def account(self, ticket) -> None:
        self.prompt_tokens += len(ticket.prompt)
        self.completion_tokens += len(ticket.tokens)
        if ticket.first_token_time is not None:
            self.ttft_sum += ticket.first_token_time
        if ticket.finished_time is not None:
            self.latency_sum += ticket.finished_time

    @staticmethod
    def finish_reason(ticket) -> str:
        return "stop" if ticket.terminated else "length"

    def response(self, rid: str, chat: bool, ticket) -> Dict[str, Any]:
        text = self.text(ticket.tokens)
        choice = {"index": 0, "finish_reason": self.finish_reason(ticket), "token_ids": list(ticket.tokens)}
        choice.update({"message": {"role": "assistant", "content": text}} if chat else {"text": text})
        return {"id": rid, "object": "chat.completion" if chat else "text_completion", "created": int(time.time()), "model": self.name, "choices": [choice],
                "usage": {"prompt_tokens": len(ticket.prompt), "completion_tokens": len(ticket.tokens), "total_tokens": len(ticket.prompt) + len(ticket.tokens)}}

    def metrics_text(self) -> str:
        s = self.server
        rows = {"requests_total": self.requests, "requests_failed_total": self.failed, "prompt_tokens_total": self.prompt_tokens,
                "completion_tokens_total": self.completion_tokens, "queue_depth": s.queued, "occupancy": s.occupancy, "steps_total": s.steps,
                "time_to_first_token_seconds_sum": self.ttft_sum, "request_latency_seconds_sum": self.latency_sum,
                "prefix_cache_hits_total": s.ledger.hits, "prefix_cache_lookups_total": s.ledger.lookups}
        return "".join(f"dew_serving_{k} {v:g}\n" for k, v in rows.items())

    # ------------------------------------------------------------------ threads
    def _run(self) -> None:
        while True:
            with self._wake:
                while not self._stop and not self.server.busy:
                    self._wake.wait(0.05)
                if self._stop:
                    return
            try:
                self.server.step()
            except BaseException as e:                                   # a failed step fails the requests in flight, not the service
                self.server.fail(e)
            with self._wake:
                self._wake.notify_all()

    def start(self) -> "CompletionService":
        self._stop = False
        self._loop = threading.Thread(target=self._run, name="serving-loop", daemon=True)
        self._loop.start()
        self._http = threading.Thread(target=self.httpd.serve_forever, name="serving-http", daemon=True)
        self._http.start()
        return self

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
        with self._wake:
            self._stop = True
            self._wake.notify_all()
        if self._loop is not None:
            self._loop.join(timeout=10)

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
