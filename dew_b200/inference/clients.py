"""Thin HTTP clients for OpenAI-compatible and Ollama chat endpoints (used by judges / reward models in RL recipes and by
comparisons against external engines).  Standard library only; a ``transport`` callable can replace the network in tests.
Reference: src/dew/inference/clients.py (674 lines)."""
from __future__ import annotations

import json
import urllib.request
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence


def _post(url: str, payload: Mapping[str, Any], headers: Mapping[str, str], timeout: float) -> Dict[str, Any]:
    req = urllib.request.Request(url, data=json.dumps(payload).encode(), headers={"Content-Type": "application/json", **headers})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read().decode())


@dataclass
class OpenAIClient:
    base_url: str = "http://127.0.0.1:8000/v1"
    model: str = "default"
    api_key: Optional[str] = None
    timeout: float = 60.0
    transport: Callable[..., Dict[str, Any]] = field(default=_post, repr=False)

    def chat(self, messages: Sequence[Mapping[str, str]], max_tokens: int = 256, temperature: float = 0.0, **extra) -> str:
        headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
        body = {"model": self.model, "messages": list(messages), "max_tokens": max_tokens, "temperature": temperature, **extra}
        out = self.transport(self.base_url.rstrip("/") + "/chat/completions", body, headers, self.timeout)
        return out["choices"][0]["message"]["content"]

    def complete(self, prompt: str, max_tokens: int = 256, temperature: float = 0.0, **extra) -> str:
        headers = {"Authorization": f"Bearer {self.api_key}"} if self.api_key else {}
        body = {"model": self.model, "prompt": prompt, "max_tokens": max_tokens, "temperature": temperature, **extra}
        out = self.transport(self.base_url.rstrip("/") + "/completions", body, headers, self.timeout)
        return out["choices"][0]["text"]


@dataclass
class OllamaClient:
    base_url: str = "http://127.0.0.1:11434"
    model: str = "llama3"
    timeout: float = 120.0
    transport: Callable[..., Dict[str, Any]] = field(default=_post, repr=False)

    def chat(self, messages: Sequence[Mapping[str, str]], **options) -> str:
        body = {"model": self.model, "messages": list(messages), "stream": False, "options": options}
        return self.transport(self.base_url.rstrip("/") + "/api/chat", body, {}, self.timeout)["message"]["content"]
