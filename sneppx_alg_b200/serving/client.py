"""HTTP client for the serving API (the reference's ``serving_client.py``): generate, batch, chat, stream, health."""
from __future__ import annotations

import json
from typing import Iterator, List, Optional

import requests


class ServingClient:
    def __init__(self, base_url="http://127.0.0.1:8000", api_key: Optional[str] = None, timeout=60.0, session=None):
        self.base, self.timeout = base_url.rstrip("/"), timeout
        self.s = session or requests.Session()
        if api_key:
            self.s.headers["Authorization"] = f"Bearer {api_key}"

    def _post(self, path, body):
        r = self.s.post(self.base + path, json=body, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def health(self) -> dict:
        r = self.s.get(self.base + "/v1/health", timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def models(self) -> dict:
        return self.s.get(self.base + "/v1/models", timeout=self.timeout).json()

    def generate(self, prompt: str, **params) -> dict:
        return self._post("/v1/generate", {"prompt": prompt, **params})

    def generate_batch(self, prompts: List[str], **params) -> dict:
        return self._post("/v1/generate/batch", {"prompts": prompts, **params})

    def chat(self, messages: List[dict], **params) -> dict:
        return self._post("/v1/chat/completions", {"messages": messages, **params})

    def stream(self, prompt: str, **params) -> Iterator[dict]:
        with self.s.post(self.base + "/v1/generate/stream", json={"prompt": prompt, **params}, stream=True,
                         timeout=self.timeout) as r:
            r.raise_for_status()
            for line in r.iter_lines():
                if line.startswith(b"data: "):
                    payload = line[6:]
                    if payload == b"[DONE]":
                        return
                    yield json.loads(payload)
