"""Client of a local Ollama daemon for the notebook AI assist
(crates/axonml-server/src/llm/ollama.rs:9-260): availability probe, plain generation, code and
markdown suggestions with the reference's prompt framing."""
from __future__ import annotations

import json
import re
import urllib.error
import urllib.request

DEFAULT_URL = "http://localhost:11434"
DEFAULT_MODEL = "qwen2.5-coder:7b"


class OllamaError(RuntimeError):
    pass


class OllamaClient:
    def __init__(self, base_url: str = DEFAULT_URL, model: str = DEFAULT_MODEL, timeout: float = 120.0):
        self.base_url, self.model, self.timeout = base_url.rstrip("/"), model, timeout

    def _call(self, method: str, route: str, body: dict | None = None, timeout: float | None = None):
        req = urllib.request.Request(self.base_url + route, method=method,
                                     data=None if body is None else json.dumps(body).encode())
        req.add_header("Content-Type", "application/json")
        try:
            with urllib.request.urlopen(req, timeout=timeout or self.timeout) as r:
                return json.loads(r.read() or b"{}")
        except urllib.error.HTTPError as e:
            raise OllamaError(f"Ollama answered {e.code}") from e
        except (urllib.error.URLError, OSError, json.JSONDecodeError) as e:
            raise OllamaError(f"Ollama service unavailable: {e}") from e

    def is_available(self) -> bool:
        try:
            self._call("GET", "/api/tags", timeout=2.0)
            return True
        except OllamaError:
            return False

    def list_models(self) -> list:
        return [m.get("name") for m in self._call("GET", "/api/tags").get("models", [])]

    def generate(self, prompt: str, system: str | None = None, temperature: float = 0.2, max_tokens: int = 1024) -> str:
        body = {"model": self.model, "prompt": prompt, "stream": False,
                "options": {"temperature": temperature, "num_predict": max_tokens}}
        if system:
            body["system"] = system
        out = self._call("POST", "/api/generate", body)
        if "response" not in out:
            raise OllamaError("Ollama returned no response text")
        return out["response"]

    @staticmethod
    def _strip_fence(text: str) -> str:
        m = re.search(r"```[a-zA-Z0-9_+-]*\n(.*?)```", text, re.S)
        return (m.group(1) if m else text).strip()

    def generate_code(self, prompt: str, context: str = "", language: str = "python") -> dict:
        system = (f"You write {language} code for a machine-learning notebook. Answer with one code block and nothing else.")
        full = (f"Existing notebook cells:\n{context}\n\n" if context else "") + f"Task: {prompt}"
        text = self.generate(full, system=system)
        return {"kind": "code", "language": language, "content": self._strip_fence(text), "model": self.model}

    def generate_markdown(self, prompt: str, context: str = "") -> dict:
        system = "You write concise markdown documentation cells for a machine-learning notebook."
        full = (f"Existing notebook cells:\n{context}\n\n" if context else "") + f"Write: {prompt}"
        return {"kind": "markdown", "language": "markdown", "content": self.generate(full, system=system).strip(),
                "model": self.model}
