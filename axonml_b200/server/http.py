"""HTTP front end (stdlib ``http.server``, threaded): ``/health``, ``/info``, ``/metrics``
(Prometheus text), ``/predict`` and ``/batch`` for StateDict models (the reference CLI server's
routes, crates/axonml-cli/src/commands/serve.rs:178-193), ``/api/inference/predict/<name>``
(crates/axonml-server/src/api/inference.rs:396) and ``/v1/completions`` for the LLM engine.  LLM
requests from all connections are funnelled into one engine thread that runs the continuous
batching loop, so concurrent clients share decode steps."""
from __future__ import annotations

import json
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .inference import InferenceServer
from .metrics import InferenceMetrics


class _EngineThread(threading.Thread):
    def __init__(self, engine):
        super().__init__(daemon=True)
        self.engine, self._cv, self._stop = engine, threading.Condition(), False

    def submit(self, prompt, max_new_tokens, eos=None):
        with self._cv:
            r = self.engine.add_request(prompt, max_new_tokens, eos)
            self._cv.notify()
        return r

    def run(self):
        while not self._stop:
            with self._cv:
                while not (self.engine.waiting or self.engine.running) and not self._stop:
                    self._cv.wait(0.1)
                if self._stop:
                    return
            with self._cv:
                self.engine.step()

    def stop(self):
        self._stop = True
        with self._cv:
            self._cv.notify_all()


class AxonmlHTTPServer:
    def __init__(self, host: str = "127.0.0.1", port: int = 3021, inference: InferenceServer | None = None,
                 llm_engine=None, tokenizer=None):
        self.inference = inference or InferenceServer()
        self.metrics = InferenceMetrics()
        self.engine, self.tokenizer = llm_engine, tokenizer
        self._engine_thread = _EngineThread(llm_engine) if llm_engine is not None else None
        self.started = time.time()
        outer = self

        class Handler(BaseHTTPRequestHandler):
            def log_message(self, *a): pass

            def _send(self, code, body, ctype="application/json"):
                data = body.encode() if isinstance(body, str) else json.dumps(body).encode()
                self.send_response(code)
                self.send_header("Content-Type", ctype)
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                self.wfile.write(data)

            def _body(self):
                n = int(self.headers.get("Content-Length", 0))
                return json.loads(self.rfile.read(n) or b"{}")

            def do_GET(self):
                if self.path == "/health":
                    return self._send(200, {"status": "healthy", "uptime_s": time.time() - outer.started})
                if self.path == "/info":
                    return self._send(200, outer.info())
                if self.path in ("/metrics", "/api/metrics"):
                    return self._send(200, outer.prometheus(), "text/plain; version=0.0.4")
                if self.path == "/api/inference/metrics":
                    return self._send(200, outer.metrics.snapshot())
                self._send(404, {"error": "not found"})

            def do_POST(self):
                path = self.path
                timer = outer.metrics.time_request(path)
                try:
                    body = self._body()
                    if path == "/predict":
                        out = {"output": outer.inference.predict(body.get("model", "default"), body["input"])}
                    elif path == "/batch":
                        out = {"outputs": outer.inference.predict(body.get("model", "default"), body["inputs"])}
                    elif path.startswith("/api/inference/predict/"):
                        out = {"output": outer.inference.predict(path.rsplit("/", 1)[-1], body["input"])}
                    elif path == "/v1/completions":
                        out = outer.complete(body)
                    else:
                        timer.finish_error()
                        return self._send(404, {"error": "not found"})
                    out["latency_ms"] = timer.finish_success()
                    self._send(200, out)
                except KeyError as e:
                    timer.finish_error()
                    self._send(404 if "unknown model" in str(e) else 400, {"error": str(e)})
                except Exception as e:  # noqa: BLE001
                    timer.finish_error()
                    self._send(500, {"error": f"{type(e).__name__}: {e}"})

        self.httpd = ThreadingHTTPServer((host, port), Handler)
        self.port = self.httpd.server_address[1]
        self._thread = None

    def info(self) -> dict:
        d = {"name": "axonml_b200 inference server", "models": self.inference.list_models(), "llm": self.engine is not None}
        if self.engine is not None:
            c = self.engine.model.cfg
            d["llm_config"] = {"layers": c.num_hidden_layers, "hidden": c.hidden_size, "vocab": c.vocab_size,
                               "tp": self.engine.model.tp, "weight_bytes": self.engine.model.weight_bytes()}
        return d

    def prometheus(self) -> str:
        extra = {"endpoints_running": len(self.inference.list_models()) + (1 if self.engine else 0)}
        if self.engine is not None:
            s = self.engine.stats()
            extra.update({"llm_ttft_p50_seconds": s["ttft_p50_s"] or 0.0, "llm_decode_tokens_per_second": s["decode_tokens_per_s"],
                          "llm_queue_depth": s["queue_depth"], "llm_kv_page_occupancy": s["kv_page_occupancy"]})
        return self.metrics.prometheus(extra)

    def complete(self, body: dict) -> dict:
        if self.engine is None:
            raise KeyError("unknown model llm")
        prompt = body.get("prompt_ids")
        if prompt is None:
            if self.tokenizer is None:
                raise KeyError("prompt_ids (no tokenizer loaded)")
            prompt = self.tokenizer.encode(body["prompt"])
        r = self._engine_thread.submit(prompt, int(body.get("max_tokens", 16)), body.get("eos_token_id"))
        while not r.done():
            time.sleep(0.001)
        out = {"token_ids": r.output, "ttft_ms": (r.ttft() or 0.0) * 1e3,
               "decode_tokens_per_s": (len(r.output) - 1) / max(r.finished_at - r.first_token_at, 1e-9) if len(r.output) > 1 else 0.0}
        if self.tokenizer is not None:
            out["text"] = self.tokenizer.decode(r.output)
        return out

    def start(self) -> "AxonmlHTTPServer":
        if self._engine_thread is not None:
            self._engine_thread.start()
        self._thread = threading.Thread(target=self.httpd.serve_forever, daemon=True)
        self._thread.start()
        return self

    def serve_forever(self) -> None:
        if self._engine_thread is not None:
            self._engine_thread.start()
        self.httpd.serve_forever()

    def stop(self) -> None:
        self.httpd.shutdown()
        self.httpd.server_close()
        if self._engine_thread is not None:
            self._engine_thread.stop()
