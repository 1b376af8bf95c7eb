"""Inference serving: quantised LLM engine (paged KV, continuous batching), StateDict model
service, metrics and the HTTP front end (crates/axonml-server inference parts +
crates/axonml-cli/src/commands/serve.rs)."""
from .engine import LLMEngine, Request
from .http import AxonmlHTTPServer
from .inference import InferenceServer, ModelPool, build_model_from_state_dict
from .kv_cache import OutOfPages, PagedKVCache
from .metrics import EndpointMetrics, InferenceMetrics, RequestTimer
from .model import QuantizedLlama
