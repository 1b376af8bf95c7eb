"""File formats and sniffing (crates/axonml-serialize/src/format.rs:13-118)."""
from __future__ import annotations

import enum
import os


class Format(enum.Enum):
    Axonml = "axonml"
    Json = "json"
    SafeTensors = "safetensors"
    Gguf = "gguf"

    def extension(self) -> str: return self.value
    def name_str(self) -> str:
        return {"axonml": "Axonml Native", "json": "JSON", "safetensors": "SafeTensors", "gguf": "GGUF"}[self.value]
    def is_binary(self) -> bool: return self is not Format.Json
    def supports_streaming(self) -> bool: return self in (Format.SafeTensors, Format.Gguf)

    @staticmethod
    def all(): return list(Format)


def detect_format(path) -> Format:
    ext = os.path.splitext(str(path))[1].lower().lstrip(".")
    if ext in ("axonml", "bin"): return Format.Axonml
    if ext == "json": return Format.Json
    if ext in ("safetensors", "st"): return Format.SafeTensors
    if ext in ("gguf", "ggml"): return Format.Gguf
    return Format.Axonml


def detect_format_from_bytes(data: bytes):
    if len(data) >= 4 and data[:4] == b"GGUF":
        return Format.Gguf
    head = data[:64].lstrip()
    if head[:1] in (b"{", b"["):
        return Format.Json
    if len(data) >= 9:
        n = int.from_bytes(data[:8], "little")
        if 2 <= n <= len(data) - 8 and data[8:9] == b"{":
            return Format.SafeTensors
        return Format.Axonml
    return None
