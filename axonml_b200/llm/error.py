"""Errors of the language-model package.

Parity: crates/axonml-llm/src/error.rs (``LLMError`` with the variants InvalidConfig, ShapeMismatch
{expected, actual}, InvalidInput, GenerationError, LoadError, CoreError, IoError, NetworkError,
ParseError, ModelNotFound, WeightNotFound, UnsupportedFormat, TensorError and their messages).
Each variant is a subclass, so callers can catch one kind or all of them; where a built-in
exception means the same thing the subclass derives from it too."""
from __future__ import annotations


class LLMError(Exception):
    prefix = ""

    def __str__(self) -> str:
        msg = super().__str__()
        return f"{self.prefix}: {msg}" if self.prefix else msg


class InvalidConfig(LLMError, ValueError): prefix = "Invalid configuration"
class InvalidInput(LLMError, ValueError): prefix = "Invalid input"
class GenerationError(LLMError): prefix = "Generation error"
class LoadError(LLMError): prefix = "Model loading error"
class CoreError(LLMError): prefix = "Core error"
class IoError(LLMError, OSError): prefix = "IO error"
class NetworkError(LLMError): prefix = "Network error"
class ParseError(LLMError, ValueError): prefix = "Parse error"
class ModelNotFound(LLMError, FileNotFoundError): prefix = "Model not found"
class WeightNotFound(LLMError, KeyError): prefix = "Weight not found"
class UnsupportedFormat(LLMError, ValueError): prefix = "Unsupported format"
class TensorError(LLMError): prefix = "Tensor error"


class ShapeMismatch(LLMError, ValueError):
    def __init__(self, expected, actual):
        super().__init__(f"Shape mismatch: expected {expected}, got {actual}")
        self.expected, self.actual = expected, actual
