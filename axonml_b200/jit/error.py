"""Errors of the JIT (crates/axonml-jit/src/error.rs:12-42), one subclass per variant; each also
derives from the built-in exception that callers would expect for that failure."""
from __future__ import annotations


class JitError(Exception):
    pass


class InvalidGraph(JitError, ValueError):
    def __init__(self, what): super().__init__(f"Invalid graph: {what}")


class TypeMismatch(JitError, TypeError):
    def __init__(self, expected, found):
        super().__init__(f"Type mismatch: expected {expected}, found {found}")
        self.expected, self.found = expected, found


class ShapeMismatch(JitError, ValueError):
    def __init__(self, expected, found):
        super().__init__(f"Shape mismatch: expected {list(expected)}, found {list(found)}")
        self.expected, self.found = list(expected), list(found)


class UnsupportedOp(JitError, NotImplementedError):
    def __init__(self, op): super().__init__(f"Unsupported operation: {op}")


class CodegenError(JitError):
    def __init__(self, what): super().__init__(f"Code generation failed: {what}")


class JitRuntimeError(JitError, RuntimeError):
    def __init__(self, what): super().__init__(f"Runtime error: {what}")


class InputNotFound(JitError, KeyError):
    def __init__(self, name):
        super().__init__(f"Input not found: {name}")
        self.name = name

    def __str__(self) -> str: return self.args[0]


class OutputNotFound(JitError, KeyError):
    def __init__(self, name):
        super().__init__(f"Output not found: {name}")
        self.name = name

    def __str__(self) -> str: return self.args[0]


class CompilationFailed(JitError, RuntimeError):
    def __init__(self, what): super().__init__(f"Compilation failed: {what}")
