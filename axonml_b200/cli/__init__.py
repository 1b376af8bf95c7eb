"""Command line and project configuration (crates/axonml-cli)."""
from .config import ProjectConfig
from .main import build_parser, main

__all__ = ["ProjectConfig", "build_parser", "main"]
