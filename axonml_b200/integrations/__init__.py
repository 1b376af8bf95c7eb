"""Clients of external services the reference CLI talks to: Weights & Biases and Kaggle.  Both
work without a network: W&B runs are written in offline-run layout on disk, Kaggle keeps the
credential and download bookkeeping and reports that the service cannot be reached."""
from .kaggle import KaggleClient, OfflineError
from .wandb import WandbConfig, WandbRun

__all__ = ["KaggleClient", "OfflineError", "WandbConfig", "WandbRun"]
