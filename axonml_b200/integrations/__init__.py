"""Clients of external services the reference talks to: Weights & Biases and Kaggle (CLI),
HashiCorp Vault / environment secrets, the Resend e-mail API and a local Ollama daemon (platform
server).  All work without a network: W&B runs are written in offline-run layout on disk, Kaggle
keeps the credential and download bookkeeping and reports that the service cannot be reached,
and the server degrades (environment secrets, accounts approved at once, AI assist answers 503)
when Vault, Resend or Ollama are not configured."""
from .email import EmailError, EmailService
from .kaggle import KaggleClient, OfflineError
from .ollama import OllamaClient, OllamaError
from .secrets import EnvBackend, SecretKey, SecretsError, SecretsManager, VaultBackend
from .wandb import WandbConfig, WandbRun

__all__ = ["EmailError", "EmailService", "EnvBackend", "KaggleClient", "OfflineError", "OllamaClient", "OllamaError",
           "SecretKey", "SecretsError", "SecretsManager", "VaultBackend", "WandbConfig", "WandbRun"]
