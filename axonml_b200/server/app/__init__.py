"""The platform server (users, training runs, model registry, datasets, inference endpoints,
notebooks, system information, dashboard) on top of the inference server of ``axonml_b200.server``.

    from axonml_b200.server.app import PlatformServer
    PlatformServer(port=3021, data_dir="~/.axonml/server", admin_password="…").serve_forever()
"""
from .api import HttpError, PlatformServer, Request, Router
from .auth import AuthError, JwtAuth, RecoveryAuth, TotpAuth, hash_password, verify_password
from .notebooks import NotebookKernel, NotebookService
from .registry import DatasetCatalog, EndpointManager, ModelRegistry
from .store import AlreadyExists, Collection, DbError, DocumentStore, NotFound
from .system import SystemMonitor, list_gpus, run_benchmark, system_info
from .training import RunRepository, TrainingExecutor, TrainingTracker

__all__ = ["PlatformServer", "Request", "Router", "HttpError", "AuthError", "JwtAuth", "TotpAuth", "RecoveryAuth",
           "hash_password", "verify_password", "DocumentStore", "Collection", "DbError", "NotFound", "AlreadyExists",
           "RunRepository", "TrainingTracker", "TrainingExecutor", "ModelRegistry", "DatasetCatalog", "EndpointManager",
           "NotebookService", "NotebookKernel", "SystemMonitor", "system_info", "list_gpus", "run_benchmark"]
