"""The six views of the terminal interface (crates/axonml-tui/src/views/mod.rs)."""
from .data import ClassInfo, DatasetInfo, DataView, FeatureInfo, SplitInfo
from .files import FileEntry, FilesView, FileType
from .graphs import BrailleCanvas, ChartType, DataSeries, GraphsView
from .help import HelpView
from .model import LayerInfo, ModelInfo, ModelView
from .training import (EpochMetrics, TrainingConfig, TrainingSession, TrainingStatus, TrainingView, find_training_log,
                       parse_training_log, sparkline)

__all__ = ["ClassInfo", "DatasetInfo", "DataView", "FeatureInfo", "SplitInfo", "FileEntry", "FilesView", "FileType", "BrailleCanvas",
           "ChartType", "DataSeries", "GraphsView", "HelpView", "LayerInfo", "ModelInfo", "ModelView", "EpochMetrics", "TrainingConfig",
           "TrainingSession", "TrainingStatus", "TrainingView", "find_training_log", "parse_training_log", "sparkline"]
