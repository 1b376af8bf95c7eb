"""Profiling (crates/axonml-profile)."""
from .bottleneck import Bottleneck, BottleneckAnalyzer, BottleneckType
from .profiler import (ComputeProfiler, MemoryProfiler, OperationStats, ProfileGuard, Profiler,
                       TimelineEvent, TimelineProfiler, global_profiler, profile_scope)
from .report import ProfileReport, ReportFormat
