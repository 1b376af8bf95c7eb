"""Profiling (crates/axonml-profile)."""
from .bottleneck import AnalyzerConfig, Bottleneck, BottleneckAnalyzer, BottleneckType, Severity
from .profiler import (AllocationRecord, ComputeProfiler, Event, EventType, MemoryProfiler, MemoryStats, OperationStats,
                       ProfiledOp, ProfileError, ProfileGuard, Profiler, TimelineEvent, TimelineProfiler, TimingGuard,
                       format_bytes, format_duration, global_profiler, profile_scope, record_alloc, record_free, start, stop)
from .report import ComputeSummary, MemorySummary, OperationSummary, ProfileReport, ReportFormat
