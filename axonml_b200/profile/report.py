"""Profile reports in text / JSON / Markdown / HTML (crates/axonml-profile/src/report.rs:17-359)."""
from __future__ import annotations

import dataclasses
import enum
import json

from .bottleneck import BottleneckAnalyzer


class ReportFormat(enum.Enum):
    Text = "text"
    Json = "json"
    Markdown = "markdown"
    Html = "html"


@dataclasses.dataclass
class MemorySummary:
    current_usage: int = 0
    peak_usage: int = 0
    total_allocated: int = 0
    total_freed: int = 0
    allocation_count: int = 0


@dataclasses.dataclass
class OperationSummary:
    name: str
    total_time_ns: int
    call_count: int
    avg_time_ns: int
    time_percentage: float


@dataclasses.dataclass
class ComputeSummary:
    operation_count: int = 0
    total_time_ns: int = 0
    top_operations: list = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class ProfileReport:
    operations: list
    total_time_ms: float
    peak_memory: int
    current_memory: int
    bottlenecks: list
    device_memory: dict
    memory: MemorySummary = dataclasses.field(default_factory=MemorySummary)
    compute: ComputeSummary = dataclasses.field(default_factory=ComputeSummary)

    @classmethod
    def generate(cls, profiler) -> "ProfileReport":
        ops = profiler.compute.top(1000)
        total_ns = profiler.compute.total_time_ns()
        m = profiler.memory.stats()
        top = [OperationSummary(s.name, int(s.total_ns), s.count, int(s.avg_ns()), 100.0 * s.total_ns / total_ns if total_ns else 0.0)
               for s in ops[:10]]
        return cls([dataclasses.asdict(s) | {"avg_ns": s.avg_ns(), "gflops": s.gflops(), "gbps": s.gbps()} for s in ops],
                   total_ns / 1e6, profiler.memory.peak, profiler.memory.current,
                   [dataclasses.asdict(b) | {"kind": b.kind.value, "severity": b.severity.name} for b in BottleneckAnalyzer().analyze(profiler)],
                   profiler.memory.device_stats(),
                   MemorySummary(m.current_usage, m.peak_usage, m.total_allocated, m.total_freed, m.allocation_count),
                   ComputeSummary(len(ops), int(total_ns), top))

    def format(self, fmt: ReportFormat) -> str:
        return {ReportFormat.Text: self.to_text, ReportFormat.Json: self.to_json,
                ReportFormat.Markdown: self.to_markdown, ReportFormat.Html: self.to_html}[fmt]()

    def _rows(self):
        for o in self.operations:
            yield (o["name"], o["count"], o["total_ns"] / 1e6, o["avg_ns"] / 1e3, o["gflops"], o["gbps"])

    def to_text(self) -> str:
        lines = [f"=== Profile: {self.total_time_ms:.3f} ms total, peak memory {self.peak_memory} B ===",
                 f"{'operation':32s} {'calls':>8s} {'total ms':>10s} {'avg us':>10s} {'GFLOPS':>9s} {'GB/s':>8s}"]
        for n, c, t, a, g, b in self._rows():
            lines.append(f"{n[:32]:32s} {c:8d} {t:10.3f} {a:10.2f} {g:9.2f} {b:8.2f}")
        for b in self.bottlenecks:
            lines.append(f"[{b['severity']}] [{b['kind']}] {b['description']} -> {b['suggestion']}")
        return "\n".join(lines)

    def to_json(self) -> str: return json.dumps(dataclasses.asdict(self), indent=2, default=str)

    def to_markdown(self) -> str:
        lines = [f"# Profile report\n\nTotal {self.total_time_ms:.3f} ms, peak memory {self.peak_memory} bytes\n",
                 "| operation | calls | total ms | avg us | GFLOPS | GB/s |", "|---|---|---|---|---|---|"]
        for n, c, t, a, g, b in self._rows():
            lines.append(f"| {n} | {c} | {t:.3f} | {a:.2f} | {g:.2f} | {b:.2f} |")
        if self.bottlenecks:
            lines.append("\n## Bottlenecks\n")
            lines += [f"- **{b['kind']}** {b['description']} — {b['suggestion']}" for b in self.bottlenecks]
        return "\n".join(lines)

    def to_html(self) -> str:
        rows = "".join(f"<tr><td>{n}</td><td>{c}</td><td>{t:.3f}</td><td>{a:.2f}</td><td>{g:.2f}</td><td>{b:.2f}</td></tr>"
                       for n, c, t, a, g, b in self._rows())
        return ("<html><body><h1>Profile report</h1>"
                f"<p>Total {self.total_time_ms:.3f} ms, peak memory {self.peak_memory} bytes</p>"
                "<table border=1><tr><th>operation</th><th>calls</th><th>total ms</th><th>avg us</th>"
                f"<th>GFLOPS</th><th>GB/s</th></tr>{rows}</table></body></html>")

    def export(self, path, fmt: ReportFormat | None = None) -> None:
        """Writes the report; the format follows the file extension unless given (report.rs ``export``)."""
        self.save(path, fmt)

    def __str__(self) -> str:
        return self.to_text()

    def save(self, path, fmt: ReportFormat | None = None) -> None:
        if fmt is None:
            ext = str(path).rsplit(".", 1)[-1].lower()
            fmt = {"json": ReportFormat.Json, "md": ReportFormat.Markdown, "html": ReportFormat.Html}.get(ext, ReportFormat.Text)
        with open(path, "w") as f:
            f.write(self.format(fmt))
