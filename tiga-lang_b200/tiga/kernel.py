"""What a kernel object remembers about the launch plans it has used.

A ``Kernel`` (``MessagePassing`` and the reducers derive from it) keeps one
``CompiledVariant`` per specialisation it has executed.  In this build a
variant is a record of a launch plan of the native CUDA library -- which
recogniser matched, which kernels run, what the degree planner found -- not a
compiled module: the kernels are precompiled into the shared library.

The names a program can read are those of the reference's kernel model
(python/tiga/kernel/model.py:7-229 of walkerchi/TIGA-lang): ``variants``,
``last_variant``, ``cache_info``, ``explain()``, ``diagnostics``,
``schedules``, ``ir(stage)``, ``code(kind)``, and on a variant ``key``,
``backend``, ``provider``, ``lowering``, ``passes``, ``remarks``,
``findings``, ``artifacts``.  ``explain()`` prints the same line layout
(``backend: / provider: / lowering: / passes: / <disposition>: [stage] text /
variant cache: hits=.., misses=..``) because programs and tests grep it.
"""
from __future__ import annotations

import dataclasses
from collections import OrderedDict
from typing import Any, Iterator

DISPOSITIONS = frozenset({"accepted", "rejected", "warning", "unknown", "remark"})


@dataclasses.dataclass(frozen=True)
class AnalysisFinding:
    """One line of planner output: where it came from, how it was disposed of, the text."""

    stage: str
    disposition: str
    message: str
    source_location: str | None = None
    affected_resource: str | None = None
    target_contract: str | None = None
    estimate: str | None = None
    suggested_action: str | None = None

    def __post_init__(self) -> None:
        for name in ("stage", "message"):
            if not getattr(self, name):
                raise ValueError(f"an analysis finding needs a non-empty {name}")
        if self.disposition not in DISPOSITIONS:
            raise ValueError(f"disposition must be one of {sorted(DISPOSITIONS)}, got {self.disposition!r}")

    def line(self) -> str:
        return f"{self.disposition}: [{self.stage}] {self.message}"


@dataclasses.dataclass(frozen=True)
class CompiledVariant:
    """The record of one specialisation: cache key, where it runs, how it was lowered."""

    key: tuple[object, ...]
    backend: str
    provider: str
    domain_plan: str
    passes: tuple[str, ...]
    lowering: str | None = None
    provider_key: tuple[str, ...] = ()
    artifacts: dict[str, str] = dataclasses.field(default_factory=dict)
    remarks: tuple[str, ...] = ()
    findings: tuple[AnalysisFinding, ...] = ()
    schedules: tuple[Any, ...] = ()

    # ---------------------------------------------------------------- findings
    def _all_findings(self) -> Iterator[AnalysisFinding]:
        yield from self.findings
        for text in self.remarks:
            yield AnalysisFinding(stage="planning", disposition="remark", message=text)

    @property
    def diagnostics(self) -> tuple[AnalysisFinding, ...]:
        """Structured findings first, then every free-text remark as a ``remark`` finding."""
        return tuple(self._all_findings())

    # --------------------------------------------------------------- artifacts
    def _stages(self) -> list[str]:
        return ["domain", *sorted(self.artifacts)]

    def ir(self, stage: str = "domain") -> str:
        """Text of one stage.  Only the domain plan always exists; this build keeps no MLIR."""
        if stage in ("domain", "domain-plan"):
            return self.domain_plan
        text = self.artifacts.get(stage)
        if not isinstance(text, str):
            raise KeyError(f"IR/artifact stage {stage!r} is unavailable; have: {', '.join(self._stages())}")
        return text

    def code(self, kind: str) -> str:
        if kind not in self.artifacts:
            raise KeyError(f"artifact {kind!r} is unavailable for provider {self.provider!r}")
        return self.artifacts[kind]

    # ----------------------------------------------------------------- report
    def explain(self) -> str:
        report = [
            ("backend", self.backend),
            ("provider", self.provider),
            ("lowering", self.lowering if self.lowering else "(unspecified)"),
            ("passes", ", ".join(self.passes) if self.passes else "(none)"),
        ]
        if self.provider_key:
            report.append(("provider cache key", " | ".join(self.provider_key)))
        lines = [f"{label}: {text}" for label, text in report]
        lines += [finding.line() for finding in self._all_findings()]
        return "\n".join(lines)


class VariantCache:
    """Insertion-ordered map from specialisation key to variant, with hit / miss counters
    and a pointer to the variant used last."""

    def __init__(self) -> None:
        self.entries: "OrderedDict[tuple[object, ...], CompiledVariant]" = OrderedDict()
        self.hits = 0
        self.misses = 0
        self.last: CompiledVariant | None = None

    def find(self, key) -> CompiledVariant | None:
        hit = self.entries.get(key)
        if hit is not None:
            self.last = hit
        return hit

    def store(self, variant: CompiledVariant) -> None:
        self.entries[variant.key] = variant
        self.last = variant

    def counters(self) -> dict[str, int]:
        return {"hits": self.hits, "misses": self.misses, "variants": len(self.entries)}


class Kernel:
    """Base of everything callable in the package: owns the variant cache and the reporting API."""

    def __init__(self) -> None:
        self._cache = VariantCache()

    # The counters are plain attributes of the reference's Kernel; subclasses here bump them too.
    @property
    def _cache_hits(self) -> int:
        return self._cache.hits

    @_cache_hits.setter
    def _cache_hits(self, value: int) -> None:
        self._cache.hits = value

    @property
    def _cache_misses(self) -> int:
        return self._cache.misses

    @_cache_misses.setter
    def _cache_misses(self, value: int) -> None:
        self._cache.misses = value

    def _lookup_variant(self, key) -> CompiledVariant | None:
        return self._cache.find(key)

    def _record_variant(self, variant: CompiledVariant) -> None:
        self._cache.store(variant)

    # ------------------------------------------------------------------ public
    @property
    def variants(self) -> tuple[CompiledVariant, ...]:
        return tuple(self._cache.entries.values())

    @property
    def last_variant(self) -> CompiledVariant:
        if self._cache.last is None:
            raise RuntimeError("kernel has not been called, so no JIT variant exists")
        return self._cache.last

    @property
    def cache_info(self) -> dict[str, int]:
        return self._cache.counters()

    @property
    def diagnostics(self) -> tuple[AnalysisFinding, ...]:
        return self.last_variant.diagnostics

    @property
    def schedules(self) -> tuple[Any, ...]:
        return self.last_variant.schedules

    def ir(self, stage: str = "domain") -> str:
        return self.last_variant.ir(stage)

    def code(self, kind: str = "ptx") -> str:
        return self.last_variant.code(kind)

    def explain(self) -> str:
        counters = self._cache.counters()
        tail = f"variant cache: hits={counters['hits']}, misses={counters['misses']}"
        return f"{self.last_variant.explain()}\n{tail}"


__all__ = ["AnalysisFinding", "CompiledVariant", "Kernel", "VariantCache"]
