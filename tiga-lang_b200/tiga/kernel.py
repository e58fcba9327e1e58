"""Kernel base: variant cache, CompiledVariant, explain()/cache_info.

Mirrors python/tiga/kernel/model.py:7-229 of the reference (same public
attributes and explain() line format) without the MLIR-specific schedule
parsing: a variant here describes a launch plan of the native CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class AnalysisFinding:
    stage: str
    disposition: str
    message: str
    source_location: str | None = None
    affected_resource: str | None = None
    target_contract: str | None = None
    estimate: str | None = None
    suggested_action: str | None = None

    def __post_init__(self) -> None:
        if not self.stage or not self.message:
            raise ValueError("analysis findings require a stage and message")
        if self.disposition not in {"accepted", "rejected", "warning", "unknown", "remark"}:
            raise ValueError("invalid analysis finding disposition")


@dataclass(frozen=True)
class CompiledVariant:
    key: tuple[object, ...]
    backend: str
    provider: str
    domain_plan: str
    passes: tuple[str, ...]
    lowering: str | None = None
    provider_key: tuple[str, ...] = ()
    artifacts: dict[str, str] = field(default_factory=dict)
    remarks: tuple[str, ...] = ()
    findings: tuple[AnalysisFinding, ...] = ()
    schedules: tuple[Any, ...] = ()

    @property
    def diagnostics(self) -> tuple[AnalysisFinding, ...]:
        return (*self.findings, *(AnalysisFinding("planning", "remark", remark) for remark in self.remarks))

    def ir(self, stage: str = "domain") -> str:
        if stage in {"domain", "domain-plan"}:
            return self.domain_plan
        artifact = self.artifacts.get(stage)
        if isinstance(artifact, str):
            return artifact
        available = ", ".join(["domain", *sorted(self.artifacts)])
        raise KeyError(f"IR/artifact stage {stage!r} is unavailable; have: {available}")

    def code(self, kind: str) -> str:
        try:
            return self.artifacts[kind]
        except KeyError as exc:
            raise KeyError(f"artifact {kind!r} is unavailable for provider {self.provider!r}") from exc

    def explain(self) -> str:
        lines = [
            f"backend: {self.backend}",
            f"provider: {self.provider}",
            f"lowering: {self.lowering or '(unspecified)'}",
            f"passes: {', '.join(self.passes) if self.passes else '(none)'}",
        ]
        if self.provider_key:
            lines.append(f"provider cache key: {' | '.join(self.provider_key)}")
        lines.extend(f"{finding.disposition}: [{finding.stage}] {finding.message}" for finding in self.diagnostics)
        return "\n".join(lines)


class Kernel:
    def __init__(self) -> None:
        self._variants: dict[tuple[object, ...], CompiledVariant] = {}
        self._last_variant: CompiledVariant | None = None
        self._cache_hits = 0
        self._cache_misses = 0

    @property
    def variants(self) -> tuple[CompiledVariant, ...]:
        return tuple(self._variants.values())

    @property
    def last_variant(self) -> CompiledVariant:
        if self._last_variant is None:
            raise RuntimeError("kernel has not been called, so no JIT variant exists")
        return self._last_variant

    def ir(self, stage: str = "domain") -> str:
        return self.last_variant.ir(stage)

    def code(self, kind: str = "ptx") -> str:
        return self.last_variant.code(kind)

    def explain(self) -> str:
        return "\n".join((self.last_variant.explain(),
                          f"variant cache: hits={self._cache_hits}, misses={self._cache_misses}"))

    @property
    def diagnostics(self) -> tuple[AnalysisFinding, ...]:
        return self.last_variant.diagnostics

    @property
    def schedules(self) -> tuple[Any, ...]:
        return self.last_variant.schedules

    @property
    def cache_info(self) -> dict[str, int]:
        return {"hits": self._cache_hits, "misses": self._cache_misses, "variants": len(self._variants)}

    def _record_variant(self, variant: CompiledVariant) -> None:
        self._variants[variant.key] = variant
        self._last_variant = variant

    def _lookup_variant(self, key: tuple[Any, ...]) -> CompiledVariant | None:
        variant = self._variants.get(key)
        if variant is not None:
            self._last_variant = variant
        return variant
