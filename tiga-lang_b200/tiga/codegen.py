"""The ``b200-native`` code-generation provider and the registry it lives in.

The reference selects vendor back ends through a provider registry: entry-point
group ``tiga.codegen``, objects with a ``capabilities`` record and a
``compile(module, *, target, options)`` method, and a conformance report
(python/tiga/codegen/registry.py:11-97 of walkerchi/TIGA-lang).  This module
offers the same names -- ``ProviderCapabilities`` with the same fields,
``register_provider / get_provider / discover_providers /
provider_conformance`` -- and registers one provider, ``b200-native``.

The provider does not generate code.  Its kernels are hand-written CUDA,
precompiled for sm_100a into ``libtiga_b200.so``; ``compile`` resolves a
lowering name (what ``kernel.last_variant.lowering`` reports) to the C-ABI
entry points that implement it, and fails for anything else.  Its
``input_ir`` is ``"vendor-ir"``: the unit it accepts is a lowering name, not
TTIR or LLVM IR.

``adapt_to(registry_module)`` builds the same provider against another
registry module's own ``ProviderCapabilities`` class, which is what the
reference's ``provider_conformance`` type-checks; an installation that keeps
the reference's Python package registers it with
``tiga.codegen.register_provider("b200-native", adapt_to(tiga.codegen.registry))``
or through the entry point ``b200-native = tiga.codegen:provider_factory``.
"""
from __future__ import annotations

import dataclasses
from importlib import metadata
from typing import Any, Callable, Mapping

ABI_VERSION = 1
INPUT_IRS = ("ttir", "llvm", "msl", "vendor-ir")
ENTRY_POINT_GROUP = "tiga.codegen"


@dataclasses.dataclass(frozen=True)
class ProviderCapabilities:
    name: str
    target_family: str
    devices: tuple[str, ...]
    input_ir: str
    artifacts: tuple[str, ...]
    supports_async: bool
    supports_distributed: bool
    abi_version: int = ABI_VERSION

    def __post_init__(self) -> None:
        if self.abi_version != ABI_VERSION:
            raise ValueError("unsupported Tiga provider ABI")
        if not (self.name and self.target_family and self.devices):
            raise ValueError("provider capabilities must name a target/device")
        if self.input_ir not in INPUT_IRS:
            raise ValueError("provider input_ir is not recognized")


# lowering name -> the C-ABI entry points (include/tiga_b200.h) that implement it
LOWERINGS: dict[str, tuple[str, ...]] = {
    "b200-csr-weighted-sum-degree-bucket": ("tgb_csr_reduce_fwd", "tgb_csr_reduce_bwd_dx", "tgb_csr_reduce_bwd_dw"),
    "b200-csr-mean-degree-bucket": ("tgb_csr_reduce_fwd", "tgb_csr_reduce_bwd_dx", "tgb_csr_reduce_bwd_dw"),
    "b200-csr-max-degree-bucket": ("tgb_csr_reduce_fwd", "tgb_csr_reduce_bwd_dx", "tgb_csr_reduce_bwd_dw"),
    "b200-csr-additive-tuple-state": ("tgb_csr_reduce_fwd", "tgb_csr_reduce_bwd_dx", "tgb_csr_reduce_bwd_dw"),
    "b200-csr-edge-attention-online-softmax": ("tgb_gat_node_scores", "tgb_gat_fwd", "tgb_gat_bwd"),
    "b200-csr-stable-weighted-online-softmax": ("tgb_softmax_field_fwd", "tgb_softmax_field_bwd"),
    "b200-dense-streaming-reduction-tcgen05": ("tgb_varlen_attn_fwd", "tgb_varlen_attn_bwd"),
    "b200-halo-csr-weighted-sum": ("tgb_csr_reduce_fwd", "tgb_csr_reduce_bwd_dx", "tgb_csr_reduce_bwd_dw",
                                   "tgb_rows_gather", "tgb_rows_scatter_add"),
    "b200-dense-linear-3xtf32": ("tgb_linear_f32", "tgb_linear_dw_f32"),
}


@dataclasses.dataclass(frozen=True)
class CompiledLowering:
    """What ``compile`` returns: the library and the entry points of one lowering."""

    lowering: str
    library: str
    entry_points: tuple[str, ...]
    target: str


class B200NativeProvider:
    """Resolves lowering names to precompiled sm_100a kernels."""

    def __init__(self, capabilities_type=ProviderCapabilities) -> None:
        self.capabilities = capabilities_type(
            name="b200-native", target_family="cuda-sm100a", devices=("cuda",), input_ir="vendor-ir",
            artifacts=("shared-library",), supports_async=True, supports_distributed=True)

    def compile(self, module: str, *, target: Any | None = None, options: Mapping[str, Any] | None = None):
        from . import _native

        if module not in LOWERINGS:
            raise NotImplementedError(
                f"the b200-native provider has no kernel for {module!r}; it implements: {', '.join(sorted(LOWERINGS))}")
        if target not in (None, "cuda", "sm_100a", "cuda-sm100a"):
            raise NotImplementedError(f"the b200-native provider targets sm_100a only, not {target!r}")
        missing = [name for name in LOWERINGS[module] if name not in _native.exported_symbols()]
        if missing:
            raise RuntimeError(f"library interface lacks {missing}")
        return CompiledLowering(lowering=module, library=_native.library_path(), entry_points=LOWERINGS[module],
                                target="sm_100a")


def provider_factory() -> B200NativeProvider:
    return B200NativeProvider()


def adapt_to(registry_module) -> B200NativeProvider:
    """The provider with `registry_module`'s own ProviderCapabilities class."""
    return B200NativeProvider(registry_module.ProviderCapabilities)


# ------------------------------------------------------------------------------ registry
_registered: dict[str, Any] = {}
_entry_points_loaded = False


def _looks_like_provider(candidate) -> bool:
    return hasattr(candidate, "capabilities") and callable(getattr(candidate, "compile", None))


def register_provider(name: str, factory: Callable[[], Any] | Any, *, replace: bool = False) -> None:
    if not name:
        raise ValueError("provider name must not be empty")
    if not replace and name in _registered:
        raise ValueError(f"provider {name!r} is already registered")
    _registered[name] = factory


def discover_providers() -> tuple[str, ...]:
    """Names of all providers, after loading the ``tiga.codegen`` entry points once."""
    global _entry_points_loaded
    if not _entry_points_loaded:
        _entry_points_loaded = True
        for entry in metadata.entry_points(group=ENTRY_POINT_GROUP):
            register_provider(entry.name, entry.load(), replace=True)
    return tuple(sorted(_registered))


def get_provider(name: str):
    names = discover_providers()
    if name not in _registered:
        raise LookupError(f"Tiga codegen provider {name!r} is unavailable; installed: {', '.join(names) or 'none'}")
    candidate = _registered[name]
    provider = candidate if _looks_like_provider(candidate) else candidate()
    if not _looks_like_provider(provider):
        raise TypeError(f"provider {name!r} does not implement CodegenProvider")
    return provider


def provider_conformance(provider) -> dict[str, object]:
    """The stable-ABI report of a provider (says nothing about hardware correctness)."""
    if not _looks_like_provider(provider):
        raise TypeError("provider does not implement CodegenProvider")
    capabilities = provider.capabilities
    wanted = [f.name for f in dataclasses.fields(ProviderCapabilities)]
    if any(not hasattr(capabilities, name) for name in wanted):
        raise TypeError("provider capabilities have the wrong type")
    report = {name: getattr(capabilities, name) for name in wanted}
    return {"abi_version": report.pop("abi_version"), **report}


register_provider("b200-native", provider_factory)

__all__ = ["B200NativeProvider", "CompiledLowering", "LOWERINGS", "ProviderCapabilities", "adapt_to",
           "discover_providers", "get_provider", "provider_conformance", "provider_factory", "register_provider"]
