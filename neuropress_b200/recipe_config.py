"""Serialisable configuration of the kernel-lowering pass.

Mirrors the kernel-lowering part of the reference's ``neuropress/recipe_config.py``
(:209-286): a pydantic base class with a ``type`` discriminator, a registry filled by a class
decorator, and the ``"auto"`` configuration whose :meth:`build` returns an
:class:`~neuropress_b200.kernel_lowering.AutoKernelLowering`.  The rest of that file (recipes,
estimators, adapters) configures calibration and is outside this package.
"""

from __future__ import annotations

from typing import Callable, Literal

from pydantic import BaseModel

from .kernel_lowering import AutoKernelLowering, KernelLowering
from .nn.backends import EmbeddingBackend, LinearBackend, NormBackend, VQBackend

__all__ = ["AutoKernelLoweringConfig", "KERNEL_LOWERING_CONFIG_REGISTRY", "KernelLoweringConfig",
           "kernel_lowering_config", "resolve_kernel_lowering_config"]


class KernelLoweringConfig(BaseModel):
    """Base class of the JSON-serialisable lowering configurations (reference :209-225)."""

    type: str

    def build(self) -> KernelLowering:
        raise NotImplementedError(f"{type(self).__name__}.build()")


KERNEL_LOWERING_CONFIG_REGISTRY: dict[str, type[KernelLoweringConfig]] = {}


def kernel_lowering_config(name: str) -> Callable[[type[KernelLoweringConfig]], type[KernelLoweringConfig]]:
    """Class decorator: register a configuration class under *name* (its ``type`` value)."""

    def _decorate(cls: type[KernelLoweringConfig]) -> type[KernelLoweringConfig]:
        KERNEL_LOWERING_CONFIG_REGISTRY[name] = cls
        return cls

    return _decorate


@kernel_lowering_config("auto")
class AutoKernelLoweringConfig(KernelLoweringConfig):
    """Configuration of :class:`AutoKernelLowering` (reference :252-286): one backend per path,
    each constrained to the valid choices of that path."""

    type: Literal["auto"] = "auto"
    linear_backend: LinearBackend = LinearBackend.AUTO
    vq_backend: VQBackend = VQBackend.AUTO
    embedding_backend: EmbeddingBackend = EmbeddingBackend.AUTO
    norm_backend: NormBackend = NormBackend.AUTO

    def build(self) -> AutoKernelLowering:
        return AutoKernelLowering(
            linear_backend=self.linear_backend.value,
            vq_backend=self.vq_backend.value,
            embedding_backend=self.embedding_backend.value,
            norm_backend=self.norm_backend.value,
        )


def resolve_kernel_lowering_config(data: dict | KernelLoweringConfig | None) -> KernelLoweringConfig | None:
    """A configuration object from its dict form (``{"type": "auto", ...}``), by registry lookup;
    objects and ``None`` pass through.  Unknown types raise ``ValueError``."""
    if data is None or isinstance(data, KernelLoweringConfig):
        return data
    kind = data.get("type")
    if kind not in KERNEL_LOWERING_CONFIG_REGISTRY:
        raise ValueError(f"Unknown kernel lowering type {kind!r}; valid: {sorted(KERNEL_LOWERING_CONFIG_REGISTRY)}")
    return KERNEL_LOWERING_CONFIG_REGISTRY[kind].model_validate(data)
