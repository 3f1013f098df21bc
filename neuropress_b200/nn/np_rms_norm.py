"""NPRMSNorm: RMSNorm as one fused kernel, the step on the input side of the lowered linears.

Mirrors the reference's ``neuropress/nn/np_rms_norm.py``: :class:`NPRMSNorm` (:42-103) holds
the scale as a buffer and calls ``kernels.rms_norm``; :func:`linearize_rms_norms` (:158-208)
swaps every unfused RMSNorm of a model (class name contains ``RMSNorm``, one 1-D ``weight``
parameter, an ``eps`` attribute) whose weight is on a CUDA device.  Two conventions exist:
``x_normed * weight`` (Llama, Mistral) and ``x_normed * (1 + weight)`` (Gemma, Qwen3.5); the
kernel computes the first, so the ``+1`` is folded into the weight handed to the module, and
which convention a source module uses is found by probing it with its weight zeroed (:129-155).
"""

from __future__ import annotations

import logging

import torch
from torch import nn

__all__ = ["NPRMSNorm", "linearize_rms_norms"]

log = logging.getLogger(__name__)


class NPRMSNorm(nn.Module):
    """``x * rsqrt(mean(x**2, -1) + eps) * weight`` in one kernel, fp32 arithmetic."""

    def __init__(self, weight: torch.Tensor, eps: float = 1e-6, source: nn.Module | None = None) -> None:
        super().__init__()
        self.register_buffer("weight", weight.clone())
        self.eps = eps
        self.__dict__["_source"] = source  # outside the module tree: no state_dict entries

    def to_source_module(self) -> nn.Module | None:
        """The norm this module replaced (its own weight is unchanged, so it is the exact
        inverse of the swap), moved to this module's device; ``None`` when not recorded."""
        source = self.__dict__.get("_source")
        return None if source is None else source.to(self.weight.device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .. import kernels

        *leading, h = x.shape
        out = kernels.rms_norm(x.reshape(-1, h), self.weight.to(x.dtype), self.eps)
        return out.reshape(*leading, h)

    def extra_repr(self) -> str:
        return f"H={self.weight.shape[0]}, eps={self.eps}"


def _eps_of(module: nn.Module) -> float | None:
    """The epsilon of a source norm.  The reference looks for ``eps`` only
    (np_rms_norm.py:121-122); HuggingFace's Llama / Mistral / Qwen2 norms call it
    ``variance_epsilon``, which is accepted here as well."""
    for attr in ("eps", "variance_epsilon"):
        if hasattr(module, attr):
            return float(getattr(module, attr))
    return None


def _is_unfused_rms_norm(module: nn.Module) -> bool:
    if isinstance(module, NPRMSNorm) or "RMSNorm" not in type(module).__name__:
        return False
    params = dict(module.named_parameters(recurse=False))
    return set(params) == {"weight"} and params["weight"].dim() == 1 and _eps_of(module) is not None


def _uses_plus_one_convention(module: nn.Module, weight: torch.Tensor) -> bool:
    """Run the module's own forward on a random probe with its weight zeroed: a ``1 + weight``
    module still returns the normalised probe, a plain one returns zeros."""
    probe = torch.randn(1, weight.shape[0], device=weight.device, dtype=weight.dtype)
    saved = weight.clone()
    try:
        weight.zero_()
        with torch.no_grad():
            out = module(probe)
    finally:
        weight.copy_(saved)
    return bool(out.float().abs().max().item() > 1e-3)


def linearize_rms_norms(model: nn.Module, require_cuda: bool = True) -> int:
    """Replace the unfused RMSNorm modules of *model* in place; returns how many were replaced.
    Norms whose weight is not on a CUDA device are left alone (the kernel is CUDA-only) unless
    ``require_cuda`` is False (construction-only use, e.g. tests of the swap itself)."""
    from .. import _cabi

    if require_cuda and not _cabi.library_available():
        log.debug("linearize_rms_norms: kernel library not built - skipping")
        return 0
    targets = [(name, mod) for name, mod in model.named_modules()
               if _is_unfused_rms_norm(mod)
               and (not require_cuda or next(mod.parameters()).device.type == "cuda")]
    n_plus_one = 0
    for name, mod in targets:
        weight = next(mod.parameters()).data
        if _uses_plus_one_convention(mod, weight):
            effective = 1.0 + weight
            n_plus_one += 1
        else:
            effective = weight.clone()
        fused = NPRMSNorm(effective, eps=_eps_of(mod), source=mod).to(weight.device, weight.dtype)
        parent_name, _, attr = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, attr, fused)
    if targets:
        log.debug("linearize_rms_norms: replaced %d module(s) (%d used the '+1' convention)",
                  len(targets), n_plus_one)
    return len(targets)
