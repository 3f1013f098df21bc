"""Kernel lowering: swap QTensor-backed ``nn.Linear`` modules for the CUDA-backed NP* modules.

Same surface as the reference's ``neuropress/kernel_lowering.py``: :class:`LoweringConfig`
(:43-116; four string fields, unknown keys rejected, YAML / dict / ``None``),
:class:`AutoKernelLowering` (:154-249), :func:`is_lowered` (:257-277), :func:`unlower_model`
(:280-368).  The two linear passes (``linearize_qtensor_weights`` then ``linearize_vq_weights``, in the
reference's order) and the RMSNorm pass exist here; the embedding pass of the reference is
outside this package, so ``embedding_backend`` is carried in the configuration but has no
effect.
"""

from __future__ import annotations

import logging
from abc import ABC, abstractmethod
from dataclasses import asdict, dataclass
from pathlib import Path

import torch
from torch import nn

__all__ = ["AutoKernelLowering", "KernelLowering", "LoweringConfig", "is_lowered", "unlower_model"]

LOGGER = logging.getLogger(__name__)

_VALID_FIELDS = frozenset({"vq_backend", "linear_backend", "embedding_backend", "norm_backend"})


@dataclass
class LoweringConfig:
    """Per-path backend names; ``"auto"`` picks the CUDA kernels of this package."""

    vq_backend: str = "auto"
    linear_backend: str = "auto"
    embedding_backend: str = "auto"
    norm_backend: str = "auto"

    @classmethod
    def from_dict(cls, d: dict) -> "LoweringConfig":
        unknown = set(d) - _VALID_FIELDS
        if unknown:
            raise ValueError(
                f"Unknown lowering config key(s): {sorted(unknown)}. Valid: {sorted(_VALID_FIELDS)}"
            )
        return cls(**{k: str(v) for k, v in d.items()})

    @classmethod
    def from_file(cls, path: Path | str) -> "LoweringConfig":
        import yaml

        with open(path) as fh:
            data = yaml.safe_load(fh) or {}
        if not isinstance(data, dict):
            raise ValueError(f"{path}: expected a YAML mapping, got {type(data).__name__}")
        return cls.from_dict(data)

    @classmethod
    def load(cls, src: Path | str | dict | None) -> "LoweringConfig":
        if src is None:
            return cls()
        if isinstance(src, dict):
            return cls.from_dict(src)
        return cls.from_file(src)

    def save(self, path: Path | str) -> None:
        import yaml

        p = Path(path)
        p.parent.mkdir(parents=True, exist_ok=True)
        with p.open("w") as fh:
            yaml.safe_dump(asdict(self), fh, default_flow_style=False, sort_keys=True)


class KernelLowering(ABC):
    """Replace QTensor-backed modules with hardware-specific modules, in place."""

    @abstractmethod
    def apply(self, model: nn.Module) -> None:
        """Lower *model* in place."""


class AutoKernelLowering(KernelLowering):
    """Run the linearize passes with per-path backends (reference :154-249)."""

    def __init__(self, linear_backend: str = "auto", vq_backend: str = "auto",
                 embedding_backend: str = "auto", norm_backend: str = "auto") -> None:
        self.linear_backend = linear_backend
        self.vq_backend = vq_backend
        self.embedding_backend = embedding_backend
        self.norm_backend = norm_backend

    @classmethod
    def from_config(cls, src: Path | str | dict | LoweringConfig | None = None) -> "AutoKernelLowering":
        cfg = src if isinstance(src, LoweringConfig) else LoweringConfig.load(src)
        return cls(linear_backend=cfg.linear_backend, vq_backend=cfg.vq_backend,
                   embedding_backend=cfg.embedding_backend, norm_backend=cfg.norm_backend)

    def apply(self, model: nn.Module) -> None:
        """The five passes in the reference's order (:200-249): affine embeddings, affine
        linears, VQ linears, VQ embeddings, RMSNorm modules."""
        from .nn.np_embedding import NPEmbedding, linearize_qtensor_embeddings
        from .nn.np_linear import NPLinear, linearize_qtensor_weights
        from .nn.np_vq_embedding import NPVQEmbedding, linearize_vq_embeddings
        from .nn.np_vq_linear import NPVQLinear, linearize_vq_weights

        linearize_qtensor_embeddings(model, backend=self.embedding_backend)
        linearize_qtensor_weights(model, backend=self.linear_backend)
        linearize_vq_weights(model, backend=self.vq_backend)
        linearize_vq_embeddings(model)
        n_norms = 0
        if self.norm_backend in ("auto", "cuda"):  # "default" keeps the model's own norms
            from .nn.np_rms_norm import linearize_rms_norms

            n_norms = linearize_rms_norms(model)
        # A lowered lm_head no longer shares storage with the embedding (reference :221-227).
        if hasattr(model, "config") and hasattr(model.config, "tie_word_embeddings"):
            model.config.tie_word_embeddings = False
        counts: dict[str, int] = {}
        for m in model.modules():
            if isinstance(m, NPLinear | NPVQLinear | NPEmbedding):
                key = f"{type(m).__name__}({m.backend.value})"
                counts[key] = counts.get(key, 0) + 1
            elif isinstance(m, NPVQEmbedding):
                counts["NPVQEmbedding"] = counts.get("NPVQEmbedding", 0) + 1
        if n_norms:
            counts["NPRMSNorm(cuda)"] = n_norms
        if counts:
            LOGGER.warning("Kernel lowering applied: %s",
                           ", ".join(f"{v}x {k}" for k, v in sorted(counts.items())))
        else:
            LOGGER.warning("Kernel lowering: no modules were lowered.")


def is_lowered(model: nn.Module) -> bool:
    """``True`` if *model* contains any lowered NP* module (reference :257-277)."""
    from .nn.np_embedding import NPEmbedding
    from .nn.np_linear import NPLinear
    from .nn.np_vq_embedding import NPVQEmbedding
    from .nn.np_vq_linear import NPVQLinear

    return any(isinstance(m, NPLinear | NPVQLinear | NPEmbedding | NPVQEmbedding) for m in model.modules())


def unlower_model(model: nn.Module) -> None:
    """Inverse of :meth:`AutoKernelLowering.apply`: put each NP* module's ``to_qtensor()`` back
    into a plain ``nn.Linear`` built on the meta device (no dense weight is allocated), then
    drop the ``_vq_proxy_*`` modules from the model root (reference :280-368)."""
    from .nn.np_linear import NPLinear
    from .nn.np_vq_linear import NPVQLinear

    replacements: list[tuple[str, nn.Module]] = []
    for name, module in model.named_modules():
        if isinstance(module, NPLinear | NPVQLinear):
            qtensor = module.to_qtensor()
            has_bias = module.bias is not None
            with torch.device("meta"):
                linear = nn.Linear(module.in_features, module.out_features, bias=has_bias)
            linear._parameters["weight"] = qtensor
            if has_bias:
                linear._parameters["bias"] = module.bias
            replacements.append((name, linear))
    for name, new_mod in replacements:
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], new_mod)
    # embeddings go back to nn.Embedding shells holding their QTensor (reference :316-352)
    from .nn.np_embedding import NPEmbedding
    from .nn.np_vq_embedding import NPVQEmbedding

    for name, module in list(model.named_modules()):
        if not isinstance(module, NPEmbedding | NPVQEmbedding):
            continue
        qtensor = module.to_qtensor()
        if isinstance(module, NPEmbedding):
            vocab, dim, pad = module.num_embeddings, module.embedding_dim, module.padding_idx
        else:
            vocab, dim, pad = module.all_indices.shape[0], module.embedding_dim, None
        with torch.device("meta"):
            emb = nn.Embedding(vocab, dim, padding_idx=pad)
        emb._parameters["weight"] = qtensor
        scale = module.embed_scale if isinstance(module, NPEmbedding) else module.scale
        if scale != 1.0:
            emb.embed_scale = scale
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], emb)
        replacements.append((name, emb))
    for pname in [n for n, _ in model.named_children()
                  if n.startswith("_vq_proxy_") or n.startswith("_vq_emb_proxy_")]:
        delattr(model, pname)
    # fused norms go back to the modules they replaced
    from .nn.np_rms_norm import NPRMSNorm

    for name, module in list(model.named_modules()):
        if isinstance(module, NPRMSNorm):
            source = module.to_source_module()
            if source is not None:
                parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
                setattr(parent, name.rsplit(".", 1)[-1], source)
    LOGGER.info("unlower_model: restored %d module(s) to QTensor form", len(replacements))
