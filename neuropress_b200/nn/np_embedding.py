"""NPEmbedding: ``nn.Embedding`` replacement whose weight is a packed group-affine table.

Same surface as the reference module (neuropress/nn/np_embedding.py): buffers ``u8_blob``
``[V, D * nbits / 8]``, ``scale`` and ``zero_point`` (flattened fp16, one per group), the
constructor arguments of :233-301, ``from_embedding`` / ``to_qtensor`` / ``set_backend``.  The
reference's ``cuda`` backend gathers the selected rows in packed space and dequantises them with
eager PyTorch ops (``_emb_dequant``, :120-183); here that is one CUDA kernel
(``npb_q_embedding``) with the same arithmetic: ``fp16((q - zp) * s)`` in fp32 with one rounding
per operation, the padding row zeroed, a cast to ``out_dtype`` and the ``embed_scale`` multiply
(:449-473).  ``auto`` resolves to ``cuda``; ``default`` / ``compile`` are accepted as names and
raise at forward time (no eager, compiled or CPU path exists in this package).
"""

from __future__ import annotations

import logging

import torch
import torch.nn as nn

from .backends import Backend, EmbeddingBackend

log = logging.getLogger(__name__)


def _resolve_backend_emb(backend: str | EmbeddingBackend | Backend | None, nbits: int | None = None,
                         group_size: int | None = None) -> EmbeddingBackend:
    """Alias -> concrete :class:`EmbeddingBackend` (reference :77-112; ``auto`` -> ``cuda``:
    the lookup kernel needs no warm-up and there is no compiled path here)."""
    if backend is None or backend == "torch":
        return EmbeddingBackend.DEFAULT
    val = backend.value if isinstance(backend, EmbeddingBackend | Backend) else str(backend)
    if val == "auto":
        return EmbeddingBackend.CUDA
    return EmbeddingBackend(val)  # raises ValueError for unknown strings (gemlite included)


class NPEmbedding(nn.Module):
    """Embedding layer with packed n-bit group-quantized weight (reference :203-526)."""

    def __init__(self, u8_blob: torch.Tensor, scale: torch.Tensor, num_embeddings: int, embedding_dim: int,
                 group_size: int, nbits: int, qtype: str, backend: str | EmbeddingBackend | None,
                 padding_idx: int | None = None, zero_point: torch.Tensor | None = None,
                 weight_q=None, qtensor_meta: dict | None = None, embed_scale: float = 1.0,
                 out_dtype: torch.dtype | None = None) -> None:
        super().__init__()
        if qtype not in ("sym", "asym"):
            raise ValueError("qtype must be 'sym' or 'asym'.")
        if (qtype == "asym") != (zero_point is not None):
            raise ValueError("zero_point goes with qtype='asym' and only with it.")
        self._qtensor_meta = qtensor_meta
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.group_size = group_size
        self.nbits = nbits
        self.qtype = qtype
        self.padding_idx = padding_idx
        self.embed_scale = embed_scale
        self.out_dtype = out_dtype
        self.backend = _resolve_backend_emb(backend, nbits=nbits, group_size=group_size)
        if weight_q is not None:
            object.__setattr__(self, "_weight_q", weight_q)
        self.register_buffer("u8_blob", u8_blob.contiguous())
        self.register_buffer("scale", scale.reshape(-1).to(torch.float16).contiguous())
        self.register_buffer("zero_point", None if zero_point is None
                             else zero_point.reshape(-1).to(torch.float16).contiguous())

    @classmethod
    def from_embedding(cls, embedding: nn.Embedding,
                       backend: str | EmbeddingBackend | None = EmbeddingBackend.AUTO) -> "NPEmbedding":
        """Build from an ``nn.Embedding`` whose ``weight`` is a group-affine QTensor (reference
        :303-375).  The weight is read by attribute, like ``NPLinear.from_linear`` reads it:
        ``weight.qscheme.{n_bits, group_size, scale, per_group_zero_point()}``, ``weight.u8_blob``."""
        from .np_linear import _kernel_blob

        w = embedding._parameters.get("weight")
        qs = getattr(w, "qscheme", None)
        if qs is None or not hasattr(qs, "n_bits") or not hasattr(w, "u8_blob"):
            raise TypeError(f"Unsupported weight type {type(w).__name__!r}: expected a group-affine QTensor.")
        zp = qs.per_group_zero_point() if hasattr(qs, "per_group_zero_point") else None
        es = getattr(embedding, "embed_scale", None)
        embed_scale = 1.0 if es is None else float(es.item() if isinstance(es, torch.Tensor) else es)
        meta = w.serde_metadata() if hasattr(w, "serde_metadata") else {}
        return cls(_kernel_blob(w), qs.scale.detach().clone(), embedding.num_embeddings, embedding.embedding_dim,
                   qs.group_size, qs.n_bits, "sym" if zp is None else "asym", backend,
                   padding_idx=embedding.padding_idx, zero_point=None if zp is None else zp.detach().clone(),
                   qtensor_meta=meta, embed_scale=embed_scale,
                   out_dtype=getattr(w, "dequant_to_dtype", None) or getattr(w, "dtype", None))

    def to_qtensor(self):
        """Rebuild the group-affine QTensor stand-in for saving / unlowering (reference :381-408)."""
        if self._qtensor_meta is None:
            raise RuntimeError("Cannot reconstruct QTensor: no serde metadata stored. "
                               "Build via NPEmbedding.from_embedding() to enable to_qtensor().")
        from ..qtensor import AffineQTensor, AffineScheme

        scheme = AffineScheme(self.nbits, self.group_size, self.scale, self.zero_point)
        meta = {k: v for k, v in self._qtensor_meta.items() if k not in ("type", "shape")}
        return AffineQTensor(self.u8_blob, scheme, (self.num_embeddings, self.embedding_dim),
                             self.out_dtype or torch.float16, meta)

    def set_backend(self, backend: str | EmbeddingBackend | None) -> "NPEmbedding":
        bk = _resolve_backend_emb(backend, nbits=self.nbits, group_size=self.group_size)
        if bk == EmbeddingBackend.DEFAULT and not hasattr(self, "_weight_q"):
            raise RuntimeError("Cannot switch to EmbeddingBackend.DEFAULT: the original QTensor was not retained.")
        self.backend = bk
        return self

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.backend != EmbeddingBackend.CUDA:
            raise NotImplementedError(f"backend {self.backend.value!r} is not implemented by this package: "
                                      "only 'cuda' exists here; there is no eager or compiled path.")
        from .. import kernels

        return kernels.q_embedding(x, self.u8_blob, self.scale, self.nbits, self.group_size, self.zero_point,
                                   self.padding_idx, float(self.embed_scale), self.out_dtype)

    def extra_repr(self) -> str:
        parts = [f"num_embeddings={self.num_embeddings}", f"embedding_dim={self.embedding_dim}",
                 f"nbits={self.nbits}", f"group_size={self.group_size}", f"qtype={self.qtype}",
                 f"backend={self.backend.value}"]
        if self.padding_idx is not None:
            parts.append(f"padding_idx={self.padding_idx}")
        return ", ".join(parts)


def _is_affine_weight(w) -> bool:
    q = getattr(w, "qscheme", None)
    return q is not None and hasattr(q, "n_bits") and hasattr(q, "group_size") and hasattr(w, "u8_blob")


def linearize_qtensor_embeddings(model: nn.Module,
                                 backend: str | EmbeddingBackend | None = EmbeddingBackend.AUTO) -> nn.Module:
    """Replace every ``nn.Embedding`` whose weight is a group-affine QTensor by an
    :class:`NPEmbedding` (reference :528-595).  Returns *model*."""
    replacements: list[tuple[str, NPEmbedding]] = []
    for name, module in model.named_modules():
        if not isinstance(module, nn.Embedding) or not _is_affine_weight(module._parameters.get("weight")):
            continue
        try:
            replacements.append((name, NPEmbedding.from_embedding(module, backend)))
        except (TypeError, ValueError) as exc:
            log.warning("linearize_qtensor_embeddings: skipping %s — %s", name, exc)
    for name, emb in replacements:
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], emb)
    log.info("linearize_qtensor_embeddings: replaced %d layer(s) with NPEmbedding[%s]", len(replacements),
             _resolve_backend_emb(backend).value)
    return model
