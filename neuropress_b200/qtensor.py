"""Duck-typed stand-ins for the QTensor weight classes the lowering reads.

The reference's quantized weights are ``torch_to_nnef`` QTensor subclasses
(neuropress/transforms/vq.py ``QTensorTractVQ`` / ``VQScheme``;
neuropress/transforms/weight_only.py ``QTensorScaleZp``; torch_to_nnef's
``QTensorTractScaleOnly``).  That third-party package is not a dependency here.  The lowering
(``linearize_*``, ``from_qtensor_linear``, ``from_linear``) only reads a handful of attributes,
listed in each class below; any object that has them — the reference's real classes included —
is accepted.  These plain containers provide them for tests, benchmarks and ``to_qtensor()``.
They hold data only: no arithmetic happens here.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(eq=False)
class VQScheme:
    """Attributes read by ``NPVQLinear.from_qtensor_linear`` (reference np_vq_linear.py:863-879)."""

    centroids: torch.Tensor                 # [NC, VL]
    vector_len: int
    is_packed_indices: int                  # bits per index
    column_permutation: torch.Tensor | None = None
    use_tiered: bool = False
    tier_bits: list[int] | None = None
    zero_escape: bool = False
    original_shape: tuple[int, int] | None = None   # read by linearize_vq_embeddings (np_vq_embedding.py:206-212)


@dataclass(eq=False)
class VQQTensor:
    """A VQ weight: ``u8_blob`` (LSB-first index bit-stream) + ``qscheme``."""

    u8_blob: torch.Tensor
    qscheme: VQScheme
    shape: tuple[int, int]
    meta: dict = field(default_factory=dict)

    dequant_to_dtype: torch.dtype | None = None

    def __post_init__(self) -> None:
        if self.dequant_to_dtype is None:
            self.dequant_to_dtype = getattr(torch, self.meta.get("dequant_to_dtype", "float16"))
        else:
            self.meta.setdefault("dequant_to_dtype", str(self.dequant_to_dtype).replace("torch.", ""))

    def serde_metadata(self) -> dict:
        """What a lowered module keeps to rebuild this weight: the checkpoint fields that are not
        buffers of the module (plus type and shape, for inspection)."""
        return {"type": "QTensorTractVQ", "shape": list(self.shape) if self.shape else None, **self.meta}


@dataclass(eq=False)
class AffineScheme:
    """Attributes read by ``NPLinear.from_linear`` (reference np_linear.py:573-610)."""

    n_bits: int
    group_size: int
    scale: torch.Tensor                     # fp16, N*K/group_size elements (any shape)
    zero_point: torch.Tensor | None = None  # fp16 per group, or None for the symmetric scheme

    def per_group_zero_point(self) -> torch.Tensor | None:
        return self.zero_point


@dataclass(eq=False)
class AffineQTensor:
    """A group-affine weight: ``u8_blob`` is ``[N, K*n_bits/8]`` codes packed LSB-first."""

    u8_blob: torch.Tensor
    qscheme: AffineScheme
    shape: tuple[int, int]
    dequant_to_dtype: torch.dtype = torch.float16
    meta: dict = field(default_factory=dict)

    @property
    def symmetric(self) -> bool:
        return self.qscheme.zero_point is None

    def serde_metadata(self) -> dict:
        name = "QTensorTractScaleOnly" if self.symmetric else "QTensorScaleZp"
        return {"type": name, "shape": list(self.shape), **self.meta}
