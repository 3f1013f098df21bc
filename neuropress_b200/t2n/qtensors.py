"""Checkpoint serde of the quantized weights, in the reference's on-disk layout.

The reference stores every QTensor as a few safetensors entries plus a string-to-string metadata
dict, looked up by the QTensor's class name (neuropress/t2n/qtensors.py: ``QTensorTractScaleOnly``
:292-352, ``QTensorScaleZp`` :360-423, ``QTensorTractVQ`` :431-556).  Its QTensor classes come
from ``torch_to_nnef``, which is not a dependency here; the handlers below read and build the
duck-typed stand-ins of :mod:`neuropress_b200.qtensor` instead, and produce / accept exactly the
same entries, shapes, metadata keys and values, so a file written by either side loads on the
other.  Identical codebooks are shared again on load through a content-hash cache (:57-70,
:506-523), which is what keeps one ``VQProxy`` per codebook after lowering.
"""

from __future__ import annotations

import hashlib
import json
from typing import Any
from weakref import WeakValueDictionary

import torch

from ..qtensor import AffineQTensor, AffineScheme, VQQTensor, VQScheme

_TYPE_KEY = "__qtensor_type__"
_vq_centroid_cache: "WeakValueDictionary[str, torch.Tensor]" = WeakValueDictionary()


def _centroid_hash(centroids: torch.Tensor) -> str:
    """SHA-256 of the codebook's fp16 bytes (reference :66-69)."""
    return hashlib.sha256(centroids.to(torch.float16).cpu().contiguous().numpy().tobytes()).hexdigest()


def _dtype_name(dtype: torch.dtype) -> str:
    return str(dtype).replace("torch.", "")


def qtensor_type_name(q: Any) -> str | None:
    """The reference's class name for a quantized weight, or ``None`` for anything else."""
    if isinstance(q, VQQTensor):
        return "QTensorTractVQ"
    if isinstance(q, AffineQTensor):
        return "QTensorTractScaleOnly" if q.symmetric else "QTensorScaleZp"
    name = type(q).__name__
    return name if name in _SERDE_REGISTRY and hasattr(q, "u8_blob") else None


class QTensorSerde:
    """One handler per reference class name: tensors + metadata <-> stand-in object."""

    name = ""

    def to_tensors(self, q: Any) -> dict[str, torch.Tensor]:
        raise NotImplementedError

    def to_metadata(self, q: Any) -> dict[str, str]:
        raise NotImplementedError

    def from_parts(self, tensors: dict[str, torch.Tensor], metadata: dict[str, str]) -> Any:
        raise NotImplementedError


class _AffineSerde(QTensorSerde):
    """``QTensorTractScaleOnly`` (reference :292-352) and, with a zero-point, ``QTensorScaleZp``
    (:360-423).  Entries ``u8_blob`` (as stored), ``scale`` / ``zero_point`` as ``[groups, 1]``."""

    def __init__(self, name: str, asym: bool) -> None:
        self.name, self.asym = name, asym

    def to_tensors(self, q: Any) -> dict[str, torch.Tensor]:
        out = {"u8_blob": q.u8_blob, "scale": q.qscheme.scale.reshape(-1, 1)}
        if self.asym:
            out["zero_point"] = q.qscheme.zero_point.reshape(-1, 1)
        return out

    def to_metadata(self, q: Any) -> dict[str, str]:
        meta = getattr(q, "meta", {}) or {}
        n_bits = q.qscheme.n_bits
        packed = q.u8_blob.numel() < q.shape[0] * q.shape[1]
        md = {
            "shape": json.dumps([int(d) for d in q.shape]),
            "packing": meta.get("packing", json.dumps([n_bits] if packed else [])),
            "n_bits": str(n_bits),
            "group_size": str(q.qscheme.group_size),
            "dequant_to_dtype": _dtype_name(q.dequant_to_dtype),
            "nnef_name": meta.get("nnef_name", ""),
        }
        if self.asym:
            md["export_as_float"] = meta.get("export_as_float", "0")
        return md

    def from_parts(self, tensors: dict[str, torch.Tensor], metadata: dict[str, str]) -> Any:
        zp = tensors["zero_point"] if self.asym else None
        scheme = AffineScheme(int(metadata["n_bits"]), int(metadata["group_size"]), tensors["scale"], zp)
        blob = tensors["u8_blob"]
        if "shape" in metadata:
            shape = tuple(json.loads(metadata["shape"]))
        else:  # files from before the shape was recorded: rows x unpacked columns
            shape = (blob.shape[0], blob.shape[1] * (8 // scheme.n_bits))
        keep = {k: metadata[k] for k in ("packing", "nnef_name", "export_as_float") if k in metadata}
        return AffineQTensor(blob, scheme, shape, getattr(torch, metadata["dequant_to_dtype"]), keep)


class _VQSerde(QTensorSerde):
    """``QTensorTractVQ`` (reference :431-556): entries ``u8_blob``, ``centroids`` (fp16) and the
    optional ``column_permutation``."""

    name = "QTensorTractVQ"

    def to_tensors(self, q: Any) -> dict[str, torch.Tensor]:
        out = {"u8_blob": q.u8_blob.cpu(), "centroids": q.qscheme.centroids.to(torch.float16).cpu().clone()}
        if q.qscheme.column_permutation is not None:
            out["column_permutation"] = q.qscheme.column_permutation.cpu()
        return out

    def to_metadata(self, q: Any) -> dict[str, str]:
        meta = getattr(q, "meta", {}) or {}
        shape = q.qscheme.original_shape or q.shape
        return {
            "proxy_selector": meta.get("proxy_selector", "l2"),
            "original_shape": ",".join(str(int(d)) for d in shape) if shape else "",
            "bits_per_index": str(q.qscheme.is_packed_indices),
            "dequant_to_dtype": meta.get("dequant_to_dtype", "float16"),
            "proxy_content_hash": _centroid_hash(q.qscheme.centroids),
            "has_column_perm": "1" if q.qscheme.column_permutation is not None else "0",
            "use_tiered": "1" if q.qscheme.use_tiered else "0",
            "zero_escape": "1" if q.qscheme.zero_escape else "0",
        }

    def from_parts(self, tensors: dict[str, torch.Tensor], metadata: dict[str, str]) -> Any:
        centroids = tensors["centroids"]
        h = metadata.get("proxy_content_hash")
        if h is not None:
            key = f"{h}@{centroids.device}"
            cached = _vq_centroid_cache.get(key)
            if cached is not None:
                centroids = cached
            else:
                _vq_centroid_cache[key] = centroids
        shape_str = metadata.get("original_shape", "")
        shape = tuple(int(d) for d in shape_str.split(",")) if shape_str else None
        perm = tensors["column_permutation"] if metadata.get("has_column_perm") == "1" else None
        scheme = VQScheme(centroids, centroids.shape[-1], int(metadata["bits_per_index"]), perm,
                          use_tiered=metadata.get("use_tiered", "0") == "1",
                          zero_escape=metadata.get("zero_escape", "0") == "1", original_shape=shape)
        keep = {k: metadata[k] for k in ("proxy_selector", "dequant_to_dtype") if k in metadata}
        return VQQTensor(tensors["u8_blob"], scheme, shape, keep)


_SERDE_REGISTRY: dict[str, QTensorSerde] = {
    "QTensorTractScaleOnly": _AffineSerde("QTensorTractScaleOnly", False),
    "QTensorScaleZp": _AffineSerde("QTensorScaleZp", True),
    "QTensorTractVQ": _VQSerde(),
}


def save_qtensor(q: Any, path) -> None:
    """One quantized weight to a safetensors file (reference :134-157)."""
    from safetensors.torch import save_file

    name = qtensor_type_name(q)
    if name is None:
        raise ValueError(f"No QTensorSerde registered for type {type(q).__name__!r}.")
    serde = _SERDE_REGISTRY[name]
    save_file({k: v.contiguous() for k, v in serde.to_tensors(q).items()}, str(path),
              metadata={**serde.to_metadata(q), _TYPE_KEY: name})


def load_qtensor(path) -> Any:
    """Inverse of :func:`save_qtensor` (reference :160-191)."""
    from safetensors import safe_open

    with safe_open(str(path), framework="pt") as f:
        metadata = f.metadata() or {}
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    name = metadata.get(_TYPE_KEY)
    if name is None or name not in _SERDE_REGISTRY:
        raise ValueError(f"{path!r}: missing or unknown {_TYPE_KEY!r} metadata ({name!r}).")
    return _SERDE_REGISTRY[name].from_parts(tensors, metadata)
