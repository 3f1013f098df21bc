"""Whole-model checkpoints in the reference's layout: save, load, and load-then-lower.

File format (neuropress/t2n/model_io.py:44-58, 214-312): one safetensors file; a regular
parameter or buffer sits under its ``state_dict`` path, a quantized weight is split by its serde
handler into ``{param_path}::{key}`` entries, and the file's metadata holds one JSON manifest
under ``__neuropress_manifest__``: ``format_version``, the ordered ``transforms`` (here the
``qtensor_assignment`` entry: per parameter path the QTensor type, its entry keys and its string
metadata) and the optional ``recipe_config``.

``save_quantized_model`` unlowers a lowered model first (NP* modules hand their weights back
as QTensors), writes, and lowers again (reference :247-263, :308-312);
``load_quantized_model`` restores regular tensors with ``load_state_dict``, rebuilds each
QTensor on the device of the parameter it replaces, and lowers the model onto the CUDA kernels
unless told not to (:463-598).  A checkpoint written by the reference loads here and, saved
again, is byte-identical; the ``mixed_precision_split`` transform of the reference (a
calibration-time structure change) is not replayed.
"""

from __future__ import annotations

import json
import logging
from pathlib import Path
from typing import Any, Literal

import torch
from pydantic import BaseModel, Field
from torch import nn

from .qtensors import _SERDE_REGISTRY, qtensor_type_name

_log = logging.getLogger(__name__)

_MANIFEST_META_KEY = "__neuropress_manifest__"
_QT_SEP = "::"
_FORMAT_VERSION = "2"


class QtensorEntry(BaseModel):
    """Serde descriptor of one quantized parameter."""

    type: str
    tensor_keys: list[str]
    metadata: dict[str, Any]


class QtensorAssignmentTransform(BaseModel):
    """Which parameters are QTensors, and how to rebuild them."""

    type: Literal["qtensor_assignment"]
    qtensor_params: dict[str, QtensorEntry]


ManifestTransform = QtensorAssignmentTransform | dict[str, Any]


class QuantizationManifest(BaseModel):
    """The transformations a checkpointed model went through (reference :127-144)."""

    transforms: list[ManifestTransform] = Field(default_factory=list)
    recipe_config_json: str | None = None

    @property
    def qtensor_params(self) -> dict[str, str]:
        for t in self.transforms:
            if isinstance(t, QtensorAssignmentTransform):
                return {k: v.type for k, v in t.qtensor_params.items()}
        return {}


def _named_qtensors(model: nn.Module):
    """``(path, value, serde type name or None)`` for every entry of ``named_parameters``."""
    for name, param in model.named_parameters():
        yield name, param, qtensor_type_name(param)


def attach_manifest(model: nn.Module, recipe_config_json: str | None = None) -> QuantizationManifest:
    """Scan *model* for quantized parameters and (re)write the ``qtensor_assignment`` entry of
    its manifest, keeping every other entry (reference :147-206)."""
    manifest = getattr(model, "__neuropress_manifest__", None) or QuantizationManifest()
    entries: dict[str, QtensorEntry] = {}
    for name, param, type_name in _named_qtensors(model):
        if type_name is not None:
            serde = _SERDE_REGISTRY[type_name]
            entries[name] = QtensorEntry(type=type_name, tensor_keys=list(serde.to_tensors(param).keys()),
                                         metadata=serde.to_metadata(param))
    if entries:
        manifest.transforms = [t for t in manifest.transforms if not isinstance(t, QtensorAssignmentTransform)]
        manifest.transforms.append(QtensorAssignmentTransform(type="qtensor_assignment", qtensor_params=entries))
    if recipe_config_json is not None:
        manifest.recipe_config_json = recipe_config_json
    model.__neuropress_manifest__ = manifest
    return manifest


def save_quantized_model(model: nn.Module, path: str | Path, recipe_config_json: str | None = None) -> None:
    """Write *model* to a safetensors checkpoint (reference :214-312)."""
    from safetensors.torch import save_file

    from ..kernel_lowering import is_lowered, unlower_model

    lowering = getattr(model, "__neuropress_kernel_lowering__", None)
    was_lowered = is_lowered(model)
    if was_lowered:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        unlower_model(model)
    try:
        manifest = attach_manifest(model, recipe_config_json=recipe_config_json)
        tensors: dict[str, torch.Tensor] = {}
        for name, param, type_name in _named_qtensors(model):
            if type_name is not None:
                for key, t in _SERDE_REGISTRY[type_name].to_tensors(param).items():
                    tensors[f"{name}{_QT_SEP}{key}"] = t
            else:
                tensors[name] = param.data
        for name, buf in model.named_buffers():
            if buf is not None and name not in tensors:
                tensors[name] = buf
        rc = json.loads(manifest.recipe_config_json) if manifest.recipe_config_json else None
        manifest_dict = {
            "format_version": _FORMAT_VERSION,
            "transforms": [t.model_dump() if isinstance(t, BaseModel) else t for t in manifest.transforms],
            "recipe_config": rc,
        }
        save_file({k: v.cpu().contiguous() for k, v in tensors.items()}, str(path),
                  metadata={_MANIFEST_META_KEY: json.dumps(manifest_dict)})
    finally:
        if was_lowered and lowering is not None:
            lowering.apply(model)


def _set_param(model: nn.Module, param_path: str, value: Any) -> None:
    """Assign into ``_parameters`` / ``_buffers`` directly: ``__setattr__`` would refuse a
    non-``Parameter`` (reference :318-341)."""
    *mods, attr = param_path.split(".")
    mod = model
    for part in mods:
        mod = getattr(mod, part)
    if attr in mod._parameters:
        mod._parameters[attr] = value
    elif attr in mod._buffers:
        mod._buffers[attr] = value
    else:
        setattr(mod, attr, value)


def load_quantized_model(model: nn.Module, path: str | Path,
                         kernel_lowering: str | None = "auto") -> QuantizationManifest:
    """Load a checkpoint written by :func:`save_quantized_model` (or by the reference) into
    *model*, a float model of the same architecture, then lower it (reference :463-598).
    ``kernel_lowering=None`` leaves the QTensors in place (inspection, re-saving)."""
    from safetensors import safe_open

    with safe_open(str(path), framework="pt") as f:
        raw_meta = f.metadata() or {}
        all_tensors = {k: f.get_tensor(k) for k in f.keys()}
    manifest_str = raw_meta.get(_MANIFEST_META_KEY)
    if manifest_str is None:
        raise ValueError(f"File {str(path)!r} is missing the {_MANIFEST_META_KEY!r} metadata key.  "
                         "Was it written by save_quantized_model()?")
    manifest_dict = json.loads(manifest_str)
    manifest = QuantizationManifest.model_validate({"transforms": manifest_dict.get("transforms", [])})
    for t in manifest.transforms:
        if isinstance(t, dict) and t.get("type") == "mixed_precision_split":
            raise NotImplementedError("checkpoints with a mixed_precision_split transform are not supported: "
                                      "that structure change belongs to calibration, outside this package.")
    entries: dict[str, QtensorEntry] = {}
    for t in manifest.transforms:
        if isinstance(t, QtensorAssignmentTransform):
            entries = t.qtensor_params
            break
    regular = {k: v for k, v in all_tensors.items() if _QT_SEP not in k and k not in entries}
    model.load_state_dict(regular, strict=False)
    saved = set(entries) | set(regular)
    tied: dict[int, list[str]] = {}
    for p_path, param in model.named_parameters(remove_duplicate=False):
        tied.setdefault(id(param), []).append(p_path)
    for p_path, entry in entries.items():
        serde = _SERDE_REGISTRY.get(entry.type)
        if serde is None:
            raise ValueError(f"No QTensorSerde registered for type {entry.type!r} (needed for parameter "
                             f"{p_path!r}).  Available: {sorted(_SERDE_REGISTRY)}")
        previous = model.get_parameter(p_path)
        device = previous.device
        parts = {k: all_tensors[f"{p_path}{_QT_SEP}{k}"] for k in entry.tensor_keys}
        if device.type != "meta":
            parts = {k: t.to(device) for k, t in parts.items()}
        q = serde.from_parts(parts, entry.metadata)
        # a tied parameter is stored once: names the file does not list share this tensor
        for other in tied[id(previous)]:
            if other == p_path or other not in saved:
                _set_param(model, other, q)
    rc = manifest_dict.get("recipe_config")
    manifest.recipe_config_json = json.dumps(rc) if rc is not None else None
    model.__neuropress_manifest__ = manifest
    if kernel_lowering is not None:
        if kernel_lowering != "auto":
            raise ValueError(f"kernel_lowering must be 'auto' or None, got {kernel_lowering!r}")
        from ..kernel_lowering import AutoKernelLowering

        _log.warning("Weights loaded — applying kernel lowering…")
        lowering = AutoKernelLowering()   # "auto" backends: chosen for this machine, not the saver's
        model.__neuropress_kernel_lowering__ = lowering
        lowering.apply(model)
    return manifest
