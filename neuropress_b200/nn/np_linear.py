"""NPLinear: ``nn.Linear`` replacement with a packed n-bit group-affine weight (Q4_0 / HQQ).

    ``W[n, k] = ((q[n, k] - zp[n, k // g]) * scale[n, k // g]).to(x.dtype)``       (fp32 math)

Same module surface as the reference (neuropress/nn/np_linear.py:426-788): buffers ``u8_blob``
(``[N, K*nbits/8]``, value ``j`` of a byte at bits ``[j*nbits, (j+1)*nbits)``), ``scale`` and
``zero_point`` (flattened fp16, one per group; ``zero_point=None`` is the symmetric scheme with
the implicit zero-point ``2**(nbits-1)``), ``bias``; ``backend`` is resolved once and is always
concrete.  ``forward`` runs CUDA kernels of this package only:

    rows <= 8     fused unpack + dequant + dot GEMV
    rows <= 384   tile-dequant tensor-core GEMM (weight never written to HBM)
    otherwise     one-pass dequant + dense tensor-core GEMM

The reference runs a single warp-per-output GEMV for every row count (q4_linear.cu:137-140) and
casts bf16 activations to fp16 around it (np_linear.py:748-761); here bf16 is computed natively.
``auto`` resolves to ``cuda`` (the reference prefers the third-party ``gemlite`` Triton kernels
when installed, :201-213; they are not used here).  ``default`` / ``compile`` / ``gemlite`` are
accepted as names but not implemented: ``forward`` raises.
"""

from __future__ import annotations

import logging
from typing import Any

import torch
import torch.nn as nn

from .backends import Backend, LinearBackend

log = logging.getLogger(__name__)


def _unpack_u8(u8_blob: torch.Tensor, nbits: int) -> torch.Tensor:
    """``[N, K*nbits/8]`` packed bytes -> ``[N, K]`` uint8 values (reference :78-96)."""
    from ..t2n.packing import BitPacking

    return BitPacking(nbits).decompress(u8_blob)


def _pack_u8(values: torch.Tensor, nbits: int) -> torch.Tensor:
    """Inverse of :func:`_unpack_u8` (reference :99-117)."""
    from ..t2n.packing import BitPacking

    return BitPacking(nbits).compress(values)


def _kernel_blob(weight_q: Any) -> torch.Tensor:
    """Codes of *weight_q* in the kernels' ``[N, K*nbits/8]`` layout (reference :120-138).
    A 2-D ``u8_blob`` already has that layout; otherwise ``decompress_to_u8()`` is packed."""
    blob = weight_q.u8_blob
    if blob.dim() == 2:
        return blob
    return _pack_u8(weight_q.decompress_to_u8(), weight_q.qscheme.n_bits)


def _resolve_backend(backend: str | LinearBackend | Backend | None, nbits: int | None = None,
                     group_size: int | None = None) -> LinearBackend:
    """Alias -> concrete :class:`LinearBackend` (reference :166-213).  ``None`` / ``"torch"``
    mean DEFAULT, ``"auto"`` means CUDA, unknown strings raise ``ValueError``."""
    if backend is None or backend == "torch":
        return LinearBackend.DEFAULT
    val = backend.value if isinstance(backend, LinearBackend | Backend) else str(backend)
    if val != "auto":
        return LinearBackend(val)
    return LinearBackend.CUDA


class NPLinear(nn.Module):
    """Linear layer with a packed n-bit quantized weight.  Constructor as in the reference
    (:450-465)."""

    def __init__(
        self,
        u8_blob: torch.Tensor,
        scale: torch.Tensor,
        out_features: int,
        in_features: int,
        group_size: int,
        nbits: int,
        qtype: str,
        backend: str | LinearBackend | None,
        bias: torch.Tensor | None = None,
        zero_point: torch.Tensor | None = None,
        weight_q: Any | None = None,
        qtensor_meta: dict[str, str] | None = None,
        compute_dtype: torch.dtype = torch.float16,
    ) -> None:
        super().__init__()
        if qtype not in ("sym", "asym"):
            raise ValueError("qtype must be 'sym' or 'asym'.")
        if (qtype == "asym") != (zero_point is not None):
            raise ValueError("zero_point must be given exactly for qtype='asym'.")
        if in_features % group_size:
            raise ValueError("group_size must divide in_features.")
        self._qtensor_meta = qtensor_meta
        self.out_features = out_features
        self.in_features = in_features
        self.group_size = group_size
        self.nbits = nbits
        self.qtype = qtype
        self.backend = _resolve_backend(backend, nbits=nbits, group_size=group_size)
        self._compute_dtype = compute_dtype
        if self.backend == LinearBackend.DEFAULT:
            if weight_q is None:
                raise ValueError("weight_q is required when backend='default'.")
            object.__setattr__(self, "_weight_q", weight_q)
        self.register_buffer("u8_blob", u8_blob.contiguous())
        self.register_buffer("scale", scale.to(torch.float16).reshape(-1).contiguous())
        self.register_buffer("zero_point", None if zero_point is None
                             else zero_point.to(torch.float16).reshape(-1).contiguous())
        self.register_buffer("bias", None if bias is None else bias.contiguous())
        n_groups = out_features * (in_features // group_size)
        if self.scale.numel() != n_groups:
            raise ValueError(f"scale must have {n_groups} elements.")
        self._bias_f32: torch.Tensor | None = None
        self._bias_key = None

    @classmethod
    def from_linear(cls, linear: nn.Linear,
                    backend: str | LinearBackend | None = LinearBackend.AUTO) -> "NPLinear":
        """Build from an ``nn.Linear`` whose weight is a group-affine QTensor (reference
        :539-611).  Read by attribute: ``weight.qscheme.{n_bits, group_size, scale,
        per_group_zero_point()}``, ``weight.u8_blob``, ``weight.dequant_to_dtype``."""
        weight_q = linear._parameters.get("weight")
        q = getattr(weight_q, "qscheme", None)
        if q is None or not hasattr(q, "n_bits") or not hasattr(q, "group_size"):
            raise TypeError(f"Unsupported weight type {type(weight_q).__name__!r}: expected a "
                            "group-affine QTensor.")
        zp = q.per_group_zero_point() if hasattr(q, "per_group_zero_point") else None
        bk = _resolve_backend(backend, nbits=q.n_bits, group_size=q.group_size)
        meta = weight_q.serde_metadata() if hasattr(weight_q, "serde_metadata") else {}
        return cls(
            u8_blob=_kernel_blob(weight_q),
            scale=q.scale.detach().clone(),
            out_features=linear.out_features,
            in_features=linear.in_features,
            group_size=q.group_size,
            nbits=q.n_bits,
            qtype="sym" if zp is None else "asym",
            backend=bk,
            bias=linear.bias.detach().clone() if linear.bias is not None else None,
            zero_point=None if zp is None else zp.detach(),
            weight_q=weight_q if bk == LinearBackend.DEFAULT else None,
            qtensor_meta=meta,
            compute_dtype=getattr(weight_q, "dequant_to_dtype", torch.float16),
        )

    def to_qtensor(self):
        """Rebuild the group-affine QTensor stand-in (reference :613-645)."""
        if self._qtensor_meta is None:
            raise RuntimeError(
                "Cannot reconstruct QTensor: no serde metadata stored. "
                "Build via NPLinear.from_linear() to enable to_qtensor()."
            )
        if self.backend == LinearBackend.DEFAULT:
            return self._weight_q
        from ..qtensor import AffineQTensor, AffineScheme

        scheme = AffineScheme(self.nbits, self.group_size, self.scale, self.zero_point)
        meta = {k: v for k, v in self._qtensor_meta.items() if k not in ("type", "shape")}
        return AffineQTensor(self.u8_blob, scheme, (self.out_features, self.in_features),
                             self._compute_dtype, meta)

    def set_backend(self, backend: str | LinearBackend | None) -> "NPLinear":
        """Switch backend in place (reference :651-700)."""
        bk = _resolve_backend(backend, nbits=self.nbits, group_size=self.group_size)
        if bk == LinearBackend.DEFAULT and not hasattr(self, "_weight_q"):
            raise RuntimeError(
                "Cannot switch to LinearBackend.DEFAULT: the original QTensor was not retained."
            )
        self.backend = bk
        return self

    def _apply(self, fn, recurse: bool = True):
        self._bias_f32 = None
        return super()._apply(fn, recurse)

    def _bias32(self) -> torch.Tensor | None:
        """fp32 copy of the bias.  The reference re-casts on every call
        (vq_linear_wmma.cu:512-515); here the copy is kept and remade whenever the ``bias``
        buffer was replaced, moved or written in place (``load_state_dict`` copies in place
        and bumps the tensor's version counter)."""
        if self.bias is None:
            return None
        key = (self.bias.data_ptr(), self.bias._version, self.bias.device)
        if self._bias_f32 is None or self._bias_key != key:
            self._bias_f32 = self.bias.detach().to(torch.float32).contiguous()
            self._bias_key = key
        return self._bias_f32


    def forward(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """``gather`` (not in the reference): a ``sharding.PushGather`` when this module holds an
        out-feature shard; the all-gathered ``[..., N_full]`` is then returned."""
        if self.backend == LinearBackend.CUDA:
            return self._forward_cuda(x, gather)
        raise NotImplementedError(
            f"backend {self.backend.value!r} is not implemented by this package: only 'cuda' "
            "exists here; there is no eager, compiled or gemlite path."
        )

    def _forward_cuda(self, x: torch.Tensor, gather=None) -> torch.Tensor:
        """Banded CUDA forward (reference :732-761 runs one GEMV kernel for all row counts)."""
        from .. import kernels

        return kernels.q_linear(x.contiguous(), self.u8_blob, self.scale, self.nbits,
                                self.group_size, self.zero_point, self._bias32(), gather=gather)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, nbits={self.nbits}, "
                f"group_size={self.group_size}, qtype={self.qtype}, backend={self.backend.value}")


def _is_affine_weight(w) -> bool:
    q = getattr(w, "qscheme", None)
    return q is not None and hasattr(q, "n_bits") and hasattr(q, "group_size") and hasattr(w, "u8_blob")


def linearize_qtensor_weights(model: nn.Module,
                              backend: str | LinearBackend | None = LinearBackend.AUTO) -> nn.Module:
    """Replace every ``nn.Linear`` whose weight is a group-affine QTensor by an
    :class:`NPLinear` (reference :796-871).  Returns *model*."""
    replacements: list[tuple[str, NPLinear]] = []
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear) and _is_affine_weight(module._parameters.get("weight")):
            try:
                replacements.append((name, NPLinear.from_linear(module, backend)))
            except (TypeError, ValueError) as exc:
                log.warning("linearize_qtensor_weights: skipping %s — %s", name, exc)
    for name, layer in replacements:
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], layer)
    log.info("linearize_qtensor_weights: replaced %d layer(s)", len(replacements))
    return model
