"""Backend enums and the toolchain probe for the quantized modules.

Same names and values as the reference (neuropress/nn/backends.py:102-159).  The reference
JIT-builds its kernels and therefore probes for ninja + nvcc (``is_cuda_jit_available``,
:26-99); here the kernels are built ahead of time into one shared library, so the probe reports
whether that library is present (``NEUROPRESS_FORCE_CUDA_JIT=1`` still forces ``True``).
"""

from __future__ import annotations

import enum
import logging
import os

_log = logging.getLogger(__name__)

_cuda_jit_ok: bool | None = None


def is_cuda_jit_available() -> bool:
    """``True`` when the CUDA kernels can run: the in-tree shared library exists.

    Cached after the first call, like the reference's probe.  The environment variable
    ``NEUROPRESS_FORCE_CUDA_JIT`` (``1`` / ``true`` / ``yes``) skips the check.
    """
    global _cuda_jit_ok
    if _cuda_jit_ok is not None:
        return _cuda_jit_ok
    if os.environ.get("NEUROPRESS_FORCE_CUDA_JIT", "").strip() in ("1", "true", "yes"):
        _cuda_jit_ok = True
        return True
    from .. import _cabi

    _cuda_jit_ok = _cabi.library_available()
    if not _cuda_jit_ok:
        _log.warning(
            "libneuropress_b200.so is not built — CUDA backends will raise at forward time; "
            "run `python -m neuropress_b200.build`."
        )
    return _cuda_jit_ok


class LinearBackend(enum.StrEnum):
    """Valid backends for scalar-quantized ``nn.Linear`` (:class:`NPLinear`)."""

    AUTO = "auto"
    DEFAULT = "default"
    COMPILE = "compile"
    CUDA = "cuda"
    GEMLITE = "gemlite"


class VQBackend(enum.StrEnum):
    """Valid backends for vector-quantized ``nn.Linear`` (:class:`NPVQLinear`)."""

    AUTO = "auto"
    DEFAULT = "default"
    COMPILE = "compile"
    CUDA = "cuda"
    CUDA_WMMA = "cuda_wmma"
    CUDA_LUT = "cuda_lut"
    CUDA_TIERED = "cuda_tiered"
    CUDA_NTIER = "cuda_ntier"
    CUDA_ZERO_ESCAPE = "cuda_zero_escape"


class EmbeddingBackend(enum.StrEnum):
    """Valid backends for quantized ``nn.Embedding`` (kept for configuration files)."""

    AUTO = "auto"
    DEFAULT = "default"
    COMPILE = "compile"
    CUDA = "cuda"


class NormBackend(enum.StrEnum):
    """Valid backends for RMSNorm modules (kept for configuration files)."""

    AUTO = "auto"
    DEFAULT = "default"
    CUDA = "cuda"


class Backend(enum.StrEnum):
    """Superset backend enum (backward compatibility with the reference)."""

    DEFAULT = "default"
    COMPILE = "compile"
    CUDA = "cuda"
    CUDA_WMMA = "cuda_wmma"
    CUDA_LUT = "cuda_lut"
    CUDA_TIERED = "cuda_tiered"
    CUDA_NTIER = "cuda_ntier"
    CUDA_ZERO_ESCAPE = "cuda_zero_escape"
    GEMLITE = "gemlite"
    AUTO = "auto"
