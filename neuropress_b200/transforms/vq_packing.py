"""Fixed-width index packing: the wire format of ``NPVQLinear.packed_indices``.

Same format and API as ``IndexPacking`` of the reference
(neuropress/transforms/vq_packing.py:97-295): index ``i`` occupies bits
``[i*bits, (i+1)*bits)`` of an LSB-first bit stream stored as ``uint8``; 8-bit is one byte per
index, 4-bit puts the even index in the low nibble, 16-bit equals a little-endian ``uint16``
view.  The implementation differs: instead of one pass per bit, every index is shifted to its
in-byte offset once and its (at most three) bytes are scattered / gathered in one step.
Offline tool (lowering time), not on the forward path.
"""

from __future__ import annotations

import math

import torch


class IndexPacking:
    """Static pack / unpack utilities; no instance needed."""

    _MIN_BITS: int = 4
    _MAX_BITS: int = 20
    _MAX_CENTROIDS: int = 1 << 20

    @staticmethod
    def bits_for(num_centroids: int) -> int:
        """``max(4, ceil(log2(num_centroids)))``; ``ValueError`` outside ``[2, 2**20]``
        (reference: vq_packing.py:111-133)."""
        if num_centroids < 2:
            raise ValueError(f"num_centroids must be >= 2, got {num_centroids}.")
        if num_centroids > IndexPacking._MAX_CENTROIDS:
            raise ValueError(
                f"num_centroids={num_centroids} exceeds the maximum supported value of "
                f"{IndexPacking._MAX_CENTROIDS} (20-bit indices)."
            )
        return max(IndexPacking._MIN_BITS, math.ceil(math.log2(num_centroids)))

    @staticmethod
    def _check_bits(bits: int) -> None:
        if not (IndexPacking._MIN_BITS <= bits <= IndexPacking._MAX_BITS):
            raise ValueError(
                f"bits must be in [{IndexPacking._MIN_BITS}, {IndexPacking._MAX_BITS}], got {bits}."
            )

    @staticmethod
    def packed_nbytes(n_indices: int, bits: int) -> int:
        """Byte length of a stream of *n_indices* indices."""
        return (n_indices * bits + 7) // 8

    @staticmethod
    def pack(indices: torch.Tensor, bits: int) -> torch.Tensor:
        """Pack integer indices (any shape, flattened) into a 1-D ``uint8`` stream of
        ``ceil(n * bits / 8)`` bytes.  4-bit needs an even count (reference: :135-176)."""
        IndexPacking._check_bits(bits)
        flat = indices.flatten().to(torch.int64)
        n = flat.numel()
        if bits == 8:
            return flat.to(torch.uint8)
        if bits == 4 and n % 2 != 0:
            raise ValueError(
                f"IndexPacking(bits=4): index count ({n}) must be even for 4-bit packing."
            )
        if bits == 16:
            lo = (flat & 0xFF).to(torch.uint8)
            hi = ((flat >> 8) & 0xFF).to(torch.uint8)
            return torch.stack([lo, hi], dim=1).flatten()
        n_bytes = IndexPacking.packed_nbytes(n, bits)
        pos = torch.arange(n, dtype=torch.int64, device=flat.device) * bits
        byte0 = pos >> 3
        shifted = (flat & ((1 << bits) - 1)) << (pos & 7)  # at most 7 + 20 = 27 bits
        out = torch.zeros(n_bytes + 4, dtype=torch.int64, device=flat.device)
        for k in range((bits + 7 + 7) // 8):
            out.index_add_(0, byte0 + k, (shifted >> (8 * k)) & 0xFF)
        return out[:n_bytes].to(torch.uint8)

    @staticmethod
    def unpack(packed: torch.Tensor, bits: int, n_indices: int) -> torch.Tensor:
        """Inverse of :meth:`pack`: 1-D ``int64`` tensor of *n_indices* indices
        (reference: :178-208, :255-295)."""
        IndexPacking._check_bits(bits)
        if bits == 8:
            return packed.to(torch.int64)[:n_indices]
        p = torch.cat([packed.flatten().to(torch.int64),
                       torch.zeros(4, dtype=torch.int64, device=packed.device)])
        pos = torch.arange(n_indices, dtype=torch.int64, device=packed.device) * bits
        byte0 = pos >> 3
        window = p[byte0]
        for k in range(1, (bits + 7 + 7) // 8):
            window = window | (p[byte0 + k] << (8 * k))
        return (window >> (pos & 7)) & ((1 << bits) - 1)


# The entropy-coded packers live in a module of their own; the reference exports them from this
# one (``neuropress.transforms.vq_packing``), so they are importable from here too.
from .entropy_packing import (  # noqa: E402
    NTieredIndexPacking,
    TieredIndexPacking,
    ZeroEscapePacking,
    describe_entropy_buffer,
)
