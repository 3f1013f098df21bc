"""Bit packing of group-affine codes: ``[N, K]`` uint8 values <-> ``[N, K*nbits/8]`` bytes.

Same layout as the reference's ``BitPacking`` compressor (neuropress/t2n/packing.py:99-192) and
``_pack_u8`` / ``_unpack_u8`` (neuropress/nn/np_linear.py:78-117): value ``j`` of a byte sits at
bits ``[j*nbits, (j+1)*nbits)`` — for 4 bits the even column is the low nibble.  Offline tool
(lowering time), not on the forward path.
"""

from __future__ import annotations

import torch


class BitPacking:
    """Packs ``8 // nbits`` values per byte along the last dimension."""

    def __init__(self, nbits: int) -> None:
        if nbits not in (1, 2, 4, 8):
            raise ValueError(f"nbits must be one of 1, 2, 4, 8, got {nbits}.")
        self.nbits = nbits

    @property
    def values_per_byte(self) -> int:
        return 8 // self.nbits

    def compress(self, values: torch.Tensor) -> torch.Tensor:
        vpb = self.values_per_byte
        if values.shape[-1] % vpb:
            raise ValueError(f"last dimension must be a multiple of {vpb}.")
        v = values.to(torch.int32).reshape(*values.shape[:-1], values.shape[-1] // vpb, vpb)
        shifts = torch.arange(vpb, device=values.device, dtype=torch.int32) * self.nbits
        return ((v & ((1 << self.nbits) - 1)) << shifts).sum(dim=-1).to(torch.uint8)

    def decompress(self, packed: torch.Tensor) -> torch.Tensor:
        vpb = self.values_per_byte
        shifts = torch.arange(vpb, device=packed.device, dtype=torch.int32) * self.nbits
        v = (packed.to(torch.int32).unsqueeze(-1) >> shifts) & ((1 << self.nbits) - 1)
        return v.reshape(*packed.shape[:-1], packed.shape[-1] * vpb).to(torch.uint8)
