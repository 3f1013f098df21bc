"""Entropy-coded index streams: the three prefix codes the reference offers for frequency-sorted
codebooks, in the reference's wire formats (``neuropress/transforms/vq_packing.py``):

* ``TieredIndexPacking`` (:298-610) -- one prefix bit per index (0 = hot, 1 = cold), then a
  ``hot_bits`` stream and a ``cold_bits`` stream; 16-byte header ``n, n_hot, cold_bits, hot_bits``
  (uint32 LE; the 12-byte legacy header without ``hot_bits`` reads as ``hot_bits = 4``).
* ``NTieredIndexPacking`` (:612-1034) -- 2..4 tiers by cascaded one-bit prefixes: prefix stream k
  has one bit per index that is not in tiers ``< k`` (0 = tier k, 1 = rest); tier k stores
  ``index - 2**tier_bits[k-1]`` in ``tier_bits[k]`` bits; header ``magic, n, D, (count_k, bits_k)*D``.
* ``ZeroEscapePacking`` (:1037-1384) -- a flat two-bit prefix per index: 0 = centroid 0 (no
  payload), 1 = centroids 1..16 (4 bits, stored minus 1), 2 = centroids 17..256 (8 bits, stored
  minus 17), 3 = the rest (``cold_bits``, stored minus 257); 24-byte header.

All sub-streams use ``IndexPacking``'s LSB-first bit order.  The byte streams produced here are
identical to the reference's (pinned by golden vectors); the implementation is vectorised torch
(the reference walks rows in Python loops for the row offsets) and runs on whatever device the
indices live on.  ``compute_row_offsets`` returns, like the reference, int32 CPU tensors of
length ``n_rows + 1`` with the cumulative number of tier-k indices in the rows before row i --
what a kernel needs to start decoding at any row.
"""

from __future__ import annotations

import math

import torch

from .vq_packing import IndexPacking

__all__ = ["TieredIndexPacking", "NTieredIndexPacking", "ZeroEscapePacking", "describe_entropy_buffer"]


def _bits_pack(values: torch.Tensor, bits: int) -> torch.Tensor:
    """LSB-first bit stream of ``bits``-wide values (1 <= bits <= 20): value i occupies stream bits
    ``[i * bits, (i + 1) * bits)`` -- the layout of the reference's ``_pack_bitstream`` (:209-253),
    which the prefix streams use with one or two bits per index."""
    flat = values.flatten().to(torch.int64)
    n = flat.numel()
    n_bytes = (n * bits + 7) // 8
    pos = torch.arange(n, dtype=torch.int64, device=flat.device) * bits
    shifted = (flat & ((1 << bits) - 1)) << (pos & 7)
    out = torch.zeros(n_bytes + 4, dtype=torch.int64, device=flat.device)
    for k in range((bits + 7 + 7) // 8):
        out.index_add_(0, (pos >> 3) + k, (shifted >> (8 * k)) & 0xFF)
    return out[:n_bytes].to(torch.uint8)


def _bits_unpack(buf: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    """Inverse of ``_bits_pack`` for the first ``count`` values of ``buf`` (int64)."""
    p = torch.cat([buf.flatten().to(torch.int64), torch.zeros(4, dtype=torch.int64, device=buf.device)])
    pos = torch.arange(count, dtype=torch.int64, device=buf.device) * bits
    window = p[pos >> 3]
    for k in range(1, (bits + 7 + 7) // 8):
        window = window | (p[(pos >> 3) + k] << (8 * k))
    return (window >> (pos & 7)) & ((1 << bits) - 1)


def _pack_stream(values: torch.Tensor, bits: int) -> torch.Tensor:
    """``IndexPacking.pack`` of a possibly empty value list; four-bit streams are padded to an
    even count with a zero, as the reference does before packing nibbles."""
    if values.numel() == 0:
        return torch.zeros(0, dtype=torch.uint8, device=values.device)
    if bits == 4 and values.numel() % 2:
        values = torch.cat([values, values.new_zeros(1)])
    return IndexPacking.pack(values, bits)


def _unpack_stream(buf: torch.Tensor, bits: int, count: int) -> torch.Tensor:
    if count == 0:
        return torch.zeros(0, dtype=torch.int64, device=buf.device)
    return IndexPacking.unpack(buf, bits, count)


def _header_words(packed: torch.Tensor, n_bytes: int) -> list[int]:
    return [int(v) for v in packed[:n_bytes].cpu().contiguous().view(torch.int32).tolist()]


def _check_bits(name: str, bits: int) -> None:
    lo, hi = IndexPacking._MIN_BITS, IndexPacking._MAX_BITS
    if not lo <= bits <= hi:
        raise ValueError(f"{name} must be in [{lo}, {hi}], got {bits}.")


def _row_cumsum(tier_id: torch.Tensor, n_tiers: int, n_rows: int, n_groups: int) -> list[torch.Tensor]:
    """Per tier: cumulative count of its indices in the rows before row i, int32 CPU ``[n_rows+1]``."""
    rows = tier_id.view(n_rows, n_groups)
    out = []
    for k in range(n_tiers):
        per_row = (rows == k).sum(dim=1, dtype=torch.int64)
        off = torch.zeros(n_rows + 1, dtype=torch.int64, device=per_row.device)
        off[1:] = torch.cumsum(per_row, 0)
        out.append(off.to(torch.int32).cpu())
    return out


class TieredIndexPacking:
    """Two tiers behind a one-bit prefix (reference :298-610)."""

    DEFAULT_HOT_BITS: int = 4
    HEADER_BYTES: int = 16
    _LEGACY_HEADER_BYTES: int = 12

    @staticmethod
    def hot_threshold(hot_bits: int) -> int:
        return 1 << hot_bits

    @staticmethod
    def pack(indices: torch.Tensor, cold_bits: int, hot_bits: int = 4) -> torch.Tensor:
        _check_bits("cold_bits", cold_bits)
        if not 4 <= hot_bits <= 16:
            raise ValueError(f"hot_bits must be in [4, 16], got {hot_bits}.")
        flat = indices.flatten().to(torch.int64)
        cold = flat >= (1 << hot_bits)
        header = torch.tensor([flat.numel(), int((~cold).sum()), cold_bits, hot_bits], dtype=torch.int32,
                              device=flat.device).view(torch.uint8)
        return torch.cat([header, _bits_pack(cold.to(torch.int64), 1),
                          _pack_stream(flat[~cold], hot_bits), _pack_stream(flat[cold], cold_bits)])

    @staticmethod
    def _parse_header(packed: torch.Tensor) -> tuple[int, int, int, int, int]:
        legacy, full = TieredIndexPacking._LEGACY_HEADER_BYTES, TieredIndexPacking.HEADER_BYTES
        if packed.numel() < legacy:
            raise ValueError(f"TieredIndexPacking: buffer too short ({packed.numel()} bytes, need at least {legacy}).")
        n, n_hot, cold_bits = _header_words(packed, legacy)
        if packed.numel() >= full:
            hot_bits = _header_words(packed[legacy:], 4)[0]
            if 4 <= hot_bits <= 16:       # a plausible fourth field: the current header
                return n, n_hot, cold_bits, hot_bits, full
        return n, n_hot, cold_bits, 4, legacy

    @staticmethod
    def _layout(packed: torch.Tensor) -> dict:
        n, n_hot, cold_bits, hot_bits, h = TieredIndexPacking._parse_header(packed)
        prefix = h
        hot = prefix + (n + 7) // 8
        cold = hot + math.ceil(n_hot * hot_bits / 8)
        return {"n": n, "counts": [n_hot, n - n_hot], "bits": [hot_bits, cold_bits], "lo": [0, 0],
                "prefix_off": [prefix], "tier_off": [hot, cold],
                "end": cold + math.ceil((n - n_hot) * cold_bits / 8), "kind": 1}

    @staticmethod
    def unpack(packed: torch.Tensor) -> torch.Tensor:
        lay = TieredIndexPacking._layout(packed)
        n, (n_hot, n_cold) = lay["n"], lay["counts"]
        cold = _bits_unpack(packed[lay["prefix_off"][0]:lay["tier_off"][0]], 1, n) == 1
        out = torch.zeros(n, dtype=torch.int64, device=packed.device)
        out[~cold] = _unpack_stream(packed[lay["tier_off"][0]:lay["tier_off"][1]], lay["bits"][0], n_hot)
        out[cold] = _unpack_stream(packed[lay["tier_off"][1]:lay["end"]], lay["bits"][1], n_cold)
        return out

    @staticmethod
    def compute_row_offsets(packed: torch.Tensor, n_rows: int, n_groups: int) -> tuple[torch.Tensor, torch.Tensor]:
        lay = TieredIndexPacking._layout(packed)
        if lay["n"] != n_rows * n_groups:
            raise ValueError(f"compute_row_offsets: n_rows*n_groups={n_rows * n_groups} != n_indices={lay['n']} in header.")
        tier = _bits_unpack(packed[lay["prefix_off"][0]:lay["tier_off"][0]], 1, lay["n"])
        hot, cold = _row_cumsum(tier, 2, n_rows, n_groups)
        return hot, cold

    @staticmethod
    def effective_bits(n_hot: int, n_total: int, cold_bits: int, hot_bits: int = 4) -> float:
        if n_total == 0:
            return float(cold_bits)
        p_hot = n_hot / n_total
        return 1.0 + hot_bits * p_hot + cold_bits * (1.0 - p_hot)


class NTieredIndexPacking:
    """Two to four tiers behind cascaded one-bit prefixes (reference :612-1034)."""

    MAGIC: int = 0x4E565154
    MIN_TIERS: int = 2
    MAX_TIERS: int = 4

    @staticmethod
    def tier_thresholds(tier_bits: list[int]) -> list[int]:
        return [1 << b for b in tier_bits]

    @staticmethod
    def _validate_tier_bits(tier_bits: list[int]) -> None:
        d = len(tier_bits)
        if not NTieredIndexPacking.MIN_TIERS <= d <= NTieredIndexPacking.MAX_TIERS:
            raise ValueError(f"tier_bits length must be in [{NTieredIndexPacking.MIN_TIERS}, "
                             f"{NTieredIndexPacking.MAX_TIERS}], got {d}.")
        for i, b in enumerate(tier_bits):
            _check_bits(f"tier_bits[{i}]", b)
        for a, b in zip(tier_bits, tier_bits[1:]):
            if b <= a:
                raise ValueError(f"tier_bits must be strictly increasing, got {tier_bits}.")

    @staticmethod
    def _tier_of(flat: torch.Tensor, tier_bits: list[int]) -> torch.Tensor:
        """Tier of every index: the first k with ``index < 2**tier_bits[k]``, else the last tier."""
        bounds = torch.tensor([1 << b for b in tier_bits[:-1]], dtype=torch.int64, device=flat.device)
        return torch.bucketize(flat, bounds, right=True)

    @staticmethod
    def pack(indices: torch.Tensor, tier_bits: list[int]) -> torch.Tensor:
        NTieredIndexPacking._validate_tier_bits(tier_bits)
        flat = indices.flatten().to(torch.int64)
        d = len(tier_bits)
        tier = NTieredIndexPacking._tier_of(flat, tier_bits)
        counts = [int((tier == k).sum()) for k in range(d)]
        prefixes, streams = [], []
        for k in range(d):
            lo = 0 if k == 0 else 1 << tier_bits[k - 1]
            if k < d - 1:   # one bit for every index not yet placed: 0 = this tier, 1 = later
                prefixes.append(_bits_pack((tier[tier >= k] > k).to(torch.int64), 1))
            streams.append(_pack_stream(flat[tier == k] - lo, tier_bits[k]))
        words = [NTieredIndexPacking.MAGIC, flat.numel(), d]
        for k in range(d):
            words += [counts[k], tier_bits[k]]
        header = torch.tensor(words, dtype=torch.int32, device=flat.device).view(torch.uint8)
        return torch.cat([header, *prefixes, *streams])

    @staticmethod
    def _parse_header(packed: torch.Tensor) -> tuple[int, int, list[int], list[int], int]:
        if packed.numel() < 12:
            raise ValueError(f"NTieredIndexPacking: buffer too short ({packed.numel()} bytes, need at least 12).")
        magic, n, d = _header_words(packed, 12)
        if magic != NTieredIndexPacking.MAGIC:
            raise ValueError(f"NTieredIndexPacking: bad magic 0x{magic & 0xFFFFFFFF:08X}, "
                             f"expected 0x{NTieredIndexPacking.MAGIC:08X}.")
        h = 12 + 8 * d
        if packed.numel() < h:
            raise ValueError(f"NTieredIndexPacking: buffer too short for {d} tiers ({packed.numel()} < {h}).")
        words = _header_words(packed[12:], 8 * d)
        return n, d, words[0::2], words[1::2], h

    @staticmethod
    def _layout(packed: torch.Tensor) -> dict:
        n, d, counts, bits, h = NTieredIndexPacking._parse_header(packed)
        off, remaining, prefix_off, tier_off = h, n, [], []
        for k in range(d - 1):
            prefix_off.append(off)
            off += (remaining + 7) // 8
            remaining -= counts[k]
        for k in range(d):
            tier_off.append(off)
            off += math.ceil(counts[k] * bits[k] / 8)
        return {"n": n, "counts": counts, "bits": bits, "lo": [0] + [1 << b for b in bits[:-1]],
                "prefix_off": prefix_off, "tier_off": tier_off, "end": off, "kind": 1}

    @staticmethod
    def _tiers_from_prefixes(packed: torch.Tensor, lay: dict) -> torch.Tensor:
        n, d = lay["n"], len(lay["bits"])
        tier = torch.full((n,), d - 1, dtype=torch.int64, device=packed.device)
        alive = torch.arange(n, dtype=torch.int64, device=packed.device)   # positions not yet placed
        for k in range(d - 1):
            bits = _bits_unpack(packed[lay["prefix_off"][k]:], 1, alive.numel())
            tier[alive[bits == 0]] = k
            alive = alive[bits == 1]
        return tier

    @staticmethod
    def unpack(packed: torch.Tensor) -> torch.Tensor:
        lay = NTieredIndexPacking._layout(packed)
        tier = NTieredIndexPacking._tiers_from_prefixes(packed, lay)
        out = torch.zeros(lay["n"], dtype=torch.int64, device=packed.device)
        ends = lay["tier_off"][1:] + [lay["end"]]
        for k, count in enumerate(lay["counts"]):
            if count:
                out[tier == k] = _unpack_stream(packed[lay["tier_off"][k]:ends[k]], lay["bits"][k], count) + lay["lo"][k]
        return out

    @staticmethod
    def compute_row_offsets(packed: torch.Tensor, n_rows: int, n_groups: int) -> list[torch.Tensor]:
        lay = NTieredIndexPacking._layout(packed)
        if lay["n"] != n_rows * n_groups:
            raise ValueError(f"compute_row_offsets: n_rows*n_groups={n_rows * n_groups} != n_indices={lay['n']}.")
        tier = NTieredIndexPacking._tiers_from_prefixes(packed, lay)
        return _row_cumsum(tier, len(lay["bits"]), n_rows, n_groups)

    @staticmethod
    def effective_bits(tier_counts: list[int], tier_bits: list[int]) -> float:
        total = sum(tier_counts)
        if total == 0:
            return float(tier_bits[-1])
        prefix, remaining = 0.0, total
        for k in range(len(tier_bits) - 1):
            prefix += remaining / total
            remaining -= tier_counts[k]
        return prefix + sum(b * c / total for b, c in zip(tier_bits, tier_counts))

    @staticmethod
    def is_ntier_buffer(packed: torch.Tensor) -> bool:
        return packed.numel() >= 4 and (_header_words(packed, 4)[0] & 0xFFFFFFFF) == NTieredIndexPacking.MAGIC


class ZeroEscapePacking:
    """Flat two-bit prefix with a payload-free code for centroid 0 (reference :1037-1384)."""

    MAGIC: int = 0x5A455343
    HEADER_BYTES: int = 24
    TIER_0_MAX: int = 1
    TIER_1_MAX: int = 17
    TIER_2_MAX: int = 257
    _LO = (0, 1, 17, 257)

    @staticmethod
    def _tier_of(flat: torch.Tensor) -> torch.Tensor:
        bounds = torch.tensor([1, 17, 257], dtype=torch.int64, device=flat.device)
        return torch.bucketize(flat, bounds, right=True)

    @staticmethod
    def pack(indices: torch.Tensor, cold_bits: int) -> torch.Tensor:
        _check_bits("cold_bits", cold_bits)
        flat = indices.flatten().to(torch.int64)
        tier = ZeroEscapePacking._tier_of(flat)
        counts = [int((tier == k).sum()) for k in range(4)]
        header = torch.tensor([ZeroEscapePacking.MAGIC, flat.numel(), cold_bits, counts[0], counts[1], counts[2]],
                              dtype=torch.int32, device=flat.device).view(torch.uint8)
        streams = [_pack_stream(flat[tier == k] - ZeroEscapePacking._LO[k], b)
                   for k, b in ((1, 4), (2, 8), (3, cold_bits))]
        return torch.cat([header, _bits_pack(tier, 2), *streams])

    @staticmethod
    def _parse_header(packed: torch.Tensor) -> tuple[int, int, int, int, int, int]:
        h = ZeroEscapePacking.HEADER_BYTES
        if packed.numel() < h:
            raise ValueError(f"ZeroEscapePacking: buffer too short ({packed.numel()} bytes, need at least {h}).")
        magic, n, cold_bits, n_zero, n_hot, n_warm = _header_words(packed, h)
        if magic != ZeroEscapePacking.MAGIC:
            raise ValueError(f"ZeroEscapePacking: bad magic 0x{magic & 0xFFFFFFFF:08X}, "
                             f"expected 0x{ZeroEscapePacking.MAGIC:08X}.")
        return n, cold_bits, n_zero, n_hot, n_warm, h

    @staticmethod
    def _layout(packed: torch.Tensor) -> dict:
        n, cold_bits, n_zero, n_hot, n_warm, h = ZeroEscapePacking._parse_header(packed)
        n_cold = n - n_zero - n_hot - n_warm
        hot = h + (2 * n + 7) // 8
        warm = hot + math.ceil(n_hot * 4 / 8)
        cold = warm + n_warm
        return {"n": n, "counts": [n_zero, n_hot, n_warm, n_cold], "bits": [0, 4, 8, cold_bits],
                "lo": list(ZeroEscapePacking._LO), "prefix_off": [h], "tier_off": [hot, hot, warm, cold],
                "end": cold + math.ceil(n_cold * cold_bits / 8), "kind": 2}

    @staticmethod
    def unpack(packed: torch.Tensor) -> torch.Tensor:
        lay = ZeroEscapePacking._layout(packed)
        tier = _bits_unpack(packed[lay["prefix_off"][0]:lay["tier_off"][1]], 2, lay["n"])
        out = torch.zeros(lay["n"], dtype=torch.int64, device=packed.device)
        ends = lay["tier_off"][1:] + [lay["end"]]
        for k in (1, 2, 3):
            if lay["counts"][k]:
                out[tier == k] = _unpack_stream(packed[lay["tier_off"][k]:ends[k]], lay["bits"][k],
                                                lay["counts"][k]) + lay["lo"][k]
        return out

    @staticmethod
    def compute_row_offsets(packed: torch.Tensor, n_rows: int, n_groups: int) -> list[torch.Tensor]:
        lay = ZeroEscapePacking._layout(packed)
        if lay["n"] != n_rows * n_groups:
            raise ValueError(f"compute_row_offsets: n_rows*n_groups={n_rows * n_groups} != n_indices={lay['n']}.")
        tier = _bits_unpack(packed[lay["prefix_off"][0]:lay["tier_off"][1]], 2, lay["n"])
        return _row_cumsum(tier, 4, n_rows, n_groups)

    @staticmethod
    def effective_bits(n_zero: int, n_hot: int, n_warm: int, n_cold: int, cold_bits: int) -> float:
        total = n_zero + n_hot + n_warm + n_cold
        if total == 0:
            return float(cold_bits)
        return (2 * n_zero + 6 * n_hot + 10 * n_warm + (2 + cold_bits) * n_cold) / total

    @staticmethod
    def is_zero_escape_buffer(packed: torch.Tensor) -> bool:
        return packed.numel() >= 4 and (_header_words(packed, 4)[0] & 0xFFFFFFFF) == ZeroEscapePacking.MAGIC


def describe_entropy_buffer(packed: torch.Tensor, scheme: str) -> dict:
    """Where the sub-streams of an entropy-coded buffer sit: ``n`` indices, per-tier ``counts`` /
    ``bits`` / ``lo`` (value added to a payload), byte offsets of the prefix streams and of each
    tier's payload stream, ``kind`` 1 (cascaded one-bit prefixes) or 2 (flat two-bit prefix).
    ``scheme`` is ``"tiered"``, ``"ntier"`` or ``"zero_escape"``.  This is what the expansion
    kernel takes beside the buffer and the row offsets."""
    if scheme == "tiered":
        return TieredIndexPacking._layout(packed)
    if scheme == "ntier":
        return NTieredIndexPacking._layout(packed)
    if scheme == "zero_escape":
        return ZeroEscapePacking._layout(packed)
    raise ValueError(f"unknown entropy-coded scheme {scheme!r}")
