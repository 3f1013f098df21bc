"""Output-feature sharding of one quantized linear across the GPUs of one box.

The reference has no distributed code at all; this is new.  Output rows are independent, so
rank ``r`` of ``P`` owns rows ``[r*N/P, (r+1)*N/P)``: a contiguous byte range of the index
stream (flat order ``n*G + g``), the matching slice of the residual stream / row scale / bias /
group-affine codes and scales, and a full replica of the codebook(s).  Activations are
replicated.  Each rank runs the single-GPU kernels on its shard; one collective follows, an
all-gather of the ``[M, N/P]`` outputs over NCCL (NVLink / NVSwitch).  Nothing else is
exchanged, and the single-GPU path never touches ``torch.distributed``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from .nn.np_linear import NPLinear
from .nn.np_vq_linear import NPVQLinear


def shard_rows(out_features: int, world_size: int, rank: int) -> tuple[int, int]:
    """Row range ``[begin, end)`` of *rank*; ``out_features`` must divide evenly."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}.")
    if out_features % world_size:
        raise ValueError(f"out_features={out_features} is not divisible by world_size={world_size}.")
    per = out_features // world_size
    return rank * per, (rank + 1) * per


def _stream_slice(packed: torch.Tensor, bits: int, groups: int, begin: int, end: int) -> torch.Tensor:
    """Bytes of a bit-stream that hold rows ``[begin, end)``; the cut must fall on a byte."""
    b0, b1 = begin * groups * bits, end * groups * bits
    if b0 % 8 or b1 % 8:
        raise ValueError("shard boundary does not fall on a byte of the index stream "
                         f"(rows {begin}:{end}, {groups} groups of {bits} bits).")
    return packed[b0 // 8: b1 // 8].clone()


def shard_vq_linear(layer: NPVQLinear, world_size: int, rank: int) -> NPVQLinear:
    """The rows of *layer* that *rank* owns, as a new :class:`NPVQLinear` sharing its proxies."""
    begin, end = shard_rows(layer.out_features, world_size, rank)
    groups = layer.in_features // layer.vector_len
    res = None
    if layer.residual_indices is not None:
        res = _stream_slice(layer.residual_indices, layer.residual_bits, groups, begin, end)
    return NPVQLinear(
        layer.proxy,
        _stream_slice(layer.packed_indices, layer.bits, groups, begin, end),
        layer.bits, end - begin, layer.in_features, layer.vector_len, layer.backend,
        bias=None if layer.bias is None else layer.bias[begin:end].clone(),
        column_perm=layer.column_perm,
        residual_proxy=layer.residual_proxy, residual_indices=res,
        residual_bits=layer.residual_bits if res is not None else None,
        row_scale=None if layer.row_scale is None else layer.row_scale[begin:end].clone(),
        cols_per_codebook=layer.cols_per_codebook,
    )


def shard_q_linear(layer: NPLinear, world_size: int, rank: int) -> NPLinear:
    """The rows of *layer* that *rank* owns, as a new :class:`NPLinear`."""
    begin, end = shard_rows(layer.out_features, world_size, rank)
    gpr = layer.in_features // layer.group_size
    zp = layer.zero_point
    return NPLinear(
        layer.u8_blob[begin:end].clone(), layer.scale[begin * gpr: end * gpr].clone(),
        end - begin, layer.in_features, layer.group_size, layer.nbits, layer.qtype, layer.backend,
        bias=None if layer.bias is None else layer.bias[begin:end].clone(),
        zero_point=None if zp is None else zp[begin * gpr: end * gpr].clone(),
        compute_dtype=layer._compute_dtype,
    )


def gather_outputs(y_local: torch.Tensor, group: dist.ProcessGroup | None = None) -> torch.Tensor:
    """All-gather ``[..., N/P]`` shard outputs into ``[..., N]`` (rank order along the last
    dimension).  One ``all_gather_into_tensor``; for more than one row the rank-major result
    ``[P, M, N/P]`` is re-laid out to ``[M, N]`` by one device copy."""
    world = dist.get_world_size(group)
    if world == 1:
        return y_local
    *leading, n_local = y_local.shape
    flat = y_local.reshape(-1, n_local).contiguous()
    m = flat.shape[0]
    buf = torch.empty((world * m, n_local), dtype=flat.dtype, device=flat.device)
    dist.all_gather_into_tensor(buf, flat, group=group)
    if m == 1:
        out = buf.reshape(1, world * n_local)
    else:
        out = buf.view(world, m, n_local).permute(1, 0, 2).reshape(m, world * n_local)
    return out.reshape(*leading, world * n_local)


class ShardedLinear(nn.Module):
    """A rank's shard of a quantized linear plus the all-gather of the outputs.

    ``forward(x)`` takes the replicated activations ``[..., K]`` and returns the full
    ``[..., N]`` on every rank.  With ``gather=False`` the local ``[..., N/P]`` slice is
    returned (for consumers that are sharded along their input).
    """

    def __init__(self, local: nn.Module, out_features: int, rank: int, world_size: int,
                 group: dist.ProcessGroup | None = None, gather: bool = True) -> None:
        super().__init__()
        self.local = local
        self.out_features = out_features
        self.in_features = local.in_features
        self.rank = rank
        self.world_size = world_size
        self.group = group
        self.gather = gather

    @classmethod
    def from_layer(cls, layer: nn.Module, rank: int, world_size: int,
                   group: dist.ProcessGroup | None = None, gather: bool = True) -> "ShardedLinear":
        if isinstance(layer, NPVQLinear):
            local = shard_vq_linear(layer, world_size, rank)
        elif isinstance(layer, NPLinear):
            local = shard_q_linear(layer, world_size, rank)
        else:
            raise TypeError(f"cannot shard a {type(layer).__name__}.")
        return cls(local, layer.out_features, rank, world_size, group, gather)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.local(x)
        return gather_outputs(y, self.group) if self.gather else y

    def extra_repr(self) -> str:
        return f"rank={self.rank}/{self.world_size}, out={self.out_features}, gather={self.gather}"
