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

import os

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
    if layer._entropy_scheme is not None:
        raise ValueError("entropy-coded index streams cannot be cut at a row boundary (ranks are global); "
                         "re-pack the shard's indices instead.")
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


class PushGather:
    """All-gather of ``[M, N/P]`` shard outputs by peer stores into symmetric memory.

    Replaces the NCCL all-gather + re-layout copy by one small kernel of this library
    (``npb_allgather_push``): each rank writes its slice into every rank's ``[M, N]`` buffer over
    NVLink, then flags its peers and waits (bounded) for theirs.  Two output buffers alternate,
    so the tensor returned by a call stays valid until the call after the next one; consumers
    must run on the same stream before that.  Needs one rank per GPU and peer access between
    them (``torch.distributed._symmetric_memory``); construction is collective.

    The launch arguments do not change from call to call (the epoch lives in device memory), so
    calls can be captured in a CUDA graph; the output buffer of a call is fixed at capture
    time, so capture an even number of calls per instance for the two buffers to keep
    alternating across replays.
    """

    def __init__(self, group: dist.ProcessGroup | None, max_rows: int, n_full: int,
                 dtype: torch.dtype, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        grp = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(grp)
        self.rank = dist.get_rank(grp)
        if n_full % self.world:
            raise ValueError("n_full must be divisible by the world size.")
        self.n_full, self.max_rows, self.dtype = n_full, max_rows, dtype
        self.n_local = n_full // self.world
        if (self.n_local * dtype.itemsize) % 16:
            raise ValueError("a shard row must be a multiple of 16 bytes.")
        self.bufs, self.handles = [], []
        for _ in range(2):
            b = symm_mem.empty((max_rows, n_full), dtype=dtype, device=device)
            self.bufs.append(b)
            self.handles.append(symm_mem.rendezvous(b, grp))
        self.flags = symm_mem.empty(self.world + 2 + 62, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.flags_handle = symm_mem.rendezvous(self.flags, grp)
        torch.cuda.synchronize(device)
        dist.barrier(group=grp)
        self.epoch = 0

    def begin(self, m: int, n_local: int, dtype: torch.dtype):
        """Claim the next output buffer for a kernel that gathers by itself (fused epilogue):
        returns the ``npb_gather_sink`` to pass to it and the ``[m, N]`` view it fills."""
        from . import _cabi

        if n_local != self.n_local or dtype != self.dtype or not 0 < m <= self.max_rows:
            raise RuntimeError("PushGather: shard shape / dtype / row count outside what it was built for.")
        self.epoch += 1
        which = self.epoch & 1
        sink = _cabi.GatherSinkStruct(
            peer_out=self.handles[which].buffer_ptrs_dev, peer_flags=self.flags_handle.buffer_ptrs_dev,
            ld=self.n_full, col0=self.rank * self.n_local, rank=self.rank, world=self.world, epoch=0)
        return sink, self.bufs[which][:m]

    # Row count up to which kernels with a fused all-gather epilogue are used (above it the
    # kernel writes locally and the push kernel follows).  Fused won at every row count
    # measured on two B200s (2048 rows x 7168 columns: 124 us against 101 us + 72 us).
    fused_max_rows = int(os.environ.get("NEUROPRESS_B200_FUSED_GATHER_MAX_ROWS", str(1 << 30)))

    def can_push(self, m: int, dtype: torch.dtype) -> bool:
        """Whether an ``[m, N/P]`` result of *dtype* fits the buffers this gather was built
        with.  Callers outside that envelope (more rows than ``max_rows``, another dtype) must
        use the NCCL all-gather instead."""
        return dtype == self.dtype and 0 < m <= self.max_rows

    def accepts(self, m: int, dtype: torch.dtype) -> bool:
        """Whether a kernel with a fused all-gather epilogue should be used for *m* rows."""
        return dtype == self.dtype and 0 < m <= min(self.max_rows, self.fused_max_rows)

    def __call__(self, y_local: torch.Tensor) -> torch.Tensor:
        from . import _cabi
        from .kernels import _launch

        *leading, n_local = y_local.shape
        flat = y_local.reshape(-1, n_local).contiguous()
        m = flat.shape[0]
        if n_local != self.n_local or flat.dtype != self.dtype or m > self.max_rows:
            raise RuntimeError("PushGather: shard shape / dtype / row count outside what it was built for.")
        self.epoch += 1  # host-side call count: picks the output buffer only
        which = self.epoch & 1
        lib = _cabi.load_library()
        with torch.cuda.device(flat.device):
            rc = _launch("npb_allgather_push", lib.npb_allgather_push, flat.data_ptr(), m, n_local,
                         flat.dtype.itemsize, self.handles[which].buffer_ptrs_dev,
                         self.flags_handle.buffer_ptrs_dev, self.rank, self.world, 0,
                         _cabi.stream_ptr())
        _cabi.check(rc, "npb_allgather_push")
        return self.bufs[which][:m].reshape(*leading, self.n_full)

    def status(self) -> int:
        """Synchronise and return the status word (1 = a bounded wait gave up)."""
        return int(self.flags[self.world + 1].item())


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

    def enable_push_gather(self, max_rows: int, dtype: torch.dtype, device: torch.device) -> None:
        """Collective: switch the all-gather from NCCL to peer stores (:class:`PushGather`)."""
        self.push = PushGather(self.group, max_rows, self.out_features, dtype, device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        push = getattr(self, "push", None) if self.gather else None
        if push is not None and not push.can_push(x.numel() // max(self.in_features, 1), x.dtype):
            push = None  # outside what the peer-store buffers were built for: NCCL below
        if push is not None and isinstance(self.local, NPVQLinear | NPLinear):
            # the local kernels store into every rank's buffer themselves where they can
            return self.local(x, gather=push)
        y = self.local(x)
        if not self.gather:
            return y
        if push is not None and y.dtype == push.dtype and y.numel() // y.shape[-1] <= push.max_rows:
            return push(y)
        return gather_outputs(y, self.group)

    def extra_repr(self) -> str:
        return f"rank={self.rank}/{self.world_size}, out={self.out_features}, gather={self.gather}"
