"""Linears that share their input, run as one launch; the RMSNorm in front of them folded in.

A decoder layer feeds one tensor to its q / k / v projections and one to gate / up.  The
reference launches a kernel per linear and one per norm (np_vq_linear.py:1250-1267,
np_rms_norm.py:86-99); at one to sixteen rows every such launch costs more than the work it
does.  :func:`group_shared_input_linears` rewires those modules, without touching the model's
own ``forward`` code: each member is replaced by a :class:`GroupedLinear` whose first member
("leader") computes all outputs with ``npb_vq_gemv_grouped`` and hands the others their slices,
and the norm in front of the group is replaced by a :class:`DeferredNorm` that passes its input
through and lets the group's kernel normalise the activations while staging them.  From 17 rows
to the end of the tile-decode band the norm runs as its own kernel and the members share one
launch of ``npb_vq_gemm_fused_grouped``.  Larger batches, or weights the grouped kernels do not
take, fall back to the norm kernel and the members' own forwards -- same results, one launch each.

The group keys on the input tensor's identity between the leader's call and the followers'
calls of the SAME forward; use it only for members that really receive the same tensor.
"""

from __future__ import annotations

import torch
from torch import nn

from .np_rms_norm import NPRMSNorm
from .np_vq_linear import NPVQLinear, _FUSED_BACKENDS, _SMALL_BATCH_MAX_TOKENS, _TRITON_MAX_TOKENS

__all__ = ["LinearGroup", "GroupedLinear", "DeferredNorm", "group_shared_input_linears"]


class LinearGroup:
    """Shared state of one group (a plain object: it owns no parameters)."""

    def __init__(self, members: list[NPVQLinear], norm: NPRMSNorm | None = None) -> None:
        first = members[0]
        for m in members:
            if not isinstance(m, NPVQLinear) or m._entropy_scheme is not None \
                    or m.in_features != first.in_features or m.bits != first.bits \
                    or m.vector_len != first.vector_len or m.cols_per_codebook != first.cols_per_codebook \
                    or m.proxy.num_centroids != first.proxy.num_centroids:
                raise ValueError("grouped linears must be NPVQLinear modules of one input width, index width "
                                 "and codebook layout.")
        self.members = members
        self.norm = norm
        self._key = None
        self._outs: list[torch.Tensor | None] = []
        self._norm_w: torch.Tensor | None = None

    def _fusable(self, x2: torch.Tensor) -> bool:
        m0 = self.members[0]
        return (x2.shape[0] <= _SMALL_BATCH_MAX_TOKENS and m0.backend in _FUSED_BACKENDS
                and all(m.column_perm is None and m.residual_indices is None and m.row_scale is None
                        for m in self.members)
                and m0._small_batch_ok(x2, max(x2.shape[0], 3)))

    def _tile_fusable(self, x2: torch.Tensor) -> bool:
        """The members would all take the copy form of the tile-decode GEMM for these rows (the
        conditions of ``NPVQLinear._forward_triton`` and of ``kernels.vq_gemm_fused``)."""
        from .. import kernels

        m0 = self.members[0]
        rows = x2.shape[0]
        return (kernels.VQ_TILE_DECODE_GEMM and kernels.VQ_COPY_FORM and len(self.members) > 1
                and _SMALL_BATCH_MAX_TOKENS < rows <= _TRITON_MAX_TOKENS and m0.backend in _FUSED_BACKENDS
                and x2.dtype in (torch.bfloat16, torch.float16) and m0.vector_len == 8
                and m0.bits in (8, 12, 16) and m0.in_features % 64 == 0
                and not (m0.cols_per_codebook and m0.cols_per_codebook % 64)
                and all(m.column_perm is None and m.residual_indices is None and m.row_scale is None
                        and m.packed_indices.data_ptr() % 16 == 0 for m in self.members))

    def _split(self, y: torch.Tensor, leading) -> list[torch.Tensor]:
        outs, c = [], 0
        for m in self.members:
            outs.append(y[:, c:c + m.out_features].reshape(*leading, m.out_features))
            c += m.out_features
        return outs

    def _norm_weight(self, dtype: torch.dtype) -> torch.Tensor:
        w = self.norm.weight
        if self._norm_w is None or self._norm_w.dtype != dtype or self._norm_w.device != w.device \
                or self._norm_w._base_version != w._version:
            self._norm_w = w.to(dtype).contiguous()
            self._norm_w._base_version = w._version
        return self._norm_w

    def compute(self, x: torch.Tensor) -> list[torch.Tensor]:
        from .. import kernels

        m0 = self.members[0]
        *leading, k = x.shape
        x2 = x.reshape(-1, k).contiguous()
        if self._fusable(x2):
            weights = [(m.packed_indices, m.proxy.centroids, m.out_features, m._bias32()) for m in self.members]
            y = kernels.vq_gemv_grouped(x2, weights, m0.bits, m0.cols_per_codebook,
                                        None if self.norm is None else self._norm_weight(x2.dtype),
                                        0.0 if self.norm is None else self.norm.eps)
            if y is not None:
                return self._split(y, leading)
        xn = x if self.norm is None else self.norm(x)       # one norm launch, shared by the members
        xn2 = xn.reshape(-1, k)
        if self._tile_fusable(xn2):
            weights = [(m.packed_indices, m.proxy.centroids, m.out_features, m._bias32()) for m in self.members]
            y = kernels.vq_gemm_fused_grouped(xn2.contiguous(), weights, m0.bits, m0.cols_per_codebook)
            if y is not None:
                return self._split(y, leading)
        return [m(xn) for m in self.members]

    def output(self, index: int, x: torch.Tensor) -> torch.Tensor:
        key = (x.data_ptr(), tuple(x.shape), x.dtype)
        if index == 0 or self._key != key or self._outs[index] is None:
            if index != 0:
                # a follower called on its own (or with another tensor): compute just this member
                xn = x if self.norm is None else self.norm(x)
                return self.members[index](xn)
            self._outs = self.compute(x)
            self._key = key
        out = self._outs[index]
        self._outs[index] = None      # each slice is handed out once per leader call
        if all(o is None for o in self._outs):
            self._key = None
        return out


class GroupedLinear(nn.Module):
    """Stands where member ``index`` of a :class:`LinearGroup` stood; owns that member."""

    def __init__(self, inner: NPVQLinear, group: LinearGroup, index: int) -> None:
        super().__init__()
        self.inner = inner
        self.__dict__["group"] = group
        self.index = index
        self.in_features, self.out_features = inner.in_features, inner.out_features

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.group.output(self.index, x)

    def extra_repr(self) -> str:
        return f"member {self.index} of {len(self.group.members)}, norm_fused={self.group.norm is not None}"


class DeferredNorm(nn.Module):
    """A norm whose work moved into the group that consumes its output: passes its input through."""

    def __init__(self, norm: NPRMSNorm) -> None:
        super().__init__()
        self.norm = norm

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x


_DEFAULT_GROUPS = (("q_proj", "k_proj", "v_proj"), ("gate_proj", "up_proj"))
_DEFAULT_NORMS = {"self_attn": "input_layernorm", "mlp": "post_attention_layernorm"}


def group_shared_input_linears(model: nn.Module, groups=_DEFAULT_GROUPS, norms=_DEFAULT_NORMS) -> int:
    """Group every set of sibling linears named as in *groups* (all :class:`NPVQLinear`, same
    input width / index width / codebook layout).  *norms* maps the name of the module that holds
    a group (``self_attn``, ``mlp`` in Llama-style decoder layers) to the name of the sibling
    :class:`NPRMSNorm` whose output feeds only that module; such a norm is folded into the group.
    Run after the lowering passes.  Returns the number of groups made."""
    made = 0
    for parent_name, parent in list(model.named_modules()):
        for names in groups:
            mods = [getattr(parent, n, None) for n in names]
            if not all(isinstance(m, NPVQLinear) for m in mods):
                continue
            norm = None
            holder_name = parent_name.rsplit(".", 1)[-1]
            norm_name = norms.get(holder_name) if norms else None
            grand = model.get_submodule(parent_name.rsplit(".", 1)[0]) if "." in parent_name else model
            if norm_name and isinstance(getattr(grand, norm_name, None), NPRMSNorm) and grand is not parent:
                norm = getattr(grand, norm_name)
            try:
                group = LinearGroup(mods, norm)
            except ValueError:
                continue
            for i, n in enumerate(names):
                setattr(parent, n, GroupedLinear(mods[i], group, i))
            if norm is not None:
                setattr(grand, norm_name, DeferredNorm(norm))
            made += 1
    return made
