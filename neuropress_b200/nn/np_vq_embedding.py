"""NPVQEmbedding: embedding lookup for VQ-compressed embedding tables.

Same surface as the reference module (neuropress/nn/np_vq_embedding.py): the codebook indices
of the whole table are unpacked once at construction into the ``[vocab, n_groups]`` 16-bit
buffer ``all_indices`` (:88), the codebook lives in a shared :class:`VQProxy` that is not a
sub-module, and ``forward`` returns ``[..., embedding_dim]``.  The reference's forward is two
PyTorch gathers plus a reshape, a permutation, a scalar multiply and a cast (:119-141); here it
is one CUDA kernel (``npb_vq_embedding``) that decodes only the selected rows with exactly that
arithmetic.  There is no CPU path: ids and module must be on a CUDA device.
"""

from __future__ import annotations

import logging

import torch
import torch.nn as nn

from .np_vq_linear import VQProxy, _is_vq_weight

log = logging.getLogger(__name__)


class _WeightProxy:
    """What ``NPVQEmbedding.weight`` returns: supports ``weight[token_id]`` / ``weight[ids, ...]``
    by a lookup of those rows, never materialising the ``[vocab, dim]`` matrix (reference :23-57)."""

    __slots__ = ("_emb",)

    def __init__(self, emb: "NPVQEmbedding") -> None:
        self._emb = emb

    @property
    def shape(self) -> tuple[int, int]:
        return (self._emb.all_indices.shape[0], self._emb.embedding_dim)

    def __getitem__(self, key: object) -> torch.Tensor:
        row_key, rest = (key[0], key[1:]) if isinstance(key, tuple) else (key, ())
        scalar = isinstance(row_key, int)
        ids = torch.tensor([row_key] if scalar else list(row_key), dtype=torch.long,
                           device=self._emb.all_indices.device)
        out = self._emb(ids)
        if scalar:
            out = out[0]
        return out[rest] if rest else out


class NPVQEmbedding(nn.Module):
    """VQ-compressed embedding with pre-unpacked indices (constructor as the reference's, :77-109)."""

    def __init__(self, all_indices: torch.Tensor, proxy: VQProxy, embedding_dim: int, vector_len: int,
                 scale: float = 1.0, inv_perm: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> None:
        super().__init__()
        if all_indices.dim() != 2 or all_indices.shape[1] * vector_len != embedding_dim:
            raise ValueError("all_indices must be [vocab, embedding_dim // vector_len].")
        if proxy.vector_len != vector_len:
            raise ValueError("vector_len does not match the proxy's codebook.")
        self.register_buffer("all_indices", all_indices.to(torch.int16).contiguous())
        object.__setattr__(self, "proxy", proxy)   # shared codebook: not a sub-module
        self.embedding_dim = embedding_dim
        self.vector_len = vector_len
        self.scale = scale
        if inv_perm is not None:
            self.register_buffer("inv_perm", inv_perm.to(torch.int64).contiguous())
        else:
            self.inv_perm: torch.Tensor | None = None
        self.out_dtype = out_dtype
        self._source_qtensor = None

    def to_qtensor(self):
        """The VQ QTensor this module was lowered from (reference :111-117)."""
        if self._source_qtensor is None:
            raise RuntimeError("NPVQEmbedding._source_qtensor is None — was this module built via "
                               "linearize_vq_embeddings()? Cannot unlower for save.")
        return self._source_qtensor

    @property
    def weight(self) -> _WeightProxy:
        return _WeightProxy(self)

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        from .. import kernels

        return kernels.vq_embedding(input_ids, self.all_indices, self.proxy.centroids, self.embedding_dim,
                                    float(self.scale), self.inv_perm, self.out_dtype)

    def extra_repr(self) -> str:
        scale_str = f", scale={self.scale:.4g}" if self.scale != 1.0 else ""
        perm_str = ", perm=True" if self.inv_perm is not None else ""
        dtype_str = f", out_dtype={self.out_dtype}" if self.out_dtype else ""
        return (f"vocab={self.all_indices.shape[0]}, dim={self.embedding_dim}, vector_len={self.vector_len}, "
                f"num_centroids={self.proxy.num_centroids}{scale_str}{perm_str}{dtype_str}")


def linearize_vq_embeddings(model: nn.Module) -> int:
    """Replace every non-``nn.Linear`` module whose ``weight`` is a VQ QTensor by an
    :class:`NPVQEmbedding` (reference :161-289).  Codebooks already held by a :class:`VQProxy`
    of the model are reused; new ones are registered on the model root as ``_vq_emb_proxy_<i>``.
    A module attribute ``embed_scale`` becomes the lookup's ``scale``; entropy-coded index streams
    are skipped with a warning.  Returns the number of replacements."""
    from ..transforms.vq_packing import IndexPacking

    proxy_cache = {id(m.centroids): m for m in model.modules() if isinstance(m, VQProxy)}
    new_proxies: dict[int, VQProxy] = {}
    replacements: list[tuple[str, NPVQEmbedding]] = []
    try:
        out_dtype = next(p.dtype for p in model.parameters()
                         if getattr(p, "dtype", None) in (torch.float16, torch.bfloat16))
    except StopIteration:
        out_dtype = None
    for name, module in model.named_modules():
        if isinstance(module, NPVQEmbedding | nn.Linear):
            continue
        weight = module._parameters.get("weight") if hasattr(module, "_parameters") else None
        if weight is None:
            weight = module.__dict__.get("weight")
        if weight is None or not _is_vq_weight(weight):
            continue
        qscheme = weight.qscheme
        if getattr(qscheme, "use_tiered", False) or getattr(qscheme, "tier_bits", None) \
                or getattr(qscheme, "zero_escape", False):
            log.warning("linearize_vq_embeddings: skipping %s — tiered/ntier/zero-escape packing not "
                        "supported for embeddings.", name)
            continue
        shape = getattr(qscheme, "original_shape", None) or getattr(weight, "shape", None)
        if shape is None:
            log.warning("linearize_vq_embeddings: skipping %s — the table's shape is unknown.", name)
            continue
        vocab, dim = int(shape[0]), int(shape[1])
        vl = qscheme.vector_len
        groups = dim // vl
        cid = id(qscheme.centroids)
        proxy = proxy_cache.get(cid) or new_proxies.get(cid)
        if proxy is None:
            proxy = new_proxies[cid] = VQProxy(qscheme.centroids)
        idx = IndexPacking.unpack(weight.u8_blob, qscheme.is_packed_indices, vocab * groups)
        perm = getattr(qscheme, "column_permutation", None)
        emb = NPVQEmbedding(idx.reshape(vocab, groups).to(torch.int16), proxy, dim, vl,
                            scale=float(getattr(module, "embed_scale", 1.0)),
                            inv_perm=None if perm is None else torch.argsort(perm.detach().clone()),
                            out_dtype=out_dtype)
        emb._source_qtensor = weight
        replacements.append((name, emb))
    if not replacements:
        log.info("linearize_vq_embeddings: no VQ-weight embedding layers found.")
        return 0
    taken = {n for n, m in model.named_modules() if isinstance(m, VQProxy)}
    for i, proxy in enumerate(new_proxies.values()):
        if f"_vq_emb_proxy_{i}" not in taken:
            model.add_module(f"_vq_emb_proxy_{i}", proxy)
    for name, emb in replacements:
        parent = model.get_submodule(name.rsplit(".", 1)[0]) if "." in name else model
        setattr(parent, name.rsplit(".", 1)[-1], emb)
    log.info("linearize_vq_embeddings: replaced %d layer(s).", len(replacements))
    return len(replacements)
