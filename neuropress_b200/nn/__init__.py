"""Quantized linear modules (the reference's ``neuropress.nn`` names for this path)."""

from .backends import (Backend, EmbeddingBackend, LinearBackend, NormBackend, VQBackend,
                       is_cuda_jit_available)
from .decode_ahead import DecodeAhead
from .grouped import DeferredNorm, GroupedLinear, LinearGroup, group_shared_input_linears
from .np_embedding import NPEmbedding, linearize_qtensor_embeddings
from .np_linear import NPLinear, linearize_qtensor_weights
from .np_rms_norm import NPRMSNorm, linearize_rms_norms
from .np_vq_embedding import NPVQEmbedding, linearize_vq_embeddings
from .np_vq_linear import NPVQLinear, VQProxy, linearize_vq_weights

__all__ = [
    "Backend", "EmbeddingBackend", "LinearBackend", "NormBackend", "VQBackend",
    "is_cuda_jit_available", "NPLinear", "linearize_qtensor_weights", "NPVQLinear", "VQProxy",
    "linearize_vq_weights", "NPRMSNorm", "linearize_rms_norms", "NPEmbedding",
    "linearize_qtensor_embeddings", "NPVQEmbedding", "linearize_vq_embeddings", "LinearGroup",
    "GroupedLinear", "DeferredNorm", "group_shared_input_linears", "DecodeAhead",
]
