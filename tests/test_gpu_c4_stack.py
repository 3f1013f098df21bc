"""Decoder-stack integration test on the Llama-3.2-1B layer shapes (hidden 2048, intermediate
8192, 32 query / 8 key-value heads of 64): every linear of a two-layer ``LlamaModel`` is swapped
for an ``NPVQLinear`` (one 4096-entry codebook per 2048-column group, 16-bit and 12-bit index
streams), the way ``linearize_vq_weights`` swaps modules, and the hidden states are compared
with the same model holding the oracle-decoded dense weights.  Covers prefill (decode + dense
GEMM band), single-token decoding on the KV cache (GEMV band) and CUDA-graph replay of a
decoding step.  Random weights and activations; no tokenizer, no checkpoint."""

import copy

import pytest
import torch

import oracle
from neuropress_b200.nn import NPVQLinear, VQProxy
from synthetic import make_vq_layer

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)

transformers = pytest.importorskip("transformers")


def _build(bits: int):
    from transformers import LlamaConfig, LlamaModel

    cfg = LlamaConfig(hidden_size=2048, intermediate_size=8192, num_hidden_layers=2,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=512,
                      max_position_embeddings=512, attn_implementation="sdpa")
    torch.manual_seed(0)
    dense = LlamaModel(cfg).to(torch.bfloat16)
    vq = copy.deepcopy(dense)
    seed = 0
    for (name, mod_d), (_, mod_q) in zip(list(dense.named_modules()), list(vq.named_modules())):
        for child_name, child in list(mod_d.named_children()):
            if not isinstance(child, torch.nn.Linear):
                continue
            n, k = child.out_features, child.in_features
            seed += 1
            d = make_vq_layer(n, k, num_centroids=4096, bits=bits, seed=seed, cols_per_codebook=2048)
            w = oracle.vq_decode(d.packed, d.centroids, d.bits, n, k, torch.bfloat16, **d.ext())
            child.weight.data = w
            layer = NPVQLinear(VQProxy(d.centroids), d.packed, d.bits, n, k, 8, backend="auto",
                               cols_per_codebook=2048)
            layer.proxy.to(DEV)
            setattr(mod_q, child_name, layer)
    return dense.to(DEV).eval(), vq.to(DEV).eval()


def _rel_rms(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double(), b.double()
    return float((a - b).pow(2).mean().sqrt() / b.pow(2).mean().sqrt())


@pytest.mark.parametrize("bits", [16, 12])
def test_llama_shaped_stack_matches_dense_weights(bits):
    dense, vq = _build(bits)
    n_lowered = sum(isinstance(m, NPVQLinear) for m in vq.modules())
    assert n_lowered == 14  # 7 linears x 2 layers
    g = torch.Generator().manual_seed(1)
    prompt = torch.randn(1, 64, 2048, generator=g).to(torch.bfloat16).to(DEV)
    step = torch.randn(1, 1, 2048, generator=g).to(torch.bfloat16).to(DEV)
    batch8 = torch.randn(8, 1, 2048, generator=g).to(torch.bfloat16).to(DEV)
    with torch.no_grad():
        od = dense(inputs_embeds=prompt, use_cache=True)
        oq = vq(inputs_embeds=prompt, use_cache=True)
        # bf16 stacks with different summation orders: the dense model is the yardstick
        assert _rel_rms(oq.last_hidden_state, od.last_hidden_state) < 2e-2
        dd = dense(inputs_embeds=step, past_key_values=od.past_key_values, use_cache=True)
        dq = vq(inputs_embeds=step, past_key_values=oq.past_key_values, use_cache=True)
        assert _rel_rms(dq.last_hidden_state, dd.last_hidden_state) < 2e-2
        # a batch of 8 single-token rows without cache (GEMV band at its upper edge)
        bd = dense(inputs_embeds=batch8, use_cache=False)
        bq = vq(inputs_embeds=batch8, use_cache=False)
        assert _rel_rms(bq.last_hidden_state, bd.last_hidden_state) < 2e-2

        # CUDA-graph replay of a cache-less decoding step of the lowered model
        static_in = batch8.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            vq(inputs_embeds=static_in, use_cache=False)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                static_out = vq(inputs_embeds=static_in, use_cache=False).last_hidden_state
            static_in.copy_(torch.flip(batch8, dims=[0]))
            graph.replay()
            side.synchronize()
        assert _rel_rms(static_out, torch.flip(bq.last_hidden_state, dims=[0])) < 1e-3

        # the norms on the input side of the linears, fused (LlamaRMSNorm: plain-weight convention)
        from neuropress_b200.nn import NPRMSNorm, linearize_rms_norms

        assert linearize_rms_norms(vq) == 5  # 2 per layer + the final norm
        assert sum(isinstance(m, NPRMSNorm) for m in vq.modules()) == 5
        nq = vq(inputs_embeds=prompt, use_cache=False)
        assert _rel_rms(nq.last_hidden_state, od.last_hidden_state) < 2e-2
        assert _rel_rms(nq.last_hidden_state, oq.last_hidden_state) < 1e-2
