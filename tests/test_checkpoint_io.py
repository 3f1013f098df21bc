"""Checkpoint round trip against a file written by the reference's own ``save_quantized_model``
(``tests/golden/reference_checkpoint.safetensors``, made by ``make_checkpoint_fixture.py``):
load -> save is byte-identical, load -> lower -> save (which unlowers and lowers again) is
byte-identical, codebooks shared in the file are shared again after loading, and on a GPU the
lowered model computes what the oracle computes from the file's tensors."""

from pathlib import Path

import pytest
import torch
from torch import nn

import oracle
from helpers import assert_output_close
from neuropress_b200.kernel_lowering import is_lowered
from neuropress_b200.nn import NPEmbedding, NPLinear, NPVQLinear, VQProxy
from neuropress_b200.t2n.model_io import load_quantized_model, save_quantized_model
from neuropress_b200.t2n.qtensors import load_qtensor, save_qtensor

FIXTURE = Path(__file__).parent / "golden" / "reference_checkpoint.safetensors"


def fresh_model() -> nn.Module:
    """The float architecture the fixture was saved from."""
    m = nn.Module()
    m.q_proj = nn.Linear(64, 48, bias=True)
    m.k_proj = nn.Linear(64, 16, bias=False)
    m.o_proj = nn.Linear(64, 32, bias=False)
    m.up_proj = nn.Linear(128, 24, bias=True)
    m.embed_tokens = nn.Embedding(20, 64)
    m.norm = nn.LayerNorm(64)
    m.register_buffer("steps", torch.zeros(3, dtype=torch.int64))
    return m


def test_load_then_save_is_byte_identical(tmp_path):
    model = fresh_model()
    manifest = load_quantized_model(model, FIXTURE, kernel_lowering=None)
    assert manifest.qtensor_params == {"q_proj.weight": "QTensorTractVQ", "k_proj.weight": "QTensorTractVQ",
                                       "o_proj.weight": "QTensorTractScaleOnly", "up_proj.weight": "QTensorScaleZp",
                                       "embed_tokens.weight": "QTensorTractScaleOnly"}
    assert not is_lowered(model)
    assert torch.equal(model.steps, torch.arange(3))                   # plain buffers restored
    q, k = model.q_proj._parameters["weight"], model.k_proj._parameters["weight"]
    assert q.qscheme.centroids is k.qscheme.centroids                  # one codebook object again
    assert q.qscheme.is_packed_indices == 12 and k.qscheme.column_permutation is not None
    out = tmp_path / "again.safetensors"
    save_quantized_model(model, out)
    assert out.read_bytes() == FIXTURE.read_bytes()


def test_load_lower_save_is_byte_identical(tmp_path):
    model = fresh_model()
    load_quantized_model(model, FIXTURE)                               # lowers ("auto")
    assert is_lowered(model)
    assert isinstance(model.q_proj, NPVQLinear) and isinstance(model.k_proj, NPVQLinear)
    assert isinstance(model.o_proj, NPLinear) and isinstance(model.up_proj, NPLinear)
    assert isinstance(model.embed_tokens, NPEmbedding) and isinstance(model.norm, nn.LayerNorm)
    assert model.q_proj.proxy is model.k_proj.proxy                    # shared proxy survives the file
    assert sum(isinstance(m, VQProxy) for m in model.modules()) == 1
    assert model.up_proj.qtype == "asym" and model.up_proj.group_size == 64 and model.q_proj.bits == 12
    assert model.k_proj.column_perm is not None
    out = tmp_path / "again.safetensors"
    save_quantized_model(model, out)                                   # unlower -> write -> lower
    assert out.read_bytes() == FIXTURE.read_bytes()
    assert is_lowered(model) and isinstance(model.q_proj, NPVQLinear)  # and it is lowered again


def test_single_qtensor_files_round_trip(tmp_path):
    model = fresh_model()
    load_quantized_model(model, FIXTURE, kernel_lowering=None)
    for name in ("q_proj", "k_proj", "o_proj", "up_proj"):
        q = getattr(model, name)._parameters["weight"]
        save_qtensor(q, tmp_path / f"{name}.safetensors")
        r = load_qtensor(tmp_path / f"{name}.safetensors")
        assert type(r) is type(q) and torch.equal(r.u8_blob, q.u8_blob) and tuple(r.shape) == tuple(q.shape)
        # a file with several metadata keys is not byte-stable (safetensors keeps them in a hash
        # map): compare what the two objects serialize to instead
        from neuropress_b200.t2n.qtensors import _SERDE_REGISTRY, qtensor_type_name

        serde = _SERDE_REGISTRY[qtensor_type_name(q)]
        assert serde.to_metadata(r) == serde.to_metadata(q)
        tq, tr = serde.to_tensors(q), serde.to_tensors(r)
        assert list(tq) == list(tr) and all(torch.equal(tq[k2], tr[k2]) for k2 in tq)


def test_missing_manifest_is_rejected(tmp_path):
    from safetensors.torch import save_file

    save_file({"w": torch.zeros(2)}, str(tmp_path / "plain.safetensors"))
    with pytest.raises(ValueError, match="__neuropress_manifest__"):
        load_quantized_model(fresh_model(), tmp_path / "plain.safetensors")


@pytest.mark.gpu
def test_loaded_checkpoint_runs_on_the_kernels():
    from safetensors import safe_open

    model = fresh_model().cuda()
    load_quantized_model(model, FIXTURE)
    with safe_open(str(FIXTURE), framework="pt") as f:
        t = {k: f.get_tensor(k) for k in f.keys()}
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 64, generator=g).to(torch.bfloat16)
    y = model.q_proj(x.cuda())
    ref = oracle.vq_forward_f32(x, t["q_proj.weight::u8_blob"], t["q_proj.weight::centroids"], 12, 48, 64,
                                t["q_proj.bias"])
    assert_output_close(y, ref, torch.bfloat16)
    perm = t["k_proj.weight::column_permutation"]
    yk = model.k_proj(x.cuda())
    refk = oracle.vq_forward_f32(x[:, perm], t["k_proj.weight::u8_blob"], t["k_proj.weight::centroids"], 8, 16, 64)
    assert_output_close(yk, refk, torch.bfloat16)
    yo = model.o_proj(x.cuda())
    assert_output_close(yo, oracle.q_forward_f64(x, t["o_proj.weight::u8_blob"], t["o_proj.weight::scale"], 4, 32),
                        torch.bfloat16)
    xu = torch.randn(3, 128, generator=g).to(torch.bfloat16)
    yu = model.up_proj(xu.cuda())
    assert_output_close(yu, oracle.q_forward_f64(xu, t["up_proj.weight::u8_blob"], t["up_proj.weight::scale"], 4, 64,
                                                 t["up_proj.weight::zero_point"], t["up_proj.bias"]), torch.bfloat16)
    ids = torch.tensor([[0, 19, 7]])
    ye = model.embed_tokens(ids.cuda())
    want = oracle.q_embedding(ids, t["embed_tokens.weight::u8_blob"], t["embed_tokens.weight::scale"], 4, 32,
                              out_dtype=torch.bfloat16)
    assert torch.equal(ye.cpu(), want)
