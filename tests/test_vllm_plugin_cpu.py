"""The vLLM quantisation plugin: registration, per-rank parameter shapes, and the weight loader
cutting unsharded checkpoint tensors to this rank's partition (checked against the CPU oracle's
quantisation of the sliced weight).  Needs an importable vLLM; no GPU."""
import pytest
import torch

from tests import helpers as H

vllm = pytest.importorskip("vllm", reason="vLLM is not installed")


@pytest.fixture(scope="module")
def plugin():
    try:
        from sharq_b200 import vllm_plugin
    except Exception as exc:  # an installed vLLM that cannot be imported on this machine
        pytest.skip(f"vLLM could not be imported: {exc}")
    return vllm_plugin


def _quantize(oracle, w):
    qw, sfs, sfd = oracle.quantize_w32_shared(H.bits(w))
    return {"QW": torch.from_numpy(qw.reshape(w.shape[0], -1)), "SFW_sparse": torch.from_numpy(sfs),
            "SFW_dense": torch.from_numpy(sfd), "scale_b": torch.tensor([0.25])}


def test_registered_and_capability(plugin):
    from vllm.model_executor.layers.quantization import get_quantization_config

    assert get_quantization_config("sharq") is plugin.SHARQConfig
    assert plugin.SHARQConfig.get_min_capability() == 100
    assert plugin.SHARQConfig.get_supported_act_dtypes() == [torch.bfloat16]


@pytest.mark.parametrize("rank", [0, 1])
def test_partitioned_weights_load_from_unsharded_checkpoint(plugin, oracle, monkeypatch, rank):
    world = 2
    monkeypatch.setattr(plugin, "_tp", lambda: (rank, world))
    method = plugin.SHARQLinearMethod(plugin.SHARQConfig(), prefix="layers.0.self_attn.qkv_proj")
    # merged column-parallel layer: q 512 rows, k and v 256 rows each, K = 512
    nq, nk, k = 512, 256, 512
    w = H.config0_w(nq + 2 * nk, k, 5)
    w = (w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16)
    full = _quantize(oracle, w)
    layer = torch.nn.Module()
    method.create_weights(layer, k, [nq // world, nk // world, nk // world], k, nq + 2 * nk, torch.bfloat16)
    assert tuple(layer.QW.shape) == ((nq + 2 * nk) // world, k // 2)
    for name, tensor in full.items():
        getattr(layer, name).weight_loader(getattr(layer, name), tensor)
    pieces = [(rank * 256, (rank + 1) * 256), (512 + rank * 128, 512 + (rank + 1) * 128), (768 + rank * 128, 768 + (rank + 1) * 128)]
    want = _quantize(oracle, torch.cat([w[b:e] for b, e in pieces]).contiguous())
    for name in ("QW", "SFW_sparse", "SFW_dense"):
        assert torch.equal(getattr(layer, name).data.cpu(), want[name]), name
    assert layer.scale_b_value == 0.25

    # row-parallel layer: K = 1024 cut in two
    method = plugin.SHARQLinearMethod(plugin.SHARQConfig(), prefix="layers.0.self_attn.o_proj")
    n, k = 256, 1024
    w = H.config0_w(n, k, 6)
    w = (w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16)
    full = _quantize(oracle, w)
    layer = torch.nn.Module()
    method.create_weights(layer, k // world, [n], k, n, torch.bfloat16)
    assert tuple(layer.QW.shape) == (n, k // world // 2)
    for name, tensor in full.items():
        getattr(layer, name).weight_loader(getattr(layer, name), tensor)
    want = _quantize(oracle, w[:, rank * 512:(rank + 1) * 512].contiguous())
    for name in ("QW", "SFW_sparse", "SFW_dense"):
        assert torch.equal(getattr(layer, name).data.cpu(), want[name]), name


def test_unsplittable_partitions_are_rejected(plugin, monkeypatch):
    monkeypatch.setattr(plugin, "_tp", lambda: (0, 2))
    method = plugin.SHARQLinearMethod(plugin.SHARQConfig(), prefix="x")
    with pytest.raises(ValueError):
        method.create_weights(torch.nn.Module(), 192, [256], 384, 256, torch.bfloat16)  # K/rank not a multiple of 128
    with pytest.raises(ValueError):
        method.create_weights(torch.nn.Module(), 256, [64], 256, 128, torch.bfloat16)  # 64-row partitions
