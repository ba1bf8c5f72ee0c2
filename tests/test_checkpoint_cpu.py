"""Slicing a quantised SharQ checkpoint for tensor parallelism gives the bytes of quantising
the sliced weight (checked with the CPU oracle's weight quantiser)."""
import numpy as np
import pytest
import torch

from sharq_b200 import checkpoint as C
from tests import helpers as H


def _quantize(oracle, w_scaled: torch.Tensor):
    qw, sfs, sfd = oracle.quantize_w32_shared(H.bits(w_scaled))
    return {"QW": torch.from_numpy(qw.reshape(w_scaled.shape[0], -1)), "SFW_sparse": torch.from_numpy(sfs),
            "SFW_dense": torch.from_numpy(sfd), "scale_b": torch.ones(1)}


def _same(entry, want):
    for key in ("QW", "SFW_sparse", "SFW_dense"):
        assert entry[key].shape == want[key].shape, key
        assert torch.equal(entry[key], want[key]), key


@pytest.mark.parametrize("world", [2, 4])
def test_column_and_row_shards_equal_requantised_slices(oracle, world):
    n, k = 1024, 1024
    w = H.config0_w(n, k, 7)
    w = (w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16)  # pre-scaled by the GLOBAL scale
    full = _quantize(oracle, w)
    full["bias"] = torch.arange(n, dtype=torch.float32).to(torch.bfloat16)
    for rank in range(world):
        b, e = rank * n // world, (rank + 1) * n // world
        got = C.shard_rows(full, [(b, e)])
        _same(got, _quantize(oracle, w[b:e].contiguous()))
        assert torch.equal(got["bias"], full["bias"][b:e])
        kb, ke = rank * k // world, (rank + 1) * k // world
        got = C.shard_k(full, kb, ke)
        _same(got, _quantize(oracle, w[:, kb:ke].contiguous()))
        assert torch.equal(got["bias"], full["bias"])


def test_merged_layer_pieces(oracle):
    # merged qkv: 512 query rows, 256 key rows, 256 value rows, two ranks
    nq, nk, k, world = 512, 256, 512, 2
    w = H.config0_w(nq + 2 * nk, k, 3)
    w = (w.float() / (w.float().abs().max() / 2688)).to(torch.bfloat16)
    full = _quantize(oracle, w)
    for rank in range(world):
        pieces = C.merged_row_pieces([nq // world, nk // world, nk // world], world, rank)
        assert pieces == [(rank * 256, (rank + 1) * 256), (512 + rank * 128, 512 + (rank + 1) * 128),
                          (768 + rank * 128, 768 + (rank + 1) * 128)]
        local = torch.cat([w[b:e] for b, e in pieces]).contiguous()
        _same(C.shard_rows(full, pieces), _quantize(oracle, local))


def test_unaligned_slices_are_rejected(oracle):
    w = (H.config0_w(256, 256, 1).float() * 100).to(torch.bfloat16)
    full = _quantize(oracle, w)
    with pytest.raises(ValueError):
        C.shard_rows(full, [(0, 64)])
    with pytest.raises(ValueError):
        C.shard_k(full, 0, 64)


def test_checkpoint_round_trip(tmp_path, oracle):
    w = (H.config0_w(256, 256, 2).float() * 100).to(torch.bfloat16)
    entry = _quantize(oracle, w)
    tensors = {f"model.layers.0.mlp.down_proj.{k2}": v for k2, v in entry.items()}
    tensors["model.norm.weight"] = torch.ones(256, dtype=torch.bfloat16)
    path = str(tmp_path / "model.safetensors")
    C.save_checkpoint(tensors, path)
    back = C.load_checkpoint(path)
    assert set(back) == set(tensors)
    got = C.layer_entry(back, "model.layers.0.mlp.down_proj")
    _same(got, entry)
    assert C.sf_bytes(256, 256) == entry["SFW_dense"].numel()
