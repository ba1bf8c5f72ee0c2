"""The device-side plan of the grouped mixture-of-experts step (decoder.moe_grouping), checked on the CPU
against a brute-force construction: the reference's per-expert loop (model/qMixtralLayer.py:223-231) visits
the experts in ascending order and, inside an expert, its tokens in ascending order (torch.where)."""
import pytest
import torch

from sharq_b200.decoder import moe_grouping


@pytest.mark.parametrize("tokens,experts,top_k,seed", [(384, 4, 2, 0), (1000, 8, 2, 1), (7, 4, 2, 2), (513, 8, 3, 3)])
def test_grouping_matches_per_expert_order(tokens, experts, top_k, seed):
    g = torch.Generator().manual_seed(seed)
    selected = torch.stack([torch.randperm(experts, generator=g)[:top_k] for _ in range(tokens)])
    if seed == 2:
        selected[:, 0], selected[:, 1] = 1, 3  # experts 0 and 2 get no token
    dest, src_row, unit_group = moe_grouping(selected, experts)
    rows = src_row.numel()
    assert rows % 256 == 0 and unit_group.numel() == rows // 256
    assert rows == ((tokens * top_k + 255) // 256 + experts) * 256
    cursor = 0
    for e in range(experts):
        toks = (selected == e).any(dim=1).nonzero().reshape(-1)            # ascending token order, as torch.where gives
        n = toks.numel()
        padded = (n + 255) // 256 * 256
        for i, t in enumerate(toks.tolist()):
            j = int((selected[t] == e).nonzero()[0])
            assert int(dest[t, j]) == cursor + i
            assert int(src_row[cursor + i]) == t
        assert bool((src_row[cursor + n:cursor + padded] == -1).all())      # padding rows of the segment
        assert bool((unit_group[cursor // 256:(cursor + padded) // 256] == e).all())
        cursor += padded
    assert bool((src_row[cursor:] == -1).all()) and bool((unit_group[cursor // 256:] == -1).all())
    assert sorted(dest.reshape(-1).tolist()) == sorted((src_row >= 0).nonzero().reshape(-1).tolist())
