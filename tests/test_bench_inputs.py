"""The synthetic inputs `bench.py` feeds the kernels, checked on the CPU: the overlapping chunk ids that stand in for a
trained model's selections (the reference's own generator, ops/hils_fwd_bwd_head.py:96-187, restated vectorised) and
the sequence partition of the context-parallel workload."""
import torch

import bench


def test_overlap_indices_are_causal_sorted_and_overlap_as_asked():
    B, L, H, K, S, N, M = 1, 1024, 2, 8, 64, 16, 32
    idx = bench.overlap_indices(B, L, H, K, S, N, 0.8, M, torch.device("cpu"), 3)
    assert idx.shape == (B, L, H, K) and idx.dtype == torch.int32
    t = torch.arange(L).view(1, L, 1, 1)
    valid = idx >= 0
    assert bool((idx[valid] <= (t // S).expand_as(idx)[valid]).all())           # only causal chunks
    # ascending, -1 only at the tail
    filled = torch.where(valid, idx, torch.full_like(idx, N + 1))
    assert bool((filled[..., 1:] >= filled[..., :-1]).all())
    n_sel = valid.sum(-1)
    assert bool((n_sel == torch.clamp(t.squeeze(-1) // S + 1, max=K).expand_as(n_sel)).all())
    # a token inside a run keeps ~80 % of its predecessor's chunks (where both hold K of them)
    a, b = idx[:, 1:], idx[:, :-1]
    same = (a.unsqueeze(-1) == b.unsqueeze(-2)) & (a.unsqueeze(-1) >= 0)
    kept = same.any(-1).sum(-1).float()
    inside = (torch.arange(1, L) % M != 0).view(1, L - 1, 1) & (n_sel[:, 1:] == K) & (n_sel[:, :-1] == K)
    ratio = (kept[inside] / K).mean().item()
    assert 0.7 <= ratio <= 0.9, ratio
    # the first token of a run draws afresh
    first = (torch.arange(1, L) % M == 0).view(1, L - 1, 1) & (n_sel[:, 1:] == K) & (n_sel[:, :-1] == K)
    assert (kept[first] / K).mean().item() < 0.75


def test_workload_table_matches_the_baseline_configs():
    w = bench.WORKLOADS
    assert (w["c1"]["T"], w["c1"]["K"], w["c1"].get("dtype")) == (2048, 8, "f32")
    assert (w["c2"]["B"], w["c2"]["T"], w["c2"]["h_q"], w["c2"]["D"], w["c2"]["K"]) == (8, 8192, 16, 64, 32)
    assert (w["c3"]["T"], w["c3"]["h_q"], w["c3"]["D"], w["c3"]["K"]) == (65536, 32, 128, 32)
    assert (w["c4"]["B"], w["c4"]["T"]) == (32, 131072)
    assert (w["c5"]["T"], w["c5"]["T"] // w["c5"]["S"]) == (1048576, 16384)
