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


def test_reference_arm_prints_one_contract_line():
    """`bench.py --impl reference` (the CPU restatement on the host cores) prints one JSON line with the keys the
    comparison needs; no GPU is touched."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    out = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, env=env, cwd=root)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 1
    assert d["metric"] == "hils_attn_fwd_bwd_tokens_per_s" and d["unit"] == "tokens/s" and d["value"] > 0
    assert d["config"]["workload"] == "c1" and d["dtype"] == "f32"
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
