"""Pins the CPU oracle against fixtures produced by the reference's own PyTorch functions
(tests/golden/make_golden.py).  CPU only."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import hils_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _load(name):
    d = np.load(os.path.join(GOLDEN, name))
    return {k: torch.from_numpy(d[k]) for k in d.files}


@pytest.mark.parametrize("tag", ["a", "b"])
def test_pool_matches_reference(tag):
    g = _load(f"pool_{tag}.npz")
    mu = g["mu_q"].clone().requires_grad_(True)
    kc = g["k_chunked"].clone().requires_grad_(True)
    lk, lb = orc.chunk_attn_pool(mu, kc)
    torch.testing.assert_close(lk, g["lmk_k"], atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lb, g["lmk_b"], atol=1e-5, rtol=1e-5)
    ((lk * g["g_lmk_k"]).sum() + (lb * g["g_lmk_b"]).sum()).backward()
    torch.testing.assert_close(mu.grad, g["d_mu_q"], atol=1e-5, rtol=1e-4)
    torch.testing.assert_close(kc.grad, g["d_k"], atol=1e-5, rtol=1e-4)


@pytest.mark.parametrize("tag", ["shared", "bias_pq", "decode", "ragged"])
def test_selection_matches_reference(tag):
    g = _load(f"topk_{tag}.npz")
    K, S, W, qo = [int(x) for x in g["args"]]
    idx, sc = orc.topk_select(g["q"], g["lmks"], g["lse_swa"], K, S, W, True, qo,
                              bias=g.get("bias"), gumbel_noise=g.get("gumbel"))
    assert torch.equal(idx, g["indices"].to(torch.int32))          # bit-exact ids
    fin = torch.isfinite(g["scores"])
    assert torch.equal(fin, torch.isfinite(sc))
    torch.testing.assert_close(sc[fin], g["scores"][fin], atol=1e-5, rtol=1e-5)


def test_selector_tie_rule():
    keys = torch.tensor([[1.0, 3.0, 3.0, float("-inf"), 3.0, 0.5, 1.0]])
    assert orc.stable_topk_from_keys(keys, 2).tolist() == [[1, 2]]
    assert orc.stable_topk_from_keys(keys, 4).tolist() == [[0, 1, 2, 4]]
    assert orc.stable_topk_from_keys(keys, 8).tolist() == [[0, 1, 2, 4, 5, 6, -1, -1]]
    none = torch.full((1, 5), float("-inf"))
    assert orc.stable_topk_from_keys(none, 4).tolist() == [[-1, -1, -1, -1]]


@pytest.mark.parametrize("tag", ["a", "kvlong"])
def test_sparse_attn_matches_reference(tag):
    g = _load(f"sparse_{tag}.npz")
    S = int(g["args"][0])
    q, k, v, w = [g[n].clone().requires_grad_(True) for n in ("q", "k", "v", "w")]
    o = orc.sparse_attn(q, k, v, w, g["indices"], chunk_size=S, mask_last_token=True)
    torch.testing.assert_close(o, g["o"], atol=2e-5, rtol=1e-4)
    o.backward(g["do"])
    for name, t in (("dq", q), ("dk", k), ("dv", v), ("dw", w)):
        torch.testing.assert_close(t.grad, g[name], atol=5e-5, rtol=1e-4, msg=name)


@pytest.mark.parametrize("tag", ["a", "b"])
def test_log_z_matches_reference(tag):
    g = _load(f"logz_{tag}.npz")
    S, W = [int(x) for x in g["args"]]
    lz = orc.exact_chunk_log_z(g["q"], g["k"], chunk_size=S, window_size=W)
    fin = torch.isfinite(g["log_z"])
    assert torch.equal(fin, torch.isfinite(lz))
    torch.testing.assert_close(lz[fin], g["log_z"][fin], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("tag", ["mha", "gqa", "lmk"])
def test_naive_bsa_identity(tag):
    """SWA + exact log Z + stable top-k + factorised softmax + sparse attention reproduces the
    reference's dense naive-BSA output; this pins the SWA mask, the remote-chunk rule, the
    weight layout and the -1 handling in one shot."""
    g = _load(f"bsa_{tag}.npz")
    S, W, K, ml = [int(x) for x in g["args"]]
    o = orc.naive_bsa_chain(g["q"], g["k"], g["v"], chunk_size=S, window_size=W, topk=K,
                            mask_last_token=bool(ml))
    torch.testing.assert_close(o, g["o"], atol=2e-5, rtol=1e-4)
    _, lse = orc.swa(g["q"], g["k"], g["v"], W, S, mask_lmk=bool(ml), expand_to_chunk=True)
    torch.testing.assert_close(lse.permute(0, 2, 1), g["lse_swa"], atol=1e-5, rtol=1e-5)
    lz = orc.exact_chunk_log_z(g["q"], g["k"], chunk_size=S, window_size=W, mask_lmk=bool(ml))
    ref = g["log_z"].permute(0, 2, 1, 3)
    fin = torch.isfinite(ref)
    assert torch.equal(fin, torch.isfinite(lz))
    torch.testing.assert_close(lz[fin], ref[fin], atol=1e-5, rtol=1e-5)


def test_chain_runs_and_weights_sum_to_one():
    g = torch.Generator().manual_seed(7)
    B, L, H, D, S = 1, 320, 2, 32, 32
    q, k, v = (torch.randn(B, L, H, D, generator=g) / math.sqrt(D) for _ in range(3))
    o, aux = orc.hils_attention_chain(q, k, v, q, chunk_size=S, window_size=64, topk=4,
                                      pooling="mean", use_prior_bias=False, return_aux=True)
    assert o.shape == (B, L, H, D)
    torch.testing.assert_close(aux["weights"].sum(-1), torch.ones(B, L, H), atol=1e-5, rtol=0)
    idx = aux["indices"]
    lim = orc.remote_chunk_limit(torch.arange(L), 64, S).view(1, L, 1, 1)
    assert bool(((idx < lim) | (idx < 0)).all())


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_norm_rope_matches_reference(tag):
    """Oracle restatement of per-head RMSNorm + rotary embedding against fixtures produced by the
    reference's rms_norm and rotate_half_torch."""
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"normrope_{tag}.npz"))
    g = {k: torch.from_numpy(d[k]) for k in d.files}
    dt = torch.bfloat16 if int(g["args"][0]) else torch.float32
    cs_dt = torch.float32 if int(g["args"][1]) else torch.bfloat16
    x, w = g["x"].to(dt), g["w"].to(dt)
    cos, sin = g["cos"].to(cs_dt), g["sin"].to(cs_dt)
    assert torch.equal(orc.rmsnorm_rope(x, w, 1e-6, cos, sin).float(), g["out"])
    assert torch.equal(orc.rmsnorm_rope(x, w, 1e-6).float(), g["out_norm_only"])
    assert torch.equal(orc.rmsnorm_rope(x, None, 1e-6, cos, sin).float(), g["out_rope_only"])


@pytest.mark.parametrize("cfg", [(2, 512, 4, 4, 32, 32, 64, 4), (1, 640, 8, 2, 32, 64, 128, 4)])
def test_sampled_rows_oracle_equals_full_chain(cfg):
    """hils_attention_rows (the chain for a sample of query rows, used at the benchmark shapes) reproduces
    the full oracle chain on those rows: ids exactly, outputs and weights to fp32 rounding."""
    from oracle import hils_oracle as orc
    B, L, hq, hk, D, S, W, K = cfg
    g = torch.Generator().manual_seed(1)
    q = torch.randn(B, L, hq, D, generator=g)
    k, v = (torch.randn(B, L, hk, D, generator=g) for _ in range(2))
    ref, aux = orc.hils_attention_chain(q, k, v, q, chunk_size=S, window_size=W, topk=K, return_aux=True)
    b = torch.randint(0, B, (48,), generator=g)
    t = torch.randint(0, L, (48,), generator=g)
    heads = list(range(hk)) if hk < 4 else [1, 3]
    out = orc.hils_attention_rows(q, k, v, q, b, t, heads, chunk_size=S, window_size=W, topk=K)
    hq_sel = out["query_heads"]
    assert torch.equal(out["indices"], aux["indices"][b, t][:, heads])
    assert (out["o"] - ref[b, t][:, hq_sel]).abs().max() < 2e-6
    assert (out["weights"] - aux["weights"][b, t][:, hq_sel]).abs().max() < 2e-6
    # forced ids reproduce the same result and carry a gradient to the sampled rows only
    qf = q.clone().requires_grad_(True)
    out2 = orc.hils_attention_rows(qf, k, v, q, b, t, heads, chunk_size=S, window_size=W, topk=K,
                                   forced_indices=out["indices"])
    assert (out2["o"] - out["o"]).abs().max() < 2e-6
    out2["o"].sum().backward()
    touched = qf.grad.abs().sum((2, 3)) > 0
    mask = torch.zeros(B, L, dtype=torch.bool)
    mask[b, t] = True
    assert torch.equal(touched & ~mask, torch.zeros_like(mask))
