"""The whole attention chain (module level) against the oracle chain, prefill-vs-decode
consistency through the KV store, and properties at the benchmark's full size.  Needs a B200."""
import math

import pytest
import torch

from oracle import hils_oracle as orc
from tests.util import check

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def _inputs(B, T, hq, hk, D, S, seed, dtype, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, hq, D, generator=g) * scale
    k = torch.randn(B, T, hk, D, generator=g) * scale
    off = torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5 * scale
    k[:, :(T // S) * S] += off.expand(-1, -1, S, -1, -1).reshape(B, (T // S) * S, hk, D)
    v = torch.randn(B, T, hk, D, generator=g) * scale
    return [t.to(dtype) for t in (q, k, v)]


from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore  # noqa: E402


def _core(hq, hk, K, S, W, **kw):
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    return HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W, **kw))


@pytest.mark.parametrize("cfg", [
    # B, T, hq, hk, D, S, K, W, dtype, pooling kw
    (1, 2048, 4, 4, 64, 64, 8, 512, F32, dict(enable_prior_query=False, enable_chunk_pooling=True)),  # config 1, fewer heads
    (2, 1024, 4, 4, 64, 64, 8, 256, BF, dict()),
    (1, 1024, 8, 2, 64, 64, 4, 128, BF, dict()),                                                       # GQA, per-q-head keys
    (1, 1024, 4, 2, 32, 32, 4, 64, BF, dict(enable_chunk_pooling=True, enable_softmax1=True)),
])
def test_chain_matches_oracle(cfg):
    B, T, hq, hk, D, S, K, W, dtype, kw = cfg
    q, k, v = _inputs(B, T, hq, hk, D, S, 21, dtype, scale=(1 / math.sqrt(D) if dtype == F32 else 1.0))
    core = _core(hq, hk, K, S, W, **kw).train()
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o, aux = core(qd, kd, vd, qd, return_aux=True)
    pooling = "mean" if kw.get("enable_chunk_pooling") else "attn"
    ref, raux = orc.hils_attention_chain(q, k, v, q, chunk_size=S, window_size=W, topk=K, pooling=pooling,
                                         use_prior_bias=kw.get("enable_prior_query", True),
                                         softmax1=kw.get("enable_softmax1", False), return_aux=True)
    same = (aux["indices"].cpu() == raux["indices"]).all(-1)                 # (B,T,hk)
    assert same.float().mean().item() >= 0.99
    rows = same.repeat_interleave(hq // hk, dim=2)
    check(o[rows.cuda()], ref.float()[rows], dtype, "chain output")
    check(aux["lse_swa"], raux["lse_swa"], dtype, "lse_swa")
    do = torch.randn(o.shape, generator=torch.Generator().manual_seed(5)).to(dtype)
    o.backward(do.cuda())
    # gradients on identical selections: autograd through the oracle chain run with the kernel's ids
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    ref2 = orc.hils_attention_chain(qr, kr, vr, qr, chunk_size=S, window_size=W, topk=K, pooling=pooling,
                                    use_prior_bias=kw.get("enable_prior_query", True),
                                    softmax1=kw.get("enable_softmax1", False), act_dtype=dtype,
                                    forced_indices=aux["indices"].cpu())
    check(o, ref2, dtype, "chain output (kernel ids)")
    ref2.float().backward(do.float())
    for n, a, r in (("dq", qd, qr), ("dk", kd, kr), ("dv", vd, vr)):
        check(a.grad, r.grad, dtype, "chain " + n)


def test_chain_gradients_match_oracle_fp32():
    """fp32, selection frozen to the kernel's ids: gradients of the chain wrt q, k, v against
    autograd through the oracle with the same ids."""
    B, T, H, D, S, K, W = 1, 512, 2, 32, 32, 4, 64
    q, k, v = _inputs(B, T, H, H, D, S, 33, F32, scale=0.5)
    core = _core(H, H, K, S, W).train()
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o, aux = core(qd, kd, vd, qd, return_aux=True)
    do = torch.randn(o.shape, generator=torch.Generator().manual_seed(6))
    o.backward(do.cuda())
    idx = aux["indices"].cpu()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    swa_o, lse = orc.swa(qr, kr, vr, W, S)
    N = T // S
    lmk_k, pb = orc.chunk_attn_pool(qr[:, S - 1::S][:, :N], kr[:, :N * S].reshape(B, N, S, H, D))
    sel = lmk_k[torch.arange(B).view(B, 1, 1, 1), idx.clamp_min(0).long(), torch.arange(H).view(1, 1, H, 1)]
    sc = torch.einsum("blhd,blhkd->blhk", qr, sel) / math.sqrt(D)
    sc = sc.masked_fill(idx < 0, float("-inf"))
    w = orc.inter_chunk_weights(sc, idx, lse, pb)
    oh = orc.sparse_attn(qr, kr, vr, w, idx, chunk_size=S)
    ref = oh + swa_o * w[..., -1:]
    check(o, ref, F32, "o")
    ref.backward(do)
    for n, a, b in (("dq", qd, qr), ("dk", kd, kr), ("dv", vd, vr)):
        check(a.grad, b.grad, F32, n)


@pytest.mark.parametrize("B", [1, 3])
def test_prefill_then_decode_matches_full_forward(B):
    """Feeding the sequence through the KV store (prefill 700 tokens, one 100-token chunk-prefill,
    then single-token decode steps) reproduces the one-shot forward: same ids, same outputs."""
    from hils_attention_b200.cache import HiLSCache
    T, hq, hk, D, S, K, W = 832, 4, 2, 64, 64, 4, 128
    q, k, v = _inputs(B, T, hq, hk, D, S, 44, BF)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    core = _core(hq, hk, K, S, W).eval()
    with torch.no_grad():
        full, faux = core(qd, kd, vd, qd, return_aux=True)
        cache = HiLSCache()
        outs, ids = [], []
        for lo, hi in [(0, 700), (700, 800)] + [(t, t + 1) for t in range(800, T)]:
            o, aux = core(qd[:, lo:hi], kd[:, lo:hi], vd[:, lo:hi], qd[:, lo:hi], past_key_values=cache,
                          use_cache=True, return_aux=True)
            outs.append(o)
            ids.append(aux["indices"])
    got, gid = torch.cat(outs, 1), torch.cat(ids, 1)
    same = (gid == faux["indices"]).all(-1)
    assert same.float().mean().item() >= 0.99
    rows = same.repeat_interleave(hq // hk, dim=2)
    check(got[rows], full[rows], BF, "decode vs full")
    assert cache.get_seq_length(1) == T


@pytest.mark.parametrize("cfg", [(2, 4, 2, 64, BF), (3, 4, 4, 128, BF), (1, 2, 2, 64, F32)])
def test_fused_decode_step_matches_op_by_op(cfg):
    """Single-token steps through the one-call decode step (hils_decode_step) give the outputs of the
    same steps run op by op, including across a chunk boundary (where the fused path steps aside) and
    with a selection query different from the attention query."""
    from hils_attention_b200.cache import HiLSCache
    B, hq, hk, D, dtype = cfg
    T0, n_dec, S, K, W = 640, 70, 64, 4, 128
    q, k, v = _inputs(B, T0 + n_dec, hq, hk, D, S, 45, dtype)
    lq = torch.randn(q.shape, generator=torch.Generator().manual_seed(46)).to(dtype)
    qd, kd, vd, ld = q.cuda(), k.cuda(), v.cuda(), lq.cuda()
    core = _core(hq, hk, K, S, W).eval()
    outs = {}
    with torch.no_grad():
        for fused in (True, False):
            cache = HiLSCache()
            core(qd[:, :T0], kd[:, :T0], vd[:, :T0], ld[:, :T0], past_key_values=cache, use_cache=True)
            res = []
            for t in range(T0, T0 + n_dec):
                r = core(qd[:, t:t + 1], kd[:, t:t + 1], vd[:, t:t + 1], ld[:, t:t + 1], past_key_values=cache,
                         use_cache=True, return_aux=not fused)          # return_aux forces the op-by-op path
                res.append(r if fused else r[0])
            outs[fused] = torch.cat(res, 1)
            assert cache.get_seq_length(1) == T0 + n_dec
    check(outs[True], outs[False], dtype, "fused vs op-by-op decode")


@pytest.mark.parametrize("B", [1])
def test_full_size_properties(B):
    """Benchmark-sized sequence (T=8192, 16 heads, D=64, K=32): size-independent properties.
    ids ascending, in the causal remote range, -1 only as trailing padding with the right count;
    the sparse attention is linear in v and in the weights; weights sum to one."""
    import hils_attention_b200 as hb
    T, H, D, S, K, W = 8192, 16, 64, 64, 32, 512
    q, k, v = _inputs(B, T, H, H, D, S, 2, BF)
    core = _core(H, H, K, S, W).eval()
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    with torch.no_grad():
        o, aux = core(qd, kd, vd, qd, return_aux=True)
        idx, w = aux["indices"], aux["weights"].contiguous()
        t = torch.arange(T, device="cuda")
        lim = ((t - W + 1).div(S, rounding_mode="floor")).clamp(0, T // S).view(1, T, 1, 1)
        assert bool(((idx < lim) & (idx >= -1)).all())
        nvalid = (idx >= 0).sum(-1)
        assert torch.equal(nvalid, torch.minimum(lim.squeeze(-1).expand_as(nvalid), torch.full_like(nvalid, K)))
        srt = idx.masked_fill(idx < 0, 1 << 30)
        assert bool((srt[..., 1:] > srt[..., :-1]).logical_or(srt[..., 1:] == (1 << 30)).all())
        assert bool((w.float().sum(-1) - 1).abs().max() < 2e-2)
        o1 = hb.HiLS_block_M_head(qd, kd, vd, w, idx, block_size=S, is_training=False)
        o2 = hb.HiLS_block_M_head(qd, kd, (2 * vd.float()).to(BF), w, idx, block_size=S, is_training=False)
        check(o2, 2 * o1.float(), BF, "linearity in v")
        o3 = hb.HiLS_block_M_head(qd, kd, vd, (0.5 * w.float()).to(BF), idx, block_size=S, is_training=False)
        check(o3, 0.5 * o1.float(), BF, "linearity in weights")
        assert torch.isfinite(o.float()).all()


@pytest.mark.gpu
def test_host_pipeline_matches_direct_steps():
    """Steps fed from pinned host memory through HostPipeline give the results of the same steps run
    directly, for every queued batch (copies of neighbouring steps overlap the kernels)."""
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    from hils_attention_b200.host_pipeline import HostPipeline
    dev = torch.device("cuda", 0)
    B, T, H, D, S, K, W = 1, 1024, 4, 64, 64, 4, 128
    core = HiLSAttentionCore(HiLSAttentionConfig(H, H, K, S, W)).train()

    def step(q, k, v, do):
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = core(q, k, v, q)
        o.backward(do)
        return o.detach(), q.grad, k.grad, v.grad

    g = torch.Generator().manual_seed(77)
    batches = [[torch.randn(B, T, H, D, generator=g).to(torch.bfloat16).pin_memory() for _ in range(4)]
               for _ in range(5)]
    outs = [[torch.empty_like(b[0]).pin_memory() for _ in range(4)] for b in batches]
    pipe = HostPipeline(step, batches[0], dev, depth=2)
    for b, o in zip(batches, outs):
        pipe.submit(b, o)
    pipe.drain()
    for b, o in zip(batches, outs):
        ref = step(*[t.to(dev) for t in b])
        for got, want in zip(o, ref):   # fp32 atomics in the key-gradient accumulation: last-bit differences only
            w = want.float().cpu()
            assert (got.float() - w).abs().max() <= 2e-2 * w.abs().max()


@pytest.mark.parametrize("rope", [False, True])
def test_shared_prior_query_replaces_the_landmark_queries(rope):
    """shared_q_c (models/FlashHiLS/hils_attention.py:271-276, :425-432): the chunk pooling is queried by one
    learned vector per head, rotated to each chunk's last position when the model rotates its landmark queries.
    The chain must equal the oracle chain fed the chunk keys pooled with that query, and the learned query must
    receive a gradient."""
    from hils_attention_b200 import ops
    torch.manual_seed(3)
    B, T, hq, hk, D, S, W, K = 1, 1024, 4, 2, 64, 64, 128, 4
    g = torch.Generator().manual_seed(21)
    q, k, v = (torch.randn(B, T, h, D, generator=g) for h in (hq, hk, hk))
    cfg = HiLSAttentionConfig(hq, hk, K, S, W, shared_q_c=True, apply_hils_rope=rope, head_dim=D, initializer_range=1.0)
    core = HiLSAttentionCore(cfg).cuda().train()
    pos = torch.arange(T, dtype=torch.float32)
    inv = 1.0 / (10000 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.cat([pos[:, None] * inv[None, :]] * 2, -1)
    cos, sin = ang.cos()[None].cuda(), ang.sin()[None].cuda()
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    o, aux = core(qd, kd, vd, qd, return_aux=True, position_embeddings=(cos, sin) if rope else None)
    o.sum().backward()
    assert core.q_c.grad is not None and torch.isfinite(core.q_c.grad).all() and core.q_c.grad.abs().sum() > 0
    # the oracle chain with the same pooling queries (rotation restated in plain torch)
    mu = core.q_c.detach().float().cpu()[None, None].expand(B, T // S, -1, -1)
    if rope:
        c, sn = cos.cpu()[:, S - 1::S, None, :], sin.cpu()[:, S - 1::S, None, :]
        half = torch.cat([-mu[..., D // 2:], mu[..., :D // 2]], -1)
        mu = mu * c + half * sn
    ref = orc.hils_attention_chain(q, k, v, q, chunk_size=S, window_size=W, topk=K, mu_q=mu,
                                   forced_indices=aux["indices"].cpu())
    check(o, ref, F32, "chain output with the shared prior query")
