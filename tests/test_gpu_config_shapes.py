"""Parity at the shapes of the five benchmark configurations.

The CPU oracle cannot run these sizes in full, so each test runs the CUDA chain at the configuration's own
shape (the code paths the benchmark takes) and compares a SAMPLE of query rows with the oracle evaluated for
exactly those rows (oracle.hils_attention_rows: window branch, selection over all chunk keys, inter-chunk
softmax, sparse chunk attention, combine; cost O(rows * (W + N + K*S))).  Selection: the kernel's ids must be
the stable selector applied to the kernel's own fp32 ranking values (bit-exact) and agree with the oracle's own
choice on >= 99 % of the rows (the reference's acceptance bar, ops/topk_head_softmax.py:1472); outputs and
gradients are compared on rows whose ids agree.  Inputs follow the configurations: q, v ~ N(0,1), k ~ N(0,1) +
per-(chunk, head) offset ~ N(0, 0.5), seeded.  Needs a B200.
"""
import math

import pytest
import torch

from oracle import hils_oracle as orc
from tests.util import check

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


def _inputs(B, T, hq, hk, D, S, seed, dtype=BF, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, hq, D, generator=g) * scale
    k = torch.randn(B, T, hk, D, generator=g) * scale
    off = torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5 * scale
    k[:, :(T // S) * S] += off.expand(-1, -1, S, -1, -1).reshape(B, (T // S) * S, hk, D)
    v = torch.randn(B, T, hk, D, generator=g) * scale
    return [t.to(dtype) for t in (q, k, v)]


def _core(hq, hk, K, S, W, **kw):
    from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
    return HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W, **kw))


def _sample_rows(B, T, n, S, seed, avoid_landmarks=False):
    g = torch.Generator().manual_seed(seed)
    b = torch.randint(0, B, (n,), generator=g)
    t = torch.randint(0, T, (n,), generator=g)
    t[: n // 8] = torch.randint(0, min(T, 1024), (n // 8,), generator=g)      # rows with few or no candidates
    t[n // 8: n // 4] = T - 1 - torch.randint(0, min(T, 256), (n // 4 - n // 8,), generator=g)
    if avoid_landmarks:           # a chunk's last token is also its pooling query: its gradient is not row-local
        t = torch.where((t + 1) % S == 0, t - 1, t)
    bt = torch.unique(b * T + t)  # every (sequence, position) once
    return bt // T, bt % T


def _status_clean():
    from hils_attention_b200 import _lib
    assert _lib.load().hils_take_device_status() == 0


def test_config2_full_shape_sampled_rows():
    """B=8, T=8192, 16 heads, D=64, 128 chunks, top-k 32, bf16: forward of the whole chain at the full shape,
    640 sampled rows over all heads against the oracle."""
    B, T, H, D, S, K, W = 8, 8192, 16, 64, 64, 32, 512
    q, k, v = _inputs(B, T, H, H, D, S, 2)
    core = _core(H, H, K, S, W).eval()
    with torch.no_grad():
        o, aux = core(q.cuda(), k.cuda(), v.cuda(), q.cuda(), return_aux=True)
    _status_clean()
    b, t = _sample_rows(B, T, 640, S, 7)
    ref = orc.hils_attention_rows(q, k, v, q, b, t, range(H), chunk_size=S, window_size=W, topk=K)
    ids = aux["indices"].cpu()[b, t]
    same = (ids == ref["indices"]).all(-1)                                          # (R, H)
    assert same.float().mean().item() >= 0.99, same.float().mean().item()
    check(aux["lse_swa"].cpu()[b, t], ref["lse_swa"], BF, "c2 lse_swa")
    check(aux["weights"].cpu()[b, t][same], ref["weights"][same], BF, "c2 inter-chunk weights")
    check(o.cpu()[b, t][same], ref["o"][same], BF, "c2 chain output")


def test_config2_downscaled_forward_and_gradients():
    """B=1, T=2048, 16 heads, D=64, top-k 32, bf16: the whole chain forward AND backward against autograd through
    the full oracle chain with the selection frozen to the kernel's ids."""
    B, T, H, D, S, K, W = 1, 2048, 16, 64, 64, 32, 512
    q, k, v = _inputs(B, T, H, H, D, S, 12)
    core = _core(H, H, K, S, W).train()
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    o, aux = core(qd, kd, vd, qd, return_aux=True)
    do = torch.randn(o.shape, generator=torch.Generator().manual_seed(13)).to(BF)
    o.backward(do.cuda())
    _status_clean()
    ids = aux["indices"].cpu()
    qr, kr, vr = (x.float().requires_grad_(True) for x in (q, k, v))
    with torch.no_grad():
        _, raux = orc.hils_attention_chain(qr, kr, vr, qr, chunk_size=S, window_size=W, topk=K, act_dtype=BF,
                                           return_aux=True)
    own = (ids == raux["indices"]).all(-1)
    assert own.float().mean().item() >= 0.99
    # gradients on identical selections: the oracle re-run with the kernel's ids
    ref2 = orc.hils_attention_chain(qr, kr, vr, qr, chunk_size=S, window_size=W, topk=K, act_dtype=BF,
                                    forced_indices=ids)
    check(o, ref2, BF, "c2s chain output (kernel ids)")
    ref2.float().backward(do.float())
    for name, a, r in (("dq", qd, qr), ("dk", kd, kr), ("dv", vd, vr)):
        check(a.grad, r.grad, BF, "c2s chain " + name)


def test_config3_sampled_rows_forward_and_dq():
    """T=65536, D=128, 1024 chunks, top-k 32, bf16 (4 of the 32 heads: heads are independent): forward at the
    full sequence length and dQ of sampled rows against the oracle with the kernel's ids."""
    B, T, H, D, S, K, W = 1, 65536, 4, 128, 64, 32, 512
    q, k, v = _inputs(B, T, H, H, D, S, 3)
    core = _core(H, H, K, S, W).train()
    qd, kd, vd = (x.cuda().requires_grad_(True) for x in (q, k, v))
    o, aux = core(qd, kd, vd, qd, return_aux=True)
    g = torch.Generator().manual_seed(31)
    b, t = _sample_rows(B, T, 256, S, 8, avoid_landmarks=True)
    do = torch.zeros(o.shape, dtype=BF)
    do_rows = torch.randn(b.numel(), H, D, generator=g).to(BF)
    do[b, t] = do_rows                     # upstream gradient on the sampled rows only: dq of a row is row-local
    o.backward(do.cuda())
    _status_clean()
    ids = aux["indices"].cpu()[b, t]
    ref = orc.hils_attention_rows(q, k, v, q, b, t, range(H), chunk_size=S, window_size=W, topk=K)
    same = (ids == ref["indices"]).all(-1)
    assert same.float().mean().item() >= 0.99, same.float().mean().item()
    check(o.detach().cpu()[b, t][same], ref["o"][same], BF, "c3 chain output")
    # dq: the oracle on the kernel's ids, q of the sampled rows as the leaf
    qf = q.float().requires_grad_(True)
    out = orc.hils_attention_rows(qf, k, v, qf, b, t, range(H), chunk_size=S, window_size=W, topk=K,
                                  act_dtype=BF, forced_indices=ids)
    (out["o"].float() * do_rows.float()).sum().backward()
    check(qd.grad.cpu()[b, t], qf.grad[b, t], BF, "c3 dq of sampled rows")


def test_config4_decode_step_against_128k_store():
    """Decode: 2 sequences x 32 heads, D=128, one new token each against a 131072-token store (2048 pooled chunk
    keys), top-k 32: ids and output of the one-call decode step against the oracle."""
    from hils_attention_b200.cache import HiLSCache
    import hils_attention_b200 as hb
    B, T, H, D, S, K, W = 2, 131072, 32, 128, 64, 32, 512
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(4)
    cap = T + 8
    kbuf = torch.empty((cap, B, H, D), dtype=BF, device=dev)
    vbuf = torch.empty((cap, B, H, D), dtype=BF, device=dev)
    for t0 in range(0, T, 8192):
        off = (torch.randn((8192 // S, 1, B, H, D), generator=g, device=dev) * 0.5).expand(-1, S, -1, -1, -1)
        kbuf[t0:t0 + 8192] = (torch.randn((8192, B, H, D), generator=g, device=dev) + off.reshape(8192, B, H, D)).to(BF)
        vbuf[t0:t0 + 8192] = torch.randn((8192, B, H, D), generator=g, device=dev).to(BF)
    cache = HiLSCache()
    layer = cache.layer(1)
    layer.adopt(kbuf, vbuf, T)
    N = T // S
    with torch.no_grad():
        kf, _ = layer.folded()
        mu = torch.randn((1, N, B * H, D), generator=g, device=dev).to(BF)
        lmk_k, prior_b = hb.chunk_attn_pool(mu, kf[:, :N * S].unflatten(1, (N, S)))       # (1, N, B*H, D)
    cache._hils_prior_cache[0] = {"lmk_k": lmk_k, "prior_b": prior_b}
    core = _core(H, H, K, S, W).eval()
    qn, kn, vn = (torch.randn((B, 1, H, D), generator=g, device=dev).to(BF) for _ in range(3))
    with torch.no_grad():
        o = core(qn, kn, vn, qn, past_key_values=cache, use_cache=True)                     # fused decode step
        cache2 = HiLSCache()                                                                # same step op by op, for its ids
        l2 = cache2.layer(1)
        l2.adopt(kbuf, vbuf, T)
        cache2._hils_prior_cache[0] = {"lmk_k": lmk_k, "prior_b": prior_b}
        o2, aux = core(qn, kn, vn, qn, past_key_values=cache2, use_cache=True, return_aux=True)
    _status_clean()
    check(o, o2, BF, "c4 fused step vs op by op")
    # oracle for 3 kv heads of both sequences, on the store as the kernels saw it (new token appended at row T)
    heads = [0, 13, 31]
    ks = kbuf[:T + 1].permute(1, 0, 2, 3)[:, :, heads].float().cpu()                        # (B, T+1, 3, D)
    vs = vbuf[:T + 1].permute(1, 0, 2, 3)[:, :, heads].float().cpu()
    lk = lmk_k.view(N, B, H, D).permute(1, 0, 2, 3)[:, :, heads].float().cpu()              # (B, N, 3, D)
    pb = prior_b.view(N, B, H).permute(1, 0, 2)[:, :, heads].float().cpu()
    qs = qn[:, :, heads].float().cpu()
    ref = orc.hils_attention_rows(qs, ks, vs, qs, torch.arange(B), torch.zeros(B, dtype=torch.long), range(3),
                                  chunk_size=S, window_size=W, topk=K, lmk_k=lk, prior_b=pb, q_offset=T,
                                  act_dtype=BF)
    ids = aux["indices"].cpu()[:, 0][:, heads]                                              # (B, 3, K)
    assert (ids == ref["indices"]).all(-1).float().mean().item() >= 0.99
    same = (ids == ref["indices"]).all(-1)
    check(o.cpu()[:, 0][:, heads][same], ref["o"][same], BF, "c4 decode output")
    check(o2.cpu()[:, 0][:, heads][same], ref["o"][same], BF, "c4 decode output (op by op)")


def test_config5_selection_at_one_million_tokens():
    """T=1,048,576 (16384 chunks), D=128, top-k 32, two heads: the selection at full length.  Keys are N(0,1) with
    64 planted chunks, each set to 3x the mean query of a later 128-token query block (+ 0.1 noise); the blocks'
    queries share a block offset ~ N(0,1) so that this mean is a direction.  Checks on 32 probe blocks (4096 rows):
    the planted chunk is selected by every row of its block; ids equal the stable selector applied to the kernel's
    own ranking values and agree with the oracle on >= 99 % of the rows; the full-length launch returns the same
    ids as the per-block launches."""
    import hils_attention_b200 as hb
    B, T, H, D, S, K, W = 1, 1 << 20, 2, 128, 64, 32, 512
    N = T // S
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    q = torch.randn((B, T, H, D), generator=g, device=dev)
    k = torch.randn((B, T, H, D), generator=g, device=dev)
    gc = torch.Generator().manual_seed(55)
    nblk = T // 128
    blocks = (torch.randperm(nblk - 64, generator=gc)[:64] + 64).sort().values           # query blocks (not the first few)
    planted, used = [], set()
    for bq in blocks.tolist():                                                           # one distinct earlier chunk each
        while True:
            c = int(torch.randint(0, bq * 2 - 10, (1,), generator=gc))
            if c not in used:
                break
        used.add(c)
        planted.append(c)
    for bq, c in zip(blocks.tolist(), planted):
        q[0, bq * 128:(bq + 1) * 128] += torch.randn((1, H, D), generator=g, device=dev)
        m = q[0, bq * 128:(bq + 1) * 128].mean(0, keepdim=True)                            # (1, H, D)
        k[0, c * S:(c + 1) * S] = 3.0 * m + 0.1 * torch.randn((S, H, D), generator=g, device=dev)
    q, k = q.to(BF), k.to(BF)
    with torch.no_grad():
        _, lse = hb.flex_attn_tl(q, k, k, W, S, training=False)
        lse_act = lse.to(BF)
        lmk_k, prior_b = hb.chunk_attn_pool(q[:, S - 1::S][:, :N], k.unflatten(1, (N, S)))
        idx_full, _ = hb.online_softmax_topk_head(q, lmk_k, lse_act, K, S, W, is_training=False, q_offset=0,
                                                  bias=prior_b)
    _status_clean()
    lk_c, pb_c = lmk_k.float().cpu(), prior_b.float().cpu()
    agree, total = 0, 0
    probe = blocks[torch.linspace(0, blocks.numel() - 1, 32).long()].tolist()
    for bq in probe:
        lo = bq * 128
        aux = {}
        with torch.no_grad():
            idx_b, sc_b = hb.online_softmax_topk_head(q[:, lo:lo + 128], lmk_k, lse_act[:, lo:lo + 128], K, S, W,
                                                      is_training=False, q_offset=lo, bias=prior_b, _aux=aux)
        assert torch.equal(idx_b, idx_full[:, lo:lo + 128]), "full-length and per-block launches disagree"
        keys = aux["rank_keys"].cpu()
        assert torch.equal(idx_b.cpu(), orc.stable_topk_from_keys(keys, K)), "ids are not the stable top-k of the kernel's keys"
        ridx, _, raux = orc.topk_select(q[:, lo:lo + 128].float().cpu().view(B, 128, H, 1, D), lk_c,
                                        lse_act[:, lo:lo + 128].float().cpu(), K, S, W, True, lo, bias=pb_c,
                                        return_aux=True)
        agree += int((idx_b.cpu() == ridx).all(-1).sum())
        total += 128 * H
        c = planted[blocks.tolist().index(bq)]
        assert bool((idx_b == c).any(-1).all()), f"planted chunk {c} missing from block {bq}"
    assert agree / total >= 0.99, agree / total
