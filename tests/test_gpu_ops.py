"""Parity of the CUDA ops (called through the C ABI) with the CPU oracle and with the golden
fixtures produced by the reference's own functions.  Needs a B200."""
import math

import pytest
import torch

from oracle import hils_oracle as orc
from tests.util import check, cuda, golden, rms_ratio

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32


@pytest.fixture(scope="module")
def ops():
    import hils_attention_b200 as pkg
    return pkg


# ------------------------------------------------------------------ pooling
@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("dtype", [BF, F32])
def test_pool_golden(ops, tag, dtype):
    g = golden(f"pool_{tag}.npz")
    mu = cuda(g["mu_q"], dtype).requires_grad_(True)
    kc = cuda(g["k_chunked"], dtype).requires_grad_(True)
    lk, lb = ops.chunk_attn_pool(mu, kc)
    assert lk.dtype == dtype and lb.dtype == F32
    check(lk, g["lmk_k"], dtype, "lmk_k")
    check(lb, g["lmk_b"], F32 if dtype == F32 else BF, "lmk_b")
    (lk.float() * cuda(g["g_lmk_k"])).sum().add((lb * cuda(g["g_lmk_b"])).sum()).backward()
    check(mu.grad, g["d_mu_q"], dtype, "d_mu_q")
    check(kc.grad, g["d_k"], dtype, "d_k")


@pytest.mark.parametrize("shape", [(1, 64, 2, 128, 64), (2, 128, 4, 128, 64), (4, 256, 2, 128, 64),
                                   (1, 32, 2, 64, 64), (1, 16, 1, 128, 32)])
def test_pool_reference_shapes(ops, shape):
    """The forward cases of the reference's pool unit test, with its thresholds
    (ratio 0.005 for k', 0.01 for b')."""
    B, N, H, D, S = shape
    g = torch.Generator().manual_seed(42)
    mu = torch.randn(B, N, H, D, generator=g).to(BF)
    kc = torch.randn(B, N, S, H, D, generator=g).to(BF)
    lk_ref, lb_ref = orc.chunk_attn_pool(mu, kc)
    lk, lb = ops.chunk_attn_pool_tilelang(mu.cuda(), kc.cuda())
    assert rms_ratio(lk, lk_ref) < 0.005
    assert rms_ratio(lb, lb_ref) < 0.01


def test_pool_gqa_in_place_cache_view_and_compact(ops):
    g = torch.Generator().manual_seed(3)
    B, T, h_kv, G, D, S = 2, 200, 2, 4, 64, 64
    N = T // S
    k = torch.randn(B, T, h_kv, D, generator=g).to(BF)
    mu = torch.randn(B, N, h_kv * G, D, generator=g).to(BF)
    kc = k[:, :N * S].reshape(B, N, S, h_kv, D)
    lk_ref, lb_ref = orc.chunk_attn_pool(mu, kc)
    kd = k.cuda()
    view = kd[:, :N * S].view(B, N, S, h_kv, D)            # batch-strided view of the cache
    lk, lb = ops.chunk_attn_pool(mu.cuda(), view)
    check(lk, lk_ref, BF, "gqa lmk_k")
    check(lb, lb_ref, BF, "gqa lmk_b")
    lk0, lb0 = ops.chunk_attn_pool_tilelang(mu.cuda(), view, compact_lmk_k=True)
    assert float(lk0.float().abs().max()) == 0.0
    assert torch.equal(lb0, lb)
    mp = ops.chunk_mean_pool(view)
    check(mp, orc.chunk_mean_pool(kc), BF, "mean pool")


def test_pool_gqa_backward_and_mean_backward(ops):
    g = torch.Generator().manual_seed(4)
    B, N, h_kv, G, D, S = 1, 5, 2, 2, 32, 32
    mu0 = torch.randn(B, N, h_kv * G, D, generator=g)
    kc0 = torch.randn(B, N, S, h_kv, D, generator=g)
    gk = torch.randn(B, N, h_kv * G, D, generator=g)
    gb = torch.randn(B, N, h_kv * G, generator=g)
    mu_r, kc_r = mu0.clone().requires_grad_(True), kc0.clone().requires_grad_(True)
    lk_r, lb_r = orc.chunk_attn_pool(mu_r, kc_r)
    ((lk_r * gk).sum() + (lb_r * gb).sum() + (orc.chunk_mean_pool(kc_r) * gk[:, :, ::G]).sum()).backward()
    mu, kc = mu0.cuda().requires_grad_(True), kc0.cuda().requires_grad_(True)
    lk, lb = ops.chunk_attn_pool(mu, kc)
    ((lk * gk.cuda()).sum() + (lb * gb.cuda()).sum() + (ops.chunk_mean_pool(kc) * gk[:, :, ::G].cuda()).sum()).backward()
    check(mu.grad, mu_r.grad, F32, "gqa d_mu")
    check(kc.grad, kc_r.grad, F32, "gqa d_k")


def test_pool_errors(ops):
    with pytest.raises(ValueError):
        ops.chunk_attn_pool(torch.zeros(1, 2, 3, 8).cuda(), torch.zeros(1, 2, 4, 2, 8).cuda())   # 3 % 2
    with pytest.raises(ValueError):
        ops.chunk_attn_pool(torch.zeros(1, 2, 8).cuda(), torch.zeros(1, 2, 4, 2, 8).cuda())


# ------------------------------------------------------------------ selection
def _select_args(g):
    K, S, W, qo = [int(x) for x in g["args"]]
    return K, S, W, qo


@pytest.mark.parametrize("tag", ["shared", "bias_pq", "decode", "ragged"])
@pytest.mark.parametrize("dtype", [BF, F32])
def test_topk_golden(ops, tag, dtype):
    g = golden(f"topk_{tag}.npz")
    K, S, W, qo = _select_args(g)
    B, L, h_kv, G, D = g["q"].shape
    per_q = g["lmks"].shape[2] == h_kv * G and G > 1
    aux = {}
    idx, sc = ops.online_softmax_topk_head(
        cuda(g["q"], dtype), cuda(g["lmks"], dtype), cuda(g["lse_swa"]), K, S, W, True, qo,
        is_training=(qo == 0), bias=None if "bias" not in g else g["bias"].cuda(),
        gumbel_noise=None if "gumbel" not in g else g["gumbel"].cuda(), G=(G if per_q else 1), _aux=aux)
    assert idx.dtype == torch.int32 and idx.shape == (B, L, h_kv, K)
    # the selector itself is bit-exact on the values it ranked
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(aux["rank_keys"].cpu(), K))
    # and on these small cases it reproduces the reference's ids outright
    assert torch.equal(idx.cpu(), g["indices"].to(torch.int32))
    check(sc.view(B, L, h_kv, G, K), g["scores"], dtype, "scores")
    _, _, oaux = orc.topk_select(g["q"], g["lmks"], g["lse_swa"], K, S, W, True, qo, bias=g.get("bias"),
                                 gumbel_noise=g.get("gumbel"), return_aux=True)
    check(aux["lse_total"], oaux["lse_total"], F32, "lse_total")


@pytest.mark.parametrize("cfg", [(2, 1000, 2, 8, 64, 16, 64, 64), (1, 1024, 4, 1, 128, 32, 64, 512),
                                 (1, 700, 1, 2, 64, 64, 32, 96),
                                 # the reference's own robustness shapes (ops/topk_head_softmax.py:1807-1811)
                                 (2, 4096, 2, 8, 64, 16, 64, 64), (2, 4096, 8, 8, 64, 16, 64, 64)])
def test_topk_selector_exact_and_match_rate(ops, cfg):
    """Larger seeded cases: ids bit-exact against the stable selector fed the kernel's own fp32
    ranking values; ranking values within tolerance of the oracle; >= 99% of the ids equal to the
    oracle's own choice (the reference's acceptance threshold, ops/topk_head_softmax.py:1472)."""
    B, L, h_kv, G, D, K, S, W = cfg
    N = L // S
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, L, h_kv, G, D, generator=g).to(BF)
    lm = torch.randn(B, N, h_kv, D, generator=g).to(BF)
    lse = torch.randn(B, L, h_kv * G, generator=g) + 2
    bias = torch.randn(B, N, h_kv * G, generator=g)
    aux = {}
    idx, sc = ops.online_softmax_topk_head(q.cuda(), lm.cuda(), lse.cuda(), K, S, W, bias=bias.cuda(), _aux=aux)
    keys = aux["rank_keys"].cpu()
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(keys, K))
    ridx, rsc, raux = orc.topk_select(q, lm, lse, K, S, W, True, 0, bias=bias, return_aux=True)
    check(keys, raux["keys"], F32, "rank keys")
    match = (idx.cpu() == ridx).float().mean().item()
    assert match >= 0.99, match
    same = (idx.cpu() == ridx).all(-1)
    check(sc.view(B, L, h_kv, G, K)[same], rsc[same], BF, "scores")


@pytest.mark.parametrize("cfg", [
    # B, L, h_kv, G, D, K, S, W, per_qhead, drop, gumbel
    (1, 4096, 2, 1, 64, 32, 16, 32, False, False, False),      # N = 256: two key tiles, double-buffered
    (1, 3000, 1, 4, 128, 8, 8, 24, True, True, False),         # per-q-head keys, N = 375, ragged tail, drop mask
    (2, 1536, 2, 2, 64, 48, 16, 64, False, True, True),        # K > 32, gumbel noise
    (1, 640, 1, 16, 64, 4, 32, 64, False, False, False),       # 256 score rows per CTA
    (1, 8192, 1, 1, 128, 32, 8, 16, False, False, False),      # N = 1024: 16 tokens per CTA, key-bit rows reuse the key tiles
    (1, 4096, 2, 2, 64, 16, 4, 8, True, True, False),          # N = 1024, per-q-head keys, drop mask
])
def test_topk_tensor_core_scores_path(ops, cfg):
    """bf16 training/prefill selection (scores on the tensor cores, scores resident in shared memory):
    ids bit-exact against the stable selector fed the kernel's own ranking values, ranking values and
    lse_total within tolerance of the oracle, >= 99% of the ids equal to the oracle's."""
    B, L, h_kv, G, D, K, S, W, per_q, use_drop, use_gumbel = cfg
    N = L // S
    g = torch.Generator().manual_seed(23)
    q = torch.randn(B, L, h_kv, G, D, generator=g).to(BF)
    lm = torch.randn(B, N, h_kv * G if per_q else h_kv, D, generator=g).to(BF)
    lse = torch.randn(B, L, h_kv * G, generator=g) + 2
    bias = torch.randn(B, N, h_kv * G, generator=g)
    drop = (torch.rand(B, L, N, generator=g) < 0.2).to(torch.int32) if use_drop else None
    gum = torch.randn(1, 1, h_kv * G, N, generator=g) * 0.1 if use_gumbel else None
    aux = {}
    idx, sc = ops.online_softmax_topk_head(
        q.cuda(), lm.cuda(), lse.cuda(), K, S, W, bias=bias.cuda(), G=(G if per_q else 1),
        drop_mask=None if drop is None else drop.cuda(), gumbel_noise=None if gum is None else gum.cuda(), _aux=aux)
    keys = aux["rank_keys"].cpu()
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(keys, K))
    ridx, rsc, raux = orc.topk_select(q, lm, lse, K, S, W, True, 0, bias=bias, drop_mask=drop, gumbel_noise=gum,
                                      return_aux=True)
    check(keys, raux["keys"], F32, "rank keys")
    check(aux["lse_total"], raux["lse_total"], F32, "lse_total")
    assert (idx.cpu() == ridx).float().mean().item() >= 0.99
    same = (idx.cpu() == ridx).all(-1)
    check(sc.view(B, L, h_kv, G, K)[same], rsc[same], BF, "scores")
    # without the auxiliary outputs the kernel walks only the candidates: same ids
    idx2, _ = ops.online_softmax_topk_head(
        q.cuda(), lm.cuda(), lse.cuda(), K, S, W, bias=bias.cuda(), G=(G if per_q else 1),
        drop_mask=None if drop is None else drop.cuda(), gumbel_noise=None if gum is None else gum.cuda())
    assert torch.equal(idx2, idx)


def test_topk_ties_prefer_lower_id_and_padding(ops):
    """All chunk keys identical -> every candidate ties; the K lowest ids must win.  Rows with
    fewer than K candidates are -1 padded and their scores are -inf."""
    B, L, H, D, S, W, K = 1, 512, 1, 64, 64, 64, 4
    N = L // S
    q = torch.randn(B, L, H, D, generator=torch.Generator().manual_seed(5)).to(BF)
    lm = torch.ones(B, N, H, D).to(BF)
    lse = torch.zeros(B, L, H)
    idx, sc = ops.online_softmax_topk_head(q.cuda(), lm.cuda(), lse.cuda(), K, S, W)
    idx = idx.cpu()
    for l in (0, 63, 127, 128, 200, 320, 511):
        lim = max(0, (l - W + 1) // S)
        want = list(range(min(lim, K))) + [-1] * (K - min(lim, K))
        assert idx[0, l, 0].tolist() == want, (l, idx[0, l, 0].tolist())
    assert torch.isinf(sc.cpu().float()[idx.repeat_interleave(1, 2) < 0]).all()


def test_topk_drop_mask_and_backward(ops):
    g = torch.Generator().manual_seed(6)
    B, L, h_kv, G, D, K, S, W = 1, 384, 2, 2, 32, 4, 32, 64
    N = L // S
    q0 = torch.randn(B, L, h_kv * G, D, generator=g)
    lm0 = torch.randn(B, N, h_kv, D, generator=g)
    lse = torch.randn(B, L, h_kv * G, generator=g)
    drop = (torch.rand(B, L, N, generator=g) < 0.3).to(torch.int32)
    gs = torch.randn(B, L, h_kv * G, K, generator=g)
    q, lm = q0.cuda().requires_grad_(True), lm0.cuda().requires_grad_(True)
    idx, sc = ops.online_softmax_topk_head(q, lm, lse.cuda(), K, S, W, drop_mask=drop.cuda())
    ridx, rsc = orc.topk_select(q0.view(B, L, h_kv, G, D), lm0, lse, K, S, W, True, 0, drop_mask=drop)
    assert torch.equal(idx.cpu(), ridx)
    dropped = torch.gather(drop.unsqueeze(2).expand(-1, -1, h_kv, -1), -1, ridx.clamp_min(0).long())
    assert int((dropped * (ridx >= 0)).sum()) == 0
    valid = (idx >= 0).repeat_interleave(G, dim=2)
    (sc.float().masked_fill(~valid, 0.0) * gs.cuda()).sum().backward()
    # oracle gradient: scores = scale * <q, lmk[id]>
    qr, lr = q0.clone().requires_grad_(True), lm0.clone().requires_grad_(True)
    sel = lr[0][ridx[0].clamp_min(0).long(), torch.arange(h_kv).view(1, h_kv, 1)]          # (L,h_kv,K,D)
    s = torch.einsum("lhgd,lhkd->lhgk", qr[0].view(L, h_kv, G, D), sel) / math.sqrt(D)
    (s.reshape(1, L, h_kv * G, K).masked_fill(~valid.cpu(), 0.0) * gs).sum().backward()
    check(q.grad, qr.grad, F32, "dq")
    check(lm.grad, lr.grad, F32, "dlmk")


# ------------------------------------------------------------------ sparse attention
@pytest.mark.parametrize("tag", ["a", "kvlong"])
@pytest.mark.parametrize("dtype", [F32, BF])
def test_sparse_golden(ops, tag, dtype):
    g = golden(f"sparse_{tag}.npz")
    S = int(g["args"][0])
    q, k, v, w = [cuda(g[n], dtype).requires_grad_(True) for n in ("q", "k", "v", "w")]
    idx = g["indices"].cuda()
    if dtype == F32:
        ref = {n: g[n] for n in ("o", "dq", "dk", "dv", "dw")}
    else:                                   # oracle on the bf16-rounded inputs
        qr, kr, vr, wr = [t.detach().float().cpu().requires_grad_(True) for t in (q, k, v, w)]
        o_r = orc.sparse_attn(qr, kr, vr, wr, g["indices"], chunk_size=S)
        o_r.backward(g["do"].to(BF).float())
        ref = {"o": o_r, "dq": qr.grad, "dk": kr.grad, "dv": vr.grad, "dw": wr.grad}
    o = ops.HiLS_block_M_head(q, k, v, w, idx, block_size=S, mask_last_token=True,
                              dtype="float" if dtype == F32 else "bfloat16")
    check(o, ref["o"], dtype, "o")
    o.backward(cuda(g["do"], dtype))
    for n, t in (("dq", q), ("dk", k), ("dv", v), ("dw", w)):
        check(t.grad, ref[n], dtype, n)
        assert rms_ratio(t.grad, ref[n]) < (5e-3 if dtype == F32 else 2e-2), n


def test_sparse_head_dim_192_long_kv(ops):
    """The reference's own correctness shape (ops/hils_fwd_bwd_head.py:980-994): head dim 192, eight query heads on
    one kv head, 512 query tokens against 612 keys, four chunks per token.  Outside the tensor-core tiles, so the
    generic kernels run; forward and all gradients against the oracle."""
    g = torch.Generator().manual_seed(42)
    B, L, T, H, HQ, D, K, S = 1, 512, 612, 1, 8, 192, 4, 64
    N = T // S
    q0 = torch.randn(B, L, HQ, D, generator=g).to(BF)
    k0 = torch.randn(B, T, H, D, generator=g).to(BF)
    v0 = torch.randn(B, T, H, D, generator=g).to(BF)
    w0 = torch.softmax(torch.randn(B, L, HQ, K, generator=g), -1).to(BF)
    do = torch.randn(B, L, HQ, D, generator=g).to(BF)
    idx = torch.stack([torch.randperm(N, generator=g)[:K].sort().values for _ in range(B * L * H)]).view(B, L, H, K).int()
    q, k, v, w = [t.cuda().requires_grad_(True) for t in (q0, k0, v0, w0)]
    o = ops.HiLS_block_M_head(q, k, v, w, idx.cuda(), block_size=S, mask_last_token=True)
    o.backward(do.cuda())
    qr, kr, vr, wr = [t.float().requires_grad_(True) for t in (q0, k0, v0, w0)]
    ref = orc.sparse_attn(qr, kr, vr, wr, idx, chunk_size=S, mask_last_token=True)
    ref.backward(do.float())
    check(o, ref, BF, "o (D=192)")
    for n, a, b in (("dq", q, qr), ("dk", k, kr), ("dv", v, vr), ("dw", w, wr)):
        check(a.grad, b.grad, BF, n + " (D=192)")


def test_sparse_unsorted_ids_slope_and_eval_mode(ops):
    g = torch.Generator().manual_seed(8)
    B, L, H, HQ, D, K, S = 1, 128, 1, 2, 32, 4, 32
    q = torch.randn(B, L, HQ, D, generator=g)
    k = torch.randn(B, L, H, D, generator=g)
    v = torch.randn(B, L, H, D, generator=g)
    idx = torch.stack([torch.randperm(L // S, generator=g)[:K] for _ in range(L)]).view(B, L, H, K).to(torch.int32)
    idx[:, ::3, :, -1] = -1
    w = torch.rand(B, L, HQ, K + 1, generator=g)
    slope = torch.tensor([0.05, 0.2])
    ref = orc.sparse_attn(q, k, v, w, idx, chunk_size=S, mask_last_token=False, slope=slope)
    o = ops.HiLS_block_M_head(q.cuda(), k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=S,
                              mask_last_token=False, is_training=False, slope=slope.cuda(), dtype="float")
    check(o, ref, F32, "o slope/unsorted")
    qg = q.cuda().requires_grad_(True)
    o2 = ops.HiLS_block_M_head(qg, k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=S, is_training=False)
    with pytest.raises(RuntimeError):
        o2.sum().backward()


# ------------------------------------------------------------------ exact log Z
@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("dtype", [F32, BF])
def test_logz_golden_and_backward(ops, tag, dtype):
    g = golden(f"logz_{tag}.npz")
    S, W = [int(x) for x in g["args"]]
    q = cuda(g["q"], dtype).requires_grad_(True)
    k = cuda(g["k"], dtype).requires_grad_(True)
    lz = ops.exact_chunk_log_z_tl(q, k, chunk_size=S, window_size=W)
    qr, kr = q.detach().float().cpu().requires_grad_(True), k.detach().float().cpu().requires_grad_(True)
    ref = orc.exact_chunk_log_z(qr, kr, chunk_size=S, window_size=W)
    if dtype == F32:
        check(lz, g["log_z"], F32, "log_z vs reference")
    check(lz, ref, F32 if dtype == F32 else BF, "log_z")
    gz = torch.randn(ref.shape, generator=torch.Generator().manual_seed(1))
    fin = torch.isfinite(ref)
    (ref.masked_fill(~fin, 0.0) * gz).sum().backward()
    (lz.masked_fill(~fin.cuda(), 0.0) * gz.cuda()).sum().backward()
    check(q.grad, qr.grad, dtype, "dq")
    check(k.grad, kr.grad, dtype, "dk")


def test_logz_mask_lmk_forward_only(ops):
    g = torch.Generator().manual_seed(9)
    q = torch.randn(1, 200, 4, 32, generator=g)
    k = torch.randn(1, 200, 2, 32, generator=g)
    qg = q.cuda().requires_grad_(True)
    lz = ops.exact_chunk_log_z_tl(qg, k.cuda(), chunk_size=32, window_size=64, mask_lmk=True)
    check(lz, orc.exact_chunk_log_z(q, k, chunk_size=32, window_size=64, mask_lmk=True), F32, "logz lmk")
    with pytest.raises(NotImplementedError):
        lz[torch.isfinite(lz)].sum().backward()


@pytest.mark.parametrize("B,L,hq,hkv,D,W,ml", [
    (2, 1000, 4, 4, 64, 64, False),      # ragged length, one head per kv head, odd chunk count
    (1, 2048, 8, 1, 64, 512, True),      # 8 query heads per kv head, masked landmark column
    (1, 1100, 4, 2, 128, 128, False),    # head dim 128, ragged
    (2, 256, 2, 2, 128, 64, True),
    (1, 100, 2, 1, 64, 64, False),       # no chunk is ever defined: all -inf
])
def test_logz_tensor_core_forward_matches_oracle(ops, B, L, hq, hkv, D, W, ml):
    """bf16 at chunk size 64 runs one 128 x 128 tcgen05 product per pair of chunks; every (row, chunk) entry is
    compared, and the -inf pattern must agree exactly."""
    g = torch.Generator().manual_seed(L + D)
    q = torch.randn(B, L, hq, D, generator=g).to(BF)
    k = torch.randn(B, L, hkv, D, generator=g).to(BF)
    lz = ops.exact_chunk_log_z_tl(q.cuda(), k.cuda(), chunk_size=64, window_size=W, mask_lmk=ml)
    ref = orc.exact_chunk_log_z(q.float(), k.float(), chunk_size=64, window_size=W, mask_lmk=ml)
    assert lz.shape == ref.shape
    assert torch.equal(torch.isfinite(lz).cpu(), torch.isfinite(ref))
    check(lz, ref, BF, "log_z (tensor cores)")
    if ml:       # like the reference, the backward exists without the landmark mask only
        return
    # backward: two tensor-core passes (dQ query-major, dK key-major)
    qg, kg = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    qr, kr = q.float().requires_grad_(True), k.float().requires_grad_(True)
    lz2 = ops.exact_chunk_log_z_tl(qg, kg, chunk_size=64, window_size=W)
    ref2 = orc.exact_chunk_log_z(qr, kr, chunk_size=64, window_size=W)
    fin = torch.isfinite(ref2)
    gz = torch.randn(ref2.shape, generator=g)
    (lz2.masked_fill(~fin.cuda(), 0.0) * gz.cuda()).sum().backward()
    if fin.any():
        (ref2.masked_fill(~fin, 0.0) * gz).sum().backward()
        check(qg.grad, qr.grad, BF, "dq (tensor cores)")
        check(kg.grad, kr.grad, BF, "dk (tensor cores)")
    else:
        assert qg.grad.abs().sum() == 0 and kg.grad.abs().sum() == 0


# ------------------------------------------------------------------ sliding-window branch
SWA_CASES = [
    # B, Lq, Lk, h_q, h_kv, D, W, S, mask_lmk, expand, kv_start
    (1, 256, 256, 2, 1, 32, 64, 32, True, True, 0),
    (2, 333, 333, 4, 2, 64, 128, 64, False, True, 0),
    (1, 130, 130, 2, 2, 32, 48, 65, True, False, 0),
    (1, 70, 70, 1, 1, 64, 512, 64, True, True, 0),
    (1, 1, 300, 2, 1, 32, 64, 32, True, True, 0),       # decode
    (1, 64, 192, 2, 2, 32, 64, 32, True, True, 0),      # chunk prefill
    (1, 2, 100, 2, 1, 32, 64, 32, True, True, 156),     # truncated cache
    # head dims 64 / 128: the tensor-core path in bf16
    (1, 1024, 1024, 2, 2, 64, 512, 64, True, True, 0),
    (2, 777, 777, 8, 1, 64, 128, 64, True, True, 0),    # G = 8, ragged
    (1, 640, 640, 2, 1, 128, 256, 64, True, True, 0),
    (1, 300, 300, 2, 2, 128, 100, 65, True, False, 0),  # chunk 65, no snapping
    (1, 1, 700, 4, 2, 64, 128, 64, True, True, 0),      # decode
    (1, 100, 612, 2, 1, 128, 128, 64, False, True, 0),  # chunk prefill
    (1, 2, 200, 2, 1, 64, 64, 32, True, True, 157),     # truncated cache
]


@pytest.mark.parametrize("case", SWA_CASES)
@pytest.mark.parametrize("dtype", [F32, BF])
def test_swa_forward_backward(ops, case, dtype):
    B, Lq, Lk, hq, hk, D, W, S, ml, ex, ks = case
    g = torch.Generator().manual_seed(13)
    q0 = torch.randn(B, Lq, hq, D, generator=g).to(dtype).float()
    k0 = torch.randn(B, Lk, hk, D, generator=g).to(dtype).float()
    v0 = torch.randn(B, Lk, hk, D, generator=g).to(dtype).float()
    training = (Lq == Lk and ks == 0)
    qr, kr, vr = [t.clone().requires_grad_(True) for t in (q0, k0, v0)]
    o_r, lse_r = orc.swa(qr, kr, vr, W, S, mask_lmk=ml, expand_to_chunk=ex, kv_start=ks)
    q, k, v = [cuda(t, dtype).requires_grad_(training) for t in (q0, k0, v0)]
    o, lse = ops.flex_attn_tl(q, k, v, W, S, training=training, mask_lmk=ml, expand_to_chunk=ex, kv_start=ks)
    assert o.dtype == dtype and lse.dtype == F32
    check(o, o_r, dtype, "swa o")
    check(lse, lse_r, dtype, "swa lse")
    if not training:
        return
    do = torch.randn(o_r.shape, generator=g)
    dl = torch.randn(lse_r.shape, generator=g)
    fin = torch.isfinite(lse_r)
    ((o_r * do).sum() + (lse_r.masked_fill(~fin, 0.0) * dl).sum()).backward()
    ((o.float() * do.cuda()).sum() + (lse.masked_fill(~fin.cuda(), 0.0) * dl.cuda()).sum()).backward()
    for n, t, r in (("dq", q, qr), ("dk", k, kr), ("dv", v, vr)):
        check(t.grad, r.grad, dtype, "swa " + n)
    from hils_attention_b200 import _lib
    assert _lib.load().hils_take_device_status() == 0


def test_swa_errors(ops):
    x = torch.zeros(1, 8, 1, 32).cuda()
    with pytest.raises(ValueError):
        ops.flex_attn_tl(x, x, x, 4, 4, training=True, kv_start=3)
    o, _ = ops.flex_attn_tl(x.requires_grad_(True), x, x, 4, 4, training=False)
    with pytest.raises(RuntimeError):
        o.sum().backward()


# ------------------------------------------------------------------ whole naive block-sparse attention
@pytest.mark.parametrize("tag", ["mha", "gqa", "lmk"])
def test_naive_bsa_identity_on_gpu(ops, tag):
    """flex_attn_tl + exact_chunk_log_z_tl + stable top-k + softmax + HiLS_block_M_head + addcmul
    reproduces the reference's dense naive-BSA output (fp32)."""
    g = golden(f"bsa_{tag}.npz")
    S, W, K, ml = [int(x) for x in g["args"]]
    q, k, v = g["q"].cuda(), g["k"].cuda(), g["v"].cuda()
    B, L, hq, D = q.shape
    G = hq // k.shape[2]
    swa_o, lse = ops.flex_attn_tl(q, k, v, W, S, training=True, mask_lmk=bool(ml), expand_to_chunk=True)
    lz = ops.exact_chunk_log_z_tl(q, k, chunk_size=S, window_size=W, mask_lmk=bool(ml))
    n_chunk = lz.shape[-1]
    lse_h = torch.logsumexp(lz, -1).nan_to_num(nan=float("-inf"))
    keys = (lz - torch.logaddexp(lse, lse_h).unsqueeze(-1)).view(B, L, hq // G, G, n_chunk).max(3).values
    idx = orc.stable_topk_from_keys(keys.nan_to_num(nan=float("-inf")).cpu(), K).cuda()
    idx_hq = idx.repeat_interleave(G, 2)
    sel = torch.gather(lz, -1, idx_hq.clamp_min(0).long()).masked_fill(idx_hq < 0, float("-inf"))
    w = torch.softmax(torch.cat([sel, lse.unsqueeze(-1)], -1), -1)
    o_h = ops.HiLS_block_M_head(q, k, v, w.contiguous(), idx, block_size=S, mask_last_token=bool(ml),
                                is_training=False, dtype="float")
    o = torch.addcmul(o_h, swa_o, w[..., -1:])
    check(o, g["o"], F32, "naive bsa")


@pytest.mark.parametrize("cfg", [
    # B, L, h_kv, G, D, K, per_qhead
    (2, 500, 2, 1, 64, 8, False),
    (1, 384, 2, 4, 64, 4, False),     # shared keys, GQA: gradients of the group add up
    (1, 300, 1, 2, 128, 8, True),     # per-q-head keys
    (1, 1024, 1, 1, 64, 32, False),
    # more than 128 candidates: several key tiles, the software-pipelined kernel
    (1, 16421, 1, 1, 128, 32, False),  # N = 256, ragged last row block
    (1, 12800, 1, 4, 64, 8, False),    # N = 200, shared keys, four rows per token
    (1, 9000, 1, 2, 128, 16, True),    # N = 140, per-q-head keys
])
def test_topk_backward_bf16_tensor_core_path(ops, cfg):
    """bf16 gradients of the returned scores (tensor-core chunk-key gradient, K-sparse gather for
    dq) against autograd through scale * <q, k'[id]> on the same ids."""
    B, L, h_kv, G, D, K, per_q = cfg
    S, W = 64, 64
    N = L // S
    g = torch.Generator().manual_seed(17)
    q0 = torch.randn(B, L, h_kv * G, D, generator=g).to(BF)
    lm0 = torch.randn(B, N, h_kv * G if per_q else h_kv, D, generator=g).to(BF)
    lse = torch.randn(B, L, h_kv * G, generator=g)
    gs = torch.randn(B, L, h_kv * G, K, generator=g).to(BF)
    q, lm = q0.cuda().requires_grad_(True), lm0.cuda().requires_grad_(True)
    idx, sc = ops.online_softmax_topk_head(q, lm, lse.cuda(), K, S, W, G=(G if per_q else 1))
    valid = (idx >= 0).repeat_interleave(G, dim=2)
    (sc.float().masked_fill(~valid, 0.0) * gs.cuda().float()).sum().backward()
    from hils_attention_b200 import _lib
    assert _lib.load().hils_take_device_status() == 0
    ridx = idx.cpu().long().clamp_min(0)
    qr, lr = q0.float().requires_grad_(True), lm0.float().requires_grad_(True)
    lmv = lr.view(B, N, h_kv, G if per_q else 1, D)
    bi = torch.arange(B).view(B, 1, 1, 1)
    hi = torch.arange(h_kv).view(1, 1, h_kv, 1)
    sel = lmv[bi, ridx, hi]                                         # (B,L,h_kv,K,Gk,D)
    qv = qr.view(B, L, h_kv, G, D)
    s = torch.einsum("blhgd,blhkgd->blhgk", qv, sel.expand(-1, -1, -1, -1, G, -1)) / math.sqrt(D)
    (s.reshape(B, L, h_kv * G, K).masked_fill(~valid.cpu(), 0.0) * gs.float()).sum().backward()
    check(q.grad, qr.grad, BF, "dq")
    check(lm.grad, lr.grad, BF, "dlmk")


@pytest.mark.parametrize("cfg", [
    # B, L, N, h_kv, G, D, K, per_qhead, dtype
    (2, 1, 600, 2, 1, 128, 32, False, BF),
    (1, 3, 1000, 2, 4, 64, 16, False, BF),
    (1, 2, 520, 1, 2, 64, 8, True, F32),
])
def test_topk_decode_kernel(ops, cfg):
    """Few query rows against many chunk keys (the decode-specialised selection kernel): ids bit-exact
    on the kernel's own ranking values, ranking values and scores within tolerance of the oracle."""
    B, L, N, h_kv, G, D, K, per_q, dtype = cfg
    S, W = 64, 512
    q_offset = N * S + W + 5 - L                      # every chunk is a remote candidate for the last row
    g = torch.Generator().manual_seed(23)
    q = torch.randn(B, L, h_kv, G, D, generator=g).to(dtype)
    lm = torch.randn(B, N, h_kv * G if per_q else h_kv, D, generator=g).to(dtype)
    lse = torch.randn(B, L, h_kv * G, generator=g) + 2
    bias = torch.randn(B, N, h_kv * G, generator=g)
    aux = {}
    idx, sc = ops.online_softmax_topk_head(q.cuda(), lm.cuda(), lse.cuda(), K, S, W, q_offset=q_offset,
                                           is_training=False, bias=bias.cuda(), G=(G if per_q else 1), _aux=aux)
    keys = aux["rank_keys"].cpu()
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(keys, K))
    ridx, rsc, raux = orc.topk_select(q.float(), lm.float(), lse, K, S, W, True, q_offset, bias=bias, return_aux=True)
    check(keys, raux["keys"], F32, "rank keys")
    check(aux["lse_total"], raux["lse_total"], F32, "lse_total")
    assert (idx.cpu() == ridx).float().mean().item() >= 0.99
    same = (idx.cpu() == ridx).all(-1)
    check(sc.view(B, L, h_kv, G, K)[same], rsc[same], dtype, "scores")


@pytest.mark.parametrize("cfg", [(2, 1, 640, 2, 2, 64, 8), (1, 3, 512, 1, 4, 128, 4)])
def test_sparse_decode_kernel_fp32(ops, cfg):
    """The streaming decode form of the sparse chunk attention (few query rows, long store), fp32."""
    B, L, T, H, G, D, K = cfg
    g = torch.Generator().manual_seed(31)
    S, N = 64, T // 64
    q = torch.randn(B, L, H * G, D, generator=g)
    k = torch.randn(B, T, H, D, generator=g)
    v = torch.randn(B, T, H, D, generator=g)
    idx = torch.stack([torch.randperm(N, generator=g)[:K].sort()[0] for _ in range(B * L * H)]).view(B, L, H, K).to(torch.int32)
    idx[:, :, 0, -2:] = -1
    w = torch.rand(B, L, H * G, K + 1, generator=g)
    ref = orc.sparse_attn(q, k, v, w, idx, chunk_size=S, mask_last_token=True)
    o = ops.HiLS_block_M_head(q.cuda(), k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=S, is_training=False,
                              dtype="float")
    check(o, ref, F32, "sparse decode")


# ------------------------------------------------------------------ inter-chunk softmax, branch combination
@pytest.mark.parametrize("cfg", [
    # B, L, N, h_q, h_idx, K, softmax1, dtype
    (2, 70, 9, 4, 2, 8, False, BF),
    (1, 33, 40, 6, 6, 32, True, BF),
    (1, 20, 80, 2, 1, 64, False, F32),
    (1, 17, 5, 4, 4, 3, True, F32),
])
def test_inter_chunk_softmax(ops, cfg):
    B, L, N, HQ, HI, K, sm1, dtype = cfg
    g = torch.Generator().manual_seed(31)
    sc0 = torch.randn(B, L, HQ, K, generator=g).to(dtype)
    idx = torch.stack([torch.stack([torch.stack([torch.randperm(N, generator=g)[:min(K, N)].sort().values
                                                 if K <= N else torch.arange(K) % N
                                                 for _ in range(HI)]) for _ in range(L)]) for _ in range(B)]).int()
    pad = torch.rand(B, L, HI, generator=g) < 0.3                  # rows with empty slots at the end
    n_pad = torch.randint(1, K, (B, L, HI), generator=g)
    slot = torch.arange(K).view(1, 1, 1, K)
    empty = pad.unsqueeze(-1) & (slot >= (K - n_pad).unsqueeze(-1))
    idx = idx.masked_fill(empty, -1)
    sc0 = sc0.masked_fill(empty.repeat_interleave(HQ // HI, dim=2), float("-inf"))
    lse0 = torch.randn(B, L, HQ, generator=g).to(dtype)
    pb0 = torch.randn(B, N, HQ, generator=g)
    dw = torch.randn(B, L, HQ, K + 1 + int(sm1), generator=g).to(dtype)
    sc, lse, pb = sc0.cuda().requires_grad_(True), lse0.cuda().requires_grad_(True), pb0.cuda().requires_grad_(True)
    w = ops.inter_chunk_softmax(sc, idx.cuda(), lse, pb, sm1)
    assert w.dtype == dtype and w.shape == (B, L, HQ, K + 1 + int(sm1))
    w.backward(dw.cuda())
    scr, lser, pbr = sc0.clone().requires_grad_(True), lse0.clone().requires_grad_(True), pb0.clone().requires_grad_(True)
    wr = orc.inter_chunk_weights(scr, idx, lser, pbr, softmax1=sm1)
    wr.backward(dw)
    check(w, wr, dtype, "weights")
    check(sc.grad, scr.grad, dtype, "d_scores")
    check(lse.grad, lser.grad, dtype, "d_lse")
    check(pb.grad, pbr.grad, dtype, "d_prior_b")
    # without a prior bias
    w2 = ops.inter_chunk_softmax(sc0.cuda(), idx.cuda(), lse0.cuda(), None, sm1)
    check(w2, orc.inter_chunk_weights(sc0, idx, lse0, None, softmax1=sm1), dtype, "weights (no bias)")


@pytest.mark.parametrize("dtype", [BF, F32])
def test_sparse_attn_combine_matches_separate_ops(ops, dtype):
    """The fused op equals HiLS_block_M_head followed by addcmul, forward and backward."""
    g = torch.Generator().manual_seed(32)
    B, L, HQ, H, D, S, K = 1, 256, 4, 2, 64, 32, 4
    N = L // S
    q0, k0, v0, so0 = [torch.randn(B, L, h, D, generator=g).to(dtype) for h in (HQ, H, H, HQ)]
    w0 = torch.softmax(torch.randn(B, L, HQ, K + 2, generator=g), -1).to(dtype)
    idx = torch.stack([torch.stack([torch.stack([torch.randperm(N, generator=g)[:K].sort().values
                                                 for _ in range(H)]) for _ in range(L)]) for _ in range(B)]).int().cuda()
    do = torch.randn(B, L, HQ, D, generator=g).to(dtype).cuda()
    outs = []
    for fused in (True, False):
        q, k, v, w, so = [t.cuda().requires_grad_(True) for t in (q0, k0, v0, w0, so0)]
        if fused:
            o = ops.sparse_attn_combine(q, k, v, w, idx, so, -2, block_size=S)
        else:
            oh = ops.HiLS_block_M_head(q, k, v, w, idx, block_size=S)
            o = torch.addcmul(oh, so, w[..., -2].unsqueeze(-1))
        o.backward(do)
        outs.append([o.detach()] + [t.grad for t in (q, k, v, w, so)])
    for a, b, n in zip(outs[0], outs[1], ("o", "dq", "dk", "dv", "dw", "d_swa_o")):
        check(a, b, dtype, n)


# ------------------------------------------------------------------ per-head RMSNorm + rotary embedding
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_norm_rope_golden(ops, tag):
    g = golden(f"normrope_{tag}.npz")
    dt = BF if int(g["args"][0]) else F32
    cs_dt = F32 if int(g["args"][1]) else BF
    x = cuda(g["x"], dt).requires_grad_(True)
    w = cuda(g["w"], dt).requires_grad_(True)
    cos, sin = cuda(g["cos"], cs_dt), cuda(g["sin"], cs_dt)
    out = ops.rmsnorm_rope(x, w, cos, sin, eps=1e-6)
    assert out.dtype == dt
    check(out, g["out"], dt, "norm+rope")
    out.backward(cuda(g["do"], dt))
    check(x.grad, g["dx"], dt, "dx")
    check(w.grad, g["dw"], dt, "dw")
    check(ops.rmsnorm_rope(x.detach(), w.detach()), g["out_norm_only"], dt, "norm only")
    check(ops.single_tensor_rope_autograd(x.detach(), cos, sin), g["out_rope_only"], dt, "rope only")
    qo, ko = ops.rope_rotary_pos_emb(x.detach(), x.detach()[:, :, :1].contiguous(), cos, sin)
    check(qo, g["out_rope_only"], dt, "rope q")
    check(ko, g["out_rope_only"][:, :, :1], dt, "rope k")
    # rotation is orthogonal: the backward of the rotation alone is its inverse
    xr = x.detach().clone().requires_grad_(True)
    ops.single_tensor_rope_autograd(xr, cos.float(), sin.float()).backward(
        ops.single_tensor_rope_autograd(x.detach(), cos.float(), sin.float()))
    check(xr.grad, x.detach(), dt, "rope^T rope = id")


@pytest.mark.parametrize("cfg", [
    # B, L, N, h, D, K, bias, q_offset
    (1, 1500, 1024, 2, 128, 32, True, 65536 - 1500),     # the 64K-context shape: every chunk a candidate for the last rows
    (2, 700, 700, 1, 64, 8, False, 44100),               # ragged: 700 keys, 700 rows, head dim 64
    (1, 300, 2000, 2, 64, 32, True, 40000),              # rows with few and with ~620 candidates
    (1, 260, 600, 1, 128, 16, True, 0),                  # training offsets: the first rows have no candidate at all
])
def test_topk_long_candidate_lists_one_thread_per_token(ops, cfg):
    """Long candidate lists (N >= 512), one query head per key head: the kernel with one thread per token and tcgen05
    scores.  ids bit-exact on the kernel's own ranking values, those values / lse_total / scores within tolerance of the
    oracle, ids >= 99 % equal to the oracle's."""
    from hils_attention_b200 import _lib
    B, L, N, h, D, K, with_bias, q_offset = cfg
    S, W = 64, 512
    g = torch.Generator().manual_seed(61)
    q = torch.randn(B, L, h, 1, D, generator=g).to(BF)
    lm = (torch.randn(B, N, h, D, generator=g) + 0.5 * torch.randn(B, N, h, 1, generator=g)).to(BF)
    lse = torch.randn(B, L, h, generator=g) + 2
    bias = torch.randn(B, N, h, generator=g) if with_bias else None
    aux = {}
    idx, sc = ops.online_softmax_topk_head(q.cuda(), lm.cuda(), lse.cuda(), K, S, W, q_offset=q_offset, is_training=False,
                                           bias=None if bias is None else bias.cuda(), _aux=aux)
    assert _lib.load().hils_take_device_status() == 0
    keys = aux["rank_keys"].cpu()
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(keys, K))
    ridx, rsc, raux = orc.topk_select(q.float(), lm.float(), lse, K, S, W, True, q_offset, bias=bias, return_aux=True)
    check(keys, raux["keys"], F32, "rank keys", scale=10.0)   # x10: the keys are differences of values ~10 with the row's lse
    check(aux["lse_total"], raux["lse_total"], F32, "lse_total", scale=10.0)
    same = (idx.cpu() == ridx).all(-1)
    assert same.float().mean().item() >= 0.99
    check(sc.view(B, L, h, 1, K)[same], rsc[same], BF, "scores")
    # the production call (no diagnostics) emits through a cheap bound and evaluates only the candidates it lets
    # through exactly: ids and scores must be bit-identical to the diagnostic run, which evaluates every candidate
    idx2, sc2 = ops.online_softmax_topk_head(q.cuda(), lm.cuda(), lse.cuda(), K, S, W, q_offset=q_offset, is_training=False,
                                             bias=None if bias is None else bias.cuda())
    assert _lib.load().hils_take_device_status() == 0
    assert torch.equal(idx2, idx) and torch.equal(sc2, sc)


@pytest.mark.parametrize("L", [999, 1023, 1100])
def test_topk_ragged_lengths_and_wide_chunk_keys(ops, L):
    """Sequence lengths that are no multiple of anything (ops/topk_head_softmax.py:2431-2479) and chunk keys whose last
    dimension is 2*D, which the wrapper folds into twice as many heads (:1296-1300, test_gqa_d_reshape_correctness)."""
    B, h_kv, G, D, K, S, W = 2, 2, 2, 64, 16, 64, 64
    N = L // S
    g = torch.Generator().manual_seed(L)
    q = torch.randn(B, L, h_kv * G, D, generator=g).to(BF)
    lm_wide = torch.randn(B, N, h_kv, 2 * D, generator=g).to(BF)          # (B,N,h_kv,2D) == (B,N,h_kv*2,D): one key per q head
    lse = torch.randn(B, L, h_kv * G, generator=g) + 2
    aux = {}
    idx, sc = ops.online_softmax_topk_head(q.cuda(), lm_wide.cuda(), lse.cuda(), K, S, W, G=G, _aux=aux)
    idx2, sc2 = ops.online_softmax_topk_head(q.cuda(), lm_wide.view(B, N, h_kv * 2, D).cuda(), lse.cuda(), K, S, W, G=G)
    assert torch.equal(idx, idx2) and torch.equal(sc, sc2)
    assert idx.shape == (B, L, h_kv, K) and sc.shape == (B, L, h_kv * G, K)
    assert torch.equal(idx.cpu(), orc.stable_topk_from_keys(aux["rank_keys"].cpu(), K))
    ridx, rsc = orc.topk_select(q.float().view(B, L, h_kv, G, D), lm_wide.float().view(B, N, h_kv * G, D), lse, K, S, W)
    same = (idx.cpu() == ridx).all(-1)
    assert same.float().mean().item() >= 0.99
    check(sc.view(B, L, h_kv, G, K)[same], rsc[same], BF, "scores")
