"""CPU oracle for the HiLS sparse-attention hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 PyTorch on the CPU, the algorithm of every
stage of the reference's HiLS attention path.  It is the checker the CUDA
library is compared against; nothing in the shipped package imports it.  Only
the tests, the smoke check and the benchmark's CPU-baseline leg may call it.

Parity status: PINNED.  Every function below is checked in
``tests/test_oracle_golden.py`` against fixtures under ``tests/golden/`` that
were produced by running the reference's own PyTorch functions
(``tests/golden/make_golden.py`` imports them from the reference checkout):

  pool            ops/chunk_attn_pool_tilelang.py:693-717   (chunk_attn_pool_ref)
  selection       ops/topk_head_softmax.py:15-154           (ref_softmax_topk_max_pooling)
  sparse attn     ops/hils_fwd_bwd_head.py:21-93            (hils_torch_ref)
  exact log Z     models/NaiveBSA/naive_bsa_kernel.py:39-118 (exact_chunk_log_z)
  whole naive-BSA models/NaiveBSA/naive_bsa_ref.py:50-187   (naive_bsa_attention)
  norm + rotary   models/FlashHiLS/modeling_olmo_hils.py:105-111 (rms_norm, executed from its source
                  text) and ops/rope_tilelang_fp32.py:185-189, :244-247 (rotate_half_torch and the
                  torch formula of that file's own correctness test)
  SWA mask        ops/flex_attn_tilelang.py:1366-1376       (mask_mod of the torch reference;
                  that reference itself needs a CUDA device, so the SWA restatement is pinned
                  through the naive-BSA identity and through naive_bsa_ref's local branch)

All tensors use the reference's layouts: q (B, L, h_q, D); k, v (B, T, h_kv, D);
chunk keys (B, N, h, D); indices (B, L, h_kv, K) int32, ascending, -1 padded.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

NEG_INF = float("-inf")


# --------------------------------------------------------------------------
# chunk pooling  (ops/chunk_attn_pool_tilelang.py:693-717,
#                 models/FlashHiLS/hils_attention.py:20-53 for the GQA form)
# --------------------------------------------------------------------------
def chunk_attn_pool(mu_q: torch.Tensor, k_chunked: torch.Tensor,
                    sm_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """mu_q (B,N,h_q,D), k_chunked (B,N,S,h_kv,D) -> k' (B,N,h_q,D) in K's dtype, b' (B,N,h_q) fp32.

    l_j = scale*<mu, K_j>, the chunk's last token masked; p = softmax(l);
    k' = sum_j p_j K_j; b' = -sum_j p_j log p_j.
    """
    B, N, h_q, D = mu_q.shape
    h_kv = k_chunked.shape[3]
    G = h_q // h_kv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    mu = mu_q.float()
    kf = k_chunked.float()
    if G != 1:
        kf = kf.repeat_interleave(G, dim=3)
    logits = torch.einsum("bnhd,bnshd->bnsh", mu, kf) * sm_scale
    S = logits.shape[2]
    logits[:, :, S - 1, :] = NEG_INF
    p = F.softmax(logits, dim=2)
    lmk_k = torch.einsum("bnsh,bnshd->bnhd", p, kf)
    log_p = F.log_softmax(logits, dim=2)
    log_p = torch.where(torch.isfinite(log_p), log_p, torch.zeros_like(log_p))
    lmk_b = -(p * log_p).sum(dim=2)
    return lmk_k.to(k_chunked.dtype), lmk_b


def chunk_mean_pool(k_chunked: torch.Tensor) -> torch.Tensor:
    """k' = mean over the chunk's tokens (models/FlashHiLS/hils_attention.py:445-446)."""
    return k_chunked.float().mean(dim=2).to(k_chunked.dtype)


# --------------------------------------------------------------------------
# chunk selection  (ops/topk_head_softmax.py:15-154; tie rule of the kernel :589-624)
# --------------------------------------------------------------------------
def remote_chunk_limit(t_global: torch.Tensor, window_size: int, block_size: int) -> torch.Tensor:
    """First chunk id that is NOT a candidate for the query at absolute position t."""
    if window_size > 0:
        return torch.div(t_global - window_size + 1, block_size, rounding_mode="floor")
    return torch.div(t_global, block_size, rounding_mode="floor")


def stable_topk_from_keys(keys: torch.Tensor, topk: int) -> torch.Tensor:
    """Pure selector.  keys (..., N) fp32 ranking values (-inf = not a candidate).

    Returns ids (..., topk) int32: the `topk` largest keys, ties broken towards the
    smaller chunk id, -inf never selected, ids ascending and -1 padded at the end.
    This is the rule of the reference's select kernel: scan ids upward, insert only
    on strictly-greater (ops/topk_head_softmax.py:612-624), then sort ids (:926-964).
    """
    N = keys.shape[-1]
    k_eff = min(topk, N)
    order = torch.sort(keys, dim=-1, descending=True, stable=True).indices[..., :k_eff]
    picked = torch.gather(keys, -1, order)
    ids = torch.where(picked == NEG_INF, torch.full_like(order, N + 1000), order)
    if k_eff < topk:
        pad = torch.full(ids.shape[:-1] + (topk - k_eff,), N + 1000, dtype=ids.dtype)
        ids = torch.cat([ids, pad], dim=-1)
    ids = torch.sort(ids, dim=-1).values
    ids = torch.where(ids >= N, torch.full_like(ids, -1), ids)
    return ids.to(torch.int32)


def topk_select(q: torch.Tensor, lmks: torch.Tensor, lse_swa: torch.Tensor, topk: int,
                block_size: int, window_size: int, is_causal: bool = True, q_offset: int = 0,
                drop_mask: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
                bias: Optional[torch.Tensor] = None, gumbel_noise: Optional[torch.Tensor] = None,
                return_aux: bool = False, forced_indices: Optional[torch.Tensor] = None):
    """q (B,L,h_kv,G,D); lmks (B,N,h_kv,D) shared or (B,N,h_kv*G,D) per q-head;
    lse_swa (B,L,h_q) or (B,L,h_kv,G); bias (B,N,h_q) or (B,N,h_kv,G) fp32.
    forced_indices (B,L,h_kv,K): skip the ranking and return the scores of these ids (used to
    compare gradients on identical selections).

    Returns indices (B,L,h_kv,K) int32 and scores (B,L,h_kv,G,K) = scale*q.k' (fp32,
    -inf at -1).  With return_aux also the selection logits, lse_total and ranking keys.
    """
    B, L, h_kv, G, D = q.shape
    N = lmks.shape[1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    qf = q.float()
    if lmks.shape[2] == h_kv * G and G > 1:
        raw = torch.einsum("blhgd,bshgd->blhgs", qf, lmks.float().view(B, N, h_kv, G, D))
    elif lmks.shape[2] == h_kv:
        raw = torch.einsum("blhgd,bshd->blhgs", qf, lmks.float())
    else:
        raise AssertionError("lmks head count must be h_kv or h_kv*G")
    scaled = raw * sm_scale                               # returned scores come from here
    logits = scaled.clone()
    if is_causal:
        t = torch.arange(L).view(L, 1) + q_offset
        lim = remote_chunk_limit(t, window_size, block_size)
        masked = torch.arange(N).view(1, N) >= lim
        logits = logits.masked_fill(masked.view(1, L, 1, 1, N), NEG_INF)
    if bias is not None:
        bv = bias.float().reshape(B, N, h_kv, G).permute(0, 2, 3, 1).unsqueeze(1)
        logits = logits + bv
    if gumbel_noise is not None:
        logits = logits + gumbel_noise.float().view(1, 1, h_kv, G, N)
    lse_hils = torch.logsumexp(logits, dim=-1)
    lse_total = torch.logaddexp(lse_swa.float().reshape(B, L, h_kv, G), lse_hils)
    keys = (logits - lse_total.unsqueeze(-1)).max(dim=3).values       # (B,L,h_kv,N)
    keys = torch.where(torch.isnan(keys), torch.full_like(keys, NEG_INF), keys)
    if drop_mask is not None:
        keys = keys.masked_fill(drop_mask.bool().unsqueeze(2), NEG_INF)
    indices = stable_topk_from_keys(keys, topk) if forced_indices is None else forced_indices.to(torch.int32)
    safe = indices.clamp_min(0).long().unsqueeze(3).expand(-1, -1, -1, G, -1)
    scores = torch.gather(scaled, -1, safe)
    scores = scores.masked_fill((indices < 0).unsqueeze(3).expand_as(scores), NEG_INF)
    if return_aux:
        return indices, scores, {"logits": logits, "lse_hils": lse_hils,
                                 "lse_total": lse_total, "keys": keys}
    return indices, scores


# --------------------------------------------------------------------------
# inter-chunk softmax (module glue, models/FlashHiLS/hils_attention.py:585-610)
# --------------------------------------------------------------------------
def inter_chunk_weights(scores: torch.Tensor, indices: torch.Tensor, lse_swa: torch.Tensor,
                        prior_b: Optional[torch.Tensor] = None, softmax1: bool = False,
                        out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """scores (B,L,h_q,K) in the activation dtype, indices (B,L,h_kv,K), lse_swa (B,L,h_q)
    in the activation dtype, prior_b (B,N,h_q) fp32 -> weights (B,L,h_q,K+1[+1])."""
    B, L, h_q, K = scores.shape
    dt = out_dtype or scores.dtype
    s = scores
    if prior_b is not None:
        g = h_q // indices.shape[2]
        idx = indices.repeat_interleave(g, dim=2).clamp_min(0).long()
        src = prior_b.unsqueeze(-1).expand(-1, -1, -1, K)
        s = s + torch.gather(src, 1, idx).to(s.dtype)
    cols = [s, lse_swa.to(s.dtype).unsqueeze(-1)]
    if softmax1:
        cols.append(torch.zeros(B, L, h_q, 1, dtype=s.dtype))
    return F.softmax(torch.cat(cols, dim=-1), dim=-1).to(dt)


# --------------------------------------------------------------------------
# per-head RMSNorm followed by rotary embedding (upstream of the path)
#   rms_norm: models/FlashHiLS/modeling_olmo_hils.py:105-111 (fp32 statistics, the normalised
#   tensor rounded to the input dtype, then multiplied by the weight in that dtype)
#   rotary:   ops/rope_tilelang_fp32.py:120-134 = x*cos + rotate_half(x)*sin in fp32, rounded once
# --------------------------------------------------------------------------
def rmsnorm_rope(x: torch.Tensor, weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                 cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x (B,L,H,D); weight (D,) or None (no norm); cos, sin (L,D), (1,L,D) or (B,L,D) or None (no
    rotation).  Output in x's dtype."""
    dt = x.dtype
    y = x
    if weight is not None:
        xf = x.float()
        var = xf.pow(2).mean(-1, keepdim=True)
        y = weight.to(dt) * (xf * torch.rsqrt(var + eps)).to(dt)
    if cos is not None:
        c, s_ = cos.float(), sin.float()
        if c.dim() == 2:
            c, s_ = c.unsqueeze(0), s_.unsqueeze(0)
        c, s_ = c.unsqueeze(2), s_.unsqueeze(2)                      # (Bc, L, 1, D)
        yf = y.float()
        half = yf.shape[-1] // 2
        rot = torch.cat((-yf[..., half:], yf[..., :half]), dim=-1)
        y = (yf * c + rot * s_).to(dt)
    return y


# --------------------------------------------------------------------------
# sparse chunk attention  (ops/hils_fwd_bwd_head.py:21-93 with block_q=1)
# --------------------------------------------------------------------------
def sparse_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, weights: torch.Tensor,
                indices: torch.Tensor, *, chunk_size: int, sm_scale: Optional[float] = None,
                mask_last_token: bool = True, slope: Optional[torch.Tensor] = None) -> torch.Tensor:
    """o_i = sum_k w_{i,k} softmax_{j in chunk c_k}(scale q_i.K_j [- slope*max(0,S-2-j)]) V_j.

    Each selected chunk has its own softmax; slots with id -1 contribute nothing.
    Differentiable wrt q, k, v, weights (fp32 math).  Memory O(B*L*h_q*S) per slot.
    """
    B, L, HQ, D = q.shape
    H = k.shape[2]
    Dv = v.shape[-1]
    G = HQ // H
    S = chunk_size
    K = indices.shape[-1]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    N = k.shape[1] // S
    kc = k[:, :N * S].float().reshape(B, N, S, H, D)
    vc = v[:, :N * S].float().reshape(B, N, S, H, Dv)
    qf = q.float().reshape(B, L, H, G, D)
    wf = weights.float()[..., :K].reshape(B, L, H, G, K)
    o = torch.zeros(B, L, H, G, Dv, dtype=torch.float32)
    bidx = torch.arange(B).view(B, 1, 1)
    hidx = torch.arange(H).view(1, 1, H)
    dist = ((S - 2) - torch.arange(S, dtype=torch.float32)).clamp(min=0)

    def slot(kk, qf, kc, vc, wf):
        ids = indices[..., kk].long()                          # (B,L,H)
        valid = ids >= 0
        safe = ids.clamp_min(0)
        ksel = kc[bidx, safe, :, hidx]                         # (B,L,H,S,D)
        vsel = vc[bidx, safe, :, hidx]
        s = torch.einsum("blhgd,blhsd->blhgs", qf, ksel)
        if slope is not None:
            s = s - slope.float().view(1, 1, H, G, 1) * dist.view(1, 1, 1, 1, S)
        s = s * float(sm_scale)
        if mask_last_token:
            s = torch.cat([s[..., :-1], torch.full_like(s[..., -1:], NEG_INF)], dim=-1)
        p = torch.softmax(s, dim=-1)
        ok = torch.einsum("blhgs,blhsd->blhgd", p, vsel)
        wk = wf[..., kk] * valid.unsqueeze(-1).float()
        return ok * wk.unsqueeze(-1)

    # with gradients on, a slot's gathered K/V tiles (B*L*H*S*D each) would be kept for all K slots; beyond
    # ~2 GB the slots are recomputed in the backward pass instead
    recompute = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, weights)) and \
        2 * B * L * H * S * max(D, Dv) * 4 * K > (2 << 30)
    for kk in range(K):
        if recompute:
            from torch.utils.checkpoint import checkpoint
            o = o + checkpoint(slot, kk, qf, kc, vc, wf, use_reentrant=False)
        else:
            o = o + slot(kk, qf, kc, vc, wf)
    return o.reshape(B, L, HQ, Dv)


# --------------------------------------------------------------------------
# exact per-chunk log Z  (models/NaiveBSA/naive_bsa_kernel.py:39-118,
#                         ops/exact_chunk_log_z_tilelang.py:89-112 for mask_lmk)
# --------------------------------------------------------------------------
def exact_chunk_log_z(q: torch.Tensor, k: torch.Tensor, *, chunk_size: int, window_size: int,
                      sm_scale: Optional[float] = None, mask_lmk: bool = False) -> torch.Tensor:
    """log Z[b,i,h,c] = logsumexp_{j in chunk c, j<=i} scale*<q_i,k_j>, defined only for
    i >= (c+1)*S + W - 1 (chunk strictly left of the snapped window); else -inf.
    Returns (B, L, h_q, ceil(L/S)) fp32."""
    B, L, h_q, D = q.shape
    h_kv = k.shape[2]
    G = h_q // h_kv
    S, W = chunk_size, window_size
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    n_chunk = (L + S - 1) // S
    qf = q.float()
    kf = k.float().repeat_interleave(G, dim=2) if G > 1 else k.float()
    s = torch.einsum("bihd,bjhd->bihj", qf, kf) * sm_scale      # (B,L,h,L)
    pos = torch.arange(L)
    masked = pos.view(1, L) > pos.view(L, 1)
    if mask_lmk:
        masked = masked | ((pos + 1) % S == 0).view(1, L)
    s = s.masked_fill(masked.view(1, L, 1, L), NEG_INF)
    pad = n_chunk * S - L
    if pad:
        s = F.pad(s, (0, pad), value=NEG_INF)
    lz = torch.logsumexp(s.view(B, L, h_q, n_chunk, S), dim=-1)
    lz = torch.where(torch.isnan(lz), torch.full_like(lz, NEG_INF), lz)
    c = torch.arange(n_chunk)
    remote = pos.view(L, 1) >= ((c.view(1, n_chunk) + 1) * S + W - 1)
    return lz.masked_fill(~remote.view(1, L, 1, n_chunk), NEG_INF).contiguous()


# --------------------------------------------------------------------------
# sliding-window branch  (mask: ops/flex_attn_tilelang.py:1366-1376; positions :115-133)
# --------------------------------------------------------------------------
def swa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window_size: int, chunk_size: int,
        mask_lmk: bool = True, expand_to_chunk: bool = True, sm_scale: Optional[float] = None,
        kv_start: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense restatement.  Query i sits at absolute position t = kv_start + (Lk-Lq) + i and
    sees keys at absolute j with start <= j <= t, start = floor((t-W+1)/S)*S when
    expand_to_chunk else t-W+1, minus landmark columns (j+1)%S==0 when mask_lmk.
    Returns o (B,Lq,h_q,Dv) fp32 and natural-log lse (B,Lq,h_q); fully masked rows give 0/-inf."""
    B, Lq, h_q, D = q.shape
    Lk, h_kv = k.shape[1], k.shape[2]
    G = h_q // h_kv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    kf = k.float().repeat_interleave(G, dim=2) if G > 1 else k.float()
    vf = v.float().repeat_interleave(G, dim=2) if G > 1 else v.float()
    s = torch.einsum("bihd,bjhd->bhij", q.float(), kf) * sm_scale
    t = kv_start + (Lk - Lq) + torch.arange(Lq).view(Lq, 1)
    j = kv_start + torch.arange(Lk).view(1, Lk)
    start = t - window_size + 1
    if expand_to_chunk:
        start = torch.div(start, chunk_size, rounding_mode="floor") * chunk_size
    keep = (j >= start) & (j <= t)
    if mask_lmk:
        keep = keep & ((j + 1) % chunk_size != 0)
    s = s.masked_fill(~keep.view(1, 1, Lq, Lk), NEG_INF)
    lse = torch.logsumexp(s, dim=-1)
    lse = torch.where(torch.isnan(lse), torch.full_like(lse, NEG_INF), lse)
    p = torch.exp(s - torch.where(lse == NEG_INF, torch.zeros_like(lse), lse).unsqueeze(-1))
    o = torch.einsum("bhij,bjhd->bihd", p, vf)
    return o, lse.permute(0, 2, 1).contiguous()


# --------------------------------------------------------------------------
# the attention chain of the module (models/FlashHiLS/hils_attention.py:536-623)
# --------------------------------------------------------------------------
def hils_attention_chain(q, k, v, lmk_q, *, chunk_size: int, window_size: int, topk: int,
                         pooling: str = "attn", use_prior_bias: bool = True, softmax1: bool = False,
                         q_offset: Optional[int] = None, act_dtype: Optional[torch.dtype] = None,
                         return_aux: bool = False, forced_indices: Optional[torch.Tensor] = None,
                         mu_q: Optional[torch.Tensor] = None):
    """SWA -> chunk keys -> selection -> inter-chunk softmax -> sparse attention -> combine.

    mu_q (B,N,h_q,D): pooling queries that replace the landmark tokens' own queries (the module's shared prior
    query, models/FlashHiLS/hils_attention.py:425-432).

    q, lmk_q (B,L,h_q,D); k, v (B,T,h_kv,D) with T >= L (T > L = cached prefix).
    pooling: "attn" (k', b' from chunk_attn_pool with mu = lmk_q at each chunk's last token;
    needs T == L), "mean" (k' = chunk mean, b' from the attention pool if use_prior_bias),
    Roundings to the activation dtype follow the module: lse_swa (:547), scores
    (ops/topk_head_softmax.py:1038), weights (:610).
    """
    B, L, h_q, D = q.shape
    T, h_kv = k.shape[1], k.shape[2]
    S = chunk_size
    dt = act_dtype or q.dtype
    if q_offset is None:
        q_offset = T - L
    swa_o, lse = swa(q, k, v, window_size, S, mask_lmk=True, expand_to_chunk=True)
    swa_o = swa_o.to(dt)
    lse_act = lse.to(dt)
    N = T // S
    if N == 0:
        return swa_o
    k_chunked = k[:, :N * S].reshape(B, N, S, h_kv, D)
    prior_b = None
    if pooling == "attn" or use_prior_bias:
        assert T == L, "attention pooling in the oracle chain needs the full sequence"
        mu = lmk_q[:, S - 1::S][:, :N] if mu_q is None else mu_q
        kq = k_chunked.repeat_interleave(mu.shape[2] // h_kv, dim=3)
        lmk_k, prior_b = chunk_attn_pool(mu, kq)
        if not use_prior_bias:
            prior_b = None
    if pooling == "mean":
        lmk_k = chunk_mean_pool(k_chunked)
    g_lmk = lmk_k.shape[2] // h_kv
    G = h_q // h_kv
    idx, sc = topk_select(lmk_q.reshape(B, L, h_kv, G, D), lmk_k, lse_act, topk, S, window_size,
                          True, q_offset, bias=prior_b, forced_indices=forced_indices)
    scores = sc.reshape(B, L, h_q, -1).to(dt)
    w = inter_chunk_weights(scores, idx, lse_act, prior_b, softmax1, dt)
    o_hils = sparse_attn(q, k, v, w, idx, chunk_size=S, mask_last_token=True).to(dt)
    w_swa = w[..., -2 if softmax1 else -1]
    o = torch.addcmul(o_hils, swa_o, w_swa.unsqueeze(-1))
    if return_aux:
        return o, {"indices": idx, "scores": scores, "weights": w, "lse_swa": lse, "swa_o": swa_o,
                   "lmk_k": lmk_k, "prior_b": prior_b, "o_hils": o_hils, "g_lmk": g_lmk}
    return o


# --------------------------------------------------------------------------
# naive block-sparse attention in factorised form (models/NaiveBSA/naive_bsa_kernel.py:176-262)
# --------------------------------------------------------------------------
def naive_bsa_chain(q, k, v, *, chunk_size: int, window_size: int, topk: int,
                    sm_scale: Optional[float] = None, mask_last_token: bool = False):
    """SWA + exact log Z + stable top-k + softmax([logZ_sel, lse_swa]) + sparse attention.
    Equals dense attention restricted to window + selected chunks
    (models/NaiveBSA/naive_bsa_ref.py:50-187) when the chunk mass is exact."""
    B, L, h_q, D = q.shape
    h_kv = k.shape[2]
    G = h_q // h_kv
    S = chunk_size
    swa_o, lse_swa = swa(q, k, v, window_size, S, mask_lmk=mask_last_token,
                         expand_to_chunk=True, sm_scale=sm_scale)
    if L < S or topk <= 0:
        return swa_o
    log_z = exact_chunk_log_z(q, k, chunk_size=S, window_size=window_size, sm_scale=sm_scale,
                              mask_lmk=mask_last_token)
    n_chunk = log_z.shape[-1]
    lse_hils = torch.logsumexp(log_z, dim=-1)
    lse_hils = torch.where(torch.isnan(lse_hils), torch.full_like(lse_hils, NEG_INF), lse_hils)
    lse_total = torch.logaddexp(lse_swa, lse_hils)
    keys = (log_z - lse_total.unsqueeze(-1)).view(B, L, h_kv, G, n_chunk).max(dim=3).values
    keys = torch.where(torch.isnan(keys), torch.full_like(keys, NEG_INF), keys)
    idx = stable_topk_from_keys(keys, topk)
    idx_hq = idx.repeat_interleave(G, dim=2).clamp_min(0).long()
    sel = torch.gather(log_z, -1, idx_hq)
    sel = sel.masked_fill(idx.repeat_interleave(G, dim=2) < 0, NEG_INF)
    w = F.softmax(torch.cat([sel, lse_swa.unsqueeze(-1)], dim=-1), dim=-1)
    o_hils = sparse_attn(q, k, v, w[..., :topk].contiguous(), idx, chunk_size=S, sm_scale=sm_scale,
                         mask_last_token=mask_last_token)
    return o_hils + swa_o * w[..., -1:]


# --------------------------------------------------------------------------
# the same chain for a SAMPLE of query rows (cost O(rows * (W + N + K*S)) per head)
# --------------------------------------------------------------------------
def pooled_keys_for_heads(k: torch.Tensor, lmk_q: torch.Tensor, kv_heads, G: int, chunk_size: int,
                          chunk_batch: int = 256):
    """chunk_attn_pool over all full chunks for the listed kv heads only, in batches of chunks.
    k (B,T,h_kv,D), lmk_q (B,T,h_q,D) (its rows at each chunk's last token are the prior queries).
    Returns lmk_k (B,N,len(kv_heads)*G,D) in k's dtype and prior_b (B,N,len(kv_heads)*G) fp32."""
    S = chunk_size
    B, T, _, D = k.shape
    N = T // S
    hk = torch.as_tensor(list(kv_heads))
    hq = (hk.view(-1, 1) * G + torch.arange(G).view(1, -1)).reshape(-1)
    outs_k, outs_b = [], []
    for c0 in range(0, N, chunk_batch):
        c1 = min(N, c0 + chunk_batch)
        kc = k[:, c0 * S:c1 * S][:, :, hk].reshape(B, c1 - c0, S, len(hk), D)
        mu = lmk_q[:, S - 1::S][:, c0:c1][:, :, hq]
        a, b = chunk_attn_pool(mu, kc.repeat_interleave(G, dim=3) if G > 1 else kc)
        outs_k.append(a)
        outs_b.append(b)
    return torch.cat(outs_k, 1), torch.cat(outs_b, 1)


def hils_attention_rows(q, k, v, lmk_q, b_idx, t_idx, kv_heads, *, chunk_size: int, window_size: int,
                        topk: int, lmk_k: Optional[torch.Tensor] = None, prior_b: Optional[torch.Tensor] = None,
                        softmax1: bool = False, q_offset: int = 0, act_dtype: Optional[torch.dtype] = None,
                        forced_indices: Optional[torch.Tensor] = None):
    """The chain of `hils_attention_chain` evaluated only for the query rows (b_idx[r], t_idx[r]) and the
    kv heads `kv_heads` (all query heads of those groups).  q, lmk_q (B,L,h_q,D); k, v (B,T,h_kv,D), query
    row t sits at absolute position q_offset + t.  lmk_k (B,N,len(kv_heads)*G,D) / prior_b may be passed
    (decode against a store with cached pooled keys); otherwise they are attention-pooled from k with the
    prior queries lmk_q[:, S-1::S] (needs T == L).  forced_indices (R,len(kv_heads),K) skips the ranking.
    Differentiable with respect to q and lmk_q (rows' own gradient) with the pooled keys held constant.

    Returns dict: o (R,Hs*G,Dv) in the activation dtype, indices (R,Hs,K) int32, scores, weights,
    lse_swa (R,Hs*G) fp32, swa_o, o_hils.
    """
    S, W = chunk_size, window_size
    B, L, h_q, D = q.shape
    T, h_kv = k.shape[1], k.shape[2]
    G = h_q // h_kv
    dt = act_dtype or q.dtype
    hk = torch.as_tensor(list(kv_heads))
    Hs = len(hk)
    hq = (hk.view(-1, 1) * G + torch.arange(G).view(1, -1)).reshape(-1)          # query heads, group-major
    b_idx, t_idx = torch.as_tensor(b_idx).long(), torch.as_tensor(t_idx).long()
    R = b_idx.numel()
    scale = 1.0 / math.sqrt(D)
    N = T // S
    if lmk_k is None:
        lmk_k, pb = pooled_keys_for_heads(k, lmk_q, kv_heads, G, S)
        prior_b = pb if prior_b is None else prior_b
    qr = q[b_idx, t_idx][:, hq].float()                                            # (R, Hs*G, D)
    lr = lmk_q[b_idx, t_idx][:, hq].float()
    tabs = t_idx + q_offset
    # ---- sliding-window branch: keys [start, t], landmark columns dropped ---------------------
    start = (torch.div(tabs - W + 1, S, rounding_mode="floor") * S).clamp_min(0)
    span = W + S
    j = start.view(R, 1) + torch.arange(span).view(1, span)                        # (R, span) absolute key ids
    keep = (j <= tabs.view(R, 1)) & ((j + 1) % S != 0)
    jc = j.clamp_max(T - 1)
    kw = k[b_idx.view(R, 1), jc][:, :, hk].float()                                 # (R, span, Hs, D)
    vw = v[b_idx.view(R, 1), jc][:, :, hk].float()
    s = torch.einsum("rhgd,rjhd->rhgj", qr.view(R, Hs, G, D), kw) * scale
    s = s.masked_fill(~keep.view(R, 1, 1, span), NEG_INF)
    lse = torch.logsumexp(s, dim=-1)                                               # (R, Hs, G)
    p = torch.exp(s - lse.unsqueeze(-1))
    swa_o = torch.einsum("rhgj,rjhd->rhgd", p, vw).reshape(R, Hs * G, -1).to(dt)
    lse = lse.reshape(R, Hs * G)
    lse_act = lse.to(dt)
    # ---- selection over all chunk keys ------------------------------------------------------------
    g_lmk = lmk_k.shape[2] // Hs
    lk = lmk_k[b_idx].float()                                                      # (R, N, Hs*g_lmk, D)
    if g_lmk == G and G > 1:
        raw = torch.einsum("rhgd,rnhgd->rhgn", lr.view(R, Hs, G, D), lk.view(R, N, Hs, G, D))
    else:
        raw = torch.einsum("rhgd,rnhd->rhgn", lr.view(R, Hs, G, D), lk.view(R, N, Hs, D))
    scaled = raw * scale
    lim = remote_chunk_limit(tabs, W, S)
    logits = scaled.masked_fill((torch.arange(N).view(1, N) >= lim.view(R, 1)).view(R, 1, 1, N), NEG_INF)
    if prior_b is not None:
        logits = logits + prior_b[b_idx].float().view(R, N, Hs, G).permute(0, 2, 3, 1)
    lse_hils = torch.logsumexp(logits, dim=-1)
    lse_total = torch.logaddexp(lse_act.float().view(R, Hs, G), lse_hils)
    keys = (logits - lse_total.unsqueeze(-1)).max(dim=2).values                    # (R, Hs, N)
    keys = torch.where(torch.isnan(keys), torch.full_like(keys, NEG_INF), keys)
    idx = stable_topk_from_keys(keys, topk) if forced_indices is None else forced_indices.to(torch.int32)
    safe = idx.clamp_min(0).long().unsqueeze(2).expand(-1, -1, G, -1)
    sc = torch.gather(scaled, -1, safe).masked_fill((idx < 0).unsqueeze(2).expand(-1, -1, G, -1), NEG_INF)
    scores = sc.reshape(R, Hs * G, -1).to(dt)
    # ---- inter-chunk softmax ----------------------------------------------------------------------
    z = scores
    if prior_b is not None:
        pbr = prior_b[b_idx].float().view(R, N, Hs * G).permute(0, 2, 1)           # (R, Hs*G, N)
        z = z + torch.gather(pbr, -1, idx.repeat_interleave(G, dim=1).clamp_min(0).long()).to(z.dtype)
    cols = [z, lse_act.unsqueeze(-1)]
    if softmax1:
        cols.append(torch.zeros(R, Hs * G, 1, dtype=z.dtype))
    w = F.softmax(torch.cat(cols, dim=-1), dim=-1).to(dt)
    # ---- sparse chunk attention: one softmax per selected chunk, last key of the chunk masked -------
    Kk = idx.shape[-1]
    o_h = torch.zeros(R, Hs, G, v.shape[-1], dtype=torch.float32)
    ar = torch.arange(S)
    for kk in range(Kk):
        c = idx[:, :, kk].long()                                                   # (R, Hs)
        valid = c >= 0
        rows_k = (c.clamp_min(0) * S).unsqueeze(-1) + ar.view(1, 1, S)             # (R, Hs, S) token ids
        kc = k[b_idx.view(R, 1, 1), rows_k, hk.view(1, Hs, 1)].float()             # (R, Hs, S, D)
        vc = v[b_idx.view(R, 1, 1), rows_k, hk.view(1, Hs, 1)].float()
        sk = torch.einsum("rhgd,rhsd->rhgs", qr.view(R, Hs, G, D), kc) * scale
        sk = torch.cat([sk[..., :-1], torch.full_like(sk[..., -1:], NEG_INF)], dim=-1)
        pk = torch.softmax(sk, dim=-1)
        ok = torch.einsum("rhgs,rhsd->rhgd", pk, vc)
        wk = w[..., kk].float().view(R, Hs, G) * valid.unsqueeze(-1).float()
        o_h = o_h + ok * wk.unsqueeze(-1)
    o_hils = o_h.reshape(R, Hs * G, -1).to(dt)
    w_swa = w[..., -2 if softmax1 else -1]
    o = torch.addcmul(o_hils, swa_o, w_swa.unsqueeze(-1))
    return {"o": o, "indices": idx, "scores": scores, "weights": w, "lse_swa": lse, "swa_o": swa_o,
            "o_hils": o_hils, "keys": keys, "lse_total": lse_total, "query_heads": hq}
