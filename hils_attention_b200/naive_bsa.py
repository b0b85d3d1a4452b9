"""Naive block-sparse attention (the exact-chunk-mass baseline of the paper) on the B200 ops.

``naive_bsa_kernel`` keeps the signature, return values and error behaviour of the reference's
``models/NaiveBSA/naive_bsa_kernel.py:121-262``: sliding-window branch (flex_attn_tl) -> exact chunk masses
(exact_chunk_log_z_tl) -> lse_total and group-shared top-K on the normalised log-masses -> softmax over
[selected log Z, lse_swa] -> sparse chunk attention -> o = o_hils + w_swa * o_swa.  The selection differs from the
reference's ``torch.topk`` only where that leaves the choice open: ties go to the smaller chunk id and the ids come
out ascending (the sparse attention does not depend on the order); chunks that are no candidates are never picked
(the reference may pick them with weight zero), and missing slots carry id -1 and weight zero.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F

from . import ops


def _stable_topk_ids(keys: torch.Tensor, topk: int) -> torch.Tensor:
    """ids (..., topk) int32 of the `topk` largest keys, ties to the smaller id, -inf never, ascending, -1 padded."""
    n = keys.shape[-1]
    k_eff = min(topk, n)
    order = torch.sort(keys, dim=-1, descending=True, stable=True).indices[..., :k_eff]
    picked = torch.gather(keys, -1, order)
    ids = torch.where(torch.isneginf(picked), torch.full_like(order, n + 1), order)
    if k_eff < topk:
        ids = F.pad(ids, (0, topk - k_eff), value=n + 1)
    ids = torch.sort(ids, dim=-1).values
    return torch.where(ids >= n, torch.full_like(ids, -1), ids).to(torch.int32)


def naive_bsa_kernel(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, chunk_size: int, window_size: int, topk: int,
                     sm_scale: Optional[float] = None, mask_last_token: bool = False, return_aux: bool = False):
    """q (B,L,h_q,D); k, v (B,L,h_kv,D) -> o (B,L,h_q,D) in q's dtype [, dict of intermediates]."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise ValueError("q, k, v must be 4D: (B, L, H, D)")
    B, L, h_q, D = q.shape
    if k.shape[:2] != (B, L) or v.shape[:2] != (B, L) or k.shape[-1] != D:
        raise ValueError(f"q/k/v batch/seq/dim mismatch: q={tuple(q.shape)}, k={tuple(k.shape)}, v={tuple(v.shape)}")
    h_kv = k.shape[2]
    if v.shape[2] != h_kv:
        raise ValueError(f"k and v must share head count; got k.h_kv={h_kv}, v.h_kv={v.shape[2]}")
    if h_q % h_kv != 0:
        raise ValueError(f"h_q ({h_q}) must be a multiple of h_kv ({h_kv}) for GQA")
    G = h_q // h_kv
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    S, W, K = chunk_size, window_size, topk
    swa_o, lse_swa = ops.flex_attn_tl(q.contiguous(), k.contiguous(), v.contiguous(), window_size=W, chunk_size=S,
                                      training=True, mask_lmk=mask_last_token, expand_to_chunk=True, sm_scale=sm_scale)
    if L < S or K <= 0:
        out = swa_o.to(q.dtype)
        if return_aux:
            return out, {"swa_o": swa_o, "lse_swa": lse_swa, "log_Z": None, "indices": None, "chunk_weights": None}
        return out
    log_z = ops.exact_chunk_log_z_tl(q, k, chunk_size=S, window_size=W, sm_scale=sm_scale, mask_lmk=mask_last_token)
    n_chunk = log_z.shape[-1]
    lse_hils = torch.logsumexp(log_z, dim=-1)
    lse_hils = torch.where(torch.isnan(lse_hils), torch.full_like(lse_hils, float("-inf")), lse_hils)
    lse_total = torch.logaddexp(lse_swa.to(log_z.dtype), lse_hils)
    log_probs = log_z - lse_total.unsqueeze(-1)
    log_probs = torch.where(torch.isnan(log_probs), torch.full_like(log_probs, float("-inf")), log_probs)
    score_pool = log_probs if G == 1 else log_probs.view(B, L, h_kv, G, n_chunk).max(dim=3).values
    indices_kv = _stable_topk_ids(score_pool, K)                                     # (B,L,h_kv,K) ascending, -1 padded
    idx_hq = indices_kv if G == 1 else indices_kv.repeat_interleave(G, dim=2)
    scores_hq = log_z.gather(dim=-1, index=idx_hq.clamp_min(0).long())
    scores_hq = scores_hq.masked_fill(idx_hq < 0, float("-inf"))
    cat_scores = torch.cat([scores_hq, lse_swa.to(scores_hq.dtype).unsqueeze(-1)], dim=-1)
    chunk_weights_f32 = F.softmax(cat_scores, dim=-1)
    sparse_w = chunk_weights_f32[..., :K].to(q.dtype).contiguous()
    swa_w = chunk_weights_f32[..., -1:].to(q.dtype)
    is_training = q.requires_grad or k.requires_grad or v.requires_grad
    hils_o = ops.HiLS_block_M_head(q.contiguous(), k.contiguous(), v.contiguous(), sparse_w, indices_kv.contiguous(),
                                   block_size=S, sm_scale=sm_scale, block_M=None, mask_last_token=mask_last_token,
                                   is_training=is_training)
    o = torch.addcmul(hils_o.to(q.dtype), swa_o.to(q.dtype), swa_w)
    if return_aux:
        return o, {"swa_o": swa_o, "lse_swa": lse_swa, "log_Z": log_z, "log_probs": log_probs, "score_pool": score_pool,
                   "indices_kv": indices_kv, "chunk_weights": chunk_weights_f32}
    return o
