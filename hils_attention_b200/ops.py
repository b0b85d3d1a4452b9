"""Host-side mirror of the reference's ``ops/`` interface, backed by libhils_b200.so.

Every public function keeps the reference's name, positional order, keyword names, return
values and error behaviour, so the reference's attention module can bind them unchanged:

  chunk_attn_pool / chunk_attn_pool_tilelang   models/FlashHiLS/hils_attention.py:66-135,
                                                ops/chunk_attn_pool_tilelang.py:605-626
  online_softmax_topk_head                      ops/topk_head_softmax.py:1212-1367
  HiLS_block_M_head                             ops/hils_fwd_bwd_head.py:928-964
  exact_chunk_log_z_tl                          ops/exact_chunk_log_z_tilelang.py:481-498
  flex_attn_tl / flex_attn_tl_two_phase         ops/flex_attn_tilelang.py:1261-1352

Tensors must live on a CUDA device; there is no CPU path.  Kernels are enqueued on the current
torch stream and never synchronise with the host.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import call, dtype_code, ptr, query, stream

__all__ = [
    "chunk_attn_pool", "chunk_attn_pool_tilelang", "chunk_mean_pool", "online_softmax_topk_head",
    "HiLS_block_M_head", "exact_chunk_log_z_tl", "flex_attn_tl", "flex_attn_tl_two_phase",
]


# ------------------------------------------------------------------------------------------
# chunk pooling
# ------------------------------------------------------------------------------------------
def _chunked_k_view(k_chunked: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """Return (tensor, batch stride in elements) such that chunk rows are dense inside a batch
    entry.  A (B,N,S,h,D) view of a longer (B,T,h,D) cache is used in place (no copy)."""
    B, N, S, h, D = k_chunked.shape
    st = k_chunked.stride()
    dense_inner = (st[4] == 1 and st[3] == D and st[2] == h * D and st[1] == S * h * D) or N == 0
    if dense_inner and (B == 1 or st[0] >= N * S * h * D):
        return k_chunked, (st[0] if B > 1 else N * S * h * D)
    kc = k_chunked.contiguous()
    return kc, N * S * h * D


class _ChunkAttnPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, mu_q, k_chunked, sm_scale, compact):
        B, N, h_q, D = mu_q.shape
        S, h_kv = k_chunked.shape[2], k_chunked.shape[3]
        mu = mu_q.contiguous()
        kc, kbs = _chunked_k_view(k_chunked)
        dt = dtype_code(kc)
        if mu.dtype != kc.dtype:
            mu = mu.to(kc.dtype)
        lmk_k = torch.empty((B, N, h_q, D), dtype=kc.dtype, device=kc.device)
        lmk_b = torch.empty((B, N, h_q), dtype=torch.float32, device=kc.device)
        call("hils_pool_fwd", ptr(mu), ptr(kc), ptr(lmk_k), ptr(lmk_b), B, N, S, h_q, h_kv, D, kbs,
             float(sm_scale), int(compact), dt, stream())
        ctx.save_for_backward(mu, kc)
        ctx.meta = (B, N, S, h_q, h_kv, D, kbs, float(sm_scale), int(compact), dt, mu_q.dtype)
        return lmk_k, lmk_b

    @staticmethod
    def backward(ctx, g_k, g_b):
        mu, kc = ctx.saved_tensors
        B, N, S, h_q, h_kv, D, kbs, scale, compact, dt, mu_dtype = ctx.meta
        g_k = None if (g_k is None or compact) else g_k.contiguous().to(kc.dtype)
        g_b = None if g_b is None else g_b.contiguous().float()
        d_mu = torch.empty((B, N, h_q, D), dtype=kc.dtype, device=kc.device)
        d_k = torch.empty((B, N, S, h_kv, D), dtype=kc.dtype, device=kc.device)
        call("hils_pool_bwd", ptr(mu), ptr(kc), ptr(g_k), ptr(g_b), ptr(d_mu), ptr(d_k), B, N, S, h_q,
             h_kv, D, kbs, scale, compact, dt, stream())
        return d_mu.to(mu_dtype), d_k, None, None


def chunk_attn_pool_tilelang(mu_q: torch.Tensor, k_chunked: torch.Tensor, sm_scale: Optional[float] = None,
                             compact_lmk_k: bool = False):
    """mu_q (B,N,H,D), k_chunked (B,N,S,H,D) -> lmk_k (B,N,H,D) in K's dtype, lmk_b (B,N,H) fp32.
    Same call as ops/chunk_attn_pool_tilelang.py:605; k_chunked may also carry fewer (kv) heads,
    in which case each kv head serves h_q/h_kv query heads from one read of its keys."""
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(mu_q.shape[-1])
    return _ChunkAttnPool.apply(mu_q, k_chunked, sm_scale, bool(compact_lmk_k))


def chunk_attn_pool(mu_q: torch.Tensor, k_chunked: torch.Tensor, sm_scale: Optional[float] = None):
    """Attention-pool each chunk with its prior query (models/FlashHiLS/hils_attention.py:66-135):
    p = softmax_j(scale <mu_q[c], K[c,j]>) with the chunk's last token masked,
    k' = sum_j p_j K[c,j], b' = entropy(p).  Shape errors raise ValueError like the reference."""
    if mu_q.dim() != 4 or k_chunked.dim() != 5:
        raise ValueError(
            f"chunk_attn_pool: expected mu_q (B, N, h_q, d) and k_chunked "
            f"(B, N, S, h_kv, d); got {tuple(mu_q.shape)} and {tuple(k_chunked.shape)}")
    B, N, h_q, D = mu_q.shape
    Bk, Nk, S, h_kv, Dk = k_chunked.shape
    if (B, N, D) != (Bk, Nk, Dk):
        raise ValueError(
            f"chunk_attn_pool: mu_q vs k_chunked shape mismatch on (B, N, d) -- got "
            f"mu_q={tuple(mu_q.shape)}, k_chunked={tuple(k_chunked.shape)}")
    if h_q % h_kv != 0:
        raise ValueError(
            f"chunk_attn_pool: mu_q h_q ({h_q}) must be a multiple of k_chunked h_kv ({h_kv}) "
            f"for GQA grouping")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    return chunk_attn_pool_tilelang(mu_q, k_chunked, sm_scale)


class _ChunkMeanPool(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k_chunked):
        B, N, S, h, D = k_chunked.shape
        kc, kbs = _chunked_k_view(k_chunked)
        dt = dtype_code(kc)
        out = torch.empty((B, N, h, D), dtype=kc.dtype, device=kc.device)
        call("hils_meanpool_fwd", ptr(kc), ptr(out), B, N, S, h, D, kbs, dt, stream())
        ctx.meta = (B, N, S, h, D, dt)
        return out

    @staticmethod
    def backward(ctx, g):
        B, N, S, h, D, dt = ctx.meta
        g = g.contiguous()
        d_k = torch.empty((B, N, S, h, D), dtype=g.dtype, device=g.device)
        call("hils_meanpool_bwd", ptr(g), ptr(d_k), B, N, S, h, D, dt, stream())
        return d_k


def chunk_mean_pool(k_chunked: torch.Tensor) -> torch.Tensor:
    """k' = mean over each chunk's tokens ((B,N,S,h,D) -> (B,N,h,D)); the `.mean(dim=2)` of
    models/FlashHiLS/hils_attention.py:445-446 as one streaming kernel."""
    return _ChunkMeanPool.apply(k_chunked)


# ------------------------------------------------------------------------------------------
# chunk selection
# ------------------------------------------------------------------------------------------
class _TopkSelect(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, lmks, lse_swa, topk, block_size, window_size, is_causal, q_offset, drop_mask,
                sm_scale, bias, gumbel, per_qhead, aux):
        B, L, h_kv, G, D = q.shape
        N = lmks.shape[1]
        q_in = q.contiguous()
        k_in = lmks.contiguous()
        dt = dtype_code(q_in)
        if k_in.dtype != q_in.dtype:
            k_in = k_in.to(q_in.dtype)
        lse = lse_swa.contiguous()
        if lse.dtype not in (torch.float32, torch.bfloat16):
            lse = lse.float()
        dev = q.device
        indices = torch.empty((B, L, h_kv, topk), dtype=torch.int32, device=dev)
        scores = torch.empty((B, L, h_kv * G, topk), dtype=q_in.dtype, device=dev)
        lse_total = rank_keys = None
        if aux is not None:
            lse_total = torch.empty((B, L, h_kv, G), dtype=torch.float32, device=dev)
            rank_keys = torch.empty((B, L, h_kv, N), dtype=torch.float32, device=dev)
            aux["lse_total"], aux["rank_keys"] = lse_total, rank_keys
        scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
        ws_bytes = query("hils_topk_fwd_workspace_bytes", B, L, N, h_kv, G, D, dt)
        ws = _workspace(ws_bytes, dev)
        call("hils_topk_fwd", ptr(q_in), ptr(k_in), ptr(lse), ptr(bias), ptr(gumbel), ptr(drop_mask),
             ptr(indices), ptr(scores), ptr(lse_total), ptr(rank_keys), B, L, N, h_kv, G, D, int(topk),
             int(block_size), int(window_size), int(bool(is_causal)), int(q_offset), int(per_qhead), scale,
             dt, dtype_code(lse), ptr(ws), ws_bytes, stream())
        ctx.save_for_backward(q_in, k_in, indices)
        ctx.meta = (B, L, N, h_kv, G, D, int(topk), int(per_qhead), scale, dt, q.dtype, lmks.dtype)
        ctx.mark_non_differentiable(indices)
        return indices, scores

    @staticmethod
    def backward(ctx, _g_idx, g_scores):
        q_in, k_in, indices = ctx.saved_tensors
        B, L, N, h_kv, G, D, topk, per_qhead, scale, dt, q_dtype, k_dtype = ctx.meta
        g = g_scores.contiguous().to(q_in.dtype)
        d_q = torch.empty_like(q_in)
        acc = torch.empty(k_in.shape, dtype=torch.float32, device=k_in.device)
        d_k = torch.empty_like(k_in)
        call("hils_topk_bwd", ptr(g), ptr(indices), ptr(q_in), ptr(k_in), ptr(d_q), ptr(acc), ptr(d_k), B, L, N,
             h_kv, G, D, topk, per_qhead, scale, dt, stream())
        return (d_q.to(q_dtype), d_k.to(k_dtype)) + (None,) * 12


def online_softmax_topk_head(q: torch.Tensor, lmks: torch.Tensor, lse_swa: torch.Tensor, topk: int,
                             block_size: int, window_size: int, is_causal: bool = True, q_offset: int = 0,
                             is_training: bool = True, drop_mask: Optional[torch.Tensor] = None,
                             sm_scale: Optional[float] = None, bias: Optional[torch.Tensor] = None,
                             use_gumbel: bool = False, gumbel_noise: Optional[torch.Tensor] = None, G: int = 1,
                             _aux: Optional[dict] = None):
    """Softmax-then-max top-k chunk selection (ops/topk_head_softmax.py:1212-1367).

    q (B,L,h_q,D) or (B,L,h_kv,G,D); lmks (B,N,h_lmk,D) with h_lmk = h_kv (shared, G == 1) or h_q
    (per-q-head, G > 1); lse_swa (B,L,h_q) or (B,L,h_kv,G); bias (B,N,h_q) or (B,N,h_kv,G).
    Returns indices (B,L,h_kv,topk) int32 ascending / -1 padded and scores (B,L,h_q,topk) = raw
    scale*q.k' in q's dtype.  Gradients flow through scores only.  As in the reference,
    q_offset is ignored (0) when is_training.  `_aux`, if a dict, receives the fp32 lse_total and
    ranking keys the selector used (diagnostics for the parity tests).
    """
    if q.dim() == 4:
        B, L, h_q, D = q.shape
        lmks_h, D_lmk = lmks.shape[2], lmks.shape[3]
        if D != D_lmk:
            assert D_lmk % D == 0, f"lmks D dim ({D_lmk}) must be divisible by q D dim ({D})"
            ratio = D_lmk // D
            lmks = lmks.reshape(lmks.shape[0], lmks.shape[1], lmks_h * ratio, D)
            lmks_h *= ratio
        if G == 1:
            assert h_q % lmks_h == 0, f"h_q ({h_q}) must be divisible by lmks_h ({lmks_h})"
            h_kv, G_eff, per_qhead = lmks_h, h_q // lmks_h, False
        else:
            assert lmks_h == h_q, f"when G>1, lmks must have h_q ({h_q}) heads, got {lmks_h}"
            assert h_q % G == 0, f"h_q ({h_q}) must be divisible by G ({G})"
            h_kv, G_eff, per_qhead = h_q // G, G, True
        q = q.view(B, L, h_kv, G_eff, D)
    else:
        B, L, h_kv, G_in, D = q.shape
        h_q = h_kv * G_in
        D_lmk = lmks.shape[3]
        if D != D_lmk:
            assert D_lmk % D == 0, f"lmks D dim ({D_lmk}) must be divisible by q D dim ({D})"
            lmks = lmks.reshape(lmks.shape[0], lmks.shape[1], lmks.shape[2] * (D_lmk // D), D)
        lmks_h = lmks.shape[2]
        if G == 1:
            if lmks_h == h_kv:
                per_qhead, G_eff = False, G_in
            elif lmks_h == h_q:
                per_qhead, G_eff = True, G_in
            else:
                raise AssertionError(f"lmks_h ({lmks_h}) must be h_kv ({h_kv}) or h_q ({h_q})")
        else:
            assert lmks_h == h_q, f"when G>1, lmks must have h_q ({h_q}) heads, got {lmks_h}"
            assert h_q % G == 0, f"h_q ({h_q}) must be divisible by G ({G})"
            if (h_q // G != h_kv) or (G != G_in):
                q = q.reshape(B, L, h_q // G, G, D)
                h_kv = h_q // G
            G_eff, per_qhead = G, True
    N = lmks.shape[1]
    assert lmks.shape[0] == B and lmks.shape[3] == D
    lse_swa = lse_swa.reshape(B, L, h_kv * G_eff)
    bias_arg = None
    if bias is not None:
        bias_arg = bias.to(device=q.device, dtype=torch.float32)
        if bias_arg.dim() == 3:
            assert bias_arg.shape == (B, N, h_kv * G_eff), \
                f"bias shape {tuple(bias_arg.shape)} != ({B}, {N}, {h_kv * G_eff})"
        elif bias_arg.dim() == 4:
            assert bias_arg.shape == (B, N, h_kv, G_eff), \
                f"bias shape {tuple(bias_arg.shape)} != ({B}, {N}, {h_kv}, {G_eff})"
        else:
            raise AssertionError(f"bias must be [B, S, h_q] or [B, S, h_kv, G], got {tuple(bias_arg.shape)}")
        bias_arg = bias_arg.contiguous()
    use_gumbel = bool(use_gumbel) or (gumbel_noise is not None)
    gumbel_arg = None
    if use_gumbel:
        assert is_training, "gumbel_noise is only supported in training mode"
        if gumbel_noise is None:
            u = torch.rand(1, 1, h_kv * G_eff, N, device=q.device, dtype=torch.float32)
            u.clamp_(min=1e-20, max=1 - 1e-7)
            gumbel_arg = -torch.log(-torch.log(u))
        else:
            assert gumbel_noise.shape == (1, 1, h_kv * G_eff, N), \
                f"gumbel_noise shape {tuple(gumbel_noise.shape)} != ({1}, {1}, {h_kv * G_eff}, {N})"
            gumbel_arg = gumbel_noise.detach().to(device=q.device, dtype=torch.float32).contiguous()
    if drop_mask is not None:
        assert drop_mask.shape == (B, L, N), f"drop_mask shape {tuple(drop_mask.shape)} != ({B}, {L}, {N})"
        drop_mask = drop_mask.to(torch.int32).contiguous()
    if is_training:
        q_offset = 0
    indices, scores = _TopkSelect.apply(q, lmks, lse_swa, int(topk), int(block_size), int(window_size),
                                        bool(is_causal), int(q_offset), drop_mask, sm_scale, bias_arg,
                                        gumbel_arg, per_qhead, _aux)
    return indices, scores.view(B, L, h_kv * G_eff, -1)


# ------------------------------------------------------------------------------------------
# sparse chunk attention
# ------------------------------------------------------------------------------------------
def _workspace(nbytes: int, device) -> Optional[torch.Tensor]:
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes > 0 else None


class _SparseChunkAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, weights, indices, block_size, sm_scale, mask_last_token, is_training, slope,
                swa_o=None, swa_col=-1):
        assert q.is_contiguous() and k.is_contiguous() and v.is_contiguous()
        assert weights.is_contiguous() and indices.is_contiguous()
        B, L, HQ, D = q.shape
        T, H, Dk = k.shape[1], k.shape[2], k.shape[3]
        Dv = v.shape[-1]
        K = indices.shape[-1]
        nw = weights.shape[-1]
        assert HQ % H == 0, f"HQ={HQ} must be divisible by H={H}"
        assert Dk == D, f"Q head_dim ({D}) must equal K head_dim ({Dk})"
        if sm_scale is None:
            sm_scale = 1.0 / math.sqrt(D)
        dt = dtype_code(q)
        slope_dev = None
        if slope is not None:
            assert slope.shape == (HQ,), f"slope must be 1-D with shape ({HQ},), got {tuple(slope.shape)}"
            slope_dev = slope.to(dtype=torch.float32, device=q.device).contiguous()
        w = weights.to(q.dtype)
        idx = indices if indices.dtype == torch.int32 else indices.to(torch.int32)
        o = torch.empty((B, L, HQ, Dv), dtype=q.dtype, device=q.device)
        dims = (B, L, T, HQ, H, D, Dv, K)
        ws_bytes = query("hils_sparse_attn_fwd_workspace_bytes", *dims, int(block_size), dt)
        ws = _workspace(ws_bytes, q.device)
        call("hils_sparse_attn_fwd", ptr(q), ptr(k), ptr(v), ptr(w), ptr(idx), ptr(slope_dev), ptr(o), *dims, nw,
             int(block_size), float(sm_scale), int(bool(mask_last_token)), dt, ptr(ws), ws_bytes, stream())
        swa_col = int(swa_col) % nw if swa_o is not None else -1
        if swa_o is not None:
            # o <- o + w[..., swa_col] * swa_o (models/FlashHiLS/hils_attention.py:620-629), in place
            assert swa_o.shape == o.shape and swa_o.dtype == o.dtype and swa_o.is_contiguous()
            call("hils_combine_fwd", ptr(o), ptr(swa_o), ptr(w), ptr(o), B, L, HQ, Dv, nw, swa_col, dt, stream())
        ctx.is_training = bool(is_training)
        if is_training:
            # a sparse selection's forward leaves the chunk-major index of the id lists at the start of its workspace:
            # the backward reuses a copy of it (4 + 2 G bytes per selected slot) instead of building it again
            ix_bytes = query("hils_sparse_attn_index_bytes", *dims, int(block_size), dt) if ws_bytes > 0 else 0
            built = ws[:ix_bytes].clone() if 0 < ix_bytes <= ws_bytes else q.new_empty(0)
            ctx.save_for_backward(q, k, v, w, idx, slope_dev if slope_dev is not None else q.new_empty(0),
                                  swa_o if swa_o is not None else q.new_empty(0), built)
            ctx.meta = (dims, nw, int(block_size), float(sm_scale), int(bool(mask_last_token)), dt,
                        slope_dev is not None, weights.dtype, swa_col)
        return o

    @staticmethod
    def backward(ctx, do):
        if not getattr(ctx, "is_training", True):
            raise RuntimeError(
                "HiLS_block_M_head: the forward ran with is_training=False, which keeps nothing for "
                "the backward pass; call it with is_training=True to differentiate.")
        q, k, v, w, idx, slope_dev, swa_o, built = ctx.saved_tensors
        dims, nw, S, scale, mask_last, dt, has_slope, w_dtype, swa_col = ctx.meta
        B, L, T, HQ, H, D, Dv, K = dims
        do = do.contiguous().to(q.dtype)
        d_q = torch.empty_like(q)
        d_k = torch.empty_like(k)
        d_v = torch.empty_like(v)
        d_w = torch.empty((B, L, HQ, nw), dtype=q.dtype, device=q.device)
        ws_bytes = query("hils_sparse_attn_bwd_workspace_bytes", *dims, S, dt)
        ws = _workspace(ws_bytes, q.device)
        call("hils_sparse_attn_bwd_with_index", ptr(q), ptr(k), ptr(v), ptr(w), ptr(idx),
             ptr(slope_dev) if has_slope else None, ptr(do), ptr(d_q), ptr(d_k), ptr(d_v), ptr(d_w), *dims, nw, S, scale,
             mask_last, dt, ptr(ws), ws_bytes, ptr(built) if built.numel() else None, built.numel(), stream())
        d_swa_o = None
        if swa_col >= 0:
            d_swa_o = torch.empty_like(swa_o)
            call("hils_combine_bwd", ptr(do), ptr(swa_o), ptr(w), ptr(d_swa_o), ptr(d_w), B, L, HQ, Dv, nw, swa_col,
                 dt, stream())
        return d_q, d_k, d_v, d_w.to(w_dtype), None, None, None, None, None, None, d_swa_o, None


def HiLS_block_M_head(q, k, v, weights, indices, block_size=64, sm_scale=None, block_M=None,
                      mask_last_token=True, dtype="bfloat16", accum_dtype="float", num_threads=None,
                      num_threads_fwd=None, num_threads_bwd=None, is_training=True, slope=None):
    """Sparse chunk attention (ops/hils_fwd_bwd_head.py:928-964).

    o_i = sum_k weights[i,k] * softmax_{j in chunk indices[i,k]}(scale q_i.K_j) V_j with one softmax
    per selected chunk; ids < 0 end a row's list.  q (B,L,h_q,D); k,v (B,T,h_kv,D[v]); weights
    (B,L,h_q,num_weights >= K); indices (B,L,h_kv,K) int32; all contiguous.  The tile-shape knobs
    (block_M, num_threads*, dtype strings) are accepted for call compatibility and ignored: the
    element type follows the tensors.  Backward after is_training=False raises RuntimeError.
    """
    B, L, HQ, D = q.shape
    _, L_kv, H, Dk = k.shape
    assert D == Dk, f"Q head_dim ({D}) must equal K head_dim ({Dk})"
    assert HQ % H == 0, f"HQ={HQ} must be divisible by H={H}"
    return _SparseChunkAttention.apply(q, k, v, weights, indices, block_size, sm_scale, mask_last_token,
                                       is_training, slope, None, -1)


# ------------------------------------------------------------------------------------------
# exact per-chunk log Z
# ------------------------------------------------------------------------------------------

def sparse_attn_combine(q, k, v, weights, indices, swa_o, swa_col=-1, block_size=64, sm_scale=None,
                        mask_last_token=True, is_training=True, slope=None):
    """Sparse chunk attention followed by the combination with the sliding-window branch,
    ``HiLS_block_M_head(...) + weights[..., swa_col, None] * swa_o`` (models/FlashHiLS/hils_attention.py:619-629),
    as one differentiable op: the weight column of the window branch gets its gradient in the same
    tensor the sparse backward fills, and no intermediate is materialised."""
    return _SparseChunkAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), weights.contiguous(),
                                       indices.contiguous(), int(block_size), sm_scale, mask_last_token,
                                       is_training, slope, swa_o.contiguous(), int(swa_col))


class _ChunkWeights(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, indices, lse_swa, prior_b, softmax1):
        B, L, HQ, K = scores.shape
        h_idx = indices.shape[2]
        assert indices.shape == (B, L, h_idx, K) and HQ % h_idx == 0
        assert lse_swa.shape == (B, L, HQ), f"lse_swa shape {tuple(lse_swa.shape)} != ({B}, {L}, {HQ})"
        dt = dtype_code(scores)
        sc = scores.contiguous()
        idx = (indices if indices.dtype == torch.int32 else indices.to(torch.int32)).contiguous()
        lse = lse_swa.to(scores.dtype).contiguous()
        N = 0
        pb = None
        if prior_b is not None:
            N = prior_b.shape[1]
            assert prior_b.shape == (B, N, HQ), f"prior_b shape {tuple(prior_b.shape)} != ({B}, {N}, {HQ})"
            pb = prior_b.to(torch.float32).contiguous()
        ncol = K + 1 + (1 if softmax1 else 0)
        w = torch.empty((B, L, HQ, ncol), dtype=scores.dtype, device=scores.device)
        call("hils_chunk_weights_fwd", ptr(sc), ptr(idx), ptr(pb), ptr(lse), ptr(w), B, L, N, HQ, h_idx, K,
             int(bool(softmax1)), dt, stream())
        ctx.save_for_backward(w, idx)
        ctx.meta = (B, L, N, HQ, h_idx, K, int(bool(softmax1)), dt, prior_b is not None,
                    None if prior_b is None else prior_b.dtype, lse_swa.dtype)
        return w

    @staticmethod
    def backward(ctx, dw):
        w, idx = ctx.saved_tensors
        B, L, N, HQ, h_idx, K, softmax1, dt, has_pb, pb_dtype, lse_dtype = ctx.meta
        want_db = has_pb and ctx.needs_input_grad[3]
        dw = dw.contiguous().to(w.dtype)
        d_sc = torch.empty((B, L, HQ, K), dtype=w.dtype, device=w.device)
        d_lse = torch.empty((B, L, HQ), dtype=w.dtype, device=w.device)
        d_pb = torch.empty((B, N, HQ), dtype=torch.float32, device=w.device) if want_db else None
        call("hils_chunk_weights_bwd", ptr(w), ptr(dw), ptr(idx), ptr(d_sc), ptr(d_lse), ptr(d_pb), B, L, N, HQ,
             h_idx, K, softmax1, dt, stream())
        return d_sc, None, d_lse.to(lse_dtype), (None if d_pb is None else d_pb.to(pb_dtype)), None


def inter_chunk_softmax(scores, indices, lse_swa, prior_b=None, softmax1=False):
    """Weights of the selected chunks and of the sliding-window branch
    (models/FlashHiLS/hils_attention.py:585-610): softmax over [scores + prior_b[ids], lse_swa(, 0)].

    scores (B,L,h_q,K) and lse_swa (B,L,h_q) in the activation dtype, indices (B,L,h_kv,K) int32 with
    -1 for empty slots, prior_b (B,N,h_q) fp32 or None.  Returns (B,L,h_q,K+1[+1]) in scores' dtype;
    differentiable with respect to scores, lse_swa and prior_b."""
    return _ChunkWeights.apply(scores, indices, lse_swa, prior_b, bool(softmax1))


def decode_step(q, lmk_q, k_new, v_new, k_store, v_store, length: int, lmk_k, prior_b, topk: int, chunk_size: int = 64,
                window_size: int = 512, softmax1: bool = False, sm_scale: Optional[float] = None,
                workspace: Optional[torch.Tensor] = None, return_indices: bool = False):
    """One decode step of the whole chain in a single library call
    (models/FlashHiLS/hils_attention.py:512-633 with one new token per sequence; inference only).

    Batch folded into heads: q and lmk_q (the selection's query) (heads_q, D); k_new, v_new (heads_kv, D); k_store, v_store
    (capacity, heads_kv, D) token-major holding `length` tokens - the new token is written to row
    `length`; lmk_k (N, heads_lmk, D) pooled chunk keys, prior_b (N, heads_q) fp32 or None.
    Returns o (heads_q, D) [, indices (heads_kv, topk)].  `workspace` (uint8) is reused when large enough."""
    heads_q, D = q.shape
    heads_kv = k_new.shape[0]
    N, heads_lmk = lmk_k.shape[0], lmk_k.shape[1]
    assert k_store.shape[1:] == (heads_kv, D) and v_store.shape[1:] == (heads_kv, D)
    assert k_store.shape[0] > length, "the store has no free row"
    assert q.is_contiguous() and lmk_q.is_contiguous() and k_new.is_contiguous() and v_new.is_contiguous()
    assert lmk_q.shape == q.shape and k_store.is_contiguous() and v_store.is_contiguous() and lmk_k.is_contiguous()
    dt = dtype_code(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    pb = None if prior_b is None else prior_b.to(torch.float32).contiguous()
    need = query("hils_decode_step_workspace_bytes", heads_q, heads_kv, heads_lmk, D, int(topk), N, int(bool(softmax1)), dt)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=q.device)
    o = torch.empty_like(q)
    idx = torch.empty((heads_kv, topk), dtype=torch.int32, device=q.device) if return_indices else None
    call("hils_decode_step", ptr(q), ptr(lmk_q), ptr(k_new), ptr(v_new), ptr(k_store), ptr(v_store), int(length), ptr(lmk_k), ptr(pb),
         N, ptr(o), ptr(idx), heads_q, heads_kv, heads_lmk, D, int(topk), int(chunk_size), int(window_size),
         int(bool(softmax1)), float(sm_scale), dt, ptr(workspace), workspace.numel(), stream())
    return (o, idx, workspace) if return_indices else (o, workspace)


def decode_step_paged(q, lmk_q, k_new, v_new, k_pages, v_pages, page_table, lens, max_len: int, lmk_k, prior_b, topk: int,
                      chunk_size: int = 64, window_size: int = 512, softmax1: bool = False,
                      sm_scale: Optional[float] = None, workspace: Optional[torch.Tensor] = None,
                      return_indices: bool = False):
    """One decode step of the whole chain over a paged store, for sequences of different lengths
    (models/FlashHiLS/hils_attention.py:512-633 with one new token per sequence; inference only).

    q, lmk_q (B, h_q, D); k_new, v_new (B, h_kv, D); k_pages, v_pages (num_pages, h_kv, 64, D) the pool;
    page_table (B, max_pages) int32 and lens (B) int32 on the device: sequence b holds lens[b] tokens, chunk c
    of it lives in page page_table[b, c], and the page of position lens[b] is already in the table; max_len is
    a host-side upper bound of lens.  lmk_k (B, N, h_lmk, D) pooled chunk keys, prior_b (B, N, h_q) fp32 or
    None.  The new token is written into its page; lens is left as it is.
    Returns o (B, h_q, D) [, indices (B, h_kv, topk)] and the workspace for reuse."""
    B, h_q, D = q.shape
    h_kv = k_new.shape[1]
    N, h_lmk = lmk_k.shape[1], lmk_k.shape[2]
    num_pages = k_pages.shape[0]
    assert k_pages.shape == v_pages.shape == (num_pages, h_kv, chunk_size, D)
    assert page_table.dtype == torch.int32 and lens.dtype == torch.int32 and page_table.shape[0] == B == lens.shape[0]
    assert lmk_q.shape == q.shape and k_new.shape == v_new.shape == (B, h_kv, D) and lmk_k.shape[0] == B
    for t in (q, lmk_q, k_new, v_new, k_pages, v_pages, page_table, lens, lmk_k):
        assert t.is_contiguous()
    dt = dtype_code(q)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    pb = None if prior_b is None else prior_b.to(torch.float32).contiguous()
    assert pb is None or pb.shape == (B, N, h_q)
    need = query("hils_decode_step_paged_workspace_bytes", B, h_q, h_kv, h_lmk, D, int(topk), N, int(bool(softmax1)), dt)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(max(need, 1), dtype=torch.uint8, device=q.device)
    o = torch.empty_like(q)
    idx = torch.empty((B, h_kv, topk), dtype=torch.int32, device=q.device) if return_indices else None
    call("hils_decode_step_paged", ptr(q), ptr(lmk_q), ptr(k_new), ptr(v_new), ptr(k_pages), ptr(v_pages), ptr(page_table),
         int(page_table.shape[1]), int(num_pages), ptr(lens), int(max_len), ptr(lmk_k), ptr(pb), N, ptr(o), ptr(idx),
         B, h_q, h_kv, h_lmk, D, int(topk), int(chunk_size), int(window_size), int(bool(softmax1)), float(sm_scale), dt,
         ptr(workspace), workspace.numel(), stream())
    return (o, idx, workspace) if return_indices else (o, workspace)


# ------------------------------------------------------------------------------------------
# per-head RMSNorm + rotary embedding
# ------------------------------------------------------------------------------------------
class _NormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, cos, sin, eps):
        B, L, H, D = x.shape
        xc = x.contiguous()
        w = None if weight is None else weight.to(x.dtype).contiguous()
        cs_batched, cs_code = 0, dtype_code(xc)
        c = s_ = None
        if cos is not None:
            assert sin is not None and cos.shape == sin.shape and cos.dtype == sin.dtype
            c, s_ = cos, sin
            if c.dim() == 3 and c.shape[0] == 1:
                c, s_ = c[0], s_[0]
            if c.dim() == 3:
                assert c.shape == (B, L, D), f"cos shape {tuple(cos.shape)} != ({B}, {L}, {D})"
                cs_batched = 1
            else:
                assert c.shape == (L, D), f"cos shape {tuple(cos.shape)} != ({L}, {D})"
            if c.dtype not in (torch.float32, torch.bfloat16):
                c, s_ = c.float(), s_.float()
            c, s_ = c.contiguous(), s_.contiguous()
            cs_code = dtype_code(c)
        out = torch.empty_like(xc)
        rstd = torch.empty((B, L, H), dtype=torch.float32, device=x.device) if w is not None else None
        call("hils_norm_rope_fwd", ptr(xc), ptr(w), ptr(c), ptr(s_), ptr(out), ptr(rstd), B, L, H, D, cs_batched,
             float(eps), dtype_code(xc), cs_code, stream())
        ctx.save_for_backward(xc, *(t for t in (w, c, s_, rstd) if t is not None))
        ctx.meta = (B, L, H, D, cs_batched, cs_code, w is not None, c is not None,
                    None if weight is None else weight.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        B, L, H, D, cs_batched, cs_code, has_w, has_cs, w_dtype = ctx.meta
        saved = list(ctx.saved_tensors)
        xc = saved.pop(0)
        w = saved.pop(0) if has_w else None
        c = saved.pop(0) if has_cs else None
        s_ = saved.pop(0) if has_cs else None
        rstd = saved.pop(0) if has_w else None
        g = d_out.contiguous().to(xc.dtype)
        d_x = torch.empty_like(xc)
        d_w = torch.empty((D,), dtype=torch.float32, device=xc.device) if has_w else None
        call("hils_norm_rope_bwd", ptr(xc), ptr(w), ptr(c), ptr(s_), ptr(rstd), ptr(g), ptr(d_x), ptr(d_w), B, L, H, D,
             cs_batched, dtype_code(xc), cs_code, stream())
        return d_x, (None if d_w is None else d_w.to(w_dtype)), None, None, None


def rmsnorm_rope(x, weight=None, cos=None, sin=None, eps: float = 1e-6):
    """Per-head RMSNorm (models/FlashHiLS/modeling_olmo_hils.py:105-111) followed by the rotary embedding
    (ops/rope_tilelang_fp32.py:96-181) in one pass.  x (B,L,H,D); weight (D,) or None; cos, sin (L,D),
    (1,L,D) or (B,L,D), bf16 or fp32, or None.  Differentiable with respect to x and weight."""
    return _NormRope.apply(x, weight, cos, sin, float(eps))


def single_tensor_rope_autograd(x, x_cos, x_sin):
    """Rotary embedding of one tensor (ops/rope_tilelang_fp32.py:173-182): x (B,L,H,D); x_cos, x_sin
    (B,L,D) / (1,L,D) / (L,D), bf16 or fp32; returns x's dtype."""
    return _NormRope.apply(x, None, x_cos, x_sin, 0.0)


def rope_rotary_pos_emb(q, k, cos, sin):
    """Rotary embedding of q and k (ops/rope_tilelang_fp32.py:84-88): returns (q_out, k_out)."""
    return _NormRope.apply(q, None, cos, sin, 0.0), _NormRope.apply(k, None, cos, sin, 0.0)


class _ExactChunkLogZ(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, chunk_size, window_size, sm_scale, mask_lmk):
        assert q.dim() == 4 and k.dim() == 4
        B, L, H_q, D = q.shape
        Bk, Lk, H_kv, Dk = k.shape
        assert (Bk, Lk, Dk) == (B, L, D), f"q/k batch/seq/dim mismatch: q={tuple(q.shape)}, k={tuple(k.shape)}"
        assert H_q % H_kv == 0, f"H_q ({H_q}) must be a multiple of H_kv ({H_kv}) for GQA"
        q_c, k_c = q.contiguous(), k.contiguous()
        dt = dtype_code(q_c)
        n_chunk = (L + chunk_size - 1) // chunk_size
        log_z = torch.empty((B, L, H_q, n_chunk), dtype=torch.float32, device=q.device)
        call("hils_chunk_logz_fwd", ptr(q_c), ptr(k_c), ptr(log_z), B, L, H_q, H_kv, D, chunk_size, window_size,
             float(sm_scale), int(mask_lmk), dt, stream())
        ctx.save_for_backward(q_c, k_c, log_z)
        ctx.meta = (B, L, H_q, H_kv, D, chunk_size, window_size, float(sm_scale), bool(mask_lmk), dt)
        return log_z

    @staticmethod
    def backward(ctx, d_log_z):
        q, k, log_z = ctx.saved_tensors
        B, L, H_q, H_kv, D, S, W, scale, mask_lmk, dt = ctx.meta
        if mask_lmk:
            raise NotImplementedError(
                "exact_chunk_log_z_tl(mask_lmk=True) is forward/eval-only; backward is not implemented "
                "for the landmark-masked path.")
        g = d_log_z.contiguous().float()
        d_q, d_k = torch.empty_like(q), torch.empty_like(k)
        call("hils_chunk_logz_bwd", ptr(q), ptr(k), ptr(log_z), ptr(g), ptr(d_q), ptr(d_k), B, L, H_q, H_kv, D, S,
             W, scale, dt, stream())
        return d_q, d_k, None, None, None, None


def exact_chunk_log_z_tl(q: torch.Tensor, k: torch.Tensor, *, chunk_size: int, window_size: int,
                         sm_scale: Optional[float] = None, mask_lmk: bool = False) -> torch.Tensor:
    """Exact chunk mass log Z_{i,c} (ops/exact_chunk_log_z_tilelang.py:481-498): (B,L,H_q,ceil(L/S))
    fp32, -inf where chunk c is not strictly left of row i's snapped window.  mask_lmk=True is
    forward-only (its backward raises NotImplementedError)."""
    if sm_scale is None:
        sm_scale = (1.0 / q.shape[-1]) ** 0.5
    return _ExactChunkLogZ.apply(q, k, int(chunk_size), int(window_size), float(sm_scale), bool(mask_lmk))


# ------------------------------------------------------------------------------------------
# sliding-window branch
# ------------------------------------------------------------------------------------------
class _FlexAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, window_size, chunk_size, mask_lmk, expand_to_chunk, use_cache, sm_scale, kv_start):
        B, Lq, H, D = q.shape
        Lk, H_kv, Dv = k.shape[1], k.shape[2], v.shape[-1]
        q_c, k_c, v_c = q.contiguous(), k.contiguous(), v.contiguous()
        dt = dtype_code(q_c)
        scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
        o = torch.empty((B, Lq, H, Dv), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Lq, H), dtype=torch.float32, device=q.device)
        call("hils_swa_fwd", ptr(q_c), ptr(k_c), ptr(v_c), ptr(o), ptr(lse), B, Lq, Lk, H, H_kv, D, Dv,
             int(window_size), int(chunk_size), int(bool(mask_lmk)), int(bool(expand_to_chunk)), scale,
             int(kv_start), dt, stream())
        ctx.use_cache = bool(use_cache)
        if not use_cache:
            ctx.save_for_backward(q_c, k_c, v_c, o, lse)
            ctx.meta = (B, Lq, H, H_kv, D, Dv, int(window_size), int(chunk_size), int(bool(mask_lmk)),
                        int(bool(expand_to_chunk)), scale, dt)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse):
        if ctx.use_cache:
            raise RuntimeError("flex_attn_tl backward is not supported in inference (use_cache=True) mode")
        q, k, v, o, lse = ctx.saved_tensors
        B, L, H, H_kv, D, Dv, W, S, mask_lmk, expand, scale, dt = ctx.meta
        do = do.contiguous().to(q.dtype)
        dlse = None if dlse is None else dlse.contiguous().float()
        d_q, d_k, d_v = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws_bytes = query("hils_swa_bwd_workspace_bytes", B, L, H, H_kv, D, Dv, S, dt)
        ws = _workspace(ws_bytes, q.device)
        call("hils_swa_bwd", ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), ptr(do), ptr(dlse), ptr(d_q), ptr(d_k),
             ptr(d_v), B, L, H, H_kv, D, Dv, W, S, mask_lmk, expand, scale, dt, ptr(ws), ws_bytes, stream())
        return d_q, d_k, d_v, None, None, None, None, None, None, None


def flex_attn_tl(q, k, v, window_size: int, chunk_size: int, training: bool = True, mask_lmk: bool = True,
                 expand_to_chunk: bool = True, sm_scale: Optional[float] = None, kv_start: int = 0):
    """Sliding-window attention with a chunk-snapped left edge (ops/flex_attn_tilelang.py:1261-1310).
    q (B,Lq,H_q,D), k/v (B,Lk,H_kv,D[v]) -> o (B,Lq,H_q,Dv) in q's dtype, lse (B,Lq,H_q) fp32 natural
    log.  training=False allows Lq <= Lk and a non-zero kv_start; its backward raises RuntimeError.
    Gradients flow through both o and lse."""
    if training and int(kv_start) != 0:
        raise ValueError("flex_attn_tl only supports non-zero kv_start in inference (training=False)")
    if training and q.shape[1] != k.shape[1]:
        raise ValueError("flex_attn_tl: training mode needs q and k of equal length")
    return _FlexAttn.apply(q, k, v, window_size, chunk_size, mask_lmk, expand_to_chunk, not training,
                           sm_scale, kv_start)


def flex_attn_tl_two_phase(q, k, v, window_size: int, chunk_size: int, training: bool = True,
                           mask_lmk: bool = True, expand_to_chunk: bool = True,
                           sm_scale: Optional[float] = None, kv_start: int = 0):
    """Same call as flex_attn_tl (ops/flex_attn_tilelang.py:1313-1352).  The backward here is always
    the atomic-free two-kernel form (a dQ pass over query rows, a dK/dV pass over key rows)."""
    return flex_attn_tl(q, k, v, window_size, chunk_size, training, mask_lmk, expand_to_chunk, sm_scale,
                        kv_start)
