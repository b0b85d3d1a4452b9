"""The attention chain of the reference's HiLS attention module, on the B200 ops.

``HiLSAttentionCore.forward`` follows ``HiLSAttention.forward`` of the reference
(models/FlashHiLS/hils_attention.py:490-633) from the point where q, k, v and the landmark query
are projected, normalised and rotated (:503-508) up to the tensor handed to ``o_proj`` (:631):

  cache update (:512-523) -> flex_attn_tl (:536-547) -> chunk keys (:556, _compute_landmark_keys
  :342-464 incl. the incremental pooling of just-completed chunks during decode) -> chunk selection
  (:568-580) -> prior-bias gather and inter-chunk softmax (:585-610) -> sparse chunk attention (:619)
  -> combine with the sliding-window branch (:620-629).

Projections, RMS norms and rotary embedding stay with the caller (stock transformer plumbing).
``install_into_reference()`` registers this package's ops under the module names the reference
imports (``ops.hils_fwd_bwd_head`` ...), so the reference's own module file binds them unchanged.
"""
from __future__ import annotations

import sys
import types
from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import ops


@dataclass
class HiLSAttentionConfig:
    """The subset of the reference's HiLSConfig that the attention chain reads
    (models/FlashHiLS/hils_attention.py:226-278)."""
    num_attention_heads: int
    num_key_value_heads: int
    hils_topk: int = 32
    chunk_size: int = 64
    hils_sliding_window: int = 512
    enable_prior_query: bool = True
    enable_chunk_pooling: bool = False
    enable_softmax1: bool = False
    num_hidden_layers: int = 1
    shared_q_c: bool = False          # one learned prior query per head instead of the landmark tokens' queries (:271-276)
    apply_hils_rope: bool = False     # rotate the shared prior query to each chunk's last position (:382-387, :425-430)
    head_dim: int = 0                 # needed for the shared prior query only
    initializer_range: float = 0.02


class HiLSAttentionCore(torch.nn.Module):
    def __init__(self, config: HiLSAttentionConfig, layer_idx: int = 0):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.h_q = config.num_attention_heads
        self.h_kv = config.num_key_value_heads
        self.topk = config.hils_topk
        self.chunk_size = config.chunk_size
        self.hils_sliding_window = config.hils_sliding_window
        self.enable_prior_query = config.enable_prior_query
        self.enable_chunk_pooling = config.enable_chunk_pooling
        self.enable_softmax1 = config.enable_softmax1
        self.topk_func = ops.online_softmax_topk_head
        self.hils_func = ops.HiLS_block_M_head
        self.shared_q_c = config.shared_q_c
        self.apply_hils_rope = config.apply_hils_rope
        if self.shared_q_c:
            assert self.enable_prior_query, "shared_q_c requires enable_prior_query=True"
            assert config.head_dim > 0, "shared_q_c needs head_dim"
            self.q_c = torch.nn.Parameter(torch.empty(self.h_q, config.head_dim))
            torch.nn.init.normal_(self.q_c, mean=0.0, std=config.initializer_range)

    def _prior_queries(self, lmk_q, positions, position_embeddings):
        """Pooling queries of the chunks whose last tokens sit at `positions` (a slice or a list of indices into
        this call's tokens): the landmark tokens' own queries, or the shared learned query, rotated to those
        positions when the model rotates its landmark queries (models/FlashHiLS/hils_attention.py:382-389, :425-432)."""
        if not self.shared_q_c:
            return lmk_q[:, positions]
        n = lmk_q[:, positions].shape[1]
        q_c = self.q_c.to(lmk_q.dtype)
        if lmk_q.shape[2] != self.h_q:      # the batch is folded into the head dimension (cached decode / prefill)
            q_c = q_c.repeat(lmk_q.shape[2] // self.h_q, 1)
        mu = q_c.unsqueeze(0).unsqueeze(0).expand(lmk_q.shape[0], n, -1, -1)
        if self.apply_hils_rope:
            assert position_embeddings is not None, "apply_hils_rope needs position_embeddings=(cos, sin)"
            cos, sin = position_embeddings
            mu = ops.single_tensor_rope_autograd(mu.contiguous(), cos[:, positions, :], sin[:, positions, :])
        return mu

    # -- chunk keys: models/FlashHiLS/hils_attention.py:342-464 ---------------------------------
    def _compute_landmark_keys(self, k_src, lmk_q, L, full_seq_len, use_cache, past_key_values,
                               position_embeddings=None):
        S = self.chunk_size
        B = k_src.shape[0]
        prior_b = None
        full_chunks = full_seq_len // S

        def chunked(lo_chunk, hi_chunk):
            return k_src[:, lo_chunk * S:hi_chunk * S].unflatten(1, (hi_chunk - lo_chunk, S))

        if not self.enable_prior_query:
            if self.enable_chunk_pooling:
                return ops.chunk_mean_pool(chunked(0, full_chunks)), None
            return k_src[:, S - 1::S], None

        is_continuation = use_cache and past_key_values is not None and L < full_seq_len
        if is_continuation:
            store = past_key_values._hils_prior_cache
            cached = store.get(self.layer_idx)
            prev_len = full_seq_len - L
            prev_full = prev_len // S
            new_chunks = full_chunks - prev_full
            if new_chunks > 0:
                boundary_local = [S * (prev_full + j) - 1 - prev_len for j in range(1, new_chunks + 1)]
                new_mu = self._prior_queries(lmk_q, boundary_local, position_embeddings)
                new_k = chunked(prev_full, full_chunks)
                new_lmk_k, new_b = ops.chunk_attn_pool(new_mu, new_k)
                if self.enable_chunk_pooling:
                    new_lmk_k = ops.chunk_mean_pool(new_k)
                if cached is not None:
                    lmk_k = torch.cat([cached["lmk_k"], new_lmk_k], dim=1)
                    prior_b = torch.cat([cached["prior_b"], new_b], dim=1)
                else:
                    lmk_k, prior_b = new_lmk_k, new_b
                store[self.layer_idx] = {"lmk_k": lmk_k, "prior_b": prior_b}
            elif cached is not None:
                lmk_k, prior_b = cached["lmk_k"], cached["prior_b"]
            else:
                lmk_k, prior_b = k_src[:, S - 1::S], None
            return lmk_k, prior_b

        mu_q = self._prior_queries(lmk_q, slice(S - 1, full_chunks * S, S), position_embeddings)
        if mu_q.shape[1] == 0:
            if self.enable_chunk_pooling and full_chunks > 0:
                return ops.chunk_mean_pool(chunked(0, full_chunks)), None
            return k_src[:, S - 1::S], None
        kc = chunked(0, full_chunks)
        pooled, prior_b = ops.chunk_attn_pool(mu_q, kc)     # kv heads are shared inside the kernel
        lmk_k = ops.chunk_mean_pool(kc) if self.enable_chunk_pooling else pooled
        if use_cache and past_key_values is not None and prior_b is not None:
            past_key_values._hils_prior_cache[self.layer_idx] = {"lmk_k": lmk_k, "prior_b": prior_b}
        return lmk_k, prior_b

    def _fused_decode_step(self, q, k, v, lmk_q, layer, past_key_values):
        """One new token per sequence against the store: the whole step as one library call.  Returns
        None when the step needs the op-by-op path (training, no pooled keys yet, or the new token
        completes a chunk, whose pooled key must be formed first)."""
        S = self.chunk_size
        cached = past_key_values._hils_prior_cache.get(self.layer_idx)
        needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, lmk_q))
        if (self.training or needs_grad or not self.enable_prior_query or cached is None
                or not layer.is_initialized or self.hils_func is not ops.HiLS_block_M_head
                or self.topk_func is not ops.online_softmax_topk_head or q.dtype not in (torch.bfloat16, torch.float32)):
            return None
        length = layer.get_seq_length()
        if (length + 1) % S == 0 or length + 1 < S or cached.get("prior_b") is None:
            return None
        B, _, h_q, D = q.shape
        layer._reserve(k, v, length + 1)
        kbuf, vbuf = layer._kbuf, layer._vbuf
        lmk_k, prior_b = cached["lmk_k"], cached["prior_b"]
        o, self._step_ws = ops.decode_step(
            q.reshape(B * h_q, D), lmk_q.reshape(B * h_q, D), k.reshape(-1, D), v.reshape(-1, D),
            kbuf.view(kbuf.shape[0], -1, D), vbuf.view(vbuf.shape[0], -1, D), length,
            lmk_k.reshape(lmk_k.shape[1], -1, D), prior_b.reshape(prior_b.shape[1], -1), self.topk, S,
            self.hils_sliding_window, self.enable_softmax1, workspace=getattr(self, "_step_ws", None))
        layer._len = length + 1
        layer._publish()
        return o.view(B, 1, h_q, D)

    def decode_paged(self, q, k, v, lmk_q, store, position_embeddings=None, return_indices: bool = False):
        """One new token per sequence against a paged store (kv_store.PagedKVStore), sequences of different lengths
        in one batch: q, lmk_q (B, 1, h_q, D), k, v (B, 1, h_kv, D) with B = store.batch, between store.begin_step()
        and store.end_step().  The whole step is one library call; a sequence whose chunk this token completes then
        gets the chunk's pooled key and prior bias (models/FlashHiLS/hils_attention.py:364-410), formed from the
        page the chunk lives in.  Inference only."""
        if not self.enable_prior_query:
            raise NotImplementedError("decode_paged needs enable_prior_query=True (the pooled chunk keys live in the store)")
        B = q.shape[0]
        if B != store.batch:
            raise ValueError(f"decode_paged: {B} rows given, the store's batch is {store.batch}")
        layer = self.layer_idx
        k_pages, v_pages, table, lens, lmk_k, prior_b = store.step_args(layer)
        max_len = max((store.length(b) for b in store.active_slots()), default=0)
        out = ops.decode_step_paged(
            q[:, 0].contiguous(), lmk_q[:, 0].contiguous(), k[:, 0].contiguous(), v[:, 0].contiguous(), k_pages, v_pages,
            table, lens, max_len, lmk_k, prior_b, self.topk, self.chunk_size, self.hils_sliding_window,
            self.enable_softmax1, workspace=getattr(self, "_paged_ws", None), return_indices=return_indices)
        o, self._paged_ws = out[0], out[-1]
        done = store.completing()
        if done:
            rows = torch.tensor(done, dtype=torch.long, device=q.device)
            pe = None
            if position_embeddings is not None:
                cos, sin = position_embeddings
                pe = (cos if cos.shape[0] == 1 else cos.index_select(0, rows), sin if sin.shape[0] == 1 else sin.index_select(0, rows))
            mu = self._prior_queries(lmk_q.index_select(0, rows), slice(0, 1), pe)           # (n, 1, h_q, D)
            kc = store.chunk_keys(layer, done).unsqueeze(1)                                   # (n, 1, 64, h_kv, D)
            new_k, new_b = ops.chunk_attn_pool(mu.contiguous(), kc)
            if self.enable_chunk_pooling:
                new_k = ops.chunk_mean_pool(kc)
            store.put_chunk_keys(layer, done, new_k[:, 0], new_b[:, 0])
        o = o.unsqueeze(1)
        return (o, out[1].unsqueeze(1)) if return_indices else o

    def forward(self, q, k, v, lmk_q, past_key_values=None, use_cache: bool = False,
                return_aux: bool = False, position_embeddings=None):
        """q, lmk_q (B,L,h_q,D); k, v (B,L,h_kv,D) of the NEW tokens.  Returns (B,L,h_q,Dv), the
        tensor the reference flattens and feeds to o_proj.  position_embeddings = (cos, sin) of this call's
        tokens, (B or 1, L, D): only read when the shared prior query is rotated."""
        B, L = q.shape[0], q.shape[1]
        S, W = self.chunk_size, self.hils_sliding_window
        caching = use_cache and past_key_values is not None
        h_kv = self.h_kv
        folded = False
        if caching and hasattr(past_key_values, "layer"):
            # token-major store of this package: the batch is folded into the head dimension, so the
            # cached K/V are consumed in place as (1, T, B*h_kv, D) and only the new tokens are copied
            layer = past_key_values.layer(self.layer_idx + self.config.num_hidden_layers)
            fused = self._fused_decode_step(q, k, v, lmk_q, layer, past_key_values) if (L == 1 and not return_aux) else None
            if fused is not None:
                return fused
            layer.update(k, v)
            k, v = layer.folded()
            q = q.transpose(0, 1).reshape(1, L, B * self.h_q, q.shape[-1])
            lmk_q = lmk_q.transpose(0, 1).reshape(1, L, B * lmk_q.shape[2], lmk_q.shape[-1])
            h_kv, folded, B_orig, B = B * self.h_kv, True, B, 1
        elif caching:
            k, v = past_key_values.update(k, v, self.layer_idx + self.config.num_hidden_layers, None)
        swa_o, lse_sum = ops.flex_attn_tl(q, k, v, window_size=W, chunk_size=S,
                                          training=(past_key_values is None), mask_lmk=True,
                                          expand_to_chunk=True)
        lse_sum = lse_sum.contiguous().to(q.dtype)
        full_seq_len = k.shape[1]
        aux = {"swa_o": swa_o, "lse_swa": lse_sum}
        if full_seq_len >= S:
            lmk_k, prior_b = self._compute_landmark_keys(k, lmk_q, L, full_seq_len, use_cache, past_key_values,
                                                         position_embeddings)
            q_offset = full_seq_len - L if caching else 0
            indices, scores = self.topk_func(
                lmk_q, lmk_k, lse_sum, self.topk, block_size=S, window_size=W, is_training=self.training,
                is_causal=True, q_offset=q_offset, G=lmk_k.shape[2] // h_kv, bias=prior_b)
            # prior-bias gather, concatenation with the window branch's lse and softmax: one kernel
            chunk_weights = ops.inter_chunk_softmax(
                scores, indices, lse_sum, prior_b if self.enable_prior_query else None, self.enable_softmax1)
            swa_idx = -2 if self.enable_softmax1 else -1
            if self.hils_func is ops.HiLS_block_M_head:
                # sparse chunk attention and o = o_hils + w_swa * o_swa as one op
                o_lower = ops.sparse_attn_combine(q, k, v, chunk_weights, indices, swa_o, swa_idx, block_size=S,
                                                  mask_last_token=True, is_training=self.training)
                hils_o = None
            else:
                hils_o = self.hils_func(q, k, v, weights=chunk_weights, indices=indices, block_size=S,
                                        mask_last_token=True, is_training=self.training)
                o_lower = torch.addcmul(hils_o, swa_o, chunk_weights[:, :, :, swa_idx].unsqueeze(-1))
            aux.update(indices=indices, scores=scores, weights=chunk_weights, lmk_k=lmk_k, prior_b=prior_b,
                       hils_o=hils_o)
        elif self.enable_softmax1:
            o_lower = swa_o * torch.sigmoid(lse_sum).to(swa_o.dtype).unsqueeze(-1)
        else:
            o_lower = swa_o
        if folded:  # back to (B, L, heads, ...)
            def unfold(t):
                return t.reshape(L, B_orig, t.shape[2] // B_orig, *t.shape[3:]).transpose(0, 1)
            o_lower = unfold(o_lower)
            aux = {n: (unfold(t) if n in ("indices", "scores", "weights", "lse_swa", "swa_o", "hils_o") and t is not None else t)
                   for n, t in aux.items()}
        return (o_lower, aux) if return_aux else o_lower


def install_into_reference() -> None:
    """Register this package's ops under the module paths the reference imports from, so that
    ``from ops.hils_fwd_bwd_head import HiLS_block_M_head`` (models/FlashHiLS/hils_attention.py:9-10,
    :264-265; models/NaiveBSA/naive_bsa_kernel.py:169-171) resolves here.  Call before importing the
    reference's model code."""
    table = {
        "ops.hils_fwd_bwd_head": {"HiLS_block_M_head": ops.HiLS_block_M_head},
        "ops.topk_head_softmax": {"online_softmax_topk_head": ops.online_softmax_topk_head},
        "ops.chunk_attn_pool_tilelang": {"chunk_attn_pool_tilelang": ops.chunk_attn_pool_tilelang},
        "ops.exact_chunk_log_z_tilelang": {"exact_chunk_log_z_tl": ops.exact_chunk_log_z_tl},
        "ops.flex_attn_tilelang": {"flex_attn_tl": ops.flex_attn_tl,
                                   "flex_attn_tl_two_phase": ops.flex_attn_tl_two_phase},
        "ops.rope_tilelang_fp32": {"single_tensor_rope_autograd": ops.single_tensor_rope_autograd,
                                   "rope_rotary_pos_emb": ops.rope_rotary_pos_emb},
    }
    pkg = sys.modules.get("ops")
    if pkg is None:
        pkg = types.ModuleType("ops")
        pkg.__path__ = []  # mark as package
        sys.modules["ops"] = pkg
    for name, attrs in table.items():
        mod = types.ModuleType(name)
        for k, fn in attrs.items():
            setattr(mod, k, fn)
        sys.modules[name] = mod
        setattr(pkg, name.split(".", 1)[1], mod)
