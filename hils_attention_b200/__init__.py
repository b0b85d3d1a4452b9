"""B200-native (sm_100a) HiLS sparse-attention hot path.

`ops` mirrors the reference's ``ops/`` call signatures on top of the C-ABI CUDA library
(libhils_b200.so, declared in include/hils_b200.h); `attention` chains them the way the reference's
attention module does; `cache` is the KV store used for prefill and decode, `kv_store` the paged store
(64-token pages = chunks) for decode batches of sequences of different lengths.
"""
from . import _lib
from .naive_bsa import naive_bsa_kernel
from .ops import (HiLS_block_M_head, chunk_attn_pool, chunk_attn_pool_tilelang, chunk_mean_pool,
                  exact_chunk_log_z_tl, flex_attn_tl, flex_attn_tl_two_phase, inter_chunk_softmax,
                  online_softmax_topk_head, rmsnorm_rope, rope_rotary_pos_emb, single_tensor_rope_autograd,
                  sparse_attn_combine)

__all__ = ["HiLS_block_M_head", "chunk_attn_pool", "chunk_attn_pool_tilelang", "chunk_mean_pool",
           "exact_chunk_log_z_tl", "flex_attn_tl", "flex_attn_tl_two_phase", "inter_chunk_softmax",
           "online_softmax_topk_head", "rmsnorm_rope", "rope_rotary_pos_emb", "single_tensor_rope_autograd",
           "sparse_attn_combine", "naive_bsa_kernel"]
