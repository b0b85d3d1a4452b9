"""Context-parallel forward of the HiLS attention chain (sequence sharded over the ranks).

Each rank owns a contiguous range of `Tl` tokens (a multiple of the chunk size) with its q, k, v.
Per layer the ranks exchange only
  * the tail of each shard (window + one chunk) as the sliding-window halo of the next rank,
  * the pooled chunk keys and their bias (all-gather: N*h*D elements in total),
  * the K/V tiles of the remote chunks a rank actually selected (requested by id, sent point to point),
and everything else runs on local memory with the single-GPU kernels.  The reference has no
context-parallel HiLS path; its older HSA model all-gathers every landmark and every chunk's K/V
(models/HSA_Ultralong/hsa_layers.py:893-898).  Collectives go through torch.distributed (NCCL on
GPUs, gloo in the CPU tests of the exchange plan); no kernel reads a peer's memory.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------
# exchange plan (pure torch: works on CPU tensors with gloo and on CUDA tensors with NCCL)
# ------------------------------------------------------------------------------------------
def plan_remote_chunks(indices: torch.Tensor, first_local_chunk: int, n_local: int
                       ) -> Tuple[torch.Tensor, torch.Tensor]:
    """indices (B, L, h_kv, K) global chunk ids (-1 = padding).  Returns (remote_ids, remapped):
    the ascending unique ids that live on other ranks, and the ids rewritten as positions in the
    staging buffer [remote chunks in that order | this rank's n_local chunks]."""
    valid = indices >= 0
    is_remote = valid & ((indices < first_local_chunk) | (indices >= first_local_chunk + n_local))
    remote_ids = torch.unique(indices[is_remote])                                  # ascending
    pos = torch.searchsorted(remote_ids, indices.clamp_min(0).to(remote_ids.dtype))
    n_remote = remote_ids.numel()
    local_pos = indices - first_local_chunk + n_remote
    remapped = torch.where(is_remote, pos.to(indices.dtype), local_pos.to(indices.dtype))
    remapped = torch.where(valid, remapped, torch.full_like(indices, -1))
    return remote_ids, remapped


def exchange_chunks(k_chunks: torch.Tensor, v_chunks: torch.Tensor, remote_ids: torch.Tensor,
                    chunks_per_rank: int, group=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """k_chunks, v_chunks (B, n_local, S, h, D): this rank's chunks.  remote_ids: ascending global
    ids this rank needs from others.  Returns the requested tiles (B, n_remote, S, h, D) for K and V.
    Request lists travel by all-gather (padded), tiles by point-to-point sends."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = k_chunks.device
    n_req = torch.tensor([remote_ids.numel()], device=dev, dtype=torch.int64)
    counts = [torch.zeros_like(n_req) for _ in range(world)]
    dist.all_gather(counts, n_req, group=group)
    counts = [int(c.item()) for c in counts]
    width = max(max(counts), 1)
    mine = torch.full((width,), -1, device=dev, dtype=torch.int64)
    mine[:remote_ids.numel()] = remote_ids.to(torch.int64)
    all_req = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(all_req, mine, group=group)
    B, _, S, h, D = k_chunks.shape
    ops: List[dist.P2POp] = []
    send_keep = []
    # what every peer wants from me
    for peer in range(world):
        if peer == rank:
            continue
        req = all_req[peer][:counts[peer]]
        sel = req[(req >= rank * chunks_per_rank) & (req < (rank + 1) * chunks_per_rank)] - rank * chunks_per_rank
        if sel.numel():
            ks = k_chunks.index_select(1, sel).contiguous()
            vs = v_chunks.index_select(1, sel).contiguous()
            send_keep += [ks, vs]
            ops += [dist.P2POp(dist.isend, ks, peer, group), dist.P2POp(dist.isend, vs, peer, group)]
    # what I want from every peer (remote_ids is ascending, so per-owner groups are contiguous)
    k_out = torch.empty((B, remote_ids.numel(), S, h, D), dtype=k_chunks.dtype, device=dev)
    v_out = torch.empty_like(k_out)
    owner = torch.div(remote_ids, chunks_per_rank, rounding_mode="floor")
    recv_parts = []
    for peer in range(world):
        if peer == rank:
            continue
        n = int((owner == peer).sum().item())
        if n:
            lo = int((owner < peer).sum().item())
            kb = torch.empty((B, n, S, h, D), dtype=k_chunks.dtype, device=dev)
            vb = torch.empty_like(kb)
            recv_parts.append((lo, n, kb, vb))
            ops += [dist.P2POp(dist.irecv, kb, peer, group), dist.P2POp(dist.irecv, vb, peer, group)]
    if ops:
        for req in dist.batch_isend_irecv(ops):
            req.wait()
    for lo, n, kb, vb in recv_parts:
        k_out[:, lo:lo + n] = kb
        v_out[:, lo:lo + n] = vb
    return k_out, v_out


def exchange_halo(x: torch.Tensor, halo: int, group=None) -> Optional[torch.Tensor]:
    """x (B, Tl, h, D).  Returns the last `halo` tokens of the previous rank (None on rank 0)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tail = x[:, -halo:].contiguous()
    parts = [torch.empty_like(tail) for _ in range(world)]
    dist.all_gather(parts, tail, group=group)
    return parts[rank - 1] if rank > 0 else None


# ------------------------------------------------------------------------------------------
# the chain
# ------------------------------------------------------------------------------------------
def context_parallel_forward(q, k, v, lmk_q, *, h_kv: int, topk: int, chunk_size: int = 64,
                             window_size: int = 512, group=None, return_aux: bool = False):
    """Forward of the attention chain for this rank's tokens.  q, lmk_q (B, Tl, h_q, D); k, v
    (B, Tl, h_kv, D); every rank holds the same Tl, a multiple of chunk_size and >= window + chunk."""
    from . import ops
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, Tl, h_q, D = q.shape
    S, W = chunk_size, window_size
    assert Tl % S == 0, "the local sequence length must be a multiple of the chunk size"
    Nl = Tl // S
    halo = ((W + S - 1) // S) * S
    assert Tl >= halo, "the local sequence must cover the sliding window"
    # 1. sliding-window branch with the previous rank's tail as halo
    hk, hv = exchange_halo(k, halo, group), exchange_halo(v, halo, group)
    if rank > 0:
        k_sw, v_sw = torch.cat([hk, k], 1), torch.cat([hv, v], 1)
        swa_o, lse = ops.flex_attn_tl(q, k_sw, v_sw, W, S, training=False, mask_lmk=True, expand_to_chunk=True,
                                      kv_start=rank * Tl - halo)
    else:
        swa_o, lse = ops.flex_attn_tl(q, k, v, W, S, training=False, mask_lmk=True, expand_to_chunk=True)
    lse_act = lse.to(q.dtype)
    # 2. pooled chunk keys of the local chunks, all-gathered
    kc = k.unflatten(1, (Nl, S))
    lk, lb = ops.chunk_attn_pool(lmk_q[:, S - 1::S], kc)
    lk_all = [torch.empty_like(lk) for _ in range(world)]
    lb_all = [torch.empty_like(lb) for _ in range(world)]
    dist.all_gather(lk_all, lk.contiguous(), group=group)
    dist.all_gather(lb_all, lb.contiguous(), group=group)
    lmk_k, prior_b = torch.cat(lk_all, 1), torch.cat(lb_all, 1)
    # 3. selection over all chunk keys at this rank's absolute positions
    idx, sc = ops.online_softmax_topk_head(lmk_q, lmk_k, lse_act, topk, block_size=S, window_size=W,
                                           is_training=False, q_offset=rank * Tl, G=lmk_k.shape[2] // h_kv,
                                           bias=prior_b)
    g_b = prior_b.shape[2] // idx.shape[2]
    idx_hq = idx.repeat_interleave(g_b, dim=2) if g_b != 1 else idx
    gathered = torch.gather(prior_b.unsqueeze(-1).expand(-1, -1, -1, topk), 1, idx_hq.clamp_min(0).long())
    w = F.softmax(torch.cat([sc + gathered.to(sc.dtype), lse_act.unsqueeze(-1)], -1), -1).to(q.dtype)
    # 4. fetch the selected remote chunks into a local staging buffer, rewrite the ids
    remote_ids, idx_local = plan_remote_chunks(idx, rank * Nl, Nl)
    vc = v.unflatten(1, (Nl, S))
    rk, rv = exchange_chunks(kc, vc, remote_ids, Nl, group)
    k_stage = torch.cat([rk, kc], 1).flatten(1, 2)
    v_stage = torch.cat([rv, vc], 1).flatten(1, 2)
    # 5. sparse chunk attention on local memory only, combine
    o_h = ops.HiLS_block_M_head(q, k_stage, v_stage, w.contiguous(), idx_local.to(torch.int32).contiguous(),
                                block_size=S, mask_last_token=True, is_training=False)
    o = torch.addcmul(o_h, swa_o, w[..., -1:])
    if return_aux:
        return o, {"indices": idx, "remote_chunks": int(remote_ids.numel()), "lse_swa": lse}
    return o
