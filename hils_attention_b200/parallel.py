"""Context-parallel forward of the HiLS attention chain: the sequence is sharded over the ranks.

The sequence is cut into equal blocks (a multiple of the chunk size, at least window + chunk long).  With the
`zigzag` partition there are 2·world blocks and rank r holds blocks r and 2·world−1−r, so that every rank scores
the same number of causal candidate chunks; with `contiguous` there are `world` blocks and rank r holds block r.
A rank's tensors are its blocks concatenated in ascending order.

Per layer the ranks exchange only
  * the tail of a block (window rounded up to chunks) as the sliding-window halo of the block that follows it:
    point-to-point between the two owners, nothing else moves;
  * the pooled chunk keys and their bias: one all-gather of N·h·D elements in total;
  * the K/V tiles of the remote chunks a rank selected, per kv head: a fixed-width bitmap of wanted chunks goes
    to each owner (all-to-all), the tile counts come back to the host in ONE small copy (the only host
    synchronisation of the exchange), the tiles travel in one uneven all-to-all per tensor into a local staging
    buffer; chunk ids are rewritten to staging slots and the sparse attention then runs on local memory only.  When
    the ranks together want more than half of all remote tiles (independent random queries over a long context want
    nearly all of them) the exchange falls back to one all-gather of K and of V, which moves the same bytes without
    the gather and scatter copies on either side.
Everything else runs on local memory with the single-GPU kernels.  With `training=True` the chain is differentiable:
the three exchanges are autograd functions whose backward runs the reverse exchange (reduce-scatter of the chunk-key
gradients, halo gradients back to the block they came from, tile gradients back to their owners and summed there), as
the reference's older HSA model does for its all-gather (models/HSA_Ultralong/gather_with_grad.py:9-31).  The reference has no context-parallel HiLS
path; its older HSA model all-gathers every landmark and every chunk's K/V
(models/HSA_Ultralong/hsa_layers.py:893-898).  Collectives go through torch.distributed (NCCL on GPUs, gloo in
the CPU tests of the exchange); no kernel reads a peer's memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


# ------------------------------------------------------------------------------------------
# partition of the sequence
# ------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class SeqPartition:
    """Which blocks of the sequence a rank holds."""
    world: int
    kind: str = "zigzag"          # "zigzag" | "contiguous"

    def __post_init__(self):
        if self.kind not in ("zigzag", "contiguous"):
            raise ValueError(f"unknown partition {self.kind!r}")

    @property
    def n_blocks(self) -> int:
        return 2 * self.world if self.kind == "zigzag" else self.world

    @property
    def blocks_per_rank(self) -> int:
        return 2 if self.kind == "zigzag" else 1

    def blocks(self, rank: int) -> List[int]:
        return [rank, 2 * self.world - 1 - rank] if self.kind == "zigzag" else [rank]

    def owner(self, block: int) -> int:
        if self.kind == "contiguous" or block < self.world:
            return block
        return 2 * self.world - 1 - block

    def block_order(self) -> List[int]:
        """Blocks in the order an all-gather over ranks delivers them (rank 0's blocks, rank 1's, ...)."""
        return [b for r in range(self.world) for b in self.blocks(r)]

    def shard(self, x: torch.Tensor, rank: int, dim: int = 1) -> torch.Tensor:
        """This rank's part of a full-sequence tensor (for tests and benchmarks that start from the whole)."""
        tb = x.shape[dim] // self.n_blocks
        return torch.cat([x.narrow(dim, b * tb, tb) for b in self.blocks(rank)], dim)


# ------------------------------------------------------------------------------------------
# exchanges (pure torch: CPU tensors with gloo, CUDA tensors with NCCL)
# ------------------------------------------------------------------------------------------
def exchange_halo(x: torch.Tensor, part: SeqPartition, halo: int, group=None) -> List[Optional[torch.Tensor]]:
    """x (B, Tl, h, D) = this rank's blocks.  Returns, per local block, the `halo` tokens that precede it in the
    sequence (None for block 0), received from the rank that owns the preceding block."""
    rank = dist.get_rank(group)
    mine = part.blocks(rank)
    tb = x.shape[1] // len(mine)
    tails = {b: x[:, (i + 1) * tb - halo:(i + 1) * tb].contiguous() for i, b in enumerate(mine)}
    out: List[Optional[torch.Tensor]] = [None] * len(mine)
    ops, pending = [], []
    # sends and receives are listed in ascending block order on every rank, so the pairs match up
    for b in range(1, part.n_blocks):
        src, dst = part.owner(b - 1), part.owner(b)
        if src == rank and dst == rank:
            out[mine.index(b)] = tails[b - 1]
        elif src == rank:
            ops.append(dist.P2POp(dist.isend, tails[b - 1], dst, group))
        elif dst == rank:
            buf = torch.empty_like(tails[mine[0]])
            out[mine.index(b)] = buf
            ops.append(dist.P2POp(dist.irecv, buf, src, group))
    if ops:
        pending = dist.batch_isend_irecv(ops)
    for req in pending:
        req.wait()
    return out


def gather_chunk_keys(lk: torch.Tensor, lb: torch.Tensor, part: SeqPartition, group=None
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """lk (B, n_local, h, D'), lb (B, n_local, h): pooled keys and biases of this rank's chunks.  Returns them for
    the whole sequence in chunk order: (B, N, h, D'), (B, N, h)."""
    world = part.world
    lk_all = torch.empty((world,) + tuple(lk.shape), dtype=lk.dtype, device=lk.device)
    lb_all = torch.empty((world,) + tuple(lb.shape), dtype=lb.dtype, device=lb.device)
    dist.all_gather(list(lk_all.unbind(0)), lk.contiguous(), group=group)
    dist.all_gather(list(lb_all.unbind(0)), lb.contiguous(), group=group)
    nb = lk.shape[1] // part.blocks_per_rank
    order = part.block_order()                                   # gathered position -> block
    inv = sorted(range(len(order)), key=lambda i: order[i])      # block -> gathered position

    def reorder(t):
        t = t.transpose(0, 1)                                    # (B, world, n_local, ...)
        t = t.reshape(t.shape[0], len(order), nb, *t.shape[3:])
        return t[:, inv].flatten(1, 2)
    return reorder(lk_all), reorder(lb_all)


@dataclass
class FetchPlan:
    """Result of the request exchange: what to send, what arrives, and where it goes."""
    send_index: torch.Tensor      # (n_send, 3) [b, h, local chunk] of the tiles this rank sends, grouped by peer
    recv_index: torch.Tensor      # (n_recv, 3) [b, h, staging slot] of the tiles that arrive, in arrival order
    send_counts: List[int]
    recv_counts: List[int]
    n_stage: int                  # staging slots taken by remote chunks (the widest (b, h) list)
    remapped: torch.Tensor        # ids rewritten to staging slots (local chunks follow the remote slots)
    dense: bool = False           # all-gather instead: the staging buffer holds every chunk in rank-major order
    wanted_fraction: float = 0.0  # share of all remote (head, chunk) tiles the ranks want, over the whole group


DENSE_FETCH_FRACTION = 0.5


def plan_fetch(indices: torch.Tensor, n_chunks: int, part: SeqPartition, group=None,
               dense_fraction: float = DENSE_FETCH_FRACTION) -> FetchPlan:
    """indices (B, L, h, K): global chunk ids selected by this rank's tokens (−1 = padding), per kv head.
    Exchanges the per-head sets of wanted chunks with their owners and returns the transfer plan."""
    world, rank = part.world, dist.get_rank(group)
    B, L, h, K = indices.shape
    dev = indices.device
    nbk = n_chunks // part.n_blocks                              # chunks per block
    n_local = nbk * part.blocks_per_rank
    # chunk id -> owner * n_local + position among the owner's chunks ("rank-major" order), in int32 arithmetic:
    # block j sits at rank-major block 2 j (j < world) or 2 (2 world - 1 - j) + 1 in the zig-zag partition
    ids = indices.to(torch.int32)
    valid = ids >= 0
    safe = ids.clamp_min(0)
    blk = safe // nbk
    if part.kind == "zigzag":
        blk = torch.where(blk < world, 2 * blk, 2 * (2 * world - 1 - blk) + 1)
    rank_major = blk * nbk + safe % nbk                          # in [0, N)
    del blk, safe
    # wanted[b, h, rank-major chunk]; column N collects the padding.  One int64 tensor (the scatter index) is built.
    row = (torch.arange(B, device=dev, dtype=torch.int32).view(B, 1, 1, 1) * h
           + torch.arange(h, device=dev, dtype=torch.int32).view(1, 1, h, 1)) * (n_chunks + 1)
    flat = (torch.where(valid, rank_major, torch.full_like(rank_major, n_chunks)) + row).reshape(-1).long()
    wanted = torch.zeros(B * h * (n_chunks + 1), dtype=torch.bool, device=dev)
    wanted.scatter_(0, flat, True)
    del flat
    wanted = wanted.view(B, h, n_chunks + 1)[..., :n_chunks].reshape(B, h, world, n_local)
    wanted[:, :, rank] = False                                   # my own chunks are not fetched
    need = wanted.permute(2, 0, 1, 3).contiguous()               # (owner, B, h, local chunk)
    want = torch.empty_like(need)                                # (requester, B, h, my local chunk)
    dist.all_to_all_single(want.view(torch.uint8), need.view(torch.uint8), group=group)
    # staging slot of a remote chunk: its rank among the chunks its (b, h) wants, in rank-major order
    slot = (wanted.reshape(B, h, n_chunks).long().cumsum(-1) - 1)
    per_head = wanted.reshape(B, h, n_chunks).sum(-1)
    total_need = need.sum().reshape(1).to(torch.int64)           # over the group: decides the all-gather fallback
    dist.all_reduce(total_need, group=group)
    counts = torch.cat([want.flatten(1).sum(1), need.flatten(1).sum(1), per_head.max().reshape(1), total_need]).to(torch.int64)
    counts = counts.cpu().tolist()                               # the one host synchronisation of the exchange
    send_counts, recv_counts, n_stage = counts[:world], counts[world:2 * world], counts[2 * world]
    fraction = counts[2 * world + 1] / max(1, world * B * h * (n_chunks - n_local))
    if fraction > dense_fraction:
        remapped = torch.where(valid, rank_major, torch.full_like(rank_major, -1)).to(indices.dtype)
        empty = torch.empty((0, 3), dtype=torch.int64, device=dev)
        return FetchPlan(empty, empty, send_counts, recv_counts, n_chunks - n_local, remapped, True, fraction)
    snd = torch.nonzero_static(want, size=sum(send_counts))      # rows [peer, b, h, chunk], sorted: grouped by peer
    rcv = torch.nonzero_static(need, size=sum(recv_counts))      # rows [owner, b, h, chunk]: the arrival order
    rcv_slot = slot[rcv[:, 1], rcv[:, 2], rcv[:, 0] * n_local + rcv[:, 3]]
    recv_index = torch.stack([rcv[:, 1], rcv[:, 2], rcv_slot], 1)
    # ids -> staging slots: remote chunks by their slot, local chunks after the n_stage remote slots
    is_local = valid & (rank_major // n_local == rank)
    hh = torch.arange(h, device=dev).view(1, 1, h, 1).expand_as(ids)
    bb = torch.arange(B, device=dev).view(B, 1, 1, 1).expand_as(ids)
    remote_slot = slot[bb, hh, rank_major.long()]
    remapped = torch.where(is_local, n_stage + rank_major % n_local, remote_slot)
    remapped = torch.where(valid, remapped, torch.full_like(remapped, -1)).to(indices.dtype)
    return FetchPlan(snd[:, 1:], recv_index, send_counts, recv_counts, n_stage, remapped, False, fraction)


def fetch_chunks(x_chunks: torch.Tensor, plan: FetchPlan, group=None) -> torch.Tensor:
    """x_chunks (B, n_local, S, h, D): this rank's chunks of K or V.  Returns the staging buffer
    (B, n_stage + n_local, S, h, D): the fetched remote tiles in their slots, then the local chunks.  Slots that
    no id refers to stay uninitialised.  In the all-gather fallback the buffer is (B, N, S, h, D) in rank-major order."""
    B, n_local, S, h, D = x_chunks.shape
    if plan.dense:
        world = dist.get_world_size(group)
        every = torch.empty((world,) + tuple(x_chunks.shape), dtype=x_chunks.dtype, device=x_chunks.device)
        dist.all_gather(list(every.unbind(0)), x_chunks.contiguous(), group=group)
        return every.transpose(0, 1).reshape(B, world * n_local, S, h, D)     # a view when B == 1
    si, ri = plan.send_index, plan.recv_index
    send = x_chunks[si[:, 0], si[:, 2], :, si[:, 1], :].contiguous()          # (n_send, S, D)
    recv = torch.empty((ri.shape[0], S, D), dtype=x_chunks.dtype, device=x_chunks.device)
    dist.all_to_all_single(recv, send, output_split_sizes=plan.recv_counts, input_split_sizes=plan.send_counts,
                           group=group)
    stage = torch.empty((B, plan.n_stage + n_local, S, h, D), dtype=x_chunks.dtype, device=x_chunks.device)
    stage[ri[:, 0], ri[:, 2], :, ri[:, 1], :] = recv
    stage[:, plan.n_stage:] = x_chunks
    return stage


# ------------------------------------------------------------------------------------------
# the same exchanges as differentiable functions
# ------------------------------------------------------------------------------------------
def _reduce_scatter_sum(full: torch.Tensor, group) -> torch.Tensor:
    """full (world, ...) -> sum over ranks of slice [my rank] (gloo has no reduce-scatter: all-reduce and slice)."""
    rank = dist.get_rank(group)
    full = full.contiguous()
    if dist.get_backend(group) == "gloo":
        dist.all_reduce(full, group=group)
        return full[rank].clone()
    out = torch.empty_like(full[0])
    dist.reduce_scatter_tensor(out, full, group=group)
    return out


class _GatherChunks(torch.autograd.Function):
    """(B, n_local, ...) of every rank -> (B, N, ...) in chunk order; backward: each rank receives the sum of all
    ranks' gradients for its own chunks."""

    @staticmethod
    def forward(ctx, x, part, group):
        world = part.world
        every = torch.empty((world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        dist.all_gather(list(every.unbind(0)), x.contiguous(), group=group)
        nb = x.shape[1] // part.blocks_per_rank
        order = part.block_order()
        inv = sorted(range(len(order)), key=lambda i: order[i])      # block -> gathered position
        ctx.part, ctx.group, ctx.nb, ctx.order = part, group, nb, order
        t = every.transpose(0, 1)
        t = t.reshape(t.shape[0], len(order), nb, *t.shape[3:])
        return t[:, inv].flatten(1, 2)

    @staticmethod
    def backward(ctx, g):
        part, nb, order = ctx.part, ctx.nb, ctx.order
        g = g.reshape(g.shape[0], len(order), nb, *g.shape[2:])[:, order]          # back to rank-major blocks
        g = g.reshape(g.shape[0], part.world, part.blocks_per_rank * nb, *g.shape[3:]).transpose(0, 1)
        return _reduce_scatter_sum(g, ctx.group), None, None


class _Halo(torch.autograd.Function):
    """x (B, Tl, h, D) -> the halos of the local blocks, concatenated along dim 1 (zeros for the sequence's first
    block); backward: a halo's gradient goes back to the block it came from and is added to that block's tail."""

    @staticmethod
    def forward(ctx, x, part, halo, group):
        ctx.part, ctx.halo, ctx.group, ctx.xshape = part, halo, group, tuple(x.shape)
        hs = exchange_halo(x, part, halo, group)
        ref = x[:, :halo]
        return torch.cat([h if h is not None else torch.zeros_like(ref) for h in hs], 1)

    @staticmethod
    def backward(ctx, g):
        part, halo, group, xshape = ctx.part, ctx.halo, ctx.group, ctx.xshape
        rank = dist.get_rank(group)
        mine = part.blocks(rank)
        tb = xshape[1] // len(mine)
        gx = g.new_zeros(xshape)
        ops, recvs = [], []
        for b in range(1, part.n_blocks):                    # the forward's pairs with the direction reversed
            src, dst = part.owner(b - 1), part.owner(b)
            if dst == rank:
                i = mine.index(b)
                gh = g[:, i * halo:(i + 1) * halo].contiguous()
                if src == rank:
                    j = mine.index(b - 1)
                    gx[:, (j + 1) * tb - halo:(j + 1) * tb] += gh
                else:
                    ops.append(dist.P2POp(dist.isend, gh, src, group))
            elif src == rank:
                buf = torch.empty((xshape[0], halo) + xshape[2:], dtype=g.dtype, device=g.device)
                recvs.append((mine.index(b - 1), buf))
                ops.append(dist.P2POp(dist.irecv, buf, dst, group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        for j, buf in recvs:
            gx[:, (j + 1) * tb - halo:(j + 1) * tb] += buf
        return gx, None, None, None


class _FetchChunks(torch.autograd.Function):
    """fetch_chunks with a backward: the gradient of every fetched tile returns to its owner, where the gradients of all
    the ranks that fetched it (and the owner's own) are summed."""

    @staticmethod
    def forward(ctx, x_chunks, plan, group):
        ctx.plan, ctx.group, ctx.xshape = plan, group, tuple(x_chunks.shape)
        return fetch_chunks(x_chunks, plan, group)

    @staticmethod
    def backward(ctx, g):
        plan, group = ctx.plan, ctx.group
        B, n_local, S, h, D = ctx.xshape
        if plan.dense:
            world = dist.get_world_size(group)
            full = g.reshape(B, world, n_local, S, h, D).transpose(0, 1)
            return _reduce_scatter_sum(full, group), None, None
        si, ri = plan.send_index, plan.recv_index
        g_recv = g[ri[:, 0], ri[:, 2], :, ri[:, 1], :].contiguous()              # tiles I fetched, in arrival order
        g_send = torch.empty((si.shape[0], S, D), dtype=g.dtype, device=g.device)
        dist.all_to_all_single(g_send, g_recv, output_split_sizes=plan.send_counts, input_split_sizes=plan.recv_counts,
                               group=group)
        gx = g[:, plan.n_stage:].clone()
        gx.permute(0, 1, 3, 2, 4).index_put_((si[:, 0], si[:, 2], si[:, 1]), g_send, accumulate=True)   # a view: in place
        return gx, None, None


# ------------------------------------------------------------------------------------------
# the chain
# ------------------------------------------------------------------------------------------
def context_parallel_forward(q, k, v, lmk_q, *, h_kv: int, topk: int, chunk_size: int = 64,
                             window_size: int = 512, partition: str = "zigzag", group=None,
                             return_aux: bool = False, timings: Optional[Dict[str, float]] = None,
                             training: bool = False):
    """Forward of the attention chain for this rank's tokens.  q, lmk_q (B, Tl, h_q, D); k, v (B, Tl, h_kv, D):
    the rank's blocks concatenated (see SeqPartition); every block is a multiple of chunk_size and at least
    window + chunk long.  With `timings` (a dict) the stages are timed with CUDA events, which synchronises.
    training=True keeps what the backward needs and makes the exchanges differentiable."""
    from . import ops
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    part = SeqPartition(world, partition)
    mine = part.blocks(rank)
    B, Tl, h_q, D = q.shape
    S, W = chunk_size, window_size
    tb = Tl // len(mine)
    assert tb * len(mine) == Tl and tb % S == 0, "every block must be a whole number of chunks"
    halo = ((W + S - 1) // S) * S
    assert tb >= halo, "a block must cover the sliding window"
    nbk = tb // S
    n_chunks = nbk * part.n_blocks
    marks = []

    def mark(name):
        if timings is not None and q.is_cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((name, e))

    mark("start")
    # 1. pooled chunk keys of the local chunks, all-gathered into chunk order
    kc = k.unflatten(1, (Tl // S, S))
    lk, lb = ops.chunk_attn_pool(lmk_q[:, S - 1::S], kc)
    if training:
        lmk_k, prior_b = _GatherChunks.apply(lk, part, group), _GatherChunks.apply(lb, part, group)
    else:
        lmk_k, prior_b = gather_chunk_keys(lk, lb, part, group)
    mark("pool+allgather")
    # 2. sliding-window branch per block, with the preceding block's tail as halo
    if training:
        hk_all, hv_all = _Halo.apply(k, part, halo, group), _Halo.apply(v, part, halo, group)
        halos_k = [hk_all[:, i * halo:(i + 1) * halo] for i in range(len(mine))]
        halos_v = [hv_all[:, i * halo:(i + 1) * halo] for i in range(len(mine))]
    else:
        halos_k, halos_v = exchange_halo(k, part, halo, group), exchange_halo(v, part, halo, group)
    mark("halo")
    swa_o, lse = [], []
    for i, blk in enumerate(mine):
        sl = slice(i * tb, (i + 1) * tb)
        if blk > 0 and training:
            # The training kernels want as many queries as keys: the halo gets zero queries whose outputs are dropped.
            # Block starts and the halo are multiples of the chunk size, so positions relative to the start of the
            # halo have the chunk phase of the absolute ones and the windows of the block's own tokens are unchanged.
            zq = torch.zeros((B, halo, h_q, D), dtype=q.dtype, device=q.device)
            o_i, l_i = ops.flex_attn_tl(torch.cat([zq, q[:, sl]], 1), torch.cat([halos_k[i], k[:, sl]], 1),
                                        torch.cat([halos_v[i], v[:, sl]], 1), W, S, training=True, mask_lmk=True,
                                        expand_to_chunk=True)
            o_i, l_i = o_i[:, halo:], l_i[:, halo:]
        elif blk > 0:
            o_i, l_i = ops.flex_attn_tl(q[:, sl], torch.cat([halos_k[i], k[:, sl]], 1),
                                        torch.cat([halos_v[i], v[:, sl]], 1), W, S, training=False, mask_lmk=True,
                                        expand_to_chunk=True, kv_start=blk * tb - halo)
        else:
            o_i, l_i = ops.flex_attn_tl(q[:, sl], k[:, sl], v[:, sl], W, S, training=training, mask_lmk=True,
                                        expand_to_chunk=True)
        swa_o.append(o_i)
        lse.append(l_i)
    swa_o, lse = torch.cat(swa_o, 1), torch.cat(lse, 1)
    lse_act = lse.to(q.dtype)
    mark("swa")
    # 3. selection over all chunk keys at each block's absolute positions, inter-chunk softmax.  (is_training=False
    # only because, as in the reference, the op ignores q_offset otherwise; its scores are differentiable either way.)
    idx, sc = [], []
    for i, blk in enumerate(mine):
        sl = slice(i * tb, (i + 1) * tb)
        i_i, s_i = ops.online_softmax_topk_head(lmk_q[:, sl], lmk_k, lse_act[:, sl], topk, block_size=S,
                                                window_size=W, is_training=False, q_offset=blk * tb,
                                                G=lmk_k.shape[2] // h_kv, bias=prior_b)
        idx.append(i_i)
        sc.append(s_i)
    idx, sc = torch.cat(idx, 1), torch.cat(sc, 1)
    w = ops.inter_chunk_softmax(sc, idx, lse_act, prior_b)
    mark("selection")
    # 4. fetch the selected remote chunks per kv head into a local staging buffer, rewrite the ids
    plan = plan_fetch(idx, n_chunks, part, group)
    mark("plan")
    fetch = (lambda x: _FetchChunks.apply(x, plan, group)) if training else (lambda x: fetch_chunks(x, plan, group))
    k_stage = fetch(kc).flatten(1, 2)
    v_stage = fetch(v.unflatten(1, (Tl // S, S))).flatten(1, 2)
    mark("fetch")
    # 5. sparse chunk attention on local memory only, combine
    o_h = ops.HiLS_block_M_head(q, k_stage, v_stage, w.contiguous(), plan.remapped.to(torch.int32).contiguous(),
                                block_size=S, mask_last_token=True, is_training=training)
    o = torch.addcmul(o_h, swa_o, w[..., -1:])
    mark("sparse+combine")
    if timings is not None and marks:
        torch.cuda.synchronize()
        for (_, a), (name, b) in zip(marks[:-1], marks[1:]):
            timings[name] = timings.get(name, 0.0) + a.elapsed_time(b)
    if return_aux:
        es = k.element_size()
        fetched = B * h_kv * (n_chunks - Tl // S) if plan.dense else sum(plan.recv_counts)
        return o, {"indices": idx, "lse_swa": lse, "remote_tiles": sum(plan.recv_counts),
                   "staging_slots": plan.n_stage, "fetch_mode": "all_gather" if plan.dense else "selected_tiles",
                   "wanted_fraction": plan.wanted_fraction,
                   "fetch_bytes": 2 * fetched * S * D * es,
                   "allgather_bytes": (lmk_k.numel() * lmk_k.element_size() + prior_b.numel() * prior_b.element_size())
                   * (world - 1) // world,
                   "halo_bytes": 2 * sum(1 for b in mine if b > 0 and part.owner(b - 1) != rank) * B * halo * h_kv * D * es}
    return o
