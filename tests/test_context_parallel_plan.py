"""Host-side logic of the context-parallel path on CPU with gloo ranks: the per-head request exchange and the
uneven all-to-all of K/V tiles must reproduce a gather from the full (unsharded) tensors through the rewritten
ids; the halo exchange must deliver the tokens that precede each block; the all-gather of the pooled keys must
come back in chunk order.  Contiguous and zig-zag partitions, 2 and 4 ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, kind, dense_fraction, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hils_attention_b200.parallel import SeqPartition, exchange_halo, fetch_chunks, gather_chunk_keys, plan_fetch
        part = SeqPartition(world, kind)
        g = torch.Generator().manual_seed(5)
        B, nbk, S, h, D, K = 2, 3, 4, 2, 8, 5
        N = nbk * part.n_blocks
        n_local = nbk * part.blocks_per_rank
        L = n_local * S
        k_full = torch.randn(B, N, S, h, D, generator=g)
        v_full = torch.randn(B, N, S, h, D, generator=g)
        idx = torch.randint(-1, N, (world, B, L, h, K), generator=g, dtype=torch.int32)[rank]
        if rank == world - 1:
            idx[:, :, 1] = -1                       # a head that wants nothing at all
        kc, vc = part.shard(k_full, rank), part.shard(v_full, rank)
        plan = plan_fetch(idx, N, part, dense_fraction=dense_fraction)
        k_stage, v_stage = fetch_chunks(kc, plan), fetch_chunks(vc, plan)
        ok = plan.dense == (dense_fraction == 0.0)
        ok &= k_stage.shape[1] == (N if plan.dense else plan.n_stage + n_local)
        own = {b * nbk + c for b in part.blocks(rank) for c in range(nbk)}
        wanted = {(b, hh, int(c)) for b in range(B) for hh in range(h) for c in idx[b, :, hh].flatten().tolist()
                  if c >= 0 and c not in own}
        ok &= sum(plan.recv_counts) == len(wanted)           # every remote (head, chunk) tile travels once
        for b in range(B):
            for l in range(L):
                for hh in range(h):
                    for kk in range(K):
                        c, s = int(idx[b, l, hh, kk]), int(plan.remapped[b, l, hh, kk])
                        if c < 0:
                            ok &= s == -1
                        else:
                            ok &= torch.equal(k_stage[b, s, :, hh], k_full[b, c, :, hh])
                            ok &= torch.equal(v_stage[b, s, :, hh], v_full[b, c, :, hh])
        # halo: the tokens that precede each of my blocks
        T = N * S
        x_full = torch.arange(B * T * h * D, dtype=torch.float32).view(B, T, h, D)
        halos = exchange_halo(part.shard(x_full, rank), part, 5)
        tb = T // part.n_blocks
        for i, blk in enumerate(part.blocks(rank)):
            if blk == 0:
                ok &= halos[i] is None
            else:
                ok &= torch.equal(halos[i], x_full[:, blk * tb - 5:blk * tb])
        # pooled keys come back in chunk order
        lk_full = torch.randn(B, N, h, D, generator=g)
        lb_full = torch.randn(B, N, h, generator=g)
        lk, lb = gather_chunk_keys(part.shard(lk_full, rank), part.shard(lb_full, rank), part)
        ok &= torch.equal(lk, lk_full) and torch.equal(lb, lb_full)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,kind,dense_fraction", [(2, "contiguous", 2.0), (2, "zigzag", 2.0), (4, "zigzag", 2.0),
                                                       (2, "zigzag", 0.0)])   # 0.0: always the all-gather fallback
def test_remote_chunk_exchange(world, kind, dense_fraction):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), kind, dense_fraction, out), nprocs=world, join=True)
    assert all(out.get(r) is True for r in range(world)), dict(out)


def test_partition_balances_causal_work():
    from hils_attention_b200.parallel import SeqPartition
    part = SeqPartition(4, "zigzag")
    assert sorted(b for r in range(4) for b in part.blocks(r)) == list(range(8))
    assert all(part.owner(b) == r for r in range(4) for b in part.blocks(r))
    # candidate chunks scored by a rank are proportional to the sum of its blocks' positions: equal on every rank
    assert len({sum(part.blocks(r)) for r in range(4)}) == 1


def _grad_worker(rank, world, port, dense_fraction, out):
    """Backward of the three exchanges against autograd on the unsharded tensors (gradients all-reduced)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hils_attention_b200.parallel import SeqPartition, _FetchChunks, _GatherChunks, _Halo, plan_fetch
        part = SeqPartition(world, "zigzag")
        g = torch.Generator().manual_seed(17)
        B, nbk, S, h, D, K = 2, 3, 4, 2, 8, 5
        N = nbk * part.n_blocks
        n_local = nbk * part.blocks_per_rank
        L = n_local * S
        ok = True
        # ---- tile fetch: loss_r = sum over my ids of <stage[b, slot, :, h], U[b, l, h, k]>
        k_full = torch.randn(B, N, S, h, D, generator=g, dtype=torch.float64)
        idx = torch.randint(-1, N, (world, B, L, h, K), generator=g, dtype=torch.int32)[rank]
        U = torch.randn(world, B, L, h, K, S, D, generator=g, dtype=torch.float64)[rank]
        plan = plan_fetch(idx, N, part, dense_fraction=dense_fraction)
        x = part.shard(k_full, rank).clone().requires_grad_(True)
        stage = _FetchChunks.apply(x, plan, None)
        valid = idx >= 0
        bb = torch.arange(B).view(B, 1, 1, 1).expand_as(idx)
        hh = torch.arange(h).view(1, 1, h, 1).expand_as(idx)
        picked = stage[bb, plan.remapped.clamp_min(0).long(), :, hh, :]            # (B, L, h, K, S, D)
        (picked * U * valid[..., None, None]).sum().backward()
        kf = k_full.clone().requires_grad_(True)
        ref = kf[bb, idx.clamp_min(0).long(), :, hh, :]
        (ref * U * valid[..., None, None]).sum().backward()
        gref = kf.grad.clone()
        dist.all_reduce(gref)
        ok &= torch.allclose(x.grad, part.shard(gref, rank), atol=1e-10)
        # ---- chunk-key all-gather
        lk_full = torch.randn(B, N, h, D, generator=g, dtype=torch.float64)
        Wt = torch.randn(world, B, N, h, D, generator=g, dtype=torch.float64)
        xl = part.shard(lk_full, rank).clone().requires_grad_(True)
        y = _GatherChunks.apply(xl, part, None)
        ok &= torch.equal(y.detach(), lk_full)
        (y * Wt[rank]).sum().backward()
        ok &= torch.allclose(xl.grad, part.shard(Wt.sum(0), rank), atol=1e-10)
        # ---- halo: loss_r = <halos, V_r>; the gradient lands on the tail of the block each halo came from
        T = N * S
        halo = 5
        x_full = torch.randn(B, T, h, D, generator=g, dtype=torch.float64)
        V = torch.randn(world, B, part.blocks_per_rank * halo, h, D, generator=g, dtype=torch.float64)
        xs = part.shard(x_full, rank).clone().requires_grad_(True)
        hal = _Halo.apply(xs, part, halo, None)
        (hal * V[rank]).sum().backward()
        tb = T // part.n_blocks
        gfull = torch.zeros_like(x_full)
        for r in range(world):
            for i, blk in enumerate(part.blocks(r)):
                if blk > 0:
                    gfull[:, blk * tb - halo:blk * tb] += V[r][:, i * halo:(i + 1) * halo]
        ok &= torch.allclose(xs.grad, part.shard(gfull, rank), atol=1e-10)
        for i, blk in enumerate(part.blocks(rank)):
            want = x_full[:, blk * tb - halo:blk * tb] if blk > 0 else torch.zeros(B, halo, h, D, dtype=torch.float64)
            ok &= torch.equal(hal.detach()[:, i * halo:(i + 1) * halo], want)
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dense_fraction", [2.0, 0.0])
def test_exchanges_are_differentiable(dense_fraction):
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_grad_worker, args=(world, _free_port(), dense_fraction, out), nprocs=world, join=True)
    assert all(out.get(r) is True for r in range(world)), dict(out)
