"""Host-side logic of the context-parallel path on CPU: two gloo ranks exchange the K/V tiles of the
remote chunks they selected; the staged tiles and the rewritten ids must reproduce a gather from the
full (unsharded) tensors.  Also the halo exchange of the sliding-window branch."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hils_attention_b200.parallel import exchange_chunks, exchange_halo, plan_remote_chunks
        g = torch.Generator().manual_seed(5)
        B, Nl, S, h, D, L, K = 2, 6, 4, 2, 8, 10, 5
        N = Nl * world
        k_full = torch.randn(B, N, S, h, D, generator=g)
        v_full = torch.randn(B, N, S, h, D, generator=g)
        idx = torch.randint(-1, N, (world, B, L, h, K), generator=g, dtype=torch.int32)[rank]
        kc, vc = k_full[:, rank * Nl:(rank + 1) * Nl], v_full[:, rank * Nl:(rank + 1) * Nl]
        remote, remapped = plan_remote_chunks(idx, rank * Nl, Nl)
        assert bool(((remote < rank * Nl) | (remote >= (rank + 1) * Nl)).all())
        rk, rv = exchange_chunks(kc, vc, remote, Nl)
        k_stage, v_stage = torch.cat([rk, kc], 1), torch.cat([rv, vc], 1)
        ok = True
        for b in range(B):
            for l in range(L):
                for hh in range(h):
                    for kk in range(K):
                        c, s = int(idx[b, l, hh, kk]), int(remapped[b, l, hh, kk])
                        if c < 0:
                            ok &= s == -1
                        else:
                            ok &= torch.equal(k_stage[b, s, :, hh], k_full[b, c, :, hh])
                            ok &= torch.equal(v_stage[b, s, :, hh], v_full[b, c, :, hh])
        x = torch.arange(B * 12 * h * D, dtype=torch.float32).view(B, 12, h, D) + 1000 * rank
        halo = exchange_halo(x, 5)
        if rank == 0:
            ok &= halo is None
        else:
            ok &= torch.equal(halo, (x - 1000)[:, -5:])
        out[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_remote_chunk_exchange_two_ranks():
    world = 2
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out.get(0) is True and out.get(1) is True


def test_plan_without_remote_chunks():
    from hils_attention_b200.parallel import plan_remote_chunks
    idx = torch.tensor([[[[4, 6, -1]]]], dtype=torch.int32)
    remote, remapped = plan_remote_chunks(idx, 4, 4)
    assert remote.numel() == 0
    assert remapped.tolist() == [[[[0, 2, -1]]]]
