"""Context-parallel forward on 2, 4 and 8 GPUs (NCCL) against the single-GPU chain on the full sequence, for the
contiguous and the zig-zag partition.  Skipped when fewer GPUs are visible than ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _inputs(T):
    g = torch.Generator().manual_seed(12)
    # the long case has one query head per kv head: its selection runs the long-candidate-list kernel at an offset
    B, hq, hk, D, S = 1, (2 if T >= 65536 else 4), 2, 64, 64
    q = torch.randn(B, T, hq, D, generator=g)
    k = torch.randn(B, T, hk, D, generator=g)
    k += (torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5).expand(-1, -1, S, -1, -1).reshape(B, T, hk, D)
    v = torch.randn(B, T, hk, D, generator=g)
    return [t.to(torch.bfloat16) for t in (q, k, v)], (hq, hk, S, 256, 8)


def _worker(rank, world, port, kind, T, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
        from hils_attention_b200.parallel import SeqPartition, context_parallel_forward
        (q, k, v), (hq, hk, S, W, K) = _inputs(T)
        part = SeqPartition(world, kind)
        qd, kd, vd = (part.shard(t, rank).cuda().contiguous() for t in (q, k, v))
        with torch.no_grad():
            o, aux = context_parallel_forward(qd, kd, vd, qd, h_kv=hk, topk=K, chunk_size=S, window_size=W,
                                              partition=kind, return_aux=True)
            core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).eval()
            full, faux = core(q.cuda(), k.cuda(), v.cuda(), q.cuda(), return_aux=True)
        same = (aux["indices"] == part.shard(faux["indices"], rank)).all(-1)
        rows = same.repeat_interleave(hq // hk, dim=2)
        err = (o.float() - part.shard(full, rank).float())[rows].abs().max().item()
        out[rank] = (float(same.float().mean()), err, aux["remote_tiles"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,kind,T", [(2, "contiguous", 4096), (2, "zigzag", 65536), (4, "zigzag", 4096),
                                          (8, "zigzag", 8192)])
def test_context_parallel_matches_single_gpu(world, kind, T):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), kind, T, out), nprocs=world, join=True)
    for r in range(world):
        match, err, n_remote = out[r]
        assert match >= 0.99, (r, match)
        assert err < 2e-2, (r, err)
        assert n_remote > 0 or (kind == "contiguous" and r == 0)   # only the first contiguous shard fetches nothing


def _train_worker(rank, world, port, kind, T, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
        from hils_attention_b200.parallel import SeqPartition, context_parallel_forward
        (q, k, v), (hq, hk, S, W, K) = _inputs(T)
        do = torch.randn(q.shape, generator=torch.Generator().manual_seed(99)).to(torch.bfloat16)
        part = SeqPartition(world, kind)
        qd, kd, vd = (part.shard(t, rank).cuda().contiguous().requires_grad_(True) for t in (q, k, v))
        o, aux = context_parallel_forward(qd, kd, vd, qd, h_kv=hk, topk=K, chunk_size=S, window_size=W, partition=kind,
                                          return_aux=True, training=True)
        o.backward(part.shard(do, rank).cuda())
        core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).train()
        qf, kf, vf = (t.cuda().requires_grad_(True) for t in (q, k, v))
        full, faux = core(qf, kf, vf, qf, return_aux=True)
        full.backward(do.cuda())
        same = float((aux["indices"] == part.shard(faux["indices"], rank)).all(-1).float().mean())
        errs = {}
        for name, a, b in (("o", o, part.shard(full, rank)), ("dq", qd.grad, part.shard(qf.grad, rank)),
                           ("dk", kd.grad, part.shard(kf.grad, rank)), ("dv", vd.grad, part.shard(vf.grad, rank))):
            ref = b.float()
            errs[name] = float(((a.float() - ref).abs().max() / max(1.0, float(ref.abs().max()))))
        out[rank] = (same, errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,kind,T", [(2, "zigzag", 4096), (4, "zigzag", 8192)])
def test_context_parallel_backward_matches_single_gpu(world, kind, T):
    """Gradients of the sequence-sharded chain (reverse exchanges included) equal the single-GPU chain's, shard by shard."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_train_worker, args=(world, _free_port(), kind, T, out), nprocs=world, join=True)
    for r in range(world):
        same, errs = out[r]
        assert same >= 0.999, (r, same)          # identical selections: the gradients are then comparable element by element
        for name, e in errs.items():
            assert e < 2e-2, (r, name, e)
