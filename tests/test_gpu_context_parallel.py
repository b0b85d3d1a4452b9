"""Context-parallel forward on 2 GPUs (NCCL) against the single-GPU chain on the full sequence.
Skipped when fewer than two GPUs are visible."""
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


def _inputs():
    g = torch.Generator().manual_seed(12)
    B, T, hq, hk, D, S = 1, 4096, 4, 2, 64, 64
    q = torch.randn(B, T, hq, D, generator=g)
    k = torch.randn(B, T, hk, D, generator=g)
    k += (torch.randn(B, T // S, 1, hk, D, generator=g) * 0.5).expand(-1, -1, S, -1, -1).reshape(B, T, hk, D)
    v = torch.randn(B, T, hk, D, generator=g)
    return [t.to(torch.bfloat16) for t in (q, k, v)], (hq, hk, S, 256, 8)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from hils_attention_b200.attention import HiLSAttentionConfig, HiLSAttentionCore
        from hils_attention_b200.parallel import context_parallel_forward
        (q, k, v), (hq, hk, S, W, K) = _inputs()
        T = q.shape[1]
        Tl = T // world
        sl = slice(rank * Tl, (rank + 1) * Tl)
        qd, kd, vd = (t[:, sl].cuda().contiguous() for t in (q, k, v))
        with torch.no_grad():
            o, aux = context_parallel_forward(qd, kd, vd, qd, h_kv=hk, topk=K, chunk_size=S, window_size=W,
                                              return_aux=True)
            core = HiLSAttentionCore(HiLSAttentionConfig(hq, hk, K, S, W)).eval()
            full, faux = core(q.cuda(), k.cuda(), v.cuda(), q.cuda(), return_aux=True)
        same = (aux["indices"] == faux["indices"][:, sl]).all(-1)
        rows = same.repeat_interleave(hq // hk, dim=2)
        err = (o.float() - full[:, sl].float())[rows].abs().max().item()
        out[rank] = (float(same.float().mean()), err, aux["remote_chunks"])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_context_parallel_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    for r in range(world):
        match, err, n_remote = out[r]
        assert match >= 0.99, (r, match)
        assert err < 3e-2, (r, err)
    assert out[0][2] == 0 and all(out[r][2] > 0 for r in range(1, world))   # only later ranks fetch remote chunks
