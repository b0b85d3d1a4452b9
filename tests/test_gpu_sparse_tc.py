"""Tensor-core (tcgen05) sparse chunk attention against the CPU oracle: bf16, chunk 64, head dims
64 and 128, MHA and GQA, ragged lengths, unsorted and duplicated ids, kv longer than q."""
import pytest
import torch

from oracle import hils_oracle as orc
from tests.util import check

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _case(B, L, T, H, G, D, K, seed, sort=True, dup=False):
    g = torch.Generator().manual_seed(seed)
    S = 64
    N = T // S
    q = torch.randn(B, L, H * G, D, generator=g).to(BF)
    k = torch.randn(B, T, H, D, generator=g).to(BF)
    v = torch.randn(B, T, H, D, generator=g).to(BF)
    idx = torch.full((B, L, H, K), -1, dtype=torch.int32)
    for b in range(B):
        for t in range(L):
            lim = min((t + (T - L)) // S + 1, N)
            for h in range(H):
                n = min(K, lim, int(torch.randint(0, K + 1, (1,), generator=g)))
                sel = torch.randperm(lim, generator=g)[:n]
                if sort:
                    sel = sel.sort()[0]
                idx[b, t, h, :n] = sel.to(torch.int32)
                if dup and n >= 2:
                    idx[b, t, h, 1] = idx[b, t, h, 0]
    w = torch.rand(B, L, H * G, K + 1, generator=g).to(BF)
    return q, k, v, w, idx


@pytest.mark.parametrize("cfg", [
    # B, L, T, H, G, D, K, sort, dup
    (1, 512, 512, 2, 1, 64, 8, True, False),
    (2, 300, 300, 1, 2, 64, 4, True, False),       # ragged block, GQA
    (1, 256, 640, 2, 8, 64, 4, True, False),       # kv longer than q, G=8
    (1, 384, 384, 1, 1, 128, 8, True, False),      # head dim 128
    (1, 200, 512, 2, 4, 128, 4, True, True),       # duplicates add their weights
    (1, 256, 256, 1, 2, 64, 4, False, False),      # unsorted lists (naive block-sparse path)
    (1, 1024, 1024, 1, 1, 64, 32, True, False),    # K=32 as in the benchmark
])
def test_tc_forward_matches_oracle(cfg):
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    B, L, T, H, G, D, K, sort, dup = cfg
    q, k, v, w, idx = _case(B, L, T, H, G, D, K, 77, sort, dup)
    ref = orc.sparse_attn(q, k, v, w, idx, chunk_size=64, mask_last_token=True)
    o = hb.HiLS_block_M_head(q.cuda(), k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=64, is_training=False)
    assert _lib.load().hils_take_device_status() == 0
    check(o, ref, BF, "tc forward")


def test_tc_forward_slope_and_no_last_mask():
    import hils_attention_b200 as hb
    q, k, v, w, idx = _case(1, 256, 256, 1, 2, 64, 4, 5)
    slope = torch.tensor([0.02, 0.1])
    ref = orc.sparse_attn(q, k, v, w, idx, chunk_size=64, mask_last_token=False, slope=slope)
    o = hb.HiLS_block_M_head(q.cuda(), k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=64,
                             mask_last_token=False, is_training=False, slope=slope.cuda())
    check(o, ref, BF, "tc forward slope")


def test_tc_forward_is_deterministic():
    """Dense selections (few chunks per selected slot) run the query-block-major kernel, which sums in a fixed order."""
    import hils_attention_b200 as hb
    q, k, v, w, idx = [t.cuda() for t in _case(1, 512, 512, 2, 1, 64, 8, 9)]
    o1 = hb.HiLS_block_M_head(q, k, v, w, idx, block_size=64, is_training=False)
    o2 = hb.HiLS_block_M_head(q, k, v, w, idx, block_size=64, is_training=False)
    assert torch.equal(o1, o2)


def test_chunk_major_forward_matches_oracle_on_sparse_selections():
    """Many candidate chunks per selected slot (64 chunks, 4 slots): the chunk-major forward kernel (inverse index,
    gathered owner rows, fp32 scatter-add of the slots' partial outputs)."""
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    for (B, L, T, H, G, D, K) in [(1, 4096, 4096, 2, 1, 64, 4), (2, 2100, 4096, 1, 4, 128, 8)]:
        q, k, v, w, idx = _case(B, L, T, H, G, D, K, 55)
        ref = orc.sparse_attn(q, k, v, w, idx, chunk_size=64, mask_last_token=True)
        o = hb.HiLS_block_M_head(q.cuda(), k.cuda(), v.cuda(), w.cuda(), idx.cuda(), block_size=64, is_training=False)
        assert _lib.load().hils_take_device_status() == 0
        check(o, ref, BF, "chunk-major forward")


@pytest.mark.parametrize("cfg", [
    (1, 512, 512, 2, 1, 64, 8, True, False),
    (2, 300, 300, 1, 2, 64, 4, True, False),
    (1, 256, 640, 2, 8, 64, 4, True, False),
    (1, 384, 384, 1, 1, 128, 8, True, False),
    (1, 200, 512, 2, 4, 128, 4, True, True),
    (1, 256, 256, 1, 2, 64, 4, False, False),
    (1, 1024, 1024, 1, 1, 64, 32, True, False),
])
def test_tc_backward_matches_oracle(cfg):
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    B, L, T, H, G, D, K, sort, dup = cfg
    q, k, v, w, idx = _case(B, L, T, H, G, D, K, 91, sort, dup)
    do = torch.randn(B, L, H * G, D, generator=torch.Generator().manual_seed(3)).to(BF)
    qr, kr, vr, wr = [t.float().requires_grad_(True) for t in (q, k, v, w)]
    ref = orc.sparse_attn(qr, kr, vr, wr, idx, chunk_size=64, mask_last_token=True)
    ref.backward(do.float())
    qd, kd, vd, wd = [t.cuda().requires_grad_(True) for t in (q, k, v, w)]
    o = hb.HiLS_block_M_head(qd, kd, vd, wd, idx.cuda(), block_size=64)
    o.backward(do.cuda())
    assert _lib.load().hils_take_device_status() == 0
    check(o, ref, BF, "o")
    # gradients sum up to K*64 bf16-rounded products per element: compare at the size of the tensor
    for name, a, r in (("dq", qd, qr), ("dk", kd, kr), ("dv", vd, vr), ("dw", wd, wr)):
        check(a.grad, r.grad, BF, name)
        err = (a.grad.float().cpu() - r.grad).square().mean().sqrt() / r.grad.square().mean().sqrt().clamp_min(1e-20)
        assert float(err) < 2e-2, (name, float(err))
    assert float(wd.grad[..., K:].float().abs().max()) == 0.0


def test_tc_backward_is_deterministic():
    """dK, dV and dW come out bit-identical from run to run: they are summed inside one CTA per chunk in the order of
    the inverse index.  dQ is the sum of a token's slot contributions added to an fp32 accumulator in global memory in
    whatever order the chunks' CTAs reach it; two runs agree to fp32 rounding of at most K terms."""
    import hils_attention_b200 as hb
    q, k, v, w, idx = [t.cuda() for t in _case(1, 512, 512, 2, 2, 64, 8, 19)]
    do = torch.randn(q.shape, generator=torch.Generator().manual_seed(4)).to(BF).cuda()
    grads = []
    for _ in range(2):
        qd, kd, vd, wd = [t.clone().requires_grad_(True) for t in (q, k, v, w)]
        hb.HiLS_block_M_head(qd, kd, vd, wd, idx, block_size=64).backward(do)
        grads.append([t.grad.clone() for t in (qd, kd, vd, wd)])
    (dq1, dk1, dv1, dw1), (dq2, dk2, dv2, dw2) = grads
    assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2) and torch.equal(dw1, dw2)
    assert float((dq1.float() - dq2.float()).abs().max()) <= 2 ** -7 * float(dq1.float().abs().max())


def test_misaligned_tensors_are_refused_before_any_launch():
    """A bf16 tensor that starts 2 bytes into its buffer can feed neither the TMA tiles nor the vector loads of the
    generic kernels: the host layer refuses it with an error before anything is launched, and so does the C entry
    point for callers that bypass the host layer."""
    import ctypes
    import hils_attention_b200 as hb
    from hils_attention_b200 import _lib
    q, k, v, w, idx = _case(1, 256, 256, 2, 1, 64, 4, 7)
    buf = torch.empty(q.numel() + 1, dtype=BF, device="cuda")
    q_off = buf[1:].view(q.shape)
    q_off.copy_(q)
    assert q_off.data_ptr() % 16 != 0 and q_off.is_contiguous()
    kd, vd, wd, idd = k.cuda(), v.cuda(), w.cuda(), idx.cuda()
    with pytest.raises(ValueError, match="16-byte aligned"):
        hb.HiLS_block_M_head(q_off, kd, vd, wd, idd, block_size=64, is_training=False)
    o = torch.empty_like(q_off.clone())
    lib = _lib.load()
    rc = lib.hils_sparse_attn_fwd(q_off.data_ptr(), kd.data_ptr(), vd.data_ptr(), wd.data_ptr(), idd.data_ptr(), None,
                                  o.data_ptr(), 1, 256, 256, 2, 2, 64, 64, 4, 5, 64, ctypes.c_float(0.125), 1, 1, None, 0,
                                  torch.cuda.current_stream().cuda_stream)
    assert rc != 0 and b"16-byte aligned" in lib.hils_last_error()
    # the aligned call still works afterwards
    out = hb.HiLS_block_M_head(q.cuda(), kd, vd, wd, idd, block_size=64, is_training=False)
    check(out, orc.sparse_attn(q.float(), k.float(), v.float(), w.float(), idx, chunk_size=64), BF, "aligned call after a refusal")
