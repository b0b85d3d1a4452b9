"""The allocation-free selection backward (hils_topk_bwd_noalloc) against hils_topk_bwd.

Some callers cannot allocate device memory when they call the library (a frozen caching allocator,
a server that reserved everything at start-up); for them the fp32 accumulator of the chunk-key
gradient lives in a fixed array inside the library.  This file is named so that pytest collects it
last.  Both entry points are driven through the C ABI on the same inputs, twice in a row (the
built-in array keeps the previous call's contents, so the second call checks that it is cleared),
and the size limit is checked to be enforced."""
import pytest
import torch

from tests.util import check

pytestmark = pytest.mark.gpu


def _inputs(dtype, seed):
    g = torch.Generator().manual_seed(seed)
    B, L, N, h_kv, G, D, K = 2, 300, 20, 2, 2, 64, 8
    q = torch.randn(B, L, h_kv, G, D, generator=g).to(dtype).cuda()
    lm = torch.randn(B, N, h_kv, D, generator=g).to(dtype).cuda()
    ds = torch.randn(B, L, h_kv * G, K, generator=g).to(dtype).cuda()
    idx = torch.stack([torch.randperm(N, generator=g)[:K].sort()[0] for _ in range(B * L * h_kv)])
    idx = idx.view(B, L, h_kv, K).to(torch.int32)
    idx[:, ::5, :, -2:] = -1
    return (B, L, N, h_kv, G, D, K), q, lm, ds, idx.cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_noalloc_matches_allocating_entry_point_twice(dtype):
    from hils_attention_b200 import _lib
    from hils_attention_b200._lib import call, dtype_code, ptr, stream
    for rep in range(2):                                    # second call reuses the dirty scratch
        (B, L, N, h_kv, G, D, K), q, lm, ds, idx = _inputs(dtype, 100 + rep)
        dt = dtype_code(q)
        scale = D ** -0.5
        dq_ref, dl_ref = torch.empty_like(q), torch.empty_like(lm)
        acc = torch.empty(lm.shape, dtype=torch.float32, device="cuda")
        call("hils_topk_bwd", ptr(ds), ptr(idx), ptr(q), ptr(lm), ptr(dq_ref), ptr(acc), ptr(dl_ref),
             B, L, N, h_kv, G, D, K, 0, scale, dt, stream())
        dq, dl = torch.empty_like(q), torch.empty_like(lm)
        call("hils_topk_bwd_noalloc", ptr(ds), ptr(idx), ptr(q), ptr(lm), ptr(dq), ptr(dl),
             B, L, N, h_kv, G, D, K, 0, scale, dt, stream())
        torch.cuda.synchronize()
        assert torch.equal(dq, dq_ref)                       # dq has no accumulation order
        check(dl, dl_ref, dtype, f"d_lmks (call {rep})")
    assert _lib.load().hils_topk_bwd_noalloc_max_elems() == 1 << 20


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    from hils_attention_b200 import _lib
    from hils_attention_b200._lib import HilsError, call, ptr, stream
    B, L, N, h_kv, G, D, K = 1, 4, 4097, 4, 1, 64, 4         # 4097*4*64 > 2**20 elements
    z = torch.zeros(8, device="cuda")
    with pytest.raises(HilsError, match="exceeds the built-in scratch"):
        call("hils_topk_bwd_noalloc", ptr(z), ptr(z), ptr(z), ptr(z), ptr(z), ptr(z), B, L, N, h_kv, G, D, K, 0,
             1.0, _lib.F32, stream())
