"""Prefill -> decode through the paged K/V store on sequences of different lengths, against the same tokens
run as one full sequence (itself checked against the oracle chain in test_gpu_chain.py) and against the
oracle chain directly.  Needs a B200."""
import pytest
import torch

from oracle import hils_oracle as orc
from tests.test_gpu_chain import _core, _inputs
from tests.util import check

pytestmark = pytest.mark.gpu
BF, F32 = torch.bfloat16, torch.float32
S, K, W = 64, 4, 128


def _sequence(T, hq, hk, D, seed, dtype):
    q, k, v = _inputs(1, T, hq, hk, D, S, seed, dtype)
    lq = torch.randn(q.shape, generator=torch.Generator().manual_seed(seed + 1000)).to(dtype)
    return [t.cuda() for t in (q, k, v, lq)]


def _prefill(core, store, seq, T0):
    """Run the first T0 tokens as an ordinary forward and move their K/V and pooled chunk keys into the store."""
    q, k, v, lq = seq
    slot = store.allocate(T0)
    if T0 >= S:
        _, aux = core(q[:, :T0], k[:, :T0], v[:, :T0], lq[:, :T0], return_aux=True)
        store.write_prefill(slot, 0, k[0, :T0], v[0, :T0], aux["lmk_k"][0], aux["prior_b"][0])
    else:
        store.write_prefill(slot, 0, k[0, :T0], v[0, :T0])
    return slot


def _decode(core, store, live, steps, got):
    """`steps` decode steps of the sequences in `live` = {slot: (seq, position)}; outputs appended to got[slot]."""
    hq, hk, D = core.h_q, core.h_kv, next(iter(live.values()))[0][0].shape[-1]
    dtype = next(iter(live.values()))[0][0].dtype
    for _ in range(steps):
        B = store.batch
        qs, ls = (torch.zeros(B, 1, hq, D, dtype=dtype, device="cuda") for _ in range(2))
        ks, vs = (torch.zeros(B, 1, hk, D, dtype=dtype, device="cuda") for _ in range(2))
        for slot, (seq, pos) in live.items():
            qs[slot], ks[slot], vs[slot], ls[slot] = seq[0][0, pos:pos + 1], seq[1][0, pos:pos + 1], seq[2][0, pos:pos + 1], seq[3][0, pos:pos + 1]
        store.begin_step()
        o, idx = core.decode_paged(qs, ks, vs, ls, store, return_indices=True)
        store.end_step()
        for slot, (seq, pos) in list(live.items()):
            got[slot].append((pos, o[slot, 0].clone(), idx[slot, 0].clone()))
            live[slot] = (seq, pos + 1)


def _compare(core, seq, rec, dtype, what):
    """Outputs of the decode steps in rec = [(position, o, ids)] against the whole sequence run at once."""
    q, k, v, lq = seq
    T = max(p for p, _, _ in rec) + 1
    full, faux = core(q[:, :T], k[:, :T], v[:, :T], lq[:, :T], return_aux=True)
    pos = torch.tensor([p for p, _, _ in rec], device="cuda")
    o = torch.stack([x for _, x, _ in rec])                               # (n, hq, D)
    ids = torch.stack([x for _, _, x in rec])                             # (n, hk, K)
    if T >= S:
        same = (ids == faux["indices"][0, pos]).all(-1)                   # (n, hk)
        assert same.float().mean().item() >= 0.97, what
        rows = same.repeat_interleave(core.h_q // core.h_kv, dim=1)
    else:
        rows = torch.ones(o.shape[:2], dtype=torch.bool, device="cuda")
    check(o[rows], full[0, pos][rows], dtype, what)
    return full, faux


@pytest.mark.parametrize("cfg", [
    # hq, hk, D, dtype, pages per sequence, module options
    (4, 2, 64, BF, 512, dict()),                              # N >= 512: the streamed-keys selection, per-q-head chunk keys
    (4, 4, 128, BF, 16, dict()),
    (2, 2, 64, F32, 16, dict()),
    (4, 2, 64, BF, 16, dict(enable_chunk_pooling=True, enable_softmax1=True)),   # mean-pooled keys on the kv heads
])
def test_ragged_prefill_then_decode_matches_the_full_sequence(cfg):
    from hils_attention_b200 import _lib
    from hils_attention_b200.kv_store import PagedKVStore
    hq, hk, D, dtype, max_pages, kw = cfg
    core = _core(hq, hk, K, S, W, **kw).eval()
    h_lmk = hk if kw.get("enable_chunk_pooling") else hq
    store = PagedKVStore(64, 3, max_pages, hk, D, hq, h_lmk=h_lmk, dtype=dtype, device="cuda")
    T0 = [640, 300, 50]                                        # the last one starts inside its first chunk
    n1, n2, n3 = 70, 3, 12
    seqs = [_sequence(t0 + n1 + n2 + n3, hq, hk, D, 70 + i, dtype) for i, t0 in enumerate(T0)]
    newcomer = _sequence(200 + n3, hq, hk, D, 90, dtype)
    with torch.no_grad():
        slots = [_prefill(core, store, s, t0) for s, t0 in zip(seqs, T0)]
        assert slots == [0, 1, 2]
        live = {b: (seqs[b], T0[b]) for b in slots}
        got = {b: [] for b in slots}
        _decode(core, store, live, n1, got)                    # every sequence crosses a page boundary
        # the middle sequence ends: its row stays in the batch, inactive, for a few steps ...
        store.release(1)
        finished = got.pop(1)
        del live[1]
        _decode(core, store, live, n2, got)
        # ... then a new sequence takes the slot and the freed pages
        assert _prefill(core, store, newcomer, 200) == 1
        live[1], got[1] = (newcomer, 200), []
        _decode(core, store, live, n3, got)
        for b, seq in ((0, seqs[0]), (2, seqs[2]), (1, newcomer)):
            _compare(core, seq, got[b], dtype, f"paged decode, slot {b}")
        _compare(core, seqs[1], finished, dtype, "paged decode, released sequence")
        # the store holds exactly the tokens that were fed, page by page
        for b, seq in ((0, seqs[0]), (2, seqs[2]), (1, newcomer)):
            gk, gv = store.gather(b)
            T = store.length(b)
            assert T == live[b][1] and torch.equal(gk, seq[1][0, :T]) and torch.equal(gv, seq[2][0, :T])
    assert _lib.query("hils_take_device_status") == 0


def test_paged_decode_against_the_oracle_chain():
    """Two sequences of different lengths, bf16: the last decoded token of each against the CPU oracle chain."""
    from hils_attention_b200.kv_store import PagedKVStore
    hq, hk, D = 4, 2, 64
    core = _core(hq, hk, K, S, W).eval()
    store = PagedKVStore(32, 2, 16, hk, D, hq, dtype=BF, device="cuda")
    T0, n = [500, 190], 40
    seqs = [_sequence(t0 + n, hq, hk, D, 120 + i, BF) for i, t0 in enumerate(T0)]
    with torch.no_grad():
        for s, t0 in zip(seqs, T0):
            _prefill(core, store, s, t0)
        live = {b: (seqs[b], T0[b]) for b in range(2)}
        got = {0: [], 1: []}
        _decode(core, store, live, n, got)
    for b in range(2):
        q, k, v, lq = (t.cpu() for t in seqs[b])
        ref, raux = orc.hils_attention_chain(q, k, v, lq, chunk_size=S, window_size=W, topk=K, pooling="attn",
                                             use_prior_bias=True, softmax1=False, return_aux=True)
        pos = torch.tensor([p for p, _, _ in got[b]])
        o = torch.stack([x for _, x, _ in got[b]]).cpu()
        ids = torch.stack([x for _, _, x in got[b]]).cpu()
        same = (ids == raux["indices"][0, pos]).all(-1)
        assert same.float().mean().item() >= 0.95
        rows = same.repeat_interleave(hq // hk, dim=1)
        check(o[rows], ref.float()[0, pos][rows], BF, f"paged decode vs oracle, sequence {b}")


def test_a_page_id_outside_the_pool_is_skipped_and_reported():
    """A corrupted page table must not make a kernel read outside the pool: the access is skipped and the status
    word says so."""
    from hils_attention_b200 import _lib, ops
    hq, hk, D, N = 2, 2, 64, 16
    g = torch.Generator().manual_seed(3)
    mk = lambda *s: torch.randn(*s, generator=g).to(BF).cuda()
    k_pages, v_pages = mk(8, hk, 64, D), mk(8, hk, 64, D)
    table = torch.tensor([[1, 2, 99, 3] + [0] * 12], dtype=torch.int32, device="cuda")     # chunk 2 points nowhere
    lens = torch.tensor([250], dtype=torch.int32, device="cuda")
    o, _ = ops.decode_step_paged(mk(1, hq, D), mk(1, hq, D), mk(1, hk, D), mk(1, hk, D), k_pages, v_pages, table, lens, 250,
                                 mk(1, N, hq, D), torch.zeros(1, N, hq, device="cuda"), K, S, W)
    torch.cuda.synchronize()
    assert torch.isfinite(o.float()).all()
    assert _lib.query("hils_take_device_status") // 1000000 == 8
    assert _lib.query("hils_take_device_status") == 0
