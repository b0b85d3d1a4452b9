"""Host logic of the KV store (hils_attention_b200/cache.py) on CPU tensors: it keeps the contract of the
reference's HiLSDynamicLayer (utils/hils_cache_utils.py:9-76) - update() returns everything stored so far
in (B, T, H, D) layout - while storing token-major, growing geometrically and never re-copying old tokens
on append."""
import torch

from hils_attention_b200.cache import HiLSCache, HiLSDynamicLayer


def _kv(B, L, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(B, L, H, D, generator=g), torch.randn(B, L, H, D, generator=g)


def test_update_returns_all_tokens_in_reference_layout():
    layer = HiLSDynamicLayer()
    ks, vs = [], []
    for step, L in enumerate([5, 1, 1, 7, 1]):
        k, v = _kv(2, L, 3, 8, step)
        ks.append(k); vs.append(v)
        K, V = layer.update(k, v)
        assert K.shape == (2, sum(x.shape[1] for x in ks), 3, 8)
        assert torch.equal(K, torch.cat(ks, 1)) and torch.equal(V, torch.cat(vs, 1))
        assert layer.get_seq_length() == K.shape[1]
    assert layer.get_mask_sizes(4) == (layer.get_seq_length() + 4, 0)
    assert layer.get_max_cache_shape() == -1


def test_folded_view_is_zero_copy_and_batch_folds_into_heads():
    layer = HiLSDynamicLayer(initial_capacity=64)
    k, v = _kv(3, 10, 2, 4, 1)
    layer.update(k, v)
    kf, vf = layer.folded()
    assert kf.shape == (1, 10, 6, 4) and kf.is_contiguous()
    # head index of the folded view = b * H + h
    for b in range(3):
        for h in range(2):
            assert torch.equal(kf[0, :, b * 2 + h], k[b, :, h])
            assert torch.equal(vf[0, :, b * 2 + h], v[b, :, h])
    assert kf.data_ptr() == layer._kbuf.data_ptr()           # a view of the store, not a copy


def test_append_does_not_move_old_tokens_until_capacity_is_exhausted():
    layer = HiLSDynamicLayer(initial_capacity=32)
    k, v = _kv(1, 8, 1, 4, 2)
    layer.update(k, v)
    ptr = layer._kbuf.data_ptr()
    for t in range(24):                                       # fills the 32 preallocated rows
        layer.update(*_kv(1, 1, 1, 4, 10 + t))
    assert layer._kbuf.data_ptr() == ptr and layer.get_seq_length() == 32
    layer.update(*_kv(1, 1, 1, 4, 99))                        # one more: geometric growth, old tokens kept
    assert layer._kbuf.shape[0] >= 64 and layer.get_seq_length() == 33
    assert torch.equal(layer.keys[:, :8], k)


def test_adopt_takes_preallocated_buffers():
    kbuf, vbuf = torch.zeros(16, 2, 1, 4), torch.zeros(16, 2, 1, 4)
    kbuf[:5] = 1.0
    layer = HiLSDynamicLayer()
    layer.adopt(kbuf, vbuf, 5)
    assert layer.get_seq_length() == 5 and layer.keys.shape == (2, 5, 1, 4)
    k, v = _kv(2, 1, 1, 4, 3)
    K, _ = layer.update(k, v)
    assert layer._kbuf.data_ptr() == kbuf.data_ptr() and torch.equal(K[:, 5], k[:, 0])


def test_cache_keeps_one_layer_per_index_and_the_prior_store():
    cache = HiLSCache(initial_capacity=8)
    k, v = _kv(1, 3, 1, 4, 4)
    cache.update(k, v, 2)
    cache.update(k, v, 5)
    cache.update(k, v, 2)
    assert cache.get_seq_length(2) == 6 and cache.get_seq_length(5) == 3 and cache.get_seq_length(7) == 0
    assert cache.layer(2) is cache.layer(2)
    cache._hils_prior_cache[0] = {"lmk_k": k, "prior_b": None}
    assert 0 in cache._hils_prior_cache
