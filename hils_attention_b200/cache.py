"""KV store of the HiLS layers for prefill, chunk-prefill and decode.

Keeps the interface of the reference's ``HiLSDynamicLayer`` (utils/hils_cache_utils.py:9-76):
``update(k, v) -> (K_all, V_all)`` in (B, T, H, D) layout, ``get_seq_length``, ``get_mask_sizes``,
``get_max_cache_shape``, attributes ``keys`` / ``values``.  Differences, both on purpose:

* storage is preallocated, token-major and grows geometrically, so appending a token copies only
  that token (the reference re-allocates the whole cache with torch.cat on every step, :61-62), and
  the store doubles as a contiguous (1, T, B*H, D) tensor for the kernels;
* nothing is ever moved to host memory: a B200 holds the 128K-token, 32-head, D=128 cache
  (68.7 GB per layer for 32 sequences) in HBM, where the reference starts a CPU round trip
  (:19-23, :45-59).

``HiLSCache`` is the small ``past_key_values`` object the attention chain needs: per-layer
``update`` plus the ``_hils_prior_cache`` dictionary that holds the pooled chunk keys and their
bias between steps (models/FlashHiLS/hils_attention.py:364-410, :450-456).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

try:  # keep isinstance checks of HF code working when transformers is present
    from transformers.cache_utils import CacheLayerMixin as _Base
except Exception:  # pragma: no cover - transformers is optional
    class _Base:  # type: ignore
        def __init__(self, *a, **k):
            pass


class HiLSDynamicLayer(_Base):
    """Append-only K/V store of one HiLS layer.

    Storage is token-major, ``(capacity, B, H, D)``: appending tokens writes only the new rows, and
    the whole store is at the same time a contiguous ``(1, T, B*H, D)`` tensor - batch folded into the
    head dimension - which is what the kernels consume during decode (every stage of the path is
    independent per (batch, head), so a batch of sequences is just more heads).  ``update`` still
    returns the reference's ``(B, T, H, D)`` tensors, as zero-copy permuted views.
    """
    is_sliding = False

    def __init__(self, initial_capacity: int = 0, growth: float = 2.0):
        try:
            super().__init__()
        except TypeError:
            pass
        self.is_initialized = False
        self._capacity_hint = int(initial_capacity)
        self._growth = float(growth)
        self._len = 0
        self._kbuf: Optional[torch.Tensor] = None     # (capacity, B, H, D)
        self._vbuf: Optional[torch.Tensor] = None
        self.keys: Optional[torch.Tensor] = None
        self.values: Optional[torch.Tensor] = None

    def lazy_initialization(self, key_states: torch.Tensor, value_states: torch.Tensor = None) -> None:
        self.dtype, self.device = key_states.dtype, key_states.device
        self.is_initialized = True
        self._len = 0

    def _reserve(self, k: torch.Tensor, v: torch.Tensor, need: int) -> None:
        cap = 0 if self._kbuf is None else self._kbuf.shape[0]
        if need <= cap:
            return
        new_cap = max(need, int(cap * self._growth), self._capacity_hint, 64)
        B, _, H, D = k.shape
        kb = torch.empty((new_cap, B, H, D), dtype=k.dtype, device=k.device)
        vb = torch.empty((new_cap, B, v.shape[2], v.shape[3]), dtype=v.dtype, device=v.device)
        if self._len:
            kb[:self._len].copy_(self._kbuf[:self._len])
            vb[:self._len].copy_(self._vbuf[:self._len])
        self._kbuf, self._vbuf = kb, vb

    def adopt(self, kbuf: torch.Tensor, vbuf: torch.Tensor, length: int) -> None:
        """Take ownership of preallocated token-major buffers (capacity, B, H, D) already holding
        `length` tokens (used to set up long caches without a second copy)."""
        self.lazy_initialization(kbuf)
        self._kbuf, self._vbuf, self._len = kbuf, vbuf, int(length)
        self._publish()

    def _publish(self) -> None:
        self.keys = self._kbuf[:self._len].permute(1, 0, 2, 3)
        self.values = self._vbuf[:self._len].permute(1, 0, 2, 3)

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs
               ) -> Tuple[torch.Tensor, torch.Tensor]:
        if not self.is_initialized:
            self.lazy_initialization(key_states, value_states)
        n = key_states.shape[1]
        self._reserve(key_states, value_states, self._len + n)
        self._kbuf[self._len:self._len + n].copy_(key_states.transpose(0, 1))
        self._vbuf[self._len:self._len + n].copy_(value_states.transpose(0, 1))
        self._len += n
        self._publish()
        return self.keys, self.values

    def folded(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """The store as contiguous (1, T, B*H, D) tensors (batch folded into heads), zero-copy."""
        T = self._len
        kb, vb = self._kbuf[:T], self._vbuf[:T]
        return (kb.reshape(1, T, kb.shape[1] * kb.shape[2], kb.shape[3]),
                vb.reshape(1, T, vb.shape[1] * vb.shape[2], vb.shape[3]))

    def get_seq_length(self, *args, **kwargs) -> int:
        return self._len if self.is_initialized else 0

    def get_mask_sizes(self, cache_position_or_len, *args) -> Tuple[int, int]:
        q_len = cache_position_or_len if isinstance(cache_position_or_len, int) else int(cache_position_or_len.shape[0])
        return self.get_seq_length() + q_len, 0

    def get_max_cache_shape(self) -> int:
        return -1


class HiLSCache:
    """Minimal ``past_key_values`` for the attention chain: one HiLSDynamicLayer per cache index."""

    def __init__(self, initial_capacity: int = 0):
        self._layers: Dict[int, HiLSDynamicLayer] = {}
        self._initial_capacity = initial_capacity
        self._hils_prior_cache: Dict[int, dict] = {}

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        layer = self._layers.get(layer_idx)
        if layer is None:
            layer = self._layers[layer_idx] = HiLSDynamicLayer(self._initial_capacity)
        return layer.update(key_states, value_states, cache_kwargs)

    def layer(self, layer_idx: int) -> HiLSDynamicLayer:
        lay = self._layers.get(layer_idx)
        if lay is None:
            lay = self._layers[layer_idx] = HiLSDynamicLayer(self._initial_capacity)
        return lay

    def get_seq_length(self, layer_idx: int = 0) -> int:
        layer = self._layers.get(layer_idx)
        return 0 if layer is None else layer.get_seq_length()
