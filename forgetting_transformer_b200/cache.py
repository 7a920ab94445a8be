"""Generation cache for the FoX attention layer: keys, values, log forget gates and the
token-shift states of every layer.

Same role and call surface as upstream's ``FgateDynamicCache``
(model/forgetting_transformer/fgate_cache.py:4-203: ``update`` returns the whole
(key, value, log_fgate) history of the layer, ``update_shift_cache`` registers the
per-layer shift states, ``get_seq_length``, ``crop``, the batch helpers), but the storage is
not a ``torch.cat`` per generated token (which re-copies the whole history every step, O(T^2)
bytes over a generation): every layer owns one buffer ``(B, H, capacity, D)`` that grows
geometrically, a step writes its new rows in place and ``update`` returns views of the first
``length`` rows.  The views are strided (batch / head strides follow the capacity); the
attention kernels read strided ``(B, H, T, D)`` tensors through their tensor maps.
"""
from __future__ import annotations

from typing import Iterator, List, Optional, Tuple

import torch

__all__ = ["FgateCache"]


def _grown(n: int, granule: int) -> int:
    """Capacity for n rows: next power of two, at least one granule, a multiple of 128 so that
    row strides stay 16-byte multiples for every head dim."""
    cap = max(granule, 128)
    while cap < n:
        cap *= 2
    return cap


class _LayerStore:
    """One layer's buffers: k, v (B, H, cap, D) and log_fgate (B, H, cap) fp32."""

    def __init__(self) -> None:
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.g: Optional[torch.Tensor] = None
        self.length = 0

    def append(self, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, granule: int) -> None:
        B, H, T, D = k.shape
        need = self.length + T
        if self.k is None or need > self.k.shape[2]:
            cap = _grown(need, granule)
            nk = torch.empty((B, H, cap, D), dtype=k.dtype, device=k.device)
            nv = torch.empty((B, H, cap, v.shape[-1]), dtype=v.dtype, device=v.device)
            ng = torch.empty((B, H, cap), dtype=g.dtype, device=g.device)
            if self.k is not None and self.length:
                nk[:, :, :self.length].copy_(self.k[:, :, :self.length])
                nv[:, :, :self.length].copy_(self.v[:, :, :self.length])
                ng[:, :, :self.length].copy_(self.g[:, :, :self.length])
            self.k, self.v, self.g = nk, nv, ng
        self.k[:, :, self.length:need].copy_(k)
        self.v[:, :, self.length:need].copy_(v)
        self.g[:, :, self.length:need].copy_(g)
        self.length = need

    def views(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        n = self.length
        return self.k[:, :, :n], self.v[:, :, :n], self.g[:, :, :n]


class FgateCache:
    """Per-layer (key, value, log_fgate) history plus the K / V token-shift states.

    ``granule`` is the first capacity of a layer's buffers (rows); they double from there."""

    def __init__(self, granule: int = 1024) -> None:
        self._layers: List[_LayerStore] = []
        self.key_shift_cache: List[torch.Tensor] = []
        self.value_shift_cache: List[torch.Tensor] = []
        self._seen_tokens = 0
        self._granule = int(granule)

    # ---- shift states (upstream lines 40-49): one (B, hidden) tensor per layer, updated in place by ShiftLinear
    def update_shift_cache(self, key_shift_state: torch.Tensor, value_shift_state: torch.Tensor, layer_idx: int) -> None:
        assert layer_idx == len(self.key_shift_cache) == len(self.value_shift_cache)
        self.key_shift_cache.append(key_shift_state)
        self.value_shift_cache.append(value_shift_state)

    # ---- history
    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, log_fgate_states: torch.Tensor,
               layer_idx: int, cache_kwargs=None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Append (B, H, T, D) keys / values and (B, H, T) log gates of layer ``layer_idx``; returns the
        layer's whole history (upstream lines 77-116)."""
        assert log_fgate_states.ndim == 3, f"log_fgate must be (B, H, T), but get {log_fgate_states.size()}"
        assert key_states.ndim == 4 and value_states.ndim == 4
        assert layer_idx <= len(self._layers), "layers must be filled in order"
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[-2]
        if layer_idx == len(self._layers):
            self._layers.append(_LayerStore())
        self._layers[layer_idx].append(key_states, value_states, log_fgate_states, self._granule)
        return self._layers[layer_idx].views()

    def __len__(self) -> int:
        return len(self._layers)

    def __getitem__(self, layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        if layer_idx < len(self):
            return self._layers[layer_idx].views()
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}")

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]:
        for layer_idx in range(len(self)):
            yield self._layers[layer_idx].views()

    @property
    def key_cache(self) -> List[torch.Tensor]:
        return [s.views()[0] for s in self._layers]

    @property
    def value_cache(self) -> List[torch.Tensor]:
        return [s.views()[1] for s in self._layers]

    @property
    def log_fgate_cache(self) -> List[torch.Tensor]:
        return [s.views()[2] for s in self._layers]

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        if len(self._layers) <= layer_idx:
            return 0
        return self._layers[layer_idx].length

    def get_max_length(self) -> Optional[int]:
        return None

    def capacity(self, layer_idx: int = 0) -> int:
        s = self._layers[layer_idx]
        return 0 if s.k is None else s.k.shape[2]

    def to_legacy_cache(self):
        return tuple(self._layers[i].views() for i in range(len(self)))

    def crop(self, max_length: int) -> None:
        """Keep the first ``max_length`` tokens (negative: drop that many from the end); upstream lines 149-164.
        The buffers are kept, only the lengths move."""
        if max_length < 0:
            max_length = self.get_seq_length() - abs(max_length)
        if self.get_seq_length() <= max_length:
            return
        self._seen_tokens = max_length
        for s in self._layers:
            s.length = min(s.length, max_length)

    def batch_repeat_interleave(self, repeats: int) -> None:
        for s in self._layers:
            n = s.length
            s.k, s.v, s.g = [t[:, :, :n].repeat_interleave(repeats, dim=0) for t in (s.k, s.v, s.g)]
        self.key_shift_cache = [t.repeat_interleave(repeats, dim=0) for t in self.key_shift_cache]
        self.value_shift_cache = [t.repeat_interleave(repeats, dim=0) for t in self.value_shift_cache]

    def batch_select_indices(self, indices: torch.Tensor) -> None:
        for s in self._layers:
            n = s.length
            s.k, s.v, s.g = [t[indices, :, :n].contiguous() for t in (s.k, s.v, s.g)]
        self.key_shift_cache = [t[indices] for t in self.key_shift_cache]
        self.value_shift_cache = [t[indices] for t in self.value_shift_cache]
