"""Dual-state KV cache with the reference's ``Cache`` contract over preallocated storage.

The reference (``logo/cache.py:46-124``) grows both states with ``torch.cat`` on every step.
Here each layer owns preallocated bf16 buffers that are updated in place by
``logo_cache_append``:

* global branch ``[B, H, t_max, D]`` -- token ``p`` at row ``p``;
* local branch ``[B, H, window + 1, D]`` -- a ring, token ``p`` at row ``p % (window + 1)``.

``update()`` keeps the reference's signature and returns the same dictionary (``attn_state``
= the local keys/values to attend over, ``attn_state_full`` = the whole global state) for
callers that consume tensors; the LoGo layer of this package uses :meth:`append` and
:meth:`layer_buffers` instead and reads the buffers directly from the decode kernel.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _lib

__all__ = ["Cache"]


class _LayerState:
    __slots__ = ("k_ring", "v_ring", "k_full", "v_full", "ring", "t_max", "length", "status")

    def __init__(self):
        self.k_ring = self.v_ring = self.k_full = self.v_full = None
        self.ring = 0
        self.t_max = 0
        self.length = 0          # tokens written so far (same for every sequence of the batch)
        self.status = None


class Cache:
    """Key/value cache for LoGo's dual-branch attention (same public surface as ``logo.cache.Cache``)."""

    is_compileable = True

    def __init__(self, seen_tokens: int = 0, max_length: int = 0, growth: int = 1024) -> None:
        self.layers: List[_LayerState] = []
        self._seen_tokens = seen_tokens
        self._max_length = max_length
        self._growth = growth

    # -- container protocol (logo/cache.py:35-44) --------------------------------------------
    def __len__(self) -> int:
        return len(self.layers)

    def __getitem__(self, layer_idx: int) -> Dict[str, Any]:
        if layer_idx < len(self):
            return self._state_dict(self.layers[layer_idx])
        raise KeyError(f"Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}")

    def __iter__(self):
        for st in self.layers:
            yield self._state_dict(st)

    # -- storage ---------------------------------------------------------------------------------
    def _ensure(self, layer_idx: int, b: int, h: int, d: int, window: Optional[int], need: int, device) -> _LayerState:
        while len(self.layers) <= layer_idx:
            self.layers.append(_LayerState())
        st = self.layers[layer_idx]
        if st.k_full is None:
            st.t_max = max(self._max_length, need + self._growth)
            st.k_full = torch.empty(b, h, st.t_max, d, dtype=torch.bfloat16, device=device)
            st.v_full = torch.empty_like(st.k_full)
            st.ring = (window + 1) if window is not None else 0
            if st.ring:
                st.k_ring = torch.zeros(b, h, st.ring, d, dtype=torch.bfloat16, device=device)
                st.v_ring = torch.zeros_like(st.k_ring)
            st.status = torch.zeros(1, dtype=torch.int32, device=device)
        elif need > st.t_max:
            new_max = max(need + self._growth, 2 * st.t_max)
            for name in ("k_full", "v_full"):
                old = getattr(st, name)
                new = torch.empty(b, h, new_max, d, dtype=torch.bfloat16, device=device)
                new[:, :, : st.length].copy_(old[:, :, : st.length])
                setattr(st, name, new)
            st.t_max = new_max
        return st

    def append(self, layer_idx: int, k_local, v_local, k_global, v_global, window: int, layout: str = "bthd") -> _LayerState:
        """Writes ``t_new`` tokens per sequence in place.

        ``layout='bthd'``: tensors are ``[B, t, H, D]``; ``'bhtd'``: ``[B, H, t, D]`` (any strides
        whose last dimension is contiguous). The first layer advances the seen-token counter.
        """
        lib = _lib.load()
        given = [x for x in (k_local, v_local, k_global, v_global) if x is not None]
        for x in given:
            if x.dtype != torch.bfloat16:
                raise TypeError("the KV cache stores bf16 states")
            if not x.is_cuda:
                raise RuntimeError("the KV cache lives on a CUDA device; there is no CPU fallback")

        def bth_strides(x):
            return (x.stride(0), x.stride(1), x.stride(2)) if layout == "bthd" else (x.stride(0), x.stride(2), x.stride(1))

        ref_strides = bth_strides(k_global)
        same = all(x.stride(-1) == 1 and bth_strides(x) == ref_strides and x.data_ptr() % 16 == 0 for x in given)
        if not same or any(s % 8 for s in ref_strides):
            k_local, v_local, k_global, v_global = (None if x is None else x.contiguous()
                                                    for x in (k_local, v_local, k_global, v_global))
            ref_strides = bth_strides(k_global)
        if layout == "bthd":
            b, t_new, h, d = k_global.shape
        else:
            b, h, t_new, d = k_global.shape
        cur = self.layers[layer_idx].length if layer_idx < len(self.layers) else 0
        st = self._ensure(layer_idx, b, h, d, window if k_local is not None else None, cur + t_new, k_global.device)
        if k_local is not None and st.k_ring is not None and st.ring != window + 1:
            self._resize_ring(st, window)
        with _lib.on_device(k_global):
            rc = self._append_call(lib, st, k_local, v_local, k_global, v_global, ref_strides, b, t_new, h, d)
        _lib.check(rc, "logo_cache_append")
        st.length += t_new
        if layer_idx == 0:
            self._seen_tokens += t_new
        return st

    @staticmethod
    def _append_call(lib, st, k_local, v_local, k_global, v_global, ref_strides, b, t_new, h, d) -> int:
        return lib.logo_cache_append(_lib.ptr(k_local), _lib.ptr(v_local), k_global.data_ptr(), v_global.data_ptr(),
                                   ref_strides[0], ref_strides[1], ref_strides[2],
                                   _lib.ptr(st.k_ring) if k_local is not None else None,
                                   _lib.ptr(st.v_ring) if k_local is not None else None, st.ring,
                                   st.k_full.data_ptr(), st.v_full.data_ptr(), st.t_max, None, st.length, b, t_new, h,
                                   d, st.status.data_ptr(), _lib.current_stream_ptr(k_global.device))

    @staticmethod
    def _resize_ring(st: _LayerState, window: int) -> None:
        """Re-lays the local ring for another window size (a cache built from a legacy tuple does not
        know the layer's window until the first append). The ring holds local-branch states, which
        cannot be recomputed from the global state: tokens the old ring no longer holds are lost, so a
        ring that is too small for the new window is an error, not a silent truncation."""
        have = min(st.length, st.ring)                 # last tokens present in the old ring
        need = min(st.length, window)                  # tokens a step with this window attends over
        if have < need:
            raise ValueError(f"the cached local state holds {have} tokens but window_size {window} needs {need}; "
                             "rebuild the cache with the layer's window_size")
        keep = min(have, window + 1)
        pos = torch.arange(st.length - keep, st.length, device=st.k_ring.device)
        new_ring = window + 1
        for name in ("k_ring", "v_ring"):
            old = getattr(st, name)
            new = torch.zeros(old.shape[0], old.shape[1], new_ring, old.shape[3], dtype=old.dtype, device=old.device)
            if keep:
                new.index_copy_(2, pos % new_ring, old.index_select(2, pos % st.ring))
            setattr(st, name, new)
        st.ring = new_ring

    def layer_buffers(self, layer_idx: int) -> _LayerState:
        return self.layers[layer_idx]

    # -- reference contract ----------------------------------------------------------------------
    def _local_window(self, st: _LayerState, upto: int, window: int):
        """Last ``min(upto, window)`` local tokens before position ``upto`` as ``[B, H, t, D]`` tensors."""
        n = min(upto, window)
        idx = torch.arange(upto - n, upto, device=st.k_ring.device) % st.ring
        return st.k_ring.index_select(2, idx), st.v_ring.index_select(2, idx)

    def _state_dict(self, st: _LayerState) -> Dict[str, Any]:
        out: Dict[str, Any] = {"attn_state": None, "attn_state_full": None}
        if st.k_full is not None:
            out["attn_state_full"] = (st.k_full[:, :, : st.length], st.v_full[:, :, : st.length])
        if st.k_ring is not None:
            out["attn_state"] = self._local_window(st, st.length, st.ring - 1)
        return out

    def update(
        self,
        attn_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        attn_state_full: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        layer_idx: int = 0,
        offset: Optional[int] = 1,
        cache_kwargs: Optional[Dict[str, Any]] = None,
    ) -> Dict[str, Any]:
        """Same arguments and return value as ``logo/cache.py:46-124`` (states are ``[B, H, t, D]``)."""
        cache_kwargs = cache_kwargs or {}
        if attn_state is None or attn_state_full is None:
            raise NotImplementedError("this cache stores LoGo layers: both attn_state and attn_state_full are required")
        if not isinstance(attn_state, tuple) or len(attn_state) != 2:
            raise ValueError("`attn_state` must be a tuple of two tensors for key/value states")
        window_size = cache_kwargs.get("window_size", None)
        if window_size is None:
            raise NotImplementedError("`window_size` is required: the local state is a fixed-size ring")
        if window_size <= 0:
            raise ValueError(f"`window_size` must be positive, got {window_size}")

        first = len(self.layers) <= layer_idx or self.layers[layer_idx].k_full is None
        for_attention = attn_state
        if not first:
            st = self.layers[layer_idx]
            old_k, old_v = self._local_window(st, st.length, window_size)
            for_attention = (torch.cat([old_k, attn_state[0]], dim=-2), torch.cat([old_v, attn_state[1]], dim=-2))
        seen_before = self._seen_tokens
        st = self.append(layer_idx, attn_state[0], attn_state[1], attn_state_full[0], attn_state_full[1], window_size,
                         layout="bhtd")
        if layer_idx == 0:
            # `append` advanced by the number of tokens written; the contract advances by `offset`
            self._seen_tokens = seen_before + offset
        return {"attn_state": for_attention,
                "attn_state_full": (st.k_full[:, :, : st.length], st.v_full[:, :, : st.length])}

    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        """Number of cached tokens (0 if this layer has no state yet), logo/cache.py:126-130."""
        if len(self.layers) <= layer_idx:
            return 0
        return self._seen_tokens

    def get_max_length(self) -> Optional[int]:
        """The cache grows on demand (logo/cache.py:132-134)."""
        return None

    def to_legacy_cache(self) -> Tuple:
        return tuple(self._state_dict(st) for st in self.layers)

    @classmethod
    def from_legacy_cache(cls, past_key_values: Optional[Tuple] = None, seen_tokens: int = 0,
                          window_size: Optional[int] = None) -> "Cache":
        """Builds a cache from the legacy tuple of per-layer state dicts (logo/cache.py:136-155)."""
        cache = cls(seen_tokens)
        if isinstance(past_key_values, (list, tuple)):
            for layer_idx, state in enumerate(past_key_values):
                full = state.get("attn_state_full")
                local = state.get("attn_state")
                if full is None or local is None:
                    raise NotImplementedError("legacy states must hold both attn_state and attn_state_full")
                t = full[0].shape[-2]
                w = local[0].shape[-2]
                # The legacy local state holds the last `w` = min(t, window) tokens. Without an explicit
                # window_size the ring is sized for exactly those; the first append() passes the layer's
                # real window and re-lays the ring if it differs (nothing is lost: when t > w, w IS the
                # window; when t == w every cached token is in the state).
                window = window_size or max(w, 1)
                st = cache._ensure(layer_idx, full[0].shape[0], full[0].shape[1], full[0].shape[-1], window, t,
                                   full[0].device)
                st.k_full[:, :, :t].copy_(full[0])
                st.v_full[:, :, :t].copy_(full[1])
                idx = torch.arange(t - w, t, device=full[0].device) % st.ring
                st.k_ring.index_copy_(2, idx, local[0].to(torch.bfloat16))
                st.v_ring.index_copy_(2, idx, local[1].to(torch.bfloat16))
                st.length = t
            if seen_tokens == 0 and cache.layers:
                cache._seen_tokens = cache.layers[0].length
        return cache
