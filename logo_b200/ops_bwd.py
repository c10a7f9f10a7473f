"""Raw launchers of the backward attention kernels (used by the autograd functions in ``ops``)."""
from __future__ import annotations

import torch

from . import _lib


def _workspace(n_tokens: int, hq: int, gathered: bool, device) -> torch.Tensor:
    nbytes = _lib.load().logo_attn_bwd_workspace_bytes(n_tokens, hq, int(gathered))
    # torch's caching allocator hands out blocks aligned to 512 bytes
    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)


def sq_attn_bwd_raw(q, k, v, o, lse, d_o, m, scale: float):
    """Gradients of the query-sparse global branch: (dq [N,HQ,D], dk [N,H,D], dv [N,H,D])."""
    lib = _lib.load()
    n, hq, d = q.shape
    h = k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = _workspace(n, hq, True, q.device)
    rc = lib.logo_sq_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
                              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m.q_idx.data_ptr(), m.pos_ids.data_ptr(),
                              m.cu_seqlens_q.data_ptr(), m.cu_seqlens_k.data_ptr(), m.tile_off.data_ptr(),
                              m.meta.data_ptr(), ws.data_ptr(), ws.numel(), m.n_seq, n, hq, h, d, float(scale),
                              m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_sq_attn_bwd")
    return dq, dk, dv


def swa_bwd_raw(q, k, v, o, lse, d_o, m, window: int, scale: float):
    """Gradients of the local sliding-window branch."""
    lib = _lib.load()
    n, hq, d = q.shape
    h = k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = _workspace(n, hq, False, q.device)
    rc = lib.logo_swa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
                          dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m.cu_seqlens_k.data_ptr(),
                          m.tile_off.data_ptr(), m.meta.data_ptr(), ws.data_ptr(), ws.numel(), m.n_seq, n, hq, h, d,
                          int(window), float(scale), m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_swa_bwd")
    return dq, dk, dv
