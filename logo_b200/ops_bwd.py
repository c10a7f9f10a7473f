"""Raw launchers of the backward attention kernels (used by the autograd functions in ``ops``)."""
from __future__ import annotations

import torch

from . import _lib


_BRANCHES = {"global": 0, "local": 1}
_MODES = {"single_pass": 0, "two_kernel": 1}


def set_backward_mode(branch: str, mode: str) -> None:
    """Chooses the backward implementation of a branch for the whole process.

    ``branch``: ``"global"`` (query-sparse attention) or ``"local"`` (window attention).
    ``mode``: ``"single_pass"`` -- one kernel forms S and dP once per tile pair and produces dK, dV
    and dQ; dQ is summed with fp32 reductions whose order varies, so it can differ between two runs
    in the last bit. ``"two_kernel"`` -- the dK/dV and dQ kernels, bit-reproducible.
    """
    _lib.check(_lib.load().logo_set_backward_mode(_BRANCHES[branch], _MODES[mode]), "logo_set_backward_mode")


def get_backward_mode(branch: str) -> str:
    code = _lib.load().logo_get_backward_mode(_BRANCHES[branch])
    return {v: k for k, v in _MODES.items()}[code]


class _reproducible_if_requested:
    """Under ``torch.use_deterministic_algorithms(True)`` the two-kernel backward runs for the call."""

    def __init__(self, branch: str):
        self.branch, self.saved = branch, None

    def __enter__(self):
        if torch.are_deterministic_algorithms_enabled() and get_backward_mode(self.branch) != "two_kernel":
            self.saved = get_backward_mode(self.branch)
            set_backward_mode(self.branch, "two_kernel")

    def __exit__(self, *exc):
        if self.saved is not None:
            set_backward_mode(self.branch, self.saved)


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
    with _reproducible_if_requested("global"), torch.cuda.device(q.device):
        rc = lib.logo_sq_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                  d_o.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m.q_idx.data_ptr(),
                                  m.pos_ids.data_ptr(), m.cu_seqlens_q.data_ptr(), m.cu_seqlens_k.data_ptr(),
                                  m.tile_off.data_ptr(), m.meta.data_ptr(), ws.data_ptr(), ws.numel(), m.n_seq, n, hq,
                                  h, d, float(scale), m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_sq_attn_bwd")
    return dq, dk, dv


def swa_bwd_raw(q, k, v, o, lse, d_o, m, window: int, scale: float):
    """Gradients of the local sliding-window branch."""
    lib = _lib.load()
    n, hq, d = q.shape
    h = k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = _workspace(n, hq, False, q.device)
    with _reproducible_if_requested("local"), torch.cuda.device(q.device):
        rc = lib.logo_swa_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), d_o.data_ptr(),
                              dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), m.cu_seqlens_k.data_ptr(),
                              m.tile_off.data_ptr(), m.meta.data_ptr(), ws.data_ptr(), ws.numel(), m.n_seq, n, hq, h,
                              d, int(window), float(scale), m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_swa_bwd")
    return dq, dk, dv
