"""Host-side mirror of the reference's ``logo.ops`` package over the sm_100a CUDA library.

Same names, arguments and error behaviour as the reference (``logo/ops/__init__.py:4-23``):
``sq_full_attn``, ``build_selection``, ``SelInfo``, ``sq_full_attn_dense_ref``,
``sdpa_causal_ref``, ``get_abs_err``, ``get_err_ratio``, ``assert_close``.
Everything that computes runs in ``liblogo_b200.so``; there is no Triton, flash-attn or CPU
path. The ``*_ref`` helpers are the reference's own torch-SDPA checks, kept for API parity.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

__all__ = [
    "sq_full_attn",
    "sq_full_attn_dense_ref",
    "sdpa_causal_ref",
    "build_selection",
    "SelInfo",
    "SelMeta",
    "select_rows",
    "swa_attn",
    "get_abs_err",
    "get_err_ratio",
    "assert_close",
    "check_device_status",
    "lm_head_cross_entropy",
    "proj_rope",
]

HEAD_DIM = 128


# ----------------------------------------------------------------------------------------
# error metrics: the reference's public helpers, restated from logo/ops/common.py:24-41 (same
# names, arguments and formulas, so that checks written against `logo.ops` read the same here)
# ----------------------------------------------------------------------------------------
def get_abs_err(x, y):
    return (x.detach() - y.detach()).flatten().abs().max().item()


def get_err_ratio(x, y):
    err = (x.detach() - y.detach()).flatten().square().mean().sqrt().item()
    base = (x.detach()).flatten().square().mean().sqrt().item()
    return err / (base + 1e-8)


def assert_close(prefix, ref, tri, ratio, err_atol=1e-6):
    abs_atol = get_abs_err(ref, tri)
    msg = f"{prefix} diff: {abs_atol:.6e} ratio: {get_err_ratio(ref, tri):.6e}"
    error_rate = get_err_ratio(ref, tri)
    if abs_atol <= err_atol:
        return msg
    assert error_rate < ratio, msg
    return msg


# ----------------------------------------------------------------------------------------
# selection metadata
# ----------------------------------------------------------------------------------------
@dataclass
class SelInfo:
    """Same fields as the reference's SelInfo (logo/ops/common.py:44-68)."""

    q_idx: torch.Tensor
    pos_ids: torch.Tensor
    cu_seqlens_q: torch.Tensor
    cu_seqlens_k: torch.Tensor
    B: int
    T: int
    Nseq: int
    Sq: int


@dataclass
class SelMeta:
    """Device-resident output of the select kernel; nothing here has been copied to the host.

    ``q_idx`` / ``pos_ids`` are sized for every token; only the first ``meta[0]`` entries are valid.
    """

    q_idx: torch.Tensor          # int64 [N]
    pos_ids: torch.Tensor        # int32 [N]
    cu_seqlens_q: torch.Tensor   # int32 [Nseq+1]
    cu_seqlens_k: torch.Tensor   # int32 [Nseq+1]
    tile_off: torch.Tensor       # int32 [4, Nseq+1]
    meta: torch.Tensor           # int32 [16]: counts, then scratch of the attention kernels
    gate_sum: torch.Tensor       # fp32 [1]
    status: torch.Tensor         # int32 [1] device status word shared by the kernels using this metadata
    n_tokens: int
    n_seq: int


def check_device_status(status: torch.Tensor, what: str = "logo_b200 kernels") -> None:
    """Reads the device status word (this synchronises) and raises if a kernel reported a problem."""
    code = int(status.item())
    if code != 0:
        raise RuntimeError(f"{what}: device status {code}: {_lib.DEVICE_STATUS_TEXT.get(code, 'unknown')}")


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("logo_b200 operators run on CUDA tensors only; there is no CPU fallback")


def select_rows(gate_or_mask: torch.Tensor, thres: Optional[torch.Tensor], cu_seqlens: torch.Tensor) -> SelMeta:
    """Runs the select / compact kernel. ``gate_or_mask`` is a flat ``[N]`` float gate (compared
    ``>= thres`` in fp32, ``thres`` a one-element device tensor) or a bool mask."""
    _require_cuda(gate_or_mask, thres)   # cu_seqlens may live on the host: it is moved like the reference does
    lib = _lib.load()
    flat = gate_or_mask.reshape(-1).contiguous()
    dev = flat.device
    n = flat.numel()
    cu = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
    nseq = cu.numel() - 1
    q_idx = torch.empty(max(n, 1), dtype=torch.int64, device=dev)
    pos_ids = torch.empty(max(n, 1), dtype=torch.int32, device=dev)
    cu_q = torch.empty(nseq + 1, dtype=torch.int32, device=dev)
    tile_off = torch.empty(4, nseq + 1, dtype=torch.int32, device=dev)
    meta = torch.zeros(16, dtype=torch.int32, device=dev)   # LOGO_META_INTS
    gate_sum = torch.empty(1, dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ws_bytes = lib.logo_select_workspace_bytes(n)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    if flat.dtype == torch.bool:
        thres_ptr, thres_code = None, _lib.DTYPE_F32
    else:
        if thres is None:
            raise ValueError("a floating-point gate needs a threshold tensor")
        thres = thres.reshape(-1)[:1].contiguous()
        thres_ptr, thres_code = thres.data_ptr(), _lib.torch_dtype_code(thres.dtype)
    with _lib.on_device(flat):
        rc = lib.logo_select_rows(flat.data_ptr(), _lib.torch_dtype_code(flat.dtype), thres_ptr, thres_code,
                                  cu.data_ptr(), nseq, n, q_idx.data_ptr(), pos_ids.data_ptr(), cu_q.data_ptr(),
                                  tile_off.data_ptr(), meta.data_ptr(), gate_sum.data_ptr(), ws.data_ptr(), ws_bytes,
                                  status.data_ptr(), _lib.current_stream_ptr(dev))
    _lib.check(rc, "logo_select_rows")
    return SelMeta(q_idx, pos_ids, cu_q, cu, tile_off, meta, gate_sum, status, n, nseq)


def build_selection(selection: torch.Tensor, B: int, T: int, cu_seqlens: Optional[torch.Tensor] = None) -> SelInfo:
    """Selection metadata for packed variable-length input (logo/ops/common.py:71-107).

    Like the reference, this public helper returns a python ``Sq`` and therefore synchronises;
    ``sq_full_attn`` itself goes through :func:`select_rows` and does not.
    """
    m = select_rows(selection.reshape(-1), None, cu_seqlens)
    sq = int(m.meta[0].item())
    check_device_status(m.status, "build_selection")
    return SelInfo(q_idx=m.q_idx[:sq], pos_ids=m.pos_ids[:sq], cu_seqlens_q=m.cu_seqlens_q,
                   cu_seqlens_k=m.cu_seqlens_k, B=B, T=T, Nseq=m.n_seq, Sq=sq)


# ----------------------------------------------------------------------------------------
# raw kernel launchers (no autograd)
# ----------------------------------------------------------------------------------------
def _check_qkv(q, k, v):
    _require_cuda(q, k, v)
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("logo_b200 attention kernels take bf16 q/k/v")
    if q.shape[-1] != HEAD_DIM or k.shape[-1] != HEAD_DIM or v.shape[-1] != HEAD_DIM:
        raise NotImplementedError(f"only head_dim {HEAD_DIM} is implemented")


def sq_attn_fwd_raw(q, k, v, m: SelMeta, scale: float, zero_fill: bool = True):
    """q [N,HQ,D], k/v [N,H,D] contiguous bf16 -> (o [N,HQ,D], lse [N,HQ])."""
    _check_qkv(q, k, v)
    lib = _lib.load()
    n, hq, d = q.shape
    h = k.shape[1]
    o = torch.empty_like(q)
    lse = torch.empty(n, hq, dtype=torch.float32, device=q.device)
    with _lib.on_device(q):
        rc = lib.logo_sq_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                  m.q_idx.data_ptr(), m.pos_ids.data_ptr(), m.cu_seqlens_q.data_ptr(),
                                  m.cu_seqlens_k.data_ptr(), m.tile_off.data_ptr(), m.meta.data_ptr(), m.n_seq, n, hq, h,
                                  d, float(scale), int(zero_fill), m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_sq_attn_fwd")
    return o, lse


def swa_fwd_raw(q, k, v, m: SelMeta, window: int, scale: float):
    """Local-branch forward on packed tokens: (o [N,HQ,D], lse [N,HQ])."""
    _check_qkv(q, k, v)
    lib = _lib.load()
    n, hq, d = q.shape
    h = k.shape[1]
    o = torch.empty_like(q)
    lse = torch.empty(n, hq, dtype=torch.float32, device=q.device)
    with _lib.on_device(q):
        rc = lib.logo_swa_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                              m.cu_seqlens_k.data_ptr(), m.tile_off.data_ptr(), m.meta.data_ptr(), m.n_seq, n, hq, h, d,
                              int(window), float(scale), m.status.data_ptr(), _lib.current_stream_ptr(q.device))
    _lib.check(rc, "logo_swa_fwd")
    return o, lse


# ----------------------------------------------------------------------------------------
# autograd functions
# ----------------------------------------------------------------------------------------
# Autocast bookkeeping of the reference's autograd function (logo/ops/triton_utils.py:42-44,
# logo/ops/selected_full_attn.py:450-452,473-474): inside a torch.autocast region floating-point
# inputs are cast to bf16 (the only dtype the kernels take) and the body runs with autocast off;
# the backward runs in the autocast state of its forward. Outside autocast nothing is cast.
_fwd_bf16 = torch.amp.custom_fwd(device_type="cuda", cast_inputs=torch.bfloat16)
_fwd_plain = torch.amp.custom_fwd(device_type="cuda")
_bwd = torch.amp.custom_bwd(device_type="cuda")


class SQFullAttentionFunction(torch.autograd.Function):
    """Counterpart of logo/ops/selected_full_attn.py:449-492 (same argument order)."""

    @staticmethod
    @_fwd_bf16
    def forward(ctx, q, k, v, scale, sel: SelMeta):
        B, T, HQ, K = q.shape
        H, V = v.shape[2], v.shape[3]
        qf = q.contiguous().reshape(B * T, HQ, K)
        kf = k.contiguous().reshape(B * T, H, K)
        vf = v.contiguous().reshape(B * T, H, V)
        o, lse = sq_attn_fwd_raw(qf, kf, vf, sel, scale, zero_fill=True)
        ctx.save_for_backward(qf, kf, vf, o, lse)
        ctx.sel = sel
        ctx.scale = scale
        ctx.shapes = (B, T, HQ, H, K, V)
        return o.view(B, T, HQ, V)

    @staticmethod
    @_bwd
    def backward(ctx, do):
        from .ops_bwd import sq_attn_bwd_raw

        qf, kf, vf, o, lse = ctx.saved_tensors
        B, T, HQ, H, K, V = ctx.shapes
        dof = do.contiguous().reshape(B * T, HQ, V)
        dq, dk, dv = sq_attn_bwd_raw(qf, kf, vf, o, lse, dof, ctx.sel, ctx.scale)
        return dq.view(B, T, HQ, K), dk.view(B, T, H, K), dv.view(B, T, H, V), None, None


class SWAFunction(torch.autograd.Function):
    """Local sliding-window branch (the flash-attn call of logo/layers/logo.py:166-179)."""

    @staticmethod
    @_fwd_bf16
    def forward(ctx, q, k, v, window, scale, sel: SelMeta):
        qf, kf, vf = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = swa_fwd_raw(qf, kf, vf, sel, window, scale)
        ctx.save_for_backward(qf, kf, vf, o, lse)
        ctx.sel, ctx.window, ctx.scale = sel, window, scale
        return o

    @staticmethod
    @_bwd
    def backward(ctx, do):
        from .ops_bwd import swa_bwd_raw

        qf, kf, vf, o, lse = ctx.saved_tensors
        dq, dk, dv = swa_bwd_raw(qf, kf, vf, o, lse, do.contiguous(), ctx.sel, ctx.window, ctx.scale)
        return dq, dk, dv, None, None, None


def swa_attn(q, k, v, cu_seqlens, window: int, scale: Optional[float] = None, sel: Optional[SelMeta] = None):
    """Sliding-window causal attention on packed tokens ``[N, H, D]`` (keys ``[i-window, i]``)."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    if sel is None:
        sel = select_rows(torch.ones(q.shape[0], dtype=torch.bool, device=q.device), None, cu_seqlens)
    return SWAFunction.apply(q, k, v, window, scale, sel)


def sq_full_attn(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    selection: torch.Tensor,
    scale: Optional[float] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    r"""Selected-query full causal attention (logo/ops/selected_full_attn.py:495-527).

    Args:
        q: queries `[1, total_tokens, HQ, K]`.
        k: keys    `[1, total_tokens, H, K]` (GQA when HQ % H == 0).
        v: values  `[1, total_tokens, H, V]`.
        selection: per-token bool mask `[1, total_tokens]`.
        scale: attention scale; defaults to `K ** -0.5`.
        cu_seqlens: required `[Nseq+1]` int tensor for packed varlen input.

    Returns:
        o: `[1, total_tokens, HQ, V]`; rows for unselected query tokens are 0.
    """
    B, T, HQ, K = q.shape
    H = k.shape[2]
    assert q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q/k/v must be [B, T, H, D]"
    assert HQ % H == 0, "HQ must be a multiple of H (GQA)"
    assert selection.dtype == torch.bool and selection.shape == (B, T), "selection must be a bool mask [B, T]"
    assert B == 1, "sq_full_attn only supports B=1 packed-varlen input"
    assert cu_seqlens is not None, "sq_full_attn requires explicit cu_seqlens"
    if scale is None:
        scale = K ** -0.5
    sel = select_rows(selection.reshape(-1), None, cu_seqlens)
    return SQFullAttentionFunction.apply(q, k, v, scale, sel)


# ----------------------------------------------------------------------------------------
# the reference's dense checks (logo/ops/dense_full_attn.py), kept for API parity
# ----------------------------------------------------------------------------------------
def sq_full_attn_dense_ref(q, k, v, scale=None, cu_seqlens=None):
    """Full causal attention through the shared kernels (selection = all ones), dense_full_attn.py:12-22."""
    B, T, HQ, K = q.shape
    selection = torch.ones(B, T, dtype=torch.bool, device=q.device)
    return sq_full_attn(q, k, v, selection, scale=scale, cu_seqlens=cu_seqlens)


def sdpa_causal_ref(q, k, v, scale=None, cu_seqlens=None):
    """Independent causal-attention check with torch SDPA (dense_full_attn.py:30-69)."""
    B, T, HQ, K = q.shape
    H = k.shape[2]
    G = HQ // H
    if scale is None:
        scale = K ** -0.5

    def rep(x):
        b, t, h, d = x.shape
        return x[:, :, :, None, :].expand(b, t, h, G, d).reshape(b, t, h * G, d)

    qh, kh, vh = q.transpose(1, 2), rep(k).transpose(1, 2), rep(v).transpose(1, 2)
    if cu_seqlens is None:
        return F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, scale=scale).transpose(1, 2).contiguous()
    assert B == 1
    cu = cu_seqlens.tolist()
    outs = [F.scaled_dot_product_attention(qh[:, :, a:b], kh[:, :, a:b], vh[:, :, a:b], is_causal=True, scale=scale)
            for a, b in zip(cu[:-1], cu[1:])]
    return torch.cat(outs, dim=2).transpose(1, 2).contiguous()


# ----------------------------------------------------------------------------------------
# RMSNorm over rows of any width, inference only (logo/modules/layernorm.py:9-26)
# ----------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``weight * bf16(x * rsqrt(mean(x^2) + eps))`` over the last dimension of a bf16 CUDA tensor."""
    lib = _lib.load()
    _require_cuda(x, weight)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise TypeError("the RMSNorm kernel takes bf16 activations and a bf16 weight")
    dim = x.shape[-1]
    if weight.numel() != dim:
        raise ValueError("rmsnorm: weight must have the size of the last dimension")
    xc = x.contiguous()
    out = torch.empty_like(xc)
    with _lib.on_device(xc):
        rc = lib.logo_rmsnorm_fwd(xc.data_ptr(), weight.contiguous().data_ptr(), out.data_ptr(), xc.numel() // dim, dim,
                                  float(eps), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "logo_rmsnorm_fwd")
    return out


# ----------------------------------------------------------------------------------------
# gated MLP activation, inference only (logo/modules/mlp.py:25)
# ----------------------------------------------------------------------------------------
def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` over bf16 CUDA tensors of equal shape whose last dimension is contiguous
    (row-strided views, e.g. the two halves of a fused projection, are read in place)."""
    lib = _lib.load()
    _require_cuda(gate, up)
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.shape != up.shape:
        raise TypeError("silu_mul takes two bf16 tensors of the same shape")
    dim = gate.shape[-1]
    g2, u2 = gate.reshape(-1, dim), up.reshape(-1, dim)     # views when only the row stride is non-trivial
    if g2.stride(1) != 1 or g2.stride(0) % 8 or g2.data_ptr() % 16:
        g2 = g2.contiguous()
    if u2.stride(1) != 1 or u2.stride(0) % 8 or u2.data_ptr() % 16:
        u2 = u2.contiguous()
    out = torch.empty(gate.shape, dtype=torch.bfloat16, device=gate.device)
    with _lib.on_device(g2):
        rc = lib.logo_silu_mul(g2.data_ptr(), g2.stride(0), u2.data_ptr(), u2.stride(0), out.data_ptr(), g2.shape[0], dim,
                               _lib.current_stream_ptr(gate.device))
    _lib.check(rc, "logo_silu_mul")
    return out


# ----------------------------------------------------------------------------------------
# rotary position embedding (logo/modules/rotary.py:81-106, used at logo/layers/logo.py:136-139)
# ----------------------------------------------------------------------------------------
def _rope_call(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool) -> torch.Tensor:
    lib = _lib.load()
    n, h, d = x.shape
    if x.stride(2) != 1 or x.stride(0) % 8 or x.stride(1) % 8 or x.data_ptr() % 16:
        x = x.contiguous()      # rows must be contiguous and 16-byte aligned; any token / head strides are fine
    out = torch.empty((n, h, d), dtype=x.dtype, device=x.device)
    with _lib.on_device(x):
        rc = lib.logo_rope(x.data_ptr(), x.stride(0), x.stride(1), out.data_ptr(), cos.data_ptr(), sin.data_ptr(), n, h, d,
                           int(inverse), _lib.current_stream_ptr(x.device))
    _lib.check(rc, "logo_rope")
    return out


class RopeFunction(torch.autograd.Function):
    """``(x * cos) + (rotate_half(x) * sin)`` on packed ``[N, H, 128]`` bf16 rows, one kernel each way."""

    @staticmethod
    @_fwd_bf16
    def forward(ctx, x, cos, sin):
        _require_cuda(x, cos, sin)
        if x.dtype != torch.bfloat16 or cos.dtype != torch.bfloat16 or sin.dtype != torch.bfloat16:
            raise TypeError("the rotary kernel takes bf16 activations and bf16 cos / sin tables")
        if x.dim() != 3 or cos.shape != (x.shape[0], x.shape[2]) or sin.shape != cos.shape:
            raise ValueError("rope: x must be [N, H, D] and cos / sin [N, D]")
        cos, sin = cos.contiguous(), sin.contiguous()
        ctx.save_for_backward(cos, sin)
        return _rope_call(x, cos, sin, False)

    @staticmethod
    @_bwd
    def backward(ctx, d_out):
        cos, sin = ctx.saved_tensors
        return _rope_call(d_out, cos, sin, True), None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of ``x [N, H, 128]`` with per-token tables ``cos, sin [N, 128]`` (all bf16)."""
    return RopeFunction.apply(x, cos, sin)


# ----------------------------------------------------------------------------------------
# per-head projection of the global branch fused with the rotary embedding
# (logo/layers/logo.py:86-94 + :137-139 + the layout copies of :156-158)
# ----------------------------------------------------------------------------------------
class ProjRopeFunction(torch.autograd.Function):
    """``out[t, h] = rope(x[t, h] @ w[h])`` in one kernel; with a selection only its rows are computed.

    The backward un-rotates the gradient with the rotary kernel and forms the two gradient products
    with batched GEMMs (rows outside the selection carry a zero gradient: the attention backward
    writes zeros there)."""

    @staticmethod
    @_fwd_bf16
    def forward(ctx, x, w, cos, sin, sel):
        lib = _lib.load()
        _require_cuda(x, w, cos, sin)
        if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
            raise TypeError("proj_rope takes bf16 activations and bf16 per-head weights")
        n, heads, d = x.shape
        if x.stride(2) != 1 or x.stride(1) != d or x.stride(0) % 8 or x.data_ptr() % 16:
            x = x.contiguous()
        w = w.contiguous()
        if cos is not None:
            cos, sin = cos.contiguous(), sin.contiguous()
        out = torch.empty(n, heads, d, dtype=torch.bfloat16, device=x.device)
        status = sel.status if sel is not None else torch.zeros(1, dtype=torch.int32, device=x.device)
        with _lib.on_device(x):
            rc = lib.logo_proj_rope(x.data_ptr(), x.stride(0), w.data_ptr(),
                                    sel.q_idx.data_ptr() if sel is not None else None,
                                    sel.meta.data_ptr() if sel is not None else None, _lib.ptr(cos), _lib.ptr(sin),
                                    out.data_ptr(), n, heads, d, status.data_ptr(), _lib.current_stream_ptr(x.device))
        _lib.check(rc, "logo_proj_rope")
        ctx.save_for_backward(x, w, cos, sin)
        return out

    @staticmethod
    @_bwd
    def backward(ctx, g):
        x, w, cos, sin = ctx.saved_tensors
        if cos is not None:
            g = _rope_call(g, cos, sin, True)
        else:
            g = g.contiguous()
        dx = torch.einsum("l h e, h d e -> l h d", g, w) if ctx.needs_input_grad[0] else None
        dw = torch.einsum("l h d, l h e -> h d e", x, g) if ctx.needs_input_grad[1] else None
        return dx, dw, None, None, None


def proj_rope(x: torch.Tensor, w: torch.Tensor, cos: Optional[torch.Tensor] = None,
              sin: Optional[torch.Tensor] = None, sel: Optional[SelMeta] = None) -> torch.Tensor:
    """``x [N, H, 128]`` (rows of a token contiguous), ``w [H, 128, 128]``, ``cos / sin [N, 128]`` or None;
    returns ``[N, H, 128]`` bf16. With ``sel`` only the selected token rows are computed; the others
    are left unwritten (the query-sparse attention never reads them)."""
    return ProjRopeFunction.apply(x, w, cos, sin, sel)


# ----------------------------------------------------------------------------------------
# per-branch RMSNorm + gate mask + blend (logo/layers/logo.py:180-182,225-227,256-258)
# ----------------------------------------------------------------------------------------
class FuseFunction(torch.autograd.Function):
    """out[N, H*D] = (1-g) * RMSNorm_l(local) + g * RMSNorm_g(glob), g = gate masked below thres."""

    @staticmethod
    @_fwd_plain      # no cast: the threshold and the norm weights keep their own precision
    def forward(ctx, local, glob, gate, thres, w_local, w_global, eps, use_norm):
        lib = _lib.load()
        _require_cuda(local, glob, gate, thres)
        if local.dtype != torch.bfloat16 or glob.dtype != torch.bfloat16 or gate.dtype != torch.bfloat16:
            raise TypeError("the fused norm/blend kernel takes bf16 activations and a bf16 gate")
        local, glob = local.contiguous(), glob.contiguous()
        gate_flat = gate.reshape(-1).contiguous()
        thres = thres.reshape(-1)[:1].contiguous()
        n, h, d = local.shape
        if use_norm:
            if w_local.dtype != w_global.dtype:
                raise TypeError("both context-norm weights must share one dtype")
            w_local, w_global = w_local.contiguous(), w_global.contiguous()
            w_code = _lib.torch_dtype_code(w_local.dtype)
        else:
            w_code = _lib.DTYPE_BF16
        out = torch.empty(n, h * d, dtype=torch.bfloat16, device=local.device)
        with _lib.on_device(local):
            rc = lib.logo_fuse_fwd(local.data_ptr(), glob.data_ptr(), gate_flat.data_ptr(), _lib.DTYPE_BF16,
                                   thres.data_ptr(), _lib.torch_dtype_code(thres.dtype),
                                   _lib.ptr(w_local) if use_norm else None, _lib.ptr(w_global) if use_norm else None,
                                   w_code, out.data_ptr(), n, h, d, float(eps), int(bool(use_norm)),
                                   _lib.current_stream_ptr(local.device))
        _lib.check(rc, "logo_fuse_fwd")
        ctx.save_for_backward(local, glob, gate_flat, thres, w_local if use_norm else None,
                              w_global if use_norm else None)
        ctx.eps, ctx.use_norm, ctx.gate_shape, ctx.w_code = float(eps), bool(use_norm), gate.shape, w_code
        return out

    @staticmethod
    @_bwd
    def backward(ctx, d_out):
        lib = _lib.load()
        local, glob, gate_flat, thres, w_local, w_global = ctx.saved_tensors
        n, h, d = local.shape
        d_out = d_out.contiguous()
        d_local, d_glob = torch.empty_like(local), torch.empty_like(glob)
        d_gate = torch.empty_like(gate_flat)
        d_wl = torch.empty_like(w_local) if ctx.use_norm else None
        d_wg = torch.empty_like(w_global) if ctx.use_norm else None
        ws_bytes = lib.logo_fuse_bwd_workspace_bytes(n)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=local.device)
        with _lib.on_device(local):
            rc = lib.logo_fuse_bwd(d_out.data_ptr(), local.data_ptr(), glob.data_ptr(), gate_flat.data_ptr(),
                                   _lib.DTYPE_BF16, thres.data_ptr(), _lib.torch_dtype_code(thres.dtype),
                                   _lib.ptr(w_local), _lib.ptr(w_global), ctx.w_code, d_local.data_ptr(),
                                   d_glob.data_ptr(), d_gate.data_ptr(), _lib.ptr(d_wl), _lib.ptr(d_wg), n, h, d, ctx.eps,
                                   int(ctx.use_norm), ws.data_ptr(), ws.numel(), _lib.current_stream_ptr(local.device))
        _lib.check(rc, "logo_fuse_bwd")
        return d_local, d_glob, d_gate.view(ctx.gate_shape), None, d_wl, d_wg, None, None


def fuse_norm_blend(local, glob, gate, thres, w_local, w_global, eps: float, use_norm: bool = True):
    """local, glob [N,H,128] bf16; gate [N] or [N,1] bf16; thres one-element tensor. Returns [N, H*128]."""
    return FuseFunction.apply(local, glob, gate, thres, w_local, w_global, eps, use_norm)


# ----------------------------------------------------------------------------------------
# lm_head + shifted cross-entropy with packed-boundary masking (logo/modeling_logo.py:380-407)
# ----------------------------------------------------------------------------------------
class LmHeadLossFunction(torch.autograd.Function):
    """Mean next-token cross-entropy of ``hidden @ weight.T`` without ever holding the ``[tokens, vocab]``
    logits: rows are processed in chunks; each chunk's bf16 logits are turned into their gradient in
    place by the loss kernel and immediately contracted into the gradients of ``hidden`` and ``weight``."""

    @staticmethod
    @_fwd_plain
    def forward(ctx, hidden, weight, labels, cu_seqlens, ignore_index, chunk_rows):
        lib = _lib.load()
        _require_cuda(hidden, weight, labels)
        if hidden.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
            raise TypeError("lm_head_cross_entropy takes bf16 hidden states and a bf16 weight")
        n, hid = hidden.shape
        vocab = weight.shape[0]
        dev = hidden.device
        hidden, weight = hidden.contiguous(), weight.contiguous()
        labels = labels.reshape(-1).to(torch.int64).contiguous()
        cu = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        targets = torch.empty(n, dtype=torch.int64, device=dev)
        n_valid = torch.zeros(1, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        row_loss = torch.empty(n, dtype=torch.float32, device=dev)
        stream = _lib.current_stream_ptr(dev)
        need_h, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        d_hidden = torch.empty_like(hidden) if need_h else None
        d_weight = torch.zeros(vocab, hid, dtype=torch.float32, device=dev) if need_w else None
        with _lib.on_device(hidden):
            _lib.check(lib.logo_shift_labels(labels.data_ptr(), cu.data_ptr(), cu.numel() - 1, n, int(ignore_index),
                                             targets.data_ptr(), n_valid.data_ptr(), stream), "logo_shift_labels")
            for a in range(0, n, chunk_rows):
                b = min(a + chunk_rows, n)
                logits = hidden[a:b] @ weight.t()                       # bf16, as the bf16 lm_head produces them
                _lib.check(lib.logo_ce_rows(logits.data_ptr(), vocab, targets[a:b].data_ptr(), int(ignore_index),
                                            row_loss[a:b].data_ptr(), n_valid.data_ptr(), 1.0, b - a, vocab,
                                            int(need_h or need_w), status.data_ptr(), stream), "logo_ce_rows")
                if need_h:
                    torch.mm(logits, weight, out=d_hidden[a:b])
                if need_w:
                    d_weight += (logits.t() @ hidden[a:b]).float()
        ctx.save_for_backward(d_hidden, d_weight.to(weight.dtype) if need_w else None)
        ctx.status = status
        return (row_loss.sum() / n_valid.clamp(min=1).to(torch.float32)).reshape(())

    @staticmethod
    @_bwd
    def backward(ctx, g):
        d_hidden, d_weight = ctx.saved_tensors
        return (None if d_hidden is None else d_hidden * g.to(d_hidden.dtype),
                None if d_weight is None else d_weight * g.to(d_weight.dtype), None, None, None, None)


def lm_head_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                          cu_seqlens: Optional[torch.Tensor] = None, ignore_index: int = -100,
                          chunk_rows: int = 8192) -> torch.Tensor:
    """The loss of ``LoGoForCausalLM.forward`` (logo/modeling_logo.py:380-407) from the final hidden states.

    ``hidden`` ``[B, T, H]`` or packed ``[1, N, H]`` / ``[N, H]`` bf16, ``weight`` the lm_head weight ``[V, H]``
    bf16 (V a multiple of 8), ``labels`` the UN-shifted labels with the shape of the tokens. Token ``i`` is
    scored against ``labels[i + 1]``; the last token of every row -- or, with ``cu_seqlens``, of every
    packed sequence -- has no target, as have labels equal to ``ignore_index``. Returns the mean over the
    scored tokens as an fp32 scalar; differentiable with respect to ``hidden`` and ``weight``.
    """
    if hidden.dim() == 3:
        bsz, t, hid = hidden.shape
        flat = hidden.reshape(bsz * t, hid)
        if cu_seqlens is None:
            cu_seqlens = torch.arange(0, (bsz + 1) * t, t, dtype=torch.int32, device=hidden.device)
    else:
        flat = hidden
        if cu_seqlens is None:
            cu_seqlens = torch.tensor([0, hidden.shape[0]], dtype=torch.int32, device=hidden.device)
    return LmHeadLossFunction.apply(flat, weight, labels, cu_seqlens, ignore_index, chunk_rows)
