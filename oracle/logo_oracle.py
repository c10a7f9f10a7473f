"""CPU oracle for the LoGo attention hot path -- TEST INFRASTRUCTURE, not product code.

A plain restatement (numpy for the integer work, dense-masked torch fp32/fp64 for the
floating-point work) of what the reference computes on this path. Only the test-suite,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may
import this module; nothing under ``logo_b200/`` does.

Pinning: every function below is checked against outputs of the reference itself
(``tests/golden/*.npz``, produced by ``tests/golden/make_golden.py`` which imports the
reference package and runs its own code -- the Triton kernels under the Triton
interpreter, the layer with a dense-masked stand-in for the flash-attn wheel).
The flash-attn wheel is a third-party dependency that is not part of the reference
tree (``flash-attn>=2.3.2``, setup.py:35-37); its window semantics (keys
``[i - w, i]`` inclusive, bottom-right aligned) are restated from its public docstring
and are not pinned by any reference test.

All citations are paths inside the reference project (Pan-Yuqi/Logo).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

RCP_LN2 = 1.4426950216  # logo/ops/selected_full_attn.py:30


# ---------------------------------------------------------------------------------------
# integer work: selection metadata
# ---------------------------------------------------------------------------------------
@dataclass
class SelRef:
    """Mirror of SelInfo (logo/ops/common.py:44-68) with numpy arrays."""

    q_idx: np.ndarray          # int64 [Sq]
    pos_ids: np.ndarray        # int32 [Sq]
    cu_seqlens_q: np.ndarray   # int32 [Nseq+1]
    cu_seqlens_k: np.ndarray   # int32 [Nseq+1]
    Nseq: int
    Sq: int


def select_from_gate(gate: np.ndarray, thres: float) -> np.ndarray:
    """``gate >= gate_thres`` (logo/layers/logo.py:190), evaluated in fp32; NaN is unselected."""
    g = np.asarray(gate, dtype=np.float32)
    return g >= np.float32(thres)


def build_selection_ref(selection: np.ndarray, cu_seqlens: Sequence[int]) -> SelRef:
    """logo/ops/common.py:71-107: ascending selected indices, in-sequence positions, per-sequence counts."""
    flat = np.asarray(selection).reshape(-1).astype(bool)
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    nseq = cu.shape[0] - 1
    q_idx = np.nonzero(flat)[0].astype(np.int64)                      # :90
    seg = np.searchsorted(cu, q_idx, side="right") - 1               # :92
    pos = (q_idx - cu[seg]).astype(np.int32)                         # :93
    counts = np.bincount(seg, minlength=nseq)[:nseq] if q_idx.size else np.zeros(nseq, np.int64)
    cu_q = np.zeros(nseq + 1, dtype=np.int32)                        # :95-96
    cu_q[1:] = np.cumsum(counts).astype(np.int32)
    return SelRef(q_idx, pos, cu_q, cu.astype(np.int32), nseq, int(q_idx.size))


def prepare_chunk_indices_ref(cu_seqlens: Sequence[int], chunk: int) -> np.ndarray:
    """logo/ops/common.py:110-124: flat tile id -> (sequence id, local tile id), empty sequences skipped."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    rows = []
    for sid in range(cu.shape[0] - 1):
        n = int(cu[sid + 1] - cu[sid])
        for b in range((n + chunk - 1) // chunk):
            rows.append((sid, b))
    return np.asarray(rows, dtype=np.int32).reshape(-1, 2)


def tile_offsets_ref(cu_seqlens: Sequence[int], chunk: int) -> np.ndarray:
    """Prefix sum of ceil(len / chunk) per sequence: the device-side form of prepare_chunk_indices."""
    cu = np.asarray(cu_seqlens, dtype=np.int64)
    lens = cu[1:] - cu[:-1]
    out = np.zeros(cu.shape[0], dtype=np.int32)
    out[1:] = np.cumsum((lens + chunk - 1) // chunk).astype(np.int32)
    return out


def q_start_blk_ref(pos_ids: np.ndarray, cu_seqlens_q: np.ndarray, cu_seqlens_k: np.ndarray, bt: int) -> np.ndarray:
    """logo/ops/selected_full_attn.py:374-402: per key tile, first compacted-query tile that can see it."""
    out = []
    for s in range(len(cu_seqlens_k) - 1):
        lk = int(cu_seqlens_k[s + 1] - cu_seqlens_k[s])
        p = pos_ids[int(cu_seqlens_q[s]):int(cu_seqlens_q[s + 1])]
        for t in range((lk + bt - 1) // bt):
            first = int(np.searchsorted(p, t * bt, side="left"))
            out.append(first // bt)
    return np.asarray(out, dtype=np.int32)


# ---------------------------------------------------------------------------------------
# floating-point work: attention
# ---------------------------------------------------------------------------------------
def _repeat_kv(x: torch.Tensor, g: int) -> torch.Tensor:
    n, h, d = x.shape
    return x[:, :, None, :].expand(n, h, g, d).reshape(n, h * g, d)


def _seq_mask(cu: Sequence[int], n: int, window: Optional[int]) -> torch.Tensor:
    """Boolean [n, n]: key j visible to query i. Same sequence, causal, optional window [i-w, i]."""
    cu_t = torch.as_tensor(np.asarray(cu, dtype=np.int64))
    idx = torch.arange(n)
    seg = torch.searchsorted(cu_t, idx, right=True) - 1
    same = seg[:, None] == seg[None, :]
    causal = idx[None, :] <= idx[:, None]
    m = same & causal
    if window is not None:
        m = m & (idx[None, :] >= idx[:, None] - window)
    return m


def attention_dense_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    cu_seqlens: Sequence[int],
    scale: Optional[float] = None,
    window: Optional[int] = None,
    selection: Optional[torch.Tensor] = None,
    dtype: torch.dtype = torch.float32,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense-masked attention over packed tokens.

    q [N,HQ,D], k [N,H,D], v [N,H,Dv]. Returns (o [N,HQ,Dv], lse2 [N,HQ]) where lse2 is the
    base-2 log-sum-exp of ``scale * RCP_LN2 * q.k`` (logo/ops/selected_full_attn.py:93,118-119).
    ``window=None``: full causal (global branch, selected_full_attn.py:88-116 semantics);
    ``window=w``: keys [i-w, i] (local branch, logo/layers/logo.py:166-179 with flash-attn
    ``window_size=(w, w)`` under a causal mask).
    Rows with ``selection == False`` are zero (selected_full_attn.py:469-471).
    Differentiable with torch autograd.
    """
    n, hq, d = q.shape
    h = k.shape[1]
    g = hq // h
    if scale is None:
        scale = d ** -0.5
    qf, kf, vf = q.to(dtype), _repeat_kv(k.to(dtype), g), _repeat_kv(v.to(dtype), g)
    s = torch.einsum("ihd,jhd->hij", qf, kf) * scale
    m = _seq_mask(cu_seqlens, n, window)
    s = s.masked_fill(~m[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)                       # natural log
    p = torch.exp(s - lse[..., None])
    o = torch.einsum("hij,jhd->ihd", p, vf)
    lse2 = (lse * RCP_LN2).transpose(0, 1)                  # [N,HQ]
    if selection is not None:
        sel = selection.reshape(-1).to(torch.bool)
        o = o * sel[:, None, None].to(o.dtype)
    return o, lse2


def sq_full_attn_ref(q, k, v, selection, scale=None, cu_seqlens=None, dtype=torch.float32):
    """logo/ops/selected_full_attn.py:495-527 on [1,N,H,D] tensors; returns [1,N,HQ,Dv]."""
    assert q.dim() == 4 and q.shape[0] == 1 and cu_seqlens is not None
    o, _ = attention_dense_ref(q[0], k[0], v[0], [int(x) for x in cu_seqlens], scale, None, selection, dtype)
    return o[None]


def swa_ref(q, k, v, cu_seqlens, window: int, scale=None, dtype=torch.float32):
    """Local branch (logo/layers/logo.py:162-179): causal attention restricted to keys [i-window, i]."""
    o, _ = attention_dense_ref(q, k, v, [int(x) for x in cu_seqlens], scale, window, None, dtype)
    return o


# ---------------------------------------------------------------------------------------
# RMSNorm, gate mask, blend
# ---------------------------------------------------------------------------------------
def rmsnorm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """logo/modules/layernorm.py:17-22: fp32 normalise, round to the input dtype, then multiply by weight."""
    in_dtype = x.dtype
    xf = x.to(torch.float32)
    var = xf.pow(2).mean(-1, keepdim=True)
    xf = xf * torch.rsqrt(var + eps)
    return weight * xf.to(in_dtype)


def fuse_ref(local, glob, gate, thres, w_local, w_global, eps, use_context_norm=True):
    """logo/layers/logo.py:180-182,225-227,256-258.

    local, glob: [N,H,D]; gate: [N,1] (dtype of the activations); thres: scalar tensor.
    Returns [N, H*D] = (1-g)*norm_l(local) + g*norm_g(glob) with g = gate masked below thres.
    """
    n = local.shape[0]
    if use_context_norm:
        local = rmsnorm_ref(local, w_local, eps)
        glob = rmsnorm_ref(glob, w_global, eps)
    local = local.reshape(n, -1)
    glob = glob.reshape(n, -1)
    g = gate.masked_fill(gate < thres, 0.0)
    return (1 - g) * local + g * glob


# ---------------------------------------------------------------------------------------
# RoPE and the global re-parameterisation (inputs of the path; kept for the layer oracle)
# ---------------------------------------------------------------------------------------
def rope_cos_sin(positions: torch.Tensor, dim: int, theta: float = 10000.0, dtype=torch.float32):
    """logo/modules/rotary.py:57-78 with the default rope type: inv_freq = theta^(-2i/dim)."""
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    fr = positions.to(torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([fr, fr], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """logo/modules/rotary.py:81-106 for x [N,H,D], cos/sin [N,D]."""
    d = x.shape[-1]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    rot = torch.cat([-x2, x1], dim=-1)
    return x * cos[:, None, :] + rot * sin[:, None, :]


def logo_layer_ref(
    hidden: torch.Tensor,            # [N, hidden] packed tokens
    weights: Dict[str, torch.Tensor],
    cu_seqlens: Sequence[int],
    num_heads: int,
    num_kv_heads: int,
    window: int,
    gate_thres: float,
    eps: float,
    rope_theta: float = 10000.0,
    return_parts: bool = False,
    selection_override: Optional[torch.Tensor] = None,
):
    """logo/layers/logo.py:96-262 (either global_qk_param, chosen by the weight names), no cache, no dropout.

    ``weights`` uses the reference's parameter names (q_proj.weight, ..., q_global_proj,
    gate_proj.weight, context_norm_local.weight, context_norm_global.weight, o_proj.weight).
    ``selection_override`` (bool [N]) replaces the threshold test; the gate values themselves are
    still computed here. Tests use it to compare against a run whose gate was rounded differently.
    Returns the layer output [N, hidden] (and the intermediate tensors when asked).
    """
    n, hid = hidden.shape
    d = hid // num_heads
    cu = [int(x) for x in cu_seqlens]
    q = hidden @ weights["q_proj.weight"].T                      # :112-114
    k = hidden @ weights["k_proj.weight"].T
    v = hidden @ weights["v_proj.weight"].T
    qv, kv, vv = q.view(n, num_heads, d), k.view(n, num_kv_heads, d), v.view(n, num_kv_heads, d)
    if "q_global_scale" in weights:                                   # global_qk_param='scale_offset', :80-84
        gq = (q * weights["q_global_scale"] + weights["q_global_offset"]).view(n, num_heads, d)
        gk = (k * weights["k_global_scale"] + weights["k_global_offset"]).view(n, num_kv_heads, d)
        gv = (v * weights["v_global_scale"] + weights["v_global_offset"]).view(n, num_kv_heads, d)
    else:                                                             # 'linear_proj', :86-94
        gq = torch.einsum("lhd,hde->lhe", qv, weights["q_global_proj"])
        gk = torch.einsum("lhd,hde->lhe", kv, weights["k_global_proj"])
        gv = torch.einsum("lhd,hde->lhe", vv, weights["v_global_proj"])
    gate = torch.sigmoid(hidden @ weights["gate_proj.weight"].T)      # :130  [N,1]
    cu_t = torch.as_tensor(cu)
    idx = torch.arange(n)
    seg = torch.searchsorted(cu_t, idx, right=True) - 1
    pos = idx - cu_t[seg]
    cos, sin = rope_cos_sin(pos, d, rope_theta, hidden.dtype)        # :132-139
    ql, kl = apply_rope(qv, cos, sin), apply_rope(kv, cos, sin)
    gq, gk = apply_rope(gq, cos, sin), apply_rope(gk, cos, sin)
    local = swa_ref(ql, kl, vv, cu, window)                          # :166-179
    thres = torch.tensor(gate_thres, dtype=gate.dtype)
    selection = gate[:, 0] >= thres                                  # :190
    if selection_override is not None:
        selection = selection_override.reshape(-1).to(torch.bool)
        thres = torch.tensor(float("-inf"), dtype=gate.dtype)        # masked_fill below must not re-mask
        gate_for_blend = gate * selection[:, None].to(gate.dtype)
    else:
        gate_for_blend = gate
    glob, _ = attention_dense_ref(gq, gk, gv, cu, None, None, selection)   # :192-209
    fused = fuse_ref(local, glob, gate_for_blend, thres, weights["context_norm_local.weight"],
                     weights["context_norm_global.weight"], eps)     # :180-182,225-227,256-258
    out = fused @ weights["o_proj.weight"].T                         # :259
    if return_parts:
        return out, dict(gate=gate, selection=selection, local=local, glob=glob, fused=fused,
                         ql=ql, kl=kl, v=vv, gq=gq, gk=gk, gv=gv)
    return out


def dense_attention_layer_ref(hidden: torch.Tensor, weights: Dict[str, torch.Tensor], cu_seqlens: Sequence[int],
                              num_heads: int, num_kv_heads: int, rope_theta: float = 10000.0) -> torch.Tensor:
    """logo/layers/attn.py:54-121 (the dense causal layer of non-LoGo decoder layers), no cache, no dropout:
    projections, rotary embedding, full causal attention within each packed sequence, output projection.
    hidden [N, hidden] packed tokens; returns [N, hidden]."""
    n, hid = hidden.shape
    d = hid // num_heads
    cu = [int(x) for x in cu_seqlens]
    q = (hidden @ weights["q_proj.weight"].T).view(n, num_heads, d)        # :68-70
    k = (hidden @ weights["k_proj.weight"].T).view(n, num_kv_heads, d)
    v = (hidden @ weights["v_proj.weight"].T).view(n, num_kv_heads, d)
    cu_t = torch.as_tensor(cu)
    idx = torch.arange(n)
    pos = idx - cu_t[torch.searchsorted(cu_t, idx, right=True) - 1]
    cos, sin = rope_cos_sin(pos, d, rope_theta, hidden.dtype)             # :76-80
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o, _ = attention_dense_ref(q, k, v, cu, None, None, None)             # :102-114 (flash-attn, causal)
    return o.reshape(n, hid) @ weights["o_proj.weight"].T                 # :116-119


# ---------------------------------------------------------------------------------------
# decode step and the cache contract
# ---------------------------------------------------------------------------------------
def decode_attn_ref(q, k_cache, v_cache, ctx_lens, scale=None, window: Optional[int] = None,
                    active: Optional[torch.Tensor] = None):
    """One-token attention over a cache (logo/layers/logo.py:166-179 local, :228-249 global).

    q [B,HQ,D]; k_cache, v_cache [B,H,Tmax,D]; ctx_lens [B] = valid cached tokens INCLUDING the
    new one. window=w restricts to the last w+1 keys. Sequences with active == False give zeros
    (logo.py:248-249 and the masked gate of :256).
    """
    b, hq, d = q.shape
    h = k_cache.shape[1]
    g = hq // h
    if scale is None:
        scale = d ** -0.5
    out = torch.zeros(b, hq, v_cache.shape[-1], dtype=torch.float32)
    for i in range(b):
        if active is not None and not bool(active[i]):
            continue
        n = int(ctx_lens[i])
        lo = 0 if window is None else max(0, n - 1 - window)
        kk = k_cache[i, :, lo:n].to(torch.float32).repeat_interleave(g, dim=0)   # [HQ,t,D]
        vv = v_cache[i, :, lo:n].to(torch.float32).repeat_interleave(g, dim=0)
        s = torch.einsum("hd,htd->ht", q[i].to(torch.float32), kk) * scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.einsum("ht,htd->hd", p, vv)
    return out


class CacheRef:
    """logo/cache.py:46-124 restated with python lists of tensors ([B,H,t,D] states)."""

    def __init__(self):
        self.states: List[dict] = []
        self.seen = 0

    def update(self, attn_state, attn_state_full, layer_idx, offset, window_size):
        if layer_idx == 0:
            self.seen += offset                                       # :66-67
        for_attn = attn_state
        if len(self.states) <= layer_idx:                             # :79-92
            kc, vc = attn_state
            if kc.shape[-2] > window_size:
                kc, vc = kc[..., -window_size:, :].contiguous(), vc[..., -window_size:, :].contiguous()
            self.states.append(dict(attn_state=(kc, vc), attn_state_full=attn_state_full))
        else:                                                         # :95-118
            st = self.states[layer_idx]
            k0, v0 = st["attn_state"]
            for_attn = (torch.cat([k0, attn_state[0]], dim=-2), torch.cat([v0, attn_state[1]], dim=-2))
            kc, vc = for_attn
            if kc.shape[-2] > window_size:
                kc, vc = kc[..., -window_size:, :].contiguous(), vc[..., -window_size:, :].contiguous()
            st["attn_state"] = (kc, vc)
            kf, vf = st["attn_state_full"]
            st["attn_state_full"] = (torch.cat([kf, attn_state_full[0]], dim=-2),
                                     torch.cat([vf, attn_state_full[1]], dim=-2))
        out = dict(self.states[layer_idx])                            # :120-124
        out["attn_state"] = for_attn
        return out


# ---------------------------------------------------------------------------------------
# language-model loss
# ---------------------------------------------------------------------------------------
def lm_loss_ref(logits: torch.Tensor, labels: torch.Tensor, cu_seqlens: Optional[Sequence[int]] = None) -> torch.Tensor:
    """logo/modeling_logo.py:380-407: logits [B, T, V] (or [1, N, V] packed), labels like the tokens.
    Upcast, shift by one, do not predict across packed-sequence boundaries, mean cross-entropy."""
    vocab = logits.shape[-1]
    logits = logits.float()                                            # :385
    shift_logits = logits[..., :-1, :].contiguous().view(-1, vocab)    # :386-389
    shift_labels = labels[..., 1:].contiguous().view(-1).clone()       # :387-390
    if cu_seqlens is not None:
        cu = torch.as_tensor([int(x) for x in cu_seqlens], dtype=torch.int64)
        shift_labels[cu[1:-1] - 1] = -100                              # :392-394
    return torch.nn.functional.cross_entropy(shift_logits, shift_labels, ignore_index=-100)   # :406


# ---------------------------------------------------------------------------------------
# budget controller
# ---------------------------------------------------------------------------------------
def update_gate_thres_ref(gate_thres: np.ndarray, global_count: np.ndarray, total_count: np.ndarray,
                          target: float, rate: float) -> Tuple[np.ndarray, np.ndarray]:
    """logo/update.py:56-66: sign step on the thresholds of layers that saw tokens; returns (thres, ratio)."""
    gt = np.asarray(gate_thres, dtype=np.float32).copy()
    g = np.asarray(global_count, dtype=np.float32)
    t = np.asarray(total_count, dtype=np.float32)
    has = t > 0
    ratio = np.where(has, g / np.maximum(t, 1), 0).astype(np.float32)
    upd = np.float32(rate) * np.sign(ratio - np.float32(target))
    gt = gt + np.where(has, upd, 0).astype(np.float32)
    return gt, ratio


# ---------------------------------------------------------------------------------------
# error metrics (logo/ops/common.py:24-31)
# ---------------------------------------------------------------------------------------
def abs_err(x: torch.Tensor, y: torch.Tensor) -> float:
    return (x.detach().double() - y.detach().double()).abs().max().item()


def err_ratio(ref: torch.Tensor, out: torch.Tensor) -> float:
    r, o = ref.detach().double().flatten(), out.detach().double().flatten()
    return ((r - o).square().mean().sqrt() / (r.square().mean().sqrt() + 1e-8)).item()


def effective_flops_fwd(pos_ids: np.ndarray, hq: int, d: int) -> float:
    """4 * D * HQ * sum(pos + 1) over the selected rows: the algorithmic forward FLOPs."""
    return 4.0 * d * hq * float(np.sum(np.asarray(pos_ids, dtype=np.int64) + 1))
