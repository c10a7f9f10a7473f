"""Drop-in ``LoGoAttention`` layer over the sm_100a kernels.

Same constructor, parameter / buffer names and shapes, forward signature and return value as
the reference layer (``logo/layers/logo.py:34-262`` with its base class
``logo/layers/attn.py:22-52``), so a reference ``state_dict`` loads unchanged and
``LoGoDecoderLayer`` can call it as is. What differs is underneath:

* gate threshold test + compaction, query-sparse global attention, window local attention,
  the two context RMSNorms, the gate mask and the blend run in ``liblogo_b200.so``;
* nothing synchronises the host (the reference syncs in ``build_selection`` /
  ``prepare_chunk_indices`` and on ``active.any()``);
* both values of ``config.sparse_full_attn_backend`` use the query-sparse kernel: for tokens
  below the threshold the gate is exactly 0, so skipping their global rows gives the same
  layer output as the reference's dense ``"flash"`` backend;
* decode (``q_len == 1`` with a cache) skips the global branch per sequence instead of running
  it for the whole batch whenever any gate passes (``logo.py:229-249``).

Not provided (as in the reference's ``"triton"`` backend, ``logo.py:189-209``): padding
``attention_mask`` handling and attention dropout; activations must be bf16 and head_dim 128.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

import os

from . import _lib, ops
from .cache import Cache

# LOGO_B200_CHECK_STATUS=1: every layer call reads the device status word afterwards (this
# synchronises) and raises if a kernel reported a problem. Off by default: the layers never sync.
_CHECK_STATUS = os.environ.get("LOGO_B200_CHECK_STATUS", "0") not in ("", "0")

__all__ = ["Attention", "LoGoAttention", "RMSNorm", "RotaryEmbedding", "apply_rotary_pos_emb", "check_status",
           "rotate_half"]


class RMSNorm(nn.Module):
    """Parameter holder with the reference's RMSNorm surface (logo/modules/layernorm.py:11-25).

    The LoGo layer feeds ``weight`` / ``variance_epsilon`` to the fused kernel; ``forward`` is the
    plain torch formula for callers that use the module on its own.
    """

    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        # inference on bf16 CUDA tensors: one kernel with the same roundings as the expression below
        if (hidden_states.is_cuda and hidden_states.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16
                and hidden_states.shape[-1] % 8 == 0
                and not (torch.is_grad_enabled() and (hidden_states.requires_grad or self.weight.requires_grad))):
            return ops.rmsnorm(hidden_states, self.weight, self.variance_epsilon)
        input_dtype = hidden_states.dtype
        hidden_states = hidden_states.to(torch.float32)
        variance = hidden_states.pow(2).mean(-1, keepdim=True)
        hidden_states = hidden_states * torch.rsqrt(variance + self.variance_epsilon)
        return self.weight * hidden_states.to(input_dtype)

    def extra_repr(self) -> str:
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


class RotaryEmbedding(nn.Module):
    """Default-type RoPE tables (logo/modules/rotary.py:16-78): inv_freq = theta ** (-2i / dim)."""

    def __init__(self, config, device=None):
        super().__init__()
        scaling = getattr(config, "rope_scaling", None)
        if isinstance(scaling, dict):     # transformers >= 5 fills in {"rope_type": "default", ...} by itself
            kind = scaling.get("rope_type", scaling.get("type", "default"))
        else:
            kind = "default" if scaling is None else str(scaling)
        if kind != "default":
            raise NotImplementedError("only the default rope type is built in; pass position_embeddings for others")
        self.rope_type = "default"
        self.max_seq_len_cached = config.max_position_embeddings
        self.original_max_seq_len = config.max_position_embeddings
        self.config = config
        self.attention_scaling = 1.0
        self.register_buffer("inv_freq", self._make_inv_freq(device), persistent=False)
        self._inv_freq_fp32 = {}

    def _make_inv_freq(self, device) -> torch.Tensor:
        dim = self.config.hidden_size // self.config.num_attention_heads
        return 1.0 / (self.config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float().to(device) / dim))

    # `module.to(torch.bfloat16)` also casts the `inv_freq` buffer, which costs the rotation angle about
    # three decimal digits at position ~500. By default the tables are built from an fp32 copy. The
    # reference uses the cast buffer as it is (logo/modules/rotary.py:66-71): set this to True to
    # reproduce the angles a checkpoint saw if it was trained through a bf16-cast reference model.
    use_cast_inv_freq = False

    def _inv_freq_for(self, device) -> torch.Tensor:
        if self.use_cast_inv_freq:
            return self.inv_freq.float()
        if self.inv_freq.dtype == torch.float32 and self.inv_freq.device == device:
            return self.inv_freq
        key = str(device)
        if key not in self._inv_freq_fp32:
            self._inv_freq_fp32[key] = self._make_inv_freq(device)
        return self._inv_freq_fp32[key]

    @torch.no_grad()
    def forward(self, x: torch.Tensor, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        inv = self._inv_freq_for(x.device)[None, :, None].expand(position_ids.shape[0], -1, 1)
        pos = position_ids[:, None, :].float()
        with torch.autocast(device_type=x.device.type, enabled=False):
            freqs = (inv @ pos).transpose(1, 2)
            emb = torch.cat((freqs, freqs), dim=-1)
            cos, sin = emb.cos(), emb.sin()
        return cos.to(dtype=x.dtype), sin.to(dtype=x.dtype)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1 = x[..., : x.shape[-1] // 2]
    x2 = x[..., x.shape[-1] // 2:]
    return torch.cat((-x2, x1), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim: int = 1):
    """logo/modules/rotary.py:88-106."""
    cos = cos.unsqueeze(unsqueeze_dim)
    sin = sin.unsqueeze(unsqueeze_dim)
    return (q * cos) + (rotate_half(q) * sin), (k * cos) + (rotate_half(k) * sin)


class LoGoAttention(nn.Module):
    """Token-level dynamic local-global attention (drop-in for ``logo.layers.LoGoAttention``)."""

    def __init__(self, config, layer_idx: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx

        # logo/layers/attn.py:27-52
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.max_position_embeddings = config.max_position_embeddings
        self.rope_theta = config.rope_theta
        self.is_causal = True
        self.attention_dropout = config.attention_dropout
        if (self.head_dim * self.num_heads) != self.hidden_size:
            raise ValueError(
                f"hidden_size must be divisible by num_heads (got `hidden_size`: {self.hidden_size}"
                f" and `num_heads`: {self.num_heads})."
            )
        if self.head_dim != ops.HEAD_DIM:
            raise NotImplementedError(f"the CUDA kernels implement head_dim {ops.HEAD_DIM} only, got {self.head_dim}")
        if self.attention_dropout != 0.0:
            raise NotImplementedError("attention dropout is not implemented (the reference's sparse path ignores it)")
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=config.attention_bias)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=config.attention_bias)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=config.attention_bias)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=config.attention_out_bias)
        self.resid_dropout = nn.Dropout(config.resid_pdrop)
        self.rotary_emb = RotaryEmbedding(config=config)

        # logo/layers/logo.py:40-78
        self.local_window_size = config.window_size
        self.global_qk_param = config.global_qk_param
        if self.global_qk_param == "scale_offset":
            self.q_global_scale = nn.Parameter(torch.ones(self.num_heads * self.head_dim))
            self.q_global_offset = nn.Parameter(torch.zeros(self.num_heads * self.head_dim))
            self.k_global_scale = nn.Parameter(torch.ones(self.num_key_value_heads * self.head_dim))
            self.k_global_offset = nn.Parameter(torch.zeros(self.num_key_value_heads * self.head_dim))
            self.v_global_scale = nn.Parameter(torch.ones(self.num_key_value_heads * self.head_dim))
            self.v_global_offset = nn.Parameter(torch.zeros(self.num_key_value_heads * self.head_dim))
            self._transform_qkv = self._scale_offset_qkv
        elif self.global_qk_param == "linear_proj":
            eye = torch.eye(self.head_dim)
            self.q_global_proj = nn.Parameter(eye.unsqueeze(0).repeat(self.num_heads, 1, 1))
            self.k_global_proj = nn.Parameter(eye.unsqueeze(0).repeat(self.num_key_value_heads, 1, 1))
            self.v_global_proj = nn.Parameter(eye.unsqueeze(0).repeat(self.num_key_value_heads, 1, 1))
            self._transform_qkv = self._linear_proj_qkv
        else:
            raise ValueError(f"unknown global_qk_param {self.global_qk_param!r}")

        self.gate_proj = nn.Linear(self.hidden_size, 1, bias=False)
        self.use_context_norm = config.use_context_norm
        if self.use_context_norm:
            self.context_norm_local = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
            self.context_norm_global = RMSNorm(self.head_dim, eps=config.rms_norm_eps)
        self.sparse_full_attn_backend = config.sparse_full_attn_backend
        self.register_buffer("gate_thres", torch.full((1,), float(config.gate_thres_init)))
        self.register_buffer("gate_avg", torch.zeros(1), persistent=False)
        self.register_buffer("global_token_count", torch.zeros(1), persistent=False)
        self.register_buffer("total_token_count", torch.zeros(1), persistent=False)

    # -- global re-parameterisation (logo/layers/logo.py:80-94) ----------------------------------
    def _scale_offset_qkv(self, q, k, v):
        q = q * self.q_global_scale.view(1, 1, -1) + self.q_global_offset.view(1, 1, -1)
        k = k * self.k_global_scale.view(1, 1, -1) + self.k_global_offset.view(1, 1, -1)
        v = v * self.v_global_scale.view(1, 1, -1) + self.v_global_offset.view(1, 1, -1)
        return q, k, v

    def _linear_proj_qkv(self, q, k, v):
        bsz, q_len, _ = q.size()
        q_view = q.view(bsz, q_len, self.num_heads, self.head_dim)
        k_view = k.view(bsz, q_len, self.num_key_value_heads, self.head_dim)
        v_view = v.view(bsz, q_len, self.num_key_value_heads, self.head_dim)
        # [B, L, H, E] results (views of the head-major buffers the batched product writes): the rotary
        # kernel reads q / k through their strides, only v is packed here
        q_out = torch.einsum("b l h d, h d e -> b l h e", q_view, self.q_global_proj)
        k_out = torch.einsum("b l h d, h d e -> b l h e", k_view, self.k_global_proj)
        v_out = torch.einsum("b l h d, h d e -> b l h e", v_view, self.v_global_proj)
        return q_out, k_out, v_out.reshape(bsz, q_len, -1)

    # -- forward -----------------------------------------------------------------------------------
    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: Optional[torch.LongTensor] = None,
        position_ids: Optional[torch.LongTensor] = None,
        cu_seqlens: Optional[torch.IntTensor] = None,
        past_key_value=None,
        output_attentions: bool = False,
        use_cache: bool = False,
        cache_position: Optional[torch.LongTensor] = None,
        position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        max_seqlen: Optional[int] = None,
        **kwargs,
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[object]]:
        if not hidden_states.is_cuda:
            raise RuntimeError("logo_b200.LoGoAttention runs on CUDA only; there is no CPU fallback")
        bsz, q_len, _ = hidden_states.size()
        H, HKV, D = self.num_heads, self.num_key_value_heads, self.head_dim

        query_states = self.q_proj(hidden_states)
        key_states = self.k_proj(hidden_states)
        value_states = self.v_proj(hidden_states)
        gate = torch.sigmoid(self.gate_proj(hidden_states))              # [B, T, 1]
        if query_states.dtype != torch.bfloat16:
            raise TypeError("logo_b200.LoGoAttention needs bf16 activations (cast the model or use autocast)")
        n_tok = bsz * q_len
        is_decode = past_key_value is not None and q_len == 1
        filled = 0
        if past_key_value is not None:
            if not isinstance(past_key_value, Cache):
                raise TypeError("the cache must be a logo_b200.Cache")
            filled = (past_key_value.layers[self.layer_idx].length
                      if len(past_key_value.layers) > self.layer_idx else 0)
        # Prefill / training with the per-head projection: one kernel per global tensor does projection,
        # rotary embedding and layout, and the query projection runs over the selected rows only. Decode
        # steps, continuations of a filled cache and the scale / offset parameterisation take the eager route.
        fused_proj = self.global_qk_param == "linear_proj" and not is_decode and filled == 0

        # token-major [B, T, H, D]: the layout the kernels consume, no transposes
        q_l = query_states.view(bsz, q_len, H, D)
        k_l = key_states.view(bsz, q_len, HKV, D)
        v_l = value_states.view(bsz, q_len, HKV, D)

        if position_embeddings is None:
            cos, sin = self.rotary_emb(v_l, position_ids)
        else:
            cos, sin = position_embeddings
        # rotary embedding of both branches (logo/layers/logo.py:136-139): one kernel per tensor
        # tables may come with a broadcast batch of 1 (the reference multiplies with broadcasting)
        cos2 = cos.expand(bsz, q_len, D).reshape(n_tok, D).to(torch.bfloat16)
        sin2 = sin.expand(bsz, q_len, D).reshape(n_tok, D).to(torch.bfloat16)
        gate_flat = gate.reshape(-1).to(torch.bfloat16)
        sel = None
        if fused_proj:
            if cu_seqlens is not None:
                cu = cu_seqlens
            else:  # equal-length batch packed to one varlen batch (logo.py:200-209)
                cu = torch.arange(0, (bsz + 1) * q_len, q_len, dtype=torch.int32, device=hidden_states.device)
            sel = ops.select_rows(gate_flat, self.gate_thres, cu)
            q_g = ops.proj_rope(query_states.view(n_tok, H, D), self.q_global_proj, cos2, sin2, sel).view(bsz, q_len, H, D)
            k_g = ops.proj_rope(key_states.view(n_tok, HKV, D), self.k_global_proj, cos2, sin2).view(bsz, q_len, HKV, D)
            v_g = ops.proj_rope(value_states.view(n_tok, HKV, D), self.v_global_proj).view(bsz, q_len, HKV, D)
        else:
            gq, gk, gv = self._transform_qkv(query_states, key_states, value_states)
            q_g, k_g, v_g = gq.reshape(bsz, q_len, H, D), gk.reshape(bsz, q_len, HKV, D), gv.view(bsz, q_len, HKV, D)
            q_g = ops.rope(q_g.reshape(n_tok, H, D), cos2, sin2).view(bsz, q_len, H, D)
            k_g = ops.rope(k_g.reshape(n_tok, HKV, D), cos2, sin2).view(bsz, q_len, HKV, D)
        q_l = ops.rope(q_l.reshape(n_tok, H, D), cos2, sin2).view(bsz, q_len, H, D)
        k_l = ops.rope(k_l.reshape(n_tok, HKV, D), cos2, sin2).view(bsz, q_len, HKV, D)

        scale = D ** -0.5
        thres = self.gate_thres
        w_l = self.context_norm_local.weight if self.use_context_norm else None
        w_g = self.context_norm_global.weight if self.use_context_norm else None
        eps = self.context_norm_local.variance_epsilon if self.use_context_norm else 0.0

        if is_decode:
            if not isinstance(past_key_value, Cache):
                raise TypeError("decode needs a logo_b200.Cache")
            st = past_key_value.append(self.layer_idx, k_l, v_l, k_g, v_g, self.local_window_size, layout="bthd")
            local, glob = decode_attention(q_l.reshape(bsz, H, D), q_g.reshape(bsz, H, D), st, gate_flat, thres, scale)
            self._last_status = st.status
            fused = ops.fuse_norm_blend(local, glob, gate_flat, thres, w_l, w_g, eps, self.use_context_norm)
        else:
            n = bsz * q_len
            if filled != 0:
                # several new tokens on top of cached ones (chunked prefill, logo/cache.py:95-118)
                if cu_seqlens is not None:
                    raise NotImplementedError("a packed batch cannot continue a cache: pass [B, T] inputs")
                local, glob, sel = _continue_with_cache(past_key_value, self.layer_idx, q_l, k_l, v_l, q_g, k_g, v_g,
                                                        gate_flat, thres, self.local_window_size, scale)
            else:
                if past_key_value is not None:
                    past_key_value.append(self.layer_idx, k_l, v_l, k_g, v_g, self.local_window_size, layout="bthd")
                if sel is None:
                    if cu_seqlens is not None:
                        cu = cu_seqlens
                    else:  # equal-length batch packed to one varlen batch (logo.py:200-209)
                        cu = torch.arange(0, (bsz + 1) * q_len, q_len, dtype=torch.int32, device=hidden_states.device)
                    sel = ops.select_rows(gate_flat, thres, cu)
                local = ops.SWAFunction.apply(q_l.reshape(n, H, D), k_l.reshape(n, HKV, D), v_l.reshape(n, HKV, D),
                                              self.local_window_size, scale, sel)
                glob = ops.SQFullAttentionFunction.apply(q_g.reshape(1, n, H, D), k_g.reshape(1, n, HKV, D),
                                                         v_g.reshape(1, n, HKV, D), scale, sel).view(n, H, D)
            self._last_status = sel.status
            fused = ops.fuse_norm_blend(local, glob, gate_flat, thres, w_l, w_g, eps, self.use_context_norm)
            if self.training:   # logo.py:251-255, from the select kernel's by-products (no sync)
                with torch.no_grad():
                    if filled != 0:   # the continuation's selection also lists (never selected) cached rows
                        self.gate_avg.add_(gate.sum().to(self.gate_avg.dtype))
                    else:
                        self.gate_avg.add_(sel.gate_sum.to(self.gate_avg.dtype))
                    self.global_token_count.add_(sel.meta[0].to(self.global_token_count.dtype))
                    self.total_token_count.add_(gate.numel())

        if is_decode and self.training:
            with torch.no_grad():
                self.gate_avg.add_(gate.sum().to(self.gate_avg.dtype))
                self.global_token_count.add_((gate >= thres).sum().to(self.global_token_count.dtype))
                self.total_token_count.add_(gate.numel())

        if _CHECK_STATUS:
            ops.check_device_status(self._last_status, f"LoGoAttention layer {self.layer_idx}")
        attn_output = self.o_proj(fused.view(bsz, q_len, H * D))
        attn_output = self.resid_dropout(attn_output)
        return attn_output, None, past_key_value


def _continue_with_cache(cache, layer_idx, q_l, k_l, v_l, q_g, k_g, v_g, gate_flat, thres, window, scale):
    """Both branches for ``t`` new tokens per sequence on top of ``T0`` cached ones (inference only).

    The reference concatenates the cached states with the new ones and lets flash-attn align the
    causal mask to the bottom right (logo/cache.py:95-118, logo/layers/logo.py:141-179). Here the
    cached keys / values are laid out token-major in front of the new ones, each sequence becomes one
    packed sequence of ``T0 + t`` (global) or ``min(T0, window) + t`` (local) tokens whose leading
    rows carry no query, and the ordinary kernels run: the select kernel is given a gate of -inf
    for the cached rows, so the global branch computes the new selected rows only.
    Inputs are ``[B, t, H, D]`` (rotary embedding applied); returns ``(local, glob, sel)`` with
    ``local``, ``glob`` ``[B * t, H, D]``.
    """
    if torch.is_grad_enabled() and any(x.requires_grad for x in (q_l, k_l, v_l, q_g, k_g, v_g)):
        raise NotImplementedError("continuing a cache with several tokens is an inference path (run it under no_grad)")
    bsz, t, H, D = q_l.shape
    st = cache.layers[layer_idx]
    T0 = st.length
    w0 = min(T0, window)
    dev = q_l.device
    with torch.no_grad():
        if window > 0:
            old_kl, old_vl = cache._local_window(st, T0, window)              # [B, HKV, w0, D]
        cache.append(layer_idx, k_l, v_l, k_g, v_g, window, layout="bthd")
        st = cache.layers[layer_idx]

        def packed(old_bhtd, new_bthd):                                      # -> [B * (t_old + t), heads, D]
            return torch.cat([old_bhtd.transpose(1, 2), new_bthd], dim=1).reshape(-1, new_bthd.shape[2], D)

        # local branch: the last w0 cached tokens + the new ones, every row computed, cached rows dropped
        local = None
        if window > 0:          # (the dense layer has no local branch and passes window 0)
            zq = torch.zeros(bsz, w0, H, D, dtype=q_l.dtype, device=dev)
            ql = torch.cat([zq, q_l], dim=1).reshape(-1, H, D)
            kl, vl = packed(old_kl, k_l), packed(old_vl, v_l)
            cu_l = torch.arange(0, (bsz + 1) * (w0 + t), w0 + t, dtype=torch.int32, device=dev)
            sel_l = ops.select_rows(torch.ones(ql.shape[0], dtype=torch.bool, device=dev), None, cu_l)
            lo, _ = ops.swa_fwd_raw(ql, kl, vl, sel_l, window, scale)
            local = lo.view(bsz, w0 + t, H, D)[:, w0:].reshape(bsz * t, H, D)

        # global branch: the whole cache (it already holds the new tokens) token-major
        kg = st.k_full[:, :, : T0 + t].transpose(1, 2).reshape(-1, st.k_full.shape[1], D)
        vg = st.v_full[:, :, : T0 + t].transpose(1, 2).reshape(-1, st.v_full.shape[1], D)
        zq = torch.zeros(bsz, T0, H, D, dtype=q_g.dtype, device=dev)
        qg = torch.cat([zq, q_g], dim=1).reshape(-1, H, D)
        gate_ext = torch.full((bsz, T0 + t), float("-inf"), dtype=gate_flat.dtype, device=dev)
        gate_ext[:, T0:] = gate_flat.view(bsz, t)
        cu_g = torch.arange(0, (bsz + 1) * (T0 + t), T0 + t, dtype=torch.int32, device=dev)
        sel = ops.select_rows(gate_ext.reshape(-1), thres, cu_g)
        go, _ = ops.sq_attn_fwd_raw(qg, kg, vg, sel, scale, zero_fill=True)
        glob = go.view(bsz, T0 + t, H, D)[:, T0:].reshape(bsz * t, H, D)
    return local, glob, sel


def check_status(obj) -> None:
    """Raises if a kernel launched on behalf of ``obj`` left an error in its device status word.

    ``obj`` is a module tree holding LoGo layers (the status of each layer's most recent call is
    looked at) or a :class:`logo_b200.Cache`. The layers themselves never read the word, because
    reading it synchronises the host with the device; call this at a point where a sync is
    acceptable (end of a step, after generation), or set ``LOGO_B200_CHECK_STATUS=1`` to check after
    every layer call while debugging.
    """
    if isinstance(obj, Cache):
        for i, st in enumerate(obj.layers):
            if st.status is not None:
                ops.check_device_status(st.status, f"cache layer {i}")
        return
    for name, mod in obj.named_modules():
        status = getattr(mod, "_last_status", None)
        if status is not None:
            ops.check_device_status(status, f"layer {name or type(mod).__name__}")


def decode_attention(q_local, q_global, st, gate_flat, thres, scale: float):
    """One-token attention of both branches over a layer's cache buffers (no autograd).

    q_local, q_global ``[B, HQ, D]`` bf16; ``st`` a layer state of :class:`logo_b200.Cache`` that
    already holds the new token. Returns ``(o_local, o_global)`` as ``[B, HQ, D]`` bf16;
    ``o_global`` is 0 for sequences whose gate is below the threshold.
    """
    lib = _lib.load()
    b, hq, d = q_local.shape
    h = st.k_full.shape[1]
    dev = q_local.device
    q_local, q_global = q_local.contiguous(), q_global.contiguous()
    o_local = torch.empty(b, hq, d, dtype=torch.bfloat16, device=dev)
    o_global = torch.empty_like(o_local)
    ctx = torch.full((b,), st.length, dtype=torch.int32, device=dev)
    thres = thres.reshape(-1)[:1].contiguous()
    ws_bytes = lib.logo_decode_workspace_bytes(b, hq, st.length)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with _lib.on_device(q_local):
        rc = lib.logo_decode_attn(q_local.data_ptr(), q_global.data_ptr(), st.k_ring.data_ptr(), st.v_ring.data_ptr(),
                                  st.ring, st.k_full.data_ptr(), st.v_full.data_ptr(), st.t_max, ctx.data_ptr(),
                                  gate_flat.data_ptr(), _lib.torch_dtype_code(gate_flat.dtype), thres.data_ptr(),
                                  _lib.torch_dtype_code(thres.dtype), o_local.data_ptr(), o_global.data_ptr(), b, hq,
                                  h, d, st.length, float(scale), ws.data_ptr(), ws.numel(), st.status.data_ptr(),
                                  _lib.current_stream_ptr(dev))
    _lib.check(rc, "logo_decode_attn")
    return o_local, o_global


class Attention(nn.Module):
    """Dense causal attention layer (drop-in for ``logo.layers.attn.Attention``, logo/layers/attn.py:22-121).

    Used for layers whose ``attn_type_list`` entry is non-zero. It runs on the same kernels as the LoGo
    layer: rotary kernel, then full causal attention as the all-rows path of the attention kernels with
    a window that covers any sequence; a one-token step attends over the in-place cache with the decode
    kernel (every sequence active).
    """

    _FULL_WINDOW = 1 << 30

    def __init__(self, config, layer_idx: Optional[int] = None):
        super().__init__()
        self.config = config
        self.layer_idx = layer_idx
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.num_key_value_groups = self.num_heads // self.num_key_value_heads
        self.max_position_embeddings = config.max_position_embeddings
        self.rope_theta = config.rope_theta
        self.is_causal = True
        self.attention_dropout = config.attention_dropout
        if (self.head_dim * self.num_heads) != self.hidden_size:
            raise ValueError(
                f"hidden_size must be divisible by num_heads (got `hidden_size`: {self.hidden_size}"
                f" and `num_heads`: {self.num_heads})."
            )
        if self.head_dim != ops.HEAD_DIM:
            raise NotImplementedError(f"the CUDA kernels implement head_dim {ops.HEAD_DIM} only, got {self.head_dim}")
        if self.attention_dropout != 0.0:
            raise NotImplementedError("attention dropout is not implemented")
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=config.attention_bias)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=config.attention_bias)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=config.attention_bias)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=config.attention_out_bias)
        self.resid_dropout = nn.Dropout(config.resid_pdrop)
        self.rotary_emb = RotaryEmbedding(config=config)

    def forward(
        self,
        hidden_states: torch.Tensor,
        attention_mask: Optional[torch.Tensor] = None,
        position_ids: Optional[torch.LongTensor] = None,
        cu_seqlens: Optional[torch.IntTensor] = None,
        past_key_value=None,
        output_attentions: bool = False,
        use_cache: bool = False,
        cache_position: Optional[torch.LongTensor] = None,
        position_embeddings: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
        max_seqlen: Optional[int] = None,
        **kwargs,
    ) -> Tuple[torch.Tensor, Optional[torch.Tensor], Optional[object]]:
        if not hidden_states.is_cuda:
            raise RuntimeError("logo_b200.Attention runs on CUDA only; there is no CPU fallback")
        bsz, q_len, _ = hidden_states.size()
        H, HKV, D = self.num_heads, self.num_key_value_heads, self.head_dim
        query_states = self.q_proj(hidden_states)
        key_states = self.k_proj(hidden_states)
        value_states = self.v_proj(hidden_states)
        if query_states.dtype != torch.bfloat16:
            raise TypeError("logo_b200.Attention needs bf16 activations (cast the model or use autocast)")
        v = value_states.view(bsz, q_len, HKV, D)
        if position_embeddings is None:
            cos, sin = self.rotary_emb(v, position_ids)
        else:
            cos, sin = position_embeddings
        n_tok = bsz * q_len
        # tables may come with a broadcast batch of 1 (the reference multiplies with broadcasting)
        cos2 = cos.expand(bsz, q_len, D).reshape(n_tok, D).to(torch.bfloat16)
        sin2 = sin.expand(bsz, q_len, D).reshape(n_tok, D).to(torch.bfloat16)
        q = ops.rope(query_states.view(n_tok, H, D), cos2, sin2)          # [N, H, D]
        k = ops.rope(key_states.view(n_tok, HKV, D), cos2, sin2)
        scale = D ** -0.5

        if past_key_value is not None and q_len == 1:
            if not isinstance(past_key_value, Cache):
                raise TypeError("decode needs a logo_b200.Cache")
            kb, vb = k.view(bsz, 1, HKV, D), v
            # the decode kernel serves both LoGo branches: give it a one-entry local ring and use its
            # global output with every sequence active
            st = past_key_value.append(self.layer_idx, kb, vb, kb, vb, 0, layout="bthd")
            ones = torch.ones(bsz, dtype=torch.bfloat16, device=q.device)
            zero = torch.zeros(1, dtype=torch.float32, device=q.device)
            qd = q.view(bsz, H, D)
            _, out = decode_attention(qd, qd, st, ones, zero, scale)
            out = out.view(bsz, 1, H * D)
        else:
            filled = 0
            if past_key_value is not None:
                if not isinstance(past_key_value, Cache):
                    raise TypeError("the cache must be a logo_b200.Cache")
                filled = (past_key_value.layers[self.layer_idx].length
                          if len(past_key_value.layers) > self.layer_idx else 0)
            if filled != 0:
                if cu_seqlens is not None:
                    raise NotImplementedError("a packed batch cannot continue a cache: pass [B, T] inputs")
                # several new tokens on top of cached ones: the global-branch route of the LoGo layer
                # with every new row selected
                qb, kb = q.view(bsz, q_len, H, D), k.view(bsz, q_len, HKV, D)
                ones = torch.ones(bsz * q_len, dtype=torch.bfloat16, device=q.device)
                zero = torch.zeros(1, dtype=torch.float32, device=q.device)
                _, out, _ = _continue_with_cache(past_key_value, self.layer_idx, qb, kb, v, qb, kb, v, ones, zero, 0, scale)
                out = out.view(bsz, q_len, H * D)
            else:
                if past_key_value is not None:
                    kb = k.view(bsz, q_len, HKV, D)
                    past_key_value.append(self.layer_idx, kb, v, kb, v, 0, layout="bthd")
                if cu_seqlens is not None:
                    cu = cu_seqlens
                else:
                    cu = torch.arange(0, (bsz + 1) * q_len, q_len, dtype=torch.int32, device=hidden_states.device)
                out = ops.swa_attn(q, k, v.reshape(n_tok, HKV, D), cu, self._FULL_WINDOW, scale).view(bsz, q_len, H * D)

        attn_output = self.o_proj(out)
        attn_output = self.resid_dropout(attn_output)
        return attn_output, None, past_key_value
