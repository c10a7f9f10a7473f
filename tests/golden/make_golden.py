"""Generates the golden fixtures in this directory by running the REFERENCE's own code.

Run once, where a checkout of the reference is available (its path in ``LOGO_REFERENCE``); the
resulting ``*.npz`` files are committed and are all the tests need.

    LOGO_REFERENCE=<reference checkout> python tests/golden/make_golden.py [fixture ...]

The reference is imported unmodified. Four shims make it runnable without a GPU and with the
installed transformers 5.x (the reference pins < 4.52):
  a. register a ``"default"`` rope initialiser (dropped from ROPE_INIT_FUNCTIONS in 5.x);
  b. replace ``logo.layers.logo.flash_attention_forward`` (a thin wrapper over the third-party
     flash-attn wheel, which needs a GPU) by a dense-masked fp32 attention with flash-attn's
     documented semantics (causal, bottom-right aligned, window ``[i - w, i]``, packed sequences);
  c. make ``transformers.cache_utils.Cache.__init__`` accept the reference's bare ``super().__init__()``;
  d. run the reference's Triton kernels under the Triton interpreter, re-binding its module-level
     ``exp2`` / ``log2`` aliases to ``@triton.jit`` wrappers the interpreter accepts.
All inputs come from ``numpy.random.RandomState`` seeds so that tests can regenerate them.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch
import triton
import triton.language as tl

REF = os.environ.get("LOGO_REFERENCE")
if not REF or not Path(REF, "logo").is_dir():
    raise SystemExit("set LOGO_REFERENCE to a checkout of the reference (the directory that contains logo/)")
OUT = Path(__file__).resolve().parent
sys.path.insert(0, REF)
sys.path.insert(0, str(OUT))

from golden_inputs import (attn_case_inputs, layer_case_inputs, selection_cases, layer_weights,  # noqa: E402
                           dense_attn_inputs, dense_attn_weights, model_inputs, model_weights, ATTN_CASES,
                           DENSE_ATTN_CASE, LAYER_CASES, MODEL_CASE)


@triton.jit
def _exp2(x):
    return tl.math.exp2(x)


@triton.jit
def _log2(x):
    return tl.log2(x)


def install_shims():
    import transformers
    from transformers import modeling_rope_utils as mru

    def default_rope(config, device=None, seq_len=None, **kw):
        dim = config.hidden_size // config.num_attention_heads
        inv = 1.0 / (config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float().to(device) / dim))
        return inv, 1.0

    mru.ROPE_INIT_FUNCTIONS.setdefault("default", default_rope)
    transformers.cache_utils.Cache.__init__ = lambda self, *a, **k: None

    import logo.ops.selected_full_attn as sfa

    sfa.exp2 = _exp2
    sfa.log2 = _log2

    import logo.layers.logo as ll

    def dense_flash(q, k, v, attention_mask, query_length, is_causal=True, dropout=0.0, position_ids=None,
                    cu_seqlens=None, softmax_scale=None, sliding_window=None, **kw):
        # q [B,Tq,H,D], k/v [B,Tk,Hkv,D]
        B, Tq, H, D = q.shape
        Tk, Hkv = k.shape[1], k.shape[2]
        g = H // Hkv
        scale = softmax_scale if softmax_scale is not None else D ** -0.5
        kk = k.repeat_interleave(g, dim=2).float()
        vv = v.repeat_interleave(g, dim=2).float()
        s = torch.einsum("bihd,bjhd->bhij", q.float(), kk) * scale
        i = torch.arange(Tq)[:, None] + (Tk - Tq)
        j = torch.arange(Tk)[None, :]
        m = j <= i
        if sliding_window is not None and Tk > sliding_window:
            m = m & (j >= i - sliding_window)
        if cu_seqlens is not None:
            cu = cu_seqlens.to(torch.int64)
            seg = torch.searchsorted(cu, torch.arange(Tk), right=True) - 1
            m = m & (seg[:, None] == seg[None, :])
        s = s.masked_fill(~m[None, None], float("-inf"))
        o = torch.einsum("bhij,bjhd->bihd", torch.softmax(s, dim=-1), vv).to(q.dtype)
        return o.squeeze(0) if cu_seqlens is not None else o

    ll.flash_attention_forward = dense_flash
    import logo.layers.attn as la

    la.flash_attention_forward = dense_flash     # the dense layer calls the same wrapper (attn.py:102)


def gen_selection():
    from logo.ops.common import build_selection, prepare_chunk_indices
    from logo.ops.selected_full_attn import _compute_q_start_blk
    out = {}
    for name, (mask, cu) in selection_cases().items():
        sel = build_selection(torch.from_numpy(mask)[None], 1, mask.size, torch.tensor(cu, dtype=torch.int32))
        ck = prepare_chunk_indices(sel.cu_seqlens_k, 128)
        out[f"{name}/q_idx"] = sel.q_idx.numpy()
        out[f"{name}/pos_ids"] = sel.pos_ids.numpy()
        out[f"{name}/cu_seqlens_q"] = sel.cu_seqlens_q.numpy()
        out[f"{name}/chunks_q128"] = prepare_chunk_indices(sel.cu_seqlens_q, 128).numpy()
        out[f"{name}/chunks_k128"] = ck.numpy()
        out[f"{name}/q_start_blk"] = _compute_q_start_blk(sel.pos_ids, sel, ck, 128).numpy()
    np.savez_compressed(OUT / "selection.npz", **out)
    print("selection.npz", len(out))


def gen_attention():
    from logo.ops import sq_full_attn
    out = {}
    for name in ATTN_CASES:
        q, k, v, do, sel, cu = attn_case_inputs(name)
        qt, kt, vt = (torch.from_numpy(x)[None].requires_grad_(True) for x in (q, k, v))
        o = sq_full_attn(qt, kt, vt, torch.from_numpy(sel)[None], cu_seqlens=torch.tensor(cu, dtype=torch.int32))
        o.backward(torch.from_numpy(do)[None])
        out[f"{name}/o"] = o.detach()[0].numpy()
        out[f"{name}/dq"] = qt.grad[0].numpy()
        out[f"{name}/dk"] = kt.grad[0].numpy()
        out[f"{name}/dv"] = vt.grad[0].numpy()
        print(name, "Sq", int(sel.sum()), "o abs max", float(np.abs(out[f'{name}/o']).max()))
    np.savez_compressed(OUT / "attention.npz", **out)


def build_ref_layer(case):
    from logo.configuration_logo import LoGoConfig
    from logo.layers.logo import LoGoAttention
    cfg = LoGoConfig(hidden_size=case["hidden"], num_attention_heads=case["heads"],
                     num_key_value_heads=case["kv_heads"], window_size=case["window"],
                     global_qk_param=case.get("param", "linear_proj"), gate_thres_init=case["gate_thres"],
                     sparse_full_attn_backend=case["backend"], num_hidden_layers=1, rms_norm_eps=1e-5)
    layer = LoGoAttention(cfg, layer_idx=0)
    w = layer_weights(case)
    with torch.no_grad():
        for name, arr in w.items():
            dict(layer.named_parameters())[name].copy_(torch.from_numpy(arr))
    return layer.eval()


def gen_layer():
    out = {}
    for name, case in LAYER_CASES.items():
        layer = build_ref_layer(case)
        hidden, cu, pos = layer_case_inputs(case)
        h = torch.from_numpy(hidden)
        kwargs = dict(position_ids=torch.from_numpy(pos))
        if cu is not None:
            kwargs["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32)
        with torch.no_grad():
            y, _, _ = layer(h, **kwargs)
            gate = torch.sigmoid(layer.gate_proj(h))
        sel = (gate.squeeze(-1) >= layer.gate_thres).reshape(-1)
        out[f"{name}/q_idx"] = sel.nonzero().squeeze(-1).numpy()
        y = y.numpy()
        if case.get("subsample"):
            out[f"{name}/out_sub"] = y.reshape(-1)[:: case["subsample"]].copy()
            out[f"{name}/out_sum"] = np.array([y.astype(np.float64).sum(), np.abs(y.astype(np.float64)).sum()])
        else:
            out[f"{name}/out"] = y
        out[f"{name}/gate"] = gate.numpy().reshape(-1)
        print(name, "selected", int(sel.sum()), "of", sel.numel())

    # the dense causal layer (logo/layers/attn.py), with the same stand-in for the flash-attn wheel
    from logo.configuration_logo import LoGoConfig
    from logo.layers.attn import Attention
    case = DENSE_ATTN_CASE
    cfg = LoGoConfig(hidden_size=case["hidden"], num_attention_heads=case["heads"],
                     num_key_value_heads=case["kv_heads"], num_hidden_layers=1)
    layer = Attention(cfg, layer_idx=0).eval()
    with torch.no_grad():
        for name, arr in dense_attn_weights(case).items():
            dict(layer.named_parameters())[name].copy_(torch.from_numpy(arr))
        hidden, pos = dense_attn_inputs(case)
        y, _, _ = layer(torch.from_numpy(hidden), position_ids=torch.from_numpy(pos))
    out["dense_attn/out"] = y.numpy()
    print("dense_attn out std", float(y.std()))
    np.savez_compressed(OUT / "layer.npz", **out)


def gen_decode():
    """Prefill + single-token steps through the reference layer and its Cache."""
    from logo.cache import Cache
    out = {}
    case = dict(LAYER_CASES["small_batch"])
    layer = build_ref_layer(case)
    B, T0, steps = 2, 150, 6
    rs = np.random.RandomState(4242)
    hidden = rs.standard_normal((B, T0 + steps, case["hidden"])).astype(np.float32)
    h = torch.from_numpy(hidden)
    cache = Cache()
    outs = []
    with torch.no_grad():
        pos = torch.arange(T0)[None].expand(B, -1)
        y, _, _ = layer(h[:, :T0], position_ids=pos, past_key_value=cache, use_cache=True)
        outs.append(y.numpy())
        for s in range(steps):
            pos = torch.full((B, 1), T0 + s)
            y, _, _ = layer(h[:, T0 + s: T0 + s + 1], position_ids=pos, past_key_value=cache, use_cache=True)
            outs.append(y.numpy())
        gate = torch.sigmoid(layer.gate_proj(h)).numpy()
        full, _, _ = layer(h, position_ids=torch.arange(T0 + steps)[None].expand(B, -1))
    out["decode/prefill_out"] = outs[0]
    out["decode/step_out"] = np.concatenate(outs[1:], axis=1)
    out["decode/gate"] = gate
    out["decode/full_out"] = full.numpy()
    st = cache.states[0]
    out["decode/local_k_shape"] = np.array(st["attn_state"][0].shape)
    out["decode/full_k_shape"] = np.array(st["attn_state_full"][0].shape)
    out["decode/seen"] = np.array([cache.get_seq_length(0)])
    print("decode: local", tuple(st["attn_state"][0].shape), "full", tuple(st["attn_state_full"][0].shape),
          "max |cached - full|", float(np.abs(out["decode/step_out"] - out["decode/full_out"][:, T0:]).max()))

    # several tokens on top of a non-empty cache (logo/cache.py:95-118): prefill 100, a chunk of 50
    # (the local branch then sees 100 cached + 50 new keys and uses its window), one more token
    cache2 = Cache()
    with torch.no_grad():
        T1, chunk = 100, 50
        layer(h[:, :T1], position_ids=torch.arange(T1)[None].expand(B, -1), past_key_value=cache2, use_cache=True)
        y_chunk, _, _ = layer(h[:, T1:T1 + chunk], position_ids=torch.arange(T1, T1 + chunk)[None].expand(B, -1),
                              past_key_value=cache2, use_cache=True)
        y_last, _, _ = layer(h[:, T1 + chunk:T1 + chunk + 1], position_ids=torch.full((B, 1), T1 + chunk),
                             past_key_value=cache2, use_cache=True)
    out["decode/chunk_out"] = y_chunk.numpy()
    out["decode/after_chunk_out"] = y_last.numpy()
    print("chunk: max |chunked - full|", float(np.abs(out["decode/chunk_out"] - out["decode/full_out"][:, T1:T1 + chunk]).max()),
          "then one token", float(np.abs(out["decode/after_chunk_out"] - out["decode/full_out"][:, T1 + chunk:T1 + chunk + 1]).max()))
    np.savez_compressed(OUT / "decode.npz", **out)


def gen_misc():
    """bf16 RMSNorm + blend through the reference modules, and the budget controller."""
    from logo.modules.layernorm import RMSNorm
    from logo.update import update_gate_thres
    out = {}
    rs = np.random.RandomState(77)
    n, h, d = 64, 2, 128
    local = torch.from_numpy(rs.standard_normal((n, h, d)).astype(np.float32)).to(torch.bfloat16)
    glob = torch.from_numpy(rs.standard_normal((n, h, d)).astype(np.float32)).to(torch.bfloat16)
    gate = torch.from_numpy(rs.uniform(0, 1, (n, 1)).astype(np.float32)).to(torch.bfloat16)
    wl = torch.from_numpy((1 + 0.1 * rs.standard_normal(d)).astype(np.float32)).to(torch.bfloat16)
    wg = torch.from_numpy((1 + 0.1 * rs.standard_normal(d)).astype(np.float32)).to(torch.bfloat16)
    thres = torch.full((1,), 0.5)
    nl, ng = RMSNorm(d, eps=1e-5).to(torch.bfloat16), RMSNorm(d, eps=1e-5).to(torch.bfloat16)
    with torch.no_grad():
        nl.weight.copy_(wl)
        ng.weight.copy_(wg)
        sel = gate.squeeze(-1) >= thres
        glob = glob * sel[:, None, None]           # unselected rows are exactly 0 (selected_full_attn.py:469)
        a = nl(local).reshape(n, -1)
        b = ng(glob).reshape(n, -1)
        g = gate.masked_fill(gate < thres, 0.0)
        fused = (1 - g) * a + g * b                 # logo/layers/logo.py:256-258 in bf16
    out["fuse/out_bf16"] = fused.float().numpy()
    out["fuse/norm_local_bf16"] = a.float().numpy()

    class Fake(torch.nn.Module):
        def __init__(self, thres, g, t):
            super().__init__()
            self.register_buffer("gate_thres", torch.tensor([thres]))
            self.register_buffer("gate_avg", torch.tensor([3.0]))
            self.register_buffer("global_token_count", torch.tensor([g]))
            self.register_buffer("total_token_count", torch.tensor([t]))

    model = torch.nn.ModuleList([Fake(0.5, 30.0, 100.0), Fake(0.4, 70.0, 100.0), Fake(0.3, 0.0, 0.0),
                                 Fake(0.2, 50.0, 100.0)])
    ratio = update_gate_thres(model, target_global_ratio=0.5, update_rate=0.01)
    out["update/ratio"] = ratio.numpy()
    out["update/thres"] = np.array([m.gate_thres.item() for m in model], dtype=np.float32)
    out["update/counters"] = np.array([[m.gate_avg.item(), m.global_token_count.item(), m.total_token_count.item()]
                                       for m in model], dtype=np.float32)
    np.savez_compressed(OUT / "misc.npz", **out)
    print("misc.npz")


def gen_rope():
    """The reference's rotary embedding on bf16 tensors (its eager rounding sequence) and the gradient
    autograd gives for it; tables from the reference's RotaryEmbedding."""
    from logo.modules.rotary import apply_rotary_pos_emb
    from golden_inputs import rope_case
    x, g, pos = rope_case()
    n, h, d = x.shape
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
    fr = torch.from_numpy(pos).float()[:, None] * inv[None, :]
    emb = torch.cat([fr, fr], dim=-1)
    cos, sin = emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)       # [N, D]
    # reference layout: q [B, heads, T, D] with cos [B, T, D] broadcast over heads (unsqueeze_dim=1)
    q = torch.from_numpy(x).to(torch.bfloat16).permute(1, 0, 2)[None].contiguous().requires_grad_(True)
    k = q.detach().clone()
    q_out, _ = apply_rotary_pos_emb(q, k, cos[None], sin[None])
    q_out.backward(torch.from_numpy(g).to(torch.bfloat16).permute(1, 0, 2)[None].contiguous())
    out = {"cos": cos.float().numpy(), "sin": sin.float().numpy(),
           "out": q_out.detach()[0].permute(1, 0, 2).float().numpy(),
           "grad": q.grad[0].permute(1, 0, 2).float().numpy()}
    np.savez_compressed(OUT / "rope.npz", **out)
    print("rope.npz")


def gen_model():
    """A tiny LoGoForCausalLM (one LoGo layer + one dense layer) through the reference's own model code:
    logits of a packed varlen batch, and of a prefill followed by four single-token steps through its Cache."""
    from logo.cache import Cache
    from logo.configuration_logo import LoGoConfig
    from logo.modeling_logo import LoGoForCausalLM
    cfg = LoGoConfig(**{k: v for k, v in MODEL_CASE.items() if k != "seed"})
    model = LoGoForCausalLM(cfg).eval()
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    model.load_state_dict({k: torch.from_numpy(v) for k, v in model_weights(shapes).items()})
    packed, cu, batch = model_inputs()
    out = {}
    with torch.no_grad():
        y = model(input_ids=torch.from_numpy(packed), cu_seqlens=torch.tensor(cu, dtype=torch.int32), use_cache=False)
        out["model/packed_logits"] = y.logits[0].numpy()
        # the reference's loss (shifted labels, packed boundaries masked, logo/modeling_logo.py:380-407)
        y = model(input_ids=torch.from_numpy(packed), labels=torch.from_numpy(packed),
                  cu_seqlens=torch.tensor(cu, dtype=torch.int32), use_cache=False)
        out["model/packed_loss"] = np.array([float(y.loss)])
        y = model(input_ids=torch.from_numpy(batch), labels=torch.from_numpy(batch), use_cache=False)
        out["model/batch_loss"] = np.array([float(y.loss)])
        out["model/batch_logits"] = y.logits.numpy()
        B, T0, steps = batch.shape[0], 150, 4
        ids = torch.from_numpy(batch)
        cache = Cache()
        y = model(input_ids=ids[:, :T0], past_key_values=cache, use_cache=True)
        logits = [y.logits]
        for s in range(steps):
            y = model(input_ids=ids[:, T0 + s: T0 + s + 1], past_key_values=cache, use_cache=True)
            logits.append(y.logits)
        out["model/cached_logits"] = torch.cat(logits, dim=1).numpy()
        full = model(input_ids=ids, use_cache=False).logits.numpy()
    out["model/param_names"] = np.array(sorted(shapes))
    print("model: logits std", float(out["model/packed_logits"].std()), "max |cached - full|",
          float(np.abs(out["model/cached_logits"] - full).max()))
    np.savez_compressed(OUT / "model.npz", **out)


if __name__ == "__main__":
    import sys
    torch.set_num_threads(8)
    install_shims()
    gens = {"selection": gen_selection, "attention": gen_attention, "layer": gen_layer, "decode": gen_decode,
            "misc": gen_misc, "rope": gen_rope, "model": gen_model}
    for name in (sys.argv[1:] or list(gens)):       # `make_golden.py rope` regenerates one fixture only
        gens[name]()
