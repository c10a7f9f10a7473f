"""The CPU oracle against outputs of the reference's own code (tests/golden/*.npz)."""
import numpy as np
import pytest
import torch

from golden_inputs import (ATTN_CASES, DENSE_ATTN_CASE, LAYER_CASES, attn_case_inputs, dense_attn_inputs,
                           dense_attn_weights, layer_case_inputs, layer_weights, selection_cases)
from oracle import logo_oracle as orc


@pytest.mark.parametrize("name", sorted(selection_cases()))
def test_selection_bit_exact(golden, name):
    mask, cu = selection_cases()[name]
    g = golden["selection"]
    sel = orc.build_selection_ref(mask, cu)
    assert sel.q_idx.dtype == np.int64 and sel.pos_ids.dtype == np.int32
    np.testing.assert_array_equal(sel.q_idx, g[f"{name}/q_idx"])
    np.testing.assert_array_equal(sel.pos_ids, g[f"{name}/pos_ids"])
    np.testing.assert_array_equal(sel.cu_seqlens_q, g[f"{name}/cu_seqlens_q"])
    np.testing.assert_array_equal(orc.prepare_chunk_indices_ref(sel.cu_seqlens_q, 128), g[f"{name}/chunks_q128"])
    np.testing.assert_array_equal(orc.prepare_chunk_indices_ref(cu, 128), g[f"{name}/chunks_k128"])
    np.testing.assert_array_equal(orc.q_start_blk_ref(sel.pos_ids, sel.cu_seqlens_q, sel.cu_seqlens_k, 128),
                                  g[f"{name}/q_start_blk"])
    # the device-side tile list is the prefix-sum form of prepare_chunk_indices
    off = orc.tile_offsets_ref(sel.cu_seqlens_q, 128)
    assert off[-1] == g[f"{name}/chunks_q128"].shape[0]


@pytest.mark.parametrize("name", sorted(ATTN_CASES))
def test_attention_matches_reference_kernels(golden, name):
    q, k, v, do, sel, cu = attn_case_inputs(name)
    g = golden["attention"]
    qt, kt, vt = (torch.from_numpy(x).requires_grad_(True) for x in (q, k, v))
    o, _ = orc.attention_dense_ref(qt, kt, vt, cu, None, None, torch.from_numpy(sel))
    o.backward(torch.from_numpy(do))
    # fp32 against the reference's Triton kernels (interpreted): rounding-level agreement
    for key, val in (("o", o.detach()), ("dq", qt.grad), ("dk", kt.grad), ("dv", vt.grad)):
        ref = torch.from_numpy(g[f"{name}/{key}"])
        assert orc.abs_err(ref, val) < 2e-5, (name, key, orc.abs_err(ref, val))
    assert np.all(g[f"{name}/o"][~sel] == 0) and torch.all(o.detach()[~torch.from_numpy(sel)] == 0)


@pytest.mark.parametrize("name", sorted(LAYER_CASES))
def test_layer_matches_reference_layer(golden, name):
    case = LAYER_CASES[name]
    g = golden["layer"]
    hidden, cu, pos = layer_case_inputs(case)
    w = {k: torch.from_numpy(v) for k, v in layer_weights(case).items()}
    b, t, hid = hidden.shape
    cu_full = cu if cu is not None else list(range(0, (b + 1) * t, t))
    out, parts = orc.logo_layer_ref(torch.from_numpy(hidden).reshape(b * t, hid), w, cu_full, case["heads"],
                                    case["kv_heads"], case["window"], case["gate_thres"], 1e-5, return_parts=True)
    np.testing.assert_allclose(parts["gate"].reshape(-1).numpy(), g[f"{name}/gate"], atol=1e-6)
    np.testing.assert_array_equal(parts["selection"].nonzero().squeeze(-1).numpy(), g[f"{name}/q_idx"])
    out = out.reshape(b, t, hid).numpy()
    if case.get("subsample"):
        np.testing.assert_allclose(out.reshape(-1)[:: case["subsample"]], g[f"{name}/out_sub"], atol=2e-5)
        assert abs(out.astype(np.float64).sum() - g[f"{name}/out_sum"][0]) < 1e-2
    else:
        np.testing.assert_allclose(out, g[f"{name}/out"], atol=2e-5)


def test_dense_attention_layer_matches_reference_layer(golden):
    """The oracle's restatement of the dense causal layer against the reference's Attention module."""
    case = DENSE_ATTN_CASE
    hidden, _ = dense_attn_inputs(case)
    w = {k: torch.from_numpy(v) for k, v in dense_attn_weights(case).items()}
    b, t, hid = hidden.shape
    out = orc.dense_attention_layer_ref(torch.from_numpy(hidden).reshape(b * t, hid), w, list(range(0, (b + 1) * t, t)),
                                        case["heads"], case["kv_heads"])
    np.testing.assert_allclose(out.reshape(b, t, hid).numpy(), golden["layer"]["dense_attn/out"], atol=2e-5)


def test_chunk_on_a_filled_cache_equals_the_rows_of_the_full_forward(golden):
    """The reference layer fed 50 new tokens on top of 100 cached ones returns the rows 100..149 of its
    own uncached forward (and the following single token row 150): what a continuation has to
    reproduce is therefore the oracle layer on the whole sequence, restricted to the new rows."""
    g = golden["decode"]
    case = LAYER_CASES["small_batch"]
    w = {k: torch.from_numpy(v) for k, v in layer_weights(case).items()}
    B, T = 2, 156
    hidden = torch.from_numpy(np.random.RandomState(4242).standard_normal((B, T, case["hidden"])).astype(np.float32))
    np.testing.assert_allclose(g["decode/chunk_out"], g["decode/full_out"][:, 100:150], atol=2e-6)
    np.testing.assert_allclose(g["decode/after_chunk_out"], g["decode/full_out"][:, 150:151], atol=2e-6)
    for b in range(B):
        out = orc.logo_layer_ref(hidden[b, :151], w, [0, 151], case["heads"], case["kv_heads"], case["window"],
                                 case["gate_thres"], 1e-5)
        np.testing.assert_allclose(out[100:150].numpy(), g["decode/chunk_out"][b], atol=2e-5)
        np.testing.assert_allclose(out[150:151].numpy(), g["decode/after_chunk_out"][b], atol=2e-5)


def test_decode_and_cache_match_reference(golden):
    """Prefill + 6 single-token steps through the oracle's cache restatement and decode attention."""
    g = golden["decode"]
    case = LAYER_CASES["small_batch"]
    w = {k: torch.from_numpy(v) for k, v in layer_weights(case).items()}
    B, T0, steps = 2, 150, 6
    hidden = torch.from_numpy(np.random.RandomState(4242).standard_normal((B, T0 + steps, case["hidden"]))
                              .astype(np.float32))
    H, HKV, W = case["heads"], case["kv_heads"], case["window"]
    D = case["hidden"] // H
    thres = case["gate_thres"]
    np.testing.assert_array_equal(g["decode/local_k_shape"], [B, HKV, W, D])
    np.testing.assert_array_equal(g["decode/full_k_shape"], [B, HKV, T0 + steps, D])
    assert int(g["decode/seen"][0]) == T0 + steps

    def project(h, pos):
        n = h.shape[0]
        q = (h @ w["q_proj.weight"].T).view(n, H, D)
        k = (h @ w["k_proj.weight"].T).view(n, HKV, D)
        v = (h @ w["v_proj.weight"].T).view(n, HKV, D)
        gq = torch.einsum("lhd,hde->lhe", q, w["q_global_proj"])
        gk = torch.einsum("lhd,hde->lhe", k, w["k_global_proj"])
        gv = torch.einsum("lhd,hde->lhe", v, w["v_global_proj"])
        cos, sin = orc.rope_cos_sin(pos, D)
        return (orc.apply_rope(q, cos, sin), orc.apply_rope(k, cos, sin), v, orc.apply_rope(gq, cos, sin),
                orc.apply_rope(gk, cos, sin), gv)

    cache = orc.CacheRef()
    # prefill: the oracle layer on each sequence, then store states [B,H,T,D]
    pre = []
    states = [project(hidden[b, :T0], torch.arange(T0)) for b in range(B)]
    for b in range(B):
        pre.append(orc.logo_layer_ref(hidden[b, :T0], w, [0, T0], H, HKV, W, thres, 1e-5))
    np.testing.assert_allclose(torch.stack(pre).numpy(), g["decode/prefill_out"], atol=2e-5)
    to_bhtd = lambda xs: torch.stack(xs).transpose(1, 2)
    cache.update((to_bhtd([s[1] for s in states]), to_bhtd([s[2] for s in states])),
                 (to_bhtd([s[4] for s in states]), to_bhtd([s[5] for s in states])), 0, T0, W)
    outs = []
    for s in range(steps):
        h = hidden[:, T0 + s]
        ql, kl, v, gq, gk, gv = project(h, torch.full((B,), T0 + s))
        st = cache.update((kl[:, :, None], v[:, :, None]), (gk[:, :, None], gv[:, :, None]), 0, 1, W)
        gate = torch.sigmoid(h @ w["gate_proj.weight"].T)
        active = gate[:, 0] >= thres
        n_loc = st["attn_state"][0].shape[-2]
        assert n_loc == min(T0 + s, W) + 1
        local = orc.decode_attn_ref(ql, st["attn_state"][0], st["attn_state"][1], [n_loc] * B)
        full_k, full_v = st["attn_state_full"]
        glob = orc.decode_attn_ref(gq, full_k, full_v, [T0 + s + 1] * B, active=active)
        fused = orc.fuse_ref(local, glob, gate, torch.tensor(thres), w["context_norm_local.weight"],
                             w["context_norm_global.weight"], 1e-5)
        outs.append(fused @ w["o_proj.weight"].T)
    np.testing.assert_allclose(torch.stack(outs, dim=1).numpy(), g["decode/step_out"], atol=2e-5)
    assert cache.seen == T0 + steps
    assert cache.states[0]["attn_state"][0].shape[-2] == W


def test_fuse_bf16_rounding_matches_reference_modules(golden):
    g = golden["misc"]
    rs = np.random.RandomState(77)
    n, h, d = 64, 2, 128
    bf = lambda a: torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    local, glob = bf(rs.standard_normal((n, h, d))), bf(rs.standard_normal((n, h, d)))
    gate = bf(rs.uniform(0, 1, (n, 1)))
    wl, wg = bf(1 + 0.1 * rs.standard_normal(d)), bf(1 + 0.1 * rs.standard_normal(d))
    thres = torch.full((1,), 0.5)
    glob = glob * (gate.squeeze(-1) >= thres)[:, None, None]
    out = orc.fuse_ref(local, glob, gate, thres, wl, wg, 1e-5)
    assert out.dtype == torch.bfloat16
    np.testing.assert_array_equal(out.float().numpy(), g["fuse/out_bf16"])
    np.testing.assert_array_equal(orc.rmsnorm_ref(local, wl, 1e-5).reshape(n, -1).float().numpy(),
                                  g["fuse/norm_local_bf16"])


def test_update_gate_thres_matches_reference(golden):
    g = golden["misc"]
    thres, ratio = orc.update_gate_thres_ref([0.5, 0.4, 0.3, 0.2], [30, 70, 0, 50], [100, 100, 0, 100], 0.5, 0.01)
    np.testing.assert_allclose(thres, g["update/thres"], atol=1e-7)
    np.testing.assert_allclose(ratio, g["update/ratio"].reshape(-1), atol=1e-7)
    assert np.all(g["update/counters"] == 0)


def test_rope_bf16_graph_bit_exact(golden):
    """The oracle's rotary embedding on bf16 tensors reproduces the reference's eager bf16 graph and
    the gradient autograd gives for it."""
    from golden_inputs import rope_case

    g = golden["rope"]
    x, grad_out, _ = rope_case()
    cos, sin = torch.from_numpy(g["cos"]).to(torch.bfloat16), torch.from_numpy(g["sin"]).to(torch.bfloat16)
    xt = torch.from_numpy(x).to(torch.bfloat16).requires_grad_(True)
    out = orc.apply_rope(xt, cos, sin)
    out.backward(torch.from_numpy(grad_out).to(torch.bfloat16))
    np.testing.assert_array_equal(out.detach().float().numpy(), g["out"])
    np.testing.assert_array_equal(xt.grad.float().numpy(), g["grad"])


def test_lm_loss_matches_reference_model_loss(golden):
    """The oracle's restatement of the loss (label shift, packed-boundary masking, mean cross-entropy) on
    the reference model's own logits reproduces the loss the reference model returned."""
    from golden_inputs import model_inputs

    g = golden["model"]
    packed, cu, batch = model_inputs()
    loss = orc.lm_loss_ref(torch.from_numpy(g["model/packed_logits"])[None], torch.from_numpy(packed), cu)
    assert abs(float(loss) - float(g["model/packed_loss"][0])) < 1e-5
    loss = orc.lm_loss_ref(torch.from_numpy(g["model/batch_logits"]), torch.from_numpy(batch), None)
    assert abs(float(loss) - float(g["model/batch_loss"][0])) < 1e-5
