"""The benchmark configurations at their real sizes against the CPU oracle on a subsample.

The oracle is dense-masked fp32 and cannot run a 32768-token x 16-head problem in test time, but
sequences and heads are independent (attention never crosses a packed-sequence boundary,
logo/ops/selected_full_attn.py:62-67, and every head is its own softmax), so the full-size CUDA
launch is compared with the oracle run on a few (sequence, head) slices of the same tensors.
Tolerances are the contract's: outputs 1e-2 max-abs, gradients 2e-2 RMS-relative."""
import numpy as np
import pytest
import torch

from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu

OUT_ATOL = 1e-2
GRAD_RATIO = 2e-2


@pytest.mark.parametrize("ratio", [0.125, 0.5, 1.0])
def test_config2_full_size_subsample_vs_oracle(cuda_device, ratio):
    """sq_full_attn forward + backward on 4 x 8192 tokens packed [1, 32768, 16, 128]; heads {0, 15}
    of sequences {0, 3} are checked against the oracle."""
    from logo_b200 import ops

    t, nseq, hq, d = 8192, 4, 16, 128
    n = t * nseq
    g = torch.Generator(device="cuda").manual_seed(1234)
    mk = lambda s: (torch.randn(n, hq, d, device=cuda_device, generator=g) * s).to(torch.bfloat16)
    q, k, v, do = mk(d ** -0.25), mk(d ** -0.25), mk(1.0), mk(1.0)
    sel = (torch.rand(n, device=cuda_device, generator=g) < ratio) if ratio < 1 else \
        torch.ones(n, dtype=torch.bool, device=cuda_device)
    cu = torch.arange(0, n + 1, t, dtype=torch.int32)
    qd, kd, vd = (x[None].clone().requires_grad_(True) for x in (q, k, v))
    o = ops.sq_full_attn(qd, kd, vd, sel[None], cu_seqlens=cu)
    o.backward(do[None])
    torch.cuda.synchronize()
    assert torch.all(o[0][~sel] == 0) and torch.all(qd.grad[0][~sel] == 0)
    for seq, head in ((0, 0), (3, 15)):
        rows = slice(seq * t, (seq + 1) * t)
        cut = lambda x: x[rows, head:head + 1].float().cpu()
        qr, kr, vr = (cut(x).requires_grad_(True) for x in (q, k, v))
        sel_s = sel[rows].cpu()
        o_ref, _ = orc.attention_dense_ref(qr, kr, vr, [0, t], None, None, sel_s)
        o_ref.backward(cut(do))
        err_o = orc.abs_err(o_ref.detach(), cut(o[0]))
        ratios = {nm: orc.err_ratio(ref, cut(got.grad[0]))
                  for nm, ref, got in (("dq", qr.grad, qd), ("dk", kr.grad, kd), ("dv", vr.grad, vd))}
        print(f"config 2, ratio {ratio}, sequence {seq}, head {head}: o max-abs {err_o:.2e}, "
              + ", ".join(f"{nm} {r:.2e}" for nm, r in ratios.items()))
        assert err_o <= OUT_ATOL
        for nm, r in ratios.items():
            assert r < GRAD_RATIO, (nm, r)


def test_config3_layer_train_step_two_sequences_vs_oracle(cuda_device):
    """The layer training step of the benchmark (8 packed sequences, 32768 tokens, hidden 2048,
    16 x 128, window 128, 25 % of the tokens global): output rows and input gradients of the two
    shortest sequences against fp32 autograd through the oracle on those sequences alone."""
    import bench
    from logo_b200 import LoGoAttention
    from logo_b200.config import LoGoConfig

    lens = sorted(bench._varlen_lengths(bench.N_TOK, 8, 512, 8192, 5), reverse=True)
    cfg = LoGoConfig(hidden_size=2048, num_attention_heads=16, num_key_value_heads=16, window_size=128,
                     global_qk_param="linear_proj", num_hidden_layers=1, rms_norm_eps=1e-5,
                     max_position_embeddings=8192)
    torch.manual_seed(0)
    layer = LoGoAttention(cfg, 0)
    with torch.no_grad():   # linear weights N(0, 0.02), per-head projections identity + N(0, 0.02), norm weights near 1
        for name, p in layer.named_parameters():
            if name.endswith("_global_proj"):
                p.add_(0.02 * torch.randn_like(p))
            elif "context_norm" in name:
                p.add_(0.1 * torch.randn_like(p))
            else:
                p.normal_(0, 0.02)
    layer = layer.to(cuda_device, torch.bfloat16).train()
    n = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(1)
    hidden = torch.randn(1, n, 2048, device=cuda_device, generator=g).to(torch.bfloat16).requires_grad_(True)
    d_out = torch.randn(1, n, 2048, device=cuda_device, generator=g).to(torch.bfloat16)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    pos = torch.cat([torch.arange(l, device=cuda_device) for l in lens])[None]
    with torch.no_grad():   # threshold at the 75th percentile of the gates, a bf16-representable value
        gate = torch.sigmoid(layer.gate_proj(hidden)).float().flatten()
        thres = float(torch.quantile(gate, 0.75).to(torch.bfloat16).item())
        layer.gate_thres.fill_(thres)
    out, _, _ = layer(hidden, position_ids=pos, cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=cuda_device))
    out.backward(d_out)
    torch.cuda.synchronize()
    sel = (gate >= thres).cpu()
    assert 0.2 < sel.float().mean().item() < 0.3
    # the counters are bf16 buffers after the cast of the module (logo/layers/logo.py:73-76 registers them as
    # plain float buffers): the count is rounded like any other bf16 value
    assert layer.global_token_count.item() == torch.tensor(float(sel.sum())).to(torch.bfloat16).item()

    w = {k: v.detach().float().cpu() for k, v in layer.named_parameters()}
    for s in (len(lens) - 1, len(lens) - 2):           # the two shortest sequences
        a, b = int(cu[s]), int(cu[s + 1])
        hr = hidden.detach()[0, a:b].float().cpu().requires_grad_(True)
        ref = orc.logo_layer_ref(hr, w, [0, b - a], 16, 16, 128, thres, 1e-5, selection_override=sel[a:b])
        ref.backward(d_out[0, a:b].float().cpu())
        r_out = orc.err_ratio(ref.detach(), out[0, a:b].float().cpu())
        r_dh = orc.err_ratio(hr.grad, hidden.grad[0, a:b].float().cpu())
        print(f"config 3, sequence of {b - a} tokens ({int(sel[a:b].sum())} global): output {r_out:.2e}, d hidden {r_dh:.2e}")
        assert r_out < 2e-2 and r_dh < 3e-2


def test_config5_decode_at_32768_cached_tokens_vs_oracle(cuda_device):
    """One decode step over a 32768-token cache: two sequences (one active, one below the threshold),
    2 KV heads with a group of 2 query heads each, against the oracle."""
    from logo_b200 import Cache
    from logo_b200.layers import decode_attention

    g = torch.Generator(device="cuda").manual_seed(5)
    B, HQ, H, D, T, W = 2, 4, 2, 128, 32768, 128
    mk = lambda *s: torch.randn(*s, device=cuda_device, generator=g).to(torch.bfloat16)
    cache = Cache(max_length=T + 8)
    kl, vl, kg, vg = mk(B, T, H, D), mk(B, T, H, D), mk(B, T, H, D), mk(B, T, H, D)
    st = cache.append(0, kl, vl, kg, vg, W)
    ql, qg = mk(B, HQ, D), mk(B, HQ, D)
    gate = torch.tensor([0.75, 0.25], device=cuda_device).to(torch.bfloat16)
    thres = torch.tensor([0.5], device=cuda_device)
    o_l, o_g = decode_attention(ql, qg, st, gate, thres, D ** -0.5)
    torch.cuda.synchronize()
    assert int(st.status.item()) == 0
    bh = lambda x: x.transpose(1, 2).float().cpu()
    ref_g = orc.decode_attn_ref(qg.float().cpu(), bh(kg), bh(vg), [T] * B, active=torch.tensor([True, False]))
    ref_l = orc.decode_attn_ref(ql.float().cpu(), bh(kl), bh(vl), [T] * B, window=W)
    err_g, err_l = orc.abs_err(ref_g, o_g.float().cpu()), orc.abs_err(ref_l, o_l.float().cpu())
    print(f"config 5, context {T}: global max-abs {err_g:.2e}, local max-abs {err_l:.2e}")
    assert err_g <= OUT_ATOL and err_l <= OUT_ATOL
    assert torch.all(o_g[1] == 0)
