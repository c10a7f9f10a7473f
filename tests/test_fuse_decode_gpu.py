"""Fused RMSNorm + gate blend (forward / backward), cache append and decode attention through the
C ABI, against the oracle and the reference-module fixtures."""
import numpy as np
import pytest
import torch

from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu


def _bf(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def test_fuse_forward_reproduces_reference_bf16_graph(cuda_device, golden):
    from logo_b200 import ops

    g = golden["misc"]
    rs = np.random.RandomState(77)
    n, h, d = 64, 2, 128
    local, glob = _bf(rs.standard_normal((n, h, d))), _bf(rs.standard_normal((n, h, d)))
    gate = _bf(rs.uniform(0, 1, (n, 1)))
    wl, wg = _bf(1 + 0.1 * rs.standard_normal(d)), _bf(1 + 0.1 * rs.standard_normal(d))
    thres = torch.full((1,), 0.5)
    # rows of the global branch below the threshold are never read: poison them
    glob_poison = glob.clone()
    glob_poison[(gate.squeeze(-1) < thres)] = float("nan")
    out = ops.fuse_norm_blend(local.to(cuda_device), glob_poison.to(cuda_device), gate.to(cuda_device),
                              thres.to(cuda_device), wl.to(cuda_device), wg.to(cuda_device), 1e-5, True)
    got = out.float().cpu().numpy()
    ref = g["fuse/out_bf16"]
    assert not np.isnan(got).any()
    # identical rounding sequence; rsqrt may differ in its last bit between CPU and GPU, which can
    # flip a bf16 rounding: allow one bf16 ulp on a handful of elements, nothing more
    ulp = np.maximum(np.abs(ref), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - ref) <= ulp)
    assert np.mean(got != ref) < 0.01


@pytest.mark.parametrize("h,use_norm,w_dtype", [(2, True, torch.bfloat16), (3, True, torch.float32),
                                                (16, True, torch.bfloat16), (4, False, torch.bfloat16)])
def test_fuse_forward_backward_vs_oracle(cuda_device, h, use_norm, w_dtype):
    from logo_b200 import ops

    rs = np.random.RandomState(h)
    n, d = 777, 128
    local, glob = _bf(rs.standard_normal((n, h, d))), _bf(rs.standard_normal((n, h, d)))
    gate = _bf(rs.uniform(0, 1, (n, 1)))
    thres = torch.tensor([0.4])
    sel = gate.squeeze(-1).float() >= 0.4
    glob = glob * sel[:, None, None]
    wl = torch.from_numpy((1 + 0.1 * rs.standard_normal(d)).astype(np.float32)).to(w_dtype)
    wg = torch.from_numpy((1 + 0.1 * rs.standard_normal(d)).astype(np.float32)).to(w_dtype)
    d_out = _bf(rs.standard_normal((n, h * d)))

    ref_in = [x.detach().float().clone().requires_grad_(True) for x in (local, glob, gate, wl, wg)]
    ref = orc.fuse_ref(ref_in[0], ref_in[1], ref_in[2], thres, ref_in[3], ref_in[4], 1e-5, use_norm)
    ref.backward(d_out.float())

    dev_in = [x.detach().clone().to(cuda_device).requires_grad_(True) for x in (local, glob, gate, wl, wg)]
    out = ops.fuse_norm_blend(dev_in[0], dev_in[1], dev_in[2], thres.to(cuda_device),
                              dev_in[3] if use_norm else None, dev_in[4] if use_norm else None, 1e-5, use_norm)
    out.backward(d_out.to(cuda_device))
    assert orc.err_ratio(ref.detach(), out.float().cpu()) < 6e-3          # bf16 rounding of the result
    names = ["d_local", "d_glob", "d_gate"] + (["d_w_local", "d_w_global"] if use_norm else [])
    for nm, r, t in zip(names, ref_in, dev_in):
        assert orc.err_ratio(r.grad, t.grad.float().cpu()) < 2e-2, (nm, orc.err_ratio(r.grad, t.grad.float().cpu()))
    assert torch.all(dev_in[1].grad[~sel.to(cuda_device)] == 0)
    assert torch.all(dev_in[2].grad[~sel.to(cuda_device)] == 0)
    # weight gradients are reduced in a fixed order: two runs agree bit for bit
    if use_norm:
        dev2 = [x.detach().clone().requires_grad_(True) for x in dev_in]
        ops.fuse_norm_blend(dev2[0], dev2[1], dev2[2], thres.to(cuda_device), dev2[3], dev2[4], 1e-5,
                            True).backward(d_out.to(cuda_device))
        assert torch.equal(dev2[3].grad, dev_in[3].grad) and torch.equal(dev2[4].grad, dev_in[4].grad)


@pytest.mark.parametrize("hq,h", [(2, 2), (4, 2), (4, 1)])
def test_cache_append_and_decode_vs_oracle(cuda_device, hq, h):
    """Prefill of 300 tokens then 5 single-token steps; per-sequence skipping of the global branch."""
    from logo_b200 import Cache
    from logo_b200.layers import decode_attention

    rs = np.random.RandomState(hq * 10 + h)
    B, D, W, T0, steps = 3, 128, 128, 300, 5
    ref = orc.CacheRef()
    cache = Cache(max_length=0, growth=2)       # tiny growth: the reallocation path is exercised
    mk = lambda *s: _bf(rs.standard_normal(s))
    kl, vl, kg, vg = (mk(B, T0, h, D) for _ in range(4))
    bh = lambda x: x.transpose(1, 2)
    ref.update((bh(kl), bh(vl)), (bh(kg), bh(vg)), 0, T0, W)
    cache.append(0, kl.to(cuda_device), vl.to(cuda_device), kg.to(cuda_device), vg.to(cuda_device), W, layout="bthd")
    for s in range(steps):
        kl, vl, kg, vg = (mk(B, 1, h, D) for _ in range(4))
        ql, qg = mk(B, hq, D), mk(B, hq, D)
        gate = _bf(rs.uniform(0, 1, B))
        gate[0] = 0.9
        gate[1] = 0.1
        thres = torch.tensor([0.5])
        st_ref = ref.update((bh(kl), bh(vl)), (bh(kg), bh(vg)), 0, 1, W)
        st = cache.append(0, kl.to(cuda_device), vl.to(cuda_device), kg.to(cuda_device), vg.to(cuda_device), W)
        n = T0 + s + 1
        assert st.length == n and cache.get_seq_length(0) == n
        o_l, o_g = decode_attention(ql.to(cuda_device), qg.to(cuda_device), st, gate.to(cuda_device),
                                    thres.to(cuda_device), D ** -0.5)
        active = gate.float() >= 0.5
        n_loc = st_ref["attn_state"][0].shape[-2]
        ref_l = orc.decode_attn_ref(ql, st_ref["attn_state"][0], st_ref["attn_state"][1], [n_loc] * B)
        ref_g = orc.decode_attn_ref(qg, st_ref["attn_state_full"][0], st_ref["attn_state_full"][1], [n] * B,
                                    active=active)
        assert orc.abs_err(ref_l, o_l.float().cpu()) <= 1e-2
        assert orc.abs_err(ref_g, o_g.float().cpu()) <= 1e-2
        assert torch.all(o_g[~active.to(cuda_device)] == 0)
        assert int(st.status.item()) == 0
    # the contract view of the cache equals the reference's stored states
    state = cache[0]
    np.testing.assert_array_equal(state["attn_state_full"][0].float().cpu().numpy(),
                                  ref.states[0]["attn_state_full"][0].float().numpy())
    np.testing.assert_array_equal(state["attn_state"][1].float().cpu().numpy(),
                                  ref.states[0]["attn_state"][1].float().numpy())
    assert state["attn_state"][0].shape[-2] == W


def test_cache_update_contract(cuda_device):
    """Cache.update() with the reference's arguments returns the reference's dictionary."""
    from logo_b200 import Cache

    rs = np.random.RandomState(2)
    B, H, D, W = 2, 2, 128, 16
    ref, cache = orc.CacheRef(), Cache()
    for t_new in (40, 1, 1, 1):
        mk = lambda: _bf(rs.standard_normal((B, t_new, H, D))).transpose(1, 2)      # [B,H,t,D] views
        a, b, c, d = mk(), mk(), mk(), mk()
        want = ref.update((a, b), (c, d), 0, t_new, W)
        got = cache.update((a.to(cuda_device), b.to(cuda_device)), (c.to(cuda_device), d.to(cuda_device)),
                           layer_idx=0, offset=t_new, cache_kwargs={"window_size": W})
        for key in ("attn_state", "attn_state_full"):
            for i in range(2):
                np.testing.assert_array_equal(got[key][i].float().cpu().numpy(), want[key][i].float().numpy())
    assert cache.get_seq_length(0) == ref.seen == 43 and cache.get_seq_length(5) == 0
    assert len(cache) == 1 and cache.get_max_length() is None
    legacy = cache.to_legacy_cache()
    again = Cache.from_legacy_cache(legacy, window_size=W)
    assert again.get_seq_length(0) == 43
    np.testing.assert_array_equal(again[0]["attn_state"][0].float().cpu().numpy(),
                                  ref.states[0]["attn_state"][0].float().numpy())
    with pytest.raises(ValueError):
        cache.update((a, b), (c, d), 0, 1, {"window_size": 0})
    with pytest.raises(KeyError):
        cache[3]


def test_decode_long_context_many_splits(cuda_device):
    """A context that spans many key chunks, ragged last chunk, GQA 2."""
    from logo_b200 import Cache
    from logo_b200.layers import decode_attention

    g = torch.Generator(device="cuda").manual_seed(0)
    B, HQ, H, D, T = 4, 4, 2, 128, 5000
    cache = Cache(max_length=T + 8)
    mk = lambda *s: torch.randn(*s, device=cuda_device, generator=g).to(torch.bfloat16)
    kl, vl, kg, vg = mk(B, T, H, D), mk(B, T, H, D), mk(B, T, H, D), mk(B, T, H, D)
    st = cache.append(0, kl, vl, kg, vg, 128)
    ql, qg = mk(B, HQ, D), mk(B, HQ, D)
    gate = torch.tensor([0.9, 0.2, 0.7, 0.5], device=cuda_device).to(torch.bfloat16)
    thres = torch.tensor([0.5], device=cuda_device)
    o_l, o_g = decode_attention(ql, qg, st, gate, thres, D ** -0.5)
    bh = lambda x: x.transpose(1, 2).cpu()
    ref_g = orc.decode_attn_ref(qg.cpu(), bh(kg), bh(vg), [T] * B, active=gate.float().cpu() >= 0.5)
    ref_l = orc.decode_attn_ref(ql.cpu(), bh(kl), bh(vl), [T] * B, window=128)
    assert orc.abs_err(ref_g, o_g.float().cpu()) <= 1e-2
    assert orc.abs_err(ref_l, o_l.float().cpu()) <= 1e-2
    assert torch.all(o_g[1] == 0)


def test_rmsnorm_kernel_reproduces_reference_bf16_module(cuda_device, golden):
    """The row-wise RMSNorm kernel against the reference module's bf16 output (head rows of 128) and,
    for a decoder-width row, against the oracle's restatement of the module."""
    from logo_b200 import ops

    g = golden["misc"]
    rs = np.random.RandomState(77)
    n, h, d = 64, 2, 128
    local = _bf(rs.standard_normal((n, h, d)))
    _glob = rs.standard_normal((n, h, d))
    _gate = rs.uniform(0, 1, (n, 1))
    wl = _bf(1 + 0.1 * rs.standard_normal(d))
    got = ops.rmsnorm(local.to(cuda_device), wl.to(cuda_device), 1e-5).float().cpu().numpy().reshape(n, -1)
    ref = g["fuse/norm_local_bf16"]
    ulp = np.maximum(np.abs(ref), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - ref) <= ulp) and np.mean(got != ref) < 0.01

    x = _bf(rs.standard_normal((37, 2048)) * 3)
    w = _bf(1 + 0.1 * rs.standard_normal(2048))
    want = orc.rmsnorm_ref(x, w, 1e-5).float().numpy()
    got = ops.rmsnorm(x.to(cuda_device), w.to(cuda_device), 1e-5).float().cpu().numpy()
    ulp = np.maximum(np.abs(want), 2.0 ** -126) * 2.0 ** -7
    assert np.all(np.abs(got - want) <= ulp) and np.mean(got != want) < 0.01


def test_rmsnorm_module_uses_kernel_only_without_autograd(cuda_device):
    from logo_b200.layers import RMSNorm

    torch.manual_seed(3)
    m = RMSNorm(256, 1e-5).to(cuda_device, torch.bfloat16)
    x = torch.randn(5, 256, device=cuda_device).to(torch.bfloat16)
    with torch.no_grad():
        fast = m(x)
    slow = m(x.clone().requires_grad_(True))     # eager path: autograd needs the graph
    assert slow.requires_grad and not fast.requires_grad
    ulp = slow.detach().float().abs().clamp_min(2.0 ** -126) * 2.0 ** -7
    assert torch.all((fast.float() - slow.detach().float()).abs() <= ulp)


def test_silu_mul_matches_eager_bf16(cuda_device):
    """silu(gate) * up on the two halves of a fused projection (row-strided views), against the eager
    bf16 expression evaluated on the CPU (torch rounds silu to bf16, then multiplies in bf16)."""
    from logo_b200 import ops

    torch.manual_seed(4)
    gu = (torch.randn(37, 2 * 5632) * 2).to(torch.bfloat16)
    a, b = gu.chunk(2, dim=-1)
    want = (torch.nn.functional.silu(a) * b).float()
    gud = gu.to(cuda_device)
    ad, bd = gud.chunk(2, dim=-1)
    got = ops.silu_mul(ad, bd).float().cpu()
    ulp = want.abs().clamp_min(2.0 ** -126) * 2.0 ** -7
    assert torch.all((got - want).abs() <= ulp)       # expf differs in its last bits between CPU and GPU
    assert (got != want).float().mean().item() < 0.01
    assert ops.silu_mul(ad[:0], bd[:0]).shape == (0, 5632)
