"""Rotary-embedding kernel through the C ABI: bit-exact against the eager bf16 expression of
logo/modules/rotary.py:81-106 (evaluated on the CPU by the oracle helper), forward and gradient."""
import numpy as np
import pytest
import torch

from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu


def _tables(n, d, seed):
    rs = np.random.RandomState(seed)
    pos = rs.randint(0, 8192, size=n).astype(np.float32)
    inv = 1.0 / (10000.0 ** (np.arange(0, d, 2, dtype=np.float32) / d))
    ang = pos[:, None] * inv[None, :]
    emb = np.concatenate([ang, ang], axis=-1)
    return (torch.from_numpy(np.cos(emb)).to(torch.bfloat16), torch.from_numpy(np.sin(emb)).to(torch.bfloat16))


@pytest.mark.parametrize("n,h", [(1, 1), (37, 3), (300, 16), (4096, 16)])
def test_rope_forward_bit_exact(cuda_device, n, h):
    from logo_b200 import ops

    torch.manual_seed(n + h)
    x = torch.randn(n, h, 128).to(torch.bfloat16)
    cos, sin = _tables(n, 128, n)
    want = orc.apply_rope(x, cos, sin)
    got = ops.rope(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_rope_tables_with_unequal_halves(cuda_device):
    """Nothing may assume cos[d] == cos[d + 64]: arbitrary tables give the eager result too."""
    from logo_b200 import ops

    torch.manual_seed(5)
    x = torch.randn(50, 4, 128).to(torch.bfloat16)
    cos, sin = torch.randn(50, 128).to(torch.bfloat16), torch.randn(50, 128).to(torch.bfloat16)
    want = orc.apply_rope(x, cos, sin)
    got = ops.rope(x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)).cpu()
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


def test_rope_gradient_matches_autograd_of_eager_graph(cuda_device):
    from logo_b200 import ops

    torch.manual_seed(9)
    n, h = 257, 5
    x = torch.randn(n, h, 128).to(torch.bfloat16)
    g = torch.randn(n, h, 128).to(torch.bfloat16)
    cos, sin = _tables(n, 128, 3)
    x_ref = x.clone().requires_grad_(True)
    orc.apply_rope(x_ref, cos, sin).backward(g)
    x_dev = x.to(cuda_device).requires_grad_(True)
    ops.rope(x_dev, cos.to(cuda_device), sin.to(cuda_device)).backward(g.to(cuda_device))
    assert torch.equal(x_dev.grad.cpu().view(torch.int16), x_ref.grad.view(torch.int16))


def test_rope_in_place_and_empty(cuda_device):
    import ctypes

    from logo_b200 import _lib

    lib = _lib.load()
    x = torch.randn(64, 2, 128).to(torch.bfloat16)
    cos, sin = _tables(64, 128, 1)
    want = orc.apply_rope(x, cos, sin)
    xd, cd, sd = x.to(cuda_device), cos.to(cuda_device), sin.to(cuda_device)
    rc = lib.logo_rope(xd.data_ptr(), 256, 128, xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), 64, 2, 128, 0, None)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(xd.cpu().view(torch.int16), want.view(torch.int16))
    assert lib.logo_rope(None, 256, 128, None, None, None, 0, 2, 128, 0, None) == 0
    assert lib.logo_rope(xd.data_ptr(), 256, 128, xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), 64, 2, 64, 0, None) != 0
    assert lib.logo_rope(xd.data_ptr(), 252, 128, xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), 64, 2, 128, 0, None) != 0


def test_rope_head_major_input_view(cuda_device):
    """The global branch's per-head projection comes out as a [H, N, D] buffer viewed [N, H, D]."""
    from logo_b200 import ops

    torch.manual_seed(21)
    n, h = 130, 4
    buf = torch.randn(h, n, 128).to(torch.bfloat16)
    cos, sin = _tables(n, 128, 8)
    want = orc.apply_rope(buf.permute(1, 0, 2), cos, sin)
    got = ops.rope(buf.to(cuda_device).permute(1, 0, 2), cos.to(cuda_device), sin.to(cuda_device))
    assert got.is_contiguous()
    assert torch.equal(got.cpu().view(torch.int16), want.contiguous().view(torch.int16))


def test_rope_against_reference_fixture(cuda_device, golden):
    from golden_inputs import rope_case
    from logo_b200 import ops

    g = golden["rope"]
    x, grad_out, _ = rope_case()
    cos = torch.from_numpy(g["cos"]).to(torch.bfloat16).to(cuda_device)
    sin = torch.from_numpy(g["sin"]).to(torch.bfloat16).to(cuda_device)
    xd = torch.from_numpy(x).to(torch.bfloat16).to(cuda_device).requires_grad_(True)
    out = ops.rope(xd, cos, sin)
    out.backward(torch.from_numpy(grad_out).to(torch.bfloat16).to(cuda_device))
    np.testing.assert_array_equal(out.detach().float().cpu().numpy(), g["out"])
    np.testing.assert_array_equal(xd.grad.float().cpu().numpy(), g["grad"])


@pytest.mark.parametrize("with_rows,with_rope", [(False, True), (True, True), (False, False)])
def test_proj_rope_matches_the_eager_bf16_graph(cuda_device, with_rows, with_rope):
    """Per-head projection + rotary embedding in one kernel against the eager bf16 expressions it replaces
    (the einsum of logo/layers/logo.py:86-94 followed by apply_rotary_pos_emb): same roundings, so the
    results agree except where the two fp32 accumulation orders of the product round to neighbouring
    bf16 values. Forward and the gradients of x and w."""
    from logo_b200 import ops

    torch.manual_seed(5)
    n, heads, d = 700, 3, 128
    x = torch.randn(n, heads * d, device=cuda_device).to(torch.bfloat16)
    w = (torch.eye(d, device=cuda_device)[None] + 0.05 * torch.randn(heads, d, d, device=cuda_device)).to(torch.bfloat16)
    pos = torch.arange(n, device=cuda_device).float()
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, device=cuda_device).float() / d))
    emb = torch.cat([pos[:, None] * inv[None], pos[:, None] * inv[None]], dim=-1)
    cos, sin = (emb.cos().to(torch.bfloat16), emb.sin().to(torch.bfloat16)) if with_rope else (None, None)
    sel = None
    keep = torch.ones(n, dtype=torch.bool, device=cuda_device)
    if with_rows:
        keep = torch.rand(n, device=cuda_device) < 0.4
        sel = ops.select_rows(keep, None, torch.tensor([0, 300, 300, n], dtype=torch.int32, device=cuda_device))
    g_out = torch.randn(n, heads, d, device=cuda_device).to(torch.bfloat16) * keep[:, None, None]

    def eager(xr, wr):
        y = torch.einsum("l h d, h d e -> l h e", xr.view(n, heads, d), wr)
        if cos is None:
            return y
        rot = torch.cat((-y[..., d // 2:], y[..., : d // 2]), dim=-1)
        return (y * cos[:, None, :]) + (rot * sin[:, None, :])

    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ref = eager(xr, wr)
    ref.backward(g_out)
    xd, wd = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    out = ops.proj_rope(xd.view(n, heads, d), wd, cos, sin, sel)
    out.backward(g_out)
    torch.cuda.synchronize()
    if sel is not None:
        assert int(sel.status.item()) == 0
    got, want = out[keep].float(), ref.detach()[keep].float()
    ulp = want.abs().clamp_min(2.0 ** -126) * 2.0 ** -7
    assert torch.all((got - want).abs() <= 2 * ulp + 1e-3)       # neighbouring bf16 values at most, rotation included
    assert (got != want).float().mean().item() < 0.05
    assert oracle_err(xr.grad.float(), xd.grad.float()) < 1e-2
    assert oracle_err(wr.grad.float(), wd.grad.float()) < 1e-2


def oracle_err(ref, got):
    return ((ref - got).square().mean().sqrt() / (ref.square().mean().sqrt() + 1e-8)).item()
