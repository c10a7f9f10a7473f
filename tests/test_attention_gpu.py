"""Query-sparse global attention and window local attention, forward and backward, through the
C ABI against the CPU oracle (fp32 dense-masked) and the reference's own kernel outputs.

Tolerances are the contract's: bf16 outputs within 1e-2 max-abs of the fp32 result, gradients
within 2e-2 RMS-relative (the reference's get_err_ratio)."""
import zlib

import numpy as np
import pytest
import torch

from golden_inputs import ATTN_CASES, attn_case_inputs
from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu

OUT_ATOL = 1e-2
GRAD_RATIO = 2e-2


def _inputs(lens, hq, h, ratio, seed, scale_qk=1.0):
    rs = np.random.RandomState(seed)
    n, d = sum(lens), 128
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64).tolist()
    mk = lambda *s: torch.from_numpy(rs.standard_normal(s).astype(np.float32)).to(torch.bfloat16)
    q, k, v, do = mk(n, hq, d) * scale_qk, mk(n, h, d) * scale_qk, mk(n, h, d), mk(n, hq, d)
    sel = torch.from_numpy(rs.uniform(size=n) < ratio) if ratio < 1 else torch.ones(n, dtype=torch.bool)
    return q, k, v, do, sel, cu


def _oracle(q, k, v, do, sel, cu, window):
    qr, kr, vr = (x.float().requires_grad_(True) for x in (q, k, v))
    o, lse = orc.attention_dense_ref(qr, kr, vr, cu, None, window, sel)
    o.backward(do.float())
    return o.detach(), lse.detach(), qr.grad, kr.grad, vr.grad


GLOBAL_CASES = {
    "one_tile": ([128], 1, 1, 1.0),
    "ragged_rows": ([300], 2, 1, 1.0),
    "half_selected": ([1000], 2, 2, 0.5),
    "varlen_gqa_empty_seq": ([70, 0, 130, 513, 1, 700], 4, 2, 0.3),
    "gqa4": ([400, 90], 4, 1, 0.6),
    "heads32_kv8": ([300, 140], 32, 8, 0.5),
    "sparse_long": ([4096], 2, 1, 0.125),
    "single_token_seqs": ([1, 1, 1, 257], 2, 2, 1.0),
    # more work items than SMs in every kernel: CTAs claim several items, the record ring wraps
    "many_items": ([3000, 500], 16, 4, 0.8),
}


@pytest.fixture
def bwd_mode():
    """Sets the backward implementation of a branch for one test and restores the default afterwards."""
    import logo_b200

    saved = {b: logo_b200.get_backward_mode(b) for b in ("global", "local")}

    def choose(branch, mode):
        logo_b200.set_backward_mode(branch, mode)

    yield choose
    for b, m in saved.items():
        logo_b200.set_backward_mode(b, m)


@pytest.mark.parametrize("mode", ["single_pass", "two_kernel"])
@pytest.mark.parametrize("name", sorted(GLOBAL_CASES))
def test_sq_full_attn_fwd_bwd_vs_oracle(cuda_device, bwd_mode, name, mode):
    from logo_b200 import ops

    bwd_mode("global", mode)
    lens, hq, h, ratio = GLOBAL_CASES[name]
    q, k, v, do, sel, cu = _inputs(lens, hq, h, ratio, seed=zlib.crc32(name.encode()) % 1000)
    o_ref, lse_ref, dq_ref, dk_ref, dv_ref = _oracle(q, k, v, do, sel, cu, None)
    qd, kd, vd = (x[None].to(cuda_device).requires_grad_(True) for x in (q, k, v))
    o = ops.sq_full_attn(qd, kd, vd, sel[None].to(cuda_device), cu_seqlens=torch.tensor(cu, dtype=torch.int32))
    o.backward(do[None].to(cuda_device))
    assert o.dtype == torch.bfloat16 and o.shape == qd.shape
    assert orc.abs_err(o_ref, o[0].float().cpu()) <= OUT_ATOL
    assert torch.all(o[0][~sel.to(cuda_device)] == 0), "unselected rows must be exactly zero"
    assert torch.all(qd.grad[0][~sel.to(cuda_device)] == 0), "dq of unselected rows must be exactly zero"
    for nm, ref, got in (("dq", dq_ref, qd.grad), ("dk", dk_ref, kd.grad), ("dv", dv_ref, vd.grad)):
        got = got[0].float().cpu()
        assert not torch.isnan(got).any()
        assert orc.err_ratio(ref, got) < GRAD_RATIO, (name, nm, orc.err_ratio(ref, got))


@pytest.mark.parametrize("name", [n for n in sorted(ATTN_CASES) if ATTN_CASES[n][3] == 128])
def test_sq_full_attn_vs_reference_kernel_outputs(cuda_device, golden, name):
    """Same seeded inputs as the fixtures produced by the reference's Triton kernels (fp32)."""
    from logo_b200 import ops

    q, k, v, do, sel, cu = attn_case_inputs(name)
    g = golden["attention"]
    bf = lambda a: torch.from_numpy(a).to(torch.bfloat16)[None].to(cuda_device).requires_grad_(True)
    qd, kd, vd = bf(q), bf(k), bf(v)
    o = ops.sq_full_attn(qd, kd, vd, torch.from_numpy(sel)[None].to(cuda_device),
                         cu_seqlens=torch.tensor(cu, dtype=torch.int32))
    o.backward(torch.from_numpy(do).to(torch.bfloat16)[None].to(cuda_device))
    # inputs are rounded to bf16 here, the fixture is fp32 end to end: allow the input rounding
    assert orc.abs_err(torch.from_numpy(g[f"{name}/o"]), o[0].float().cpu()) <= 3e-2
    for nm, got in (("dq", qd.grad), ("dk", kd.grad), ("dv", vd.grad)):
        assert orc.err_ratio(torch.from_numpy(g[f"{name}/{nm}"]), got[0].float().cpu()) < GRAD_RATIO


LOCAL_CASES = {
    "short": ([100], 2, 1, 128),
    "ragged": ([300], 2, 1, 128),
    "varlen_gqa": ([70, 0, 130, 513, 1, 700], 4, 2, 128),
    "window64": ([1000], 2, 2, 64),
    "window200": ([900, 300], 2, 1, 200),
    "many_items": ([2500, 700], 16, 16, 128),
}


@pytest.mark.parametrize("mode", ["single_pass", "two_kernel"])
@pytest.mark.parametrize("name", sorted(LOCAL_CASES))
def test_swa_fwd_bwd_vs_oracle(cuda_device, bwd_mode, name, mode):
    from logo_b200 import ops

    bwd_mode("local", mode)
    lens, hq, h, window = LOCAL_CASES[name]
    q, k, v, do, _, cu = _inputs(lens, hq, h, 1.0, seed=zlib.crc32(name.encode()) % 1000)
    o_ref, _, dq_ref, dk_ref, dv_ref = _oracle(q, k, v, do, None, cu, window)
    qd, kd, vd = (x.to(cuda_device).requires_grad_(True) for x in (q, k, v))
    o = ops.swa_attn(qd, kd, vd, torch.tensor(cu, dtype=torch.int32, device=cuda_device), window)
    o.backward(do.to(cuda_device))
    assert orc.abs_err(o_ref, o.float().cpu()) <= OUT_ATOL
    for nm, ref, got in (("dq", dq_ref, qd.grad), ("dk", dk_ref, kd.grad), ("dv", dv_ref, vd.grad)):
        assert orc.err_ratio(ref, got.float().cpu()) < GRAD_RATIO, (name, nm)


def test_empty_selection_and_empty_input(cuda_device):
    from logo_b200 import ops

    q, k, v, do, _, cu = _inputs([256, 100], 2, 2, 1.0, seed=9)
    sel = torch.zeros(356, dtype=torch.bool)
    qd, kd, vd = (x[None].to(cuda_device).requires_grad_(True) for x in (q, k, v))
    o = ops.sq_full_attn(qd, kd, vd, sel[None].to(cuda_device), cu_seqlens=torch.tensor(cu, dtype=torch.int32))
    o.backward(do[None].to(cuda_device))
    for t in (o, qd.grad, kd.grad, vd.grad):
        assert torch.all(t == 0)


@pytest.mark.parametrize("mode", ["single_pass", "two_kernel"])
def test_full_size_properties(cuda_device, bwd_mode, mode):
    """The benchmark shape (4 x 8192 tokens, 16 heads): properties that need no oracle.

    * V == 1 everywhere: every selected output row is exactly 1, every other row 0;
    * all-ones selection == the local kernel with a window that covers the whole sequence;
    * linearity in V and in dO; two runs are bit-identical (dq of the single-pass backward, which is
      summed by reductions in varying order, to within the last bits of its fp32 sum).
    """
    from logo_b200 import ops, ops_bwd

    bwd_mode("global", mode)

    n, hq, d = 32768, 16, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    cu = torch.arange(0, n + 1, 8192, dtype=torch.int32, device=cuda_device)
    mk = lambda: (torch.randn(n, hq, d, device=cuda_device, generator=g) * d ** -0.25).to(torch.bfloat16)
    q, k = mk(), mk()
    sel = torch.rand(n, device=cuda_device, generator=g) < 0.5
    m = ops.select_rows(sel, None, cu)
    ones = torch.ones(n, hq, d, dtype=torch.bfloat16, device=cuda_device)
    o, lse = ops.sq_attn_fwd_raw(q, k, ones, m, d ** -0.5)
    assert torch.all(o[~sel] == 0)
    assert (o[sel].float() - 1).abs().max().item() <= 2 ** -7    # row sums of P are 1 up to bf16 rounding of P
    assert torch.isfinite(lse[sel]).all()

    v = torch.randn(n, hq, d, device=cuda_device, generator=g).to(torch.bfloat16)
    o1, lse1 = ops.sq_attn_fwd_raw(q, k, v, m, d ** -0.5)
    o2, _ = ops.sq_attn_fwd_raw(q, k, v, m, d ** -0.5)
    assert torch.equal(o1, o2)
    o_2v, _ = ops.sq_attn_fwd_raw(q, k, (v.float() * 2).to(torch.bfloat16), m, d ** -0.5)
    assert (o_2v.float() - 2 * o1.float()).abs().max().item() <= 2e-2

    # all rows selected == window attention whose window covers the sequence
    m_all = ops.select_rows(torch.ones(n, dtype=torch.bool, device=cuda_device), None, cu)
    oa, _ = ops.sq_attn_fwd_raw(q, k, v, m_all, d ** -0.5)
    ow, _ = ops.swa_fwd_raw(q, k, v, m_all, 8192, d ** -0.5)
    assert (oa.float() - ow.float()).abs().max().item() <= 1e-2

    do = torch.randn(n, hq, d, device=cuda_device, generator=g).to(torch.bfloat16)
    dq, dk, dv = ops_bwd.sq_attn_bwd_raw(q, k, v, o1, lse1, do, m, d ** -0.5)
    dq2, dk2, dv2 = ops_bwd.sq_attn_bwd_raw(q, k, v, o1, lse1, do, m, d ** -0.5)
    assert torch.equal(dk, dk2) and torch.equal(dv, dv2)
    if mode == "two_kernel":
        assert torch.equal(dq, dq2)
    else:
        assert orc.err_ratio(dq.float(), dq2.float()) < 1e-3
    assert torch.all(dq[~sel] == 0)
    # sum_i dS_ij = 0 row-wise  =>  dq is orthogonal to nothing in particular, but dv is linear in dO:
    _, _, dv_half = ops_bwd.sq_attn_bwd_raw(q, k, v, o1, lse1, (do.float() * 0.5).to(torch.bfloat16), m, d ** -0.5)
    assert orc.err_ratio(dv.float() * 0.5, dv_half.float()) < 1e-2
    # column sums: sum over tokens of dv equals P^T dO summed = sum over selected rows of dO (P rows sum to 1)
    per_seq = dv.float().view(4, 8192, hq, d).sum(1)
    ref = (do.float() * sel[:, None, None]).view(4, 8192, hq, d).sum(1)
    assert orc.err_ratio(ref, per_seq) < 2e-2
    assert int(m.status.item()) == 0 and int(m_all.status.item()) == 0


def test_umma_operand_encodings(cuda_device):
    """The tcgen05 operand encodings the attention kernels rely on, on one 128x128x128 tile."""
    from logo_b200 import _lib

    lib = _lib.load()
    g = torch.Generator(device="cuda").manual_seed(1)
    a = torch.randn(128, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    b = torch.randn(128, 128, device=cuda_device, generator=g).to(torch.bfloat16)
    abt, ab, atb = a.float() @ b.float().T, a.float() @ b.float(), a.float().T @ b.float()
    # (mode, flags, expected): flags bit 0 / bit 2 = A / B written by threads into the swizzled layout
    abt16 = abt + a.float()[:, :16] @ b.float()[:, :16].T   # mode 4: a ninth k-step from 32-byte-swizzled tiles
    # mode 5: the ninth k-step's A operand is a 256-byte tile of identical rows (a[0, 0:16]), no swizzle,
    # distance 128 bytes between its two K chunks and 0 between 8-row groups
    abt_row = abt + (b.float()[:, :16] @ a.float()[0, :16])[None, :]
    cases = ((0, 0, abt), (0, 1, abt), (1, 0, ab), (1, 4, ab), (1, 5, ab), (2, 0, ab), (3, 0, atb), (3, 4, atb),
             (4, 0, abt16), (5, 0, abt_row))
    for mode, flags, ref in cases:
        c = torch.full((128, 128), float("nan"), device=cuda_device)
        st = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        lbo, sbo, kstep = (0, 0, 128) if mode == 5 else (16384 if mode else 0, 1024, 2048)
        rc = lib.logo_umma_selftest(mode, flags, a.data_ptr(), b.data_ptr(), c.data_ptr(), lbo, sbo, kstep,
                                    st.data_ptr(), None)
        _lib.check(rc, "logo_umma_selftest")
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        assert (c - ref).abs().max().item() < 1e-3, (mode, flags)


def test_bounded_wait_runs_out_and_the_context_survives(cuda_device):
    """Every device-side wait of the library is bounded: a barrier that nothing arms makes the wait
    give up after its limit (50 ms here), the kernel returns, the status word says so, and the next
    launch on the same context works."""
    from logo_b200 import _lib

    lib = _lib.load()
    a = torch.ones(128, 128, device=cuda_device, dtype=torch.bfloat16)
    c = torch.full((128, 128), -7.0, device=cuda_device)
    st = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    flags = 8 | (50000 << 8)          # bit 3: the load barrier is never armed; wait limit 50 000 us
    _lib.check(lib.logo_umma_selftest(0, flags, a.data_ptr(), a.data_ptr(), c.data_ptr(), 0, 1024, 2048,
                                      st.data_ptr(), None), "logo_umma_selftest")
    torch.cuda.synchronize()
    assert int(st.item()) == 1          # LOGO_DEV_WAIT_TIMEOUT
    assert torch.all(c == -7.0)         # no result was written
    st.zero_()
    _lib.check(lib.logo_umma_selftest(0, 0, a.data_ptr(), a.data_ptr(), c.data_ptr(), 0, 1024, 2048,
                                      st.data_ptr(), None), "logo_umma_selftest")
    torch.cuda.synchronize()
    assert int(st.item()) == 0 and torch.all(c == 128.0)
