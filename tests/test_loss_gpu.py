"""lm_head + shifted cross-entropy with packed-boundary masking against the oracle (fp32 autograd)."""
import numpy as np
import pytest
import torch

from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu


def _case(n_rows_shape, vocab, hid, cu, seed, ignore_some=True):
    rs = np.random.RandomState(seed)
    hidden = torch.from_numpy(rs.standard_normal(n_rows_shape + (hid,)).astype(np.float32)).to(torch.bfloat16)
    weight = torch.from_numpy((rs.standard_normal((vocab, hid)) * hid ** -0.5).astype(np.float32)).to(torch.bfloat16)
    labels = torch.from_numpy(rs.randint(0, vocab, size=n_rows_shape).astype(np.int64))
    if ignore_some:
        labels.view(-1)[rs.choice(labels.numel(), labels.numel() // 7, replace=False)] = -100
    return hidden, weight, labels, cu


@pytest.mark.parametrize("name,shape,vocab,cu,chunk", [
    ("packed_varlen", (1, 700), 1000 * 8, [0, 130, 130, 131, 700], 256),      # empty and one-token sequences, several chunks
    ("batch_rows", (3, 150), 512, None, 8192),
    ("one_chunk_big_vocab", (1, 64), 32000, [0, 64], 8192),
])
def test_lm_head_cross_entropy_vs_oracle(cuda_device, name, shape, vocab, cu, chunk):
    from logo_b200 import ops

    hid = 256
    hidden, weight, labels, cu = _case(shape, vocab, hid, cu, seed=len(name))
    hr, wr = hidden.float().requires_grad_(True), weight.float().requires_grad_(True)
    # the oracle sees the logits the bf16 lm_head produces (the reference upcasts AFTER the bf16 linear)
    exact = hr @ wr.t()
    logits = exact + (exact.to(torch.bfloat16).float() - exact).detach()
    ref = orc.lm_loss_ref(logits, labels, cu)
    ref.backward()

    hd = hidden.to(cuda_device).requires_grad_(True)
    wd = weight.to(cuda_device).requires_grad_(True)
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.int32, device=cuda_device)
    loss = ops.lm_head_cross_entropy(hd, wd, labels.to(cuda_device), cu_t, chunk_rows=chunk)
    assert loss.dtype == torch.float32 and loss.dim() == 0
    (loss * 2.0).backward()          # an upstream factor must scale both gradients
    # cuBLAS accumulates the bf16 logits in another order than the CPU product: a few logits land on the
    # other side of a bf16 rounding boundary
    assert abs(float(loss) - float(ref)) < 2e-3 * max(1.0, abs(float(ref)))
    assert orc.err_ratio(2.0 * hr.grad, hd.grad.float().cpu()) < 2e-2
    assert orc.err_ratio(2.0 * wr.grad, wd.grad.float().cpu()) < 2e-2


def test_shifted_targets_are_bit_exact_and_ignored_rows_get_zero_gradient(cuda_device):
    from logo_b200 import _lib

    lib = _lib.load()
    rs = np.random.RandomState(3)
    lens = [5, 0, 1, 300, 2]
    n, vocab = sum(lens), 64
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    labels = rs.randint(0, vocab, size=n).astype(np.int64)
    labels[[2, 100, 306]] = -100
    want = np.full(n, -100, dtype=np.int64)
    for a, b in zip(cu[:-1], cu[1:]):
        want[a:b - 1] = labels[a + 1:b] if b - a > 1 else want[a:b - 1]
    lab_d = torch.from_numpy(labels).to(cuda_device)
    cu_d = torch.from_numpy(cu).to(cuda_device)
    targets = torch.empty(n, dtype=torch.int64, device=cuda_device)
    n_valid = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    _lib.check(lib.logo_shift_labels(lab_d.data_ptr(), cu_d.data_ptr(), len(lens), n, -100, targets.data_ptr(),
                                     n_valid.data_ptr(), None), "logo_shift_labels")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(targets.cpu().numpy(), want)
    assert int(n_valid.item()) == int((want != -100).sum())

    logits = torch.from_numpy(rs.standard_normal((n, vocab)).astype(np.float32)).to(torch.bfloat16).to(cuda_device)
    keep = logits.clone()
    row_loss = torch.empty(n, dtype=torch.float32, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    _lib.check(lib.logo_ce_rows(logits.data_ptr(), vocab, targets.data_ptr(), -100, row_loss.data_ptr(),
                                n_valid.data_ptr(), 1.0, n, vocab, 1, status.data_ptr(), None), "logo_ce_rows")
    torch.cuda.synchronize()
    ignored = torch.from_numpy(want == -100).to(cuda_device)
    assert torch.all(logits[ignored] == 0) and torch.all(row_loss[ignored] == 0) and int(status.item()) == 0
    ref = torch.nn.functional.cross_entropy(keep.float().cpu(), torch.from_numpy(want), ignore_index=-100, reduction="none")
    assert (row_loss.cpu() - ref).abs().max().item() < 1e-4
    # gradient rows sum to zero (softmax minus one-hot) up to bf16 rounding
    assert logits[~ignored].float().sum(-1).abs().max().item() < 1e-3
