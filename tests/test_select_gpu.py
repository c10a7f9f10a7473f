"""Row selection / compaction kernel: bit-exact against the reference's build_selection outputs."""
import numpy as np
import pytest
import torch

from golden_inputs import selection_cases
from oracle import logo_oracle as orc

pytestmark = pytest.mark.gpu


def _check_against(m, sel_ref, cu):
    sq = int(m.meta[0].item())
    assert int(m.status.item()) == 0
    assert sq == sel_ref.Sq
    assert m.q_idx.dtype == torch.int64 and m.pos_ids.dtype == torch.int32 and m.cu_seqlens_q.dtype == torch.int32
    np.testing.assert_array_equal(m.q_idx[:sq].cpu().numpy(), sel_ref.q_idx)
    np.testing.assert_array_equal(m.pos_ids[:sq].cpu().numpy(), sel_ref.pos_ids)
    np.testing.assert_array_equal(m.cu_seqlens_q.cpu().numpy(), sel_ref.cu_seqlens_q)
    off = m.tile_off.cpu().numpy()
    np.testing.assert_array_equal(off[0], orc.tile_offsets_ref(sel_ref.cu_seqlens_q, 256))
    np.testing.assert_array_equal(off[1], orc.tile_offsets_ref(cu, 128))
    np.testing.assert_array_equal(off[2], orc.tile_offsets_ref(cu, 256))
    np.testing.assert_array_equal(off[3], orc.tile_offsets_ref(sel_ref.cu_seqlens_q, 128))
    np.testing.assert_array_equal(m.meta[1:5].cpu().numpy(), off[:, -1])


@pytest.mark.parametrize("name", sorted(selection_cases()))
def test_bool_mask_matches_reference_golden(cuda_device, golden, name):
    from logo_b200 import ops

    mask, cu = selection_cases()[name]
    g = golden["selection"]
    m = ops.select_rows(torch.from_numpy(mask).to(cuda_device), None, torch.tensor(cu, dtype=torch.int32))
    sq = int(m.meta[0].item())
    np.testing.assert_array_equal(m.q_idx[:sq].cpu().numpy(), g[f"{name}/q_idx"])
    np.testing.assert_array_equal(m.pos_ids[:sq].cpu().numpy(), g[f"{name}/pos_ids"])
    np.testing.assert_array_equal(m.cu_seqlens_q.cpu().numpy(), g[f"{name}/cu_seqlens_q"])
    # the tile-offset rows are the prefix-sum form of the reference's chunk lists
    assert int(m.meta[4].item()) == g[f"{name}/chunks_q128"].shape[0]
    assert int(m.meta[2].item()) == g[f"{name}/chunks_k128"].shape[0]
    _check_against(m, orc.build_selection_ref(mask, cu), cu)
    info = ops.build_selection(torch.from_numpy(mask)[None].to(cuda_device), 1, mask.size,
                               torch.tensor(cu, dtype=torch.int32))
    assert info.Sq == sq and info.Nseq == len(cu) - 1 and info.q_idx.numel() == sq


@pytest.mark.parametrize("gate_dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("thres_dtype", [torch.float32, torch.bfloat16])
def test_gate_threshold_compare_in_fp32(cuda_device, gate_dtype, thres_dtype):
    from logo_b200 import ops

    rs = np.random.RandomState(5)
    n = 70000   # several scan blocks, ragged tail
    gate = torch.from_numpy(rs.uniform(0, 1, n).astype(np.float32)).to(gate_dtype)
    gate[17] = float("nan")
    thres = torch.tensor([0.4375], dtype=thres_dtype)       # exactly representable: ties are exercised
    gate[100:110] = 0.4375
    cu = [0, 1, 40000, 40000, n]
    m = ops.select_rows(gate.to(cuda_device), thres.to(cuda_device), torch.tensor(cu, dtype=torch.int32))
    mask = orc.select_from_gate(gate.float().numpy(), float(thres.float().item()))
    assert not mask[17] and mask[100:110].all()
    _check_against(m, orc.build_selection_ref(mask, cu), cu)
    finite = torch.nan_to_num(gate.float(), nan=0.0)
    # the by-product gate sum (NaN propagates exactly like torch.sum)
    assert torch.isnan(m.gate_sum).item()
    gate[17] = 0.25
    m = ops.select_rows(gate.to(cuda_device), thres.to(cuda_device), torch.tensor(cu, dtype=torch.int32))
    assert abs(m.gate_sum.item() - gate.float().sum().item()) < 1e-3 * n ** 0.5 + 1e-2 * (gate_dtype != torch.float32)
    del finite


def test_large_and_deterministic(cuda_device):
    from logo_b200 import ops

    n = 1 << 20
    g = torch.Generator(device="cpu").manual_seed(3)
    mask = torch.rand(n, generator=g) < 0.37
    lens = [8192] * 100 + [n - 819200]
    cu = np.concatenate([[0], np.cumsum(lens)]).tolist()
    cu_t = torch.tensor(cu, dtype=torch.int32)
    a = ops.select_rows(mask.to(cuda_device), None, cu_t)
    b = ops.select_rows(mask.to(cuda_device), None, cu_t)
    _check_against(a, orc.build_selection_ref(mask.numpy(), cu), cu)
    sq = int(a.meta[0].item())
    assert torch.equal(a.q_idx[:sq], b.q_idx[:sq]) and torch.equal(a.pos_ids[:sq], b.pos_ids[:sq])
    # properties that do not depend on the size: sorted, unique, positions restart at sequence starts
    q = a.q_idx[:sq]
    assert bool((q[1:] > q[:-1]).all())
    assert bool((a.pos_ids[:sq].long() == q - cu_t.to(cuda_device).long()[torch.searchsorted(
        cu_t.to(cuda_device).long(), q, right=True) - 1]).all())


def test_empty_inputs(cuda_device):
    from logo_b200 import ops

    m = ops.select_rows(torch.zeros(0, dtype=torch.bool, device=cuda_device), None,
                        torch.tensor([0], dtype=torch.int32))
    assert m.meta[:5].tolist() == [0, 0, 0, 0, 0] and int(m.status.item()) == 0
    m = ops.select_rows(torch.ones(5, dtype=torch.bool, device=cuda_device), None,
                        torch.tensor([0, 0, 5, 5], dtype=torch.int32))
    assert m.cu_seqlens_q.tolist() == [0, 0, 5, 5] and m.pos_ids[:5].tolist() == [0, 1, 2, 3, 4]


def test_malformed_cu_seqlens_sets_status_not_a_fault(cuda_device):
    from logo_b200 import ops

    m = ops.select_rows(torch.ones(64, dtype=torch.bool, device=cuda_device), None,
                        torch.tensor([0, 40, 30, 64], dtype=torch.int32))
    torch.cuda.synchronize()
    assert int(m.status.item()) == 2
    with pytest.raises(RuntimeError, match="out of range"):
        ops.check_device_status(m.status)
