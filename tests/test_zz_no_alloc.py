"""logo_select_rows_static: the row-selection entry point for hosts that may not allocate device
memory (its scan scratch is a static device array inside the library instead of a caller buffer).

Checked through the C ABI against the regular logo_select_rows on the same inputs, on two calls in a
row with different inputs, so a stale ticket or look-back word left by the first call would show.
The integer outputs and the ordered gate sum must be bit-identical."""
import ctypes

import numpy as np
import pytest
import torch


def _buffers(n, nseq, dev):
    return dict(q_idx=torch.full((max(n, 1),), -1, dtype=torch.int64, device=dev),
                pos_ids=torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev),
                cu_q=torch.full((nseq + 1,), -1, dtype=torch.int32, device=dev),
                tile_off=torch.full((4, nseq + 1), -1, dtype=torch.int32, device=dev),
                meta=torch.full((16,), -1, dtype=torch.int32, device=dev),
                gate_sum=torch.full((1,), float("nan"), dtype=torch.float32, device=dev),
                status=torch.zeros(1, dtype=torch.int32, device=dev))


def _call(lib, static, gate, thres, cu, dev):
    from logo_b200 import _lib

    n, nseq = gate.numel(), cu.numel() - 1
    b = _buffers(n, nseq, dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    head = (gate.data_ptr(), _lib.torch_dtype_code(gate.dtype), thres.data_ptr(), _lib.torch_dtype_code(thres.dtype),
            cu.data_ptr(), nseq, n, b["q_idx"].data_ptr(), b["pos_ids"].data_ptr(), b["cu_q"].data_ptr(),
            b["tile_off"].data_ptr(), b["meta"].data_ptr(), b["gate_sum"].data_ptr())
    if static:
        rc = lib.logo_select_rows_static(*head, b["status"].data_ptr(), stream)
    else:
        ws = torch.empty(lib.logo_select_workspace_bytes(n), dtype=torch.uint8, device=dev)
        rc = lib.logo_select_rows(*head, ws.data_ptr(), ws.numel(), b["status"].data_ptr(), stream)
    _lib.check(rc, "select")
    torch.cuda.synchronize()
    return b


@pytest.mark.gpu
def test_static_scratch_variant_matches_workspace_variant_twice(cuda_device):
    from logo_b200 import _lib

    lib = _lib.load()
    rs = np.random.RandomState(2024)
    # second call: fewer tokens and fewer scan blocks than the first, other threshold, other sequences
    for n, lens, thr in ((150_001, [70_000, 0, 1, 80_000], 0.3), (9_000, [4_096, 4_904], 0.8)):
        gate = torch.from_numpy(rs.uniform(0, 1, n).astype(np.float32)).to(torch.bfloat16).to(cuda_device)
        thres = torch.tensor([thr], dtype=torch.float32, device=cuda_device)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=cuda_device)
        want = _call(lib, False, gate, thres, cu, cuda_device)
        got = _call(lib, True, gate, thres, cu, cuda_device)
        sq = int(want["meta"][0].item())
        assert 0 < sq < n and int(got["status"].item()) == 0 and int(want["status"].item()) == 0
        assert torch.equal(got["meta"][:8], want["meta"][:8])
        assert torch.equal(got["q_idx"][:sq], want["q_idx"][:sq])
        assert torch.equal(got["pos_ids"][:sq], want["pos_ids"][:sq])
        assert torch.equal(got["cu_q"], want["cu_q"])
        assert torch.equal(got["tile_off"], want["tile_off"])
        assert torch.equal(got["gate_sum"], want["gate_sum"])


def test_static_variant_refuses_inputs_beyond_its_fixed_scratch(lib_path):
    """Rejected on the host, before any CUDA call: runs without a GPU."""
    from logo_b200 import _lib

    lib = _lib.load()
    limit = 1 << 20
    rc = lib.logo_select_rows_static(None, 3, None, 1, None, 1, limit + 1, None, None, None, None, None, None, None,
                                     None)
    assert rc == 3
    msg = _lib.last_error()
    assert "at most" in msg and str(limit) in msg
