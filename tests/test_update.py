"""update_gate_thres: same results as the reference (golden) on one process, and the counters are
summed across ranks (2 gloo ranks on CPU) before the sign step."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from logo_b200.update import update_gate_thres


class FakeLayer(torch.nn.Module):
    def __init__(self, thres, g, t, dtype=torch.float32):
        super().__init__()
        self.register_buffer("gate_thres", torch.tensor([thres], dtype=dtype))
        self.register_buffer("gate_avg", torch.tensor([3.0], dtype=dtype))
        self.register_buffer("global_token_count", torch.tensor([g], dtype=dtype))
        self.register_buffer("total_token_count", torch.tensor([t], dtype=dtype))


def test_single_process_matches_reference(golden):
    g = golden["misc"]
    model = torch.nn.ModuleList([FakeLayer(0.5, 30.0, 100.0), FakeLayer(0.4, 70.0, 100.0), FakeLayer(0.3, 0.0, 0.0),
                                 FakeLayer(0.2, 50.0, 100.0)])
    ratio = update_gate_thres(model, target_global_ratio=0.5, update_rate=0.01)
    np.testing.assert_array_equal(ratio.numpy(), g["update/ratio"])
    np.testing.assert_array_equal(np.array([m.gate_thres.item() for m in model], dtype=np.float32), g["update/thres"])
    for m in model:
        assert m.gate_avg.item() == 0 and m.global_token_count.item() == 0 and m.total_token_count.item() == 0


def test_argument_checks_and_empty_model():
    with pytest.raises(ValueError):
        update_gate_thres(torch.nn.Linear(2, 2), target_global_ratio=1.5)
    with pytest.raises(ValueError):
        update_gate_thres(torch.nn.Linear(2, 2), update_rate=-1.0)
    assert update_gate_thres(torch.nn.Linear(2, 2)) is None


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # rank 0 alone would raise the threshold of layer 0 (ratio 0.8), rank 1 alone would lower it (0.1);
    # summed: 90 / 200 = 0.45 < 0.5 -> lowered on both ranks
    counts = [(80.0, 100.0), (10.0, 100.0)][rank]
    model = torch.nn.ModuleList([FakeLayer(0.5, *counts), FakeLayer(0.5, 0.0, 0.0)])
    ratio = update_gate_thres(model, target_global_ratio=0.5, update_rate=0.01)
    out[rank] = (ratio.reshape(-1).tolist(), [m.gate_thres.item() for m in model])
    dist.destroy_process_group()


def test_counters_are_summed_over_two_gloo_ranks():
    port = _free_port()
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_rank_main, args=(2, port, out), nprocs=2, join=True)
        for rank in (0, 1):
            ratio, thres = out[rank]
            assert ratio[0] == pytest.approx(0.45) and ratio[1] == 0.0
            assert thres[0] == pytest.approx(0.49) and thres[1] == pytest.approx(0.5)
