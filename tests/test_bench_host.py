"""Host-side logic of bench.py that does not need a GPU: the sequence -> rank plan of the sharded
layer workload."""
import importlib.util
import pathlib

_spec = importlib.util.spec_from_file_location("bench", pathlib.Path(__file__).resolve().parents[1] / "bench.py")
bench = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(bench)


def test_lpt_partition_covers_every_sequence_once():
    lens = [8192, 7000, 5000, 4096, 3000, 2500, 1500, 980]
    for world in (1, 2, 4, 8):
        plan = bench.lpt_partition(lens, world, 0.25)
        assert len(plan) == world
        assert sorted(i for p in plan for i in p) == list(range(len(lens)))


def test_lpt_partition_balances_cost():
    lens = [8192, 7000, 5000, 4096, 3000, 2500, 1500, 980]
    cost = lambda l: 0.25 * l * l / 2 + 129 * l
    for world in (2, 4):
        plan = bench.lpt_partition(lens, world, 0.25)
        loads = [sum(cost(lens[i]) for i in p) for p in plan]
        # longest-processing-time-first is within 4/3 of the optimum, which is at least the mean load
        # and at least the heaviest single sequence
        assert max(loads) <= 4 / 3 * max(sum(loads) / world, cost(max(lens))) * 1.0001
    # deterministic: every rank computes the same plan
    assert bench.lpt_partition(lens, 4, 0.25) == bench.lpt_partition(lens, 4, 0.25)
