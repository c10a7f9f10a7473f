"""Training-time controller of the global-attention budget.

This is host logic whose contract is its body: it is the reference's function
(``logo/update.py:17-75``) restated, not a new design. Same entry point and behaviour: layers are found by
their four buffers (``gate_thres``, ``gate_avg``, ``global_token_count``,
``total_token_count``), the observed global ratio moves each threshold by a signed step, and
the counters are cleared. The two all-reduces of ``update.py:52-54`` are issued as one
all-reduce over a stacked ``[2, L, 1]`` tensor.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
import torch.distributed as dist

__all__ = ["update_gate_thres"]

GATE_THRES_UPDATE_RATE = float(os.getenv("GATE_THRES_UPDATE_RATE", "0.0005"))
TARGET_GLOBAL_RATIO = float(os.getenv("TARGET_GLOBAL_RATIO", "0.5"))

_BUFFERS = ("gate_thres", "gate_avg", "global_token_count", "total_token_count")


def update_gate_thres(
    model,
    target_global_ratio: float = TARGET_GLOBAL_RATIO,
    update_rate: float = GATE_THRES_UPDATE_RATE,
    process_group=None,
) -> Optional[torch.Tensor]:
    """Update gate thresholds from the accumulated global-token ratios; returns the ratios ``[L, 1]``."""
    if not 0.0 <= target_global_ratio <= 1.0:
        raise ValueError(f"`target_global_ratio` must be in [0, 1], got {target_global_ratio}")
    if update_rate < 0.0:
        raise ValueError(f"`update_rate` must be non-negative, got {update_rate}")

    layers = [m for m in model.modules() if all(hasattr(m, name) for name in _BUFFERS)]
    if not layers:
        return None

    with torch.no_grad():
        gate_thres = torch.stack([m.gate_thres for m in layers], dim=0)
        counts = torch.stack(
            [torch.stack([m.global_token_count for m in layers], dim=0),
             torch.stack([m.total_token_count for m in layers], dim=0)], dim=0)   # [2, L, 1]
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(counts, op=dist.ReduceOp.SUM, group=process_group)
        global_token_count, total_token_count = counts[0], counts[1]

        has_observations = total_token_count > 0
        global_token_ratio = torch.where(
            has_observations,
            global_token_count / total_token_count.clamp_min(1),
            torch.zeros_like(global_token_count),
        )
        update = update_rate * torch.sign(global_token_ratio - target_global_ratio)
        gate_thres.add_(torch.where(has_observations, update, torch.zeros_like(update)).to(gate_thres.dtype))

        for m, new_thres in zip(layers, gate_thres):
            m.gate_thres.copy_(new_thres)
            m.gate_avg.zero_()
            m.global_token_count.zero_()
            m.total_token_count.zero_()

    return global_token_ratio
