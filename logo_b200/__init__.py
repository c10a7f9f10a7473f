"""logo_b200: the LoGo attention hot path on B200 (sm_100a).

Public surface, mirroring the reference package ``logo``:

* ``logo_b200.ops``      -- ``sq_full_attn``, ``build_selection``, ``SelInfo`` ... (``logo.ops``)
* ``LoGoAttention``      -- the attention layer (``logo.layers.LoGoAttention``)
* ``Attention``          -- the dense causal layer for non-LoGo layers (``logo.layers.attn.Attention``)
* ``Cache``              -- the dual-state KV cache (``logo.cache.Cache``)
* ``update_gate_thres``  -- the budget controller (``logo.update.update_gate_thres``)

All compute runs in ``liblogo_b200.so`` (build it with ``python -m logo_b200.build``); there is
no Triton, flash-attn or CPU path.
"""
from . import ops
from .cache import Cache
from .layers import Attention, LoGoAttention, check_status
from .ops import SelInfo, build_selection, sq_full_attn
from .ops_bwd import get_backward_mode, set_backward_mode
from .update import update_gate_thres

__all__ = ["ops", "Attention", "Cache", "LoGoAttention", "SelInfo", "build_selection", "check_status",
           "get_backward_mode", "set_backward_mode", "sq_full_attn", "update_gate_thres"]
__version__ = "0.1.0"
