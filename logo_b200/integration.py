"""Runtime form of the layer-level integration: points an importable reference package at this one.

``logo/modeling_logo.py:29-35`` binds ``Cache``, ``Attention`` and ``LoGoAttention`` at import
time and ``LoGoDecoderLayer.__init__`` (``modeling_logo.py:48-51``) instantiates them. Replacing
those three module attributes (and the controller) is the same edit as changing the import lines,
without touching the reference's files: every ``LoGoForCausalLM`` built afterwards runs its
attention layers, cache and budget controller from this package, and a reference ``state_dict``
loads unchanged because parameter and buffer names are the same.
"""
from __future__ import annotations

__all__ = ["patch_reference"]


def patch_reference(logo_module=None):
    """Re-binds the reference package's attention layer, dense layer, cache and controller.

    ``logo_module``: the imported reference package (default: ``import logo``). Also registers the
    ``"default"`` rotary initialiser that transformers >= 5 no longer ships and the reference's
    ``RotaryEmbedding`` looks up (``logo/modules/rotary.py:34``). Returns the patched package.
    """
    import torch

    if logo_module is None:
        import logo as logo_module                      # noqa: PLC0415 - the reference must be importable
    try:
        from transformers import modeling_rope_utils as mru

        def default_rope(config, device=None, seq_len=None, **kw):
            dim = config.hidden_size // config.num_attention_heads
            inv = 1.0 / (config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.int64).float().to(device) / dim))
            return inv, 1.0

        mru.ROPE_INIT_FUNCTIONS.setdefault("default", default_rope)
    except ImportError:
        pass

    from . import Attention, Cache, LoGoAttention, update_gate_thres

    import importlib

    modeling = importlib.import_module(logo_module.__name__ + ".modeling_logo")
    modeling.LoGoAttention = LoGoAttention
    modeling.Attention = Attention
    modeling.Cache = Cache
    logo_module.update_gate_thres = update_gate_thres
    logo_module.Cache = Cache
    return logo_module
