"""Seeded inputs shared by ``make_golden.py`` (which feeds them to the reference) and by the
tests (which feed them to the oracle and to the CUDA kernels). Only ``numpy.random.RandomState``
is used, so the streams do not depend on the torch version."""
from __future__ import annotations

import numpy as np


def _cu(lens):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + int(n))
    return cu


# ----------------------------------------------------------------------------------------------
# selection masks
# ----------------------------------------------------------------------------------------------
def selection_cases():
    """name -> (bool mask [N], cu_seqlens list)."""
    cases = {}
    rs = np.random.RandomState(1)
    cases["single_half"] = (rs.uniform(size=512) < 0.5, _cu([512]))
    cases["varlen_empty_seq"] = (rs.uniform(size=200) < 0.4, [0, 70, 70, 200])
    cases["all_selected"] = (np.ones(300, dtype=bool), _cu([100, 200]))
    cases["none_selected"] = (np.zeros(260, dtype=bool), _cu([130, 130]))
    lens = [1, 513, 0, 127, 128, 129, 2048, 3]
    cases["ragged"] = (rs.uniform(size=sum(lens)) < 0.25, _cu(lens))
    m = np.zeros(1000, dtype=bool)
    m[[0, 499, 500, 999]] = True
    cases["seq_ends_only"] = (m, _cu([500, 500]))
    cases["many_blocks"] = (rs.uniform(size=9000) < 0.125, _cu([4096, 4904]))
    return cases


# ----------------------------------------------------------------------------------------------
# sq_full_attn cases (reference Triton kernels under the interpreter)
# ----------------------------------------------------------------------------------------------
ATTN_CASES = {
    #  name: (lens, HQ, H, D, selection ratio, seed)
    "d32_gqa_empty_seq": ([70, 0, 130], 4, 2, 32, 0.5, 11),
    "d128_two_seq": ([170, 130], 2, 1, 128, 0.5, 12),
    "d128_all_rows": ([260], 2, 2, 128, 1.0, 13),
    "d128_sparse": ([384], 1, 1, 128, 0.125, 14),
}


def attn_case_inputs(name):
    lens, hq, h, d, ratio, seed = ATTN_CASES[name]
    rs = np.random.RandomState(seed)
    n = sum(lens)
    q = rs.standard_normal((n, hq, d)).astype(np.float32)
    k = rs.standard_normal((n, h, d)).astype(np.float32)
    v = rs.standard_normal((n, h, d)).astype(np.float32)
    do = rs.standard_normal((n, hq, d)).astype(np.float32)
    sel = (rs.uniform(size=n) < ratio) if ratio < 1.0 else np.ones(n, dtype=bool)
    return q, k, v, do, sel, _cu(lens)


# ----------------------------------------------------------------------------------------------
# layer cases
# ----------------------------------------------------------------------------------------------
LAYER_CASES = {
    # the configuration quoted as the CPU-runnable case: B=1, T=512, hidden 2048, 16 x 128, window 128
    "config1": dict(hidden=2048, heads=16, kv_heads=16, window=128, gate_thres=0.5, backend="triton",
                    batch=1, seqlen=512, lens=None, seed=100, subsample=61),
    "small_varlen": dict(hidden=256, heads=2, kv_heads=2, window=128, gate_thres=0.5, backend="triton",
                         batch=1, seqlen=420, lens=[100, 0, 320], seed=101),
    "small_batch": dict(hidden=256, heads=2, kv_heads=1, window=128, gate_thres=0.5, backend="flash",
                        batch=2, seqlen=200, lens=None, seed=102),
    # global_qk_param='scale_offset' (logo/layers/logo.py:44-51,80-84), GQA, an empty sequence
    "scale_offset_varlen": dict(hidden=256, heads=2, kv_heads=1, window=128, gate_thres=0.5, backend="triton",
                                batch=1, seqlen=450, lens=[180, 0, 270], seed=103, param="scale_offset"),
}

# the dense causal layer used for attn_type_list != 0 (logo/layers/attn.py:22-121)
DENSE_ATTN_CASE = dict(hidden=512, heads=4, kv_heads=2, batch=2, seqlen=300, seed=104)


def dense_attn_weights(case=DENSE_ATTN_CASE):
    rs = np.random.RandomState(case["seed"])
    hid, nh, nkv = case["hidden"], case["heads"], case["kv_heads"]
    d = hid // nh
    return {"q_proj.weight": (0.05 * rs.standard_normal((nh * d, hid))).astype(np.float32),
            "k_proj.weight": (0.05 * rs.standard_normal((nkv * d, hid))).astype(np.float32),
            "v_proj.weight": (0.05 * rs.standard_normal((nkv * d, hid))).astype(np.float32),
            "o_proj.weight": (0.05 * rs.standard_normal((hid, hid))).astype(np.float32)}


def dense_attn_inputs(case=DENSE_ATTN_CASE):
    rs = np.random.RandomState(case["seed"] + 1000)
    b, t = case["batch"], case["seqlen"]
    hidden = rs.standard_normal((b, t, case["hidden"])).astype(np.float32)
    pos = np.broadcast_to(np.arange(t, dtype=np.int64)[None], (b, t)).copy()
    return hidden, pos


def layer_weights(case):
    """Reference parameter name -> fp32 array. Linear weights N(0, 0.02); the per-head global
    projections are the reference's identity initialisation perturbed by N(0, 0.02)."""
    rs = np.random.RandomState(case["seed"])
    hid, nh, nkv = case["hidden"], case["heads"], case["kv_heads"]
    d = hid // nh
    w = {}
    w["q_proj.weight"] = (0.02 * rs.standard_normal((nh * d, hid))).astype(np.float32)
    w["k_proj.weight"] = (0.02 * rs.standard_normal((nkv * d, hid))).astype(np.float32)
    w["v_proj.weight"] = (0.02 * rs.standard_normal((nkv * d, hid))).astype(np.float32)
    w["o_proj.weight"] = (0.02 * rs.standard_normal((hid, hid))).astype(np.float32)
    w["gate_proj.weight"] = (0.02 * rs.standard_normal((1, hid))).astype(np.float32)
    if case.get("param", "linear_proj") == "scale_offset":
        for name, heads in (("q", nh), ("k", nkv), ("v", nkv)):
            w[f"{name}_global_scale"] = (1 + 0.1 * rs.standard_normal(heads * d)).astype(np.float32)
            w[f"{name}_global_offset"] = (0.1 * rs.standard_normal(heads * d)).astype(np.float32)
    else:
        eye = np.eye(d, dtype=np.float32)
        w["q_global_proj"] = (eye[None] + 0.02 * rs.standard_normal((nh, d, d))).astype(np.float32)
        w["k_global_proj"] = (eye[None] + 0.02 * rs.standard_normal((nkv, d, d))).astype(np.float32)
        w["v_global_proj"] = (eye[None] + 0.02 * rs.standard_normal((nkv, d, d))).astype(np.float32)
    w["context_norm_local.weight"] = (1 + 0.1 * rs.standard_normal(d)).astype(np.float32)
    w["context_norm_global.weight"] = (1 + 0.1 * rs.standard_normal(d)).astype(np.float32)
    return w


def layer_case_inputs(case):
    """(hidden [B,T,hidden] fp32, cu_seqlens list or None, position_ids [B,T] int64)."""
    rs = np.random.RandomState(case["seed"] + 1000)
    b, t = case["batch"], case["seqlen"]
    hidden = rs.standard_normal((b, t, case["hidden"])).astype(np.float32)
    if case["lens"] is not None:
        cu = _cu(case["lens"])
        pos = np.concatenate([np.arange(n) for n in case["lens"]]).astype(np.int64)[None]
    else:
        cu = None
        pos = np.broadcast_to(np.arange(t, dtype=np.int64)[None], (b, t)).copy()
    return hidden, cu, pos


# ----------------------------------------------------------------------------------------------
# rotary embedding (bf16 eager graph of logo/modules/rotary.py:81-106)
# ----------------------------------------------------------------------------------------------
def rope_case():
    """x [N, H, D], output gradient g [N, H, D], positions [N] (fp32 arrays; the users round to bf16)."""
    rs = np.random.RandomState(11)
    n, h, d = 96, 3, 128
    x = rs.standard_normal((n, h, d)).astype(np.float32)
    g = rs.standard_normal((n, h, d)).astype(np.float32)
    pos = rs.randint(0, 8192, size=n).astype(np.int64)
    return x, g, pos


# ----------------------------------------------------------------------------------------------
# model-level drop-in: a tiny LoGoForCausalLM (one LoGo layer, one dense layer)
# ----------------------------------------------------------------------------------------------
MODEL_CASE = dict(vocab_size=128, hidden_size=256, intermediate_size=256, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=2, max_position_embeddings=1024, rms_norm_eps=1e-5, attn_type_list=[0, 1],
                  window_size=128, global_qk_param="linear_proj", sparse_full_attn_backend="flash",
                  gate_thres_init=0.5, tie_word_embeddings=False, seed=105)


def model_weights(shapes, seed=MODEL_CASE["seed"]):
    """Parameter / persistent-buffer name -> fp32 array for the tiny model, drawn in sorted name order.
    ``shapes``: name -> shape, as ``{k: tuple(v.shape) for k, v in model.state_dict().items()}`` gives it."""
    rs = np.random.RandomState(seed)
    w = {}
    for name in sorted(shapes):
        shape = tuple(shapes[name])
        if name.endswith("gate_thres"):
            w[name] = np.full(shape, 0.5, dtype=np.float32)
        elif name.endswith("_global_proj"):
            w[name] = (np.eye(shape[-1], dtype=np.float32)[None] + 0.02 * rs.standard_normal(shape)).astype(np.float32)
        elif "norm" in name:
            w[name] = (1 + 0.1 * rs.standard_normal(shape)).astype(np.float32)
        elif "embed_tokens" in name:
            w[name] = (0.5 * rs.standard_normal(shape)).astype(np.float32)
        else:
            w[name] = (0.05 * rs.standard_normal(shape)).astype(np.float32)
    return w


def model_inputs():
    """(packed ids [1, 200], cu_seqlens, batch ids [2, 154]) for the packed forward and the prefill + decode loop."""
    rs = np.random.RandomState(MODEL_CASE["seed"] + 1)
    packed = rs.randint(0, MODEL_CASE["vocab_size"], size=(1, 200)).astype(np.int64)
    batch = rs.randint(0, MODEL_CASE["vocab_size"], size=(2, 154)).astype(np.int64)
    return packed, [0, 90, 90, 200], batch
