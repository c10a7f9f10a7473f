"""Model level: the reference's own ``LoGoForCausalLM`` with its attention layers, cache and controller
re-bound to this package, against logits the unmodified reference produced on the CPU (fixture
``tests/golden/model.npz``, written by ``tests/golden/make_golden.py model``).

Needs an importable copy of the reference package under ``baseline/_ref`` (installed with
``pip install --target baseline/_ref <reference checkout>``; it is not part of the repository);
without it the test is skipped."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from golden_inputs import MODEL_CASE, model_inputs, model_weights

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parents[1] / "baseline" / "_ref"


@pytest.fixture(scope="module")
def patched_reference():
    if not (REF / "logo" / "modeling_logo.py").exists():
        pytest.skip("no reference package under baseline/_ref")
    sys.path.insert(0, str(REF))
    try:
        from logo_b200.integration import patch_reference

        import logo
        yield patch_reference(logo)
    finally:
        sys.path.remove(str(REF))


def _build(patched_reference, device):
    from logo.configuration_logo import LoGoConfig
    from logo.modeling_logo import LoGoForCausalLM

    import logo_b200

    cfg = LoGoConfig(**{k: v for k, v in MODEL_CASE.items() if k != "seed"})
    model = LoGoForCausalLM(cfg).eval()
    assert type(model.model.layers[0].self_attn) is logo_b200.LoGoAttention
    assert type(model.model.layers[1].self_attn) is logo_b200.Attention
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    missing, unexpected = model.load_state_dict({k: torch.from_numpy(v) for k, v in model_weights(shapes).items()})
    assert not missing and not unexpected
    return model.to(device, torch.bfloat16), shapes


def test_reference_model_runs_on_this_package_and_matches_its_own_cpu_logits(cuda_device, golden, patched_reference):
    import logo_b200

    g = golden["model"]
    model, shapes = _build(patched_reference, cuda_device)
    # the reference's checkpoint layout: every parameter / persistent buffer name is the reference's
    assert sorted(shapes) == [str(x) for x in g["model/param_names"]]
    packed, cu, batch = model_inputs()
    scale = float(g["model/packed_logits"].std())
    with torch.no_grad():
        y = model(input_ids=torch.from_numpy(packed).to(cuda_device),
                  cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=cuda_device), use_cache=False)
        err = np.abs(y.logits[0].float().cpu().numpy() - g["model/packed_logits"])
        print(f"packed logits: max-abs {err.max():.4f}, rms {np.sqrt((err ** 2).mean()):.5f}, logits std {scale:.3f}")
        # a token whose gate lies within bf16 rounding of the threshold may take the other branch: bound
        # the bulk tightly and the worst row loosely
        assert np.sqrt((err ** 2).mean()) < 0.02 * scale
        assert np.quantile(err.max(axis=-1), 0.95) < 0.08 * scale

        ids = torch.from_numpy(batch).to(cuda_device)
        cache = logo_b200.Cache()
        T0, steps = 150, 4
        outs = [model(input_ids=ids[:, :T0], past_key_values=cache, use_cache=True).logits]
        for s in range(steps):
            outs.append(model(input_ids=ids[:, T0 + s: T0 + s + 1], past_key_values=cache, use_cache=True).logits)
        got = torch.cat(outs, dim=1).float().cpu().numpy()
    assert cache.get_seq_length(0) == T0 + steps and len(cache) == MODEL_CASE["num_hidden_layers"]
    err = np.abs(got - g["model/cached_logits"])
    print(f"prefill + {steps} cached steps: max-abs {err.max():.4f}, rms {np.sqrt((err ** 2).mean()):.5f}")
    assert np.sqrt((err ** 2).mean()) < 0.02 * scale
    assert np.quantile(err.max(axis=-1), 0.95) < 0.08 * scale
    logo_b200.check_status(model)
    logo_b200.check_status(cache)


def test_training_step_and_controller_through_the_reference_model(cuda_device, patched_reference):
    """Loss with the reference's packed-boundary label masking, backward through this package's layers,
    then the budget controller finds the layers by their buffers."""
    import logo

    model, _ = _build(patched_reference, cuda_device)
    model.train()
    packed, cu, _ = model_inputs()
    ids = torch.from_numpy(packed).to(cuda_device)
    out = model(input_ids=ids, labels=ids.clone(), cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=cuda_device),
                use_cache=False)
    assert torch.isfinite(out.loss)
    out.loss.backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())
    ratio = logo.update_gate_thres(model, target_global_ratio=0.5, update_rate=0.01)
    assert ratio.shape == (1, 1)       # one LoGo layer (the second layer is the dense one)
    assert 0.0 < float(ratio[0, 0]) < 1.0
    assert float(model.model.layers[0].self_attn.total_token_count) == 0.0
