"""Weight residency planning and the rotating arena (CPU: copies are synchronous, the mapping logic is the same)."""
import pytest
import torch

from ninfer_fusion_b200.models.config import TINY_DENSE
from ninfer_fusion_b200.models.weights import random_weights
from ninfer_fusion_b200.runtime.weight_offload import OffloadedWeights, plan_residency


def test_plan_residency_budgets():
    w = random_weights(TINY_DENSE, "cpu", seed=0)
    everything = sum(t.numel() * t.element_size() for t in w.values())
    full = plan_residency(w, everything)
    assert full.offloaded_layers == [] and full.arena_bytes == 0 and full.device_bytes == everything
    biggest = max(full.layer_bytes.values())
    budget = full.fixed_bytes + 2 * biggest + full.layer_bytes[0]   # a 2-slot arena and exactly the first layer
    tight = plan_residency(w, budget)
    assert tight.resident_layers == [0] and tight.offloaded_layers == [1, 2, 3]
    assert tight.device_bytes <= budget and tight.host_bytes == sum(tight.layer_bytes[l] for l in (1, 2, 3))
    assert plan_residency(w, full.fixed_bytes + 2 * biggest).resident_layers == []
    with pytest.raises(MemoryError):
        plan_residency(w, full.fixed_bytes + biggest)


def test_offloaded_weights_serve_the_same_tensors():
    w = random_weights(TINY_DENSE, "cpu", seed=1)
    plan = plan_residency(w, 1 << 40)
    biggest = max(plan.layer_bytes.values())
    ow = OffloadedWeights(w, "cpu", plan.fixed_bytes + 2 * biggest + plan.layer_bytes[0])
    assert ow.plan.offloaded_layers == [1, 2, 3]
    for step in range(2):
        for layer in range(TINY_DENSE.n_layers):
            ow.note_layer(layer)
            for name, t in w.items():
                if name.startswith(f"text/layers/{layer}/"):
                    assert torch.equal(ow[name], t), name
    assert "text/embed" in ow and "text/layers/2/mlp/down" in ow and "nope" not in ow
    assert ow.get("text/layers/9/input_norm", None) is None
    assert torch.equal(ow["text/layers/3/input_norm"], w["text/layers/3/input_norm"])   # vectors stay resident
    assert ow.fetches >= 6          # three offloaded layers rotate through two slots, every step
    assert set(ow.keys()) == set(w)


def test_values_do_not_fetch():
    w = random_weights(TINY_DENSE, "cpu", seed=1)
    plan = plan_residency(w, 1 << 40)
    ow = OffloadedWeights(w, "cpu", plan.fixed_bytes + 2 * max(plan.layer_bytes.values()) + plan.layer_bytes[0])
    before = ow.fetches
    vals = list(ow.values())
    assert len(vals) == len(w) and ow.fetches == before
    assert all(isinstance(v, torch.Tensor) for v in vals)
