"""Mapuvik on the CPU: configuration, model description, checkpoint rules, the plain
implementation's own consistency, and the host bookkeeping of a model that caches nothing."""

from __future__ import annotations

import copy

import pytest
import torch

import plain_mapuvik as plain
from mapuvik_cases import LOUD, TINY_A, TINY_B, TINY_STATE_ONLY
from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.cache.storage import plan_cache
from ayaka_b200.config.mapuvik import MapuvikConfig
from ayaka_b200.engine.scheduler import Scheduler
from ayaka_b200.errors import AyakaError, ModelLoadError
from ayaka_b200.kernels import ops
from ayaka_b200.models import build_model
from ayaka_b200.models.registry import architecture_of
from ayaka_b200.sampling.params import SamplingParams
from ayaka_b200.weights.loader import TensorSource, load_into
from ayaka_b200.weights.random_init import random_state


def test_the_configuration_reads_back_as_written():
    for raw in (TINY_A, TINY_B, TINY_STATE_ONLY):
        config = MapuvikConfig.from_json_dict(raw)
        assert MapuvikConfig.from_json_dict(config.to_json_dict()) == config
        assert [layer.kind for layer in config.layers] == [e["type"] for e in raw["layers"]]
    config = MapuvikConfig.from_json_dict(TINY_A)
    assert [layer.weights_of for layer in config.layers] == [0, 1, 2, 0, 1]
    assert config.layers[1].ff is None and config.layers[0].get("mask.size") == 20


@pytest.mark.parametrize("change, text", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "rot.base"),
    (lambda c: c["layers"][1].update(type="s4"), "not a mixer"),
    (lambda c: c["layers"][2]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c["layers"][3].update(weights_of=4), "earlier"),
    (lambda c: c["layers"][3].update(mixer={**c["layers"][3]["mixer"], "heads": 5}),
     "another layer"),
    (lambda c: c["layers"][1]["mixer"].update(state=0), "at least 1"),
])
def test_a_configuration_that_lacks_or_twists_something_is_refused(change, text):
    raw = copy.deepcopy(TINY_A)
    change(raw)
    with pytest.raises(AyakaError, match=text):
        MapuvikConfig.from_json_dict(raw)


def test_layers_that_borrow_tensors_run_the_owner_again_with_their_own_cache():
    model, architecture, config = build_model(TINY_A, "float32", "cpu")
    spec = model.spec
    assert len(spec.layers) == 3 and [run.layer for run in spec.order] == [0, 1, 2, 0, 1]
    plan = plan_cache(spec.order, model.needs())
    assert len(plan.groups) == 1 and plan.groups[0].values is False
    assert plan.groups[0].head_dim == 32 + 8 and plan.groups[0].window == 20
    assert plan.slots_per_group == (2,) and plan.run_writes == (True, False, False, True, False)
    assert [state is not None for state in plan.run_state] == [False, True, True, False, True]
    assert spec.max_positions >= 1 << 30  # the design has no longest sequence of its own


def test_random_tensors_fill_the_model_exactly(tmp_path):
    for raw in (TINY_A, TINY_B, TINY_STATE_ONLY):
        model, architecture, config = build_model(raw, "float32", "cpu")
        state = random_state(raw, 3, LOUD)
        load_into(model, architecture.weight_rules(config), TensorSource(tensors=state))
        params = dict(model.named_params())
        # stacked parameters hold the stored tensors one under the other
        if raw is TINY_A:
            fused = params["layers.0.mixer.proj.weight"].tensor
            q, dkv, g = state["l0.mix.q"], state["l0.mix.dkv"], state["l0.mix.g"]
            assert torch.equal(fused, torch.cat([q, dkv, g]))
            gates = params["layers.2.mixer.gate_bias"].tensor
            assert torch.equal(gates, torch.cat([state["l2.mix.i.b"], state["l2.mix.f.b"]]))
            assert params["layers.1.mixer.conv.weight"].tensor.dtype == torch.float32
        del state["head"]
        with pytest.raises(ModelLoadError, match="missing"):
            load_into(model, architecture.weight_rules(config), TensorSource(tensors=state))
    assert architecture_of({"architecture": "Mapuvik"}).name == "Mapuvik"


def test_the_plain_recurrences_do_not_depend_on_where_a_sequence_is_cut():
    """The oracle itself: a state-space layer and a matrix memory run over a whole sequence
    give, at every position, what they give over any prefix (causality), and the attention
    window drops exactly the keys it should."""
    state = plain.cast_state(random_state(TINY_B, 5, LOUD), torch.float64)
    tokens = torch.randint(0, TINY_B["vocab"], (40,), generator=torch.Generator().manual_seed(1))
    whole = plain.logits(state, TINY_B, tokens)
    for cut in (1, 2, 8, 23):
        assert torch.allclose(plain.logits(state, TINY_B, tokens[:cut]), whole[:cut],
                              rtol=1e-10, atol=1e-10)
    # window 7: the key eight back must not matter, the key seven back must
    h = torch.randn(12, 96, dtype=torch.float64, generator=torch.Generator().manual_seed(2))
    weights = plain.sub(state, "l1.mix.")
    mixer = TINY_B["layers"][1]["mixer"]
    base = plain.latent_attention(h, weights, mixer, 1e-6)
    moved = h.clone()
    moved[11 - 7] += 1.0
    assert torch.equal(plain.latent_attention(moved, weights, mixer, 1e-6)[11], base[11])
    moved = h.clone()
    moved[11 - 6] += 1.0
    assert not torch.allclose(plain.latent_attention(moved, weights, mixer, 1e-6)[11], base[11])


def test_state_sizes_and_a_model_that_holds_no_page():
    assert ops.scan_state_floats("mamba2", heads=3, inner=4, columns=8, taps=3,
                                 channels=3 * 8 + 2 * 3 * 4) == 2 * 48 + 96
    tiles = -(-24 // ops.SCAN_COLUMNS)
    assert ops.scan_state_floats("mlstm", heads=1, inner=8, columns=24) == 192 + tiles * 9
    model, _, _ = build_model(TINY_STATE_ONLY, "float32", "cpu")
    plan = plan_cache(model.spec.order, model.needs())
    assert plan.groups == () and all(state is not None for state in plan.run_state)
    # the scheduler and the manager work with no group at all: rows and lengths only
    manager = CacheManager([], [], 16, 2, 8)
    scheduler = Scheduler(manager, max_running=2, max_tokens_per_step=32, max_waiting=8,
                          max_positions=manager.max_tokens_per_request)
    for name in ("a", "b", "c"):
        scheduler.add_request(name, tuple(range(1, 41)), SamplingParams(max_tokens=4))
    plan_1 = scheduler.schedule()
    assert [len(entry.tokens) for entry in plan_1.entries] == [32]
    scheduler.update(plan_1, {})
    plan_2 = scheduler.schedule()
    assert [len(entry.tokens) for entry in plan_2.entries] == [8, 16]  # cut at a page
    manager.check_integrity()
