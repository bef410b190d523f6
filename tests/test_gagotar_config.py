"""Gagotar on the CPU: configuration, rules, the plain model's own edges, the cache
manager's blocks of positions."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_gagotar as plain
from ayaka_b200.cache.manager import CacheManager
from ayaka_b200.config.gagotar import GagotarConfig
from ayaka_b200.errors import AyakaError
from ayaka_b200.kernels import ops
from ayaka_b200.models import build_model
from ayaka_b200.models.gagotar import gagotar_model_spec, gagotar_weight_rules
from ayaka_b200.parts.base import CacheNeed
from ayaka_b200.weights.random_init import random_state
from gagotar_cases import LOUD, TINY_A, TINY_B, TINY_C, TINY_D


@pytest.mark.parametrize("config", [TINY_A, TINY_B, TINY_C, TINY_D])
def test_configuration_round_trip(config):
    parsed = GagotarConfig.from_json_dict(config)
    again = GagotarConfig.from_json_dict(parsed.to_json_dict())
    assert parsed == again
    assert len(parsed.layers) == len(config["layers"])
    first = parsed.layers[0]
    assert first.left.chunk == config["layers"][0]["mixer"]["left"]["mask"]["size"]
    assert first.right.rank == config["layers"][0]["mixer"]["right"]["rank"]


def _broken(path: list, value=None, delete=False) -> dict:
    config = copy.deepcopy(TINY_A)
    at = config
    for key in path[:-1]:
        at = at[key]
    if delete:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return config


@pytest.mark.parametrize("config", [
    _broken(["vocab"], delete=True),
    _broken(["norm"], {}),
    _broken(["layers", 0, "type"], "serial"),
    _broken(["layers", 0, "mixer", "left", "kv_heads"], 3),
    _broken(["layers", 0, "mixer", "left", "rot", "dims"], 7),
    _broken(["layers", 0, "mixer", "left", "rot", "dims"], 18),
    _broken(["layers", 0, "mixer", "left", "mask"], delete=True),
    _broken(["layers", 0, "mixer", "right", "tau"], 0.0),
    _broken(["layers", 0, "mixer", "right"], delete=True),
    _broken(["layers", 0, "mlp", "router", "top"], 6),
    _broken(["layers", 0, "mlp", "kind"], "dense"),
    _broken(["layers", 0, "mlp", "expert", "limit"], delete=True),
])
def test_refusals(config):
    with pytest.raises(AyakaError):
        GagotarConfig.from_json_dict(config)


def test_the_decay_rank_comes_from_the_stored_tensor_when_no_key_gives_it():
    config = copy.deepcopy(TINY_A)
    for entry in config["layers"]:
        del entry["mixer"]["right"]["rank"]
    assert GagotarConfig.from_json_dict(config).layers[0].right.rank is None
    with pytest.raises(AyakaError):  # nothing says the rank
        build_model(config, "float32", "cpu")
    shapes = {name: tuple(t.shape) for name, t in random_state(TINY_A, 1, LOUD).items()}
    model, _, completed = build_model(config, "float32", "cpu", shapes.get)
    assert [layer.right.rank for layer in completed.layers] == [5, 3, 5]
    assert model.blocks[1].mixer.sides[1].decay_rank == 3


@pytest.mark.parametrize("config", [TINY_A, TINY_B, TINY_C, TINY_D])
def test_every_stored_tensor_has_a_rule_and_every_parameter_is_covered(config):
    from ayaka_b200.weights.loader import TensorSource, load_into

    state = random_state(config, 3, LOUD)
    model, architecture, parsed = build_model(config, "float32", "cpu")
    load_into(model, architecture.weight_rules(parsed), TensorSource(tensors=state))
    params = dict(model.named_params())
    # stacked: an expert's gate rows, then its up rows, expert after expert
    mlp = config["layers"][0]["mlp"]
    ff = mlp["expert"]["ff"]
    stacked = params["layers.0.feed_forward.in.weight"].tensor
    last = mlp["router"]["experts"] - 1
    assert torch.equal(stacked[last * 2 * ff:last * 2 * ff + ff], state[f"l0.mlp.e{last}.gate"])
    assert torch.equal(stacked[last * 2 * ff + ff:(last + 1) * 2 * ff], state[f"l0.mlp.e{last}.up"])
    left = config["layers"][0]["mixer"]["left"]
    proj = params["layers.0.mixer.left.proj.weight"].tensor
    q, k = left["heads"] * left["dim"], left["kv_heads"] * left["dim"]
    assert torch.equal(proj[q:q + k], state["l0.mix.left.k"])
    assert torch.equal(proj[-left["heads"]:], state["l0.mix.left.g"])
    assert torch.equal(params["layers.0.mixer_scale"].tensor, state["l0.ls1"])
    # a layer without feed-forward has neither a second norm nor a second scale
    if config is TINY_A:
        assert "layers.1.feed_forward_norm.weight" not in params
        assert "layers.1.feed_forward_scale" not in params
        rules = gagotar_weight_rules(parsed)
        assert rules.ignored("l1.norm2") and rules.ignored("l1.ls2")


def test_needs_of_a_layer():
    parsed = GagotarConfig.from_json_dict(TINY_A)
    model, _, _ = build_model(TINY_A, "float32", "cpu")
    need, state = model.needs()[0]
    assert need == CacheNeed(2, 16, 0, chunk=20, value_dim=24)
    assert state.shape == (3 * 8 * 12,)
    spec = gagotar_model_spec(parsed)
    assert spec.layers[0].layer_scale and spec.layers[1].feed_forward.kind == "none"


def test_rescaled_frequencies():
    """All three ranges of the rescaling occur, and the kernel's table equals the plain one."""
    scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 40}
    plain_f = plain.scaled_frequencies(16, 300.0, scaling)
    raw = [300.0 ** (-2.0 * i / 16) for i in range(8)]
    kinds = set()
    for f, r in zip(plain_f, raw):
        wavelength = 2 * math.pi / r
        if wavelength < 10:
            assert f == r
            kinds.add("kept")
        elif wavelength > 40:
            assert f == r / 4
            kinds.add("slowed")
        else:
            assert r / 4 < f < r
            kinds.add("between")
    assert kinds == {"kept", "slowed", "between"}
    table = ops.rope_frequencies(16, 300.0, torch.device("cpu"), (4.0, 1.0, 4.0, 40))
    assert table.tolist() == pytest.approx(plain_f, rel=1e-15)
    assert ops.rope_frequencies(16, 300.0, torch.device("cpu")).tolist() == \
        pytest.approx(raw, rel=1e-15)


def test_the_plain_model_sees_its_own_block_only():
    """Changing a token changes later logits inside its block through attention; the plain
    attention alone never looks across a block's border."""
    torch.manual_seed(0)
    T, H, G, dim, vdim, size = 23, 4, 2, 6, 5, 7
    q, k = torch.randn(T, H, dim, dtype=torch.float64), torch.randn(T, G, dim, dtype=torch.float64)
    v = torch.randn(T, G, vdim, dtype=torch.float64)
    talk, temp = torch.randn(H, H, dtype=torch.float64), torch.rand(H, dtype=torch.float64) + 0.5
    base = plain.mixed_head_attention(q, k, v, talk, temp, 0.4, size)
    k2, v2 = k.clone(), v.clone()
    k2[6] += 3.0
    v2[6] -= 2.0
    moved = plain.mixed_head_attention(q, k2, v2, talk, temp, 0.4, size)
    changed = (moved - base).abs().amax(dim=(1, 2)) > 1e-12
    assert changed.tolist() == [t == 6 for t in range(T)]  # 6 is the last of its block
    k2, v2 = k.clone(), v.clone()
    k2[7] += 3.0
    moved = plain.mixed_head_attention(q, k2, v2, talk, temp, 0.4, size)
    changed = (moved - base).abs().amax(dim=(1, 2)) > 1e-12
    # (position 7 opens its block: its only key is its own, whose weight is one whatever it is)
    assert changed.tolist() == [8 <= t < 14 for t in range(T)]
    # mixing is not a relabelling: with an identity matrix and unit factors it is plain attention
    plain_att = plain.mixed_head_attention(q, k, v, torch.eye(H, dtype=torch.float64),
                                           torch.ones(H, dtype=torch.float64), 0.4, size)
    assert (plain_att - base).abs().max() > 1e-3


def test_the_plain_memory_carries_its_state():
    torch.manual_seed(1)
    T, H, dim, vdim = 19, 2, 5, 3
    q, k, z = (torch.randn(T, H, dim, dtype=torch.float64) for _ in range(3))
    v = torch.randn(T, H, vdim, dtype=torch.float64)
    whole, last = plain.decayed_memory(q, k, v, z, 3.0)
    head, state = plain.decayed_memory(q[:8], k[:8], v[:8], z[:8], 3.0)
    tail, last2 = plain.decayed_memory(q[8:], k[8:], v[8:], z[8:], 3.0, state)
    assert torch.allclose(torch.cat([head, tail]), whole, atol=1e-13)
    assert torch.allclose(last, last2, atol=1e-13)


def test_the_cache_manager_gives_back_the_pages_of_blocks_that_are_over():
    need = CacheNeed(2, 16, 0, chunk=20, value_dim=24)
    manager = CacheManager([need], [12], 8, 2, 64)
    assert manager.allocate("a", 19) and manager.num_free_pages() == 11 - 3
    manager.commit("a", 19)
    manager.check_integrity()
    assert manager.num_free_pages() == 8  # position 19 still sees 0 .. 19
    assert manager.allocate("a", 1)
    manager.commit("a", 1)  # the next row is position 20: block 20 .. 39, pages from 2 on
    manager.check_integrity()
    assert manager.num_free_pages() == 10
    assert manager.tables[0][manager.row("a"), :3].tolist() == [0, 0, 3]
    # a long portion needs every page it passes through, and returns them when it is done
    assert manager.allocate("a", 50)
    assert manager.num_free_pages() == 10 - 6
    manager.commit("a", 50)  # 70 stored: block 60 .. 79 starts in page 7
    manager.check_integrity()
    assert manager.num_free_pages() == 11 - 2
    assert manager.max_context_tokens == 64 * 8  # blocks never bound a sequence by the pool
    manager.free("a")
    manager.check_integrity()
    assert manager.num_free_pages() == 11
