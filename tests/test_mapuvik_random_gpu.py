"""Drawn Mapuvik models through drawn schedules: a seed draws every size and constant (widths
that are no multiple of 8, one to six heads, key rows of any even size, windows from 1 to
beyond the prompt, taps 1 to 5, groups, borrowed layers, layers without feed-forward, the
order of the mixers), the requests, the page size, the pool and every step's cut; the engine
must agree with the plain model on every position. ``MAPUVIK_RANDOM_SEEDS`` widens the run."""

from __future__ import annotations

import os
import random

import pytest

import engine_support as support
from cases import random_tokens
from mapuvik_cases import latent, layer, mamba, mlstm, model, plain_logits
from ayaka_b200.weights.rules import RandomInit

pytestmark = pytest.mark.gpu

SEEDS = range(int(os.environ.get("MAPUVIK_RANDOM_SEEDS", "12")))


def draw_model(rng: random.Random) -> dict:
    width = rng.choice([24, 40, 50, 64, 72, 96, 130])
    layers, owners = [], []
    for index in range(rng.randint(1, 5)):
        if owners and rng.random() < 0.25:
            owner = rng.choice(owners)
            layers.append({**{k: v for k, v in layers[owner].items() if k != "weights_of"},
                           "weights_of": owner})
            continue
        kind = rng.choice(["latent", "mamba", "mlstm"])
        if kind == "latent":
            rot = rng.choice([2, 4, 6, 8, 16])
            entry = latent(rng.randint(1, 6), rng.choice([4, 8, 12, 16, 24]), rot,
                           rng.choice([4, 8, 10, 16, 32]), rng.choice([6, 8, 14, 16, 24, 40, 64]),
                           rng.choice([1, 2, 5, 16, 17, 31, 40, 200]),
                           turned=rng.choice([rot, rot, max(2, rot - 2)]),
                           base=rng.choice([10.0, 500.0, 10000.0, 1e6]),
                           scale=rng.choice([None, 0.2, 0.5]))
        elif kind == "mamba":
            groups = rng.choice([1, 1, 2, 3])
            heads = groups * rng.randint(1, 3)
            columns = rng.choice([4, 6, 8, 16, 20])
            divisors = [d for d in (1, 2, 3, 4) if (heads * columns) % d == 0]
            entry = mamba(heads, columns, rng.choice([2, 4, 8, 16, 24, 64, 72]), groups,
                          rng.randint(1, 5), rng.choice(divisors))
        else:
            entry = mlstm(rng.randint(1, 4), rng.choice([4, 8, 16, 20, 40, 80]),
                          rng.choice([4, 8, 12, 16, 33]), rng.choice([2.0, 8.0, 15.0, 30.0]))
        owners.append(index)
        layers.append(layer(entry, rng.choice([None, 16, 40, 70, 128])))
    return model(rng.choice([17, 64, 101, 300]), width, rng.choice([1e-5, 1e-6, 1e-3]), layers)


def draw_steps(rng: random.Random, sequences: dict[str, list[int]], pool_tokens: int
               ) -> list[dict]:
    sizes = tuple(rng.choice([1, 1, 2, 2, 3, 5, 8, 15, 16, 17, 31, 33, 64]) for _ in range(9))
    kind = rng.choice(["whole", "tail", "portions", "mixed", "mixed"])
    if kind == "whole":
        return support.schedule_whole(sequences)
    if kind == "tail":
        return support.schedule_tail(sequences, tail=rng.choice([1, 7, 40]))
    if kind == "portions":
        return support.schedule_portions(sequences, sizes=sizes)
    return support.schedule_mixed(sequences, pool_tokens=pool_tokens,
                                  live_limit=rng.choice([2, 3, 4]),
                                  decode_tail=rng.choice([0, 3, 20]), sizes=sizes)


def assert_mostly_close(got: dict, expected: dict, label: str) -> None:
    """bfloat16 against the float64 model on drawn models. Some drawn models are
    discontinuous where they stand: at a sequence's first positions an mLSTM's answer is its
    value times the *sign* of k . q once the per-head norm has scaled it to unit size, a
    norm over a group of three entries does the same to a state-space layer, and a rounding
    of the inputs to 8 bits flips a sign that float64 keeps (seen: 26 % at position 0 of a
    request, where no cache, page or state is involved, 0.1 % at its neighbours). So single
    positions may be off; what a fault of bookkeeping does is different: it moves every position
    behind it. Asked for here: all but one position in twenty (or one) within 3e-2 of the logit
    scale (row root mean square), and half of them within 1e-2. The float32 run of the same seed,
    schedule and pool is held to 1e-4 at every position."""
    import torch

    errors = []
    for rid, want in expected.items():
        have = got[rid]
        assert have.shape == want.shape and torch.isfinite(have).all(), (label, rid)
        scale = float(want.abs().max())
        errors.append(((have - want) ** 2).mean(dim=1).sqrt() / scale)
    errors = torch.cat(errors)
    off = int((errors > 3e-2).sum())
    assert off <= max(1, errors.numel() // 20) and float(errors.median()) <= 1e-2, \
        f"{label}: {off} of {errors.numel()} positions beyond 3e-2, median " \
        f"{float(errors.median()):.2e}, worst {float(errors.max()):.2e}"


@pytest.mark.parametrize("seed", SEEDS)
def test_a_drawn_model_through_a_drawn_schedule(tmp_path, seed):
    rng = random.Random(1000 + seed)
    config = draw_model(rng)
    init = RandomInit(weight_std=rng.choice([0.08, 0.15]) * (64 / config["width"]) ** 0.5,
                      scale_residual_projections=False, bias_std=0.1, norm_std=0.1)
    lengths = [rng.choice([1, 2, 3, 15, 16, 17, 33, 60, 97, 140]) for _ in range(rng.randint(1, 6))]
    sequences = {f"s{i}": random_tokens(config["vocab"], n, 7 * seed + i)
                 for i, n in enumerate(lengths)}
    page = rng.choice([8, 16, 16, 32])
    pool_tokens = max(-(-n // 64) * 64 for n in lengths) + rng.choice([0, 64, 256])
    steps = draw_steps(rng, sequences, pool_tokens)
    for dtype in ("float32", "bfloat16") if seed % 3 == 0 else ("float32",):
        folder, state = support.make_model(tmp_path / f"model-{dtype}", config, seed, init, dtype)
        core = support.build_core(folder, dtype,
                                  num_blocks=max(pool_tokens // page + 1 + 8 // page, 6),
                                  block_size=page, max_running=4,
                                  max_tokens_per_step=max(256, page))
        got = support.replay(core, steps)
        expected = plain_logits(state, config, sequences)
        if dtype == "bfloat16":
            assert_mostly_close(got, expected, f"mapuvik-drawn[{seed}]")
        else:
            support.assert_logits_close(got, expected, dtype, "mapuvik-drawn", page=page)
        assert not core.manager.live_requests()
        del core
