"""Drawn Gagotar models through drawn schedules: a seed draws every size and constant (widths
that are no multiple of 8, one to eight heads over any divisor of key/value heads, key and
value sizes of any size, rotated parts from nothing to all of a head, rescaled or plain
frequencies, blocks from one position to beyond the prompt, one to nine experts of which any
number is chosen, layers without feed-forward), the requests, the page size, the pool and
every step's cut; the engine must agree with the plain model on every position.
``GAGOTAR_RANDOM_SEEDS`` widens the run."""

from __future__ import annotations

import os
import random

import pytest
import torch

import engine_support as support
import plain_gagotar as plain
from cases import random_tokens
from gagotar_cases import layer, left, model, moe, plain_logits, right
from ayaka_b200.weights.rules import RandomInit

pytestmark = pytest.mark.gpu

SEEDS = range(int(os.environ.get("GAGOTAR_RANDOM_SEEDS", "14")))


def draw_model(rng: random.Random) -> dict:
    width = rng.choice([24, 40, 50, 64, 72, 96, 130])
    layers = []
    for _ in range(rng.randint(1, 4)):
        heads = rng.randint(1, 8)
        kv_heads = rng.choice([g for g in range(1, heads + 1) if heads % g == 0])
        dim = rng.choice([2, 4, 6, 8, 12, 16, 24, 32, 64])
        turned = rng.choice([0, dim, dim, 2 * rng.randint(0, dim // 2)])
        scaling = rng.choice([None, None, {"factor": rng.choice([2.0, 8.0]), "low": 1.0,
                                           "high": rng.choice([2.0, 4.0]),
                                           "original": rng.choice([8, 64, 512])}])
        attention = left(heads, kv_heads, dim, rng.choice([2, 4, 8, 10, 16, 24, 40]),
                         rng.choice([1, 2, 5, 16, 17, 31, 40, 64, 200]), turned=turned,
                         base=rng.choice([10.0, 500.0, 10000.0, 1e6]),
                         scale=rng.choice([None, 0.2, 0.5]), scaling=scaling)
        memory = right(rng.randint(1, 4), rng.choice([2, 4, 8, 16, 20, 40, 80]),
                       rng.choice([2, 4, 8, 12, 16, 33]), rng.choice([1.0, 4.0, 16.0, 50.0]),
                       rng.randint(1, 9))
        experts = rng.randint(1, 9)
        mlp = rng.choice([None, moe(experts, rng.randint(1, experts),
                                    rng.choice([3, 8, 16, 40, 70]),
                                    rng.choice([0.5, 1.5, 7.0]))])
        layers.append(layer(attention, memory, mlp if mlp is not None or rng.random() < 0.5
                            else moe(experts, rng.randint(1, experts), 24, 2.0)))
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
    """bfloat16 against the float64 model on drawn models, which are discontinuous in two
    places. A drawn router chooses by less than a rounding to 8 bits at some position of most
    models; another expert is then rightly chosen, and that position (and, a little, those that
    read it through a later layer) jumps. And at a sequence's first positions the linear
    attention's answer is, once the per-head norm has scaled it to unit size, its value times
    the *sign* of k . q, which a rounding flips where float64 keeps it (seen: 21 % at position
    0, 6 % to 3 % over the next ten, 0.1 % from position 30 on). A fault of bookkeeping moves
    every position behind it. Asked for: all but one position in ten (or one) within 3e-2 of
    the logit scale (row root mean square), and half of them within 1e-2. The float32 run of
    the same seed, schedule and pool is held to 1e-4 at every position where the plain routers
    choose by more than 1e-4 (60 seeds run once: no float32 run failed)."""
    errors = []
    for rid, want in expected.items():
        have = got[rid]
        assert have.shape == want.shape and torch.isfinite(have).all(), (label, rid)
        scale = float(want.abs().max())
        errors.append(((have - want) ** 2).mean(dim=1).sqrt() / scale)
    errors = torch.cat(errors)
    off = int((errors > 3e-2).sum())
    assert off <= max(1, errors.numel() // 10) and float(errors.median()) <= 1e-2, \
        f"{label}: {off} of {errors.numel()} positions beyond 3e-2, median " \
        f"{float(errors.median()):.2e}, worst {float(errors.max()):.2e}"


@pytest.mark.parametrize("seed", SEEDS)
def test_a_drawn_model_through_a_drawn_schedule(tmp_path, seed):
    rng = random.Random(2000 + seed)
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
            assert_mostly_close(got, expected, f"gagotar-drawn[{seed}]")
        else:
            wide = plain.cast_state(state, torch.float64)
            for rid, tokens in sequences.items():  # (a tie of float32 is no fault either)
                close = plain.router_margins(wide, config, torch.tensor(tokens)) < 1e-4
                got[rid] = torch.where(close[:, None], expected[rid], got[rid])
            support.assert_logits_close(got, expected, dtype, "gagotar-drawn", page=page)
        assert not core.manager.live_requests()
        del core
