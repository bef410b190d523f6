"""Gagotar through the engine against the plain implementation: whole prompts, prompts then
token-by-token decoding, portions of every size, mixed batches with pages and state slots
used again, long decoding through many blocks of positions, greedy generation through ``LLM``
and its scheduler, the replay program as a child process, and the command line."""

from __future__ import annotations

import json

import pytest
import torch

import engine_support as support
import plain_gagotar as plain
from cases import random_tokens
from gagotar_cases import LOUD, LOUD_WIDE, TINY_A, TINY_B, TINY_C, TINY_D, plain_logits

pytestmark = pytest.mark.gpu

CONFIGS = {"a": (TINY_A, LOUD), "b": (TINY_B, LOUD), "c": (TINY_C, LOUD_WIDE),
           "d": (TINY_D, LOUD)}
#: lengths around the blocks (5, 7, 16, 20, 48) and the page (16) of the configurations
LENGTHS = (1, 2, 41, 97, 16, 145)


def _sequences(config: dict, lengths=LENGTHS, seed: int = 0) -> dict[str, list[int]]:
    return {f"r{index}": random_tokens(config["vocab"], length, 50 * seed + index)
            for index, length in enumerate(lengths)}


def _model(tmp_path, name: str, dtype: str):
    config, init = CONFIGS[name]
    folder, state = support.make_model(tmp_path / f"{name}-{dtype}", config, 11, init, dtype)
    return config, folder, state


def _without_close_calls(got: dict, expected: dict, state: dict, config: dict,
                         sequences: dict, below: float) -> dict:
    """``got`` with the positions taken from ``expected`` at which some router of the plain
    model chooses by less than ``below`` of its logits' size. There the model is
    discontinuous: an engine that rounds to 8 bits rightly lands on another expert now and
    then (these random routers have such a position in every few hundred), the logits jump,
    and no comparison can rest on it. A fault of bookkeeping moves the positions around it
    too, which stay in."""
    wide = plain.cast_state(state, torch.float64)
    out = {}
    for rid, tokens in sequences.items():
        close = plain.router_margins(wide, config, torch.tensor(tokens)) < below
        out[rid] = torch.where(close[:, None], expected[rid], got[rid])
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_the_four_ways_of_cutting_the_work_agree_with_the_plain_model(tmp_path, name, dtype):
    config, folder, state = _model(tmp_path, name, dtype)
    sequences = _sequences(config)
    expected = plain_logits(state, config, sequences)
    for label, steps, blocks in (
            ("whole", support.schedule_whole(sequences), 24),
            ("tail", support.schedule_tail(sequences, tail=45), 24),
            ("portions", support.schedule_portions(sequences), 24),
            # 320 tokens of cache for six requests of 302 tokens: pages and slots come back
            ("mixed", support.schedule_mixed(sequences, pool_tokens=320), 21)):
        core = support.build_core(folder, dtype, num_blocks=blocks, max_running=4)
        got = support.replay(core, steps)
        if dtype == "bfloat16":
            got = _without_close_calls(got, expected, state, config, sequences, 1.5e-2)
        support.assert_logits_close(got, expected, dtype, f"gagotar-{name}/{label}")
        assert not core.manager.live_requests()
        del core


@pytest.mark.parametrize("page", [8, 32])
def test_other_page_sizes(tmp_path, page):
    config, folder, state = _model(tmp_path, "a", "float32")
    sequences = _sequences(config, (3, 70, 33), seed=2)
    expected = plain_logits(state, config, sequences)
    core = support.build_core(folder, "float32", num_blocks=1 + 192 // page, block_size=page,
                              max_tokens_per_step=64)
    got = support.replay(core, support.schedule_mixed(sequences, pool_tokens=192))
    support.assert_logits_close(got, expected, "float32", f"gagotar-a/page{page}", page=page)


@pytest.mark.parametrize("name", ["a", "b"])
def test_long_decoding_from_the_first_token(tmp_path, name):
    """One prompt token, then 230 single tokens: dozens of blocks of positions begin and end
    among decoded tokens, their pages are given back (checked after every step by the
    manager's own integrity check), the states run long."""
    config, folder, state = _model(tmp_path, name, "float32")
    sequences = _sequences(config, (231,), seed=3)
    expected = plain_logits(state, config, sequences)
    core = support.build_core(folder, "float32", num_blocks=17, max_running=1)
    got = support.replay(core, support.schedule_tail(sequences, tail=230))
    support.assert_logits_close(got, expected, "float32", f"gagotar-{name}/long-decode")


def test_a_batch_gives_each_request_what_it_gets_alone(tmp_path):
    """The same requests alone and side by side (portions beside single tokens): equal to a
    few rounding steps of float32, whatever row, slot or page a request got."""
    config, folder, _ = _model(tmp_path, "a", "float32")
    sequences = _sequences(config, (60, 5, 33, 18), seed=4)
    alone = support.replay(support.build_core(folder, "float32", num_blocks=24),
                           support.schedule_portions(sequences, sizes=(7, 2, 30, 1)))
    core = support.build_core(folder, "float32", num_blocks=12)
    together = support.replay(core, support.schedule_mixed(sequences, pool_tokens=160))
    for rid in sequences:
        scale = float(alone[rid].abs().max())
        assert float((alone[rid] - together[rid]).abs().max()) <= 2e-5 * scale, rid


def test_portions_of_two_tokens_across_every_border(tmp_path):
    """Portions of two and three tokens all the way: every block's and every page's border is
    crossed inside a portion, between portions, and by a portion's first token."""
    config, folder, state = _model(tmp_path, "a", "float32")
    sequences = _sequences(config, (85, 44), seed=8)
    expected = plain_logits(state, config, sequences)
    for sizes in ((2,), (3, 2), (2, 2, 1)):
        core = support.build_core(folder, "float32", num_blocks=12)
        got = support.replay(core, support.schedule_portions(sequences, sizes=sizes))
        support.assert_logits_close(got, expected, "float32", f"gagotar-a/portions{sizes}")


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_entry_point(tmp_path, graphs):
    from ayaka_b200 import LLM, EngineConfig, SamplingParams

    config, folder, state = _model(tmp_path, "a", "float32")
    prompts = [random_tokens(config["vocab"], n, 90 + n) for n in (1, 9, 40, 17, 3, 26)]
    wide = plain.cast_state(state, torch.float64)
    # a small budget and pool: prompts are cut into portions beside decoding requests, more
    # requests than running slots, so state slots and pages are used again; requests end at
    # different steps, so the decode batch shrinks one by one (five running slots: graph
    # buckets of 1, 2, 4 and 5 rows, so three live requests run in a bucket with a row of
    # padding, which must leave every state alone)
    engine = EngineConfig(model=str(folder), dtype="float32", max_running=5, num_blocks=20,
                          max_tokens_per_step=24, cuda_graph=graphs)
    with LLM.from_config(engine) as llm:
        lengths = [12, 5, 9, 12, 3, 7]
        outputs = llm.generate([tuple(p) for p in prompts],
                               [SamplingParams(temperature=0.0, max_tokens=n) for n in lengths])
        llm.core.manager.check_integrity()
        assert not llm.core.manager.live_requests()
        if graphs:
            assert llm.graphs.replays > 0
    for prompt, output, length in zip(prompts, outputs, lengths):
        assert output.error is None
        assert list(output.outputs[0].token_ids) == \
            plain.greedy_generate(wide, config, prompt, length)


def test_the_replay_program_runs_a_folder_whose_configuration_lacks_the_rank(tmp_path):
    config, folder, state = _model(tmp_path, "b", "float32")
    written = json.loads((folder / "config.json").read_text())
    for entry in written["layers"]:
        del entry["mixer"]["right"]["rank"]
    (folder / "config.json").write_text(json.dumps(written))
    sequences = _sequences(config, (41, 2, 19), seed=5)
    steps = support.schedule_mixed(sequences, pool_tokens=128)
    got = support.run_trace_program(folder, "float32", steps,
                                    support.peak_tokens(steps, sequences), tmp_path / "out",
                                    config["vocab"])
    support.assert_logits_close(got, plain_logits(state, config, sequences), "float32",
                                "gagotar-b/trace_run")


def test_the_command_line_writes_and_runs_a_folder(tmp_path):
    import subprocess
    import sys
    from pathlib import Path

    from ayaka_b200.weights.random_init import random_state
    from ayaka_b200.weights.rules import RandomInit

    root = Path(__file__).resolve().parent.parent
    config_file = tmp_path / "config.json"
    config_file.write_text(json.dumps(TINY_B))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "ayaka_b200", "random", str(config_file),
                           str(folder), "--seed", "4", "--weight-std", "0.12", "--norm-std",
                           "0.1"], capture_output=True, text=True, cwd=root, timeout=600)
    assert made.returncode == 0, made.stderr
    state = random_state(TINY_B, 4, RandomInit(weight_std=0.12, bias_std=0.0, norm_std=0.1))
    prompt = random_tokens(TINY_B["vocab"], 21, 11)
    done = subprocess.run(
        [sys.executable, "-m", "ayaka_b200", "run", str(folder), "-p",
         " ".join(map(str, prompt)), "--max-tokens", "9", "--dtype", "fp32"],
        capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr
    wide = plain.cast_state(state, torch.float64)
    assert [int(t) for t in done.stdout.split()] == plain.greedy_generate(wide, TINY_B, prompt, 9)
    assert "2 layers" in done.stderr
