"""Sukalorn through the engine on the GPU against the plain implementation, in float32 and bfloat16: requests whole,
their last tokens decoded one by one (CUDA graphs), portions down to two tokens, mixed batches with so few pages that
they are used again; decoding from the very first token across several block edges; greedy generation through the
entry point, the scheduler and the command line."""

import functools
import json
import os
import subprocess
import sys

import pytest
import torch

import replay_util as ru
import sukalorn_util as su
from plain import sukalorn_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

LENGTHS = {"S1": (1, 2, 19, 47, 130), "S2": (3, 31, 64, 131), "S3": (5, 40, 97, 200)}
MODES = ("whole", "last32", "portions", "mixed")
MAX_TOKENS = 64 * 6


@functools.lru_cache(maxsize=None)
def _run(name: str, dtype: str):
    raw, page = su.CONFIGS[name]
    folder = su.model_folder(name)
    requests = ru.make_requests(raw["vocab"], LENGTHS[name] + (70, 45), seed=11)
    expected_one = su.plain_logits(folder, raw, requests)
    combined = ru.Trace()
    spans, expected = {}, {}
    for mode in MODES:
        sub = {"whole": ru.trace_whole, "last32": ru.trace_last_decoded, "portions": ru.trace_portions,
               "mixed": lambda r: ru.trace_mixed(r, MAX_TOKENS, seed=5)}[mode](requests)
        spans[mode] = combined.extend(sub, mode + ":")
        expected.update({f"{mode}:{rid}": logits for rid, logits in expected_one.items()})
    outputs, engine = ru.run_on_device(folder, dtype, combined, MAX_TOKENS, page_size=page)
    engine.manager.check_invariants()
    assert engine.manager.free_pages() == [g.pool.count for g in engine.manager.groups]
    return combined, spans, outputs, expected, engine.runner.graph_replays


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S1", "S2", "S3"])
@pytest.mark.parametrize("mode", MODES)
def test_replay_matches_plain(name, dtype, mode):
    combined, spans, outputs, expected, replays = _run(name, dtype)
    first, last = spans[mode]
    part = ru.Trace()
    part.expect = {s: rows for s, rows in combined.expect.items() if first <= s < last}
    assert part.expect and replays > 0
    if dtype == "bfloat16":
        ru.compare_rows_to_scale(part, outputs, expected, rms_bound=0.03, peak_bound=0.15)
    else:
        ru.compare(part, outputs, expected, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S1", "S2"])
def test_decoding_from_the_first_token_across_block_edges(name, dtype):
    """One token a step from position 0 on through 150 positions, through the trace program as a user starts it:
    the first tokens of a sequence, every block edge of both block sizes, pages given back behind each block."""
    raw, page = su.CONFIGS[name]
    folder = su.model_folder(name)
    requests = ru.make_requests(raw["vocab"], (150,), seed=23)
    trace = ru.trace_last_decoded(requests, last=150)
    outputs = ru.run_subprocess(folder, dtype, trace, 192, page_size=page)
    expected = su.plain_logits(folder, raw, requests)
    if dtype == "bfloat16":
        ru.compare_rows_to_scale(trace, outputs, expected, rms_bound=0.03, peak_bound=0.15)
    else:
        ru.compare(trace, outputs, expected, dtype)


@pytest.mark.parametrize("name,lengths", [("S1", (1, 17, 45)), ("S2", (3, 30, 61, 130)), ("S3", (7, 96))])
def test_greedy_generation_equals_plain(name, lengths):
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = su.CONFIGS[name]
    folder = su.model_folder(name)
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=page, num_pages=40, max_batch_tokens=24)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in lengths]
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    w = su.plain_weights(folder)
    assert got == [plain.greedy_generate(w, raw, p, 8) for p in prompts]
    assert engine.manager.free_pages() == [40] * len(engine.manager.groups)
    engine.manager.check_invariants()


def test_bfloat16_greedy_generation_close_to_plain():
    """bfloat16 may pick another token where two logits are within rounding; every pick must still be (nearly) the
    plain model's best token given the same history."""
    from ampere_kv_engine_b200.engine.engine import Engine
    raw, page = su.CONFIGS["S3"]
    folder = su.model_folder("S3")
    engine = Engine.from_pretrained(folder, dtype="bfloat16", page_size=page, num_pages=40)
    prompts = [torch.randint(0, raw["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (5, 33, 100)]
    got = engine.generate(prompts, max_new_tokens=8, ignore_eos=True)
    w = su.plain_weights(folder)
    for prompt, out in zip(prompts, got):
        ids = list(prompt)
        for token in out:
            logits = plain.forward(w, raw, ids)[-1]
            assert float(logits.max() - logits[token]) <= 0.05 * float(logits.std())
            ids.append(token)


def test_command_line_generates(tmp_path):
    raw, page = su.CONFIGS["S2"]
    folder = su.model_folder("S2")
    prompt = [5, 9, 33, 2, 71, 8, 8, 40, 11]
    proc = subprocess.run([sys.executable, "-m", "ampere_kv_engine_b200.runner", "--model", folder, "--mode", "generate",
                           "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "5",
                           "--ignore-eos", "--page-size", str(page)], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    line = next(l for l in proc.stdout.splitlines() if l.startswith("generated_token_ids"))
    assert json.loads(line.split("=", 1)[1]) == plain.greedy_generate(su.plain_weights(folder), raw, prompt, 5)
