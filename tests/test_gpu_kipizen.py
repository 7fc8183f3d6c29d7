"""Kipizen on the GPU against the plain implementation (tests/plain/kipizen_plain.py): every mechanism's kernels alone,
then whole models through the step function, the cache and state manager, the generation loop, the command line and
replay, in both precisions.

Schedules: whole prompts; a prompt, then token by token across page borders and window edges; decoding from the first
token; prompts in portions down to two tokens; steps cut into chunks; batches of unequal requests; slots, pages and
state used again; long decoding.  Mechanisms: a score that towers over the others at the first key, far back, on both
sides of a page border, at the last key a window still holds and at the first it has dropped, and at the query itself,
with a larger one just after the query that must not be seen; the sink against scores far below zero; the cap; biases,
the rotation with stretched positions and unit lengths; the recurrence with one decay per head in one piece and in
pieces; the norm over all heads with a gate; routing by logit with a bias.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import kipizen_cases as cases
from tests.plain import kipizen_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DTYPES = ["float32", "bfloat16"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 11):
        key = (name, seed)
        if key not in made:
            cfg = cases.CONFIGS[name]()
            w = cases.random_weights(cfg, seed)
            made[key] = (cases.write_folder(cfg, w, str(tmp_path_factory.mktemp(f"kipizen-{name}-{seed}"))), cfg, w)
        return made[key]
    return get


def make_stepper(folder, dtype, max_tokens=64 * 40, chunk_tokens=2048, n_slots=None):
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.engine.step import Stepper
    from cpmcu_b200.loading import load_model

    _, _, model = load_model(folder, dtype)
    cache = Cache(model.cache_needs(), max_tokens=max_tokens, dtype=DT[dtype], device="cuda:0", n_slots=n_slots,
                  max_step_tokens=chunk_tokens)
    return Stepper(model, cache, chunk_tokens=chunk_tokens)


def run_portions(stepper, requests, portions, n_moe=0):
    """Feeds request r its tokens in portions[r] (sizes that add up to its length), step k taking the k-th portion of
    every request that still has one, all as one batch.  Returns (logits of every position per request, the experts
    the engine chose per request: a list over the layers with experts of [tokens, top], when ``n_moe`` is given)."""
    from cpmcu_b200.engine.step import SequenceStep

    slots = stepper.open(len(requests))
    at = [0] * len(requests)
    out = [[] for _ in requests]
    chosen = [[[] for _ in range(n_moe)] for _ in requests]
    for k in range(max(len(p) for p in portions)):
        batch, who = [], []
        for r, ids in enumerate(requests):
            if k < len(portions[r]):
                n = portions[r][k]
                batch.append(SequenceStep(slots[r], ids[at[r]:at[r] + n], list(range(n))))
                who.append((r, n))
                at[r] += n
        stepper.taps = {"experts": []} if n_moe else None
        logits = stepper.step(batch)
        if n_moe:
            taps = stepper.taps["experts"]                   # chunk by chunk, layer by layer
            per_layer = [torch.cat(taps[i::n_moe]).cpu() for i in range(n_moe)]
        stepper.taps = None
        o = 0
        for r, n in who:
            out[r].append(logits[o:o + n].clone())
            for i in range(n_moe):
                chosen[r][i].append(per_layer[i][o:o + n])
            o += n
        for r, _ in who:
            if at[r] == len(requests[r]) and slots[r] is not None:
                stepper.close(slots[r])
                slots[r] = None
    stepper.ops.raise_on_kernel_error()
    stepper.cache.check_consistent()
    return [torch.cat(x) for x in out], [[torch.cat(c) for c in per] for per in chosen]


def check(got, want, dtype, what=""):
    e = cases.row_errors(got, want)
    worst = int(e.argmax())
    assert float(e.max()) <= cases.TOL[dtype], f"{what}: row {worst} differs by {float(e.max()):.3e} (allowed {cases.TOL[dtype]})"
    if e.numel() >= 20:
        assert float(e.median()) <= cases.MEDIAN_TOL[dtype], f"{what}: the median row differs by {float(e.median()):.3e}"


def run_and_check(stepper, cfg, w, requests, portions, dtype, what):
    """The plain implementation uses the experts the engine chose, whose lowest logit must lie within a small slack of
    the rule's cut-off (float32: a rounding error's worth) and differ from the rule's own choice for few tokens."""
    n_moe = cases.moe_layers(cfg)
    got, chosen = run_portions(stepper, requests, portions, n_moe)
    for r, ids in enumerate(requests):
        slack = []
        want = plain.forward(cfg, w, ids, chosen=chosen[r], slack=slack)
        assert max(slack) <= cases.CHOICE_SLACK[dtype], f"{what}: a chosen expert lies {max(slack):.3e} below the cut-off"
        assert sum(1 for s in slack if s > 0) <= (0.1 if dtype == "bfloat16" else 0.01) * len(slack) + 1
        check(got[r], want, dtype, f"{what}, request {r}")


# ---------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_whole_prompt_and_first_tokens(folders, name, dtype):
    folder, cfg, w = folders(name)
    st = make_stepper(folder, dtype)
    for n in (200, 1, 2, 67):
        ids = cases.random_ids(cfg["vocab"], n, 40 + n)
        run_and_check(st, cfg, w, [ids], [[n]], dtype, f"whole prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_prompt_then_token_by_token_across_pages_and_windows(folders, name, dtype):
    """The decoded tokens carry every window of the four configurations (1 to 150 tokens) over its edge."""
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 230, 3)
    run_and_check(make_stepper(folder, dtype), cfg, w, [ids], [[15] + [1] * 215], dtype, "prompt then decode")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "c"])
def test_token_by_token_from_the_first_token(folders, name, dtype):
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 80, 4)
    run_and_check(make_stepper(folder, dtype), cfg, w, [ids], [[1] * 80], dtype, "decode from the start")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,cuts", [("a", [2] * 40 + [70]), ("a", [63, 1, 64, 2, 20]), ("c", [33, 32, 31, 3, 51]), ("d", [64, 64, 22]),
                                       ("c", [149, 1]), ("d", [1, 2, 147]), ("b", [20, 19, 2, 36, 73]), ("d", [70, 2, 78])])
def test_portions_of_a_prompt(folders, dtype, name, cuts):
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 150, 6)
    run_and_check(make_stepper(folder, dtype), cfg, w, [ids], [cuts], dtype, f"portions {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["c", "d"])
def test_step_function_cuts_long_steps_into_chunks(folders, name, dtype):
    folder, cfg, w = folders(name)
    reqs = [cases.random_ids(cfg["vocab"], n, 70 + n) for n in (130, 50, 3)]
    st = make_stepper(folder, dtype, chunk_tokens=48)
    run_and_check(st, cfg, w, reqs, [[130], [50], [3]], dtype, "chunks of 48")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_batches_of_unequal_requests(folders, name, dtype):
    folder, cfg, w = folders(name)
    reqs = [cases.random_ids(cfg["vocab"], n, 90 + n) for n in (100, 31, 66, 5)]
    portions = [[70] + [1] * 30, [21] + [1] * 10, [64, 2], [2] + [1] * 3]
    run_and_check(make_stepper(folder, dtype), cfg, w, reqs, portions, dtype, "batch")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "d"])
def test_slots_pages_and_state_are_used_again(folders, name, dtype):
    """A cache of two slots and few pages serves nine requests one after another and in pairs: every slot, every page
    and every matrix state is used again with what the last sequence left in it; windowed lanes give pages back while a
    sequence still runs."""
    folder, cfg, w = folders(name)
    st = make_stepper(folder, dtype, max_tokens=64 * 7, n_slots=2)
    for round_no in range(3):
        reqs = [cases.random_ids(cfg["vocab"], n, 100 + 7 * round_no + n) for n in (130, 9, 70)]
        run_and_check(st, cfg, w, reqs[:2], [[100] + [1] * 30, [9]], dtype, "reused slots")
        run_and_check(st, cfg, w, reqs[2:], [[3, 67]], dtype, "reused slots")
        assert st.cache.slots.n_held == 0 and all(g.pages.n_held == 0 for g in st.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["b", "c"])
def test_long_decoding(folders, name, dtype):
    folder, cfg, w = folders(name)
    ids = cases.random_ids(cfg["vocab"], 330, 5)
    run_and_check(make_stepper(folder, dtype, max_tokens=64 * 8), cfg, w, [ids], [[10] + [1] * 320], dtype, "long decode")


# ---------------------------------------------------------------------------
# through the library's own entry points
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("graph", [False, True])
def test_greedy_generation_through_llm(folders, graph):
    """fp32: the tokens of the plain implementation for a batch of unequal prompts (a comparison stops where the two
    best logits nearly tie), twice in a row so that slots and state are used again; prompts go through chunks of 16
    tokens, which the graph variant records and replays, and decoding through the decode runner."""
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("a")
    llm = LLM(folder, dtype="float32", cuda_graph=graph, max_tokens=64 * 16, chunk_length=16)
    prompts = [cases.random_ids(cfg["vocab"], n, 60 + n) for n in (41, 3, 70)]
    want = [plain.greedy(cfg, w, p, 10) for p in prompts]
    for _ in range(2):
        res = llm.generate_batch(prompts, generation_length=10)
        compared = 0
        for r, (tokens, gaps) in zip(res, want):
            firm = next((i for i, g in enumerate(gaps) if g < 1e-3), len(tokens))
            assert r.tokens[:firm] == tokens[:firm]
            compared += firm
        assert compared >= 20


def test_bfloat16_generation_with_graphs_matches_eager(folders):
    from cpmcu_b200 import LLM

    folder, cfg, w = folders("d")
    prompts = [cases.random_ids(cfg["vocab"], n, 80 + n) for n in (33, 90)]
    outs = []
    for graph in (False, True):
        llm = LLM(folder, dtype="bfloat16", cuda_graph=graph, max_tokens=64 * 16, chunk_length=32)
        outs.append([r.tokens for r in llm.generate_batch(prompts, generation_length=10)])
    assert outs[0] == outs[1]


def test_command_line_and_replay(folders, tmp_path):
    folder, cfg, w = folders("c")
    ids = cases.random_ids(cfg["vocab"], 30, 9)
    env = dict(os.environ, PYTHONPATH=ROOT)
    p = subprocess.run([sys.executable, "-m", "cpmcu_b200.cli", "--model-path", folder, "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, ids)), "--num-generate", "6", "--max-tokens", "512"],
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    tokens, gaps = plain.greedy(cfg, w, ids, 6)
    firm = next((i for i, g in enumerate(gaps) if g < 1e-3), 6)
    assert firm >= 1 and " ".join(map(str, tokens[:firm])) in p.stdout.replace(",", " ").replace("  ", " ")
    out = tmp_path / "out"
    steps = [{"step": 0, "entries": [{"id": "r", "tokens": ids[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "r", "tokens": ids[17:29], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "r", "tokens": ids[29:], "want": [0]}], "end": ["r"]}]
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = plain.forward(cfg, w, ids)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4")).view(2, -1)
    got2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4")).view(1, -1)
    assert not (out / "1.f32").exists()
    check(got0, want[[0, 16]], "float32", "replay")
    check(got2, want[[29]], "float32", "replay")
