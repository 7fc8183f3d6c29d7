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


# ---------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------

def _ctx(q_lens, starts, slots):
    """A step's description on the device for sequences that bring ``q_lens`` tokens from positions ``starts``."""
    from cpmcu_b200.parts.base import QUERY_TILE_TOKENS, StepContext

    i32 = dict(dtype=torch.int32, device="cuda")
    pos = torch.cat([torch.arange(s, s + n) for n, s in zip(q_lens, starts)]).to(**i32)
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(q_lens)]).to(**i32)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), **i32)
    kv = [s + n for n, s in zip(q_lens, starts)]
    ctx = StepContext(n_tokens=sum(q_lens), n_seqs=len(q_lens), is_decode=all(n == 1 for n in q_lens), captured=False,
                      q_lens=list(q_lens), kv_lens=kv, slots=list(slots), max_q_len=max(q_lens), max_kv_len=max(kv),
                      token_ids=torch.zeros(sum(q_lens), **i32), positions=pos, token_seq=seq, cu_q=cu,
                      kv_len_dev=torch.tensor(kv, **i32), slot_dev=torch.tensor(list(slots), **i32))
    ts = [i for i, n in enumerate(q_lens) for _ in range(0, n, QUERY_TILE_TOKENS)]
    trow = [r for n in q_lens for r in range(0, n, QUERY_TILE_TOKENS)]
    ctx.q_tiles = (torch.tensor(ts, **i32), torch.tensor(trow, **i32), len(ts))
    return ctx


def _close(got, want, dtype, tol32=3e-5, tol16=2e-2):
    got, want = got.double().cpu(), want.double().cpu()
    err = float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))
    assert err <= (tol32 if dtype == "float32" else tol16), err


def _towers(T, window):
    """(query, key) pairs whose score towers, and keys that tower but must stay unseen (later than the query, or the
    first one a window has dropped)."""
    seen, unseen = [], []
    w = window or T + 1
    for qi in (T - 1, T - 2, 150, 151, 130, 127, 128, 64, 63, 1):
        seen.append((qi, qi - w + 1 if qi - w + 1 >= 0 else 0))                # the last key a window holds, or the first key
        if qi - w >= 0:
            unseen.append((qi, qi - w))                                       # the first key the window has dropped
    seen += [(190, 190), (100, 63 if w > 37 else 100), (101, 64 if w > 37 else 101), (0, 0)]
    return seen, unseen


ATTENTION_SIZES = [
    # H, G, d, dv, window, cap, sink
    (6, 3, 128, 128, 70, 20.0, True), (8, 2, 64, 32, 64, 0.0, True), (4, 1, 32, 96, None, 7.0, True), (34, 2, 32, 32, 1, 0.0, True),
    (3, 3, 96, 64, 33, 30.0, False), (5, 5, 12, 36, 129, 15.0, True), (4, 2, 24, 40, None, 0.0, True), (2, 1, 200, 130, 65, 50.0, True),
    (16, 1, 64, 128, 200, 25.0, True), (2, 2, 128, 64, 2, 0.0, False),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("generic", [True, False])
@pytest.mark.parametrize("H,G,d,dv,window,cap,sink", ATTENTION_SIZES)
def test_sink_window_attention_sees_its_window_and_the_sink(dtype, generic, H, G, d, dv, window, cap, sink):
    """Queries and keys enter as they are (no bias, rotation or norm), so only the scores, the cap, the window, the sink
    and the weighted sum are under test.  A score towers at the last key a window still holds, at the first key, on
    both sides of page borders and at the query itself; a larger one stands at the first key the window has dropped and
    right after the query.  Some queries are zero: their weights are 1 / (keys + 1) with the sink and 1 / keys without.
    One prompt; a prompt, then single tokens; portions of 70, 2, 61, 5 and single tokens; slots and pages that are not
    the first; by the kernel of every size and by the library's choice (tensor cores where the sizes fit)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    if not generic and not (dtype == "bfloat16" and d % 32 == 0 and dv % 32 == 0 and d <= 128 and dv <= 128):
        pytest.skip("the library's choice is the kernel of every size")
    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(H * d + dv)
    T = 230
    q = torch.randn(T, H, d, generator=g) * 0.5
    k = torch.randn(T, G, d, generator=g) * 0.5
    v = torch.randn(T, G, dv, generator=g)
    spike = d - 1
    seen, unseen = _towers(T, window)
    for qi, kj in seen:
        q[qi, :, spike] = 9.0
        k[kj, :, spike] = 9.0
    marked = {qi for qi, _ in seen} | {kj for _, kj in seen}
    for qi, kj in unseen:
        if kj not in marked:
            k[kj, :, spike] = 30.0
    for qi, _ in seen:
        if qi + 1 < T and qi + 1 not in marked:
            k[qi + 1, :, spike] = 30.0                                        # later than the query
    q[110:114] = 0.0
    scale = 0.3
    rnd = lambda t: t.to(DT[dtype]).double()
    want = plain.window_attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window, sink).reshape(T, H * dv)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=1).to(DT[dtype]).float().cuda()
    needs = CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0, window=window)
    fn = ops.sink_attention_generic if generic else ops.sink_attention
    for pieces in ([T], [T - 40] + [1] * 40, [70, 2, 61, 5] + [1] * (T - 138)):
        cache = Cache([needs], max_tokens=64 * 12, dtype=DT[dtype], device="cuda:0", n_slots=3)
        cache.open_sequence()
        other = cache.open_sequence()
        cache.reserve(other, 130)
        slot = cache.open_sequence()
        lane = cache.lane(0)
        outs, at = [], 0
        for n in pieces:
            cache.reserve(slot, at + n)
            cache.sync()
            ctx = _ctx([n], [at], [slot])
            qr = ops.qk_prepare_store(ctx, proj[at:at + n].contiguous(), lane, H, G, d, dv, (None, None, None), None, 0, False, 0.0)
            outs.append(fn(ctx, qr, lane, G, dv, scale, window or 0, cap, sink))
            at += n
        got = torch.cat(outs)
        _close(got, want, dtype)
        for qi in sorted({qi for qi, _ in seen} | {110, 113}):
            _close(got[qi], want[qi], dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_sink_window_attention_batches_unequal_sequences(dtype):
    """Three sequences of different lengths and histories in one step, prompt portions and then single tokens together,
    against each sequence alone by the plain implementation."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(DT[dtype])
    H, G, d, dv, window, cap, scale = 4, 2, 64, 64, 40, 12.0, 0.25
    g = torch.Generator().manual_seed(5)
    lens = [150, 9, 77]
    data = [(torch.randn(n, H, d, generator=g), torch.randn(n, G, d, generator=g), torch.randn(n, G, dv, generator=g)) for n in lens]
    rnd = lambda t: t.to(DT[dtype]).double()
    want = [plain.window_attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window).reshape(n, H * dv) for (q, k, v), n in zip(data, lens)]
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, window=window)], max_tokens=64 * 10, dtype=DT[dtype], device="cuda:0", n_slots=4)
    cache.open_sequence()
    slots = [cache.open_sequence() for _ in lens]
    lane = cache.lane(0)
    done = [0] * 3
    got = [[] for _ in lens]
    steps = [[100, 5, 70], [45, 3, 6]] + [[1, 1, 1]] * 5
    for step in steps:
        take = [min(s, n - a) for s, n, a in zip(step, lens, done)]
        live = [i for i in range(3) if take[i] > 0]
        for i in live:
            cache.reserve(slots[i], done[i] + take[i])
        cache.sync()
        ctx = _ctx([take[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        proj = torch.cat([torch.cat([t[done[i]:done[i] + take[i]].reshape(take[i], -1) for t in data[i]], dim=1) for i in live])
        qr = ops.qk_prepare_store(ctx, proj.to(DT[dtype]).float().cuda().contiguous(), lane, H, G, d, dv, (None, None, None), None, 0,
                                  False, 0.0)
        o = ops.sink_attention(ctx, qr, lane, G, dv, scale, window, cap, True)
        at = 0
        for i in live:
            got[i].append(o[at:at + take[i]])
            at += take[i]
            done[i] += take[i]
    for i in range(3):
        _close(torch.cat(got[i]), want[i][:done[i]], dtype)


@pytest.mark.parametrize("shares", [None, 3])
@pytest.mark.parametrize("H,G,d,window,cap,sink", [(4, 2, 128, 200, 20.0, True), (2, 1, 64, 1100, 0.0, True), (4, 1, 128, None, 30.0, False),
                                                   (2, 1, 128, 128, 0.0, True), (2, 1, 128, 1, 10.0, True), (6, 3, 64, 129, 15.0, True)])
def test_prompt_portions_on_the_tcgen05_kernel(H, G, d, window, cap, sink, shares):
    """Prompt portions of two sequences of unequal lengths on the 128-row tiles of the tcgen05 kernel: windows shorter
    than, equal to and longer than a key step of 128, no window, with and without cap and sink, the keys of a tile in
    one block and shared among three.  Scores tower at the last key a window holds and at the first it has dropped
    (see ``_towers``); the second sequence ends inside the first tile; pages that a window has left are given back after
    every step, so that a tile's first key step begins in a page that now holds later keys."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(H + d)
    lens, scale = [1300, 200], 0.25
    data = [[torch.randn(n, H, d, generator=g) * 0.5, torch.randn(n, G, d, generator=g) * 0.5, torch.randn(n, G, d, generator=g)]
            for n in lens]
    for (q, k, v), n in zip(data, lens):
        seen, unseen = _towers(n, window)
        for qi, kj in seen:
            q[qi, :, 1] = 9.0
            k[kj, :, 1] = 9.0
        marked = {qi for qi, _ in seen} | {kj for _, kj in seen}
        for qi, kj in unseen:
            if kj not in marked:
                k[kj, :, 1] = 30.0
        for qi, _ in seen:
            if qi + 1 < n and qi + 1 not in marked:
                k[qi + 1, :, 1] = 30.0
    rnd = lambda t: t.bfloat16().double()
    want = [plain.window_attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window, sink).reshape(n, H * d) for (q, k, v), n in zip(data, lens)]
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, window=window)], max_tokens=64 * 30, dtype=torch.bfloat16, device="cuda:0",
                  n_slots=4)
    cache.open_sequence()
    slots = [cache.open_sequence() for _ in lens]
    lane = cache.lane(0)
    calls = []
    inner = ops.sink_attention_tcgen05
    ops.sink_attention_tcgen05 = lambda *a, **kw: (calls.append(1), inner(*a, **kw))[1]
    if shares:
        ops.prefill_key_shares = lambda *a, **kw: shares
    done, got = [0, 0], [[], []]
    for step in ([640, 200], [129, 0], [531, 0]):
        live = [i for i in range(2) if step[i] > 0]
        for i in live:
            cache.reserve(slots[i], done[i] + step[i])
        cache.sync()
        ctx = _ctx([step[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        proj = torch.cat([torch.cat([t[done[i]:done[i] + step[i]].reshape(step[i], -1) for t in data[i]], dim=1) for i in live])
        qr = ops.qk_prepare_store(ctx, proj.bfloat16().float().cuda().contiguous(), lane, H, G, d, d, (None, None, None), None, 0,
                                  False, 0.0)
        o = ops.sink_attention(ctx, qr, lane, G, d, scale, window or 0, cap, sink)
        at = 0
        for i in live:
            got[i].append(o[at:at + step[i]])
            at += step[i]
            done[i] += step[i]
            cache.set_length(slots[i], done[i])          # pages behind the window go back and are taken again below
    ops.raise_on_kernel_error()
    assert len(calls) == (3 if d == 128 else 1)          # head size 64 goes there from 1,024 keys on
    for i in range(2):
        full = torch.cat(got[i])
        _close(full, want[i], "bfloat16")
        seen, _ = _towers(lens[i], window)
        for qi in sorted({qi for qi, _ in seen}):
            _close(full[qi], want[i][qi], "bfloat16")


@pytest.mark.parametrize("H,G,d,dv,window,sink", [(6, 2, 64, 64, 700, True), (4, 1, 128, 32, None, True), (20, 1, 32, 128, 1000, False)])
def test_single_tokens_whose_keys_are_shared_among_blocks(H, G, d, dv, window, sink):
    """Two sequences of unequal lengths bring one token each; the keys of a token are divided among 1, 3 and 16 blocks
    and by the library's own choice.  The score towers at a far key (the last one the window holds, or the first key)
    for one sequence and at the query's own key for the other, so that a share that is lost or counted twice shows;
    the shorter sequence leaves most shares of 16 empty."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(torch.bfloat16)
    g = torch.Generator().manual_seed(d + dv)
    lens, scale, cap = [1500, 45], 0.2, 25.0
    data = [(torch.randn(n, H, d, generator=g) * 0.5, torch.randn(n, G, d, generator=g) * 0.5, torch.randn(n, G, dv, generator=g))
            for n in lens]
    far = lens[0] - window if window else 0
    data[0][0][-1, :, 3] = 9.0
    data[0][1][far, :, 3] = 9.0
    if far > 0:
        data[0][1][far - 1, :, 3] = 30.0                                      # the first key the window has dropped
    data[1][0][-1, :, 5] = 9.0
    data[1][1][-1, :, 5] = 9.0
    rnd = lambda t: t.bfloat16().double()
    want = torch.cat([plain.window_attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window, sink)[-1:].reshape(1, H * dv)
                      for q, k, v in data])
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0, window=window)], max_tokens=64 * 30,
                  dtype=torch.bfloat16, device="cuda:0", n_slots=3)
    cache.open_sequence()
    slots = [cache.open_sequence() for _ in lens]
    lane = cache.lane(0)
    for (q, k, v), n, slot in zip(data, lens, slots):                         # all but the last token, as a prompt
        cache.reserve(slot, n)
        cache.sync()
        ctx = _ctx([n - 1], [0], [slot])
        proj = torch.cat([t[:n - 1].reshape(n - 1, -1) for t in (q, k, v)], dim=1).bfloat16().float().cuda().contiguous()
        ops.qk_prepare_store(ctx, proj, lane, H, G, d, dv, (None, None, None), None, 0, False, 0.0)
    ctx = _ctx([1, 1], [n - 1 for n in lens], slots)
    proj = torch.cat([torch.cat([t[-1:].reshape(1, -1) for t in seq], dim=1) for seq in data]).bfloat16().float().cuda().contiguous()
    qr = ops.qk_prepare_store(ctx, proj, lane, H, G, d, dv, (None, None, None), None, 0, False, 0.0)
    assert ops.sink_attention_splits(ctx, 2, H, G, window or 0) > 1
    choose = ops.sink_attention_splits
    try:
        for n_splits in (None, 1, 3, 16):
            if n_splits is not None:
                ops.sink_attention_splits = lambda *a, n_splits=n_splits: n_splits
            got = ops.sink_attention_bf16(ctx, qr, lane, G, dv, scale, window or 0, cap, sink)
            _close(got, want, "bfloat16")
            _close(got[0], want[0], "bfloat16")
            _close(got[1], want[1], "bfloat16")
    finally:
        ops.sink_attention_splits = choose


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,rot_dim,base,factor", [(4, 2, 64, 64, 32, 20000.0, 2.0), (3, 1, 24, 40, 24, 300.0, 1.0),
                                                            (2, 2, 128, 32, 0, 1.0, 1.0), (5, 5, 20, 20, 8, 1e6, 7.5)])
def test_biases_rotation_and_unit_lengths_before_the_cache(dtype, H, G, d, dv, rot_dim, base, factor):
    """The whole mixer with identity projections against the plain one: biases on q, k and v, the rotation of the first
    channels of a head in pairs (i, i + dims/2) with stretched positions, unit root mean square per head, and a second
    layer's queries over the first layer's cached keys and values."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds
    from cpmcu_b200.parts.position import LinearlyScaledRotary

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(d + dv)
    T, eps, scale, window, cap = 140, 1e-5, 0.9, 50, 10.0
    q = torch.randn(T, H * d, generator=g)
    k = torch.randn(T, G * d, generator=g)
    v = torch.randn(T, G * dv, generator=g)
    q2 = torch.randn(T, H * d, generator=g)
    bq, bk, bv, bq2 = (torch.randn(n, generator=g) for n in (H * d, G * d, G * dv, H * d))
    W = q.shape[1] + k.shape[1] + v.shape[1]
    h = torch.cat([q, k, v], dim=1).double()
    eye = torch.eye(W, dtype=torch.float64)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale, "softcap": cap, "mask": {"size": window}}
    if rot_dim:
        m["rot"] = {"dims": rot_dim, "base": base, "scaling": {"factor": factor}}
    w = {"q": eye[:H * d], "k": eye[H * d:H * d + G * d], "v": eye[H * d + G * d:], "o": torch.eye(H * dv, dtype=torch.float64),
         "q.b": bq.double(), "k.b": bk.double(), "v.b": bv.double()}
    want = plain.window_attention(h, w, "", m, eps)
    kv = plain.attention_keys_values(h, w, "", m, eps)
    w2 = dict(w, **{"q": torch.eye(H * d, dtype=torch.float64), "q.b": bq2.double()})
    want2 = plain.window_attention(q2.double(), w2, "", m, eps, kv=kv)
    inv_freq = LinearlyScaledRotary(ops, d, base, rot_dim, factor).inv_freq if rot_dim else None
    needs = CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0, window=window)
    for pieces in ([T], [T - 20] + [1] * 20, [3, 66, 2] + [1] * (T - 71)):
        cache = Cache([needs], max_tokens=64 * 8, dtype=DT[dtype], device="cuda:0", n_slots=2)
        cache.open_sequence()
        slot = cache.open_sequence()
        lane = cache.lane(0)
        outs, outs2, at = [], [], 0
        for n in pieces:
            cache.reserve(slot, at + n)
            cache.sync()
            ctx = _ctx([n], [at], [slot])
            qr = ops.qk_prepare_store(ctx, h[at:at + n].float().cuda().contiguous(), lane, H, G, d, dv,
                                      (bq.cuda(), bk.cuda(), bv.cuda()), inv_freq, rot_dim, True, eps)
            outs.append(ops.sink_attention(ctx, qr, lane, G, dv, scale, window, cap, True))
            qr2 = ops.qk_prepare_store(ctx, q2[at:at + n].float().cuda().contiguous(), lane, H, G, d, dv, (bq2.cuda(), None, None),
                                       inv_freq, rot_dim, True, eps, has_kv=False)
            outs2.append(ops.sink_attention(ctx, qr2, lane, G, dv, scale, window, cap, True))
            at += n
        _close(torch.cat(outs), want, dtype, tol32=5e-5, tol16=3e-2)
        _close(torch.cat(outs2), want2, dtype, tol32=5e-5, tol16=3e-2)


@pytest.mark.parametrize("H,d,dv", [(3, 20, 24), (6, 32, 64), (1, 72, 16), (2, 128, 130), (5, 8, 8)])
def test_lightning_recurrence_in_one_piece_and_in_pieces(H, d, dv):
    """One decay per head (one of them 1, one small), three sequences at once in slots that hold rubbish, in one piece,
    in two and in pieces down to single tokens; the state lives on between the steps."""
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(d * dv + H)
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    decay[0] = 1.0
    decay[-1] = 0.05 if H > 1 else 0.9
    lens = [90, 1, 37]
    ins, want = [], []
    for n in lens:
        q, k, v = torch.rand(n, H, d, generator=g), torch.rand(n, H, d, generator=g) - 0.3, torch.randn(n, H, dv, generator=g)
        ins.append((q, k, v))
        want.append(plain.lightning_recurrence(q.double(), k.double(), v.double(), decay.double())[0])
    for cuts in ([1.0], [0.5, 1.0], [0.1, 0.2, 0.6, 1.0], [i / 45 for i in range(1, 46)]):
        state = torch.full((5, H, d, dv), 7.0, device="cuda")
        slots = [4, 0, 2]
        got = [[] for _ in lens]
        done = [0] * len(lens)
        for c in cuts:
            upto = [max(done[i] + 1, int(round(n * c))) if done[i] < n else n for i, n in enumerate(lens)]
            upto = [min(u, n) for u, n in zip(upto, lens)]
            live = [i for i in range(len(lens)) if upto[i] > done[i]]
            if not live:
                continue
            ctx = _ctx([upto[i] - done[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
            cat = lambda j: torch.cat([ins[i][j][done[i]:upto[i]].reshape(upto[i] - done[i], -1) for i in live]).cuda().contiguous()
            dec = decay.cuda().unsqueeze(0).expand(ctx.n_tokens, H)
            o = ops.linear_recurrence(ctx, cat(0), cat(1), cat(2), dec, None, state, H, H, d, dv, 1.0)
            at = 0
            for i in live:
                got[i].append(o[at:at + upto[i] - done[i]])
                at += upto[i] - done[i]
                done[i] = upto[i]
        for i in range(len(lens)):
            _close(torch.cat(got[i]), want[i], "float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dv,group,act", [(6, 64, 6, "sigmoid"), (3, 24, 3, "sigmoid"), (4, 16, 2, "silu"), (1, 130, 1, "sigmoid"), (5, 8, 1, "silu")])
def test_norm_over_heads_with_gate_and_activations_in_place(dtype, H, dv, group, act):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(H * dv)
    T, eps = 37, 1e-5
    o = torch.randn(T, H, dv, generator=g) * 3
    row = torch.randn(T, H * dv + 5, generator=g)                      # the gate is a slice of a wider row
    weight = torch.randn(group * dv, generator=g)
    x = o.double().view(T, H // group, group * dv)
    want = plain.rms_norm(x, weight.double(), eps).reshape(T, H * dv)
    gate = row[:, 5:].double()
    want = want * (torch.sigmoid(gate) if act == "sigmoid" else plain.silu(gate))
    got = ops.gated_group_norm(o.cuda(), row.cuda()[:, 5:], weight.cuda(), eps, group, act)
    _close(got, want, dtype)
    wide = torch.randn(T, 50, generator=g)
    got = ops.silu_columns(wide.clone().cuda(), 33)
    _close(got[:, :33], plain.silu(wide[:, :33].double()), "float32")
    assert torch.equal(got[:, 33:].cpu(), wide[:, 33:])


@pytest.mark.parametrize("E,top", [(8, 4), (10, 3), (6, 6), (5, 1), (64, 6), (300, 8)])
def test_routing_by_logit_with_bias_and_softmax_over_the_chosen(E, top):
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(E + top)
    T = 50
    z = torch.randn(T, E + 3, generator=g) * 3                           # rows wider than the experts
    z[7] = -40.0 - torch.arange(E + 3)                                   # all far below zero: still a choice and weights that sum to 1
    bias = torch.randn(E, generator=g) * 2
    chosen, weights, _ = ops.moe_route(z.cuda(), None, E, top, 1, 1, bias=bias.cuda(), top_first=True)
    full = (z[:, :E] + bias).double()
    val, idx = torch.topk(full, top, dim=-1)
    want_w = torch.softmax(val, dim=-1)
    got_idx = chosen.cpu().long()
    order = torch.argsort(got_idx, dim=1)
    want_order = torch.argsort(idx, dim=1)
    assert torch.equal(torch.gather(got_idx, 1, order), torch.gather(idx, 1, want_order))
    _close(torch.gather(weights.cpu(), 1, order), torch.gather(want_w, 1, want_order), "float32")
    assert float((weights.sum(-1) - 1).abs().max()) < 1e-5
