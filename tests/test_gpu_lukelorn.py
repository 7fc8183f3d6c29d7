"""Lukelorn on the GPU against the plain implementation (tests/plain/lukelorn_plain.py): every mechanism's kernels alone,
then whole models through the step function, the cache and state manager, the generation loop, the command line and
replay, in both precisions.

Schedules: whole prompts; a prompt, then token by token across page borders and window edges; decoding from the first
token; prompts in portions down to two tokens; steps cut into chunks; batches of unequal requests; slots, pages and
state used again; long decoding.  Mechanisms: a score that towers at the last kept first token and a larger one at the
first token that is not kept, far behind the window; towers at the last key a window still holds, on both sides of page
borders and at the query itself, with larger ones at the first key the window has dropped and right after the query;
sinks far above and far below the scores; output gates; the rotation of adjacent pairs with stretched waves; the delta
rule with a decay per key channel in one piece and in pieces; the latent attention's rotated key part; routing by
sigmoid scores with the weight on the experts' input.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import lukelorn_cases as cases
from tests.plain import lukelorn_plain as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
DTYPES = ["float32", "bfloat16"]
WHOLE = ["a", "b", "c", "d"]
ALONE = ["attention", "channel_delta", "latent_attention"]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    made = {}

    def get(name: str, seed: int = 11):
        key = (name, seed)
        if key not in made:
            cfg = cases.CONFIGS[name]()
            w = cases.random_weights(cfg, seed)
            made[key] = (cases.write_folder(cfg, w, str(tmp_path_factory.mktemp(f"lukelorn-{name}-{seed}"))), cfg, w)
        return made[key]
    return get


def make_stepper(folder, dtype, max_tokens=64 * 60, chunk_tokens=2048, n_slots=None):
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
    the engine chose per request: a list over the runs with experts of [tokens, top], when ``n_moe`` is given)."""
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
            taps = stepper.taps["experts"]                   # chunk by chunk, run by run
            per_run = [torch.cat(taps[i::n_moe]).cpu() for i in range(n_moe)]
        stepper.taps = None
        o = 0
        for r, n in who:
            out[r].append(logits[o:o + n].clone())
            for i in range(n_moe):
                chosen[r][i].append(per_run[i][o:o + n])
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
    """The plain implementation uses the experts the engine chose, whose lowest score must lie within a small slack of
    the rule's cut-off (float32: a rounding error's worth) and differ from the rule's own choice for few tokens."""
    n_moe = cases.moe_runs(cfg)
    got, chosen = run_portions(stepper, requests, portions, n_moe)
    for r, ids in enumerate(requests):
        slack = []
        want = plain.forward(cfg, w, ids, chosen=chosen[r] if n_moe else None, slack=slack)
        if slack:
            assert max(slack) <= cases.CHOICE_SLACK[dtype], f"{what}: a chosen expert lies {max(slack):.3e} below the cut-off"
            assert sum(1 for s in slack if s > 0) <= (0.1 if dtype == "bfloat16" else 0.01) * len(slack) + 1
        check(got[r], want, dtype, f"{what}, request {r}")


# ---------------------------------------------------------------------------
# whole models, and models of one mechanism alone
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", WHOLE + ALONE)
def test_whole_prompt_and_first_tokens(folders, name, dtype):
    folder, cfg, w = folders(name)
    st = make_stepper(folder, dtype)
    for n in (200, 1, 2, 67):
        ids = cases.random_ids(cfg["vocab"], n, 40 + n)
        run_and_check(st, cfg, w, [ids], [[n]], dtype, f"whole prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", WHOLE + ALONE)
def test_prompt_then_token_by_token_across_pages_and_windows(folders, name, dtype):
    """The decoded tokens carry every window of the configurations (1 to 150 tokens) over its edge, and the kept first
    tokens (1 to 130) out of the window."""
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
                                       ("c", [149, 1]), ("d", [1, 2, 147]), ("b", [20, 19, 2, 36, 73]), ("d", [70, 2, 78]),
                                       ("channel_delta", [3, 2, 1, 70, 74]), ("latent_attention", [65, 2, 83])])
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
@pytest.mark.parametrize("name", WHOLE)
def test_batches_of_unequal_requests(folders, name, dtype):
    folder, cfg, w = folders(name)
    reqs = [cases.random_ids(cfg["vocab"], n, 90 + n) for n in (100, 31, 66, 5)]
    portions = [[70] + [1] * 30, [21] + [1] * 10, [64, 2], [2] + [1] * 3]
    run_and_check(make_stepper(folder, dtype), cfg, w, reqs, portions, dtype, "batch")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "d"])
def test_slots_pages_and_state_are_used_again(folders, name, dtype):
    """A cache of two slots and few pages serves nine requests one after another and in pairs: every slot, every page,
    every matrix state and every convolution's inputs are used again with what the last sequence left in them; windowed
    lanes give pages back while a sequence still runs and keep those of the first tokens."""
    folder, cfg, w = folders(name)
    st = make_stepper(folder, dtype, max_tokens=64 * 9, n_slots=2)
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


def _tower_data(T, H, G, d, dv, window, keep, seed):
    """Random q, k, v with scores that tower: at the last key a window still holds, at the last kept first token, at the
    first key, at the query itself and on both sides of page borders (all seen); larger ones at the first key a window
    has dropped, at the first token that is not kept and right after the query (all unseen).  Returns (q, k, v, the
    queries whose rows are looked at one by one)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, H, d, generator=g) * 0.5
    k = torch.randn(T, G, d, generator=g) * 0.5
    v = torch.randn(T, G, dv, generator=g)
    spike = d - 1
    w = window or T + 1
    seen, unseen = [], []
    for qi in (T - 1, T - 2, T - 30, 150, 130, 128, 127, 65, 64, 63, 1, 0):
        if qi < 0 or qi >= T:
            continue
        first = qi - w + 1
        if first > 0:
            seen.append((qi, first))                                   # the last key the window holds
            if keep and first > keep:
                seen.append((qi, keep - 1))                            # the last kept first token, far behind the window
                unseen.append((qi, keep))                              # the first token that is not kept
            elif first - 1 >= keep:
                unseen.append((qi, first - 1))                         # the first key the window has dropped
        else:
            seen.append((qi, 0))
    seen += [(qi, qi) for qi in (T - 3, 100, 64)]
    marked = {a for a, _ in seen} | {b for _, b in seen}
    for qi, kj in seen:
        q[qi, :, spike] = 9.0
        k[kj, :, spike] = 9.0
    for qi, kj in unseen:
        if kj not in marked:
            k[kj, :, spike] = 30.0
    for qi, _ in seen:
        if qi + 1 < T and qi + 1 not in marked:
            k[qi + 1, :, spike] = 30.0                                 # later than the query
    q[110:114] = 0.0                                                   # weights 1 / (keys + the sink's share)
    rows = sorted({qi for qi, _ in seen} | {110, 113})
    return q, k, v, rows


ATTENTION_SIZES = [
    # H, G, d, dv, window, keep_first, cap
    (6, 2, 128, 128, 70, 9, 18.0), (8, 2, 64, 32, 64, 64, 0.0), (4, 1, 32, 96, None, 0, 7.0), (34, 2, 32, 32, 1, 1, 0.0),
    (3, 3, 96, 64, 33, 65, 30.0), (5, 5, 12, 36, 129, 2, 15.0), (4, 2, 24, 40, 40, 130, 0.0), (2, 1, 200, 130, 65, 3, 50.0),
    (16, 1, 64, 128, 100, 33, 25.0), (2, 2, 128, 64, 2, 70, 0.0), (4, 2, 64, 64, 90, 0, 10.0),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("generic", [True, False])
@pytest.mark.parametrize("H,G,d,dv,window,keep,cap", ATTENTION_SIZES)
def test_attention_sees_its_window_the_kept_first_tokens_and_the_sink(dtype, generic, H, G, d, dv, window, keep, cap):
    """Queries and keys enter as they are (no rotation), so the scores, the cap, the window with its kept first tokens,
    the sinks, the gates and the weighted sum are under test.  The sinks of the heads range from far below the scores to
    far above them.  One prompt; a prompt, then single tokens; portions of 70, 2, 61, 5 and single tokens; in slots and
    pages that are not the first, with the pages behind the window given back between the steps; by the kernel of
    every size and by the library's choice (tensor cores where the sizes fit)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    if not generic and not (dtype == "bfloat16" and d % 32 == 0 and dv % 32 == 0 and d <= 128 and dv <= 128):
        pytest.skip("the library's choice is the kernel of every size")
    ops = Ops(DT[dtype])
    T = 230
    q, k, v, rows = _tower_data(T, H, G, d, dv, window, keep, H * d + dv)
    g = torch.Generator().manual_seed(7)
    sinks = torch.linspace(-12.0, 12.0, H)[torch.randperm(H, generator=g)]
    gate = torch.randn(T, H, generator=g) * 2.0
    scale = 0.3
    rnd = lambda t: t.to(DT[dtype]).double()
    want = plain.attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window, keep, sinks.double())
    want = (want * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * dv)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], dim=1).to(DT[dtype]).float()
    proj[:, -H:] = gate
    proj = proj.cuda()
    needs = CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv if dv != d else 0, window=window, keep_first=keep if window else 0)
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
            rows_in = proj[at:at + n].contiguous()
            qr = ops.qk_prepare_store(ctx, rows_in, lane, H, G, d, dv, (None, None, None), None, 0, False, 0.0, extra_cols=H)
            outs.append(fn(ctx, qr, lane, G, dv, scale, window or 0, cap, True, keep_first=keep, sinks=sinks.cuda(),
                           gate=rows_in[:, -H:]))
            at += n
            cache.set_length(slot, at)               # pages behind the window go back; the kept ones stay
        got = torch.cat(outs)
        _close(got, want, dtype)
        for qi in rows:
            _close(got[qi], want[qi], dtype)


@pytest.mark.parametrize("shares", [None, 3])
@pytest.mark.parametrize("H,G,d,window,keep,cap", [(4, 2, 128, 200, 70, 20.0), (2, 1, 64, 300, 129, 0.0), (4, 1, 128, None, 0, 30.0),
                                                   (2, 1, 128, 128, 128, 0.0), (2, 1, 128, 1, 1, 10.0), (6, 3, 64, 129, 300, 15.0)])
def test_tcgen05_attention_with_kept_first_tokens(H, G, d, window, keep, cap, shares, monkeypatch):
    """Prompt portions on the tcgen05 kernel (bfloat16, head sizes 128 and 64) against the plain implementation: kept
    first tokens below, at and above its key step of 128, towers on both sides of the kept tokens' end, two sequences
    in one step, a portion after a history, and a tile's keys shared among blocks."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds

    ops = Ops(torch.bfloat16)
    if shares:
        monkeypatch.setattr(Ops, "prefill_key_shares", lambda self, q_lens, keys, heads: shares)
    T = 1150
    q, k, v, rows = _tower_data(T, H, G, d, d, window, keep, 3 * H + d)
    g = torch.Generator().manual_seed(9)
    sinks = torch.linspace(-6.0, 8.0, H)
    gate = torch.randn(T, H, generator=g) * 2.0
    scale = 0.25
    rnd = lambda t: t.bfloat16().double()
    want = plain.attention_core(rnd(q), rnd(k), rnd(v), scale, cap, window, keep, sinks.double())
    want = (want * torch.sigmoid(gate.double())[:, :, None]).reshape(T, H * d)
    proj = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), gate], dim=1).bfloat16().float()
    proj[:, -H:] = gate
    proj = proj.cuda()
    needs = CacheNeeds(kv_heads=G, head_dim=d, window=window, keep_first=keep if window else 0)
    cache = Cache([needs], max_tokens=64 * 60, dtype=torch.bfloat16, device="cuda:0", n_slots=3)
    cache.open_sequence()
    a, b = cache.open_sequence(), cache.open_sequence()
    lane = cache.lane(0)
    done = {a: 0, b: 0}
    got = {a: [], b: []}
    for step in ([(a, 700), (b, 130)], [(a, 450), (b, 1020)]):
        for slot, n in step:
            cache.reserve(slot, done[slot] + n)
        cache.sync()
        ctx = _ctx([n for _, n in step], [done[s] for s, _ in step], [s for s, _ in step])
        rows_in = torch.cat([proj[done[s]:done[s] + n] for s, n in step]).contiguous()
        qr = ops.qk_prepare_store(ctx, rows_in, lane, H, G, d, d, (None, None, None), None, 0, False, 0.0, extra_cols=H)
        o = ops.sink_attention_tcgen05(ctx, qr, lane, G, scale, window or 0, cap, True, keep_first=keep, sinks=sinks.cuda(),
                                       gate=rows_in[:, -H:])
        at = 0
        for slot, n in step:
            got[slot].append(o[at:at + n])
            at += n
            done[slot] += n
            cache.set_length(slot, done[slot])
    ops.raise_on_kernel_error()
    for slot in (a, b):
        out = torch.cat(got[slot])
        _close(out, want, "bfloat16")
        for qi in rows:
            _close(out[qi], want[qi], "bfloat16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,rot,adjacent", [(64, 64, True), (24, 16, True), (40, 6, True)])
def test_rotation_of_adjacent_pairs_with_stretched_waves(dtype, d, rot, adjacent):
    """The prepared queries and the cached keys against the plain rotation (64-bit angles; the engine's are 32-bit, whose
    rounding grows with the position, so the positions stay in the hundreds)."""
    from cpmcu_b200.cache import Cache
    from cpmcu_b200.ops.ops import Ops
    from cpmcu_b200.parts.base import CacheNeeds
    from cpmcu_b200.parts.position import WavelengthScaledRotary

    ops = Ops(DT[dtype])
    H, G, dv, n, start = 3, 1, 8, 70, 200
    cfg = {"dims": rot, "base": 3000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 256}}
    enc = WavelengthScaledRotary(ops, d, cfg["base"], rot, factor=8.0, low=1.0, high=4.0, original=256, adjacent=adjacent)
    assert torch.allclose(enc.inv_freq.cpu().double(), plain.frequencies(cfg), rtol=1e-7)
    g = torch.Generator().manual_seed(d)
    proj = torch.randn(n, (H + G) * d + G * dv, generator=g).to(DT[dtype]).float()
    cache = Cache([CacheNeeds(kv_heads=G, head_dim=d, value_dim=dv)], max_tokens=64 * 60, dtype=DT[dtype], device="cuda:0", n_slots=1)
    slot = cache.open_sequence()
    cache.reserve(slot, start + n)
    cache.sync()
    ctx = _ctx([n], [start], [slot])
    lane = cache.lane(0)
    q = ops.qk_prepare_store(ctx, proj.cuda(), lane, H, G, d, dv, (None, None, None), enc.inv_freq, rot, False, 0.0,
                             adjacent=adjacent)
    x = torch.zeros(start + n, H + G, d, dtype=torch.float64)
    x[start:] = proj[:, :(H + G) * d].double().view(n, H + G, d)
    want = plain.rotate_pairs(x, cfg)[start:]
    _close(q, want[:, :H], dtype, tol32=3e-5, tol16=1e-2)
    pages = lane.page_table[slot].tolist()
    keys = torch.stack([lane.k[pages[p // 64], 0, p % 64] for p in range(start, start + n)])
    _close(keys, want[:, H], dtype, tol32=3e-5, tol16=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("which", ["rotated", "plain"])
def test_latent_attention_where_one_part_of_the_score_decides(folders, dtype, which):
    """The latent layers alone, with the rotated part of queries and keys (or the plain part) scaled up so that it
    decides the softmax: a rotation that paired other channels, a key part that lost its position or a window one token
    off would move nearly all of a token's weight.  A prompt, then single tokens across the windows' edges."""
    folder, cfg, w = folders("latent_attention")
    w = {k: v.clone() for k, v in w.items()}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}.mix."
        H, d, dr, R = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
        uq = w[p + "uq"].float().view(H, d + dr, -1)
        if which == "rotated" and dr:
            uq[:, d:] *= 6.0
            w[p + "dkv"] = torch.cat([w[p + "dkv"][:R], (w[p + "dkv"][R:].float() * 6.0).bfloat16()])
        elif which == "plain":
            uq[:, :d] *= 6.0
            w[p + "uk"] = (w[p + "uk"].float() * 4.0).bfloat16()
        w[p + "uq"] = uq.reshape(H * (d + dr), -1).bfloat16()
    import tempfile
    folder = cases.write_folder(cfg, w, tempfile.mkdtemp(prefix=f"lukelorn-latent-{which}-"))
    ids = cases.random_ids(cfg["vocab"], 160, 8)
    run_and_check(make_stepper(folder, dtype), cfg, w, [ids], [[60, 2, 18] + [1] * 80], dtype, f"latent attention, {which} part scaled")


@pytest.mark.parametrize("H,G,d,dv", [(3, 3, 16, 40), (6, 2, 40, 8), (2, 1, 70, 20), (4, 4, 64, 64), (2, 2, 128, 32)])
def test_delta_rule_with_a_decay_per_key_channel(H, G, d, dv):
    """channel_decay and the recurrence (fp32) against the plain recurrence: one piece, and pieces for three sequences at
    once whose state starts as rubbish in its slot (a sequence's first token ignores it)."""
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(H * d + dv)
    lens = [90, 7, 41]
    state = torch.randn(5, H, d, dv, generator=g).cuda()
    a_log, dt_bias = torch.randn(H, generator=g) * 0.7 - 1.0, torch.randn(H * d, generator=g)
    data, want = [], []
    for n in lens:
        q = torch.nn.functional.normalize(torch.randn(n, G, d, generator=g), dim=-1) * d ** -0.5
        k = torch.nn.functional.normalize(torch.randn(n, G, d, generator=g), dim=-1)
        v, beta, z = torch.randn(n, H, dv, generator=g), torch.rand(n, H, generator=g), torch.randn(n, H * d, generator=g) * 2
        decay = torch.exp(-torch.exp(a_log.double())[None, :, None] * plain.softplus(z.double() + dt_bias.double()).view(n, H, d))
        rep = H // G
        o, _ = plain.delta_recurrence(q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1), v.double(),
                                      beta.double(), decay)
        data.append((q, k, v, beta, z))
        want.append(o)
    slots = [3, 0, 4]
    done = [0, 0, 0]
    got = [[] for _ in lens]
    for step in ([50, 7, 2], [1, 0, 1], [39, 0, 38]):
        live = [i for i in range(3) if step[i] > 0]
        ctx = _ctx([step[i] for i in live], [done[i] for i in live], [slots[i] for i in live])
        cat = lambda j, width: torch.cat([data[i][j][done[i]:done[i] + step[i]].reshape(step[i], width) for i in live]).cuda()
        decay = ops.channel_decay(cat(4, H * d).contiguous(), a_log.cuda(), dt_bias.cuda(), H, d)
        o = ops.linear_recurrence(ctx, cat(0, G * d), cat(1, G * d), cat(2, H * dv), decay, cat(3, H), state, H, G, d, dv, 1.0,
                                  vector_decay=True)
        at = 0
        for i in live:
            got[i].append(o[at:at + step[i]])
            at += step[i]
            done[i] += step[i]
    for i in range(3):
        _close(torch.cat(got[i]), want[i], "float32", tol32=2e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,top,W,ff,n", [(8, 1, 64, 24, 5), (8, 3, 64, 24, 300), (3, 3, 100, 20, 40), (16, 2, 96, 40, 2), (5, 2, 30, 7, 150)])
def test_experts_chosen_by_sigmoid_scores_with_the_weight_on_their_input(dtype, E, top, W, ff, n):
    """Routing (scores, choice, weights) and the experts' products by pair and by tiles against the plain expert."""
    from cpmcu_b200.ops.ops import Ops

    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(E * W + n)
    z = torch.randn(n, E, generator=g) * 3
    z[0] = torch.linspace(-40, 40, E)                        # saturated scores
    chosen, weights, _ = ops.moe_route(z.cuda(), None, E, top, 1, 1, sigmoid=True)
    s = torch.sigmoid(z.double())
    val, idx = torch.topk(s, top, dim=-1)
    assert torch.equal(chosen.cpu().long()[1:], idx[1:])
    assert torch.allclose(weights.cpu().double(), torch.gather(s, 1, chosen.cpu().long()), atol=1e-6)
    x = (torch.randn(n, W, generator=g)).to(DT[dtype])
    wu = (torch.randn(E, ff, W, generator=g) * W ** -0.5).to(DT[dtype])
    wd = (torch.randn(E, W, ff, generator=g) * ff ** -0.5).to(DT[dtype])
    pairs = ops.moe_experts(x.cuda(), chosen, None, wu.cuda(), wd.cuda(), input_scale=weights)
    out = ops.moe_combine(pairs, None, None, None, top=top).double().cpu()
    want = torch.zeros(n, W, dtype=torch.float64)
    for t in range(n):
        for j in range(top):
            e = int(chosen[t, j])
            w = {"up": wu[e].double(), "down": wd[e].double()}
            want[t] += plain.expert(float(weights[t, j]) * x[t].double()[None], w, "")[0]
    _close(out, want, dtype, tol32=2e-5, tol16=3e-2)
