"""Suposun through the engine against the plain implementation: whole requests, the last tokens one by one, prompts in
portions down to two tokens, unequal batches with reused slots, blocks and kept tokens, the first tokens, long decoding
past every window, a step of seventy sequences, greedy generation through the package's entry point and a replay through
bin/trace_run — in 32-bit and in bfloat16, on four small models whose sizes all differ."""
import pytest
import torch

import plain_suposun as plain
from conftest import random_ids, record_error
from engine_drives import drive_batches, drive_portions, drive_tail_one_by_one, drive_whole, poison
from suposun_models import MODELS, SHARP_FACTOR, write_model

pytestmark = pytest.mark.gpu

#: largest absolute logit error over the largest absolute logit of the plain implementation
TOL = {"float32": 1e-4, "bfloat16": 5e-2}
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"sup_a": [1 + 12, 17 + 12, 64 + 12, 65 + 12, 150, 215], "sup_b": [3 + 10, 63 + 10, 129 + 10, 200],
           "sup_odd": [2 + 8, 40 + 8, 100 + 8, 141], "sup_sharp": [5 + 16, 64 + 16, 127 + 16, 260]}
DECODE = {"sup_a": 12, "sup_b": 10, "sup_odd": 8, "sup_sharp": 16}
NAMES = list(MODELS)
#: per model and request: the leading positions without a close call of a router (plain.decided_prefix)
DECIDED: dict = {}


def poison_states(engine):
    """NaN in every block of the cache and an impossible token in the kept tokens of every slot that no sequence holds: a
    slot that is taken must be zeroed, not trusted."""
    poison(engine)
    for g in engine.cache._groups:
        if hasattr(g, "state"):
            for s in range(engine.cache.n_slots):
                if not engine.cache.slots.is_held(s):      # (a kept token that no vocabulary has: reading it raises the error word)
                    g.state[:, s].fill_(float("nan") if g.state.is_floating_point() else 1 << 30)


@pytest.fixture(scope="module")
def sup_dirs(tmp_path_factory):
    out = {}
    for i, (name, cfg) in enumerate(MODELS.items()):
        d = tmp_path_factory.mktemp(name)
        write_model(cfg, 40 + i, d, sharp=SHARP_FACTOR if name == "sup_sharp" else 1.0)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def truth(sup_dirs):
    out = {}
    for name, d in sup_dirs.items():
        cfg, w = plain.read_model_dir(d)
        reqs = [random_ids(cfg["vocab"], n, 11 + i) for i, n in enumerate(LENGTHS[name])]
        out[name] = (cfg, w, reqs, [plain.logits_all_positions(cfg, w, ids) for ids in reqs])
        DECIDED[name] = [plain.decided_prefix(cfg, w, ids) for ids in reqs]
    return out


def make_engine(sup_dirs, name, dtype, max_tokens):
    from vlrf_b200.engine import Engine, load_model
    eng = Engine(load_model(sup_dirs[name], dtype), max_tokens=max_tokens)
    poison_states(eng)
    return eng


def compare(got, want, dtype, what, model, decided=None):
    """32-bit: every position.  bfloat16: the positions before a router's first close call (`decided`, per request;
    None: all), since rounding may choose another expert there and everything later in the sequence depends on that token."""
    worst = 0.0
    for i, (g, t) in enumerate(zip(got, want)):
        assert g.shape == t.shape, f"{what}: request {i} has shape {tuple(g.shape)}, expected {tuple(t.shape)}"
        assert torch.isfinite(g).all(), f"{what}: request {i} has non-finite logits (something unwritten was read)"
        err = (g.double() - t).abs().max(dim=1).values / float(t.abs().max())
        if dtype != "float32" and decided is not None:
            err = err[:decided[i]]
            if err.numel() == 0:
                continue
        bad = (err > TOL[dtype]).nonzero()
        assert bad.numel() == 0, (f"{what} ({model}, {dtype}): request {i} (length {len(t)}) first differs at position "
                                  f"{int(bad[0])} with error {float(err[bad[0]]):.3e} of the logit scale")
        worst = max(worst, float(err.max()))
    record_error("suposun " + what, model, dtype, worst)


def test_the_sharp_model_is_sharp_and_decided(truth):
    """Its last position must depend on single tokens at the edges of the first layer's mask: another token at the last kept
    position (8 of its nine, 251 positions back) and another at the oldest position inside its window of 48 each move
    the last logits far beyond rounding; and none of its routers has a choice to make, so bfloat16 is compared at every
    position."""
    cfg, w, reqs, want = truth["sup_sharp"]
    for place in (8, len(reqs[3]) - 48):
        ids = [(t + 1) % cfg["vocab"] if i == place else t for i, t in enumerate(reqs[3])]
        moved = plain.logits_all_positions(cfg, w, ids)[-1]
        assert float((moved - want[3][-1]).abs().max() / want[3].abs().max()) > 0.02, place
    assert DECIDED["sup_sharp"] == [len(r) for r in reqs]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(sup_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    eng = make_engine(sup_dirs, name, dtype, 320)
    compare(drive_whole(eng, reqs), want, dtype, "whole", name, DECIDED[name])
    eng.cache.check()
    assert eng.cache.slots.n_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_last_tokens_one_by_one(sup_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    eng = make_engine(sup_dirs, name, dtype, 320)
    compare(drive_tail_one_by_one(eng, reqs, 32), want, dtype, "prefix + 32 single tokens", name, DECIDED[name])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("portion", [2, 3, 7, 64, 65])
def test_prompts_in_portions(sup_dirs, truth, portion, dtype):
    """Portions of an even and of an odd number of tokens (the two copies of the kept token), down to two tokens."""
    for name in ("sup_a", "sup_odd", "sup_sharp"):
        _, _, reqs, want = truth[name]
        eng = make_engine(sup_dirs, name, dtype, 320)
        compare(drive_portions(eng, reqs[1:], portion), want[1:], dtype, f"portions of {portion}", name, DECIDED[name][1:])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_with_reused_slots_blocks_and_states(sup_dirs, truth, name, dtype):
    _, _, reqs, want = truth[name]
    prompt_lens = [max(1, len(r) - DECODE[name]) for r in reqs]
    batch = 3
    order = list(reversed(range(len(reqs))))

    def need_of(rs):
        return max(sum((len(r) + 63) // 64 * 64 for r in rs[b:b + batch]) for b in range(0, len(rs), batch))

    eng = make_engine(sup_dirs, name, dtype, max(need_of(reqs), need_of([reqs[i] for i in order])))
    compare(drive_batches(eng, reqs, batch, prompt_lens), want, dtype, "unequal batches", name, DECIDED[name])
    assert eng.cache.slots.n_held == 0
    poison_states(eng)           # what the second pass reads it must have written (or zeroed) itself
    got = drive_batches(eng, [reqs[i] for i in order], batch, [prompt_lens[i] for i in order])
    compare(got, [want[i] for i in order], dtype, "unequal batches, reused cache", name, [DECIDED[name][i] for i in order])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_first_tokens(sup_dirs, truth, name, dtype):
    cfg, w, _, _ = truth[name]
    reqs = [random_ids(cfg["vocab"], n, 70 + n) for n in (1, 2, 3, 1)]
    want = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    decided = [plain.decided_prefix(cfg, w, ids) for ids in reqs]
    eng = make_engine(sup_dirs, name, dtype, 256)
    compare(drive_whole(eng, reqs), want, dtype, "first tokens, whole", name, decided)
    compare(drive_batches(eng, reqs, 4, [1, 1, 1, 1]), want, dtype, "first tokens, batch", name, decided)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_one_token(sup_dirs, truth, dtype):
    for name in ("sup_a", "sup_sharp"):
        cfg, w, _, _ = truth[name]
        ids = random_ids(cfg["vocab"], 200, 5)
        want = plain.logits_all_positions(cfg, w, ids)
        eng = make_engine(sup_dirs, name, dtype, 256)
        compare(drive_tail_one_by_one(eng, [ids], tail=len(ids) - 1), [want], dtype, "decoding 200 positions", name,
                [plain.decided_prefix(cfg, w, ids)])


def test_a_batch_of_seventy_sequences(sup_dirs, truth):
    """More rows in a decode step than the few-row products take."""
    cfg, w, _, _ = truth["sup_odd"]
    reqs = [random_ids(cfg["vocab"], 4 + (i * 7) % 30, 300 + i) for i in range(70)]
    want = [plain.logits_all_positions(cfg, w, ids) for ids in reqs]
    decided = [plain.decided_prefix(cfg, w, ids) for ids in reqs]
    for dtype in DTYPES:
        eng = make_engine(sup_dirs, "sup_odd", dtype, 70 * 64)
        compare(drive_batches(eng, reqs, 70, [max(1, len(r) - 3) for r in reqs]), want, dtype, "seventy sequences", "sup_odd", decided)


@pytest.mark.parametrize("name", ["sup_a", "sup_b"])
def test_greedy_generation_through_the_entry_point(tmp_path, name):
    """Seven requests over three rows: requests wait, take over rows (and kept tokens) of those that ended, and decode in the
    replayed session beside padding rows, whose first step runs twice; every request gets what it gets alone from the
    plain implementation (32-bit, so that no argmax rests on rounding)."""
    from vlrf_b200.api import Model
    from vlrf_b200.sampling.params import SamplingParams
    write_model(MODELS[name], 77, tmp_path)
    cfg, w = plain.read_model_dir(tmp_path)
    prompts = [random_ids(cfg["vocab"], n, 900 + n) for n in (3, 20, 1, 66, 9, 33, 5)]
    new = [6, 3, 9, 4, 7, 2, 8]
    model = Model.load(tmp_path, "float32", max_tokens=3 * 128, n_slots=3)
    params = [SamplingParams(max_new_tokens=n, do_sample=False) for n in new]
    results = model.generate_ids(prompts, params)
    want = [plain.greedy_generate(cfg, w, p, n) for p, n in zip(prompts, new)]
    assert [r.new_tokens for r in results] == want
    assert len({t for ts in want for t in ts}) > 10, "the model just repeats itself: the test would show nothing"
    assert model.engine.cache.slots.n_held == 0
    model.engine.cache.check()


def test_trace_replay_of_a_batch_of_unequal_requests(sup_dirs, truth, tmp_path):
    """`bin/trace_run` on a Suposun folder: twelve requests of 1 to 70 tokens start together in one step, go on one token
    a step and end one after another.  32-bit, every wanted position."""
    from test_trace_run import Replay, read
    cfg, w, _, _ = truth["sup_a"]
    V = cfg["vocab"]
    reqs = {f"q{i}": random_ids(V, n, 500 + i) for i, n in enumerate([1, 2, 3, 5, 8, 13, 21, 34, 55, 70, 4, 1])}
    want = {k: plain.logits_all_positions(cfg, w, ids) for k, ids in reqs.items()}
    decode = 4
    fed = {k: max(1, len(ids) - decode) for k, ids in reqs.items()}
    rp = Replay(sup_dirs["sup_a"], "float32", tmp_path / "out", sum(len(v) for v in reqs.values()))
    f = rp.send([{"id": k, "tokens": ids[:fed[k]], "want": [fed[k] - 1]} for k, ids in reqs.items()],
                end=[k for k, ids in reqs.items() if fed[k] == len(ids)])
    got = read(f, V)
    for r, k in enumerate(reqs):
        assert float((got[r].double() - want[k][fed[k] - 1]).abs().max() / want[k].abs().max()) < TOL["float32"], (k, "prompt")
    live = [k for k, ids in reqs.items() if fed[k] < len(ids)]
    while live:
        f = rp.send([{"id": k, "tokens": [reqs[k][fed[k]]], "want": [0]} for k in live],
                    end=[k for k in live if fed[k] + 1 == len(reqs[k])])
        got = read(f, V)
        for r, k in enumerate(live):
            assert float((got[r].double() - want[k][fed[k]]).abs().max() / want[k].abs().max()) < TOL["float32"], (k, fed[k])
            fed[k] += 1
        live = [k for k in live if fed[k] < len(reqs[k])]
    rp.close()
