"""Rakelorn configurations drawn at random (every size, count, constant and the order of layers from a seeded generator;
keys that may be absent are absent now and then) through the engine against the plain implementation: whole, the last
tokens one by one, prompts in portions and an unequal batch.  What the hand-made models happen not to combine shows here:
larger widths and heads, routers with many outputs, loops over any range, layers of one kind only.

The 32-bit comparison covers every position.  In bfloat16 only the positions before a router's first close call are
held against the plain implementation, with a wide bound: it is there to show a kernel of the bfloat16 path that a size
sends wrong, not to grade rounding."""
import random

import pytest

import plain_rakelorn as plain
from conftest import random_ids
from engine_drives import drive_batches, drive_portions, drive_tail_one_by_one, drive_whole
from rakelorn_models import att, gru, layer, moe, write_model
from test_rakelorn import compare, poison_states

pytestmark = pytest.mark.gpu


def draw_router(r: random.Random) -> dict | None:
    if r.random() < 0.12:
        return None
    count = r.choice([1, 1, 2, 3, 4, 8])
    per = r.choice([1, 2, 3, 4, 5, 9])
    n_out = count * per
    keep = r.randint(1, count)
    identity = r.choice([0, 0, 1, 2, n_out]) if n_out <= 6 else r.choice([0, 1, 2, 3, 5])
    identity = min(identity, n_out)
    top = r.randint(1, min(keep * per, 6))
    return moe(r.choice([24, 40, 64, 96, 136, 200]), n_out - identity, identity, top, count, keep, r.choice([0.5, 1.0, 2.0, 2.5]))


def draw_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([48, 64, 72, 100, 128, 160, 192, 256, 320, 384])
    cfg = {"architecture": "Rakelorn", "vocab": r.choice([97, 200, 333, 512, 777, 1500]), "width": width,
           "norm": {"eps": r.choice([1e-5, 1e-6, 1e-4])}}
    if r.random() < 0.8:
        cfg["embedding"] = {"scale": r.choice([0.7, 1.0, 2.5, 8.0, 16.0])}
    n_layers = r.choice([1, 2, 3, 4, 5])
    kinds = r.choice(["mixed", "mixed", "mixed", "attention", "recurrence"])
    layers = []
    for _ in range(n_layers):
        if kinds == "recurrence" or (kinds == "mixed" and r.random() < 0.45):
            mixer = gru(r.choice([32, 52, 64, 100, 128, 256, 300, 512, width]))
        else:
            dim = r.choice([8, 12, 16, 24, 32, 48, 64, 96, 128])
            rot_dim = r.choice([2, 4, 6, 8, 16, 32, 64])
            half = rot_dim // 2
            rot_dims = r.choice([rot_dim, rot_dim, rot_dim, half if half >= 2 and half % 2 == 0 else rot_dim])
            mixer = att(r.choice([1, 2, 3, 4, 6, 8, 12]), dim, rot_dim, r.choice([8, 16, 20, 32, 48, 64, 128]),
                        r.choice([16, 24, 40, 64, 96, 128, 192]), r.choice([16, 24, 48, 72, 128, 160]),
                        round((dim + rot_dim) ** -0.5 * r.choice([0.8, 1.0, 1.4]), 4), base=r.choice([100.0, 10000.0, 1e6]), rot_dims=rot_dims)
        layers.append(layer(mixer, draw_router(r)))
    cfg["layers"] = layers
    if r.random() < 0.75:
        a = r.randrange(0, n_layers)
        b = r.randrange(a + 1, n_layers + 1)
        cfg["loop"] = {"start": a, "stop": b, "times": r.choice([1, 2, 2, 3, 4])}
    return cfg


@pytest.mark.parametrize("seed", range(14))
def test_a_random_model_whole_decoded_in_portions_and_batched(tmp_path, seed):
    from vlrf_b200.engine import Engine, load_model
    cfg = draw_config(2000 + seed)
    write_model(cfg, seed, tmp_path)
    pc, w = plain.read_model_dir(tmp_path)
    reqs = [random_ids(cfg["vocab"], n, 37 * seed + i) for i, n in enumerate((1 + seed % 3, 66 + 5 * seed, 141))]
    want = [plain.logits_all_positions(pc, w, ids) for ids in reqs]
    decided = [plain.decided_prefix(pc, w, ids) for ids in reqs]
    for dtype in ("float32", "bfloat16"):
        eng = Engine(load_model(tmp_path, dtype), max_tokens=512)
        poison_states(eng)
        name = f"random {seed}"
        compare(drive_whole(eng, reqs), want, dtype, "whole", name, decided)
        compare(drive_tail_one_by_one(eng, reqs, 36), want, dtype, "prefix + 36 single tokens", name, decided)
        compare(drive_portions(eng, reqs, 2 + seed % 9), want, dtype, "portions", name, decided)
        poison_states(eng)
        compare(drive_batches(eng, reqs, 3, [1, 33, 100]), want, dtype, "unequal batch", name, decided)
        assert eng.cache.slots.n_held == 0
