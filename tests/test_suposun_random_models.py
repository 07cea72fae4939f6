"""Suposun configurations drawn at random (every size, count, constant and the order of layers from a seeded generator;
keys that may be absent are absent now and then) through the engine against the plain implementation: whole, the last
tokens one by one, prompts in portions and an unequal batch.  What the hand-made models happen not to combine shows here:
larger widths and heads, windows around the requests' lengths, kept tokens beyond the window, layers of one kind only,
several layers reading one layer's keys.

The 32-bit comparison covers every position.  In bfloat16 only the positions before a router's first close call are
held against the plain implementation; every other configuration is therefore drawn with corrections so wide that they
alone decide the choice of experts, and is compared at every position in bfloat16 too."""
import random

import pytest

import plain_suposun as plain
from conftest import random_ids
from engine_drives import drive_batches, drive_portions, drive_tail_one_by_one, drive_whole
from suposun_models import att, att2, dense, layer, moe, write_model
from test_suposun import compare, poison_states

pytestmark = pytest.mark.gpu


def draw_mlp(r: random.Random):
    x = r.random()
    if x < 0.12:
        return None
    if x < 0.5:
        return dense(r.choice([24, 40, 64, 100, 136, 304]))
    experts = r.choice([1, 2, 3, 4, 6, 11, 17, 40])
    return moe(r.choice([24, 40, 64, 96, 136]), r.choice([0.5, 1.0, 1.5, 3.0, 7.0]), experts, r.randint(1, min(experts, 6)))


def draw_config(seed: int) -> dict:
    r = random.Random(seed)
    width = r.choice([48, 64, 72, 100, 128, 160, 192, 256, 320, 384])
    cfg = {"architecture": "Suposun", "vocab": r.choice([97, 200, 333, 512, 777, 1500]), "width": width,
           "norm": {"eps": r.choice([1e-5, 1e-6, 1e-4])}}
    if r.random() < 0.8:
        cfg["logit_scale"] = r.choice([0.5, 1.0, 2.0, 3.7])
    if r.random() < 0.85:
        cfg["embedding"] = {}
        if r.random() < 0.85:
            cfg["embedding"]["scale"] = r.choice([0.7, 1.0, 2.5, 8.0, 16.0])
        if r.random() < 0.8:
            cfg["embedding"]["bigram"] = {"buckets": r.choice([1, 7, 64, 521, 4099]), "mul_prev": r.choice([0, 1, 131, 100003]),
                                          "mul_cur": r.choice([0, 1, 5, 31])}
    n_layers = r.choice([1, 2, 3, 4, 5, 6])
    kinds = r.choice(["mixed", "mixed", "mixed", "attention", "attention_2"])
    layers, owners = [], {}
    for i in range(n_layers):
        first = kinds == "attention" or (kinds == "mixed" and r.random() < 0.55)
        if first:
            dim = r.choice([8, 12, 16, 24, 32, 48, 64, 96, 128])
            kv = r.choice([1, 1, 2, 3, 4])
            heads = kv * r.choice([1, 2, 4, 6])
            rot = r.choice([d for d in (2, 4, 6, 8, 16, 32, 64, 128) if d <= dim])
            scaling = (r.choice([2.0, 8.0, 32.0]), r.choice([16, 64, 1024]), r.choice([4.0, 24.0]), r.choice([0.5, 1.0, 2.0])) if r.random() < 0.7 else None
            mask = None
            if r.random() < 0.85:
                mask = (r.choice([1, 5, 31, 64, 65, 100, 128, 140, 200]), r.choice([None, 0, 1, 24, 64, 70, 150]))
            mixer = att(heads, kv, dim, round(dim ** -0.5 * r.choice([0.8, 1.0, 1.4]), 4), rot, base=r.choice([100.0, 10000.0, 1e6]),
                        scaling=scaling, softcap=r.choice([None, 5.0, 18.0, 50.0]), mask=mask)
        else:
            if owners and r.random() < 0.45:
                j = r.choice(list(owners))
                mixer = att2(*owners[j][:4], round(owners[j][4] * r.choice([0.9, 1.0, 1.2]), 4), *owners[j][5:], kv_from=j)
            else:
                dim = r.choice([8, 12, 16, 20, 32, 64, 128])
                kv = r.choice([1, 2, 4])
                heads = kv * r.choice([1, 1, 2, 4])
                rot = r.choice([d for d in (2, 4, 8, 16, 20, 32, 64, 128) if d <= dim and d % 2 == 0])
                shape = (heads, kv, dim, r.choice([8, 16, 20, 32, 64, 128]), round(dim ** -0.5 * r.choice([0.8, 1.0, 1.4]), 4), rot,
                         r.choice([100.0, 10000.0, 1e6]))
                owners[i] = shape
                mixer = att2(*shape)
        layers.append(layer(mixer, draw_mlp(r)))
    cfg["layers"] = layers
    return cfg


@pytest.mark.parametrize("seed", range(14))
def test_a_random_model_whole_decoded_in_portions_and_batched(tmp_path, seed):
    from vlrf_b200.engine import Engine, load_model
    cfg = draw_config(3000 + seed)
    write_model(cfg, seed, tmp_path, correction=100.0 if seed % 2 else 10.0)
    pc, w = plain.read_model_dir(tmp_path)
    reqs = [random_ids(cfg["vocab"], n, 37 * seed + i) for i, n in enumerate((1 + seed % 3, 66 + 5 * seed, 141, 230))]
    want = [plain.logits_all_positions(pc, w, ids) for ids in reqs]
    decided = [plain.decided_prefix(pc, w, ids) for ids in reqs]
    for dtype in ("float32", "bfloat16"):
        eng = Engine(load_model(tmp_path, dtype), max_tokens=768)
        poison_states(eng)
        name = f"random {seed}"
        compare(drive_whole(eng, reqs), want, dtype, "whole", name, decided)
        compare(drive_tail_one_by_one(eng, reqs, 36), want, dtype, "prefix + 36 single tokens", name, decided)
        compare(drive_portions(eng, reqs, 2 + seed % 9), want, dtype, "portions", name, decided)
        poison_states(eng)
        compare(drive_batches(eng, reqs, 4, [1, 33, 100, 199]), want, dtype, "unequal batch", name, decided)
        assert eng.cache.slots.n_held == 0
