"""Suposun without a GPU: the configuration reader (every key read, absent keys, refusals), the tensor list, what every
layer keeps and whose keys it reads, the cache's kept first blocks, and the plain functions' own edge cases."""
import copy
import math

import pytest
import torch

import plain_suposun as plain
from suposun_models import MODELS, SUP_A, SUP_B, SUP_ODD


def parse(cfg):
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    return parse_config(cfg)


def test_every_key_is_read():
    arch, c = parse(SUP_A)
    assert arch.name == "Suposun" and (c.vocab, c.width, c.norm_eps, c.logit_scale, c.embedding_scale) == (311, 96, 1e-5, 0.7, 3.0)
    assert (c.bigram.buckets, c.bigram.mul_prev, c.bigram.mul_cur) == (53, 31, 5)
    m = c.mixers[0]
    assert (m.kind, m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.rot_base, m.rot_dims) == ("attention", 6, 2, 16, 16, 0.3, 1000.0, 8)
    assert m.rot_scaling == (4.0, 64.0, 8.0, 2.0) and (m.softcap, m.window, m.keep_first) == (8.0, 40, 5)
    assert (c.mixers[2].window, c.mixers[2].keep_first, c.mixers[2].rot_scaling) == (70, 0, None)
    assert c.mixers[3].kv_from == 1 and c.mixers[1].kv_from is None and c.mixers[1].vdim == 16
    assert (c.mlps[0].kind, c.mlps[0].ff, c.mlps[0].limit, c.mlps[0].experts, c.mlps[0].top) == ("moe", 40, 1.2, 5, 2)
    assert (c.mlps[1].kind, c.mlps[1].ff) == ("dense", 72) and c.mlps[2] is None


def test_absent_keys():
    _, c = parse(SUP_B)
    assert c.bigram is None and c.embedding_scale == 1.0 and c.logit_scale == 1.0
    assert (c.mixers[1].window, c.mixers[1].softcap) == (0, None)


@pytest.mark.parametrize("change,where", [
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=24), "vdim"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=0.0), "softcap"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_heads=1), "differ"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].update(limit=0.0), "limit"),
    (lambda c: c["layers"][1]["mlp"].update(kind="gated"), "kind"),
    (lambda c: c["layers"][1].update(type="attention_3"), "type"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "buckets"),
    (lambda c: c["norm"].update(eps=0.0), "eps"),
])
def test_refusals(change, where):
    from vlrf_b200.config import ConfigError
    cfg = copy.deepcopy(SUP_A)
    change(cfg)
    with pytest.raises(ConfigError, match=where):
        parse(cfg)


def test_tensor_list():
    arch, c = parse(SUP_A)
    spec = {s.name: tuple(s.shape) for s in arch.weight_spec(c) if not s.optional}
    assert spec["embed"] == (311, 96) and spec["bigram"] == (54, 96) and spec["final.norm"] == (96,)
    assert spec["l0.mix.q"] == (96, 96) and spec["l0.mix.k"] == (32, 96) and "l0.mix.v" not in spec
    assert spec["l0.mix.q.norm"] == (16,) and spec["l0.mix.k.norm"] == (16,) and spec["l0.mix.sink"] == (6,) and spec["l0.mix.g"] == (6, 96)
    assert spec["l1.mix.q.norm"] == (72,) and spec["l1.mix.k.norm"] == (72,) and spec["l1.mix.v"] == (48, 96) and spec["l1.mix.o"] == (96, 48)
    assert "l3.mix.k" not in spec and "l3.mix.v" not in spec and "l3.mix.k.norm" not in spec and spec["l3.mix.q.norm"] == (72,)
    assert spec["l0.mlp.e4.down"] == (96, 40) and spec["l0.mlp.router"] == (5, 96) and spec["l0.mlp.correction"] == (5,)
    assert "l2.norm2" not in spec and "l2.ls2" not in spec and spec["l2.ls1"] == (96,)
    _, b = parse(SUP_B)
    assert "bigram" not in {s.name for s in arch.weight_spec(b)}
    drawn = arch.random_weights(c, torch.Generator().manual_seed(1))
    assert set(drawn) == set(spec) and all(tuple(drawn[n].shape) == sh for n, sh in spec.items())


def test_cache_keeps_the_first_blocks_of_a_window():
    """A window need with keep_first: the blocks that hold them stay while later ones behind the window go back."""
    from vlrf_b200.cache import KVNeed, SequenceCache
    need = KVNeed(2, 8, "window", 33, keep_first=70)
    c = SequenceCache([need, KVNeed(2, 8, "window", 33)], max_tokens=64 * 12, max_seq_len=4096, dtype=torch.float32, device="cpu")
    s = c.acquire()
    c.reserve(s, 500)
    c.advance(s, 500)
    kept, plain_window = c._groups[0], c._groups[1]
    assert [i for i, b in enumerate(kept.table_host[s]) if b >= 0] == [0, 1, 7]
    assert [i for i, b in enumerate(plain_window.table_host[s]) if b >= 0] == [7]
    for n in range(60):
        c.reserve(s, 501 + n)
        c.advance(s, 1)
    assert [i for i, b in enumerate(kept.table_host[s]) if b >= 0] == [0, 1, 8]
    c.check()
    c.release(s)
    c.check()
    assert kept.pool.n_held == 0
    with pytest.raises(Exception):
        SequenceCache([KVNeed(2, 8, "full", 0, keep_first=3)], max_tokens=64, max_seq_len=64, dtype=torch.float32, device="cpu")


def test_what_layers_keep_and_read():
    """The need of every layer as the model states it, without a GPU: built from the parts' constructors."""
    from vlrf_b200.cache import KVNeed
    from vlrf_b200.parts import get_part
    att = get_part("mixer", "window_attention")
    w = torch.zeros
    own = att(w(24, 10), w(8, 10), None, w(10, 24), n_heads=3, n_kv_heads=1, dim=8, vdim=8, scale=1.0, window=9, keep_first=2,
              sink=w(3), w_gate=w(3, 10), qk_norm="head", q_norm=w(8), k_norm=w(8), norm_eps=1e-5, softcap=4.0)
    assert own.cache_need() == KVNeed(1, 8, "window", 9, keep_first=2) and own.in_width == 24 + 8 + 3 and own.v_off == own.k_off
    reader = att(w(24, 10), None, None, w(10, 12), n_heads=3, n_kv_heads=1, dim=8, vdim=4, scale=1.0, qk_norm="all", q_norm=w(24),
                 norm_eps=1e-5)
    assert reader.cache_need() == KVNeed(1, 8, "full", 0, v_dim=4) and reader.in_width == 24 and not reader.own_kv
    with pytest.raises(ValueError):
        att(w(24, 10), w(8, 10), None, w(10, 24), n_heads=3, n_kv_heads=1, dim=8, vdim=8, scale=1.0, keep_first=2)   # no window
    with pytest.raises(ValueError):
        att(w(24, 10), w(8, 10), None, w(10, 12), n_heads=3, n_kv_heads=1, dim=8, vdim=4, scale=1.0)                  # values are keys


def test_norm_offset_and_scale_fold_into_one_factor():
    from vlrf_b200.parts import get_part
    w, ls = torch.tensor([0.25, -0.5, 0.0]), torch.tensor([2.0, 0.5, -1.0])
    n = get_part("norm", "group_rmsnorm")(w, 1e-5, 1, offset=1.0, post_scale=ls)
    assert torch.equal(n.weight, torch.tensor([2.5, 0.25, -1.0])) and n.stored_weight is w
    assert get_part("norm", "group_rmsnorm")(w, 1e-5).weight is w


def test_rotation_table_of_the_part_matches_the_plain_one():
    from vlrf_b200.parts import get_part
    rot = {"base": 1000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}}
    f, mag = plain.rotary_frequencies(rot)
    part = get_part("position", "rotary")(1000.0, 16, "cpu", yarn=(4.0, 64, 8.0, 2.0), pairing="interleaved")
    assert torch.allclose(part.inv_freq.double(), torch.tensor(f, dtype=torch.float64), rtol=1e-6) and part.magnitude == pytest.approx(mag) and part.interleaved
    # the fastest pair is untouched, the slowest is slowed by the whole factor, and one between is blended
    base = [1000.0 ** (-2.0 * i / 16) for i in range(8)]
    assert f[0] == base[0] and f[-1] == pytest.approx(base[-1] / 4.0) and any(b / 4.0 < x < b for x, b in zip(f, base))
    assert mag == pytest.approx(0.1 * math.log(4.0) + 1.0)
    assert plain.rotary_frequencies({"base": 10.0, "dims": 4}) == ([1.0, 10.0 ** -0.5], 1.0)


def test_plain_visibility_and_sink():
    mask = {"size": 4, "keep_first": 2}
    assert [j for j in range(10) if plain.visible(9, j, mask)] == [0, 1, 6, 7, 8, 9]
    assert [j for j in range(4) if plain.visible(2, j, mask)] == [0, 1, 2]
    assert [j for j in range(10) if plain.visible(9, j, {"size": 4})] == [6, 7, 8, 9]
    assert all(plain.visible(9, j, None) for j in range(10))
    # one key, one head: the weight of the only key is 1 / (1 + exp(sink − score))
    q, k, v = torch.ones(1, 1, 2, dtype=torch.float64), torch.ones(1, 1, 2, dtype=torch.float64), torch.tensor([[[3.0, 5.0]]], dtype=torch.float64)
    out = plain.attend(q, k, v, 0.5, sink=torch.tensor([2.0], dtype=torch.float64))
    assert torch.allclose(out[0, 0], v[0, 0] / (1.0 + math.exp(2.0 - 1.0)))
    capped = plain.attend(q * 100, k, v, 0.5, softcap=3.0, sink=torch.tensor([3.0], dtype=torch.float64))
    assert torch.allclose(capped[0, 0], v[0, 0] / (1.0 + math.exp(3.0 - 3.0 * math.tanh(100.0 / 3.0))))


def test_plain_bigram_rows_and_router():
    assert plain.bigram_rows([5, 7, 7, 0], 11, 3, 2).tolist() == [11, (15 + 14) % 11, (21 + 14) % 11, 21 % 11]
    w = {"r.router": torch.tensor([[1.0], [2.0], [-1.0]], dtype=torch.float64), "r.correction": torch.tensor([0.0, -0.9, 0.5], dtype=torch.float64)}
    idx, wt = plain.route(torch.tensor([[1.0]], dtype=torch.float64), w, "r.", {"router": {"top": 2}})
    s = torch.sigmoid(torch.tensor([1.0, 2.0, -1.0], dtype=torch.float64))
    # the correction changes who is chosen (expert 1 has the best score and loses), never the weights
    assert idx.tolist() == [[2, 0]] and torch.allclose(wt[0], s[[2, 0]])
    e = {"e.gate": torch.tensor([[4.0]], dtype=torch.float64), "e.up": torch.tensor([[-4.0]], dtype=torch.float64), "e.down": torch.tensor([[1.0]], dtype=torch.float64)}
    assert plain.expert(torch.tensor([[1.0]], dtype=torch.float64), e, "e.", 1.5).item() == pytest.approx(1.5 / (1 + math.exp(-1.702 * 1.5)) * (-1.5 + 1.0))


def test_configurations_differ():
    sizes = [(c["width"], c["vocab"], len(c["layers"])) for c in MODELS.values()]
    assert len(set(sizes)) == len(sizes) and SUP_ODD["embedding"]["bigram"]["buckets"] == 1
