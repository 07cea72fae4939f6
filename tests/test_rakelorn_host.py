"""Rakelorn without a GPU: its configuration, its tensor list, its schedule, what its layers keep in the cache, and the
plain implementation's own mechanisms on cases worked out by hand."""
import copy
import math

import pytest
import torch

import plain_rakelorn as plain
from rakelorn_models import MODELS, RAK_A, RAK_B, RAK_ODD, RAK_SHARP, write_model


def test_config_json_selects_the_architecture_and_reads_every_layer():
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.config.rakelorn import RecurrenceConfig
    from vlrf_b200.registry import parse_config
    arch, cfg = parse_config(RAK_A)
    assert arch.name == "Rakelorn" and cfg.n_layer == 4 and cfg.embedding_scale == 3.0 and cfg.norm_eps == 1e-5
    assert isinstance(cfg.mixers[1], RecurrenceConfig) and cfg.mixers[1].width == 112
    assert cfg.mixers[2].rot_dim == 16 and cfg.mixers[2].rot_dims == 8 and cfg.mixers[2].rot_base == 500.0 and cfg.mixers[0].q_rank == 56
    assert cfg.mlps[2] is None and (cfg.mlps[0].experts, cfg.mlps[0].identity, cfg.mlps[0].groups, cfg.mlps[0].keep) == (6, 2, 4, 2)
    assert cfg.mlps[3].identity == 0 and cfg.mlps[3].scale == 0.7
    assert cfg.layer_order == [0, 1, 2, 1, 2, 3] and cfg.pass_begins == [None, 0, None, 1, None, None]
    assert cfg.to_dict() == RAK_A
    _, b = parse_config(RAK_B)
    assert b.embedding_scale == 1.0 and b.layer_order == [0, 1, 2, 3] and b.pass_begins == [None] * 4 and b.loop_times == 0
    _, o = parse_config(RAK_ODD)
    assert o.layer_order == [0, 1] * 3 and o.pass_begins == [0, None, 1, None, 2, None]
    _, s = parse_config(RAK_SHARP)
    assert s.layer_order == [0, 1, 2] and s.pass_begins == [None, None, 0]


@pytest.mark.parametrize("edit,text", [
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),            # two kept groups of two
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=5), "groups"),
    (lambda c: c["layers"][1]["mixer"].pop("width"), "width"),
    (lambda c: c["layers"][2]["mixer"].pop("q_rank"), "q_rank"),
    (lambda c: c["loop"].update(stop=5), "loop"),
    (lambda c: c["loop"].update(times=0), "loop"),
    (lambda c: c["norm"].pop("eps"), "eps"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_configurations_that_describe_no_model_are_refused(edit, text):
    from vlrf_b200.config.base import ConfigError
    from vlrf_b200.registry import parse_config
    cfg = copy.deepcopy(RAK_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=text):
        parse_config(cfg)


def test_tensor_list_follows_the_layers(tmp_path):
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights.model_dir import open_model_dir
    arch, cfg = parse_config(RAK_A)
    names = {s.name: s for s in arch.weight_spec(cfg)}
    assert tuple(names["loop.step"].shape) == (2, 96) and tuple(names["l0.norm1"].shape) == () and tuple(names["final.norm"].shape) == ()
    assert tuple(names["l0.mix.g"].shape) == (3, 96) and tuple(names["l0.mix.dkv"].shape) == (48, 96) and tuple(names["l0.mix.uq"].shape) == (72, 56)
    assert tuple(names["l1.mix.z"].shape) == (112, 96) and tuple(names["l1.mix.o"].shape) == (96, 112) and "l1.mix.dq" not in names
    assert tuple(names["l0.mlp.router"].shape) == (8, 96) and "l0.mlp.e5.down" in names and "l0.mlp.e6.up" not in names
    assert names["l2.norm2"].optional and "l2.mlp.router" not in names and tuple(names["l3.mlp.correction"].shape) == (4,)
    write_model(RAK_A, 3, tmp_path)
    arch2, _, checked = open_model_dir(tmp_path)
    assert arch2.name == "Rakelorn" and set(checked.tensors) == set(names) - {"l2.norm2"}
    arch_b, cfg_b = parse_config(RAK_B)
    names_b = {s.name for s in arch_b.weight_spec(cfg_b)}
    assert "loop.step" not in names_b and "l1.mlp.router" in names_b and "l1.mlp.e0.up" not in names_b


def test_what_the_layers_keep_and_the_schedule(tmp_path):
    """Every layer run has an entry of its own: the mixer's need and, behind it, the row of the first norm's token shift."""
    from vlrf_b200.cache import LatentNeed, SequenceCache, StateNeed
    from vlrf_b200.engine.model import BuildOptions
    from vlrf_b200.weights.model_dir import open_model_dir
    write_model(RAK_A, 5, tmp_path)
    arch, cfg, weights = open_model_dir(tmp_path)
    model = arch.build(cfg, weights, BuildOptions(torch.float32, torch.device("cpu")))     # (parts only; nothing runs)
    needs = model.cache_needs()
    assert [c.layer for c in model.schedule] == [0, 1, 2, 1, 2, 3]
    assert [c.add_before is not None for c in model.schedule] == [False, True, False, True, False, False]
    assert not torch.equal(model.schedule[1].add_before, model.schedule[3].add_before)
    shift = StateNeed((2, 96), torch.float32)
    assert needs[0] == (LatentNeed(40 + 8), shift) and needs[1] == (StateNeed((2, 112), torch.float32), shift) == needs[3]
    assert needs[2] == (LatentNeed(48 + 16), shift) == needs[4]
    cache = SequenceCache(needs, max_tokens=256, max_seq_len=512, dtype=torch.float32, device="cpu")
    v1, v3 = cache.view(1), cache.view(3)
    assert len(v1.parts) == 2 and v1.parts[0].state.shape[1:] == (2, 112) and v1.parts[1].state.shape[1:] == (2, 96)
    assert v1.parts[0].state.data_ptr() != v3.parts[0].state.data_ptr() and v1.parts[1].state.data_ptr() != v3.parts[1].state.data_ptr()
    assert cache.view(0).parts[1].state.data_ptr() not in (v1.parts[1].state.data_ptr(), v3.parts[1].state.data_ptr())
    assert model.replayable


# ---- the plain implementation's mechanisms on cases worked out by hand ------------------------------------------------

def test_plain_token_shift_and_norm():
    h = torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0]], dtype=torch.float64)
    mu = torch.tensor([0.0, 1.0], dtype=torch.float64)
    assert torch.equal(plain.token_shift(h, mu), torch.tensor([[1.0, 0.0], [3.0, 2.0], [5.0, 4.0]], dtype=torch.float64))
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(plain.scalar_rms_norm(x, 2.0, 0.0), x / math.sqrt(12.5) * 2.0)
    assert float(plain.scalar_rms_norm(torch.zeros(1, 2, dtype=torch.float64), 2.0, 1e-6).abs().max()) == 0.0


def test_plain_rotation_pairs_neighbours():
    v = torch.tensor([[1.0, 0.0, 0.0, 1.0, 7.0, 9.0]], dtype=torch.float64)
    out = plain.rotate_pairs(v, torch.tensor([2]), 100.0, 4)
    a0, a1 = 2.0, 2.0 * 100.0 ** -0.5
    want = [math.cos(a0), math.sin(a0), -math.sin(a1), math.cos(a1), 7.0, 9.0]
    assert torch.allclose(out[0], torch.tensor(want, dtype=torch.float64))
    assert torch.equal(plain.rotate_pairs(v, torch.tensor([0]), 100.0, 4), v)


def test_plain_recurrence_written_out():
    z = torch.tensor([[0.5], [0.25], [1.0]], dtype=torch.float64)
    c = torch.tensor([[2.0], [4.0], [-1.0]], dtype=torch.float64)
    S = plain.mingru_scan(z, c)
    assert torch.allclose(S[:, 0], torch.tensor([1.0, 0.75 * 1.0 + 1.0, -1.0], dtype=torch.float64))
    w = {"z": torch.zeros(1, 1), "z.b": torch.zeros(1), "x": torch.ones(1, 1), "x.b": torch.zeros(1), "g": torch.ones(1, 1), "o": torch.ones(1, 1)}
    w = {k: v.double() for k, v in w.items()}
    out = plain.mingru(torch.tensor([[1.0], [-1.0]], dtype=torch.float64), w, "")
    sig = lambda v: 1.0 / (1.0 + math.exp(-v))
    s0 = 0.5 * 1.5
    s1 = 0.5 * s0 + 0.5 * sig(-1.0)
    assert torch.allclose(out[:, 0], torch.tensor([s0 * 1.0 * sig(1.0), s1 * -1.0 * sig(-1.0)], dtype=torch.float64))


def test_plain_routing_by_groups_correction_and_identity():
    r = {"experts": 4, "identity": 2, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    z = torch.log(torch.tensor([[0.05, 0.30, 0.25, 0.20, 0.15, 0.05]], dtype=torch.float64))
    s = torch.softmax(z, -1)
    # without a correction group 1 (0.25, 0.20) loses to group 0 (0.05, 0.30): the group's best counts, not its sum
    ids, wts = plain.route(z, torch.zeros(6, dtype=torch.float64), r)
    assert ids == [[1, 0]] and wts[0] == pytest.approx([0.6, 0.1])
    # the correction moves the choice and not the weights; a negative choice score still beats a dropped group's
    corr = torch.tensor([0.0, -0.5, 0.0, 0.0, 0.2, -0.3], dtype=torch.float64)
    ids, wts = plain.route(z, corr, r)
    assert ids == [[4, 5]] and wts[0] == pytest.approx([2 * float(s[0, 4]), 2 * float(s[0, 5])])
    # identity experts return their input, times the weight
    w = {"router": torch.zeros(6, 3, dtype=torch.float64), "correction": corr}
    h = torch.tensor([[1.0, -2.0, 0.5]], dtype=torch.float64)
    ml = {"router": dict(r, groups={"count": 3, "keep": 1})}
    out = plain.routed_ff(h, w, "", ml)                      # z = 0: s = 1/6 everywhere, group 2 wins by the correction
    assert torch.allclose(out, h * (2.0 / 6.0) * 2)
    # ties go to the lower index
    ids, _ = plain.route(torch.zeros(1, 6, dtype=torch.float64), torch.zeros(6, dtype=torch.float64), r)
    assert ids == [[0, 1]]


def test_plain_schedule_and_layers_kept(tmp_path):
    assert plain.schedule(RAK_A) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    assert plain.schedule(RAK_B) == [(i, None) for i in range(4)]
    assert plain.schedule(RAK_SHARP) == [(0, None), (1, None), (2, 0)]
    write_model(RAK_SHARP, 9, tmp_path)
    cfg, w = plain.read_model_dir(tmp_path)
    logits, layers = plain.forward(cfg, w, [5, 6, 7, 8], keep_layers=True)
    assert layers.shape == (3, 4, 64) and logits.shape == (4, 311)
    # a token sees nothing behind it
    again = plain.forward(cfg, w, [5, 6, 7, 9])
    assert torch.equal(again[:3], logits[:3]) and not torch.equal(again[3], logits[3])
    # the vector before a pass counts: without it the logits move
    w2 = dict(w)
    w2["loop.step"] = torch.zeros_like(w["loop.step"])
    assert float((plain.forward(cfg, w2, [5, 6, 7, 8]) - logits).abs().max()) > 1e-3
