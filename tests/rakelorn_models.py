"""Small Rakelorn configurations for the tests: every size differs from layer to layer and between the models, and what
a configuration could make equal by accident (the recurrence's width and the model's, query/key size and value size,
rotated size and rotated dimensions, one head, one group, every group kept, top = 1, top = every allowed expert, no
identity expert, nothing but identity experts, a loop over all layers, over one layer once, none) is covered somewhere."""
import json
from pathlib import Path

import torch


def att(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, rot_dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                      "scale": scale, "rot": {"base": base, "dims": rot_dims or rot_dim}}}


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def moe(ff, experts, identity, top, count, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}, "scale": scale}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


#: the loop covers the two middle layers (a recurrence wider than the model, an attention without feed-forward); groups of
#: two and of three, of which some are dropped; rotated dimensions fewer than the rotated size
RAK_A = {"architecture": "Rakelorn", "vocab": 301, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
         "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    layer(att(3, 16, 8, 24, 40, 56, 0.2), moe(48, 6, 2, 3, 4, 2, 1.5)),
    layer(gru(112), moe(40, 5, 1, 2, 3, 1, 2.5)),
    layer(att(5, 8, 16, 16, 48, 32, 0.3, base=500.0, rot_dims=8), None),
    layer(att(2, 32, 8, 8, 24, 72, 0.18), moe(56, 4, 0, 1, 1, 1, 0.7)),
]}
#: neither a loop nor an embedding scale; one head; a recurrence first; a feed-forward of identity experts only; top = 1
RAK_B = {"architecture": "Rakelorn", "vocab": 257, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    layer(gru(64), moe(32, 8, 0, 1, 2, 2, 1.0)),
    layer(att(1, 64, 32, 32, 64, 48, 0.11, base=1e6), moe(24, 0, 3, 2, 1, 1, 3.0)),
    layer(gru(128), None),
    layer(att(6, 16, 16, 8, 96, 40, 0.25, base=1000.0), moe(64, 3, 3, 2, 3, 2, 0.9)),
]}
#: sizes that are no multiples of 8; the loop covers every layer, three times
RAK_ODD = {"architecture": "Rakelorn", "vocab": 199, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 0.5},
           "loop": {"start": 0, "stop": 2, "times": 3}, "layers": [
    layer(att(3, 12, 6, 20, 36, 30, 0.21, base=3000.0), moe(28, 4, 2, 3, 2, 1, 1.7)),
    layer(gru(52), moe(44, 7, 2, 2, 3, 2, 1.0)),
]}
#: attention made sharp (the query projections are drawn larger, see `write_model`) so that a wrong key, scale or mask
#: edge moves the logits by far more than rounding does; every feed-forward takes all the experts it may choose from, so
#: that no choice rests on rounding and bfloat16 can be held against the plain implementation at every position; the
#: loop runs its one layer once (its vector is still added)
RAK_SHARP = {"architecture": "Rakelorn", "vocab": 311, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
             "loop": {"start": 2, "stop": 3, "times": 1}, "layers": [
    layer(att(2, 16, 16, 16, 32, 40, 0.25), moe(96, 2, 1, 3, 1, 1, 0.5)),
    layer(gru(64), None),
    layer(att(4, 8, 16, 8, 32, 24, 0.3, rot_dims=16), moe(64, 3, 1, 4, 2, 2, 0.4)),
]}
SHARP_FACTOR = 6.0
MODELS = {"rak_a": RAK_A, "rak_b": RAK_B, "rak_odd": RAK_ODD, "rak_sharp": RAK_SHARP}


def write_model(cfg: dict, seed: int, out_dir, sharp: float = 1.0, head: float = 1.0) -> None:
    """The package's random draw for the configuration, the matrices that make queries multiplied by `sharp`, the router
    matrices by 4 (fewer close calls between experts, see the plain `decided_prefix`) and the head by `head`."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights import write_safetensors
    arch, parsed = parse_config(cfg)
    tensors = arch.random_weights(parsed, torch.Generator().manual_seed(seed))
    for name in tensors:
        if name.endswith("mix.uq"):
            tensors[name] = tensors[name] * sharp
        if name.endswith("mlp.router"):
            tensors[name] = tensors[name] * 4.0
        if name == "head":
            tensors[name] = tensors[name] * head
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    (Path(out_dir) / "config.json").write_text(json.dumps(cfg, indent=2))
    write_safetensors(Path(out_dir) / "model.safetensors",
                      {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in tensors.items()})
