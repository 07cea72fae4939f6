"""Small Suposun configurations for the tests: every size differs from layer to layer and between the models, and what a
configuration could make equal by accident (query heads and key/value heads, query/key size and value size, rotated
dimensions and head size, one head, one bucket, a window of one block, kept tokens of more than a block, top = 1, top =
every expert, absent embedding section, absent scaling, mask, cap and feed-forward) is covered somewhere."""
import json
from pathlib import Path

import torch


def att(heads, kv_heads, dim, scale, rot_dims, base=10000.0, scaling=None, softcap=None, mask=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if softcap is not None:
        m["softcap"] = softcap
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]} if mask[1] is not None else {"size": mask[0]}
    return {"type": "attention", "mixer": m}


def att2(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"base": base, "dims": rot_dims}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


#: windows of 40 and 70 with 5 and no kept tokens, a window of exactly one block with a kept block; a layer that reads the
#: keys of the layer two before it; a layer without feed-forward; experts of which all are taken
SUP_A = {"architecture": "Suposun", "vocab": 311, "width": 96, "norm": {"eps": 1e-5}, "logit_scale": 0.7,
         "embedding": {"scale": 3.0, "bigram": {"buckets": 53, "mul_prev": 31, "mul_cur": 5}}, "layers": [
    layer(att(6, 2, 16, 0.3, 8, base=1000.0, scaling=(4.0, 64, 8.0, 2.0), softcap=8.0, mask=(40, 5)), moe(40, 1.2, 5, 2)),
    layer(att2(3, 3, 24, 16, 0.2, 24), dense(72)),
    layer(att(2, 1, 32, 0.18, 32, base=500.0, softcap=15.0, mask=(70, None)), None),
    layer(att2(3, 3, 24, 16, 0.25, 24, kv_from=1), moe(24, 0.8, 3, 3)),
    layer(att(4, 4, 8, 0.35, 4, mask=(64, 64)), dense(56)),
]}
#: no embedding section and no logit scale; the second kind first, with grouped heads and values larger than keys; an
#: attention without mask and without cap; kept tokens of more than a block under a window of 33; top = 1
SUP_B = {"architecture": "Suposun", "vocab": 257, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    layer(att2(4, 2, 16, 32, 0.25, 8, base=1e6), moe(32, 2.0, 6, 1)),
    layer(att(1, 1, 64, 0.125, 16, scaling=(8.0, 128, 16.0, 1.0)), dense(96)),
    layer(att2(4, 2, 16, 32, 0.2, 8, base=1e6, kv_from=0), None),
    layer(att(8, 2, 8, 0.4, 8, softcap=30.0, mask=(33, 70)), moe(48, 1.0, 4, 2)),
]}
#: sizes that are no multiples of 8 (the attention kernels of the CUDA cores); one bucket; a multiplier of zero; a window of 7
SUP_ODD = {"architecture": "Suposun", "vocab": 199, "width": 100, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
           "embedding": {"scale": 0.5, "bigram": {"buckets": 1, "mul_prev": 0, "mul_cur": 3}}, "layers": [
    layer(att(5, 1, 12, 0.28, 6, base=3000.0, scaling=(2.0, 32, 4.0, 1.0), softcap=5.0, mask=(7, 3)), moe(28, 1.4, 7, 3)),
    layer(att2(2, 1, 20, 28, 0.22, 10, base=700.0), dense(44)),
    layer(att(3, 3, 12, 0.3, 12, mask=(130, 1)), moe(36, 0.6, 2, 1)),
]}
#: attention made sharp (the query projections are drawn larger, see `write_model`) so that a wrong key, scale or mask
#: edge moves the logits by far more than rounding does; every feed-forward of experts takes all of them, so that no choice
#: rests on rounding and bfloat16 can be held against the plain implementation at every position
SUP_SHARP = {"architecture": "Suposun", "vocab": 307, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 2.5,
             "embedding": {"scale": 2.0, "bigram": {"buckets": 101, "mul_prev": 7, "mul_cur": 13}}, "layers": [
    layer(att(2, 1, 16, 0.25, 16, softcap=12.0, mask=(48, 9)), moe(64, 1.0, 3, 3)),
    layer(att2(4, 2, 8, 16, 0.35, 8), dense(80)),
    layer(att(4, 2, 16, 0.25, 8, scaling=(4.0, 32, 4.0, 1.0), softcap=25.0, mask=(100, 20)), moe(48, 2.0, 2, 2)),
    layer(att2(4, 2, 8, 16, 0.3, 8, kv_from=1), None),
]}
SHARP_FACTOR = 5.0
MODELS = {"sup_a": SUP_A, "sup_b": SUP_B, "sup_odd": SUP_ODD, "sup_sharp": SUP_SHARP}


def write_model(cfg: dict, seed: int, out_dir, sharp: float = 1.0, correction: float = 10.0) -> None:
    """The package's random draw for the configuration, the matrices that make queries multiplied by `sharp`, and the
    routers' corrections drawn `correction` times wider: ten times leaves fewer close calls between experts (see the
    plain `decided_prefix`) while the scores still take part in the choice; a hundred times lets the corrections decide
    alone, so that no choice rests on rounding and bfloat16 can be compared at every position."""
    import vlrf_b200.models  # noqa: F401
    from vlrf_b200.registry import parse_config
    from vlrf_b200.weights import write_safetensors
    arch, parsed = parse_config(cfg)
    tensors = arch.random_weights(parsed, torch.Generator().manual_seed(seed))
    for name in tensors:
        if name.endswith("mix.q"):
            tensors[name] = tensors[name] * sharp
        if name.endswith("mlp.correction"):
            tensors[name] = tensors[name] * correction
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    (Path(out_dir) / "config.json").write_text(json.dumps(cfg, indent=2))
    write_safetensors(Path(out_dir) / "model.safetensors",
                      {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in tensors.items()})
