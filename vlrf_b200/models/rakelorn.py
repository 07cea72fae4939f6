"""Rakelorn: a decoder of latent-attention and minGRU layers with routed feed-forwards, a token shift ahead of every
mixer, norms with a single weight, and a range of layers that runs several times.

Tensors (all linear weights [out, in]): `embed` [vocab, width]; `loop.step` [times, width] (with a loop); per layer i
`l<i>.norm1`, `l<i>.norm2` (one number each), `l<i>.shift` [width]; the mixer's `l<i>.mix.*`; the feed-forward's
`l<i>.mlp.router` [experts + identity, width], `l<i>.mlp.correction` [experts + identity], `l<i>.mlp.e<k>.up / .down`;
`final.norm` (one number); `head` [vocab, width].

  mixer "latent_attention"   mix.dq, mix.dq.norm, mix.uq (queries through a latent, per head [dim | rot_dim]), mix.dkv
                             ([kv_rank + rot_dim, width]), mix.dkv.norm, mix.uk, mix.uv, mix.g ([heads, width]: a sigmoid
                             gate per head), mix.o; the rot_dim parts rotate with entry 2i paired with entry 2i + 1
  mixer "mingru"             mix.z, mix.z.b, mix.x, mix.x.b, mix.g, mix.o

  x = embed[token] · embedding.scale
  per scheduled layer:  x += mixer(shift(norm1(x)));  x += experts(norm2(x))        (parts/block.py, "pre_norm")
  logits = head · norm(x)

A layer inside the loop appears several times in the schedule; every appearance has a cache and state of its own, and the
first layer of pass t is preceded by x += loop.step[t].
"""
from __future__ import annotations

import torch

from ..config.rakelorn import RakelornConfig, RecurrenceConfig
from ..engine.model import BuildOptions, DecoderModel, LayerCall
from ..parts import LMHead, TokenEmbedding, get_part
from ..registry import Architecture, register_architecture
from ..weights.spec import CheckedWeights, TensorSpec, place

#: positions a sequence may reach: the design has no position table, so this only sizes the block tables
MAX_POSITIONS = 1 << 17


def weight_spec(cfg: RakelornConfig) -> list[TensorSpec]:
    d = cfg.width
    specs = [TensorSpec("embed", (cfg.vocab, d))]
    if cfg.loop_times:
        specs.append(TensorSpec("loop.step", (cfg.loop_times, d), "vector"))
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}."
        specs += [TensorSpec(p + "norm1", (), "vector"), TensorSpec(p + "norm2", (), "vector", optional=ml is None)]
        q = p + "mix."
        if isinstance(m, RecurrenceConfig):
            W = m.width
            specs += [TensorSpec(q + "z", (W, d)), TensorSpec(q + "z.b", (W,), "vector"), TensorSpec(q + "x", (W, d)),
                      TensorSpec(q + "x.b", (W,), "vector"), TensorSpec(q + "g", (W, d)), TensorSpec(q + "o", (d, W))]
        else:
            per_q = m.dim + m.rot_dim
            specs += [TensorSpec(q + "dq", (m.q_rank, d)), TensorSpec(q + "dq.norm", (m.q_rank,), "vector"),
                      TensorSpec(q + "uq", (m.heads * per_q, m.q_rank)), TensorSpec(q + "dkv", (m.kv_rank + m.rot_dim, d)),
                      TensorSpec(q + "dkv.norm", (m.kv_rank,), "vector"), TensorSpec(q + "uk", (m.heads * m.dim, m.kv_rank)),
                      TensorSpec(q + "uv", (m.heads * m.vdim, m.kv_rank)), TensorSpec(q + "g", (m.heads, d)),
                      TensorSpec(q + "o", (d, m.heads * m.vdim))]
        if ml is not None:
            for e in range(ml.experts):
                specs += [TensorSpec(p + f"mlp.e{e}.up", (ml.ff, d)), TensorSpec(p + f"mlp.e{e}.down", (d, ml.ff))]
            specs += [TensorSpec(p + "mlp.router", (ml.experts + ml.identity, d)),
                      TensorSpec(p + "mlp.correction", (ml.experts + ml.identity,), "vector")]
        specs.append(TensorSpec(p + "shift", (d,), "vector"))
    specs += [TensorSpec("final.norm", (), "vector"), TensorSpec("head", (cfg.vocab, d))]
    return specs


def random_weights(cfg: RakelornConfig, gen: torch.Generator) -> dict:
    """Matrices N(0, 1/in), norm weights 1 + N(0, 0.1), biases N(0, 0.5) (the recurrence's gate biases spread from gates
    that forget within a few tokens to gates that keep hundreds), shift coefficients uniform in 0…1, the router's
    correction N(0, 0.05) (of the order of the scores it is added to), the vectors between passes N(0, 0.5), the embedding
    N(0, 1) and the head N(0, 1/width): no term of a formula is hidden by a zero or a one."""
    out = {}
    for spec in weight_spec(cfg):
        if spec.optional:                  # (the second norm of a layer without feed-forward)
            continue
        name, shape = spec.name, spec.shape
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        if name.endswith(".shift"):
            t = torch.rand(shape, generator=gen)
        elif name.endswith(".z.b"):
            t = -4.0 + 6.0 * torch.rand(shape, generator=gen)
        elif name.endswith(".b") or name == "loop.step":
            t = 0.5 * t
        elif name.endswith(".correction"):
            t = 0.05 * t
        elif spec.kind == "vector":
            t = 1.0 + 0.1 * t
        elif name == "embed":
            pass
        else:
            t = t / float(shape[-1]) ** 0.5
        out[name] = t
    return out


def build(cfg: RakelornConfig, weights: CheckedWeights, options: BuildOptions) -> DecoderModel:
    dt, dev = options.dtype, options.device
    d = cfg.width

    def matrix(name):
        return place(weights[name], "matrix", dt, dev)

    def vector(name):
        return place(weights[name], "vector", dt, dev)

    def one_weight(name, width=d):
        """A norm's single weight as the vector that the norm kernels take."""
        return vector(name).reshape(1).expand(width).contiguous()

    plain_norm, shifted_norm = get_part("norm", "group_rmsnorm"), get_part("norm", "rmsnorm_shift")
    block_cls = get_part("block", "pre_norm")
    rotations, layers = {}, []
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}."
        q = p + "mix."
        if isinstance(m, RecurrenceConfig):
            mixer = get_part("mixer", "mingru")(matrix(q + "z"), vector(q + "z.b"), matrix(q + "x"), vector(q + "x.b"),
                                                matrix(q + "g"), matrix(q + "o"))
        else:
            rk = (m.rot_base, m.rot_dims)
            if rk not in rotations:
                rotations[rk] = get_part("position", "rotary")(m.rot_base, m.rot_dims, dev, pairing="interleaved")
            mixer = get_part("mixer", "latent_attention")(
                n_heads=m.heads, dim=m.dim, vdim=m.vdim, kv_rank=m.kv_rank, rot_dim=m.rot_dim, scale=m.scale, eps=cfg.norm_eps,
                w_dq=matrix(q + "dq"), dq_norm=vector(q + "dq.norm"), w_uq=matrix(q + "uq"), w_dkv=matrix(q + "dkv"),
                dkv_norm=vector(q + "dkv.norm"), w_uk=matrix(q + "uk"), w_uv=matrix(q + "uv"), w_gate=matrix(q + "g"),
                w_out=matrix(q + "o"), rotary=rotations[rk])
        ffn = norm2 = None
        if ml is not None:
            norm2 = plain_norm(one_weight(p + "norm2"), cfg.norm_eps, 1)

            def stack(what):
                if ml.experts == 0:
                    return None
                return torch.stack([matrix(p + f"mlp.e{e}.{what}") for e in range(ml.experts)]).contiguous()
            ffn = get_part("feed_forward", "routed_experts")(
                matrix(p + "mlp.router"), None, None, stack("up"), stack("down"), top=ml.top, scoring="softmax_all",
                correction=vector(p + "mlp.correction"), groups=ml.groups, keep=ml.keep, weight_scale=ml.scale,
                n_identity=ml.identity)
        layers.append(block_cls(shifted_norm(one_weight(p + "norm1"), vector(p + "shift"), cfg.norm_eps), mixer, norm2, ffn))
    steps = vector("loop.step") if cfg.loop_times else None
    schedule = [LayerCall(i, add_before=steps[t].contiguous() if t is not None else None)
                for i, t in zip(cfg.layer_order, cfg.pass_begins)]
    embedding = TokenEmbedding(matrix("embed"), None, scale=cfg.embedding_scale)
    return DecoderModel(config=cfg, embedding=embedding, layers=layers, schedule=schedule,
                        final_norm=plain_norm(one_weight("final.norm"), cfg.norm_eps, 1), head=LMHead(matrix("head")),
                        options=options, max_seq_len=MAX_POSITIONS)


RAKELORN = register_architecture(Architecture(
    name="Rakelorn", config_cls=RakelornConfig, weight_spec=weight_spec, random_weights=random_weights, build=build))
