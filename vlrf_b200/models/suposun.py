"""Suposun: a decoder of softmax-attention layers of two kinds with dense or routed feed-forwards, a bigram table beside
the token embedding, and the norm on every sublayer's output.

Tensors (all linear weights [out, in]): `embed` [vocab, width]; `bigram` [buckets + 1, width] where the configuration
has one; per layer i `l<i>.norm1`, `l<i>.ls1` and, with a feed-forward, `l<i>.norm2`, `l<i>.ls2`; the mixer's `l<i>.mix.*`
and the feed-forward's `l<i>.mlp.*`; `final.norm`.  The head is the embedding table.

  mixer "attention"     mix.q, mix.k (the values are the projected keys), mix.q.norm / mix.k.norm [dim] (per head, one
                        weight for all heads), mix.sink [heads], mix.g [heads, width] (a sigmoid gate per head), mix.o
  mixer "attention_2"   mix.q, mix.k, mix.v, mix.q.norm [heads·dim] / mix.k.norm [kv_heads·dim] (over the whole
                        projection), mix.o; with kv_from only mix.q, mix.q.norm, mix.o
  mlp "dense"           mlp.gate, mlp.up, mlp.down (tanh GELU on the gate)
  mlp "moe"             mlp.router, mlp.correction, mlp.e<k>.gate / .up / .down

  x = embed[token] · embedding.scale + bigram[(token before · mul_prev + token · mul_cur) mod buckets]   (last row at position 0)
  per layer: x += ls1 ⊙ norm1(mixer(x)); x += ls2 ⊙ norm2(ffn(x)), the norms RMS norms whose factor is 1 + the stored weight
  logits = logit_scale · embed · norm(x)

A layer with `kv_from` reads that layer's keys and values (as its cache holds them) and writes none.
"""
from __future__ import annotations

import torch

from ..config.suposun import SuposunConfig
from ..engine.model import BuildOptions, DecoderModel, LayerCall
from ..parts import LMHead, TokenEmbedding, get_part
from ..registry import Architecture, register_architecture
from ..weights.spec import CheckedWeights, TensorSpec, place

#: positions a sequence may reach: the design has no position table, so this only sizes the block tables
MAX_POSITIONS = 1 << 17

#: the factor inside the sigmoid of an expert's gate, g · sigmoid(1.702 g): fixed by the design
EXPERT_GATE_ALPHA = 1.702


def weight_spec(cfg: SuposunConfig) -> list[TensorSpec]:
    d = cfg.width
    specs = [TensorSpec("embed", (cfg.vocab, d))]
    if cfg.bigram is not None:
        specs.append(TensorSpec("bigram", (cfg.bigram.buckets + 1, d)))
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}."
        specs += [TensorSpec(p + "norm1", (d,), "vector"), TensorSpec(p + "norm2", (d,), "vector", optional=ml is None)]
        q = p + "mix."
        specs.append(TensorSpec(q + "q", (m.heads * m.dim, d)))
        if m.kind == "attention":
            specs += [TensorSpec(q + "k", (m.kv_heads * m.dim, d)), TensorSpec(q + "q.norm", (m.dim,), "vector"),
                      TensorSpec(q + "k.norm", (m.dim,), "vector"), TensorSpec(q + "sink", (m.heads,), "vector"),
                      TensorSpec(q + "g", (m.heads, d))]
        else:
            if m.kv_from is None:
                specs += [TensorSpec(q + "k", (m.kv_heads * m.dim, d)), TensorSpec(q + "v", (m.kv_heads * m.vdim, d)),
                          TensorSpec(q + "k.norm", (m.kv_heads * m.dim,), "vector")]
            specs.append(TensorSpec(q + "q.norm", (m.heads * m.dim,), "vector"))
        specs.append(TensorSpec(q + "o", (d, m.heads * m.vdim)))
        if ml is not None:
            q = p + "mlp."
            if ml.kind == "dense":
                specs += [TensorSpec(q + "gate", (ml.ff, d)), TensorSpec(q + "up", (ml.ff, d)), TensorSpec(q + "down", (d, ml.ff))]
            else:
                for e in range(ml.experts):
                    specs += [TensorSpec(q + f"e{e}.gate", (ml.ff, d)), TensorSpec(q + f"e{e}.up", (ml.ff, d)),
                              TensorSpec(q + f"e{e}.down", (d, ml.ff))]
                specs += [TensorSpec(q + "router", (ml.experts, d)), TensorSpec(q + "correction", (ml.experts,), "vector")]
        specs += [TensorSpec(p + "ls1", (d,), "vector"), TensorSpec(p + "ls2", (d,), "vector", optional=ml is None)]
    specs.append(TensorSpec("final.norm", (d,), "vector"))
    return specs


def random_weights(cfg: SuposunConfig, gen: torch.Generator) -> dict:
    """Matrices N(0, 1/in); the norms on sublayer outputs and the model's norm (whose stored weights are offsets from one) N(0, 0.1); the norms of
    queries and keys 1 + N(0, 0.1); layer scales 0.5 + N(0, 0.1); sinks N(0, 1); the routers' corrections N(0, 0.05): no
    term of a formula is hidden by a zero or a one.  The embedding is drawn so that a scaled row has a size of 0.06, and
    the bigram table N(0, 0.3): with the embedding as head a token's own embedding otherwise dominates its logits, and
    a random model does nothing but repeat its last token whatever its layers compute."""
    out = {}
    for spec in weight_spec(cfg):
        if spec.optional:
            continue
        name = spec.name
        t = torch.randn(spec.shape, generator=gen, dtype=torch.float32)
        if name.endswith(".ls1") or name.endswith(".ls2"):
            t = 0.5 + 0.1 * t
        elif name.endswith(".correction"):
            t = 0.05 * t
        elif name.endswith(".sink"):
            pass
        elif name.endswith("q.norm") or name.endswith("k.norm"):
            t = 1.0 + 0.1 * t
        elif spec.kind == "vector":
            t = 0.1 * t
        elif name == "embed":
            t = t * (0.06 / max(abs(cfg.embedding_scale), 1e-6))
        elif name == "bigram":
            t = 0.3 * t
        else:
            t = t / float(spec.shape[-1]) ** 0.5
        out[name] = t
    return out


def build(cfg: SuposunConfig, weights: CheckedWeights, options: BuildOptions) -> DecoderModel:
    dt, dev = options.dtype, options.device

    def matrix(name):
        return place(weights[name], "matrix", dt, dev)

    def vector(name):
        return place(weights[name], "vector", dt, dev)

    norm_cls = get_part("norm", "group_rmsnorm")

    def out_norm(name, scale_name=None):
        """An RMS norm with the factor 1 + stored weight, times the layer scale where there is one."""
        return norm_cls(vector(name), cfg.norm_eps, 1, offset=1.0, post_scale=vector(scale_name) if scale_name else None)

    embed = matrix("embed")
    bigram = (matrix("bigram"), cfg.bigram.mul_prev, cfg.bigram.mul_cur) if cfg.bigram is not None else None
    embedding = TokenEmbedding(embed, None, scale=cfg.embedding_scale, bigram=bigram)
    mixer_cls, block_cls = get_part("mixer", "window_attention"), get_part("block", "sublayer_norm")
    layers, schedule, rotations = [], [], {}
    for i, (m, ml) in enumerate(zip(cfg.mixers, cfg.mlps)):
        p = f"l{i}.mix."
        first_kind = m.kind == "attention"
        rotary = None
        if m.rot_dims > 0:
            rk = (m.rot_base, m.rot_dims, m.rot_scaling, first_kind)
            if rk not in rotations:
                rotations[rk] = get_part("position", "rotary")(m.rot_base, m.rot_dims, dev, yarn=m.rot_scaling,
                                                               pairing="interleaved" if first_kind else "half")
            rotary = rotations[rk]
        own = m.kv_from is None
        common = dict(n_heads=m.heads, n_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim, scale=m.scale, rotary=rotary,
                      q_norm=vector(p + "q.norm"), norm_eps=cfg.norm_eps)
        if first_kind:
            mixer = mixer_cls(matrix(p + "q"), matrix(p + "k"), None, matrix(p + "o"), qk_norm="head", k_norm=vector(p + "k.norm"),
                              softcap=m.softcap, window=m.window, keep_first=m.keep_first if m.window > 0 else 0,
                              sink=vector(p + "sink"), w_gate=matrix(p + "g"), **common)
        else:
            mixer = mixer_cls(matrix(p + "q"), matrix(p + "k") if own else None, matrix(p + "v") if own else None, matrix(p + "o"),
                              qk_norm="all", k_norm=vector(p + "k.norm") if own else None, **common)
        ffn = norm2 = None
        if ml is not None:
            q = f"l{i}.mlp."
            norm2 = out_norm(f"l{i}.norm2", f"l{i}.ls2")
            if ml.kind == "dense":
                ffn = get_part("feed_forward", "gated_mlp")(matrix(q + "gate"), matrix(q + "up"), matrix(q + "down"),
                                                            activation="gelu_tanh")
            else:
                def stack(what):
                    return torch.stack([matrix(q + f"e{e}.{what}") for e in range(ml.experts)]).contiguous()
                ffn = get_part("feed_forward", "routed_experts")(
                    matrix(q + "router"), None, stack("gate"), stack("up"), stack("down"), top=ml.top, scoring="sigmoid",
                    correction=vector(q + "correction"), gate="clamped", limit=ml.limit, gate_alpha=EXPERT_GATE_ALPHA)
        layers.append(block_cls(out_norm(f"l{i}.norm1", f"l{i}.ls1"), mixer, norm2, ffn))
        schedule.append(LayerCall(i, reads_cache_of=m.kv_from))
    return DecoderModel(config=cfg, embedding=embedding, layers=layers, schedule=schedule, final_norm=out_norm("final.norm"),
                        head=LMHead(embed, scale=cfg.logit_scale), options=options, max_seq_len=MAX_POSITIONS)


SUPOSUN = register_architecture(Architecture(
    name="Suposun", config_cls=SuposunConfig, weight_spec=weight_spec, random_weights=random_weights, build=build))
