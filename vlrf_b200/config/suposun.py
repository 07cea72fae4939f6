"""Suposun's configuration: a decoder whose layers are listed one by one in config.json.

    {"architecture": "Suposun", "vocab": …, "width": …, "norm": {"eps": …}, "logit_scale": …,
     "embedding": {"scale": …, "bigram": {"buckets": …, "mul_prev": …, "mul_cur": …}},
     "layers": [{"type": "attention" | "attention_2", "mixer": {…}, "mlp": {…} | null}, …]}

A layer names its mixer's kind and sizes and its feed-forward.  Both mixers: `heads`, `kv_heads`, `dim`, `vdim`, `scale`,
`rot` (`base`, `dims`, optionally `scaling`: `factor`, `original`, `fast`, `slow`).  "attention" also reads `softcap` and
`mask` (`size`, `keep_first`); "attention_2" may name with `kv_from` the earlier layer whose keys and values it reads.
A feed-forward is "dense" (`ff`) or "moe" (`expert.ff`, `expert.limit`, `router.experts`, `router.top`).  `embedding`,
its `scale` and its `bigram`, `logit_scale`, a mixer's `mask`, `softcap`, `rot.scaling` and `kv_from`, and a layer's
`mlp` may each be absent.
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key
from .kuvusun import _need

MIXER_TYPES = ("attention", "attention_2")
MLP_KINDS = ("dense", "moe")


@dataclasses.dataclass(frozen=True)
class AttentionConfig:
    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float = 0.0
    rot_dims: int = 0                    # 0: no rotation
    rot_scaling: tuple | None = None     # (factor, original, fast, slow)
    softcap: float | None = None
    window: int = 0                      # 0: every earlier key is visible
    keep_first: int = 0
    kv_from: int | None = None


@dataclasses.dataclass(frozen=True)
class FeedForwardConfig:
    kind: str
    ff: int
    experts: int = 0
    top: int = 0
    limit: float = 0.0


@dataclasses.dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclasses.dataclass
class SuposunConfig(ModelConfig):
    model_type = "Suposun"

    vocab: int = key()
    width: int = key()
    norm: dict = key()
    layers: list = key()
    embedding: dict = key(default=None, nullable=True)
    logit_scale: float = key(default=1.0)

    def to_dict(self) -> dict:
        out = {"architecture": self.model_type, "vocab": self.vocab, "width": self.width, "norm": self.norm,
               "logit_scale": self.logit_scale, "layers": self.layers}
        if self.embedding is not None:
            out["embedding"] = self.embedding
        return out

    def validate(self) -> None:
        self._positive("vocab", self.vocab)
        self._positive("width", self.width)
        self.norm_eps = _need(self.norm, "eps", float, "norm")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        self.logit_scale = float(self.logit_scale)
        self.embedding_scale, self.bigram = 1.0, None
        if self.embedding is not None:
            if "scale" in self.embedding:
                self.embedding_scale = _need(self.embedding, "scale", float, "embedding")
            b = self.embedding.get("bigram")
            if b is not None:
                self.bigram = BigramConfig(*(_need(b, name, int, "embedding.bigram") for name in ("buckets", "mul_prev", "mul_cur")))
                if self.bigram.buckets <= 0 or self.bigram.mul_prev < 0 or self.bigram.mul_cur < 0:
                    raise ConfigError("embedding.bigram: buckets must be positive and the multipliers not negative")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        self.mixers, self.mlps = [], []
        for i, layer in enumerate(self.layers):
            self.mixers.append(self._mixer(i, layer))
            self.mlps.append(self._mlp(i, layer))

    def _mixer(self, i: int, layer) -> AttentionConfig:
        where = f"layers[{i}]"
        kind = _need(layer, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {', '.join(MIXER_TYPES)}")
        m = _need(layer, "mixer", dict, where)
        mw = where + ".mixer"
        fields = dict(kind=kind, heads=_need(m, "heads", int, mw), kv_heads=_need(m, "kv_heads", int, mw), dim=_need(m, "dim", int, mw),
                      vdim=_need(m, "vdim", int, mw), scale=_need(m, "scale", float, mw))
        rot = m.get("rot")
        if rot is not None:
            fields.update(rot_base=_need(rot, "base", float, mw + ".rot"), rot_dims=_need(rot, "dims", int, mw + ".rot"))
            sc = rot.get("scaling")
            if sc is not None:
                fields["rot_scaling"] = tuple(_need(sc, name, float, mw + ".rot.scaling") for name in ("factor", "original", "fast", "slow"))
        if kind == "attention":
            if m.get("softcap") is not None:
                fields["softcap"] = _need(m, "softcap", float, mw)
            mask = m.get("mask")
            if mask is not None:
                fields["window"] = _need(mask, "size", int, mw + ".mask")
                if mask.get("keep_first") is not None:
                    fields["keep_first"] = _need(mask, "keep_first", int, mw + ".mask")
        elif m.get("kv_from") is not None:
            fields["kv_from"] = _need(m, "kv_from", int, mw)
        mc = AttentionConfig(**fields)
        if min(mc.heads, mc.kv_heads, mc.dim, mc.vdim) <= 0 or mc.heads % mc.kv_heads != 0:
            raise ConfigError(f"config.json: {mw}: heads, kv_heads, dim and vdim must be positive and kv_heads divide heads")
        if kind == "attention" and mc.vdim != mc.dim:
            raise ConfigError(f"config.json: {mw}: the values of this mixer are its keys, so vdim ({mc.vdim}) must equal dim ({mc.dim})")
        if rot is not None and (mc.rot_dims <= 0 or mc.rot_dims % 2 != 0 or mc.rot_dims > mc.dim or not mc.rot_base > 0):
            raise ConfigError(f"config.json: {mw}: rot.dims ({mc.rot_dims}) must be even, positive and at most dim ({mc.dim}), and "
                              f"rot.base positive")
        if mc.rot_scaling is not None and (min(mc.rot_scaling) <= 0.0 or mc.rot_base == 1.0):
            raise ConfigError(f"config.json: {mw}.rot.scaling: factor, original, fast and slow must be positive")
        if mc.softcap is not None and not mc.softcap > 0.0:
            raise ConfigError(f"config.json: {mw}.softcap must be positive")
        if (m.get("mask") is not None and mc.window <= 0) or mc.keep_first < 0:
            raise ConfigError(f"config.json: {mw}.mask: size must be positive and keep_first not negative")
        if mc.kv_from is not None:
            j = mc.kv_from
            if not (0 <= j < i) or self.mixers[j].kind != "attention_2" or self.mixers[j].kv_from is not None:
                raise ConfigError(f"config.json: {mw}.kv_from = {j} must name an earlier layer of the same kind with keys and values of its own")
            o = self.mixers[j]
            if (o.heads, o.kv_heads, o.dim, o.vdim, o.rot_base, o.rot_dims, o.rot_scaling) != \
                    (mc.heads, mc.kv_heads, mc.dim, mc.vdim, mc.rot_base, mc.rot_dims, mc.rot_scaling):
                raise ConfigError(f"config.json: {mw}: head counts, sizes and rot differ from those of layer {j}, whose keys and values it reads")
        return mc

    def _mlp(self, i: int, layer):
        ml = layer.get("mlp") if isinstance(layer, dict) else None
        if ml is None:
            return None
        lw = f"layers[{i}].mlp"
        mk = _need(ml, "kind", str, lw)
        if mk not in MLP_KINDS:
            raise ConfigError(f"config.json: {lw}.kind '{mk}' is not one of {', '.join(MLP_KINDS)}")
        if mk == "dense":
            cfg = FeedForwardConfig("dense", _need(ml, "ff", int, lw))
        else:
            expert, router = _need(ml, "expert", dict, lw), _need(ml, "router", dict, lw)
            cfg = FeedForwardConfig("moe", _need(expert, "ff", int, lw + ".expert"), experts=_need(router, "experts", int, lw + ".router"),
                                    top=_need(router, "top", int, lw + ".router"), limit=_need(expert, "limit", float, lw + ".expert"))
            if cfg.experts <= 0 or not (0 < cfg.top <= cfg.experts):
                raise ConfigError(f"config.json: {lw}.router: top ({cfg.top}) must lie in 1…experts ({cfg.experts})")
            if not cfg.limit > 0.0:
                raise ConfigError(f"config.json: {lw}.expert.limit must be positive")
        if cfg.ff <= 0:
            raise ConfigError(f"config.json: {lw}: the inner size must be positive")
        return cfg

    @property
    def n_layer(self) -> int:
        return len(self.layers)
