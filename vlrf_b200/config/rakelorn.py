"""Rakelorn's configuration: a decoder whose layers are listed one by one in config.json.

    {"architecture": "Rakelorn", "vocab": …, "width": …, "norm": {"eps": …}, "embedding": {"scale": …},
     "loop": {"start": …, "stop": …, "times": …},
     "layers": [{"type": "latent_attention" | "mingru", "mixer": {…}, "mlp": {…} | null}, …]}

A layer names its mixer's kind and sizes and its feed-forward.  "latent_attention": `heads`, `dim` (unrotated query/key
size), `rot_dim` (rotated), `vdim`, `kv_rank`, `q_rank`, `scale`, `rot` (`base`, `dims`).  "mingru": `width` of the
recurrence.  A feed-forward of kind "moe": `expert.ff`, `router.experts`, `router.top`, `router.identity` (experts that
return their input), `router.groups` (`count`, `keep`), `router.scale`.  `embedding` and `loop` may be absent (no
scaling; every layer once and no vectors between passes).
"""
from __future__ import annotations

import dataclasses

from .base import ConfigError, ModelConfig, key
from .kuvusun import LatentMixerConfig, _need

MIXER_TYPES = ("latent_attention", "mingru")
MLP_KINDS = ("moe",)


@dataclasses.dataclass(frozen=True)
class RecurrenceConfig:
    width: int


@dataclasses.dataclass(frozen=True)
class ScoredMoeConfig:
    ff: int
    experts: int                     # experts with matrices
    identity: int                    # experts that return their input (the router's last outputs)
    top: int
    groups: int
    keep: int
    scale: float


@dataclasses.dataclass
class RakelornConfig(ModelConfig):
    model_type = "Rakelorn"

    vocab: int = key()
    width: int = key()
    norm: dict = key()
    layers: list = key()
    embedding: dict = key(default=None, nullable=True)
    loop: dict = key(default=None, nullable=True)

    def to_dict(self) -> dict:
        out = {"architecture": self.model_type, "vocab": self.vocab, "width": self.width, "norm": self.norm, "layers": self.layers}
        for name in ("embedding", "loop"):
            if getattr(self, name) is not None:
                out[name] = getattr(self, name)
        return out

    def validate(self) -> None:
        self._positive("vocab", self.vocab)
        self._positive("width", self.width)
        self.norm_eps = _need(self.norm, "eps", float, "norm")
        if not self.norm_eps > 0.0:
            raise ConfigError(f"norm.eps must be positive, got {self.norm_eps}")
        self.embedding_scale = _need(self.embedding, "scale", float, "embedding") if self.embedding is not None else 1.0
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        self.mixers, self.mlps = [], []
        for i, layer in enumerate(self.layers):
            self.mixers.append(self._mixer(i, layer))
            self.mlps.append(self._mlp(i, layer))
        n = len(self.layers)
        #: the layers in the order they run, and for each run the number of the pass it begins (or None)
        self.layer_order, self.pass_begins = list(range(n)), [None] * n
        self.loop_times = 0
        if self.loop is not None:
            a, b, k = (_need(self.loop, name, int, "loop") for name in ("start", "stop", "times"))
            if not (0 <= a < b <= n) or k < 1:
                raise ConfigError(f"loop: start {a}, stop {b}, times {k} do not name a range of the {n} layers run at least once")
            self.loop_times = k
            self.layer_order = list(range(a)) + list(range(a, b)) * k + list(range(b, n))
            self.pass_begins = [None] * a + [t if i == a else None for t in range(k) for i in range(a, b)] + [None] * (n - b)

    def _mixer(self, i: int, layer):
        where = f"layers[{i}]"
        kind = _need(layer, "type", str, where)
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {where}.type '{kind}' is not one of {', '.join(MIXER_TYPES)}")
        m = _need(layer, "mixer", dict, where)
        mw = where + ".mixer"
        if kind == "mingru":
            r = RecurrenceConfig(_need(m, "width", int, mw))
            if r.width <= 0:
                raise ConfigError(f"config.json: {mw}.width must be positive")
            return r
        rot = _need(m, "rot", dict, mw)
        mc = LatentMixerConfig(heads=_need(m, "heads", int, mw), dim=_need(m, "dim", int, mw), vdim=_need(m, "vdim", int, mw),
                               kv_rank=_need(m, "kv_rank", int, mw), scale=_need(m, "scale", float, mw),
                               q_rank=_need(m, "q_rank", int, mw), rot_dim=_need(m, "rot_dim", int, mw),
                               rot_base=_need(rot, "base", float, mw + ".rot"), rot_dims=_need(rot, "dims", int, mw + ".rot"),
                               gated=True)
        if min(mc.heads, mc.dim, mc.vdim, mc.kv_rank, mc.q_rank) <= 0:
            raise ConfigError(f"config.json: {mw}: heads, dim, vdim, kv_rank and q_rank must be positive")
        if mc.rot_dim <= 0 or mc.rot_dims <= 0 or mc.rot_dims % 2 != 0 or mc.rot_dims > mc.rot_dim or not mc.rot_base > 0:
            raise ConfigError(f"config.json: {mw}: rot.dims ({mc.rot_dims}) must be even, positive and at most rot_dim "
                              f"({mc.rot_dim}), and rot.base positive")
        return mc

    def _mlp(self, i: int, layer):
        ml = layer.get("mlp") if isinstance(layer, dict) else None
        if ml is None:
            return None
        lw = f"layers[{i}].mlp"
        mk = _need(ml, "kind", str, lw)
        if mk not in MLP_KINDS:
            raise ConfigError(f"config.json: {lw}.kind '{mk}' is not one of {', '.join(MLP_KINDS)}")
        router = _need(ml, "router", dict, lw)
        rw = lw + ".router"
        groups = router.get("groups")
        cfg = ScoredMoeConfig(
            ff=_need(_need(ml, "expert", dict, lw), "ff", int, lw + ".expert"), experts=_need(router, "experts", int, rw),
            identity=_need(router, "identity", int, rw) if "identity" in router else 0, top=_need(router, "top", int, rw),
            groups=_need(groups, "count", int, rw + ".groups") if groups is not None else 1,
            keep=_need(groups, "keep", int, rw + ".groups") if groups is not None else 1,
            scale=_need(router, "scale", float, rw) if "scale" in router else 1.0)
        outputs = cfg.experts + cfg.identity
        if cfg.ff <= 0 or cfg.experts < 0 or cfg.identity < 0 or outputs <= 0:
            raise ConfigError(f"config.json: {lw}: the inner size must be positive and there must be an expert")
        if cfg.groups < 1 or outputs % cfg.groups != 0 or not (1 <= cfg.keep <= cfg.groups):
            raise ConfigError(f"config.json: {rw}.groups: {outputs} router outputs cannot form {cfg.groups} equal groups of which "
                              f"{cfg.keep} are kept")
        if not (0 < cfg.top <= cfg.keep * (outputs // cfg.groups)):
            raise ConfigError(f"config.json: {rw}: top ({cfg.top}) must lie in 1…{cfg.keep * (outputs // cfg.groups)}, the experts of the kept groups")
        return cfg

    @property
    def n_layer(self) -> int:
        return len(self.layers)
