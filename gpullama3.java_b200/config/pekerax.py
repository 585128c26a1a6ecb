"""Typed configuration of the Pekerax decoder, read from ``config.json``.

A Pekerax model is a list of layers over one residual stream, each a pre-norm pair of a mixer and an optional
feed-forward; every norm is a layer norm with weight and bias (``norm.eps``); the embedding rows are multiplied with
``embedding.scale`` on their way in, and the output head is the embedding table as stored.

* ``layers[i].type`` names the mixer, ``layers[i].mixer`` gives its sizes:
  ``delta``: the gated delta rule with one decay per head behind a short convolution (``heads``, ``kv_heads``, ``dim``,
  ``vdim``, ``conv`` taps);
  ``attention``: grouped-query attention without rotation (``heads``, ``kv_heads``, ``dim``, ``vdim``, score ``scale``),
  with a weighted RMS norm over the whole query and key projections, a distance penalty per head, a sliding window
  ``mask.size`` behind which the first ``mask.keep_first`` positions stay visible (no ``mask``: no window), a learned sink per head, an output
  gate per head, and, where ``v_mix`` is set, values mixed with those of the first such layer;
* ``layers[i].mlp`` is null, ``{"kind": "dense", "ff", "limit"}`` or ``{"kind": "moe", "expert": {"ff", "limit"},
  "router": {"experts", "top", "groups": {"count", "keep"}}}``; both kinds use the clamped gated unit
  min(g, limit) sigmoid(1.702 min(g, limit)) (clamp(u, -limit, limit) + 1).

Constants the design fixes stand here: the unit's sigmoid slope, the slope base of the distance penalty, the epsilons of
the delta rule's unit vectors and of the routing weights."""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, as_float, as_int, require_keys
from .registry import register_architecture

MIXER_TYPES = ("attention", "delta")
UNIT_SIGMOID_SLOPE = 1.702
DISTANCE_SLOPE_BASE = 8.0      # slope of head h: 2^(-8 (h + 1) / heads)
UNIT_VECTOR_EPS = 1e-6
ROUTING_WEIGHT_EPS = 1e-20


def _positive(d: dict, key: str, where: str) -> float:
    v = as_float(d, key)
    if not v > 0:
        raise ConfigError(f"{where}: {key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class PekeraxLayer:
    type: str
    mixer: dict        # the mixer's record as config.json has it (checked when read)
    mlp: dict | None   # the feed-forward's record, None for a layer without one


@dataclass(frozen=True)
class PekeraxConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    layers: tuple
    norm_eps: float
    embed_scale: float = 1.0
    initializer_range: float = 0.02
    tie_word_embeddings: bool = True
    stop_token_ids: tuple[int, ...] = ()

    architecture = "Pekerax"

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "PekeraxConfig":
        require_keys(d, ["vocab", "width", "layers", "norm"], "Pekerax config.json")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("Pekerax config.json: 'layers' must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("Pekerax config.json: 'norm' must be an object with 'eps'")
        require_keys(d["norm"], ["eps"], "Pekerax norm")
        eps = _positive(d["norm"], "eps", "norm")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("Pekerax config.json: 'embedding' must be an object with 'scale'")
        scale = as_float(emb, "scale") if emb.get("scale") is not None else 1.0
        layers = []
        for i, L in enumerate(d["layers"]):
            where = f"layer {i}"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"{where}: needs 'type' and a 'mixer' object")
            kind, m = L.get("type"), dict(L["mixer"])
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            need = {"attention": ["heads", "kv_heads", "dim", "vdim", "scale"],
                    "delta": ["heads", "kv_heads", "dim", "vdim", "conv"]}[kind]
            require_keys(m, need, where)
            for key in need:
                if key == "scale":
                    _positive(m, key, where)
                else:
                    as_int(m, key)
            if kind == "attention" and m.get("mask") is not None:      # (no mask: every earlier position is visible)
                if not isinstance(m["mask"], dict):
                    raise ConfigError(f"{where}: mask must be an object with 'size' (and 'keep_first')")
                require_keys(m["mask"], ["size"], where + " mask")
                as_int(m["mask"], "size")
                if m["mask"].get("keep_first") is not None:
                    as_int(m["mask"], "keep_first", minimum=0)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            mlp = L.get("mlp")
            if mlp is not None:
                mlp = cls._checked_mlp(mlp, where)
            layers.append(PekeraxLayer(kind, m, mlp))
        mixing = [L.mixer for L in layers if L.type == "attention" and L.mixer.get("v_mix")]
        if any((m["kv_heads"], m["vdim"]) != (mixing[0]["kv_heads"], mixing[0]["vdim"]) for m in mixing):
            raise ConfigError("layers that mix their values must agree on kv_heads and vdim")
        eos = d.get("eos_token_id")
        stop = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab_size=as_int(d, "vocab"), hidden_size=as_int(d, "width"), layers=tuple(layers), norm_eps=eps,
                   embed_scale=scale, initializer_range=float(d.get("initializer_range", 0.02)), stop_token_ids=stop)

    @staticmethod
    def _checked_mlp(mlp, where: str) -> dict:
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"{where}: mlp must be null or an object of kind 'dense' or 'moe', got {mlp!r}")
        if mlp["kind"] == "dense":
            require_keys(mlp, ["ff", "limit"], where + " mlp")
            as_int(mlp, "ff")
            _positive(mlp, "limit", where + " mlp")
            return dict(mlp)
        require_keys(mlp, ["expert", "router"], where + " mlp")
        ex, ro = mlp["expert"], mlp["router"]
        if not isinstance(ex, dict) or not isinstance(ro, dict):
            raise ConfigError(f"{where} mlp: 'expert' and 'router' must be objects")
        require_keys(ex, ["ff", "limit"], where + " mlp.expert")
        as_int(ex, "ff")
        _positive(ex, "limit", where + " mlp.expert")
        require_keys(ro, ["experts", "top"], where + " mlp.router")
        n, top = as_int(ro, "experts"), as_int(ro, "top")
        groups = ro.get("groups") or {"count": 1, "keep": 1}
        if not isinstance(groups, dict):
            raise ConfigError(f"{where} mlp.router: groups must be an object with 'count' and 'keep'")
        require_keys(groups, ["count", "keep"], where + " mlp.router.groups")
        count, keep = as_int(groups, "count"), as_int(groups, "keep")
        if n % count or keep > count or top > keep * (n // count):
            raise ConfigError(f"{where} mlp.router: {top} of {n} experts in {count} groups of which {keep} are kept")
        return {"kind": "moe", "expert": dict(ex), "router": {"experts": n, "top": top, "groups": {"count": count, "keep": keep}}}

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embed_scale}, "norm": {"eps": self.norm_eps},
             "initializer_range": self.initializer_range,
             "layers": [{"type": L.type, "mixer": dict(L.mixer), "mlp": dict(L.mlp) if L.mlp else None} for L in self.layers]}
        if self.stop_token_ids:
            d["eos_token_id"] = list(self.stop_token_ids)
        return d

    # ---- the model as data
    def embedding_scale(self) -> float:
        return self.embed_scale

    def _norm(self) -> PartSpec:
        return PartSpec("norm", "layernorm", {"dim": self.hidden_size, "eps": self.norm_eps})

    def _value_mix(self, i: int):
        """None, "source" (the first value-mixing layer) or "mixed"."""
        if not (self.layers[i].type == "attention" and self.layers[i].mixer.get("v_mix")):
            return None
        first = next(j for j, L in enumerate(self.layers) if L.type == "attention" and L.mixer.get("v_mix"))
        return "source" if i == first else "mixed"

    def _mixer(self, i: int) -> PartSpec:
        L = self.layers[i]
        m, h = L.mixer, self.hidden_size
        if L.type == "attention":
            return PartSpec("mixer", "attention", {
                "hidden_size": h, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "position": PartSpec("position", "none", {}),
                "window": (m.get("mask") or {}).get("size"), "keep_first": int((m.get("mask") or {}).get("keep_first") or 0),
                "qk_norm_eps": self.norm_eps, "projection_norm": True,
                "scale": float(m["scale"]), "distance_slope_base": DISTANCE_SLOPE_BASE, "sink": True,
                "value_mix": self._value_mix(i), "output_gate": True})
        return PartSpec("mixer", "head_delta", {
            "hidden_size": h, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": self.norm_eps, "unit_eps": UNIT_VECTOR_EPS,
            "gate_activation": "silu"})

    def _feed_forward(self, mlp: dict) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("feed_forward", "gated", {
                "hidden_size": self.hidden_size, "intermediate_size": mlp["ff"], "activation": "clamped_sigmoid",
                "limit": float(mlp["limit"]), "slope": UNIT_SIGMOID_SLOPE})
        ro, ex = mlp["router"], mlp["expert"]
        return PartSpec("feed_forward", "routed", {
            "hidden_size": self.hidden_size, "intermediate_size": ex["ff"], "n_experts": ro["experts"], "top": ro["top"],
            "groups": ro["groups"]["count"], "keep_groups": ro["groups"]["keep"], "activation": "clamped_sigmoid",
            "limit": float(ex["limit"]), "slope": UNIT_SIGMOID_SLOPE, "weight_eps": ROUTING_WEIGHT_EPS})

    def layer_specs(self) -> list[LayerSpec]:
        specs = []
        for i, L in enumerate(self.layers):
            parts = {"mixer": self._mixer(i), "mixer_norm": self._norm()}
            if L.mlp is not None:
                parts["feed_forward"] = self._feed_forward(L.mlp)
                parts["feed_forward_norm"] = self._norm()
            specs.append(LayerSpec("connected", parts))
        return specs

    def final_norm(self) -> PartSpec:
        return self._norm()

    def tensor_names(self) -> dict[str, str]:
        names = {"embedding.table": "embed", "final_norm.weight": "final.norm", "final_norm.bias": "final.norm.b"}
        for i, L in enumerate(self.layers):
            p, c = f"layers.{i}.", f"l{i}."
            names[p + "mixer_norm.weight"], names[p + "mixer_norm.bias"] = c + "norm1", c + "norm1.b"
            if L.mlp is not None:
                names[p + "feed_forward_norm.weight"], names[p + "feed_forward_norm.bias"] = c + "norm2", c + "norm2.b"
                if L.mlp["kind"] == "dense":
                    for w in ("gate", "up", "down"):
                        names[p + f"feed_forward.{w}"] = c + f"mlp.{w}"
                else:
                    names[p + "feed_forward.router"] = c + "mlp.router"
                    for e in range(L.mlp["router"]["experts"]):
                        for w in ("gate", "up", "down"):
                            names[p + f"feed_forward.e{e}.{w}"] = c + f"mlp.e{e}.{w}"
            m = p + "mixer."
            if L.type == "attention":
                for w in ("q", "k", "v", "o", "g", "sink"):
                    names[m + w] = c + f"mix.{w}"
                names[m + "q_norm"], names[m + "k_norm"] = c + "mix.q.norm", c + "mix.k.norm"
                if L.mixer.get("v_mix"):
                    names[m + "vmix"] = c + "mix.vmix"
            else:
                for w in ("q", "k", "v", "b", "A_log", "norm", "a", "dt_bias", "g", "o"):
                    names[m + w] = c + f"mix.{w}"
                for w in ("q", "k", "v"):
                    names[m + w + "_conv"] = c + f"mix.{w}.conv"
        return names

    def init_std(self) -> float:
        return self.initializer_range


register_architecture("Pekerax", PekeraxConfig)
