"""Typed configuration of the Guduzen decoder, read from ``config.json``.

A Guduzen model is a list of layers, each with its own mixer and an optional gated feed-forward, over several
residual streams:

* ``layers[i].type`` names the mixer: ``attention`` (grouped-query attention without rotation, biases on the three
  projections, an unweighted RMS norm over every query and key head, a sliding window ``mask.size``, the score
  ``scale`` of the configuration; with ``kv_from: j`` it has no key and value projections and reads layer j's
  cache), ``latent_attention`` (queries and keys/values through latents of ``q_rank`` and ``kv_rank``; causal),
  ``channel_delta`` (the gated delta rule with a decay per key channel behind a short convolution of ``conv`` taps);
* ``layers[i].mixer`` gives that mixer's sizes (``heads``, ``kv_heads``, ``dim``, ``vdim``, ...), ``layers[i].mlp`` is
  ``{"kind": "dense", "ff": n}`` or null;
* ``streams`` residual streams with learned read / write / mix weights per sublayer; ``norm.eps`` for every RMS norm
  (weights are stored around zero and applied as 1 + w); the output head is the embedding table, and logits pass
  ``logit_softcap`` * tanh(. / ``logit_softcap``).

The inner sizes of the delta mixer's two low-rank products are not configuration keys; they are read from the
checkpoint's shapes (``a_rank`` / ``g_rank`` may be given in the mixer's record, which the random-weights mode needs)."""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, ScheduleEntry, as_float, as_int, require_keys
from .registry import register_architecture

MIXER_TYPES = ("attention", "latent_attention", "channel_delta")


def _optional_int(d: dict, key: str, minimum: int = 1):
    return as_int(d, key, minimum=minimum) if d.get(key) is not None else None


def _window(mixer: dict, where: str):
    mask = mixer.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"{where}: mask must be an object with 'size', got {mask!r}")
    return _optional_int(mask, "size")


@dataclass(frozen=True)
class GuduzenLayer:
    type: str
    mixer: dict      # the mixer's record as config.json has it (checked when read)
    ff: int | None   # width of the dense feed-forward, None for a layer without one


@dataclass(frozen=True)
class GuduzenConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    layers: tuple
    norm_eps: float
    streams: int | None
    logit_softcap: float | None
    initializer_range: float = 0.02
    tie_word_embeddings: bool = True
    stop_token_ids: tuple[int, ...] = ()

    architecture = "Guduzen"

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "GuduzenConfig":
        require_keys(d, ["vocab", "width", "layers", "norm"], "Guduzen config.json")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("Guduzen config.json: 'layers' must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("Guduzen config.json: 'norm' must be an object with 'eps'")
        require_keys(d["norm"], ["eps"], "Guduzen norm")
        eps = as_float(d["norm"], "eps")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        layers = []
        for i, L in enumerate(d["layers"]):
            where = f"layer {i}"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"{where}: needs 'type' and a 'mixer' object")
            kind, m = L.get("type"), dict(L["mixer"])
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            need = {"attention": ["heads", "kv_heads", "dim", "vdim", "scale"],
                    "latent_attention": ["heads", "dim", "vdim", "kv_rank", "q_rank", "scale"],
                    "channel_delta": ["heads", "kv_heads", "dim", "vdim", "conv"]}[kind]
            require_keys(m, need, where)
            for key in need:
                if key == "scale":
                    if as_float(m, key) <= 0:
                        raise ConfigError(f"{where}: scale must be positive")
                else:
                    as_int(m, key)
            if "kv_heads" in need and m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
            _window(m, where)
            if kind == "attention" and m.get("kv_from") is not None:
                j = as_int(m, "kv_from", minimum=0)
                if j >= i or d["layers"][j].get("type") != "attention" or d["layers"][j]["mixer"].get("kv_from") is not None:
                    raise ConfigError(f"{where}: kv_from {j} must name an earlier attention layer with projections of its own")
                other = d["layers"][j]["mixer"]
                if any(other.get(k) != m.get(k) for k in ("heads", "kv_heads", "dim", "vdim")):
                    raise ConfigError(f"{where}: its head counts and sizes differ from those of layer {j}, whose cache it reads")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"{where}: mlp must be null or {{'kind': 'dense', 'ff': n}}, got {mlp!r}")
                require_keys(mlp, ["ff"], where + " mlp")
                ff = as_int(mlp, "ff")
            layers.append(GuduzenLayer(kind, m, ff))
        cap = as_float(d, "logit_softcap") if d.get("logit_softcap") is not None else None
        if cap is not None and cap <= 0:
            raise ConfigError("logit_softcap must be positive")
        eos = d.get("eos_token_id")
        stop = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab_size=as_int(d, "vocab"), hidden_size=as_int(d, "width"), layers=tuple(layers), norm_eps=eps,
                   streams=_optional_int(d, "streams"), logit_softcap=cap,
                   initializer_range=float(d.get("initializer_range", 0.02)), stop_token_ids=stop)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "initializer_range": self.initializer_range,
             "layers": [{"type": L.type, "mixer": dict(L.mixer), "mlp": {"kind": "dense", "ff": L.ff} if L.ff else None}
                        for L in self.layers]}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.stop_token_ids:
            d["eos_token_id"] = list(self.stop_token_ids)
        return d

    # ---- the model as data
    def _norm(self) -> PartSpec:
        return PartSpec("norm", "rmsnorm", {"dim": self.hidden_size, "eps": self.norm_eps, "offset": 1.0})

    def _cache_window(self, j: int):
        """What layer j's cache entry must keep: the longest window among the layers that read it (None: everything)."""
        windows = [_window(L.mixer, f"layer {i}") for i, L in enumerate(self.layers)
                   if i == j or (L.type == "attention" and L.mixer.get("kv_from") == j)]
        return None if any(w is None for w in windows) else max(windows)

    def _mixer(self, i: int) -> PartSpec:
        L = self.layers[i]
        m, h = L.mixer, self.hidden_size
        if L.type == "attention":
            source = m.get("kv_from")
            return PartSpec("mixer", "attention", {
                "hidden_size": h, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "position": PartSpec("position", "none", {}), "window": _window(m, f"layer {i}"),
                "bias": True, "qk_norm_eps": self.norm_eps, "scale": float(m["scale"]), "shares_cache": source is not None,
                "cache_window": self._cache_window(i if source is None else source)})
        if L.type == "latent_attention":
            return PartSpec("mixer", "latent_attention", {
                "hidden_size": h, "n_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "norm_eps": self.norm_eps, "scale": float(m["scale"]),
                "window": _window(m, f"layer {i}")})
        return PartSpec("mixer", "channel_delta", {
            "hidden_size": h, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "conv_taps": m["conv"], "norm_eps": self.norm_eps,
            "decay_rank": m.get("a_rank"), "gate_rank": m.get("g_rank")})

    def layer_specs(self) -> list[LayerSpec]:
        specs = []
        for i, L in enumerate(self.layers):
            parts = {"mixer": self._mixer(i), "mixer_norm": self._norm()}
            if self.streams is not None:
                parts["mixer_connection"] = PartSpec("connection", "streams", {"streams": self.streams})
            if L.ff is not None:
                parts["feed_forward"] = PartSpec("feed_forward", "gated", {
                    "hidden_size": self.hidden_size, "intermediate_size": L.ff, "activation": "gelu_tanh"})
                parts["feed_forward_norm"] = self._norm()
                if self.streams is not None:
                    parts["feed_forward_connection"] = PartSpec("connection", "streams", {"streams": self.streams})
            specs.append(LayerSpec("connected", parts))
        return specs

    def schedule(self) -> list[ScheduleEntry]:
        out = []
        for i, L in enumerate(self.layers):
            source = L.mixer.get("kv_from") if L.type == "attention" else None
            out.append(ScheduleEntry(layer=i, cache=i if source is None else source, writes_cache=source is None))
        return out

    def final_norm(self) -> PartSpec:
        return self._norm()

    def output_softcap(self) -> float | None:
        return self.logit_softcap

    def tensor_names(self) -> dict[str, str]:
        names = {"embedding.table": "embed", "final_norm.weight": "final.norm"}
        for i, L in enumerate(self.layers):
            p, c = f"layers.{i}.", f"l{i}."
            names[p + "mixer_norm.weight"] = c + "norm1"
            subs = [("mixer_connection", "hc1")]
            if L.ff is not None:
                names[p + "feed_forward_norm.weight"] = c + "norm2"
                subs.append(("feed_forward_connection", "hc2"))
                for w in ("gate", "up", "down"):
                    names[p + f"feed_forward.{w}"] = c + f"mlp.{w}"
            if self.streams is not None:
                for part, hc in subs:
                    for local, stored in (("read", "in"), ("write", "out"), ("mix", "mix")):
                        names[p + f"{part}.{local}"] = c + f"{hc}.{stored}"
            m = p + "mixer."
            if L.type == "attention":
                for w in ("q", "o") if L.mixer.get("kv_from") is not None else ("q", "k", "v", "o"):
                    names[m + w] = c + f"mix.{w}"
                    if w != "o":
                        names[m + w + "_bias"] = c + f"mix.{w}.b"
            elif L.type == "latent_attention":
                for w in ("dq", "uq", "dkv", "uk", "uv", "o"):
                    names[m + w] = c + f"mix.{w}"
                names[m + "dq_norm"], names[m + "dkv_norm"] = c + "mix.dq.norm", c + "mix.dkv.norm"
            else:
                for w in ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o"):
                    names[m + w] = c + f"mix.{w}"
                for w in ("q", "k", "v"):
                    names[m + w + "_conv"] = c + f"mix.{w}.conv"
        return names

    def init_std(self) -> float:
        return self.initializer_range


register_architecture("Guduzen", GuduzenConfig)
